"""Call plans (nn/plan.py): the recorder's bookkeeping on the CPU with a stand-in library, and on the GPU
the replayed / captured forward pass against the node-by-node one."""
import ctypes

import numpy as np
import pytest

from onnx_translator_b200.capi import CQConvCall, CTensor, TensorP
from onnx_translator_b200.nn.plan import _Recorder


class _FakeLib:
    """Counts references like the library does; operator calls just log their name."""

    def __init__(self):
        self.refs, self.log = {}, []

    def _key(self, handle):
        return ctypes.addressof(handle.contents)

    def tops_retain(self, handle):
        self.refs[self._key(handle)] = self.refs.get(self._key(handle), 1) + 1

    def free_tensor(self, handle):
        self.refs[self._key(handle)] = self.refs.get(self._key(handle), 1) - 1

    def add_forward(self, a, b, o):
        self.log.append("add")

    def tops_qconv_forward(self, call):
        self.log.append("qconv")
        return 0

    def tops_last_error(self):
        return 0

    def tops_download(self, *args):
        return 0


def _tensor():
    return ctypes.pointer(CTensor())


def test_recorder_keeps_operator_calls_and_holds_their_tensors():
    lib = _FakeLib()
    rec = _Recorder(lib)
    a, b, o = _tensor(), _tensor(), _tensor()
    assert isinstance(a, TensorP)
    rec.add_forward(a, b, o)
    rec.tops_retain(a)                       # passed through, not recorded
    rec.free_tensor(a)
    assert lib.log == ["add"] and len(rec.calls) == 1
    assert all(lib.refs[lib._key(t)] == 2 for t in (a, b, o))          # one more reference each, held by the recording
    # a tensor handle inside the QConvCall struct is held too
    y = _tensor()
    call = CQConvCall()
    call.y = ctypes.cast(y, ctypes.c_void_p)
    rec.tops_qconv_forward(ctypes.byref(call))
    assert lib.refs[lib._key(y)] == 2 and len(rec.calls) == 2
    # replaying issues the same calls with the same argument objects
    for fn, args in rec.calls:
        fn(*args)
    assert lib.log == ["add", "qconv", "add", "qconv"]
    rec.release()
    assert all(lib.refs[lib._key(t)] == 1 for t in (a, b, o, y))


def test_recorder_refuses_host_reads_during_recording():
    from onnx_translator_b200.capi import TensorOpsError
    rec = _Recorder(_FakeLib())
    with pytest.raises(TensorOpsError):
        rec.tops_download(_tensor(), None, 0)


# ---- on the device ------------------------------------------------------------------------------------------------
def _bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


@pytest.mark.gpu
def test_small_cnn_plan_replays_and_captures_bit_for_bit():
    from onnx_translator_b200 import nn
    graph, x = nn.small_cnn(seed=0)
    prob, side = (t.numpy() for t in graph.forward(x))
    plan = graph.plan(x)
    assert len(plan.calls) == 11                     # 12 nodes, Flatten is a view
    p1, s1 = (t.numpy() for t in plan.run())
    assert np.array_equal(_bits(p1), _bits(prob)) and np.array_equal(_bits(s1), _bits(side))
    # another input of the same shape, given as a host tensor
    rng = np.random.default_rng(5)
    x2 = nn.Tensor(1, 3, 32, 32, dtype="float32", data=rng.standard_normal((1, 3, 32, 32)).astype(np.float32))
    want2 = [t.numpy() for t in graph.forward(x2)]
    got2 = [t.numpy() for t in plan.run(x2)]
    assert all(np.array_equal(_bits(g), _bits(w)) for g, w in zip(got2, want2))
    assert plan.capture(), "the small CNN's forward pass must be capturable as one CUDA graph"
    got3 = [t.numpy() for t in plan.run(x)]
    assert np.array_equal(_bits(got3[0]), _bits(prob)) and np.array_equal(_bits(got3[1]), _bits(side))
    got4 = [t.numpy() for t in plan.run(x2)]
    assert all(np.array_equal(_bits(g), _bits(w)) for g, w in zip(got4, want2))
    with pytest.raises(ValueError):
        plan.run(nn.Tensor(2, 3, 32, 32, dtype="float32"))
    plan.close()


@pytest.mark.gpu
def test_channels_last_edges_do_not_change_the_fused_graph_result():
    """The fourth fusion pass (float32 edges between fused convolutions kept [N, H, W, C]) moves bytes, not values:
    same logits, bit for bit, as the fused graph whose float32 edges are all NCHW -- and the plan gives them too."""
    from onnx_translator_b200 import nn
    graph, x = nn.qdq_resnet50(batch=3, seed=1, image=64, stages=(2, 2, 1, 1), widths=(8, 16, 24, 32), classes=20)
    graph.output_name = ["logits"]
    with_cl = graph.fused()
    n_cl = sum(getattr(op, "y_channels_last", False) for op in with_cl.ops.values())
    # every block output but the last one (MaxPool reads that), and the four shortcut convolutions
    assert n_cl == (6 - 1) + 4
    assert sum(getattr(op, "residual_channels_last", False) for op in with_cl.ops.values()) == 6
    assert sum(getattr(op, "x_channels_last", False) for op in with_cl.ops.values()) >= 3      # stride-2 shortcuts read the block input as float32
    nchw = graph.fused(channels_last=False)
    assert not any(getattr(op, "y_channels_last", False) for op in nchw.ops.values())
    a = with_cl.forward(x).numpy()
    b = nchw.forward(x).numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    plan = with_cl.plan(x)
    assert np.array_equal(plan.run().numpy().view(np.uint32), a.view(np.uint32))
    if plan.capture():
        assert np.array_equal(plan.run().numpy().view(np.uint32), a.view(np.uint32))
    plan.close()
