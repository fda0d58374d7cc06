"""The resident graph runner: topology rules on the CPU (with stand-in nodes), and on the GPU the
two benchmark graphs against the oracle executing the same nodes."""
import numpy as np
import pytest

from onnx_translator_b200.nn.graph import Graph


class _Value:
    def __init__(self, v):
        self.v = v
        self.uploads = 0

    def to_device(self):
        self.uploads += 1
        return self


class _Node:
    """Stand-in operator: adds its inputs (no library, no GPU)."""
    log = []

    def __init__(self, inputs, outputs, name=None):
        self.inputs, self.outputs, self.name = inputs, outputs, name

    def forward(self, *args):
        _Node.log.append((self.name, len(args)))
        return {"tensor": _Value(sum(a.v for a in args))}


class _Other(_Node):
    pass


def test_graph_runs_nodes_in_order_feeds_initializers_and_returns_outputs():
    w = _Value(10)
    g = Graph([_Node(["x", "w"], ["a"]), _Other(["a", "a"], ["b"]), _Node(["b", "x"], ["y"])], "x", initializers={"w": w})
    assert list(g.ops) == ["_Node.0", "_Other.0", "_Node.1"]
    assert g.output_name == ["y"]                       # inferred: the edge nobody reads
    out = g.forward(_Value(1))
    assert out.v == (1 + 10) * 2 + 1
    g.forward(_Value(2))
    assert w.uploads == 1                               # weights are made resident once


def test_graph_returns_a_tuple_for_several_outputs_and_skips_absent_optional_inputs():
    _Node.log = []
    g = Graph([_Node(["x", ""], ["a"], name="first"), _Node(["a"], ["b"]), _Node(["a"], ["c"])], ["x"], ["b", "c"])
    b, c = g.forward(_Value(3))
    assert (b.v, c.v) == (3, 3)
    assert _Node.log[0] == ("first", 1)                 # the empty optional input is not passed


def test_graph_rejects_bad_topology():
    with pytest.raises(ValueError):
        Graph([_Node(["nowhere"], ["a"])], "x")
    with pytest.raises(ValueError):
        Graph([_Node(["x"], ["a"]), _Node(["x"], ["a"])], "x")
    with pytest.raises(ValueError):
        Graph([_Node(["x"], ["a"])], "x", ["missing"])
    with pytest.raises(ValueError):
        Graph([_Node(["x"], ["a"])], "x").forward()


# ---- on the device --------------------------------------------------------------------------------------------
def _bits_equal(got, want):
    return got.shape == want.shape and np.array_equal(np.ascontiguousarray(got).view(np.uint8), np.ascontiguousarray(want).view(np.uint8))


@pytest.mark.gpu
def test_small_cnn_graph_matches_the_oracle(port):
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import nn
    graph, x = nn.small_cnn(seed=0)
    prob, side = graph.forward(x)
    want_prob, want_side = oracle_graph.run(graph, port, x)
    assert _bits_equal(side.numpy(), want_side)          # conv, add, sub, mul, div, abs, cos: bit for bit
    assert np.allclose(prob.numpy(), want_prob, rtol=1e-6, atol=0)
    again, _ = graph.forward(x)                          # a second run on resident weights gives the same bits
    assert _bits_equal(again.numpy(), prob.numpy())


@pytest.mark.gpu
def test_qdq_resnet_shaped_graph_matches_the_oracle_node_for_node(port):
    """A small instance of the QDQ ResNet-50-shaped graph (same node pattern, one block per stage).
    With every convolution on the exact kernel the logits agree bit for bit; the softmax within 1e-6."""
    import os
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import nn
    os.environ["TOPS_DISABLE_TC"] = "1"
    try:
        graph, x = nn.qdq_resnet50(batch=2, seed=0, image=64, stages=(1, 1, 1, 1), widths=(8, 16, 24, 32), classes=20)
        kinds = [type(op).__name__ for op in graph.ops.values()]
        assert kinds.count("Conv") == 1 + 4 * 4 and kinds.count("QuantizeLinear") == kinds.count("Conv")
        assert kinds.count("DequantizeLinear") == 2 * kinds.count("Conv") and kinds.count("ADD") == 4
        graph.output_name = ["logits", "prob"]
        logits, prob = graph.forward(x)
        want_logits, want_prob = oracle_graph.run(graph, port, x)
    finally:
        del os.environ["TOPS_DISABLE_TC"]
    assert _bits_equal(logits.numpy(), want_logits)
    assert np.allclose(prob.numpy(), want_prob, rtol=1e-6, atol=1e-45)
    assert np.allclose(prob.numpy().sum(axis=1), 1.0, atol=1e-5)


@pytest.mark.gpu
def test_fused_graph_replaces_every_qdq_conv_chain_and_stays_close_to_the_oracle(port):
    """Graph.fused() turns each Q -> DQ -> Conv(DQ(w)) [-> Relu] chain into one node.  The fused
    convolutions differ from the chain within the tensor-core tolerance, which moves a few activation
    codes by one step in later layers; the logits stay within 1 % (relative L2) of the oracle's."""
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import nn
    graph, x = nn.qdq_resnet50(batch=2, seed=0, image=64, stages=(1, 1, 1, 1), widths=(8, 16, 24, 32), classes=20)
    graph.output_name = ["logits", "prob"]
    fused = graph.fused()
    kinds = [type(op).__name__ for op in fused.ops.values()]
    convs = sum(type(op).__name__ == "Conv" for op in graph.ops.values())
    assert kinds.count("QLinearConv") == convs and kinds.count("Conv") == 0 and kinds.count("DequantizeLinear") == 0
    assert kinds.count("QuantizeLinear") == 0 and kinds.count("RELU") == 0 and kinds.count("ADD") == 0
    assert sum(len(op.inputs) >= 7 and bool(op.inputs[6]) for op in fused.ops.values()) == 4     # the four residual tails
    logits, prob = fused.forward(x)
    want_logits, want_prob = oracle_graph.run(graph, port, x)
    got = logits.numpy().astype(np.float64)
    err = np.linalg.norm(got - want_logits) / np.linalg.norm(want_logits)
    assert err < 1e-2, err
    assert np.allclose(prob.numpy().sum(axis=1), 1.0, atol=1e-5)
    assert np.abs(prob.numpy() - want_prob).max() < 1e-2 * want_prob.max()


# ---- golden outputs of the small CNN (made by tests/golden/make_graph_golden.py from the compiled reference) ----
def _small_cnn_golden():
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "small_cnn.npz"))


def test_oracle_port_reproduces_the_small_cnn_golden_outputs(port):
    """No GPU involved: building the graph needs none, and the C restatement runs it on the host."""
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import nn
    graph, x = nn.small_cnn(seed=0)
    prob, side = oracle_graph.run(graph, port, x)
    gold = _small_cnn_golden()
    assert _bits_equal(side, gold["side"]) and _bits_equal(prob, gold["prob"])


@pytest.mark.gpu
def test_small_cnn_graph_reproduces_the_golden_outputs():
    from onnx_translator_b200 import nn
    graph, x = nn.small_cnn(seed=0)
    prob, side = graph.forward(x)
    gold = _small_cnn_golden()
    assert _bits_equal(side.numpy(), gold["side"])
    assert np.allclose(prob.numpy(), gold["prob"], rtol=1e-6, atol=0)


def _hand_built_qdq_block(shared_codes=False, weight_zero=0, stride=1, group=1):
    """x -> Q -> DQ -> Conv(DQ(w)) -> Relu -> Q -> DQ -> Conv(DQ(w2)) -> Add(., x) -> Relu, built without a GPU."""
    from onnx_translator_b200 import nn
    from onnx_translator_b200.nn import Operators as ops
    f32 = "float32"
    T = lambda a, dt: nn.Tensor(*np.asarray(a).shape, dtype=dt, data=np.asarray(a))
    init = {"s": T(np.array([0.1], np.float32), f32), "z": T(np.zeros(1, np.int8), "int8"),
            "w1": T(np.ones((8, 8, 3, 3), np.int8), "int8"), "w1s": T(np.full((8, 1, 1, 1), 0.01, np.float32), f32),
            "w1z": T(np.full((8, 1, 1, 1), weight_zero, np.int8), "int8"),
            "w2": T(np.ones((8, 8, 1, 1), np.int8), "int8"), "w2s": T(np.full((8, 1, 1, 1), 0.01, np.float32), f32),
            "w2z": T(np.zeros((8, 1, 1, 1), np.int8), "int8"), "b": T(np.zeros(8, np.float32), f32)}
    nodes = [
        ops.QuantizeLinear(["x", "s", "z"], ["xq"], axis=1, dtype="int8"),
        ops.DequantizeLinear(["xq", "s", "z"], ["xdq"], dtype=f32),
        ops.DequantizeLinear(["w1", "w1s", "w1z"], ["w1dq"], dtype=f32),
        ops.Conv(["xdq", "w1dq", "b"], ["c1"], pads=[1, 1, 1, 1], strides=[stride, stride], dilations=[1, 1], group=group, dtype=f32),
        ops.RELU(["c1"], ["r1"], dtype=f32),
        ops.QuantizeLinear(["r1", "s", "z"], ["r1q"], axis=1, dtype="int8"),
        ops.DequantizeLinear(["r1q", "s", "z"], ["r1dq"], dtype=f32),
        ops.DequantizeLinear(["w2", "w2s", "w2z"], ["w2dq"], dtype=f32),
        ops.Conv(["r1dq", "w2dq"], ["c2"], pads=[0, 0, 0, 0], strides=[1, 1], dilations=[1, 1], group=1, dtype=f32),
        ops.ADD(["c2", "x"], ["sum"], dtype=f32),
        ops.RELU(["sum"], ["y"], dtype=f32),
    ]
    outputs = ["y", "xq"] if shared_codes else ["y"]
    return Graph(nodes, "x", outputs, "block", init)


def test_fusion_pass_rewrites_chains_and_residual_tails_without_a_gpu():
    fused = _hand_built_qdq_block().fused()
    kinds = [type(op).__name__ for op in fused.ops.values()]
    assert kinds == ["QLinearConv", "QLinearConv"]
    first, second = fused.ops.values()
    assert first.from_float and first.relu and first.inputs == ["x", "s", "z", "w1", "w1s", "b", "", "s", "z"] and first.outputs == ["r1"]
    assert first.next_conv == dict(pads=[0, 0, 0, 0], strides=[1, 1], dilations=[1, 1], kernel=[1, 1]) and not first.levels_in
    assert second.levels_in and second.next_conv is None                       # the edge r1 carries integer levels
    assert second.from_float and second.relu and second.inputs == ["r1", "s", "z", "w2", "w2s", "", "x"] and second.outputs == ["y"]


def test_fusion_pass_leaves_what_it_must_not_touch():
    # the codes are a graph output too: the QuantizeLinear stays and the fused node starts from the codes
    g = _hand_built_qdq_block(shared_codes=True).fused()
    kinds = [type(op).__name__ for op in g.ops.values()]
    assert kinds[0] == "QuantizeLinear" and kinds[1] == "QLinearConv" and not list(g.ops.values())[1].from_float
    # non-zero weight zero points, grouped or stride-3 convolutions are not what the fused kernel computes
    for bad in (dict(weight_zero=3), dict(group=2), dict(stride=3)):
        kinds = [type(op).__name__ for op in _hand_built_qdq_block(**bad).fused().ops.values()]
        # (the Q -> DQ pair in front of the untouched convolution still becomes one round-trip node)
        assert kinds[:4] == ["QuantizeDequantize", "DequantizeLinear", "Conv", "RELU"], bad
        assert kinds.count("QLinearConv") == 1                                   # the second chain is still taken


def test_fusion_conditions_on_scale_shape_and_dtypes():
    """DequantizeLinear has no axis: only a weight scale shaped [M, 1, 1, 1] scales per output channel.  A flat [M]
    scale, a float16 DequantizeLinear or a zero point of another type than the codes leave the chain unfused."""
    from onnx_translator_b200 import nn
    T = lambda a, dt: nn.Tensor(*np.asarray(a).shape, dtype=dt, data=np.asarray(a))
    def conv_kinds(mutate):
        g = _hand_built_qdq_block()
        mutate(g)
        return [type(op).__name__ for op in Graph(list(g.ops.values()), "x", ["y"], "block", g.initializers).fused().ops.values()]
    def flat_scale(g):
        g.initializers["w1s"] = T(np.full(8, 0.01, np.float32), "float32")
        g.initializers["w1z"] = T(np.zeros(8, np.int8), "int8")
    def half_dq(g):
        list(g.ops.values())[2].dtype = "float16"
    def zero_type(g):
        g.initializers["z"] = T(np.zeros(1, np.uint8), "uint8")
    assert conv_kinds(lambda g: None).count("Conv") == 0
    for mutate in (flat_scale, half_dq, zero_type):
        assert conv_kinds(mutate).count("Conv") >= 1, mutate.__name__


def _hand_built_quantised_add(relu=True, second_reader=False):
    """a, b int8 codes -> DQ, DQ -> Add [-> Relu] -> Q -> DQ -> (output), and x -> Q -> DQ beside it."""
    from onnx_translator_b200 import nn
    from onnx_translator_b200.nn import Operators as ops
    f32 = "float32"
    T = lambda a, dt: nn.Tensor(*np.asarray(a).shape, dtype=dt, data=np.asarray(a))
    init = {"sa": T(np.array([0.05], np.float32), f32), "za": T(np.array([3], np.int8), "int8"),
            "sb": T(np.array([0.02], np.float32), f32), "zb": T(np.array([100], np.uint8), "uint8"),
            "sy": T(np.array([0.04], np.float32), f32), "zy": T(np.array([-5], np.int8), "int8")}
    nodes = [ops.DequantizeLinear(["a", "sa", "za"], ["da"], dtype=f32),
             ops.DequantizeLinear(["b", "sb", "zb"], ["db"], dtype=f32),
             ops.ADD(["da", "db"], ["sum"], dtype=f32)]
    edge = "sum"
    if relu:
        nodes.append(ops.RELU(["sum"], ["act"], dtype=f32))
        edge = "act"
    nodes += [ops.QuantizeLinear([edge, "sy", "zy"], ["yq"], axis=1, dtype="int8"),
              ops.DequantizeLinear(["yq", "sy", "zy"], ["y"], dtype=f32),
              ops.QuantizeLinear(["x", "sy", "zy"], ["xq"], axis=1, dtype="int8"),
              ops.DequantizeLinear(["xq", "sy", "zy"], ["xr"], dtype=f32)]
    outputs = ["y", "xr"] + (["sum"] if second_reader else [])
    return Graph(nodes, ["a", "b", "x"], outputs, "qadd", init)


def test_elementwise_qdq_fusion_pass_without_a_gpu():
    fused = _hand_built_quantised_add().fused()
    kinds = [type(op).__name__ for op in fused.ops.values()]
    assert kinds == ["DequantAddQuant", "DequantizeLinear", "QuantizeDequantize"]
    first, _, third = fused.ops.values()
    assert first.relu and first.inputs == ["a", "sa", "za", "b", "sb", "zb", "sy", "zy"] and first.outputs == ["yq"]
    assert third.inputs == ["x", "sy", "zy"] and third.outputs == ["xr"] and not third.with_codes
    assert not list(_hand_built_quantised_add(relu=False).fused().ops.values())[0].relu
    # the float32 sum is a graph output too: the chain must stay as it is
    kinds = [type(op).__name__ for op in _hand_built_quantised_add(second_reader=True).fused().ops.values()]
    assert kinds[:3] == ["DequantizeLinear", "DequantizeLinear", "ADD"] and "DequantAddQuant" not in kinds


@pytest.mark.gpu
def test_levels_edges_do_not_change_the_fused_graph_result():
    """The third fusion pass (integer levels between consecutive fused convolutions) is exact: same logits, bit for
    bit, as the fused graph whose edges are float32 tensors."""
    from onnx_translator_b200 import nn
    graph, x = nn.qdq_resnet50(batch=2, seed=0, image=64, stages=(1, 2, 1, 1), widths=(8, 16, 24, 32), classes=20)
    graph.output_name = ["logits"]
    with_levels = graph.fused()
    # conv2 and conv3 of each of the five blocks, plus the first convolution reading each later block's input
    assert sum(getattr(op, "levels_in", False) for op in with_levels.ops.values()) == 2 * 5 + 4
    assert sum(getattr(op, "also_float", False) for op in with_levels.ops.values()) == 4
    plain = graph.fused(channels_last=False)
    for op in plain.ops.values():
        if type(op).__name__ == "QLinearConv":
            if op.next_conv is not None:
                op.next_conv, op.inputs, op.also_float, op.outputs = None, op.inputs[:7], False, op.outputs[:1]
            if op.levels_in:
                op.levels_in, op.inputs = False, [op.inputs[0].replace(".levels", "")] + list(op.inputs[1:])
    plain = Graph(list(plain.ops.values()), "x", ["logits"], "plain", plain.initializers)     # recount the edge readers
    a = with_levels.forward(x).numpy()
    b = plain.forward(x).numpy()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
