"""The QDQ ResNet-50-shaped graph at the size the benchmark runs it (224 x 224 input, stages [3, 4, 6, 3],
widths 64 .. 512 with 4x expansion, K up to 4608), two images, against the oracle executing the unfused
nodes (QuantizeLinear, DequantizeLinear, Conv, Relu, Add: tensor_ops.c:999-1034, 1036-1114, 708-728, 864-997).

Two gates.

Layer by layer, on identical inputs: every fused convolution (Q -> DQ -> Conv(DQ(W)) [-> Add] [-> Relu] in one
tensor-core call) is run on the ORACLE's input to that layer, and its float32 result is quantised with the scale and
zero point of every QuantizeLinear that reads it in the unfused graph.  Those codes must equal the codes of the
oracle's own result except for at most 1e-4 of the elements, and never by more than one step.  (Why not zero:
the fused call accumulates exact integer products and applies x_scale * w_scale[m] once, the reference rounds every
dequantised operand to float32 and accumulates in double; the results differ by ~1e-7 relative, which moves a
value across a rounding tie now and then.)  Results no QuantizeLinear reads are compared as floats.

End to end: one flipped code perturbs hundreds of outputs of the next layer by a fraction of a step, so over 53
quantised layers the two runs decorrelate at the level of the quantisation noise itself; what stays bounded is the
size of that noise.  The gate is on the logits (relative L2) and on the probabilities, with the measured values
printed so the margin can be seen.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CODE_MISMATCH_RATE = 1e-4          # per layer, on identical inputs
LOGITS_REL_L2 = 5e-2               # end to end
PROB_MAX_ABS = 5e-2                # end to end, relative to the largest probability


@pytest.fixture(scope="module")
def full_size(port):
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import nn
    graph, x = nn.qdq_resnet50(batch=2, seed=0, image=224)
    graph.output_name = ["logits", "prob"]
    (want_logits, want_prob), edges = oracle_graph.run(graph, port, x, all_edges=True)
    return graph, x, edges, want_logits, want_prob


def test_every_fused_convolution_matches_the_oracle_on_the_oracles_input(port, full_size):
    from onnx_translator_b200.nn import Tensor
    from onnx_translator_b200.nn.fused_ops import QLinearConv
    graph, x, edges, _, _ = full_size
    fused = graph.fused()
    quantisers = {}
    for op in graph.ops.values():
        if type(op).__name__ == "QuantizeLinear":
            quantisers.setdefault(op.inputs[0], []).append(op)
    T = lambda a, dt: Tensor(*a.shape, dtype=dt, data=np.ascontiguousarray(a))
    checked = worst_rate = 0
    report = []
    for node in fused.ops.values():
        if type(node).__name__ != "QLinearConv":
            continue
        assert node.from_float
        names = list(node.inputs) + [""] * 9
        x_edge = names[0][:-len(".levels")] if names[0].endswith(".levels") else names[0]
        init = graph.initializers
        alone = QLinearConv([], [], node.pads, node.strides, node.dilations, node.relu, "float32", from_float=True)
        got = alone.forward(T(edges[x_edge], "float32"), init[names[1]], init[names[2]], init[names[3]], init[names[4]],
                            init[names[5]] if names[5] else None,
                            T(edges[names[6]], "float32") if names[6] else None)["tensor"].numpy()
        want = edges[node.outputs[0]]
        assert got.shape == want.shape, node.name
        readers = quantisers.get(node.outputs[0], [])
        for q in readers:
            scale, zero = init[q.inputs[1]].numpy(), init[q.inputs[2]].numpy()
            zdt = init[q.inputs[2]].dtype
            a = port.quantize(got, "float32", scale, "float32", zero, zdt, zdt).astype(np.int32)
            b = port.quantize(want, "float32", scale, "float32", zero, zdt, zdt).astype(np.int32)
            rate = float(np.mean(a != b))
            step = int(np.abs(a - b).max())
            report.append((node.name, got.size, rate, step))
            worst_rate = max(worst_rate, rate)
            assert step <= 1, (node.name, step)
            assert rate <= CODE_MISMATCH_RATE, (node.name, rate)
            assert np.unique(b).size > 8, node.name                       # a real spread of codes, not a saturated tensor
            checked += 1
        if not readers:                                                   # e.g. the last block, read by MaxPool
            tol = 1e-5 * np.abs(want).max()
            assert np.abs(got.astype(np.float64) - want).max() <= tol, node.name
            checked += 1
    print(f"\n{checked} layer checks, worst code mismatch rate {worst_rate:.2e}")
    for name, size, rate, step in sorted(report, key=lambda r: -r[2])[:5]:
        print(f"  {name}: {size} elements, mismatch rate {rate:.2e}, max step {step}")
    assert checked >= 53


def test_fused_graph_end_to_end_at_benchmark_size(full_size):
    graph, x, _, want_logits, want_prob = full_size
    fused = graph.fused()
    kinds = [type(op).__name__ for op in fused.ops.values()]
    assert kinds.count("QLinearConv") == 53 and kinds.count("Conv") == 0
    assert sum(getattr(op, "y_channels_last", False) for op in fused.ops.values()) >= 16      # block outputs and shortcuts stay channels-last
    logits, prob = fused.forward(x)
    got_logits, got_prob = logits.numpy().astype(np.float64), prob.numpy().astype(np.float64)
    rel = np.linalg.norm(got_logits - want_logits) / np.linalg.norm(want_logits)
    dp = np.abs(got_prob - want_prob).max() / want_prob.max()
    print(f"\nlogits relative L2 {rel:.3e}; max |prob difference| / max prob {dp:.3e}")
    assert rel < LOGITS_REL_L2, rel
    assert dp < PROB_MAX_ABS, dp
    assert np.allclose(got_prob.sum(axis=1), 1.0, atol=1e-5)
    # the recorded call plan and the captured CUDA graph give the same bits as the node-by-node run
    plan = fused.plan(x)
    again = [t.numpy() for t in plan.run()]
    assert np.array_equal(again[0].view(np.uint32), logits.numpy().view(np.uint32))
    if plan.capture():
        third = [t.numpy() for t in plan.run()]
        assert np.array_equal(third[0].view(np.uint32), logits.numpy().view(np.uint32))
    plan.close()
