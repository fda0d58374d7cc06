"""Test infrastructure, like the rest of this package: runs a ``Graph`` of onnx_translator_b200 on the
CPU oracle, node by node -- the checker for whole graphs and the CPU baseline of the graph benchmark.  Edges are numpy arrays in storage convention; node attributes are read from the very
operator objects the device runner executes."""
import numpy as np


def run(graph, port, *inputs, all_edges=False):
    """Outputs of the graph; with ``all_edges`` also the dict of every edge (name -> array) for layer-by-layer checks."""
    edges = {name: (t.numpy(), t.dtype) for name, t in graph.initializers.items()}
    for name, t in zip(graph.input_name, inputs):
        edges[name] = (t.numpy(), t.dtype)
    for op in graph.ops.values():
        kind = type(op).__name__
        args = [edges[e] for e in op.inputs if e]
        out_dt = op.dtype or "float32"
        if kind in ("RELU", "ABS", "COS"):
            (x, xd), = args
            y = port.unary(kind.lower(), x, xd, out_dt)
        elif kind in ("ADD", "SUB", "MUL", "DIV"):
            (a, ad), (b, bd) = args
            y = port.binary(kind.lower(), a, ad, b, bd, out_dt)
        elif kind == "QuantizeLinear":
            (x, xd), (s, sd), (z, zd) = args
            y = port.quantize(x, xd, s, sd, z, zd, out_dt, axis=op.axis)
        elif kind == "DequantizeLinear":
            (x, xd), (s, sd), (z, zd) = args
            y = port.dequantize(x, xd, s, sd, z, zd, out_dt)
        elif kind == "Conv":
            (x, xd), (w, wd) = args[:2]
            b, bd = args[2] if len(args) > 2 else (None, "float32")
            y = port.conv2d(x, xd, w, wd, b, bd, out_dt, tuple(op.pads), tuple(op.strides), tuple(op.dilations), op.group)
        elif kind == "MaxPool":
            (x, xd), = args
            y = port.max_pool(x, xd, out_dt, tuple(op.kernel_shape), tuple(op.pads), tuple(op.strides), tuple(op.dilations))
        elif kind == "Gemm":
            (a, ad), (b, bd) = args[:2]
            c, cd = args[2] if len(args) > 2 else (None, "float32")
            y = port.gemm(a, ad, b, bd, c, cd, out_dt, op.alpha, op.beta, op.transA, op.transB)
        elif kind == "Softmax":
            (x, xd), = args
            y = port.softmax(x, xd, out_dt, op.axis)
        elif kind in ("Flatten", "Reshape"):
            (x, xd), = args[:1]
            y = x.reshape(x.shape[0], -1) if kind == "Flatten" else x.reshape(op.shape)
        else:
            raise NotImplementedError(kind)
        edges[op.outputs[0]] = (np.asarray(y), out_dt)
    outs = tuple(edges[e][0] for e in graph.output_name)
    outs = outs[0] if len(outs) == 1 else outs
    if all_edges:
        return outs, {name: value for name, (value, _) in edges.items()}
    return outs
