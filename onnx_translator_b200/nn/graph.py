"""Resident graph runner and the two graph-shaped benchmark workloads.

``Graph`` mirrors the reference's graph object (nn/__init__.py:346-456: a list of operator nodes
with named input and output edges, executed in list order) with the three things a resident runner
needs and the reference lacks: initializers (weights, scales) are fed to the nodes and uploaded
once, every edge stays on the device between nodes, and ``forward`` returns the graph outputs.

The builders construct the graphs from operator constructor calls -- the same objects an ONNX import
would create -- so no model file or ``onnx`` package is involved:

* ``small_cnn``      the small CNN of the first benchmark configuration;
* ``qdq_resnet50``   a ResNet-50-shaped network (stem 7x7/2, bottleneck stages [3, 4, 6, 3], widths
                     64/128/256/512 with 4x expansion) in which every convolution reads its input
                     through QuantizeLinear -> DequantizeLinear (int8, per tensor) and its weights
                     through DequantizeLinear (int8, per output channel).  Weights are random
                     (seeded); only the well-known layer shapes are taken from the architecture.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

import numpy as np


class Graph:
    """Operator nodes with named edges, executed in list order (which must be topological)."""

    def __init__(self, ops, input_name, output_name=None, model_name=None, initializers: Optional[Dict[str, object]] = None):
        self.input_name = input_name if isinstance(input_name, list) else [input_name]
        self.ops = OrderedDict()
        self.model_name = model_name
        self.initializers = dict(initializers or {})
        self._resident = False
        counts: Dict[str, int] = {}
        produced = set(self.input_name) | set(self.initializers)
        self.consumers: Dict[str, int] = {}
        for op in ops:
            kind = type(op).__name__
            counts[kind] = counts.get(kind, -1) + 1
            if not getattr(op, "name", None):
                op.name = f"{kind}.{counts[kind]}"
            if op.name in self.ops:
                raise ValueError(f"node name {op.name} repeats")
            for edge in op.inputs:
                if edge and edge not in produced:
                    raise ValueError(f"{op.name} reads edge {edge!r} before any node produces it")
                if edge:
                    self.consumers[edge] = self.consumers.get(edge, 0) + 1
            for edge in op.outputs:
                if edge in produced:
                    raise ValueError(f"output edge name {edge} repeats")
                produced.add(edge)
            self.ops[op.name] = op
        if output_name is None or output_name == [None]:
            # edges nobody reads are the outputs (what the reference infers)
            output_name = [e for op in self.ops.values() for e in op.outputs if self.consumers.get(e, 0) == 0]
        self.output_name = output_name if isinstance(output_name, list) else [output_name]
        for edge in self.output_name:
            if edge not in produced:
                raise ValueError(f"graph output {edge!r} is not produced by any node")

    def fused(self, channels_last: bool = True) -> "Graph":
        """A graph computing the same function with every

            QuantizeLinear -> DequantizeLinear -> Conv(weights = DequantizeLinear(initializers)) [-> Relu]

        chain executed by one ``QLinearConv`` node (the QuantizeLinear is part of it unless something else
        reads the codes); a following Add of another float32 tensor [-> Relu] -- the tail of a residual
        block -- joins that node's epilogue; and where one such node feeds another, the edge between them
        carries integer levels in the consumer's layout instead of (or, when the float32 values have
        other readers, besides) a float32 tensor.
        A chain is taken only when nothing else reads its inner edges, the weight zero points are all
        zero and the convolution is one the fused kernel covers (group 1; stride 1, or stride 2 with
        dilation 1); everything else is left as it is.  Initializers are shared with this graph.
        ``channels_last=False`` keeps every float32 edge NCHW (the fourth pass below is skipped)."""
        from .fused_ops import QLinearConv
        nodes = list(self.ops.values())
        producer = {e: op for op in nodes for e in op.outputs}
        kind = lambda op: type(op).__name__
        dropped, replaced = set(), {}

        def sole_consumer(edge):
            return self.consumers.get(edge, 0) == 1 and edge not in self.output_name

        for conv in nodes:
            if kind(conv) != "Conv" or len(conv.inputs) < 2:
                continue
            dq_x, dq_w = producer.get(conv.inputs[0]), producer.get(conv.inputs[1])
            if dq_x is None or dq_w is None or kind(dq_x) != "DequantizeLinear" or kind(dq_w) != "DequantizeLinear":
                continue
            q = producer.get(dq_x.inputs[0])
            if q is None or kind(q) != "QuantizeLinear" or q.inputs[1:3] != dq_x.inputs[1:3] or q.dtype not in ("int8", "uint8"):
                continue
            if not all(e in self.initializers for e in dq_w.inputs) or not all(e in self.initializers for e in q.inputs[1:3]):
                continue
            if not (sole_consumer(dq_x.outputs[0]) and sole_consumer(dq_w.outputs[0])):
                continue
            w_codes, w_scale, w_zero = (self.initializers[e] for e in dq_w.inputs)
            strides, dil = list(conv.strides), list(conv.dilations)
            covered = conv.group == 1 and (strides == [1, 1] or (strides == [2, 2] and dil == [1, 1]))
            m_out = int(w_codes.size[0])
            # DequantizeLinear has no axis: its scale broadcasts over TRAILING dimensions, so only [M, 1, 1, 1] scales per
            # output channel, which is what the fused node applies; a float16 DequantizeLinear would round each
            # dequantised value, which the fused node does not
            per_channel = tuple(w_scale.size) == (m_out, 1, 1, 1) and tuple(w_zero.size) == tuple(w_scale.size)
            x_zero = self.initializers[q.inputs[2]]
            if (not covered or not per_channel or w_codes.dtype != "int8" or w_scale.dtype != "float32" or np.any(w_zero.numpy() != 0)
                    or (dq_x.dtype or "float32") != "float32" or (dq_w.dtype or "float32") != "float32" or x_zero.dtype != q.dtype
                    or self.initializers[q.inputs[1]].data_size != 1 or x_zero.data_size != 1):
                continue
            relu, out_edge = False, conv.outputs[0]
            if sole_consumer(out_edge):
                nxt = next((op for op in nodes if out_edge in op.inputs), None)
                if nxt is not None and kind(nxt) == "RELU" and (nxt.dtype or "float32") == (conv.dtype or "float32"):
                    relu, out_edge = True, nxt.outputs[0]
                    dropped.add(nxt.name)
            bias = conv.inputs[2] if len(conv.inputs) > 2 and conv.inputs[2] else ""
            # the QuantizeLinear joins the call when only this chain reads its codes
            from_float = sole_consumer(q.outputs[0]) and q.name not in dropped
            if from_float:
                dropped.add(q.name)
            node = QLinearConv([q.inputs[0] if from_float else q.outputs[0], q.inputs[1], q.inputs[2], dq_w.inputs[0], dq_w.inputs[1], bias],
                               [out_edge], conv.pads, strides, dil, relu, conv.dtype or "float32", from_float=from_float)
            node.name = conv.name + ".fused"
            dropped.update((dq_x.name, dq_w.name))
            replaced[conv.name] = node
        kept = [replaced.get(op.name, op) for op in nodes if op.name not in dropped]

        # second pass: QLinearConv -> Add(., other float32 tensor) [-> Relu] joins the convolution's epilogue
        order = {op.name: i for i, op in enumerate(kept)}
        made_by = {e: op for op in kept for e in op.outputs}
        readers: Dict[str, list] = {}
        for op in kept:
            for e in op.inputs:
                if e:
                    readers.setdefault(e, []).append(op)
        gone = set()
        for add in kept:
            if kind(add) != "ADD" or add.name in gone or (add.dtype or "float32") != "float32":
                continue
            cands = []
            for mine, other in ((add.inputs[0], add.inputs[1]), (add.inputs[1], add.inputs[0])):
                conv = made_by.get(mine)
                if (conv is not None and kind(conv) == "QLinearConv" and not conv.relu and conv.dtype == "float32" and mine != other
                        and len(conv.inputs) == 6 and len(readers.get(mine, [])) == 1 and mine not in self.output_name
                        and order.get(getattr(made_by.get(other), "name", None), -1) < order[conv.name]):
                    cands.append((order[conv.name], conv, other))
            if not cands:
                continue
            _, conv, other = max(cands, key=lambda t: t[0])
            out_edge, relu = add.outputs[0], False
            after = readers.get(out_edge, [])
            if len(after) == 1 and kind(after[0]) == "RELU" and out_edge not in self.output_name and (after[0].dtype or "float32") == "float32":
                relu, out_edge = True, after[0].outputs[0]
                gone.add(after[0].name)
            gone.add(add.name)
            conv.inputs = list(conv.inputs) + [other]
            conv.outputs = [out_edge]
            conv.relu = relu
        kept = [op for op in kept if op.name not in gone]

        # third pass: a float32 edge between two fused convolutions that nobody else reads never needs to exist:
        # the producer quantises with the consumer's scale and writes the integer levels in the consumer's layout
        made_by = {e: op for op in kept for e in op.outputs}
        readers = {}
        for op in kept:
            for e in op.inputs:
                if e:
                    readers.setdefault(e, []).append(op)
        # a producer serves one reader: stride-1 readers first (they read every pixel; a 1 x 1 stride-2 reader's own
        # layout pass only touches a quarter of them)
        by_preference = sorted(kept, key=lambda op: 0 if list(getattr(op, "strides", [1, 1])) == [1, 1] else 1)
        for consumer in by_preference:
            if kind(consumer) != "QLinearConv" or not consumer.from_float:
                continue
            edge = consumer.inputs[0]
            producer_node = made_by.get(edge)
            if (producer_node is None or kind(producer_node) != "QLinearConv" or producer_node.next_conv is not None
                    or producer_node.dtype != "float32" or len(producer_node.outputs) != 1):
                continue
            shared = len(readers.get(edge, [])) != 1 or edge in self.output_name    # the float32 values are needed elsewhere too
            w_codes = self.initializers[consumer.inputs[3]]
            if self.initializers[producer_node.inputs[3]].size[0] % 8:
                continue                                    # the levels layout wants channel groups of eight
            producer_node.next_conv = dict(pads=list(consumer.pads), strides=list(consumer.strides), dilations=list(consumer.dilations),
                                           kernel=[int(w_codes.size[2]), int(w_codes.size[3])])
            producer_node.inputs = (list(producer_node.inputs) + ["", ""])[:7] + [consumer.inputs[1], consumer.inputs[2]]
            consumer.levels_in = True
            if shared:                                      # second output: the levels; the float32 edge stays for the others
                producer_node.also_float = True
                producer_node.outputs = [edge, edge + ".levels"]
                consumer.inputs = [edge + ".levels"] + list(consumer.inputs[1:])
        # fourth pass: a float32 edge that only fused convolutions touch (as activations to quantise, or as the
        # residual) never meets the ABI's NCHW rule, so it is kept channels-last -- the order the tensor-core
        # kernel produces and consumes (contiguous 64-byte pieces per pixel instead of one element per plane)
        readers = {}
        for op in kept:
            for slot, e in enumerate(op.inputs):
                if e:
                    readers.setdefault(e, []).append((op, slot))
        for op in kept if channels_last else ():
            if kind(op) != "QLinearConv" or op.dtype != "float32" or (op.next_conv is not None and not op.also_float):
                continue
            edge = op.outputs[0]
            users = readers.get(edge, [])
            fused_only = all(kind(u) == "QLinearConv" and ((slot == 0 and u.from_float and not u.levels_in) or slot == 6) for u, slot in users)
            if not users or not fused_only or edge in self.output_name or self.initializers[op.inputs[3]].size[0] % 4:
                continue
            op.y_channels_last = True
            for u, slot in users:
                if slot == 0:
                    u.x_channels_last = True
                else:
                    u.residual_channels_last = True
        kept = self._fuse_elementwise_qdq(kept)
        g = Graph(kept, list(self.input_name), list(self.output_name), self.model_name, self.initializers)
        g._resident = self._resident
        if hasattr(self, "macs_per_image"):
            g.macs_per_image = self.macs_per_image
        return g

    def _fuse_elementwise_qdq(self, nodes):
        """Q/DQ chains that no convolution absorbed, fused with their elementwise neighbours:

            DequantizeLinear(a), DequantizeLinear(b) -> Add [-> Relu] -> QuantizeLinear      one DequantAddQuant node
            QuantizeLinear -> DequantizeLinear (same scale and zero point)                   one QuantizeDequantize node

        A chain is taken only when its inner edges have no other reader and are not graph outputs (the codes of a
        Q -> DQ pair may have other readers: the fused node then writes them as a second output)."""
        from .fused_ops import DequantAddQuant, QuantizeDequantize
        kind = lambda op: type(op).__name__
        made_by = {e: op for op in nodes for e in op.outputs}
        readers: Dict[str, list] = {}
        for op in nodes:
            for e in op.inputs:
                if e:
                    readers.setdefault(e, []).append(op)
        inner = lambda e: len(readers.get(e, [])) == 1 and e not in self.output_name
        one = lambda name: name in self.initializers and self.initializers[name].data_size == 1
        gone, replaced = set(), {}
        for add in nodes:
            if kind(add) != "ADD" or (add.dtype or "float32") != "float32" or len(add.inputs) != 2 or add.inputs[0] == add.inputs[1]:
                continue
            dqs = [made_by.get(e) for e in add.inputs]
            if not all(d is not None and kind(d) == "DequantizeLinear" and (d.dtype or "float32") == "float32" and inner(d.outputs[0])
                       and d.name not in gone and all(one(n) for n in d.inputs[1:3]) for d in dqs):
                continue
            tail, relu = add, False
            if not inner(add.outputs[0]):
                continue
            nxt = readers[add.outputs[0]][0]
            if kind(nxt) == "RELU" and (nxt.dtype or "float32") == "float32" and inner(nxt.outputs[0]):
                tail, relu, nxt = nxt, True, readers[nxt.outputs[0]][0]
            if kind(nxt) != "QuantizeLinear" or nxt.dtype not in ("int8", "uint8") or not all(one(n) for n in nxt.inputs[1:3]):
                continue
            if any(self.initializers[d.inputs[2]].dtype not in ("int8", "uint8") for d in dqs) or self.initializers[nxt.inputs[2]].dtype != nxt.dtype:
                continue
            node = DequantAddQuant(list(dqs[0].inputs[:3]) + list(dqs[1].inputs[:3]) + list(nxt.inputs[1:3]), [nxt.outputs[0]], relu, nxt.dtype)
            node.name = add.name + ".fused"
            gone.update(d.name for d in dqs)
            gone.update((add.name, nxt.name))
            if relu:
                gone.add(tail.name)
            replaced[nxt.name] = node                       # the fused node sits where the chain ended
        for q in nodes:
            if kind(q) != "QuantizeLinear" or q.name in gone or q.dtype not in ("int8", "uint8", "float8_e4m3", "float8_e5m2"):
                continue
            dq = next((r for r in readers.get(q.outputs[0], []) if kind(r) == "DequantizeLinear" and r.inputs[0] == q.outputs[0]
                       and r.inputs[1:3] == q.inputs[1:3] and (r.dtype or "float32") == "float32" and r.name not in gone), None)
            if dq is None:
                continue
            scale = self.initializers.get(q.inputs[1])
            # DequantizeLinear has no axis: the pair is the same function for every element only when the scale is one
            # value or already shaped for plain broadcasting
            if scale is None or not (scale.data_size == 1 or len(scale.size) != 1):
                continue
            shared = not inner(q.outputs[0])
            node = QuantizeDequantize(list(q.inputs[:3]), [dq.outputs[0]] + ([q.outputs[0]] if shared else []), q.axis, q.dtype, "float32", shared)
            node.name = q.name + ".fused"
            gone.update((q.name, dq.name))
            replaced[q.name] = node                         # where the QuantizeLinear stood: before every reader of the codes
        out = []
        for op in nodes:
            if op.name in replaced:
                out.append(replaced[op.name])
            elif op.name not in gone:
                out.append(op)
        return out

    def make_resident(self) -> None:
        """Upload every initializer once; later calls of ``forward`` reuse the device copies."""
        if not self._resident:
            for t in self.initializers.values():
                t.to_device()
            self._resident = True

    def plan(self, *inputs):
        """Records one forward pass on ``inputs`` as a list of library calls (``nn.plan.GraphPlan``): later runs
        replay that list -- or, after ``capture()``, launch one CUDA graph -- instead of walking the nodes."""
        from .plan import GraphPlan
        return GraphPlan(self, inputs)

    def forward(self, *inputs):
        """Runs the graph on device-resident edges and returns the output tensor (or a tuple of
        them).  Intermediate edges are dropped as soon as their last consumer has run."""
        if len(inputs) != len(self.input_name):
            raise ValueError(f"graph takes {len(self.input_name)} inputs, got {len(inputs)}")
        self.make_resident()
        edges = dict(self.initializers)
        for name, value in zip(self.input_name, inputs):
            edges[name] = value.to_device() if hasattr(value, "to_device") else value
        left = dict(self.consumers)
        keep = set(self.output_name) | set(self.initializers)
        for op in self.ops.values():
            args = [edges[e] if e else None for e in op.inputs]
            while args and args[-1] is None:
                args.pop()
            result = op.forward(*args)["tensor"]
            if len(op.outputs) == 1:
                edges[op.outputs[0]] = result
            else:
                for edge, value in zip(op.outputs, result):
                    edges[edge] = value
            for e in op.inputs:
                if e and e not in keep:
                    left[e] -= 1
                    if left[e] == 0:
                        edges.pop(e, None)
        outs = tuple(edges[e] for e in self.output_name)
        return outs[0] if len(outs) == 1 else outs


# ---------------------------------------------------------------------------------------------------
# builders
# ---------------------------------------------------------------------------------------------------
def _tensor(array, dtype):
    from . import Tensor
    array = np.ascontiguousarray(array)
    return Tensor(*array.shape, dtype=dtype, data=array)


def small_cnn(seed: int = 0):
    """Conv 3->16 k3 p1 -> Relu -> MaxPool 2x2 -> Flatten -> Gemm 4096->10 -> Softmax, plus the side
    branch Add/Sub/Mul with a [16,1,1] tensor, Div by a [16,1,1] tensor, Abs, Cos on the conv output.
    Returns (graph, x) with x the seeded float32 [1,3,32,32] input; outputs: ("prob", "side")."""
    from . import Operators as ops
    rng = np.random.default_rng(seed)
    f32 = "float32"
    x = rng.standard_normal((1, 3, 32, 32)).astype(np.float32)
    init = {
        "conv.w": _tensor(rng.normal(0, 0.1, (16, 3, 3, 3)).astype(np.float32), f32),
        "conv.b": _tensor(np.zeros(16, np.float32), f32),
        "fc.w": _tensor(rng.normal(0, 0.02, (10, 4096)).astype(np.float32), f32),
        "fc.b": _tensor(rng.normal(0, 1, 10).astype(np.float32), f32),
        "t": _tensor(rng.uniform(-1, 1, (16, 1, 1)).astype(np.float32), f32),
        "d": _tensor(rng.uniform(0.5, 2, (16, 1, 1)).astype(np.float32), f32),
    }
    nodes = [
        ops.Conv(["x", "conv.w", "conv.b"], ["conv"], pads=[1, 1, 1, 1], strides=[1, 1], dilations=[1, 1], group=1, dtype=f32),
        ops.RELU(["conv"], ["relu"], dtype=f32),
        ops.MaxPool(["relu"], ["pool"], kernel_shape=[2, 2], pads=[0, 0, 0, 0], strides=[2, 2], dtype=f32),
        ops.Flatten(["pool"], ["flat"], axis=1, dtype=f32),
        ops.Gemm(["flat", "fc.w", "fc.b"], ["logits"], alpha=1.0, beta=1.0, transA=0, transB=1, dtype=f32),
        ops.Softmax(["logits"], ["prob"], axis=1, dtype=f32),
        ops.ADD(["conv", "t"], ["s1"], dtype=f32),
        ops.SUB(["s1", "t"], ["s2"], dtype=f32),
        ops.MUL(["s2", "t"], ["s3"], dtype=f32),
        ops.DIV(["s3", "d"], ["s4"], dtype=f32),
        ops.ABS(["s4"], ["s5"], dtype=f32),
        ops.COS(["s5"], ["side"], dtype=f32),
    ]
    return Graph(nodes, "x", ["prob", "side"], "small_cnn", init), _tensor(x, f32)


class _QdqBuilder:
    """Accumulates nodes and initializers of a QDQ convolutional network.  Activation scales come
    from a calibration run: the builder executes each new float32 edge eagerly on a small seeded
    batch, so the scale of a convolution input is amax / 127 of the very tensor it will quantise."""

    def __init__(self, rng, calibration):
        from . import Operators as ops
        self.ops_module = ops
        self.rng = rng
        self.nodes: List[object] = []
        self.init: Dict[str, object] = {}
        self.live = {"x": calibration}          # calibration values of the float32 edges
        self.counter = 0
        self.macs_per_image = 0                 # multiply-accumulates of the convolutions and the classifier

    def _name(self, stem):
        self.counter += 1
        return f"{stem}{self.counter}"

    def _run(self, node, *edge_names):
        args = [self.live[e] if e in self.live else self.init[e] for e in edge_names]
        return node.forward(*args)["tensor"]

    def add(self, node, calibrate: bool = True):
        self.nodes.append(node)
        if calibrate:
            self.live[node.outputs[0]] = self._run(node, *[e for e in node.inputs if e])
        return node.outputs[0]

    def qdq_conv(self, x_edge, c_in, c_out, k, stride, pad, relu=True):
        """QuantizeLinear -> DequantizeLinear -> Conv (weights through DequantizeLinear) [-> Relu]."""
        ops, f32 = self.ops_module, "float32"
        tag = self._name("conv")
        fan_in = c_in * k * k
        w = self.rng.normal(0, np.sqrt(2.0 / fan_in), (c_out, c_in, k, k)).astype(np.float32)
        w_scale = (np.abs(w).reshape(c_out, -1).max(axis=1) / 127.0).astype(np.float32)
        w_q = np.clip(np.rint(w / w_scale.reshape(-1, 1, 1, 1)), -127, 127).astype(np.int8)
        amax = float(np.abs(self.live[x_edge].numpy()).max())
        x_scale = np.float32(max(amax, 1e-6) / 127.0)
        self.init[f"{tag}.x_scale"] = _tensor(np.array([x_scale], np.float32), f32)
        self.init[f"{tag}.x_zero"] = _tensor(np.zeros(1, np.int8), "int8")
        self.init[f"{tag}.w_q"] = _tensor(w_q, "int8")
        self.init[f"{tag}.w_scale"] = _tensor(w_scale.reshape(c_out, 1, 1, 1), f32)
        self.init[f"{tag}.w_zero"] = _tensor(np.zeros((c_out, 1, 1, 1), np.int8), "int8")
        self.init[f"{tag}.b"] = _tensor(self.rng.normal(0, 0.05, c_out).astype(np.float32), f32)
        q = self.add(ops.QuantizeLinear([x_edge, f"{tag}.x_scale", f"{tag}.x_zero"], [f"{tag}.xq"], axis=1, dtype="int8"))
        dq = self.add(ops.DequantizeLinear([q, f"{tag}.x_scale", f"{tag}.x_zero"], [f"{tag}.xdq"], dtype=f32))
        wdq = self.add(ops.DequantizeLinear([f"{tag}.w_q", f"{tag}.w_scale", f"{tag}.w_zero"], [f"{tag}.wdq"], dtype=f32))
        y = self.add(ops.Conv([dq, wdq, f"{tag}.b"], [f"{tag}.y"], pads=[pad] * 4, strides=[stride, stride], dilations=[1, 1],
                              group=1, dtype=f32))
        for edge in (q, dq, wdq):
            self.live.pop(edge, None)
        _, _, oh, ow = self.live[y].data.shape
        self.macs_per_image += oh * ow * c_out * c_in * k * k
        if relu:
            y = self.add(ops.RELU([y], [f"{tag}.relu"], dtype=f32))
        return y


def qdq_resnet50(batch: int = 256, seed: int = 0, image: int = 224, stages: Sequence[int] = (3, 4, 6, 3),
                 widths: Sequence[int] = (64, 128, 256, 512), classes: int = 1000, calibration_batch: int = 2):
    """Builds the QDQ ResNet-50-shaped graph and its seeded input.  Returns (graph, x) with
    x float32 [batch, 3, image, image] ~ N(0, 1); the graph output is the [batch, classes] softmax.
    The stride of each stage sits on its 3x3 convolution; BatchNorm is folded (convolutions carry
    a bias).  Smaller ``image`` / ``stages`` / ``widths`` give the same structure at test size."""
    from . import Operators as ops
    rng = np.random.default_rng(seed)
    f32 = "float32"
    x = rng.standard_normal((batch, 3, image, image)).astype(np.float32)
    b = _QdqBuilder(rng, _tensor(x[:max(1, min(calibration_batch, batch))], f32).to_device())
    stem = widths[0]
    y = b.qdq_conv("x", 3, stem, 7, 2, 3)
    y = b.add(ops.MaxPool([y], ["stem.pool"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2], dtype=f32))
    c_in = stem
    for stage, (blocks, width) in enumerate(zip(stages, widths)):
        for block in range(blocks):
            stride = 2 if (block == 0 and stage > 0) else 1
            c_out = width * 4
            shortcut = y
            if block == 0:
                shortcut = b.qdq_conv(y, c_in, c_out, 1, stride, 0, relu=False)
            z = b.qdq_conv(y, c_in, width, 1, 1, 0)
            z = b.qdq_conv(z, width, width, 3, stride, 1)
            z = b.qdq_conv(z, width, c_out, 1, 1, 0, relu=False)
            tag = f"s{stage}b{block}"
            z = b.add(ops.ADD([z, shortcut], [f"{tag}.sum"], dtype=f32))
            y = b.add(ops.RELU([z], [f"{tag}.out"], dtype=f32))
            c_in = c_out
    side = b.live[y].data.shape[2]
    y = b.add(ops.MaxPool([y], ["head.pool"], kernel_shape=[side, side], pads=[0, 0, 0, 0], strides=[1, 1], dtype=f32))
    y = b.add(ops.Flatten([y], ["head.flat"], axis=1, dtype=f32))
    b.init["fc.w"] = _tensor(rng.normal(0, 0.01, (classes, c_in)).astype(np.float32), f32)
    b.init["fc.b"] = _tensor(np.zeros(classes, np.float32), f32)
    y = b.add(ops.Gemm([y, "fc.w", "fc.b"], ["logits"], alpha=1.0, beta=1.0, transA=0, transB=1, dtype=f32))
    b.add(ops.Softmax([y], ["prob"], axis=1, dtype=f32))
    graph = Graph(b.nodes, "x", ["prob"], "qdq_resnet50", b.init)
    graph.macs_per_image = b.macs_per_image + classes * c_in
    return graph, _tensor(x, f32)
