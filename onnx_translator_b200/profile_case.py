"""Run ONE operator case a few times on the current GPU and print its event-timed throughput.

Small, self-contained command lines for profilers (one kernel, few launches, bounded memory):

    python -m onnx_translator_b200.profile_case --op add --dtype float32 --rows 16 --b row --iters 3
    python -m onnx_translator_b200.profile_case --op quantize --out int8 --rows 2048 --iters 3
    python -m onnx_translator_b200.profile_case --op gemm --dtype bfloat16 --m 4096 --n 4096 --k 4096

Elementwise cases use A[rows,512,1024] with B of shape [1,512,1] (row), [1024] (vec) or full;
quantize / dequantize use X[rows,8192]; softmax X[rows,1000]; maxpool X[rows,64,112,112] k3 s2 p1.
"""
from __future__ import annotations

import argparse
import time

import numpy as np

from . import capi
from .device import DeviceArray
from .capi import CConvParams, CPoolParams
import ctypes

ITEM = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "int8": 1, "uint8": 1, "float64": 8,
        "float8_e4m3": 1, "float8_e5m2": 1, "int16": 2, "int64": 8, "int4": 1}


def _rand(rng, shape, dtype, lo=-100, hi=100):
    st = capi.DTYPE_TO_NUMPY[dtype]
    if dtype in ("int8", "int4"):
        return rng.integers(-7, 8, shape).astype(st)
    if dtype in ("uint8", "float8_e4m3", "float8_e5m2"):
        return rng.integers(0, 120, shape).astype(st)
    if dtype in ("int16", "int32", "int64"):
        return rng.integers(-1000, 1001, shape).astype(st)
    v = rng.uniform(lo, hi, shape).astype(np.float32)
    if dtype == "bfloat16":
        u = v.view(np.uint32).astype(np.uint64)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return v.astype(st)


def _ints(vals):
    arr = (ctypes.c_int * len(vals))(*vals)
    return arr, ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", required=True)
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--b-dtype", default=None)
    ap.add_argument("--out", default=None)
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--b", default="row", choices=("row", "vec", "full"))
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--channels", type=int, default=256)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--ksize", type=int, default=1)
    args = ap.parse_args()

    lib = capi.load()
    lib.init_cos_lut()
    capi.check(lib)
    rng = np.random.default_rng(0)
    dt = args.dtype
    out_dt = args.out or dt
    flops = 0
    keep = []
    if args.op in ("add", "sub", "mul", "div"):
        shape = (args.rows, 512, 1024)
        bshape = {"row": (1, 512, 1), "vec": (1024,), "full": shape}[args.b]
        bdt = args.b_dtype or dt
        a = DeviceArray.from_numpy(_rand(rng, shape, dt), dt)
        b = DeviceArray.from_numpy(_rand(rng, bshape, bdt, 0.5, 100), bdt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, b.handle, o.handle)
        n = a.size
        nbytes = n * (ITEM[dt] + ITEM[out_dt]) + b.size * ITEM[bdt]
    elif args.op in ("relu", "abs", "cos"):
        shape = (args.rows, 512, 1024)
        a = DeviceArray.from_numpy(_rand(rng, shape, dt, -10, 10), dt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, o.handle)
        nbytes = a.size * (ITEM[dt] + ITEM[out_dt])
    elif args.op in ("exp", "log", "sqrt", "sigmoid", "tanh", "neg", "reciprocal", "ceil", "floor", "sin", "tan", "atan", "softplus", "softsign",
                     "hard_swish", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "round", "erf", "gelu", "cast"):
        shape = (args.rows, 512, 1024)
        a = DeviceArray.from_numpy(_rand(rng, shape, dt, -3, 3), dt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, o.handle)
        nbytes = a.size * (ITEM[dt] + ITEM[out_dt])
    elif args.op == "dynamic_quantize":
        # range pass + quantise pass over float32 [rows, 8192]: x read twice, uint8 codes written once
        shape = (args.rows, 8192)
        x = DeviceArray.from_numpy(rng.standard_normal(shape).astype(np.float32), "float32")
        o = DeviceArray.empty(shape, "uint8")
        sc, zp = DeviceArray.empty((1,), "float32"), DeviceArray.empty((1,), "uint8")
        call = lambda: lib.dynamic_quantize_linear_forward(x.handle, o.handle, sc.handle, zp.handle)
        nbytes = x.size * 9
        dt, out_dt = "float32", "uint8"
    elif args.op == "batch_norm":
        shape = (args.batch, args.channels, args.hw, args.hw)
        x = DeviceArray.from_numpy(rng.standard_normal(shape).astype(np.float32), "float32")
        o = DeviceArray.empty(shape, "float32")
        ps = [DeviceArray.from_numpy(v.astype(np.float32), "float32") for v in (rng.normal(1, 0.1, args.channels), rng.normal(0, 0.1, args.channels),
                                                                                rng.normal(0, 0.1, args.channels), rng.uniform(0.5, 2, args.channels))]
        keep = ps
        call = lambda: lib.batch_norm_forward(x.handle, ps[0].handle, ps[1].handle, ps[2].handle, ps[3].handle, o.handle, ctypes.c_float(1e-5))
        nbytes = x.size * 8
        dt = out_dt = "float32"
    elif args.op == "global_average_pool":
        shape = (args.batch, args.channels, args.hw, args.hw)
        x = DeviceArray.from_numpy(rng.standard_normal(shape).astype(np.float32), "float32")
        o = DeviceArray.empty(shape[:2] + (1, 1), "float32")
        call = lambda: lib.global_average_pool_forward(x.handle, o.handle)
        nbytes = x.size * 4
        dt = out_dt = "float32"
    elif args.op in ("quantize", "dequantize"):
        shape = (args.rows, 8192)
        if args.op == "quantize":
            out_dt = args.out or "int8"
            x = DeviceArray.from_numpy(rng.standard_normal(shape).astype(np.float32), "float32")
            zdt = out_dt if out_dt in ("int8", "uint8") else "int8"
        else:
            dt = args.dtype if args.dtype != "float32" else "int8"
            out_dt = args.out or "float32"
            x = DeviceArray.from_numpy(_rand(rng, shape, dt), dt)
            zdt = dt if dt in ("int8", "uint8") else "int8"
        if args.b == "vec":
            s = DeviceArray.from_numpy(rng.uniform(0.01, 0.05, (1, 8192)).astype(np.float32), "float32")
            z = DeviceArray.from_numpy(rng.integers(0, 9, (1, 8192)).astype(capi.DTYPE_TO_NUMPY[zdt]), zdt)
        else:
            s = DeviceArray.from_numpy(np.array([0.02], np.float32), "float32")
            z = DeviceArray.from_numpy(np.array([0]).astype(capi.DTYPE_TO_NUMPY[zdt]), zdt)
        o = DeviceArray.empty(shape, out_dt)
        fn = lib.quantize_linear_forward if args.op == "quantize" else lib.dequantize_linear_forward
        call = lambda: fn(x.handle, s.handle, z.handle, o.handle)
        nbytes = x.size * (ITEM[x.dtype_name] + ITEM[out_dt])
    elif args.op == "softmax":
        shape = (args.rows, 1000)
        x = DeviceArray.from_numpy(_rand(rng, shape, dt, -10, 10), dt)
        o = DeviceArray.empty(shape, out_dt)
        call = lambda: lib.softmax_forward(x.handle, o.handle, 1)
        nbytes = x.size * (ITEM[dt] + ITEM[out_dt])
    elif args.op == "maxpool":
        shape = (args.rows, 64, 112, 112)
        x = DeviceArray.from_numpy(_rand(rng, shape, dt), dt)
        o = DeviceArray.empty((args.rows, 64, 56, 56), out_dt)
        keep = [_ints([1, 1, 1, 1]), _ints([2, 2]), _ints([1, 1]), _ints([3, 3])]
        prm = CPoolParams(keep[0][1], keep[1][1], keep[2][1], keep[3][1])
        call = lambda: lib.max_pool_forward(x.handle, o.handle, ctypes.byref(prm))
        nbytes = x.size * ITEM[dt] + o.size * ITEM[out_dt]
    elif args.op == "gemm":
        a = DeviceArray.from_numpy(_rand(rng, (args.m, args.k), dt, -0.05, 0.05), dt)
        b = DeviceArray.from_numpy(_rand(rng, (args.n, args.k), dt, -0.05, 0.05), dt)
        c = DeviceArray.from_numpy(rng.standard_normal((1, args.n)).astype(np.float32), "float32")
        o = DeviceArray.empty((args.m, args.n), out_dt)
        call = lambda: lib.gemm_forward(a.handle, b.handle, c.handle, o.handle, 1.0, 1.0, 0, 1)
        nbytes = a.size * ITEM[dt] + b.size * ITEM[dt] + o.size * ITEM[out_dt]
        flops = 2.0 * args.m * args.n * args.k
    elif args.op == "conv":
        n_, c_, hw = args.batch, args.channels, args.hw
        x = DeviceArray.from_numpy(_rand(rng, (n_, c_, hw, hw), dt, -1, 1), dt)
        w = DeviceArray.from_numpy(_rand(rng, (c_, c_, 3, 3), dt, -0.05, 0.05), dt)
        o = DeviceArray.empty((n_, c_, hw, hw), out_dt)
        keep = [_ints([1, 1, 1, 1]), _ints([1, 1]), _ints([1, 1])]
        prm = CConvParams(keep[0][1], keep[1][1], keep[2][1], 1)
        call = lambda: lib.conv2d_forward(x.handle, w.handle, None, o.handle, ctypes.byref(prm))
        nbytes = x.size * ITEM[dt] + w.size * ITEM[dt] + o.size * ITEM[out_dt]
        flops = 2.0 * n_ * hw * hw * c_ * c_ * 9
    elif args.op == "qconv":
        # one Q -> DQ -> Conv(DQ(W)) -> Relu chain in one call: float32 [batch, channels, hw, hw] -> [batch, n, hw, hw],
        # ksize x ksize filters (stride 1, "same" padding)
        n_, c_, hw, ks, m_ = args.batch, args.channels, args.hw, args.ksize, args.n
        x = DeviceArray.from_numpy(rng.standard_normal((n_, c_, hw, hw)).astype(np.float32), "float32")
        wq = DeviceArray.from_numpy(rng.integers(-127, 128, (m_, c_, ks, ks)).astype(np.int8), "int8")
        ws = DeviceArray.from_numpy(rng.uniform(0.005, 0.02, m_).astype(np.float32), "float32")
        sx = DeviceArray.from_numpy(np.array([0.03], np.float32), "float32")
        zx = DeviceArray.from_numpy(np.zeros(1, np.int8), "int8")
        o = DeviceArray.empty((n_, m_, hw, hw), "float32")
        pad = ks // 2
        keep = [_ints([pad] * 4), _ints([1, 1]), _ints([1, 1])]
        prm = CConvParams(keep[0][1], keep[1][1], keep[2][1], 1)
        call = lambda: lib.tops_qdq_conv_forward(x.handle, sx.handle, zx.handle, wq.handle, ws.handle, None, None, o.handle,
                                                 ctypes.byref(prm), 1)
        nbytes = x.size * 4 + o.size * 4
        flops = 2.0 * n_ * hw * hw * m_ * c_ * ks * ks
        dt = out_dt = "float32"
    elif args.op == "qdq_resnet50":
        # the QDQ ResNet-50-shaped graph through Graph.fused(); --batch images of 224 x 224
        from . import nn
        graph, x_host = nn.qdq_resnet50(batch=args.batch, seed=0)
        fused = graph.fused()
        xd = x_host.to_device()
        keep = [graph, fused, xd]
        call = lambda: fused.forward(xd)
        nbytes = 0
        flops = 2.0 * graph.macs_per_image * args.batch
        dt = out_dt = "float32"
    else:
        raise SystemExit(f"unknown op {args.op}")

    import torch
    stream = torch.cuda.ExternalStream(lib.tops_get_stream())
    for _ in range(args.warmup):
        call()
    lib.tops_sync()
    capi.check(lib)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.iters + 1)]
    ev[0].record(stream)
    for i in range(args.iters):
        call()
        ev[i + 1].record(stream)
    lib.tops_sync()
    torch.cuda.synchronize()
    capi.check(lib)
    ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.iters)]
    best = min(ms)
    msg = f"{args.op} {dt}->{out_dt}: {best:.4f} ms best of {args.iters} ({np.mean(ms):.4f} mean), {nbytes / 1e9 / (best / 1e3):.1f} GB/s algorithmic"
    if flops:
        msg += f", {flops / 1e12 / (best / 1e3):.1f} TFLOP/s"
    print(msg)


if __name__ == "__main__":
    main()
