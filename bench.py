#!/usr/bin/env python
"""Benchmark of the tensor_ops hot path on B200.

Workload (N = 1): the broadcast elementwise sweep -- Add/Sub/Mul/Div of A[64,512,1024] with B of
shape [1,512,1], [1024] and [64,512,1024] over seven dtype pairs, Relu/Abs on the same shape over
the five A dtypes, Cos on float32.  One "step" is one pass over all 95 operator calls.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is algorithmic GB/s of the whole job with inputs resident in HBM,
`e2e` the same metric through the C ABI with pinned HOST buffers (H2D of both operands and D2H of
the result inside the timed region; two streams so uploads overlap downloads), `roofline` the achieved bandwidth of the dominant kernel
family against the measured HBM copy peak, `cpu_baseline` the reference C library timed on this
machine's cores on a bounded slab of the same sweep.

Under torchrun every rank runs the same sweep on its own GPU (weak scaling, no data-path
collective); times are device-measured and the maximum over ranks is used.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FULL_ROWS = 64
MID, INNER = 512, 1024
BINARY_OPS = ("add", "sub", "mul", "div")
# (A dtype, B dtype, output dtype): the reference's promotion gives float64 for int32 + float16
DTYPE_PAIRS = (("float32", "float32", "float32"), ("float16", "float16", "float16"),
               ("bfloat16", "bfloat16", "bfloat16"), ("int32", "int32", "int32"), ("int8", "int8", "int8"),
               ("int8", "float32", "float32"), ("int32", "float16", "float64"))
UNARY_DTYPES = ("float32", "float16", "bfloat16", "int32", "int8")
ITEM = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "int8": 1, "float64": 8}
STORAGE = {"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16, "int32": np.int32,
           "int8": np.int8, "float64": np.float64}


def b_shapes(rows):
    return {"row": (1, MID, 1), "vec": (INNER,), "full": (rows, MID, INNER)}


# ---- synthetic data (seeded; value distributions of the benchmark configuration) ---------------------
def _bf16(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def make_a(rng, rows, dtype):
    shape = (rows, MID, INNER)
    if dtype == "int8":
        return rng.integers(-11, 12, shape).astype(np.int8)           # products stay inside int8
    if dtype == "int32":
        return rng.integers(-1000, 1001, shape).astype(np.int32)
    v = rng.uniform(-100, 100, shape).astype(np.float32)
    return v if dtype == "float32" else (v.astype(np.float16) if dtype == "float16" else _bf16(v))


def make_b(rng, shape, dtype, divisor):
    if dtype in ("int8", "int32"):
        hi = 11 if dtype == "int8" else 1000
        v = rng.integers(1 if divisor else -hi, hi + 1, shape)
        if divisor:
            v = v * rng.choice([-1, 1], shape)
        return v.astype(STORAGE[dtype])
    v = rng.uniform(0.5, 100, shape) * rng.choice([-1, 1], shape) if divisor else rng.uniform(-100, 100, shape)
    v = v.astype(np.float32)
    return v if dtype == "float32" else (v.astype(np.float16) if dtype == "float16" else _bf16(v))


def sweep_plan(rows):
    """List of launches in an order that never uses the same big tensor twice in a row."""
    n = rows * MID * INNER
    plan = []
    for op in BINARY_OPS:
        for bname, bshape in b_shapes(rows).items():
            for a_dt, b_dt, o_dt in DTYPE_PAIRS:
                nbytes = n * (ITEM[a_dt] + ITEM[o_dt]) + (n * ITEM[b_dt] if bname == "full" else int(np.prod(bshape)) * ITEM[b_dt])
                plan.append(dict(kind="binary", op=op, a=a_dt, b=b_dt, o=o_dt, bname=bname, divisor=(op == "div"), bytes=nbytes,
                                 label=f"{op}[{bname}] {a_dt},{b_dt}->{o_dt}"))
    for op in ("relu", "abs"):
        for dt in UNARY_DTYPES:
            plan.append(dict(kind="unary", op=op, a=dt, o=dt, bytes=n * 2 * ITEM[dt], label=f"{op} {dt}"))
    plan.append(dict(kind="unary", op="cos", a="float32", o="float32", bytes=n * 8, label="cos float32"))
    return plan


def host_inputs(rows, seed=0):
    rng = np.random.default_rng(seed)
    a = {dt: make_a(rng, rows, dt) for dt in UNARY_DTYPES}
    a_cos = rng.uniform(-10, 10, (rows, MID, INNER)).astype(np.float32)
    b = {}
    for bname, bshape in b_shapes(rows).items():
        for dt in ("float32", "float16", "bfloat16", "int32", "int8"):
            for divisor in (False, True):
                b[(bname, dt, divisor)] = make_b(rng, bshape, dt, divisor)
    return a, a_cos, b


# ---- clocks -----------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while running."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
                 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
                 0x100: "display_clock_setting"}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self.ok:
            self.thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.ok:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ---- our arm ------------------------------------------------------------------------------------------
def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def run_ours(args):
    import torch
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (there is no CPU fallback; use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = capi.load()
    if lib.tops_set_device(local):
        capi.check(lib)
    lib.init_cos_lut()
    stream = torch.cuda.ExternalStream(lib.tops_get_stream(), device=local)

    rows = FULL_ROWS
    plan = sweep_plan(rows)
    a_host, a_cos_host, b_host = host_inputs(rows, seed=rank)
    dev_a = {dt: DeviceArray.from_numpy(v, dt) for dt, v in a_host.items()}
    dev_cos = DeviceArray.from_numpy(a_cos_host, "float32")
    dev_b = {k: DeviceArray.from_numpy(v, k[1]) for k, v in b_host.items()}
    dev_out = {dt: DeviceArray.empty((rows, MID, INNER), dt) for dt in ("float32", "float16", "bfloat16", "int32", "int8", "float64")}
    capi.check(lib)

    def fn_of(item):
        return getattr(lib, item["op"] + "_forward")

    def launch(item):
        out = dev_out[item["o"]].handle
        if item["kind"] == "binary":
            fn_of(item)(dev_a[item["a"]].handle, dev_b[(item["bname"], item["b"], item["divisor"])].handle, out)
        else:
            src = dev_cos if item["op"] == "cos" else dev_a[item["a"]]
            fn_of(item)(src.handle, out)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        lib.tops_sync()
        torch.cuda.synchronize()

    # -- device-resident timing ------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        for item in plan:
            launch(item)
    capi.check(lib)
    n_launch = len(plan)
    # the timed region: K steps back to back, one event before and one after
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with ClockSampler(local) as clocks:
        with torch.cuda.stream(stream):
            t_begin.record(stream)
            for s in range(args.steps):
                for item in plan:
                    launch(item)
            t_end.record(stream)
        barrier()
    capi.check(lib)
    step_ms = t_begin.elapsed_time(t_end) / args.steps
    # per-launch durations (per-op table, roofline of the dominant kernel family): the same K steps
    # again with an event after every launch
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(n_launch + 1)] for _ in range(args.steps)]
    with torch.cuda.stream(stream):
        for s in range(args.steps):
            marks[s][0].record(stream)
            for i, item in enumerate(plan):
                launch(item)
                marks[s][i + 1].record(stream)
    barrier()
    capi.check(lib)
    per_launch_ms = np.zeros(n_launch)
    for s in range(args.steps):
        for i in range(n_launch):
            per_launch_ms[i] += marks[s][i].elapsed_time(marks[s][i + 1])
    per_launch_ms /= args.steps
    bytes_step = sum(item["bytes"] for item in plan)

    # -- end to end through the C ABI with pinned host buffers --------------------------------------
    pinned = {}

    def pin(arr):
        key = id(arr)
        if key not in pinned:
            ptr = lib.tops_host_alloc(arr.nbytes)
            if not ptr:
                capi.check(lib)
            ctypes.memmove(ptr, arr.ctypes.data, arr.nbytes)
            pinned[key] = ptr
        return pinned[key]

    # Several lanes, each with its own stream, device operands and pinned result buffer: the uploads of
    # some calls overlap the downloads of others (PCIe is full duplex); measured on one B200: 79 GB/s with
    # 2 lanes, 90 with 3, 92 with 4, 97 with 6.
    n_lanes = max(1, args.e2e_lanes)
    lane_streams = [torch.cuda.Stream(device=local) for _ in range(n_lanes)]
    out_pinned = [lib.tops_host_alloc(rows * MID * INNER * 8) for _ in range(n_lanes)]
    lanes = [dict(a=dev_a, cos=dev_cos, b=dev_b, out=dev_out)]
    for _ in range(1, n_lanes):
        lanes.append(dict(a={dt: DeviceArray.empty(v.shape, dt) for dt, v in a_host.items()},
                          cos=DeviceArray.empty(a_cos_host.shape, "float32"),
                          b={k: DeviceArray.empty(v.shape, k[1]) for k, v in b_host.items()},
                          out={dt: DeviceArray.empty((rows, MID, INNER), dt) for dt in dev_out}))
    capi.check(lib)
    h2d = d2h = 0
    e2e_items = []
    for item in plan:
        a_arr = a_cos_host if item["op"] == "cos" else a_host[item["a"]]
        ent = dict(item=item, a_ptr=pin(a_arr), a_bytes=a_arr.nbytes)
        if item["kind"] == "binary":
            b_arr = b_host[(item["bname"], item["b"], item["divisor"])]
            ent.update(b_ptr=pin(b_arr), b_bytes=b_arr.nbytes)
            h2d += b_arr.nbytes
        h2d += a_arr.nbytes
        ent["o_bytes"] = rows * MID * INNER * ITEM[item["o"]]
        d2h += ent["o_bytes"]
        e2e_items.append(ent)

    def e2e_step():
        for i, ent in enumerate(e2e_items):
            k = i % n_lanes
            lane = lanes[k]
            lib.tops_set_stream(lane_streams[k].cuda_stream)
            item = ent["item"]
            out = lane["out"][item["o"]].handle
            src = lane["cos"] if item["op"] == "cos" else lane["a"][item["a"]]
            lib.tops_upload(src.handle, ent["a_ptr"], ent["a_bytes"])
            if item["kind"] == "binary":
                bdev = lane["b"][(item["bname"], item["b"], item["divisor"])]
                lib.tops_upload(bdev.handle, ent["b_ptr"], ent["b_bytes"])
                fn_of(item)(src.handle, bdev.handle, out)
            else:
                fn_of(item)(src.handle, out)
            lib.tops_download_async(out, out_pinned[k], ent["o_bytes"])

    def e2e_sync():
        for st in lane_streams:
            st.synchronize()

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    e2e_sync()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(lane_streams[0])
    for st in lane_streams[1:]:
        st.wait_event(e0)
    for _ in range(e2e_steps):
        e2e_step()
    for st in lane_streams[1:]:
        lane_streams[0].wait_stream(st)
    e1.record(lane_streams[0])
    e2e_sync()
    lib.tops_set_stream(None)
    barrier()
    capi.check(lib)
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # -- max over ranks -----------------------------------------------------------------------------
    times = torch.tensor([step_ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    step_ms_max, e2e_ms_max = (float(t) for t in times.cpu())

    qdq_cnn = None
    if not args.no_extra:                       # every rank runs its own batch; the time is reduced inside
        try:
            qdq_cnn = qdq_cnn_throughput(lib, stream, world, local)
        except Exception as exc:
            if world > 1:
                raise                            # the ranks must stay in step
            qdq_cnn = {"error": str(exc)[:300]}

    if rank == 0:
        peak, peak_kind = peaks()
        binary_idx = [i for i, it in enumerate(plan) if it["kind"] == "binary"]
        fam_bytes = sum(plan[i]["bytes"] for i in binary_idx)
        # the family's share of a step comes from the pass with an event after every launch (events between
        # launches cost time and prevent the next kernel from being scheduled early); its duration inside the
        # timed region is that share of the un-instrumented step
        fam_share = float(sum(per_launch_ms[i] for i in binary_idx)) / float(per_launch_ms.sum())
        fam_ms = step_ms * fam_share
        achieved = fam_bytes / 1e9 / (fam_ms / 1e3)
        per_launch_ms = per_launch_ms * (step_ms / float(per_launch_ms.sum()))
        per_op = {}
        for i, it in enumerate(plan):
            per_op[it["label"]] = round(it["bytes"] / 1e9 / (per_launch_ms[i] / 1e3), 1)
        worst = sorted(per_op.items(), key=lambda kv: kv[1])[:5]
        line = {
            "metric": "per-op GB/s (aggregate over the broadcast elementwise sweep)",
            "value": round(world * bytes_step / 1e9 / (step_ms_max / 1e3), 2),
            "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(step_ms_max, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32/f16/bf16/i32/i8 elementwise (f64 where the output is float64)",
            "data": "synthetic",
            "config": {"workload": "config 2: broadcast elementwise sweep, A[64,512,1024] x B{[1,512,1],[1024],full} x 7 dtype pairs x Add/Sub/Mul/Div + Relu/Abs x 5 dtypes + Cos f32 (95 launches per step, per GPU)",
                       "l2": "inputs larger than L2 in aggregate: 1.9 GB of distinct tensors cycle between reuses of any one",
                       "timing": "K steps between two CUDA events on the launching stream; per-launch split from a second pass "
                                 "of K steps with an event after every launch, scaled to the timed step",
                       "parallelism": f"replicated sweep per GPU x{world}, no data-path collective"},
            "roofline": {"bound": "hbm", "kernel": "ew_kernel<BinaryBody> (84 launches per step)",
                         "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
                         "algorithmic_bytes_per_launch": int(fam_bytes / len(binary_idx)),
                         "launch_ms": round(fam_ms / len(binary_idx), 5), "share_of_step": round(fam_share, 4),
                         "traffic": BINARY_DRAM_BYTES_PER_LAUNCH},
            "e2e": {"value": round(world * bytes_step / 1e9 / (e2e_ms_max / 1e3), 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms_max, 3)},
            "gpu_launches": n_launch * args.steps,
            "clocks": clocks.summary(),
            "slowest_ops_GBps": dict(worst),
        }
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0) if world == 1 else None
        if qdq_cnn is not None:
            line["qdq_cnn"] = qdq_cnn
        if world == 1 and not args.no_extra:
            try:
                line["other_ops"] = other_ops(lib, stream, peak)
            except Exception as exc:                      # the headline numbers stand on their own
                line["other_ops"] = {"error": str(exc)[:200]}
        details = os.path.join(ROOT, "gpurun_out")
        try:
            os.makedirs(details, exist_ok=True)
            with open(os.path.join(details, "bench_per_op.json"), "w") as f:
                json.dump({"per_op_GBps": per_op, "per_launch_ms": [round(float(x), 5) for x in per_launch_ms]}, f, indent=1)
        except OSError:
            pass
        print(json.dumps(line), flush=True)
    for ptr in list(pinned.values()) + out_pinned:
        lib.tops_host_free(ptr)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ---- the other operators of the hot path (reported beside the headline, device-resident, event-timed) --------
def other_ops(lib, stream, hbm_peak):
    """QuantizeLinear / DequantizeLinear at 8192 x 8192, Softmax, MaxPool (GB/s and fraction of the HBM
    peak) and Gemm 8192^3 / Conv 256x256x56x56 k3 (TFLOP/s) -- the sizes of benchmark configs 3 and 4."""
    import torch
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    from onnx_translator_b200.capi import CConvParams, CPoolParams
    rng = np.random.default_rng(0)
    out = {}

    def timed(call, iters=5):
        call()
        lib.tops_sync()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        ev[0].record(stream)
        for i in range(iters):
            call()
            ev[i + 1].record(stream)
        lib.tops_sync()
        torch.cuda.synchronize()
        capi.check(lib)
        return float(np.median([ev[i].elapsed_time(ev[i + 1]) for i in range(iters)]))

    def mem(label, nbytes, call):
        ms = timed(call)
        gbs = nbytes / 1e9 / (ms / 1e3)
        out[label] = {"GBps": round(gbs, 1), "frac_hbm": round(gbs / hbm_peak, 3), "ms": round(ms, 4)}

    def ints(vals):
        arr = (ctypes.c_int * len(vals))(*vals)
        return arr, ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))

    n = 8192 * 8192
    x = DeviceArray.from_numpy(rng.standard_normal((8192, 8192)).astype(np.float32), "float32")
    s1 = DeviceArray.from_numpy(np.array([0.02], np.float32), "float32")
    s16 = DeviceArray.from_numpy(np.array([1 / 16], np.float32), "float32")
    sax = DeviceArray.from_numpy(rng.uniform(0.01, 0.05, (1, 8192)).astype(np.float32), "float32")
    z8 = DeviceArray.from_numpy(np.array([0], np.int8), "int8")
    zu8 = DeviceArray.from_numpy(np.array([128], np.uint8), "uint8")
    zax = DeviceArray.from_numpy(rng.integers(-8, 9, (1, 8192)).astype(np.int8), "int8")
    back = DeviceArray.empty((8192, 8192), "float32")
    for label, dt, sc, zp in (("int8", "int8", s1, z8), ("uint8", "uint8", s1, zu8), ("int8_per_axis", "int8", sax, zax),
                              ("float8_e4m3", "float8_e4m3", s16, z8), ("float8_e5m2", "float8_e5m2", s16, z8)):
        q = DeviceArray.empty((8192, 8192), dt)
        mem(f"quantize_f32_to_{label}", n * 5, lambda: lib.quantize_linear_forward(x.handle, sc.handle, zp.handle, q.handle))
        mem(f"dequantize_{label}_to_f32", n * 5, lambda: lib.dequantize_linear_forward(q.handle, sc.handle, zp.handle, back.handle))
        del q
    # the range-driven quantiser: x is read twice (range, then codes), the codes written once
    dq = DeviceArray.empty((8192, 8192), "uint8")
    dsc, dzp = DeviceArray.empty((1,), "float32"), DeviceArray.empty((1,), "uint8")
    mem("dynamic_quantize_f32_to_uint8", n * 9, lambda: lib.dynamic_quantize_linear_forward(x.handle, dq.handle, dsc.handle, dzp.handle))
    del dq
    # operators next to the hot path, same elementwise engine (float32 8192 x 8192)
    half = DeviceArray.empty((8192, 8192), "float16")
    mem("cast_f32_to_f16", n * 6, lambda: lib.cast_forward(x.handle, half.handle))
    del half
    lo_t, hi_t = DeviceArray.from_numpy(np.array([-1.0], np.float32), "float32"), DeviceArray.from_numpy(np.array([1.0], np.float32), "float32")
    mem("clip_f32", n * 8, lambda: lib.clip_forward(x.handle, back.handle, lo_t.handle, hi_t.handle))
    mem("max_f32_f32", n * 12, lambda: lib.max_forward(x.handle, back.handle, back.handle))
    for fn in ("exp", "sigmoid", "gelu", "sqrt"):
        mem(f"{fn}_f32", n * 8, lambda: getattr(lib, fn + "_forward")(x.handle, back.handle))
    del x, back
    bx = DeviceArray.from_numpy(rng.standard_normal((64, 256, 56, 56)).astype(np.float32), "float32")
    by = DeviceArray.empty((64, 256, 56, 56), "float32")
    bp = [DeviceArray.from_numpy(v.astype(np.float32), "float32") for v in (rng.normal(1, 0.1, 256), rng.normal(0, 0.1, 256),
                                                                              rng.normal(0, 0.1, 256), rng.uniform(0.5, 2, 256))]
    mem("batch_norm_f32_64x256x56x56", bx.size * 8, lambda: lib.batch_norm_forward(bx.handle, bp[0].handle, bp[1].handle, bp[2].handle, bp[3].handle,
                                                                                    by.handle, ctypes.c_float(1e-5)))
    gy = DeviceArray.empty((64, 256, 1, 1), "float32")
    mem("global_average_pool_f32_64x256x56x56", bx.size * 4, lambda: lib.global_average_pool_forward(bx.handle, gy.handle))
    del bx, by, gy

    sx = DeviceArray.from_numpy(rng.uniform(-10, 10, (65536, 1000)).astype(np.float32), "float32")
    sy = DeviceArray.empty((65536, 1000), "float32")
    mem("softmax_f32_65536x1000", sx.size * 8, lambda: lib.softmax_forward(sx.handle, sy.handle, 1))
    del sx, sy
    px = DeviceArray.from_numpy(rng.standard_normal((64, 64, 112, 112)).astype(np.float32), "float32")
    py = DeviceArray.empty((64, 64, 56, 56), "float32")
    keep = [ints([1, 1, 1, 1]), ints([2, 2]), ints([1, 1]), ints([3, 3])]
    pool = CPoolParams(keep[0][1], keep[1][1], keep[2][1], keep[3][1])
    mem("maxpool_f32_64x64x112x112_k3s2p1", (px.size + py.size) * 4, lambda: lib.max_pool_forward(px.handle, py.handle, ctypes.byref(pool)))
    del px, py

    def bf16(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    m = 8192
    a32 = rng.normal(0, 0.02, (m, m)).astype(np.float32)
    b32 = rng.normal(0, 0.02, (m, m)).astype(np.float32)
    bias = DeviceArray.from_numpy(rng.standard_normal((1, m)).astype(np.float32), "float32")
    flops = 2.0 * m * m * m
    import ml_dtypes
    variants = (("bf16_in_f32_out", "bfloat16", bf16, "float32"), ("bf16_in_bf16_out", "bfloat16", bf16, "bfloat16"),
                ("fp16_in_fp16_out", "float16", lambda v: v.astype(np.float16), "float16"),
                ("fp8_e4m3_in_bf16_out", "float8_e4m3", lambda v: (v * 16).astype(ml_dtypes.float8_e4m3fn).view(np.uint8), "bfloat16"))
    for label, dt, conv, odt in variants:
        a = DeviceArray.from_numpy(conv(a32), dt)
        b = DeviceArray.from_numpy(conv(b32), dt)
        y = DeviceArray.empty((m, m), odt)
        before = lib.tops_tensor_core_launches()
        ms = timed(lambda: lib.gemm_forward(a.handle, b.handle, bias.handle, y.handle, 1.0, 1.0, 0, 1))
        out[f"gemm_8192_{label}"] = {"TFLOPs": round(flops / 1e12 / (ms / 1e3), 1), "ms": round(ms, 4),
                                     "tensor_core_path": lib.tops_tensor_core_launches() > before}
        if label == "fp8_e4m3_in_bf16_out":
            # the DQ -> Gemm -> Q chain of config 4 in one call: per-tensor operand scales, e4m3 result
            sa = DeviceArray.from_numpy(np.array([1 / 16], np.float32), "float32")
            sy = DeviceArray.from_numpy(np.array([1 / 64], np.float32), "float32")
            yq = DeviceArray.empty((m, m), "float8_e4m3")
            before = lib.tops_tensor_core_launches()
            ms = timed(lambda: lib.tops_gemm_qdq_forward(a.handle, sa.handle, b.handle, sa.handle, bias.handle, sy.handle, yq.handle,
                                                         1.0, 1.0, 0, 1))
            out["gemm_8192_fp8_e4m3_dq_gemm_q_fused"] = {"TFLOPs": round(flops / 1e12 / (ms / 1e3), 1), "ms": round(ms, 4),
                                                         "tensor_core_path": lib.tops_tensor_core_launches() > before}
            del yq
        del a, b, y
    del a32, b32
    # MatMul: [8, 2048, 4096] x [4096, 4096] (one B: a single tall problem) and 64 heads of [1024, 128] x [128, 1024]
    for label, a_shape, b_shape in (("8x2048x4096_by_4096x4096", (8, 2048, 4096), (4096, 4096)), ("64x1024x128_by_64x128x1024", (64, 1024, 128), (64, 128, 1024))):
        a = DeviceArray.from_numpy(bf16(rng.normal(0, 0.02, a_shape).astype(np.float32)), "bfloat16")
        b = DeviceArray.from_numpy(bf16(rng.normal(0, 0.02, b_shape).astype(np.float32)), "bfloat16")
        y = DeviceArray.empty(a_shape[:-1] + (b_shape[-1],), "bfloat16")
        before = lib.tops_tensor_core_launches()
        ms = timed(lambda: lib.matmul_forward(a.handle, b.handle, y.handle))
        mm_flops = 2.0 * np.prod(a_shape) * b_shape[-1]
        out[f"matmul_bf16_{label}"] = {"TFLOPs": round(mm_flops / 1e12 / (ms / 1e3), 1), "ms": round(ms, 4),
                                       "tensor_core_path": lib.tops_tensor_core_launches() > before, "includes": "transposition of B"}
        del a, b, y

    cx = DeviceArray.from_numpy(bf16(rng.standard_normal((256, 256, 56, 56)).astype(np.float32)), "bfloat16")
    cw = DeviceArray.from_numpy(bf16(rng.normal(0, 0.02, (256, 256, 3, 3)).astype(np.float32)), "bfloat16")
    cy = DeviceArray.empty((256, 256, 56, 56), "bfloat16")
    keep2 = [ints([1, 1, 1, 1]), ints([1, 1]), ints([1, 1])]
    cprm = CConvParams(keep2[0][1], keep2[1][1], keep2[2][1], 1)
    before = lib.tops_tensor_core_launches()
    ms = timed(lambda: lib.conv2d_forward(cx.handle, cw.handle, None, cy.handle, ctypes.byref(cprm)), iters=3)
    out["conv_256x256x56x56_k3_bf16"] = {"TFLOPs": round(2.0 * 256 * 56 * 56 * 256 * 2304 / 1e12 / (ms / 1e3), 1), "ms": round(ms, 4),
                                         "tensor_core_path": lib.tops_tensor_core_launches() > before,
                                         "includes": "NCHW -> padded NHWC copy of X and tap-major copy of W"}
    # the same convolution with int8 weight codes and per-output-channel scales (DequantizeLinear -> Conv in one call)
    wq = DeviceArray.from_numpy(rng.integers(-127, 128, (256, 256, 3, 3)).astype(np.int8), "int8")
    ws = DeviceArray.from_numpy(rng.uniform(0.005, 0.02, 256).astype(np.float32), "float32")
    before = lib.tops_tensor_core_launches()
    ms = timed(lambda: lib.tops_conv2d_dqw_forward(cx.handle, wq.handle, ws.handle, None, cy.handle, ctypes.byref(cprm)), iters=3)
    out["conv_256x256x56x56_k3_bf16_int8_qdq_weights"] = {"TFLOPs": round(2.0 * 256 * 56 * 56 * 256 * 2304 / 1e12 / (ms / 1e3), 1),
                                                          "ms": round(ms, 4), "tensor_core_path": lib.tops_tensor_core_launches() > before}
    return out


def qdq_cnn_throughput(lib, stream, world, local, batch=256):
    """Images per second of the QDQ ResNet-50-shaped graph (benchmark config 5: batch 256 per GPU, float32
    [N,3,224,224] input, int8 QDQ around every convolution), input resident, every rank its own batch
    (batch sharding, no collective), time = max over ranks.  The graph runs through Graph.fused(): each
    Q -> DQ -> Conv [-> Relu] chain is one tensor-core call; the other nodes are the plain operators."""
    import torch
    from onnx_translator_b200 import capi, nn
    graph, x = nn.qdq_resnet50(batch=batch, seed=0)
    fused = graph.fused()
    xd = x.to_device()
    fused.forward(xd)                                   # warm-up: weights become resident, pools grow
    fused.forward(xd)
    lib.tops_sync()
    iters = 3
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    before = lib.tops_tensor_core_launches()
    ev[0].record(stream)
    for i in range(iters):
        out = fused.forward(xd)
        ev[i + 1].record(stream)
    lib.tops_sync()
    torch.cuda.synchronize()
    capi.check(lib)
    ms = float(np.median([ev[i].elapsed_time(ev[i + 1]) for i in range(iters)]))
    t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.cpu()[0])
    prob = out.numpy()
    flops = 2.0 * graph.macs_per_image * batch
    cpu = None
    if world == 1:
        # the same graph (unfused, as the reference would run it) on the host cores, one image
        import oracle
        from oracle import graph as oracle_graph
        kind = "reference" if oracle.available("ref") else "port"
        host = oracle.HostOracle("ref" if kind == "reference" else "port")
        cores = oracle.use_all_host_threads()
        one = nn.Tensor(1, 3, 224, 224, dtype="float32", data=np.ascontiguousarray(x.numpy()[:1]))
        t0 = time.perf_counter()
        oracle_graph.run(graph, host, one)
        dt = time.perf_counter() - t0
        cpu = {"images_per_s": round(1.0 / dt, 3), "cores": cores, "kind": kind, "sample": f"1 image, {dt:.1f} s, C functions node by node"}
    return {"cpu_baseline": cpu, "images_per_s": round(world * batch / (ms / 1e3), 1), "ms_per_batch": round(ms, 3), "batch_per_gpu": batch,
            "n_gpus": world, "TFLOPs_per_gpu": round(flops / 1e12 / (ms / 1e3), 1), "gflop_per_image": round(2.0 * graph.macs_per_image / 1e9, 2),
            "tensor_core_launches_per_batch": int((lib.tops_tensor_core_launches() - before) // iters),
            "nodes": len(fused.ops), "nodes_unfused": len(graph.ops),
            "softmax_rows_sum_to_one": bool(np.allclose(prob.sum(axis=1), 1.0, atol=1e-4))}


# DRAM read + write bytes of one ew_kernel<BinaryBody> launch, averaged over the 84 launches of one
# pass of this sweep at full size: dram__bytes_read.sum + dram__bytes_write.sum from an ncu launch
# list of `bench.py --steps 1 --warmup 3 --no-extra` (15.860 GB over 84 launches; the summary is
# profiles/bench_sweep_launch_list.md).  It is below the algorithmic bytes because part of each
# output is still in the 126 MB L2 when its kernel ends.
BINARY_DRAM_BYTES_PER_LAUNCH = 188_800_000


# ---- the reference's CPU implementation ------------------------------------------------------------------
def cpu_sweep(rows, steps, warmup):
    """Times the reference C library (or, if no compiled copy is present, the oracle port) on the
    sweep at `rows` rows of A, operands pre-broadcast to full size as its ABI requires.
    Returns (GB/s, seconds per step, kind, cores)."""
    import oracle
    kind = "reference" if oracle.available("ref") else "port"
    host = oracle.HostOracle("ref" if kind == "reference" else "port")
    cores = oracle.use_all_host_threads()
    a_host, a_cos_host, b_host = host_inputs(rows, seed=0)
    plan = sweep_plan(rows)
    full = (rows, MID, INNER)
    prepared = []
    for item in plan:
        a = a_cos_host if item["op"] == "cos" else a_host[item["a"]]
        wa = oracle._Wrapped(a, item["a"])
        wo = oracle._out(full, item["o"])
        if item["kind"] == "binary":
            b = np.ascontiguousarray(np.broadcast_to(b_host[(item["bname"], item["b"], item["divisor"])], full))
            prepared.append((host._fn[item["op"]], (wa.ref, oracle._Wrapped(b, item["b"]).ref, wo.ref), (wa, b, wo)))
        else:
            prepared.append((host._fn[item["op"]], (wa.ref, wo.ref), (wa, wo)))
    bytes_step = sum(item["bytes"] for item in plan)

    def one_step():
        for fn, fargs, _keep in prepared:
            fn(*fargs)

    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt = (time.perf_counter() - t0) / steps
    return bytes_step / 1e9 / dt, dt, kind, cores


def cpu_baseline(budget_s=20.0):
    rows = 4
    gbs, dt, kind, cores = cpu_sweep(rows, steps=1, warmup=0)
    if dt * 4 < budget_s:                       # a 4x larger slab still fits the budget
        rows = 16
        gbs, dt, kind, cores = cpu_sweep(rows, steps=1, warmup=0)
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"one pass of the 95-call sweep on A[{rows},512,1024] ({rows}/{FULL_ROWS} of the rows), C functions only, "
                      f"operands pre-broadcast on the host outside the timed region, {dt:.2f} s"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 8
    steps, warmup = max(1, args.steps), max(0, min(args.warmup, 1))
    gbs, dt, kind, cores = cpu_sweep(rows, steps, warmup)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference",
        "metric": "per-op GB/s (aggregate over the broadcast elementwise sweep)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64 arithmetic over f32/f16/bf16/i32/i8 storage", "data": "synthetic",
        "config": {"workload": f"config 2 sweep, bounded sample: A[{rows},512,1024] ({rows}/{FULL_ROWS} of the rows), 95 calls per step",
                   "parallelism": f"OpenMP, {cores} host threads"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{steps} timed passes of the sweep on A[{rows},512,1024], C functions only, operands pre-broadcast"},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--e2e-lanes", type=int, default=6, help="independent upload -> operator -> download pipelines of the end-to-end measurement")
    ap.add_argument("--no-extra", action="store_true", help="skip the QDQ / Softmax / MaxPool / Gemm / Conv side measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
