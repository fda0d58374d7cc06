#!/usr/bin/env python
"""Benchmark of the tensor_ops hot path on B200.

Workload (N = 1): the broadcast elementwise sweep -- Add/Sub/Mul/Div of A[64,512,1024] with B of
shape [1,512,1], [1024] and [64,512,1024] over seven dtype pairs, Relu/Abs on the same shape over
the five A dtypes, Cos on float32.  One "step" is one pass over all 95 operator calls.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case <operator> [--dtype ...] [--rows ...] ...      one operator case, for profilers (see run_case)

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

    sharded = None
    if world > 1 and not args.no_extra:
        sharded = sharded_leg(lib, stream, world, rank, local)

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
        if os.environ.get("BENCH_ALL_OPS"):                         # every launch of the sweep, slowest first, on stderr
            for label, gbps in sorted(per_op.items(), key=lambda kv: kv[1]):
                print(f"{gbps:8.1f} GB/s  {label}", file=sys.stderr)
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
                         "traffic": int(BINARY_DRAM_TRAFFIC_RATIO * fam_bytes / len(binary_idx)),
                         "traffic_how": "ncu dram read + write bytes of one float32 broadcast Add launch of this sweep without cache flushes, as a ratio (0.9886) of its algorithmic bytes, applied to the family's average"},
            "e2e": {"value": round(world * bytes_step / 1e9 / (e2e_ms_max / 1e3), 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_ms_max, 3)},
            "gpu_launches": n_launch * args.steps,
            "clocks": clocks.summary(),
            "slowest_ops_GBps": dict(worst),
        }
        line["cpu_baseline"] = cpu_baseline(budget_s=20.0) if world == 1 else None
        if qdq_cnn is not None:
            line["qdq_cnn"] = qdq_cnn
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_extra:
            try:
                line["small_cnn"] = small_cnn_latency(lib, stream)
            except Exception as exc:
                line["small_cnn"] = {"error": str(exc)[:200]}
        if world == 1 and not args.no_extra:
            try:
                line["other_ops"] = other_ops(lib, stream, peak)
            except Exception as exc:                      # the headline numbers stand on their own
                line["other_ops"] = {"error": str(exc)[:200]}
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
        # config 3 as what it is, a round trip: Q -> DQ in one pass (8 bytes per element), against the two calls above (10)
        codes = None if zp.dtype_name == dt else q.handle       # float8 codes with an int8 zero point: the code type comes from a codes tensor
        mem(f"qdq_roundtrip_f32_{label}", n * 8, lambda: lib.tops_quantize_dequantize_forward(x.handle, sc.handle, zp.handle, codes, back.handle))
        if codes is not None:
            out[f"qdq_roundtrip_f32_{label}"]["note"] = "the codes are stored too (9 bytes per element moved, 8 counted)"
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
    variants = (("f32_in_f32_out", "float32", lambda v: v, "float32"),
                ("bf16_in_f32_out", "bfloat16", bf16, "float32"), ("bf16_in_bf16_out", "bfloat16", bf16, "bfloat16"),
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
        if label == "f32_in_f32_out":
            out[f"gemm_8192_{label}"]["how"] = "three bfloat16 planes per operand, six plane products accumulated in float32 (judged against the bf16 peak / 6)"
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
    del cx, cw, cy, wq, ws
    out["cpu_slabs"] = cpu_slab_baselines()
    return out


def cpu_slab_baselines():
    """The reference C library on this machine's cores for the two contractions of config 4, timed on a slab and
    scaled (rows of a Gemm and images of a convolution are independent: tensor_ops.c:1174-1176, 1064-1066):
    Gemm float32 M = 32 of 8192 rows x 256; Conv float32 1 of 256 images x 256."""
    import oracle
    kind = "reference" if oracle.available("ref") else "port"
    host = oracle.HostOracle("ref" if kind == "reference" else "port")
    cores = oracle.use_all_host_threads()
    rng = np.random.default_rng(1)
    f32 = "float32"
    res = {}
    a = rng.normal(0, 0.02, (32, 8192)).astype(np.float32)
    b = rng.normal(0, 0.02, (8192, 8192)).astype(np.float32)
    c = rng.standard_normal(8192).astype(np.float32)
    t0 = time.perf_counter()
    host.gemm(a, f32, b, f32, c, f32, f32, 1.0, 1.0, 0, 1)
    dt = time.perf_counter() - t0
    res["gemm_8192_f32"] = {"slab": "M = 32 of 8192 rows", "slab_s": round(dt, 3), "factor": 256, "full_problem_s": round(dt * 256, 1),
                            "GFLOPs": round(2.0 * 32 * 8192 * 8192 / 1e9 / dt, 2), "cores": cores, "kind": kind}
    del a, b, c
    x = rng.standard_normal((1, 256, 56, 56)).astype(np.float32)
    w = rng.normal(0, 0.02, (256, 256, 3, 3)).astype(np.float32)
    t0 = time.perf_counter()
    host.conv2d(x, f32, w, f32, None, f32, f32, (1, 1, 1, 1), (1, 1), (1, 1), 1)
    dt = time.perf_counter() - t0
    res["conv_256x256x56x56_k3_f32"] = {"slab": "1 of 256 images", "slab_s": round(dt, 3), "factor": 256, "full_problem_s": round(dt * 256, 1),
                                       "GFLOPs": round(2.0 * 56 * 56 * 256 * 2304 / 1e9 / dt, 2), "cores": cores, "kind": kind}
    return res


def sharded_leg(lib, stream, world, rank, local):
    """Strong scaling of two fixed-size problems over the ranks (N > 1), results gathered ON THE DEVICE with NCCL:
    the bf16 Gemm 8192^3 of config 4 sharded along N (each rank a block of rows of B and of the bias, A replicated;
    tensor_ops.c:1174-1176 makes rows independent) followed by the all-gather of column blocks, and one float32
    broadcast Add of config 2 sharded by rows followed by the all-gather of row blocks.  Rank 0 also computes both
    problems whole and compares the gathered results bit for bit.  Times are device-measured, max over ranks."""
    import torch
    import torch.distributed as dist
    from onnx_translator_b200 import capi, shard
    from onnx_translator_b200.device import DeviceArray
    rng = np.random.default_rng(7)                       # the same operands on every rank

    def bf16(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)

    def timed(call, iters=5):
        call()
        lib.tops_sync()
        torch.cuda.synchronize()
        dist.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
        with torch.cuda.stream(stream):
            ev[0].record(stream)
            for i in range(iters):
                call()
                ev[i + 1].record(stream)
        lib.tops_sync()
        torch.cuda.synchronize()
        ms = float(np.median([ev[i].elapsed_time(ev[i + 1]) for i in range(iters)]))
        t = torch.tensor([ms], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.cpu()[0])

    out = {}
    # -- Gemm sharded along N --------------------------------------------------------------------------
    m = 8192
    a_host = bf16(rng.normal(0, 0.02, (m, m)).astype(np.float32))
    b_host = bf16(rng.normal(0, 0.02, (m, m)).astype(np.float32))
    bias_host = rng.standard_normal((1, m)).astype(np.float32)
    b_blk, bias_blk, (n0, n1) = shard.gemm_shard(b_host, bias_host, world, rank)
    a = DeviceArray.from_numpy(a_host, "bfloat16")
    b = DeviceArray.from_numpy(np.ascontiguousarray(b_blk), "bfloat16")
    bias = DeviceArray.from_numpy(np.ascontiguousarray(bias_blk), "float32")
    y = DeviceArray.empty((m, n1 - n0), "bfloat16")
    gathered = {}

    def gemm_compute():
        lib.gemm_forward(a.handle, b.handle, bias.handle, y.handle, 1.0, 1.0, 0, 1)

    def gemm_gather():
        with torch.cuda.stream(stream):
            gathered["y"] = shard.gather_columns(y.as_torch(), m)

    compute_ms = timed(gemm_compute)
    gather_ms = timed(gemm_gather)
    same = None
    if rank == 0:
        b_full = DeviceArray.from_numpy(b_host, "bfloat16")
        bias_full = DeviceArray.from_numpy(bias_host, "float32")
        y_full = DeviceArray.empty((m, m), "bfloat16")
        lib.gemm_forward(a.handle, b_full.handle, bias_full.handle, y_full.handle, 1.0, 1.0, 0, 1)
        lib.tops_sync()
        same = bool(torch.equal(gathered["y"].view(torch.int16), y_full.as_torch().view(torch.int16)))
        del b_full, bias_full, y_full
    out["gemm_8192_bf16_sharded_along_N"] = {
        "compute_ms": round(compute_ms, 4), "gather_ms": round(gather_ms, 4), "TFLOPs_compute": round(2.0 * m ** 3 / 1e12 / (compute_ms / 1e3), 1),
        "TFLOPs_with_gather": round(2.0 * m ** 3 / 1e12 / ((compute_ms + gather_ms) / 1e3), 1),
        "collective": "NCCL all-gather of [N/g, M] row blocks of the transposed result + transposes", "collective_share": round(gather_ms / (compute_ms + gather_ms), 3),
        "gathered_equals_single_gpu_result": same}
    del a, b, bias, y
    gathered.clear()
    # -- broadcast Add sharded by rows ------------------------------------------------------------------------
    a_host = rng.uniform(-100, 100, (FULL_ROWS, MID, INNER)).astype(np.float32)
    b_host = rng.uniform(-100, 100, (1, MID, 1)).astype(np.float32)
    mine = np.ascontiguousarray(shard.split_rows(a_host, world, rank))
    a = DeviceArray.from_numpy(mine, "float32")
    b = DeviceArray.from_numpy(b_host, "float32")
    o = DeviceArray.empty(mine.shape, "float32")

    def add_compute():
        lib.add_forward(a.handle, b.handle, o.handle)

    def add_gather():
        with torch.cuda.stream(stream):
            gathered["o"] = shard.gather_rows(o.as_torch(), FULL_ROWS)

    compute_ms = timed(add_compute)
    gather_ms = timed(add_gather)
    same = None
    if rank == 0:
        a_full = DeviceArray.from_numpy(a_host, "float32")
        o_full = DeviceArray.empty(a_host.shape, "float32")
        lib.add_forward(a_full.handle, b.handle, o_full.handle)
        lib.tops_sync()
        same = bool(torch.equal(gathered["o"].view(torch.int32), o_full.as_torch().view(torch.int32)))
    nbytes = a_host.nbytes * 2
    out["add_f32_A64x512x1024_row_sharded"] = {
        "compute_ms": round(compute_ms, 4), "gather_ms": round(gather_ms, 4), "GBps_compute": round(nbytes / 1e9 / (compute_ms / 1e3), 1),
        "collective": "NCCL all-gather of row blocks", "collective_share": round(gather_ms / (compute_ms + gather_ms), 3),
        "gathered_equals_single_gpu_result": same}
    capi.check(lib)
    return out


def small_cnn_latency(lib, stream):
    """Config 1: microseconds per forward pass of the small CNN (12 nodes), replayed from its call plan as one
    CUDA graph, with the reference C library running the same nodes on the host beside it."""
    import torch
    import oracle
    from oracle import graph as oracle_graph
    from onnx_translator_b200 import capi, nn
    graph, x = nn.small_cnn(seed=0)
    plan = graph.plan(x)
    plan.run()
    captured = plan.capture()
    iters = 200
    for _ in range(20):
        plan.run()
    lib.tops_sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(iters):
        plan.run()
    e1.record(stream)
    lib.tops_sync()
    torch.cuda.synchronize()
    device_us = e0.elapsed_time(e1) * 1e3 / iters
    t0 = time.perf_counter()
    for _ in range(50):                                  # latency a caller sees: enqueue one pass and wait for it
        plan.run()
        lib.tops_sync()
    wall_us = (time.perf_counter() - t0) * 1e6 / 50
    capi.check(lib)
    kind = "reference" if oracle.available("ref") else "port"
    host = oracle.HostOracle("ref" if kind == "reference" else "port")
    cores = oracle.use_all_host_threads()
    oracle_graph.run(graph, host, x)
    t0 = time.perf_counter()
    for _ in range(20):
        oracle_graph.run(graph, host, x)
    cpu_us = (time.perf_counter() - t0) * 1e6 / 20
    n_calls = len(plan.calls)
    plan.close()
    return {"us_per_graph_device": round(device_us, 2), "us_per_graph_enqueue_and_wait": round(wall_us, 1), "cuda_graph": bool(captured),
            "library_calls_per_forward": n_calls,
            "cpu_baseline": {"us_per_graph": round(cpu_us, 1), "cores": cores, "kind": kind, "sample": "20 passes, C functions node by node"}}


def qdq_cnn_throughput(lib, stream, world, local, batch=256):
    """Images per second of the QDQ ResNet-50-shaped graph (benchmark config 5: batch 256 per GPU, float32
    [N,3,224,224] input, int8 QDQ around every convolution), input resident, every rank its own batch
    (batch sharding, no collective), time = max over ranks.  The graph runs through Graph.fused() (each
    Q -> DQ -> Conv [-> Add] [-> Relu] chain is one tensor-core call) and Graph.plan(): the forward pass is
    recorded once and replayed as one CUDA graph launch.  Host time per forward (the call that enqueues a
    pass, no synchronisation) is reported beside the device time, with the spread over ranks."""
    import torch
    from onnx_translator_b200 import capi, nn
    graph, x = nn.qdq_resnet50(batch=batch, seed=0)
    fused = graph.fused()
    xd = x.to_device()
    before = lib.tops_tensor_core_launches()
    plan = fused.plan(xd)                               # the recording pass: weights become resident, filter caches fill
    tc_launches = int(lib.tops_tensor_core_launches() - before)
    plan.run()
    captured = plan.capture()
    plan.run()
    lib.tops_sync()
    capi.check(lib)
    iters = 5
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
    host = []
    ev[0].record(stream)
    for i in range(iters):
        t0 = time.perf_counter()
        out = plan.run()
        host.append((time.perf_counter() - t0) * 1e3)
        ev[i + 1].record(stream)
    lib.tops_sync()
    torch.cuda.synchronize()
    capi.check(lib)
    ms = float(np.median([ev[i].elapsed_time(ev[i + 1]) for i in range(iters)]))
    host_ms = float(np.median(host))
    # the node-by-node interpreter on the same graph, host side only (what a plan saves)
    t0 = time.perf_counter()
    fused.forward(xd)
    walk_ms = (time.perf_counter() - t0) * 1e3
    lib.tops_sync()
    per_rank = torch.tensor([[ms, host_ms, walk_ms]], dtype=torch.float64, device=f"cuda:{local}")
    if world > 1:
        import torch.distributed as dist
        gathered = [torch.zeros_like(per_rank) for _ in range(world)]
        dist.all_gather(gathered, per_rank)
        per_rank = torch.cat(gathered)
    per_rank = per_rank.cpu().numpy()
    ms = float(per_rank[:, 0].max())
    prob = out.numpy()
    flops = 2.0 * graph.macs_per_image * batch
    cpu = None
    prob_diff = None
    if world == 1:
        # the same graph (unfused, as the reference would run it) on the host cores, one image
        import oracle
        from oracle import graph as oracle_graph
        kind = "reference" if oracle.available("ref") else "port"
        host_oracle = oracle.HostOracle("ref" if kind == "reference" else "port")
        cores = oracle.use_all_host_threads()
        one = nn.Tensor(1, 3, 224, 224, dtype="float32", data=np.ascontiguousarray(x.numpy()[:1]))
        t0 = time.perf_counter()
        cpu_prob = oracle_graph.run(graph, host_oracle, one)
        dt = time.perf_counter() - t0
        cpu = {"images_per_s": round(1.0 / dt, 3), "cores": cores, "kind": kind, "sample": f"1 image, {dt:.1f} s, C functions node by node"}
        prob_diff = float(np.abs(prob[0].astype(np.float64) - cpu_prob[0]).max())
    n_calls = len(plan.calls)
    plan.close()
    return {"cpu_baseline": cpu, "images_per_s": round(world * batch / (ms / 1e3), 1), "ms_per_batch": round(ms, 3), "batch_per_gpu": batch,
            "n_gpus": world, "TFLOPs_per_gpu": round(flops / 1e12 / (ms / 1e3), 1), "gflop_per_image": round(2.0 * graph.macs_per_image / 1e9, 2),
            "tensor_core_launches_per_batch": tc_launches,
            "nodes": len(fused.ops), "nodes_unfused": len(graph.ops), "library_calls_per_forward": n_calls,
            "cuda_graph": bool(captured),
            "device_ms_per_rank": {"min": round(float(per_rank[:, 0].min()), 3), "max": round(float(per_rank[:, 0].max()), 3)},
            "host_ms_per_forward": {"min": round(float(per_rank[:, 1].min()), 3), "max": round(float(per_rank[:, 1].max()), 3),
                                    "what": "time for plan.run() to return (one CUDA graph launch when captured), no synchronisation"},
            "host_ms_node_by_node": {"min": round(float(per_rank[:, 2].min()), 3), "max": round(float(per_rank[:, 2].max()), 3),
                                     "what": "Graph.forward walking the fused nodes in Python, no synchronisation"},
            "max_abs_prob_diff": prob_diff,
            "max_abs_prob_diff_what": "image 0 of the batch: fused GPU graph against the unfused graph on the CPU (largest probability about 1e-3)" if prob_diff is not None else None,
            "softmax_rows_sum_to_one": bool(np.allclose(prob.sum(axis=1), 1.0, atol=1e-4))}


# DRAM read + write bytes of one ew_kernel<BinaryBody> launch as a fraction of its algorithmic bytes: measured with
# ncu (dram__bytes_read.sum + dram__bytes_write.sum, caches NOT flushed around the kernel, so that the write-backs a
# launch leaves in L2 are counted with the next one) on the float32 broadcast Add of this sweep at full size:
# 265.37 MB moved for 268.44 MB of algorithmic bytes.
BINARY_DRAM_TRAFFIC_RATIO = 0.9886


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
    wrapped_a, wrapped_b, wrapped_o = {}, {}, {}            # one host copy per distinct operand, shared by the calls that use it

    def a_of(item):
        key = "cos" if item["op"] == "cos" else item["a"]
        if key not in wrapped_a:
            wrapped_a[key] = oracle._Wrapped(a_cos_host if key == "cos" else a_host[key], item["a"])
        return wrapped_a[key]

    def b_of(item):
        key = (item["bname"], item["b"], item["divisor"])
        if key not in wrapped_b:
            wrapped_b[key] = oracle._Wrapped(np.ascontiguousarray(np.broadcast_to(b_host[key], full)), item["b"])
        return wrapped_b[key]

    def o_of(item):
        if item["o"] not in wrapped_o:
            wrapped_o[item["o"]] = oracle._out(full, item["o"])
        return wrapped_o[item["o"]]

    for item in plan:
        wa, wo = a_of(item), o_of(item)
        if item["kind"] == "binary":
            wb = b_of(item)
            prepared.append((host._fn[item["op"]], (wa.ref, wb.ref, wo.ref), (wa, wb, wo)))
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
    # the full workload of our arm (A[64,512,1024], about 4 GB of host operands) when the host has the memory for it
    rows = FULL_ROWS
    try:
        with open("/proc/meminfo") as f:
            avail_kb = next(int(line.split()[1]) for line in f if line.startswith("MemAvailable"))
        if avail_kb < 12 * 1024 * 1024:
            rows = 16
    except Exception:
        rows = 16
    steps, warmup = max(1, min(args.steps, 20)), max(0, min(args.warmup, 1))
    gbs, dt, kind, cores = cpu_sweep(rows, steps, warmup)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference",
        "metric": "per-op GB/s (aggregate over the broadcast elementwise sweep)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64 arithmetic over f32/f16/bf16/i32/i8 storage", "data": "synthetic",
        "config": {"workload": ("config 2: broadcast elementwise sweep, A[64,512,1024] x B{[1,512,1],[1024],full} x 7 dtype pairs x Add/Sub/Mul/Div + Relu/Abs x 5 dtypes + Cos f32 (95 calls per step), operands pre-broadcast on the host as the reference's ABI requires"
                                if rows == FULL_ROWS else f"config 2 sweep, bounded sample: A[{rows},512,1024] ({rows}/{FULL_ROWS} of the rows), 95 calls per step"),
                   "parallelism": f"OpenMP, {cores} host threads"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{steps} timed passes of the sweep on A[{rows},512,1024], C functions only, operands pre-broadcast"},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---- single operator cases (profiler command lines) ------------------------------------------------------------
CASE_ITEM = {"float32": 4, "float16": 2, "bfloat16": 2, "int32": 4, "int8": 1, "uint8": 1, "float64": 8,
        "float8_e4m3": 1, "float8_e5m2": 1, "int16": 2, "int64": 8, "int4": 1}


def _case_rand(rng, shape, dtype, lo=-100, hi=100):
    from onnx_translator_b200 import capi
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


def _case_ints(vals):
    arr = (ctypes.c_int * len(vals))(*vals)
    return arr, ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))


def run_case(case, argv):
    """One operator case a few times, event-timed: small self-contained command lines for profilers (one kernel,
    few launches, bounded memory).  Elementwise cases use A[rows,512,1024] with B of shape [1,512,1] (row), [1024]
    (vec) or full; quantize / dequantize X[rows,8192]; softmax X[rows,1000]; maxpool X[rows,64,112,112] k3 s2 p1;
    qdq_resnet50 the fused benchmark graph on --batch images (replayed from its call plan)."""
    import ctypes
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    from onnx_translator_b200.capi import CConvParams, CPoolParams
    ap = argparse.ArgumentParser(prog="bench.py --case " + case)
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
    args = ap.parse_args(argv)
    args.op = case

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
        a = DeviceArray.from_numpy(_case_rand(rng, shape, dt), dt)
        b = DeviceArray.from_numpy(_case_rand(rng, bshape, bdt, 0.5, 100), bdt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, b.handle, o.handle)
        n = a.size
        nbytes = n * (CASE_ITEM[dt] + CASE_ITEM[out_dt]) + b.size * CASE_ITEM[bdt]
    elif args.op in ("relu", "abs", "cos"):
        shape = (args.rows, 512, 1024)
        a = DeviceArray.from_numpy(_case_rand(rng, shape, dt, -10, 10), dt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, o.handle)
        nbytes = a.size * (CASE_ITEM[dt] + CASE_ITEM[out_dt])
    elif args.op in ("exp", "log", "sqrt", "sigmoid", "tanh", "neg", "reciprocal", "ceil", "floor", "sin", "tan", "atan", "softplus", "softsign",
                     "hard_swish", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "round", "erf", "gelu", "cast"):
        shape = (args.rows, 512, 1024)
        a = DeviceArray.from_numpy(_case_rand(rng, shape, dt, -3, 3), dt)
        o = DeviceArray.empty(shape, out_dt)
        fn = getattr(lib, args.op + "_forward")
        call = lambda: fn(a.handle, o.handle)
        nbytes = a.size * (CASE_ITEM[dt] + CASE_ITEM[out_dt])
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
            x = DeviceArray.from_numpy(_case_rand(rng, shape, dt), dt)
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
        nbytes = x.size * (CASE_ITEM[x.dtype_name] + CASE_ITEM[out_dt])
    elif args.op == "softmax":
        shape = (args.rows, 1000)
        x = DeviceArray.from_numpy(_case_rand(rng, shape, dt, -10, 10), dt)
        o = DeviceArray.empty(shape, out_dt)
        call = lambda: lib.softmax_forward(x.handle, o.handle, 1)
        nbytes = x.size * (CASE_ITEM[dt] + CASE_ITEM[out_dt])
    elif args.op == "maxpool":
        shape = (args.rows, 64, 112, 112)
        x = DeviceArray.from_numpy(_case_rand(rng, shape, dt), dt)
        o = DeviceArray.empty((args.rows, 64, 56, 56), out_dt)
        keep = [_case_ints([1, 1, 1, 1]), _case_ints([2, 2]), _case_ints([1, 1]), _case_ints([3, 3])]
        prm = CPoolParams(keep[0][1], keep[1][1], keep[2][1], keep[3][1])
        call = lambda: lib.max_pool_forward(x.handle, o.handle, ctypes.byref(prm))
        nbytes = x.size * CASE_ITEM[dt] + o.size * CASE_ITEM[out_dt]
    elif args.op == "gemm":
        a = DeviceArray.from_numpy(_case_rand(rng, (args.m, args.k), dt, -0.05, 0.05), dt)
        b = DeviceArray.from_numpy(_case_rand(rng, (args.n, args.k), dt, -0.05, 0.05), dt)
        c = DeviceArray.from_numpy(rng.standard_normal((1, args.n)).astype(np.float32), "float32")
        o = DeviceArray.empty((args.m, args.n), out_dt)
        call = lambda: lib.gemm_forward(a.handle, b.handle, c.handle, o.handle, 1.0, 1.0, 0, 1)
        nbytes = a.size * CASE_ITEM[dt] + b.size * CASE_ITEM[dt] + o.size * CASE_ITEM[out_dt]
        flops = 2.0 * args.m * args.n * args.k
    elif args.op == "conv":
        n_, c_, hw = args.batch, args.channels, args.hw
        x = DeviceArray.from_numpy(_case_rand(rng, (n_, c_, hw, hw), dt, -1, 1), dt)
        w = DeviceArray.from_numpy(_case_rand(rng, (c_, c_, 3, 3), dt, -0.05, 0.05), dt)
        o = DeviceArray.empty((n_, c_, hw, hw), out_dt)
        keep = [_case_ints([1, 1, 1, 1]), _case_ints([1, 1]), _case_ints([1, 1])]
        prm = CConvParams(keep[0][1], keep[1][1], keep[2][1], 1)
        call = lambda: lib.conv2d_forward(x.handle, w.handle, None, o.handle, ctypes.byref(prm))
        nbytes = x.size * CASE_ITEM[dt] + w.size * CASE_ITEM[dt] + o.size * CASE_ITEM[out_dt]
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
        keep = [_case_ints([pad] * 4), _case_ints([1, 1]), _case_ints([1, 1])]
        prm = CConvParams(keep[0][1], keep[1][1], keep[2][1], 1)
        call = lambda: lib.tops_qdq_conv_forward(x.handle, sx.handle, zx.handle, wq.handle, ws.handle, None, None, o.handle,
                                                 ctypes.byref(prm), 1)
        nbytes = x.size * 4 + o.size * 4
        flops = 2.0 * n_ * hw * hw * m_ * c_ * ks * ks
        dt = out_dt = "float32"
    elif args.op == "qdq_resnet50":
        # the QDQ ResNet-50-shaped graph through Graph.fused(); --batch images of 224 x 224
        from onnx_translator_b200 import nn
        graph, x_host = nn.qdq_resnet50(batch=args.batch, seed=0)
        fused = graph.fused()
        xd = x_host.to_device()
        plan = fused.plan(xd)
        keep = [graph, fused, xd, plan]
        call = lambda: plan.run()
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



def main():
    if "--case" in sys.argv:
        i = sys.argv.index("--case")
        return run_case(sys.argv[i + 1], sys.argv[1:i] + sys.argv[i + 2:])
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
