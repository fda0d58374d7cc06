"""Two ranks on two GPUs over NCCL (skipped on a one-GPU box): DynamicQuantizeLinear of a tensor whose row
blocks live on different GPUs -- the one operator on the widened path with a data-path exchange (an all-reduce of
the two ends of the range) -- must give the codes, scale and zero point of the single-GPU call, bit for bit; and a
row-sharded broadcast Add gathered over NCCL must equal the oracle's result.  The gathers run on device memory (the
library's tensors seen as torch tensors, no host hop).  A second test drives two devices from ONE process: the
opt-in for large dynamic shared memory is per device, so the first tensor-core and cosine launches on the second
device must work too.  NVLS is switched off for the tests."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LOCAL_RANK=str(rank), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import datetime
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    # a short timeout: a rank whose peer died leaves its collective with an error instead of waiting
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    try:
        import oracle
        from onnx_translator_b200 import capi, shard
        from onnx_translator_b200.device import DeviceArray
        lib = capi.load()
        port_lib = oracle.HostOracle("port")
        rng = np.random.default_rng(99)                           # the same data on both ranks
        x = rng.normal(0.3, 1.2, (513, 777)).astype(np.float32)
        x[7, 7], x[400, 1], x[100, 100] = 11.5, -6.25, np.nan      # the extremes sit in different row blocks
        want_y, want_s, want_z = port_lib.dynamic_quantize_linear(x, "float32")
        block = np.ascontiguousarray(shard.split_rows(x, world, rank))
        y, s, z = shard.dynamic_quantize_rows(DeviceArray.from_numpy(block, "float32"), "float32", lib)
        stream = torch.cuda.ExternalStream(lib.tops_get_stream(), device=rank)
        with torch.cuda.stream(stream):                           # device-resident gather, ordered after the library's work
            codes = shard.gather_rows(y.as_torch(), x.shape[0])
        stream.synchronize()
        codes = codes.cpu().numpy()
        ok_dq = np.array_equal(codes, want_y) and s.numpy().tobytes() == want_s.tobytes() and np.array_equal(z.numpy(), want_z)
        a = rng.uniform(-100, 100, (9, 12, 16)).astype(np.float32)
        b = rng.uniform(-100, 100, (1, 12, 1)).astype(np.float32)
        from onnx_translator_b200 import nn
        from onnx_translator_b200.nn import Operators as ops
        mine = np.ascontiguousarray(shard.split_rows(a, world, rank))
        out = ops.ADD([], [], dtype="float32").forward(nn.Tensor(*mine.shape, dtype="float32", data=mine),
                                                       nn.Tensor(*b.shape, dtype="float32", data=b))["tensor"]
        with torch.cuda.stream(stream):
            full = shard.gather_rows(out.data.as_torch(), 9)
        stream.synchronize()
        full = full.cpu().numpy()
        ok_add = np.array_equal(full, port_lib.binary("add", a, "float32", b, "float32", "float32"))
        ret[rank] = (bool(ok_dq), bool(ok_add))
        torch.cuda.synchronize()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    ret = manager.dict()
    port = 29600 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=300)
    finally:
        for p in procs:                                  # never leave a rank behind holding a GPU
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    assert [p.exitcode for p in procs] == [0, 0]
    assert dict(ret) == {0: (True, True), 1: (True, True)}


def _second_device(ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import ctypes
    import oracle
    from datagen import from_f64, to_f64
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    port_lib = oracle.HostOracle("port")
    rng = np.random.default_rng(3)
    results = []
    for device in (0, 1):
        assert lib.tops_set_device(device) == 0
        x = rng.uniform(-10, 10, (64, 1024)).astype(np.float32)
        y = DeviceArray.empty(x.shape, "float32")
        xd = DeviceArray.from_numpy(x, "float32")
        lib.cos_forward(xd.handle, y.handle)
        ok_cos = np.array_equal(y.numpy().view(np.uint32), port_lib.unary("cos", x, "float32", "float32").view(np.uint32))
        a = from_f64(rng.normal(0, 1, (256, 512)), "bfloat16")
        b = from_f64(rng.normal(0, 1, (384, 512)), "bfloat16")
        ad, bd = DeviceArray.from_numpy(a, "bfloat16"), DeviceArray.from_numpy(b, "bfloat16")
        out = DeviceArray.empty((256, 384), "float32")
        before = lib.tops_tensor_core_launches()
        lib.gemm_forward(ad.handle, bd.handle, None, out.handle, 1.0, 1.0, 0, 1)
        got = out.numpy().astype(np.float64)
        want = to_f64(a, "bfloat16") @ to_f64(b, "bfloat16").T
        s_mag = np.abs(to_f64(a, "bfloat16")) @ np.abs(to_f64(b, "bfloat16")).T
        ok_gemm = lib.tops_tensor_core_launches() == before + 1 and bool(np.all(np.abs(got - want) <= 1e-6 * s_mag + 1e-6))
        keep = [(ctypes.c_int * 4)(1, 1, 1, 1), (ctypes.c_int * 2)(1, 1), (ctypes.c_int * 2)(1, 1)]
        prm = capi.CConvParams(*[ctypes.cast(k, ctypes.POINTER(ctypes.c_int)) for k in keep], 1)
        cx = DeviceArray.from_numpy(from_f64(rng.normal(0, 1, (8, 32, 12, 12)), "bfloat16"), "bfloat16")
        cw = DeviceArray.from_numpy(from_f64(rng.normal(0, 0.1, (64, 32, 3, 3)), "bfloat16"), "bfloat16")
        cy = DeviceArray.empty((8, 64, 12, 12), "float32")
        before = lib.tops_tensor_core_launches()
        lib.conv2d_forward(cx.handle, cw.handle, None, cy.handle, ctypes.byref(prm))
        ok_conv = lib.tops_tensor_core_launches() == before + 1 and bool(np.isfinite(cy.numpy()).all()) and bool(np.abs(cy.numpy()).max() > 0)
        err = lib.tops_last_error()
        results.append((device, bool(ok_cos), bool(ok_gemm), bool(ok_conv), int(err)))
        del xd, y, ad, bd, out, cx, cw, cy
    ret["results"] = results


def test_one_process_drives_two_devices():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    ret = manager.dict()
    p = ctx.Process(target=_second_device, args=(ret,))
    p.start()
    try:
        p.join(timeout=300)
    finally:
        if p.is_alive():
            p.terminate()
            p.join(10)
    assert p.exitcode == 0
    assert ret["results"] == [(0, True, True, True, 0), (1, True, True, True, 0)]
