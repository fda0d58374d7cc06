"""Two ranks on two GPUs over NCCL (skipped on a one-GPU box): DynamicQuantizeLinear of a tensor whose row
blocks live on different GPUs -- the one operator on the widened path with a data-path exchange (an all-reduce of
the two ends of the range) -- must give the codes, scale and zero point of the single-GPU call, bit for bit; and a
row-sharded broadcast Add gathered over NCCL must equal the oracle's result.  NVLS is switched off for the test."""
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
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
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
        codes = shard.gather_rows(torch.from_numpy(y.numpy()).cuda(), x.shape[0]).cpu().numpy()
        ok_dq = np.array_equal(codes, want_y) and s.numpy().tobytes() == want_s.tobytes() and np.array_equal(z.numpy(), want_z)
        a = rng.uniform(-100, 100, (9, 12, 16)).astype(np.float32)
        b = rng.uniform(-100, 100, (1, 12, 1)).astype(np.float32)
        from onnx_translator_b200 import nn
        from onnx_translator_b200.nn import Operators as ops
        mine = np.ascontiguousarray(shard.split_rows(a, world, rank))
        out = ops.ADD([], [], dtype="float32").forward(nn.Tensor(*mine.shape, dtype="float32", data=mine),
                                                       nn.Tensor(*b.shape, dtype="float32", data=b))["tensor"].numpy()
        full = shard.gather_rows(torch.from_numpy(out).cuda(), 9).cpu().numpy()
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
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert dict(ret) == {0: (True, True), 1: (True, True)}
