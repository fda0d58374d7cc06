"""Multi-rank sharding on CPU: two gloo ranks split each operator's work by rows (Gemm by columns of
Y), compute their block with the CPU oracle, gather, and must reproduce the single-process result
bit for bit.  This exercises the same shard.py helpers bench.py and a multi-GPU caller use."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OMP_NUM_THREADS"] = "2"
    import torch.distributed as dist
    import oracle
    from onnx_translator_b200 import shard
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        port_lib = oracle.HostOracle("port")
        rng = np.random.default_rng(123)                       # same data on every rank
        # broadcast Add, uneven row split (7 rows over 2 ranks), B replicated
        a = rng.uniform(-100, 100, (7, 12, 16)).astype(np.float32)
        b = rng.uniform(-100, 100, (1, 12, 1)).astype(np.float32)
        full = port_lib.binary("add", a, "float32", b, "float32", "float32")
        mine = port_lib.binary("add", shard.split_rows(a, world, rank), "float32", b, "float32", "float32")
        ok_add = np.array_equal(shard.gather_rows(mine, 7), full)
        # per-axis quantize to int8 (scale / zero point replicated)
        x = rng.standard_normal((9, 32)).astype(np.float32)
        s = rng.uniform(0.01, 0.05, 32).astype(np.float32)
        z = rng.integers(-8, 9, 32).astype(np.int8)
        fullq = port_lib.quantize(x, "float32", s, "float32", z, "int8", "int8", axis=1)
        mineq = port_lib.quantize(shard.split_rows(x, world, rank), "float32", s, "float32", z, "int8", "int8", axis=1)
        ok_q = np.array_equal(shard.gather_rows(mineq, 9), fullq)
        # bfloat16 codes survive the gather
        codes = rng.integers(0, 65535, (5, 6)).astype(np.uint16)
        ok_bf16 = np.array_equal(shard.gather_rows(shard.split_rows(codes, world, rank), 5), codes)
        # conv: batch shard
        cx = rng.standard_normal((3, 4, 6, 6)).astype(np.float32)
        cw = rng.normal(0, 0.1, (5, 4, 3, 3)).astype(np.float32)
        cargs = ("float32", cw, "float32", None, "float32", "float32", (1, 1, 1, 1), (1, 1), (1, 1), 1)
        fullc = port_lib.conv2d(cx, *cargs)
        minec = port_lib.conv2d(shard.split_rows(cx, world, rank), *cargs)
        ok_conv = np.array_equal(shard.gather_rows(minec, 3), fullc)
        # Gemm sharded along N with a per-column bias
        ga = rng.normal(0, 1, (6, 10)).astype(np.float32)
        gb = rng.normal(0, 1, (9, 10)).astype(np.float32)
        gc = rng.normal(0, 1, 9).astype(np.float32)
        fullg = port_lib.gemm(ga, "float32", gb, "float32", gc, "float32", "float32", 1.0, 1.0, 0, 1)
        bb, cb, (n0, n1) = shard.gemm_shard(gb, gc, world, rank)
        mineg = port_lib.gemm(ga, "float32", bb, "float32", cb, "float32", "float32", 1.0, 1.0, 0, 1)
        ok_gemm = mineg.shape == (6, n1 - n0) and np.array_equal(shard.gather_columns(mineg, 9), fullg)
        # DynamicQuantizeLinear: the one operator with an exchange -- ranges of the row blocks are combined
        # (all-reduce of two numbers), then every rank quantises its block with the common range
        dx = rng.normal(0.2, 1.5, (11, 40)).astype(np.float32)
        dx[2, 7], dx[9, 1] = 9.5, -7.25                       # the extremes sit in different blocks
        dx[0, 3], dx[8, 3] = np.nan, np.nan                   # NaNs never enter the range
        full_y, full_s, full_z = port_lib.dynamic_quantize_linear(dx, "float32")
        block = shard.split_rows(dx, world, rank)
        local = port_lib.dynamic_quantize_range(block, "float32")
        common = shard.combine_ranges(local.copy())
        my_y, my_s, my_z = port_lib.dynamic_quantize_apply(block, "float32", common)
        ok_dq = (np.array_equal(shard.gather_rows(my_y, 11), full_y) and my_s.tobytes() == full_s.tobytes() and
                 np.array_equal(my_z, full_z) and not np.array_equal(local, common))
        ret[rank] = (ok_add, ok_q, ok_bf16, ok_conv, ok_gemm, ok_dq)
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_result():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    ret = manager.dict()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(timeout=180)
    finally:
        for p in procs:                                  # a rank stuck in a collective after its peer died is ended here
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    assert [p.exitcode for p in procs] == [0, 0]
    assert dict(ret) == {0: (True,) * 6, 1: (True,) * 6}


def test_row_range_covers_everything_once():
    from onnx_translator_b200 import shard
    for total in (0, 1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            blocks = [shard.row_range(total, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == total
            for (b0, c0), (b1, _) in zip(blocks, blocks[1:]):
                assert b1 == b0 + c0
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1
    with pytest.raises(ValueError):
        shard.row_range(4, 2, 2)
