"""Row / batch sharding of the hot-path operators across the GPUs of one box.

Every operator on the path is independent over its leading dimension (elements, rows, images), so a
job is split into contiguous row blocks, one per rank (one process per GPU), small broadcast operands
(scale, zero point, bias, weights) are replicated, and nothing is exchanged during compute.  The only
collective is the optional final gather of results.  Gemm shards along N instead: each rank takes a
block of rows of B (stored [N, K], used transposed) and the matching slice of a per-column bias, and
produces a block of columns of Y.

The helpers are backend-agnostic: arrays are numpy on the host or torch tensors on any device, and
the gather runs over whatever ``torch.distributed`` backend the process group was created with
(NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np


def row_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """(begin, count) of the contiguous block of ``total`` rows owned by ``rank``: the first
    ``total % world`` ranks get one extra row."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(int(total), world)
    begin = rank * base + min(rank, extra)
    return begin, base + (1 if rank < extra else 0)


def split_rows(array, world: int, rank: int):
    """This rank's block along dimension 0 (a view, no copy)."""
    begin, count = row_range(array.shape[0], world, rank)
    return array[begin:begin + count]


def gemm_shard(b, bias, world: int, rank: int):
    """Gemm with transB = 1 sharded along N: rows [n0, n1) of B and, for a per-column bias of
    length N (1-D or shaped (1, N)), the matching slice.  Any other bias is replicated."""
    n_total = b.shape[0]
    n0, count = row_range(n_total, world, rank)
    b_block = b[n0:n0 + count]
    bias_block = bias
    if bias is not None:
        shape = tuple(bias.shape)
        if shape == (n_total,):
            bias_block = bias[n0:n0 + count]
        elif len(shape) == 2 and shape == (1, n_total):
            bias_block = bias[:, n0:n0 + count]
    return b_block, bias_block, (n0, n0 + count)


def _dist():
    import torch.distributed as dist
    return dist


def gather_rows(local, total_rows: int, group=None):
    """All-gather row blocks produced under ``row_range`` into the full array on every rank.
    ``local`` is a torch tensor (any device) or a numpy array; the result has the same kind."""
    import torch
    dist = _dist()
    if not (dist.is_available() and dist.is_initialized()):
        return local
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    as_numpy = isinstance(local, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(local)) if as_numpy else local.contiguous()
    restore = t.dtype                                # gather raw bytes: every backend moves uint8
    if t.ndim == 1:
        t = t.reshape(-1, 1)
        flat = True
    else:
        flat = False
    t = t.view(torch.uint8)
    counts = [row_range(total_rows, world, r)[1] for r in range(world)]
    widest = max(counts)
    padded = t
    if t.shape[0] != widest:                         # collectives want equal shapes: pad the short blocks
        pad = torch.zeros((widest - t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        padded = torch.cat([t, pad], dim=0)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    full = torch.cat([parts[r][:counts[r]] for r in range(world)], dim=0)
    full = full.view(restore)
    if flat:
        full = full.reshape(-1)
    return full.numpy() if as_numpy else full


def gather_columns(local, total_cols: int, group=None):
    """All-gather column blocks of an [M, n_local] result (Gemm sharded along N) into [M, N]."""
    import torch
    as_numpy = isinstance(local, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(local)) if as_numpy else local
    full_t = gather_rows(t.transpose(0, 1).contiguous(), total_cols, group=group)   # [N, M] by row blocks
    full = full_t.transpose(0, 1).contiguous()
    return full.numpy() if as_numpy else full


def combine_ranges(value_range, group=None):
    """DynamicQuantizeLinear over row blocks: every rank holds [min, max] of its own rows (a float64 torch
    tensor on any device, or a numpy array); afterwards every rank holds the range of the whole tensor.
    One all-reduce of two numbers -- the only exchange the operator needs, since scale and zero point follow
    from the range and the codes from them (tensor_ops.c:3760-3809)."""
    import torch
    dist = _dist()
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value_range
    as_numpy = isinstance(value_range, np.ndarray)
    t = torch.from_numpy(np.ascontiguousarray(value_range, dtype=np.float64)) if as_numpy else value_range
    both = torch.stack([-t[0], t[1]])                 # min(a, b) = -max(-a, -b): one MAX reduction serves both ends
    dist.all_reduce(both, op=dist.ReduceOp.MAX, group=group)
    if as_numpy:
        return np.array([-float(both[0]), float(both[1])], dtype=np.float64)
    t[0], t[1] = -both[0], both[1]
    return t


def dynamic_quantize_rows(x_rows, x_dtype: str, lib, group=None):
    """DynamicQuantizeLinear of a tensor whose row blocks live on different GPUs.  ``x_rows`` is this rank's
    block (a DeviceArray); returns (codes of the block, scale, zero point) as DeviceArrays -- scale and zero
    point are identical on every rank.  The range buffer is a torch tensor so that the process group's backend
    (NCCL) can reduce it in place; the library sees it through tops_wrap."""
    import ctypes
    import torch
    from . import capi
    from .device import DeviceArray
    device = torch.device("cuda", torch.cuda.current_device())
    value_range = torch.empty(2, dtype=torch.float64, device=device)
    shape = (ctypes.c_int * 1)(2)
    handle = lib.tops_wrap(ctypes.c_void_p(value_range.data_ptr()), shape, 1, capi.DTYPE_MAP["float64"])
    try:
        if lib.tops_dynamic_quantize_range(x_rows.handle, handle):
            capi.check(lib)
        lib.tops_sync()                               # the library's stream is not torch's
        combine_ranges(value_range, group=group)
        torch.cuda.synchronize(device)
        y = DeviceArray.empty(x_rows.shape, "uint8", lib=lib)
        scale, zero = DeviceArray.empty((1,), "float32", lib=lib), DeviceArray.empty((1,), "uint8", lib=lib)
        if lib.tops_dynamic_quantize_apply(x_rows.handle, handle, y.handle, scale.handle, zero.handle):
            capi.check(lib)
        lib.tops_sync()
    finally:
        lib.free_tensor(handle)
    return y, scale, zero


def init_from_env(backend: Optional[str] = None):
    """Create the default process group from torchrun's environment (no-op for a single process).
    Returns (rank, world, local_rank)."""
    import os
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        dist = _dist()
        if not dist.is_initialized():
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            dist.init_process_group(backend)
    return rank, world, local
