"""Multi-GPU partitioning of the two compute paths: no exchange during compute.

GEMM: rank g of G owns a block of output columns; it needs all of A and B[:, block] (addressed in
place through the leading dimension) and writes C[:, block]. Attention: the B*Hkv (batch, kv-head)
groups are dealt out in contiguous ranges. The only collective is an optional all-gather of the
finished blocks (NCCL on GPUs; the same code runs over gloo on CPU tensors for tests).
The reference has no counterpart: its benchmark.py:546-551 only spreads different problems over GPUs.
"""
from __future__ import annotations

from typing import Callable


def column_blocks(n: int, world: int, align: int = 256) -> list[tuple[int, int]]:
    """Splits [0, n) into `world` contiguous blocks whose interior boundaries are multiples of `align`
    (the widest GEMM tile), as evenly as that allows. Trailing ranks may get empty blocks."""
    if n < 0 or world < 1 or align < 1:
        raise ValueError('column_blocks needs n >= 0, world >= 1, align >= 1')
    units = -(-n // align)
    bounds = [min(n, ((units * r) // world) * align) for r in range(world)] + [n]
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def group_range(groups: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous range of the (batch, kv-head) groups owned by `rank`."""
    if groups < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError('group_range needs groups >= 0 and 0 <= rank < world')
    return (groups * rank) // world, (groups * (rank + 1)) // world


def gemm_column_shard(a, b, rank: int, world: int, mode: str = 'bf16x3', out=None, gemm: Callable | None = None):
    """C[:, block(rank)] = A @ B[:, block(rank)]. Returns (local_c, (begin, end)).

    `b` is the full [K, N] matrix resident on this rank (or any tensor whose columns [begin, end) are
    valid); the block is a strided view, not a copy. `gemm` defaults to the native operator.
    """
    if gemm is None:
        from .ops import gemm as native_gemm
        gemm = native_gemm
    begin, end = column_blocks(b.shape[1], world)[rank]
    if end == begin:
        return a.new_empty((a.shape[0], 0)), (begin, end)
    local = gemm(a, b[:, begin:end], mode, out)
    return local, (begin, end)


def gqa_group_shard(q, k, v, scale: float, rank: int, world: int, out=None, attention: Callable | None = None):
    """Computes the attention output of this rank's (batch, kv-head) groups into `out` (full-size
    [B,Hq,S,D] buffer; only the owned heads are written). Returns (out, (group_begin, group_end))."""
    if attention is None:
        from .ops import gqa_attention
        attention = gqa_attention
    groups = q.shape[0] * k.shape[1]
    begin, end = group_range(groups, world, rank)
    out = attention(q, k, v, scale, out=out, groups=(begin, end))
    return out, (begin, end)


def all_gather_columns(local, blocks: list[tuple[int, int]], group=None):
    """All-gathers equally wide column blocks into the full [M, N] matrix on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    widths = {end - begin for begin, end in blocks}
    if len(widths) != 1 or len(blocks) != world:
        raise ValueError('all_gather_columns needs one equally wide block per rank')
    rows, width = local.shape
    staged = torch.empty((world, rows, width), dtype=local.dtype, device=local.device)
    dist.all_gather(list(staged.unbind(0)), local.contiguous(), group=group)
    return staged.permute(1, 0, 2).reshape(rows, world * width)


def all_gather_groups(out, heads_per_group: int, ranges: list[tuple[int, int]], group=None):
    """All-gathers attention outputs sharded by equal (batch, kv-head) group ranges; `out` is the
    full-size [B,Hq,S,D] buffer whose owned heads this rank has filled."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = {end - begin for begin, end in ranges}
    if len(sizes) != 1 or len(ranges) != world:
        raise ValueError('all_gather_groups needs one equally long group range per rank')
    b, hq, s, d = out.shape
    flat = out.view(b * hq // heads_per_group, heads_per_group * s * d)  # one row per group
    begin, end = ranges[rank]
    gathered = torch.empty_like(flat)
    size = end - begin
    dist.all_gather([gathered[r * size:(r + 1) * size] for r in range(world)], flat[begin:end].contiguous(), group=group)
    return gathered.view(b, hq, s, d)
