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


def row_blocks_for_overlap(m: int, blocks: int = 2, align: int = 256) -> list[tuple[int, int]]:
    """Row ranges a rank's product is computed in when finished rows are pushed to the peers while the rest is
    multiplied: `blocks` ranges with interior boundaries on multiples of `align` (the tallest GEMM tile)."""
    if m < 0 or blocks < 1 or align < 1:
        raise ValueError('row_blocks_for_overlap needs m >= 0, blocks >= 1, align >= 1')
    units = -(-m // align)
    bounds = [min(m, ((units * i) // blocks) * align) for i in range(blocks)] + [m]
    return [(bounds[i], bounds[i + 1]) for i in range(blocks) if bounds[i + 1] > bounds[i]]


class GatheredProduct:
    """C = A @ B with B's columns dealt out over the ranks and the full C on every rank, the exchange overlapped with
    the products.

    The full [M, N] result lives in symmetric memory (every rank can address every rank's copy). A rank multiplies its
    column block a row block at a time into its own copy; as soon as a row block is done, a side stream writes it into
    the same place of every peer's copy (`dtn_push_block`: peer stores over NVLink) while the next row block is being
    multiplied. A
    barrier over the ranks at the end makes every copy complete. Collective: every rank constructs it and calls
    `run` the same number of times. No reference counterpart (the reference runs one GPU per problem).
    """

    def __init__(self, m: int, n: int, rank: int, world: int, device, group=None, row_blocks: int | None = None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric
        self.rank, self.world = rank, world
        self.blocks = column_blocks(n, world)
        # measured on B200: two row blocks are best with one peer (2.61 against 2.68 ms), four with seven (4.83 against 5.1 ms)
        self.rows = row_blocks_for_overlap(m, row_blocks or (2 if world <= 2 else 4))
        self.full = symmetric.empty((m, n), dtype=torch.float32, device=device)
        group = group if group is not None else dist.group.WORLD
        self.handle = symmetric.rendezvous(self.full, group.group_name)
        self.peers = [None if r == rank else self.handle.get_buffer(r, (m, n), torch.float32) for r in range(world)]
        self.push = torch.cuda.Stream(device=device)

    def run(self, a, b_block, mode: str = 'bf16x3', gemm: Callable | None = None):
        """Multiplies `a` [M, K] by this rank's column block `b_block` [K, width]; returns the full product (this rank's
        symmetric buffer), complete on return of the stream's work."""
        import torch
        from .ops import push_block
        if gemm is None:
            from .ops import gemm as native_gemm
            gemm = native_gemm
        begin, end = self.blocks[self.rank]
        compute = torch.cuda.current_stream()
        self.push.wait_stream(compute)   # an earlier run's readers are done with the buffers
        for index, (row0, row1) in enumerate(self.rows):
            mine = self.full[row0:row1, begin:end]
            if end > begin:
                # B's planes are split once; they stay where they are as long as the row blocks are equally tall
                keep_b = index > 0 and row1 - row0 == self.rows[0][1] - self.rows[0][0]
                gemm(a[row0:row1], b_block, mode, out=mine, phase=3 | (8 if keep_b else 0))
            done = torch.cuda.Event()
            done.record(compute)
            self.push.wait_event(done)
            if end > begin:
                with torch.cuda.stream(self.push):
                    # one kernel reads the block once and stores it into every peer's copy, 512 contiguous bytes per warp
                    # and destination; the next rank first, so that no peer is everyone's first target
                    order = [(self.rank + offset) % self.world for offset in range(1, self.world)]
                    for first in range(0, len(order), 7):
                        push_block(mine, [self.peers[r][row0:row1, begin:end] for r in order[first:first + 7]])
        compute.wait_stream(self.push)
        self.handle.barrier()   # every rank's pushes have been issued and completed before anyone reads its copy
        return self.full
