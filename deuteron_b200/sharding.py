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
        self._workspace = None   # operand planes of the tallest row block; allocated at the first run, then fixed

    def _planes(self, mode: str, k: int, device):
        """This object's own scratch for the operand planes, sized for the tallest row block, and never replaced: the B
        planes split during the first row block stay valid for the later ones only while the pointer does not move."""
        import torch
        from .ops import gemm_workspace_bytes
        begin, end = self.blocks[self.rank]
        tallest = max((row1 - row0 for row0, row1 in self.rows), default=0)
        need = gemm_workspace_bytes(mode, tallest, end - begin, k) + 1024
        if self._workspace is None or self._workspace[0] != (mode, k) or self._workspace[1].numel() < need:
            self._workspace = ((mode, k), torch.empty(need, dtype=torch.uint8, device=device))
        return self._workspace[1]

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
        planes = self._planes(mode, a.shape[1], a.device) if end > begin and self.rows else None
        if planes is not None:
            # B's planes are split once, before the first row block (1|4: split B only); their place in the workspace
            # depends on the width and depth of B alone, so row blocks of any heights multiply by them (3|8)
            row0, row1 = self.rows[0]
            gemm(a[row0:row1], b_block, mode, out=self.full[row0:row1, begin:end], workspace=planes, phase=1 | 4)
        for row0, row1 in self.rows:
            mine = self.full[row0:row1, begin:end]
            if end > begin:
                gemm(a[row0:row1], b_block, mode, out=mine, workspace=planes, phase=3 | 8)
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


def a_feed_plan(m: int, world: int, row_blocks: int, align: int = 256) -> list[tuple[int, int, int]]:
    """How the rows of A reach the ranks when every rank feeds only its share from host memory.

    A is walked in `row_blocks` row blocks (boundaries on multiples of `align`). Inside a block of `height` rows every
    rank owns `share = ceil(height / world)` consecutive rows (the last owners may own fewer, or none), copies them from
    its host and receives the others' over the interconnect, so that after the exchange of block j every rank holds the
    whole block j. Returns one `(row0, row1, share)` per block; rank r owns rows
    `[row0 + r * share, min(row0 + (r + 1) * share, row1))` of it.
    """
    if world < 1:
        raise ValueError('a_feed_plan needs world >= 1')
    return [(row0, row1, -(-(row1 - row0) // world)) for row0, row1 in row_blocks_for_overlap(m, row_blocks, align)]


def owned_rows(plan: list[tuple[int, int, int]], rank: int) -> list[tuple[int, int]]:
    """Global row ranges of A that `rank` feeds, one per block of `plan` (empty ranges have begin == end)."""
    ranges = []
    for row0, row1, share in plan:
        begin = min(row0 + rank * share, row1)
        ranges.append((begin, min(begin + share, row1)))
    return ranges


class ShardedHostProduct:
    """One C = A @ B over `world` ranks with every operand byte crossing the host link once.

    Rank r owns a block of C's columns. From ITS host memory it feeds its block of B's columns and 1/world of A's rows;
    the ranks exchange their rows of A over the interconnect (all-gather: NCCL over NVLink on GPUs, gloo on CPU
    tensors), so that no rank pulls all of A through the host. The walk is pipelined over row blocks of A: while block
    j is multiplied, block j+1 is being copied in and exchanged and the finished rows of C return to the host.
    Per-element arithmetic is that of the one-launch GEMM: same bits.

    Collective: every rank constructs it with the same arguments and calls `execute` the same number of times.
    The reference has no counterpart (one GPU per problem, benchmark.py:546-551); `compiled` is the Compilation that
    compile_kernel returned for the whole product.
    """

    def __init__(self, compiled, rank: int, world: int, device, group=None, row_blocks: int | None = None,
                 gemm: Callable | None = None):
        import torch
        plan = getattr(compiled, 'plan', None)
        if plan is None or plan.kind != 'gemm':
            raise ValueError('ShardedHostProduct takes the Compilation of a contraction')
        self.m, self.n, self.k, self.mode = plan.params['m'], plan.params['n'], plan.params['k'], plan.params['mode']
        if not 0 <= rank < world:
            raise ValueError('rank must lie in [0, world)')
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device(device)
        self.on_gpu = self.device.type == 'cuda'
        self.columns = column_blocks(self.n, world)[rank]
        if row_blocks is None:
            # enough blocks to overlap the three legs; each at least 512 rows so that a block still fills the tiles
            row_blocks = max(1, min(8, self.m // 1024))
        self.plan = a_feed_plan(self.m, world, row_blocks)
        self.owned = owned_rows(self.plan, rank)
        width = self.columns[1] - self.columns[0]
        # device buffers: one padded [world * share, K] tensor per row block of A, B's column block, C's column block
        self.a_blocks = [torch.empty((world * share, self.k), dtype=torch.float32, device=self.device) for _, _, share in self.plan]
        self.b_block = torch.empty((self.k, width), dtype=torch.float32, device=self.device)
        self.c_block = torch.empty((self.m, width), dtype=torch.float32, device=self.device)
        self.workspace = None
        if gemm is None:
            from .ops import gemm as native_gemm, gemm_workspace_bytes
            gemm = native_gemm
            tallest = max((row1 - row0 for row0, row1, _ in self.plan), default=0)
            need = gemm_workspace_bytes(self.mode, tallest, width, self.k) if width and tallest else 0
            if need:
                self.workspace = torch.empty(need + 1024, dtype=torch.uint8, device=self.device)
        self.gemm = gemm
        if self.on_gpu:
            self.compute = torch.cuda.Stream(device=self.device)
            self.copy_in = torch.cuda.Stream(device=self.device)
            self.exchange = torch.cuda.Stream(device=self.device)
            self.copy_out = torch.cuda.Stream(device=self.device)

    # -- shapes of the caller's host arrays ------------------------------------------------------

    @property
    def owned_row_count(self) -> int:
        return sum(end - begin for begin, end in self.owned)

    def pack_rows(self, full_a):
        """The rows of a full [M, K] host array this rank feeds, in feeding order (what `execute` takes as `a_rows`)."""
        import numpy as np
        parts = [full_a[begin:end] for begin, end in self.owned if end > begin]
        return np.concatenate(parts, axis=0) if parts else np.empty((0, self.k), dtype=np.float32)

    def host_bytes(self) -> tuple[int, int]:
        """(host -> device, device -> host) bytes one `execute` moves on this rank."""
        width = self.columns[1] - self.columns[0]
        return 4 * (self.owned_row_count * self.k + self.k * width), 4 * self.m * width

    # -- one product -----------------------------------------------------------------------------

    def execute(self, a_rows, b_block, c_block=None, *, synchronize: bool = True):
        """a_rows [owned_row_count, K], b_block [K, width]: this rank's HOST arrays (float32, C-contiguous; page-locked
        for full copy rate). Returns C[:, columns] in the host array `c_block` [M, width] (allocated if omitted)."""
        import numpy as np
        import torch
        import torch.distributed as dist
        width = self.columns[1] - self.columns[0]
        if tuple(a_rows.shape) != (self.owned_row_count, self.k) or tuple(b_block.shape) != (self.k, width):
            raise ValueError(f'a_rows must be [{self.owned_row_count}, {self.k}] and b_block [{self.k}, {width}]')
        if a_rows.dtype != np.float32 or b_block.dtype != np.float32:
            raise ValueError('operands must be float32')
        if c_block is None:
            c_block = np.empty((self.m, width), dtype=np.float32)
        if tuple(c_block.shape) != (self.m, width) or c_block.dtype != np.float32:
            raise ValueError(f'c_block must be a float32 array of shape [{self.m}, {width}]')
        a_host = torch.from_numpy(np.ascontiguousarray(a_rows))
        b_host = torch.from_numpy(np.ascontiguousarray(b_block))
        c_host = torch.from_numpy(c_block)
        gpu = self.on_gpu

        class _Lane:
            """A CUDA stream as a context, or nothing on CPU tensors (everything then runs in program order)."""
            def __init__(self, stream):
                self.stream = stream
            def __enter__(self):
                if gpu:
                    self.context = torch.cuda.stream(self.stream)
                    self.context.__enter__()
                return self
            def __exit__(self, *exc):
                if gpu:
                    self.context.__exit__(*exc)
            def mark(self):
                if not gpu:
                    return None
                event = torch.cuda.Event()
                event.record(self.stream)
                return event
            def after(self, event):
                if gpu and event is not None:
                    self.stream.wait_event(event)

        compute = _Lane(self.compute if gpu else None)
        copy_in = _Lane(self.copy_in if gpu else None)
        exchange = _Lane(self.exchange if gpu else None)
        copy_out = _Lane(self.copy_out if gpu else None)
        if gpu:
            # the previous call's readers (products, copies out) are done with the device buffers
            idle = compute.mark()
            for lane in (copy_in, exchange, copy_out):
                lane.after(idle)
            copy_in.after(copy_out.mark())

        fed, at = [], 0
        with copy_in:
            if width:
                self.b_block.copy_(b_host, non_blocking=True)
            b_ready = copy_in.mark()
            for (begin, end), (row0, _, share), block in zip(self.owned, self.plan, self.a_blocks):
                count = end - begin
                if count:
                    first = self.rank * share
                    block[first:first + count].copy_(a_host[at:at + count], non_blocking=True)
                    at += count
                fed.append(copy_in.mark())
        gathered = []
        with exchange:
            for event, (_, _, share), block in zip(fed, self.plan, self.a_blocks):
                exchange.after(event)
                if self.world > 1:
                    mine = block[self.rank * share:(self.rank + 1) * share]
                    dist.all_gather_into_tensor(block, mine, group=self.group)
                gathered.append(exchange.mark())
        done = []
        with compute:
            compute.after(b_ready)
            if width and self.plan:
                row0, row1, _ = self.plan[0]
                # B is split once, before any row block (1|4); every block then multiplies by those planes (3|8)
                self.gemm(self.a_blocks[0][:row1 - row0], self.b_block, self.mode, out=self.c_block[row0:row1],
                          workspace=self.workspace, phase=1 | 4)
            for event, (row0, row1, _), block in zip(gathered, self.plan, self.a_blocks):
                compute.after(event)
                if width:
                    self.gemm(block[:row1 - row0], self.b_block, self.mode, out=self.c_block[row0:row1], workspace=self.workspace,
                              phase=3 | 8)
                done.append(compute.mark())
        with copy_out:
            for event, (row0, row1, _) in zip(done, self.plan):
                copy_out.after(event)
                if width:
                    c_host[row0:row1].copy_(self.c_block[row0:row1], non_blocking=True)
            finished = copy_out.mark()
        if gpu:
            compute.after(finished)
            compute.after(exchange.mark())
            if synchronize:
                self.compute.synchronize()
        return c_block
