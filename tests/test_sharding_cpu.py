"""Multi-GPU partition logic on CPU: world_size-2 gloo ranks, the oracle standing in for the kernels.

The data path has no collective; what is tested is that the column-block / group partition covers the
output exactly once and that the optional all-gather reassembles it, with the same functions
(sharding.*) the GPU path uses.
"""
import multiprocessing as mp
import os

import numpy as np
import pytest

from deuteron_b200 import sharding
from oracle import reference_math as R


def test_column_blocks_cover_exactly_once():
    for n, world in ((8192, 1), (8192, 2), (8192, 8), (1000, 4), (256, 8), (0, 3), (777, 2)):
        blocks = sharding.column_blocks(n, world)
        assert len(blocks) == world and blocks[0][0] == 0 and blocks[-1][1] == n
        assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        assert all(begin % 256 == 0 for begin, end in blocks if begin < n)
    assert sharding.column_blocks(8192, 8) == [(1024 * r, 1024 * (r + 1)) for r in range(8)]
    with pytest.raises(ValueError):
        sharding.column_blocks(10, 0)


def test_group_ranges_cover_exactly_once():
    for groups, world in ((32, 1), (32, 2), (32, 8), (5, 4), (0, 2)):
        ranges = [sharding.group_range(groups, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == groups
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        sharding.group_range(4, 2, 2)


def _worker(rank: int, world: int, port: int, queue) -> None:
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        a = torch.from_numpy(R.seeded_uniform(7, (64, 96)))
        b = torch.from_numpy(R.seeded_uniform(11, (96, 512)))

        def cpu_gemm(left, right, mode, out):
            return torch.from_numpy(R.gemm_f64(left.numpy(), right.numpy()).astype(np.float32))

        local, (begin, end) = sharding.gemm_column_shard(a, b, rank, world, gemm=cpu_gemm)
        full = sharding.all_gather_columns(local, sharding.column_blocks(512, world))
        expected = R.gemm_f64(a.numpy(), b.numpy()).astype(np.float32)
        gemm_ok = bool(np.array_equal(full.numpy(), expected)) and (begin, end) == (256 * rank, 256 * (rank + 1))

        q = torch.from_numpy(R.seeded_normal(1, (2, 4, 16, 8)))
        k = torch.from_numpy(R.seeded_normal(2, (2, 2, 16, 8)))
        v = torch.from_numpy(R.seeded_normal(3, (2, 2, 16, 8)))

        def cpu_attention(q, k, v, scale, out=None, groups=None):
            out = torch.zeros(q.shape, dtype=torch.float32) if out is None else out
            ratio = q.shape[1] // k.shape[1]
            heads = [(g // k.shape[1], (g % k.shape[1]) * ratio + j) for g in range(*groups) for j in range(ratio)]
            result = R.gqa_attention_f64(q.numpy(), k.numpy(), v.numpy(), scale, heads=heads)
            for bi, hi in heads:
                out[bi, hi] = torch.from_numpy(result[bi, hi].astype(np.float32))
            return out

        mine, owned = sharding.gqa_group_shard(q, k, v, 0.35, rank, world, attention=cpu_attention)
        ranges = [sharding.group_range(4, world, r) for r in range(world)]
        gathered = sharding.all_gather_groups(mine, 2, ranges)
        expected = R.gqa_attention_f64(q.numpy(), k.numpy(), v.numpy(), 0.35).astype(np.float32)
        attention_ok = bool(np.array_equal(gathered.numpy(), expected)) and owned == ranges[rank]

        # host-fed product: each rank feeds 1/world of A's rows and its block of B's columns, A's rows are exchanged
        from deuteron_b200 import Options, compile_kernel, schedules
        m, n, k = 1280, 512, 128
        compiled = compile_kernel(*schedules.matmul_example(m, n, k), options=Options(contraction_precision='bf16x3'))
        full_a, full_b = R.seeded_uniform(7, (m, k)), R.seeded_uniform(11, (k, n))
        calls = []

        def cpu_phase_gemm(left, right, mode, out=None, workspace=None, phase=3):
            calls.append((tuple(left.shape), phase))
            if phase & 2:
                out.copy_(torch.from_numpy(R.gemm_f64(left.numpy(), right.numpy()).astype(np.float32)))
            return out

        product = sharding.ShardedHostProduct(compiled, rank, world, 'cpu', row_blocks=3, gemm=cpu_phase_gemm)
        begin, end = product.columns
        fed = product.pack_rows(full_a)
        block = product.execute(fed, np.ascontiguousarray(full_b[:, begin:end]))
        expected = R.gemm_f64(full_a, full_b).astype(np.float32)[:, begin:end]
        host_ok = (bool(np.array_equal(block, expected)) and fed.shape[0] * world == m
                   and calls[0][1] == 5 and all(phase == 11 for _, phase in calls[1:]) and len(calls) == 4
                   and product.host_bytes() == (4 * (fed.shape[0] * k + k * (end - begin)), 4 * m * (end - begin)))
        queue.put((rank, gemm_ok, attention_ok, host_ok))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_assemble_sharded_outputs():
    context = mp.get_context('spawn')
    queue = context.Queue()
    port = 29500 + os.getpid() % 400
    workers = [context.Process(target=_worker, args=(rank, 2, port, queue)) for rank in range(2)]
    for worker in workers:
        worker.start()
    results = sorted(queue.get(timeout=60) for _ in workers)
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    assert results == [(0, True, True, True), (1, True, True, True)]


def test_row_blocks_for_overlap_cover_the_rows_on_tile_boundaries():
    from deuteron_b200 import sharding
    for m, blocks in ((8192, 2), (8192, 4), (300, 4), (256, 2), (1, 3), (0, 2), (5000, 3)):
        ranges = sharding.row_blocks_for_overlap(m, blocks)
        assert [r[0] for r in ranges] == ([0] + [r[1] for r in ranges[:-1]] if ranges else [])
        assert (ranges[-1][1] if ranges else 0) == m
        assert all(end > begin for begin, end in ranges) and len(ranges) <= blocks
        assert all(begin % 256 == 0 for begin, _ in ranges)
    with pytest.raises(ValueError):
        sharding.row_blocks_for_overlap(8, 0)


def test_a_feed_plan_gives_every_row_to_exactly_one_rank():
    for m, world, blocks in ((8192, 8, 8), (8192, 2, 4), (1000, 3, 2), (300, 4, 4), (256, 8, 1), (0, 2, 2), (5000, 7, 3)):
        plan = sharding.a_feed_plan(m, world, blocks)
        seen = np.zeros(m, dtype=np.int32)
        for rank in range(world):
            owned = sharding.owned_rows(plan, rank)
            assert len(owned) == len(plan)
            for (begin, end), (row0, row1, share) in zip(owned, plan):
                assert row0 <= begin <= end <= row1 and end - begin <= share
                seen[begin:end] += 1
        assert (seen == 1).all()
    assert sharding.a_feed_plan(8192, 8, 4) == [(2048 * j, 2048 * (j + 1), 256) for j in range(4)]
    assert sharding.owned_rows(sharding.a_feed_plan(8192, 8, 4), 3) == [(2048 * j + 768, 2048 * j + 1024) for j in range(4)]
    with pytest.raises(ValueError):
        sharding.a_feed_plan(8, 0, 1)


def test_tile_schedule_covers_the_output_once_and_balances_the_pairs():
    import ctypes as ct
    from deuteron_b200 import native

    def schedule(m, n, pairs=74):
        entries, rounds = (ct.c_uint32 * 640)(), ct.c_int()
        longest, uniform = ct.c_double(), ct.c_double()
        native.call('dtn_gemm_tile_schedule', m, n, pairs, entries, 640, ct.byref(rounds), ct.byref(longest), ct.byref(uniform))
        table = np.array(entries[:rounds.value * pairs], dtype=np.uint32).reshape(rounds.value, pairs) if rounds.value else None
        return table, longest.value, uniform.value

    for m, n in ((8192, 2048), (4096, 4096), (1024, 1024), (1536, 1536), (768, 520), (8192, 2000)):
        table, longest, uniform = schedule(m, n)
        assert table is not None and longest <= 0.97 * uniform, (m, n)
        cover = np.zeros(((m + 255) // 256, (n + 31) // 32), dtype=int)
        for entry in table.ravel():
            if entry:
                band, first, width = int(entry & 0xfff), int((entry >> 12) & 0xfff), int(entry >> 24)
                assert 1 <= width <= 8
                cover[band, first:first + width] += 1
        assert (cover == 1).all()
        # rounds walk the bands in order: no tile of a round lies above a tile of the round before
        top = [min(int(e & 0xfff) for e in row if e) for row in table]
        bottom = [max(int(e & 0xfff) for e in row if e) for row in table]
        assert all(bottom[j] <= top[j + 1] + 1 for j in range(len(top) - 1))
    # a quarter of the 8192^3 product on 74 pairs: 3.46 rounds of 256-wide tiles; three of them and one 128-wide tile
    # per pair instead of four rounds (a 128-wide tile costs 0.56 of a 256-wide one, widths in between cost as 256)
    table, longest, uniform = schedule(8192, 2048)
    widths = sorted({int(e >> 24) * 32 for e in table.ravel() if e})
    assert widths == [128, 256] and longest < 0.92 * uniform
    per_pair = [sorted(int(e >> 24) * 32 for e in table[:, w] if e) for w in range(74)]
    assert max(sum(p) for p in per_pair) <= 3 * 256 + 128 + 128
    # an eighth of it: 1.73 rounds; nothing cheaper than two rounds of 256-wide tiles exists, the plain walk stays;
    # large outputs keep it too
    assert schedule(8192, 1024)[0] is None and schedule(8192, 8192)[0] is None and schedule(8192, 4096)[0] is None


def test_skinny_plan_gives_every_cta_the_same_share_and_orders_the_contributors():
    """The streamed kernel for at most 16 rows: units of 64 k-rows x 128 columns, one contiguous range per CTA."""
    import ctypes as ct
    from deuteron_b200 import native

    def plan(n, k, workers):
        k_tiles, n_tiles = (k + 63) // 64, (n + 127) // 128
        begin, first, last = (ct.c_int64 * (workers + 1))(), (ct.c_int * n_tiles)(), (ct.c_int * n_tiles)()
        native.call('dtn_gemm_skinny_plan', n, k, workers, begin, first, last)
        return k_tiles, n_tiles, list(begin), list(first), list(last)

    for n, k, workers in ((8192, 8192, 148), (4100, 2052, 148), (128, 65536, 148), (65536, 64, 148), (2084, 1028, 148), (8192, 8192, 132), (256, 128, 4)):
        k_tiles, n_tiles, begin, first, last = plan(n, k, workers)
        units = k_tiles * n_tiles
        assert begin[0] == 0 and begin[-1] == units
        sizes = [begin[w + 1] - begin[w] for w in range(workers)]
        assert min(sizes) >= 1 and max(sizes) - min(sizes) <= 1          # equal shares: every SM reads the same bytes
        owner = np.repeat(np.arange(workers), sizes)                      # CTA of every unit
        slots = set()
        for block in range(n_tiles):
            inside = owner[block * k_tiles:(block + 1) * k_tiles]
            assert first[block] == inside[0] and last[block] == inside[-1]
            assert sorted(set(inside.tolist())) == list(range(first[block], last[block] + 1))   # contiguous, in order
            for w in range(first[block], last[block] + 1):
                slots.add((w + block, w, block))
        # the workspace slot of a (CTA, column block) pair is CTA + block: no two pairs share one, none beyond workers + blocks
        keys = [slot for slot, _, _ in slots]
        assert len(keys) == len(set(keys)) and max(keys) < workers + n_tiles
    with pytest.raises(ValueError):
        plan(128, 64, 2)   # one unit cannot be shared by two CTAs
