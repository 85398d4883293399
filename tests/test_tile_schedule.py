"""Tile order of the GEMM kernels, checked on the host with the kernels' own scheduling code (no GPU):
every output element is produced exactly once, the tail wave is halved only when that pays, the fused forms visit
the row shards in the order their protocols rely on."""
import itertools

import pytest


@pytest.fixture(scope="module")
def cu():
    import easyllm_b200.ops.cuda as cu
    if not cu.available():
        pytest.skip("kernel library not built")
    cu.lib()
    return cu


def _coverage(units, M, N, bn):
    seen = {}
    for mt, nt, n0, w in units:
        assert 0 <= mt < (M + 127) // 128 and w in (bn, bn // 2) and n0 >= nt * bn and n0 + w <= (nt + 1) * bn
        for c in range(n0, n0 + w, 64 if w >= 64 else w):
            key = (mt, c)
            assert key not in seen, f"column block {key} produced twice"
            seen[key] = 1
    step = 64
    want = {(mt, c) for mt in range((M + 127) // 128) for nt in range((N + bn - 1) // bn)
            for c in range(nt * bn, (nt + 1) * bn, step)}
    assert set(seen) == want


@pytest.mark.parametrize("M,N,ctas", [(128, 256, 148), (4096, 12288, 148), (4096, 4096, 148), (4096, 11008, 148),
                                      (1000, 520, 148), (8192, 8192, 148), (2176, 768, 148), (4096, 32000, 148),
                                      (384, 320, 7), (4096, 4096, 140)])
def test_plain_launch_covers_every_tile_once(cu, M, N, ctas):
    for bn in (256, 128):
        for split in (True, False):
            units = cu.gemm_work_units(M, N, bn=bn, ctas=ctas, allow_split=split)
            _coverage(units, M, N, bn)
            tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
            tail = tiles % ctas
            halved = split and bn == 256 and 0 < tail and 2 * tail <= ctas
            assert len(units) == tiles + (tail if halved else 0)
            assert all(w == bn for *_, w in units[:tiles - (tail if halved else 0)])
            if halved:                          # the two halves of a tail tile are neighbours in the unit order
                rest = units[tiles - tail:]
                assert all(a[:2] == b[:2] and a[3] == b[3] == bn // 2 and b[2] == a[2] + bn // 2
                           for a, b in zip(rest[0::2], rest[1::2]))
    # grouped rasterisation: 16 row tiles share a column tile before the next column tile starts (B stays in L2)
    u = cu.gemm_work_units(4096, 12288, allow_split=False)
    assert [x[0] for x in u[:16]] == list(range(16)) and {x[1] for x in u[:16]} == {0} and u[16][:2] == (0, 1)


@pytest.mark.parametrize("tp,rank", [(2, 0), (2, 1), (4, 0), (4, 3), (8, 5)])
def test_fused_launch_orders(cu, tp, rank):
    M, N = 128 * 8 * tp, 2048
    rows_per_rank_tiles = 8
    for bn in (256, 128):
        tiles_n = N // bn
        ag = cu.gemm_work_units(M, N, bn=bn, fuse=1, tp=tp, rank=rank)
        _coverage(ag, M, N, bn)
        per_phase = rows_per_rank_tiles * tiles_n
        for phase in range(tp):                 # all-gather: own shard first, then the shards in ring order
            owners = {mt // rows_per_rank_tiles for mt, *_ in ag[phase * per_phase:(phase + 1) * per_phase]}
            assert owners == {(rank + phase) % tp}
        rs = cu.gemm_work_units(M, N, bn=bn, fuse=2, tp=tp, rank=rank)
        _coverage(rs, M, N, bn)
        first = [mt // rows_per_rank_tiles for mt, *_ in rs[:tp]]
        assert sorted(first) == list(range(tp))           # reduce-scatter: consecutive tiles feed different owners


@pytest.mark.parametrize("M,N", [(256, 256), (4096, 12288), (1000, 520), (384, 320), (22016, 4096), (4352, 1280)])
def test_pair_kernel_tile_order(cu, M, N):
    tiles = cu.gemm_pair_tiles(M, N)
    tm, tn = (M + 255) // 256, (N + 255) // 256
    assert sorted(tiles) == sorted(itertools.product(range(tm), range(tn)))
    g = min(8, tm)
    assert [t[0] for t in tiles[:g]] == list(range(g)) and {t[1] for t in tiles[:g]} == {0}


@pytest.mark.parametrize("M,N", [(256, 256), (4096, 4096), (4096, 12288), (1000, 520), (4096, 11008), (22016, 4096),
                                 (4096, 32000), (2304, 1280)])
@pytest.mark.parametrize("split", [True, False])
def test_pair_kernel_units_cover_the_output_once_and_halve_only_the_tail(cu, M, N, split):
    clusters, units = cu.gemm_pair_units(M, N, resident=74, allow_split=split)
    tm, tn = (M + 255) // 256, (N + 255) // 256
    cover = {}
    for mt, nt, n0, bn in units:
        assert bn in (128, 256) and n0 == nt * 256 + (0 if bn == 256 or (n0 % 256) == 0 else 128)
        for c in range(n0, n0 + bn, 128):
            assert (mt, c) not in cover
            cover[(mt, c)] = 1
    assert sorted(cover) == sorted((m, c) for m in range(tm) for c in range(0, tn * 256, 128))
    halves = [u for u in units if u[3] == 128]
    if not split:
        assert not halves
    else:
        tail = (tm * tn) % clusters
        want = 2 * tail if (tail and 2 * tail <= clusters) else 0
        assert len(halves) == want
        assert all(u[3] == 256 for u in units[:len(units) - want])     # only the last wave is cut
        if want:                                                        # and it now fits half a wave's worth of clusters
            assert want <= clusters


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("M,N", [(4096, 4096), (4096, 6144), (8192, 2048)])
def test_pair_kernel_fused_orders(cu, tp, M, N):
    """CTA-pair fused launches: every 256-row tile once; all-gather form starts on the local shard and takes the
    others in ring order; reduce forms feed every owner from the first tiles on and are never halved."""
    tm, tn = M // 256, (N + 255) // 256
    tpr = tm // tp
    for rank in (0, tp - 1):
        clusters, ag = cu.gemm_pair_units(M, N, resident=74, fuse=1, tp=tp, rank=rank, n_comm=8)
        assert clusters == 70
        cover = {}
        for mt, nt, n0, bn in ag:
            for c in range(n0, n0 + bn, 128):
                assert (mt, c) not in cover
                cover[(mt, c)] = 1
        assert len(cover) == tm * tn * 2
        whole = [u for u in ag if u[3] == 256]
        per_phase = tpr * tn
        for phase in range(tp - 1):           # the last phase may end in half-width units
            owners = {mt // tpr for mt, *_ in whole[phase * per_phase:(phase + 1) * per_phase]}
            assert owners == {(rank + phase) % tp}
        for fuse in (2, 3):
            ncl, rs = cu.gemm_pair_units(M, N, resident=74, fuse=fuse, tp=tp, rank=rank, n_comm=8 if fuse == 3 else 0)
            if fuse == 3:
                assert all(u[3] == 256 for u in rs) and len(rs) == tm * tn
                assert sorted((u[0], u[1]) for u in rs) == sorted(itertools.product(range(tm), range(tn)))
                assert sorted(mt // tpr for mt, *_ in rs[:tp]) == list(range(tp))
                continue
            # an under-filled last wave is cut into half-width units only where every tile of it is the rank's own
            halves = [u for u in rs if u[3] == 128]
            assert all(mt // tpr == rank for mt, *_ in halves) and len(halves) % 2 == 0
            assert len(halves) // 2 <= min(tpr * tn, -(-2 * ncl // tp))
            cover = sorted((mt, c) for mt, nt, n0, bn in rs for c in range(n0, n0 + bn, 128))
            assert cover == sorted(itertools.product(range(tm), range(0, tn * 256, 128)))
            rs = [u for i, u in enumerate(rs) if u[3] == 256 or rs[i - 1][:2] != u[:2] or rs[i - 1][3] == 256]
            assert len(rs) == tm * tn
            # reduce-scatter (summed in the epilogue): every owner's tiles come in the same (raster) order on every
            # rank, and an own tile trails the position where the peers compute the same tile by about two waves
            n = tpr * tn
            lag = min(n, -(-2 * ncl // tp))
            per_owner = {o: [(mt - o * tpr, nt) for mt, nt, *_ in rs if mt // tpr == o] for o in range(tp)}
            assert all(per_owner[o] == per_owner[rank] for o in range(tp))
            pos = {(mt, nt): i for i, (mt, nt, *_) in enumerate(rs)}
            for k, (mi, nt) in enumerate(per_owner[rank]):
                own_at = pos[(rank * tpr + mi, nt)]
                for o in range(tp):
                    if o != rank:
                        # position of tile k of owner `rank` in the PEER's order equals, by symmetry, the position
                        # of tile k of owner o' = (o shifted) here; the peers' tiles of round k sit at or before it
                        assert pos[(o * tpr + mi, nt)] <= own_at
                if k + lag < n:
                    assert own_at > pos[((rank + 1) % tp * tpr + per_owner[rank][k + lag][0], per_owner[rank][k + lag][1])]
            assert [mt // tpr for mt, *_ in rs[-lag:]] == [rank] * lag
        _, rs = cu.gemm_pair_units(M, N, resident=74, fuse=3, tp=tp, rank=rank, n_comm=8)
        # the reduce role's queue visits every owned 128-row tile once, in the order the owner's tiles are emitted
        order = cu.reduce_tile_order(M // tp, tn, tp, pair=True)
        assert sorted(order) == sorted(itertools.product(range(2 * tpr), range(tn)))
        emitted = []
        for mt, nt, *_ in rs:
            if mt // tpr == rank:
                emitted += [(2 * (mt - rank * tpr), nt), (2 * (mt - rank * tpr) + 1, nt)]
        assert order == emitted
        single = cu.reduce_tile_order(M // tp, tn, tp, pair=False)
        assert sorted(single) == sorted(order)
        rs1 = cu.gemm_work_units(M, N, bn=256, fuse=2, tp=tp, rank=rank)
        assert single == [(mt - rank * 2 * tpr, nt) for mt, nt, *_ in rs1 if mt // (2 * tpr) == rank]


def _row_starts(T, doc_lens):
    rs, start = [], 0
    for n in doc_lens:
        rs += [start] * n
        start += n
    assert len(rs) == T
    return rs


@pytest.mark.parametrize("T,docs", [(512, [512]), (1000, [1000]), (1024, [100, 28, 128, 256, 1, 511]),
                                    (777, [255, 2, 520]), (640, [129, 127, 128, 256]), (300, [300]),
                                    (2048, [5] * 409 + [3]), (1536, [1, 1535])])
def test_attention_forward_plan_covers_visible_keys_and_skips_masks_only_when_safe(cu, T, docs):
    rs = _row_starts(T, docs)
    plan = cu.flash_fwd_plan(rs)
    assert len(plan) == 2 * ((T + 255) // 256)
    for idx, (kv_lo, n, bits) in enumerate(plan):
        first = (idx // 2) * 256 + (idx % 2) * 128
        rows = range(first, min(first + 128, T))
        if not rows:
            assert n == 0
            continue
        assert kv_lo == rs[(idx // 2) * 256]
        # every key a row may see lies inside the walked range, and the last walked tile is not wasted
        assert all(kv_lo <= rs[i] and i < kv_lo + n * 128 for i in rows)
        assert rows[-1] >= kv_lo + (n - 1) * 128
        for j in range(min(n, 31)):
            if bits >> j & 1:
                continue
            k0 = kv_lo + j * 128                # an unmasked tile: every (row, key) pair in it must be visible
            assert k0 + 127 < T
            assert all(rs[i] <= k0 and k0 + 127 <= i for i in rows), (idx, j)


@pytest.mark.parametrize("tp", [2, 4, 8])
@pytest.mark.parametrize("M,N,resident", [(4096, 4096, 74), (2048, 1024, 74), (8192, 2048, 70), (4096, 8192, 37)])
def test_reduce_scatter_schedule_cannot_deadlock_across_ranks(cu, tp, M, N, resident):
    """The reduce-scatter kernel walks its units in order on every cluster; a tile the rank owns waits for the flags of
    all peers, a tile another rank owns never waits.  Replay that with the kernel's own unit order for every rank:
    clusters advance in lock step, a unit finishes when its dependencies finished in an EARLIER round.  Every rank must
    drain (no cycle of waits between ranks), and an own tile must find its peers' partial sums finished at least one
    round before its own turn in the steady state, so that the epilogue does not stall the tensor core."""
    tm = M // 256
    if tm % tp:
        pytest.skip("row tiles do not divide over the ranks")
    tpr = tm // tp
    order = {}
    for rank in range(tp):
        ncl, units = cu.gemm_pair_units(M, N, resident=resident, fuse=2, tp=tp, rank=rank, n_comm=0)
        order[rank] = (ncl, units)
    done_round = {}                              # (producer rank, mt, nt) -> round in which its partial was finished
    ptr = {(r, c): c for r in range(tp) for c in range(order[r][0])}      # next unit of every cluster
    waits = 0
    for rnd in range(10000):
        progressed, finished = False, []
        for (r, c), u in ptr.items():
            ncl, units = order[r]
            if u >= len(units):
                continue
            mt, nt, n0, bn = units[u]
            owner = mt // tpr
            if owner == r:
                ready = all(done_round.get((s, mt, nt), 1 << 30) < rnd for s in range(tp) if s != r)
                if not ready:
                    waits += 1
                    continue
            finished.append((r, c, mt, nt, owner))
        for r, c, mt, nt, owner in finished:
            if owner != r:
                done_round[(r, mt, nt)] = rnd
            ptr[(r, c)] += order[r][0]
            progressed = True
        if all(u >= len(order[r][1]) for (r, c), u in ptr.items()):
            break
        assert progressed, f"ranks wait for one another in round {rnd}"
    else:
        raise AssertionError("schedule did not drain")
    n_units = sum(len(order[r][1]) for r in range(tp))
    ideal_rounds = -(-len(order[0][1]) // order[0][0])
    assert rnd + 1 <= ideal_rounds + 1, (rnd + 1, ideal_rounds)      # at most one round lost to waiting
    assert waits <= order[0][0] * tp, (waits, n_units)               # and only around the start
