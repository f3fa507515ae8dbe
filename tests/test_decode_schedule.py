"""Host-side restatement of the balanced decode schedule (csrc/tc_fwd2.cuh: sched_tiles, line_locate,
cursor_init, cursor_next) checked for every property the kernel relies on, on CPU, for random batches:
every 256-key tile of every sequence is attended exactly once, a sequence is never cut into more pieces
than the plan promises (so no piece is written past the partial slabs), piece indices are 0 .. n-1, and a
length beyond what the page table describes is clamped.  The plan itself (schedule and minimum run length)
comes from the library through fdmla_decode_plan, which needs no GPU.
"""
import ctypes
import random

T = 256            # keys per tile
MAX_IN_KERNEL_PIECES = 4


def plan(L, B, H, page_size, max_pages, splits):
    qmin, units = ctypes.c_int(0), ctypes.c_int(0)
    mode = L.fdmla_decode_plan(B, H, 576, 512, page_size, max_pages, splits, 1, ctypes.byref(qmin), ctypes.byref(units))
    return mode, qmin.value, units.value


def sched_tiles(seq):
    return max((seq + T - 1) // T, 1)


def walk(lens, cap, n_clusters, quota_min):
    """(cluster, g, first tile, end tile, piece index, pieces) of every item, in the order each cluster visits them."""
    seqs = [min(max(s, 0), cap) for s in lens]
    nts = [sched_tiles(s) for s in seqs]
    first_of, total = [], 0
    for nt in nts:
        first_of.append(total)
        total += nt
    q = max((total + n_clusters - 1) // n_clusters, quota_min, 1)
    items = []
    for cid in range(n_clusters):
        lo = cid * q
        if lo >= total:
            continue
        hi = min(lo + q, total)
        locate = lambda pos: max(g for g in range(len(nts)) if first_of[g] <= pos)
        g_first, g_last = locate(lo), locate(hi - 1)
        order = ([g_last] + list(range(g_first, g_last))) if g_last != g_first else [g_first]
        for g in order:
            first, nt = first_of[g], nts[g]
            a, b = max(first, lo), min(first + nt, hi)
            pieces = (first + nt - 1) // q - first // q + 1
            items.append((cid, g, a - first, b - first, cid - first // q, pieces))
    return items, nts, q


def check(lens, cap, n_clusters, quota_min, max_pieces):
    items, nts, q = walk(lens, cap, n_clusters, quota_min)
    seen = [[0] * nt for nt in nts]
    piece_ids = [set() for _ in nts]
    for cid, g, ta, tb, split, pieces in items:
        assert 0 <= ta < tb <= nts[g]
        assert 1 <= pieces <= max_pieces, (pieces, max_pieces, lens, q)
        assert 0 <= split < pieces
        assert split not in piece_ids[g]
        piece_ids[g].add(split)
        for t in range(ta, tb):
            seen[g][t] += 1
    for g, nt in enumerate(nts):
        assert seen[g] == [1] * nt, f"sequence {g} not covered exactly once"
        assert piece_ids[g] == set(range(len(piece_ids[g])))
    # the runs are contiguous: cluster c's items together hold tiles [c q, (c + 1) q)
    per_cluster = {}
    for cid, g, ta, tb, split, pieces in items:
        per_cluster[cid] = per_cluster.get(cid, 0) + (tb - ta)
    assert all(v <= q for v in per_cluster.values())


def test_balanced_schedule_properties_on_random_batches():
    from flashdmla import _lib
    L = _lib.lib()
    rnd = random.Random(5)
    modes = set()
    for case in range(400):
        B = rnd.choice([1, 2, 8, 40, 74, 75, 128, 150, 500])
        H = rnd.choice([2, 16, 128])
        page = rnd.choice([64, 128])
        mx = rnd.choice([64, 300, 1000, 4096, 9000, 131072])
        max_pages = (mx + page - 1) // page
        splits = rnd.choice([2, 3, 4, 5, 9, 33, 64])
        mode, qmin, units = plan(L, B, H, page, max_pages, splits)
        modes.add(mode)
        if mode == 0:
            continue
        assert units == 74 and qmin >= 1          # no device here: the B200 constant
        max_pieces = splits if mode == 1 else min(splits - 1, MAX_IN_KERNEL_PIECES)
        cap = max_pages * page
        # lengths: ragged, empty, and some beyond what the page table can describe (clamped by the kernels)
        lens = [rnd.choice([0, 1, rnd.randint(1, mx), mx, mx, cap + rnd.randint(1, 10 ** 6), -3]) for _ in range(B)]
        check(lens, cap, units, qmin, max_pieces)
        check([mx] * B, cap, units, qmin, max_pieces)
    assert modes == {0, 1, 2}, f"the random cases should reach every schedule, got {modes}"


def test_plan_of_the_headline_decode_configuration():
    """B=128, H=128, Skv=4096: one work item per sequence (the balanced runs would save four of 32 tiles per CTA
    pair, the partial rows and merges they need cost more); forty such sequences with four slabs are handed out as
    balanced runs merged in the attention kernel, a sequence cut into three pieces at most."""
    from flashdmla import _lib
    L = _lib.lib()
    splits = L.fdmla_decode_suggest_splits(128, 128, 4096, 576, 512, 64, 1)
    assert splits == 1 and plan(L, 128, 128, 64, 64, splits)[0] == 0
    mode, qmin, units = plan(L, 40, 64, 64, 64, 4)
    assert (mode, units, qmin) == (2, 74, 8)
    items, nts, q = walk([4096] * 40, 4096, units, qmin)
    assert q == 9 and max(p for *_, p in items) == 3
    # few long sequences are cut many times: never merged by single thread blocks inside the attention kernel
    splits = L.fdmla_decode_suggest_splits(8, 128, 131072, 576, 512, 64, 1)
    mode, qmin, units = plan(L, 8, 128, 64, 2048, splits)
    assert mode in (0, 1) and splits >= 6
    # unsupported shapes and single slabs stay on the plain schedule
    assert plan(L, 8, 128, 64, 64, 1)[0] == 0
    assert L.fdmla_decode_plan(8, 128, 160, 128, 64, 64, 4, 1, None, None) == 0
    assert L.fdmla_decode_plan(0, 128, 576, 512, 64, 64, 4, 1, None, None) < 0
