"""Host-side model of the balanced schedule's arithmetic (spmm_sm100.cu: Flat, SegGen, sum_split_items_kernel):
equal contiguous ranges of the flattened (item, step) sequence, the owner of a position, which scratch tile a
segment goes to and which block of the summation kernel adds which tiles.  The CUDA code uses the same integer
formulas; the GPU test test_balanced_schedule_for_skewed_matrices checks the kernels themselves."""
import numpy as np


def _check(ns_list, n_tiles, G, rng):
    gsp = np.concatenate([[0], np.cumsum(ns_list)])
    total = int(gsp[-1]) * n_tiles
    if total == 0:
        return
    rb = lambda c: total * c // G                     # Flat::range_begin
    owner = lambda p: ((p + 1) * G - 1) // total      # Flat::range_owner
    for p in rng.integers(0, total, 100):
        c = owner(int(p))
        assert rb(c) <= p < rb(c + 1)

    def locate(p):                                    # Flat::group_of + the skip over empty groups
        g = int(np.searchsorted(gsp * n_tiles, p, side="right") - 1)
        while gsp[g + 1] * n_tiles <= p:
            g += 1
        ns = int(gsp[g + 1] - gsp[g])
        off = p - int(gsp[g]) * n_tiles
        t = off // ns
        return g, t, ns, int(gsp[g]) * n_tiles + t * ns, off - t * ns

    segs = {}
    for c in range(G):                                # SegGen::next, balanced branch
        p, pe = rb(c), rb(c + 1)
        while p < pe:
            g, t, ns, p0, k0 = locate(p)
            k1 = min(ns, k0 + (pe - p))
            segs.setdefault((g, t), []).append((k0, k1, k0 != 0 or k1 != ns, c * 2 + (1 if rb(c) < p0 else 0)))
            p += k1 - k0
    handled = {}
    for c in range(1, G):                             # sum_split_items_kernel, block c - 1
        b = rb(c)
        if b <= 0 or b >= total:
            continue
        g, t, ns, p0, _ = locate(b)
        if b == p0 or (c > 1 and rb(c - 1) > p0):
            continue
        assert (g, t) not in handled
        handled[(g, t)] = [cc * 2 + (1 if rb(cc) < p0 else 0) for cc in range(c - 1, owner(p0 + ns - 1) + 1)
                           if rb(cc) != rb(cc + 1)]
    for item, ss in segs.items():
        assert sum(k1 - k0 for k0, k1, _, _ in ss) == int(gsp[item[0] + 1] - gsp[item[0]])  # every step exactly once
        if any(cut for _, _, cut, _ in ss):
            assert [slot for _, _, _, slot in ss] == handled[item]  # the summation reads exactly the tiles written
        else:
            assert item not in handled and len(ss) == 1
    slots = [slot for ss in segs.values() for _, _, cut, slot in ss if cut]
    assert len(slots) == len(set(slots))              # no tile is written twice in a launch


def test_balanced_schedule_arithmetic():
    rng = np.random.default_rng(0)
    for _ in range(300):
        ng = int(rng.integers(1, 40))
        ns = rng.integers(0, 50, ng)
        if rng.random() < 0.3:
            ns[rng.integers(0, ng)] = int(rng.integers(500, 5000))  # one heavy group
        if rng.random() < 0.2:
            ns = rng.integers(0, 3, ng)                              # fewer steps than CTAs
        _check(ns, int(rng.integers(1, 4)), int(rng.integers(1, 149)), rng)


def test_cut_last_round_at_multiples_of_a_quantum():
    """The round-robin schedule cuts the items of the last round into P segments at k = (ns / q) * j / P * q
    (spmm_sched.cuh, SegGen<0>): q = 1 for the 16-row kernels, q = 2 for the tall kernel, whose plans pad every group
    to an even number of steps and whose MMA warps take the steps two at a time.  Restated here: the segments tile
    [0, ns) in order, every cut is a multiple of q, and the last segment ends at ns whatever ns is."""
    rng = np.random.default_rng(1)
    for _ in range(2000):
        q = int(rng.choice([1, 2]))
        ns = int(rng.integers(0, 4000))
        if q == 2:
            ns += ns & 1  # tall plans: even step counts
        P = int(rng.integers(1, 5))  # kMaxTailParts = 4
        nq = ns // q
        cuts = [(nq * j // P) * q for j in range(P)] + [ns]
        for j in range(P):
            k0, k1 = cuts[j], (ns if j + 1 == P else (nq * (j + 1) // P) * q)
            assert k1 == cuts[j + 1] and 0 <= k0 <= k1 <= ns
            assert k0 % q == 0 and (k1 % q == 0 or k1 == ns)
            if q == 2:
                assert (k1 - k0) % 2 == 0  # a pair of steps never spans two segments
        assert cuts[0] == 0 and cuts[-1] == ns
