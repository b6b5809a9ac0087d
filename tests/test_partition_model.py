"""A host-side model of the decode kernel's index arithmetic (tile list, per-CTA ranges,
partial-slot numbering, arrival counts of the one- and two-level split-K merge), checked
for the invariants the device code relies on.  Constants mirror
peerkv_b200/csrc/decode_kernel.cuh; the scratch sizes mirror pkv_shard_create."""
import random

import pytest

TILE, GROUP_CTAS, GROUP_THRESHOLD, MAX_WPH, MAX_CTAS = 16, 16, 32, 2, 256


def seq_tiles(length, page_size):
    tpp = (page_size + TILE - 1) // TILE
    full, rem = divmod(length, page_size)
    return full * tpp + (rem + TILE - 1) // TILE


def uniform_bounds(total, n_cta):
    per = (total + n_cta - 1) // n_cta
    return [min(total, c * per) for c in range(n_cta + 1)]


def weighted_bounds(total, weights):
    w = [min(max(x, 0.5), 2.0) for x in weights]
    tot = sum(w)
    cum, out = 0.0, [0]
    for i, x in enumerate(w):
        cum += x
        b = min(max(int(total * cum / tot), 0), total)
        out.append(total if i == len(w) - 1 else b)
    return out


def find_cta(bound, g):
    lo, hi = 0, len(bound) - 1
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if bound[mid] <= g:
            lo = mid
        else:
            hi = mid
    return lo


def simulate(lens, page_size, n_cta, wph, bound_fn):
    """Returns per-sequence (expected arrivals per kv-head, slots written, group slots)."""
    B = len(lens)
    prefix = [0]
    for L in lens:
        prefix.append(prefix[-1] + (seq_tiles(L, page_size) if L > 0 else 0))
    total = prefix[-1]
    bound = bound_fn(total, n_cta)
    assert bound[0] == 0 and bound[-1] == total and all(a <= b for a, b in zip(bound, bound[1:]))
    grp_slot0 = (n_cta + B) * MAX_WPH
    n_slots = grp_slot0 + (n_cta + GROUP_CTAS - 1) // GROUP_CTAS + B
    covered = [0] * total
    sib_slot0 = grp_slot0 // MAX_WPH          # where the second warp of a head parks its partial
    flushes = {}            # seq -> list of (cta, slot): what the merge of the sequence reads
    parked = set()
    for c in range(n_cta):
        g0, g1 = bound[c], bound[c + 1]
        g = g0
        while g < g1:
            s = max(i for i in range(B) if prefix[i] <= g and prefix[i + 1] > g)
            seg_end = min(g1, prefix[s + 1])
            for t in range(g, seg_end):
                covered[t] += 1
            # with two warps per head the second one parks its partial in a slot of its own,
            # the first folds it in: ONE slot per (CTA, sequence) reaches the merge either way
            slot = c + s
            assert 0 <= slot < sib_slot0
            flushes.setdefault(s, []).append((c, slot))
            if wph > 1:
                park = sib_slot0 + c + s
                assert sib_slot0 <= park < grp_slot0 and park not in parked, "parking slots do not collide"
                parked.add(park)
            g = seg_end
    assert all(x == 1 for x in covered), "every tile is processed exactly once"
    seen_slots, seen_gslots = set(), set()
    for s in range(B):
        t0, t1 = prefix[s], prefix[s + 1]
        if t1 == t0:
            assert s not in flushes
            continue
        c0, c1 = find_cta(bound, t0), find_cta(bound, t1 - 1)
        assert sorted({c for c, _ in flushes[s]}) == list(range(c0, c1 + 1)), "consecutive CTAs, none empty"
        slot_lo, slot_hi = c0 + s, c1 + s
        slots = sorted(sl for _, sl in flushes[s])
        assert slots == list(range(slot_lo, slot_hi + 1)), "the merge reads exactly the slots that were written"
        assert not (set(slots) & seen_slots), "no slot is shared by two sequences"
        seen_slots |= set(slots)
        if slot_hi - slot_lo + 1 > GROUP_THRESHOLD:
            g_lo, g_hi = c0 // GROUP_CTAS, c1 // GROUP_CTAS
            arrivals = 0
            for gi in range(g_lo, g_hi + 1):
                cg0, cg1 = max(c0, gi * GROUP_CTAS), min(c1, gi * GROUP_CTAS + GROUP_CTAS - 1)
                members = [f for f in flushes[s] if f[0] // GROUP_CTAS == gi]
                assert len(members) == cg1 - cg0 + 1, "group arrival count"
                gslot = grp_slot0 + gi + s
                assert grp_slot0 <= gslot < n_slots and gslot not in seen_gslots
                seen_gslots.add(gslot)
                arrivals += 1
            assert arrivals == g_hi - g_lo + 1
            assert (g_hi + s) < (MAX_CTAS // GROUP_CTAS + B), "group counter index in range"
        else:
            assert len(flushes[s]) == slot_hi - slot_lo + 1, "sequence arrival count"
    return total


@pytest.mark.parametrize("wph", [1, 2])
@pytest.mark.parametrize("n_cta", [148, 37, 18, 1])
def test_uniform_split_invariants(wph, n_cta):
    rng = random.Random(n_cta * 10 + wph)
    cases = [[16384] * 16, [1], [0, 0, 5, 0], [131072], [4096] * 3, [17, 16, 15, 1, 0, 33],
             [rng.randint(0, 3000) for _ in range(64)], [rng.randint(4096, 262144) for _ in range(8)],
             [1] * 500, [100000, 1, 100000]]
    for lens in cases:
        for ps in (16, 32, 48):
            if sum(lens) == 0:
                continue
            simulate(lens, ps, n_cta, wph, uniform_bounds)


@pytest.mark.parametrize("wph", [1, 2])
def test_weighted_split_invariants(wph):
    rng = random.Random(7)
    for trial in range(20):
        n_cta = rng.choice([148, 132, 37])
        lens = [rng.randint(2000, 200000) for _ in range(rng.choice([1, 4, 16, 64]))]
        weights = [rng.uniform(0.3, 2.5) for _ in range(n_cta)]
        total = sum(seq_tiles(L, 16) for L in lens)
        assert total >= 8 * n_cta
        bound = weighted_bounds(total, weights)
        assert all(b > a for a, b in zip(bound, bound[1:])), "no empty range in the adaptive split"
        simulate(lens, 16, n_cta, wph, lambda t, n: weighted_bounds(t, weights))


def test_tiles_of_partial_pages():
    assert seq_tiles(0, 16) == 0 and seq_tiles(1, 16) == 1 and seq_tiles(16, 16) == 1 and seq_tiles(17, 16) == 2
    assert seq_tiles(48, 48) == 3 and seq_tiles(49, 48) == 4 and seq_tiles(40, 24) == 2 + 1
    # a page whose size is not a multiple of 16 has a short last tile in every page
    assert seq_tiles(100, 40) == 2 * 3 + 2
