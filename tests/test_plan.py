"""Host logic of the work partition (csrc/schedule.h), exercised through the C boundary.

The kernel's split-row protocol is replayed on the CPU: every chunk's pieces of split rows
write to numbered slots, the last arriver sums them in owner order.  The properties checked
are the ones the kernel relies on: chunks tile the sequence, slot ids are unique and within
the budget, and every block derives the same owner range for a row."""
import numpy as np
import pytest

SHAPES = [(56, 112), (216, 144), (72, 144), (288, 144), (72, 576), (96, 192), (1, 1), (1, 500), (300, 1), (3, 7), (2, 2)]


def pieces(cb, tiles_k):
    """[(cta, row, first_tile, last_tile_exclusive, whole)] in block order."""
    out = []
    for g in range(len(cb) - 1):
        t = cb[g]
        while t < cb[g + 1]:
            row = t // tiles_k
            end = min(cb[g + 1], (row + 1) * tiles_k)
            out.append((g, row, t, end, t == row * tiles_k and end == (row + 1) * tiles_k))
            t = end
    return out


@pytest.mark.parametrize("tiles", SHAPES)
@pytest.mark.parametrize("max_ctas", [148, 4, 1])
@pytest.mark.parametrize("slots", [10 ** 6, 140, 17, 0])
def test_partition_properties(sp, tiles, max_ctas, slots):
    tiles_m, tiles_k = tiles
    cb, above, used = sp.plan(tiles_m, tiles_k, max_ctas, slots)
    n = len(cb) - 1
    assert 1 <= n <= max_ctas and cb[0] == 0 and cb[-1] == tiles_m * tiles_k
    assert np.all(np.diff(cb) > 0)
    assert used <= slots
    seen = {}
    for g, row, t0, t1, whole in pieces(cb, tiles_k):
        if whole:
            continue
        head_row = cb[g] // tiles_k
        head_partial = (cb[g] % tiles_k != 0) or (cb[g + 1] < (head_row + 1) * tiles_k)
        slot = g + above[g] + (1 if (row != head_row and head_partial) else 0)
        assert 0 <= slot < used
        assert slot not in seen, "two pieces share a slot"
        seen[slot] = (g, row)
    # pieces of one row own consecutive blocks and consecutive slots, as the reader assumes
    by_row = {}
    for slot, (g, row) in seen.items():
        by_row.setdefault(row, []).append((g, slot))
    for row, items in by_row.items():
        items.sort()
        gs = [g for g, _ in items]
        assert gs == list(range(gs[0], gs[0] + len(gs))) and len(gs) >= 2
        assert len({s - g for g, s in items}) == 1


def test_balance_with_ample_workspace(sp):
    for tiles_m, tiles_k in [(56, 112), (216, 144), (72, 144), (288, 144), (72, 576)]:
        cb, above, used = sp.plan(tiles_m, tiles_k, 148, 10 ** 6)
        sizes = np.diff(cb)
        assert len(sizes) == 148 and sizes.max() - sizes.min() <= 1


def test_no_workspace_means_no_split_rows(sp):
    cb, above, used = sp.plan(56, 112, 148, 0)
    assert used == 0 and np.all(cb % 112 == 0)


def test_replayed_reduction_is_exact(sp):
    tiles_m, tiles_k = 7, 13
    cb, above, used = sp.plan(tiles_m, tiles_k, 16, 1000)
    rng = np.random.default_rng(0)
    contrib = rng.integers(-8, 8, size=tiles_m * tiles_k).astype(np.float64)  # one number per tile
    slots = np.full(used, np.nan)
    result = np.zeros(tiles_m)
    arrivals = np.zeros(tiles_m, int)
    ps = pieces(cb, tiles_k)
    order = rng.permutation(len(ps))  # blocks finish in any order
    for i in order:
        g, row, t0, t1, whole = ps[i]
        part = contrib[t0:t1].sum()
        if whole:
            result[row] = part
            continue
        g_first = max(x for x in range(len(cb) - 1) if cb[x] <= row * tiles_k)
        g_last = min(x for x in range(len(cb) - 1) if cb[x + 1] >= (row + 1) * tiles_k)
        head_row = cb[g] // tiles_k
        head_partial = (cb[g] % tiles_k != 0) or (cb[g + 1] < (head_row + 1) * tiles_k)
        ab = above[g] + (1 if (row != head_row and head_partial) else 0)
        slots[g + ab] = part
        arrivals[row] += 1
        if arrivals[row] == g_last - g_first + 1:
            result[row] = sum(slots[x + ab] for x in range(g_first, g_last + 1))
    assert np.array_equal(result, contrib.reshape(tiles_m, tiles_k).sum(axis=1))


def test_built_in_scratch_holds_every_partition_over_148_sms(sp):
    """The slot arithmetic behind spmm_b200_spmm_own_scratch's refusal: a partition over 148 thread blocks parks at
    most 295 partial tiles, 9.7 MB at N = 64, inside the 10 MiB array, so no shape is refused on a B200 for lack of
    scratch; with the 304 blocks the schedule allows at most (a device with more SMs) some shapes would not fit,
    which is what the refusal is for."""
    scratch = 10 << 20
    slot = 128 * 64 * 4
    worst = 0
    for tiles_m, tiles_k in ((72, 144), (216, 144), (288, 144), (72, 576), (56, 112), (1, 4096), (8192, 3), (148, 149), (295, 7)):
        _, _, used = sp.plan(tiles_m, tiles_k, 148, 1 << 40)
        worst = max(worst, used)
        assert used * slot <= scratch, (tiles_m, tiles_k, used)
    assert worst <= 295
    _, _, used = sp.plan(1000, 7, 304, 1 << 40)
    assert used * slot > scratch
