"""CPU model of the integer logic of the paged-decode kernel (csrc/paged_decode.cu): the stream-K cut of the tile
stream into per-CTA ranges, which ranges emit a partial result into which workspace slot, how many tickets a split
sequence expects before it is combined, and which slots the combining CTA reads back.  Property-tested against brute
force: every tile is served exactly once, every output row is written exactly once, the ticket count equals the
number of partials written, and the combine step reads exactly the slots that were written for its sequence."""
import numpy as np
from hypothesis import given, settings, strategies as st

TILE = 64
ITEM_COST = 4  # kItemCostDefault: units a sequence boundary costs in front of the sequence's tiles


def tiles_of(ctx):
    return (ctx + TILE - 1) // TILE


def units_of(tb):
    return tb + ITEM_COST if tb > 0 else 0


def main_kernel_model(ctx, num_groups):
    """Returns (direct, partial, served, first_unit, total): direct = set of sequences written straight to `out`;
    partial[(group, slot)] = (b, t0, t1); first_unit[b] = unit of b's tile 0 on the cost line."""
    tiles = [tiles_of(c) for c in ctx]
    units = [units_of(t) for t in tiles]
    total = sum(units)
    start = np.concatenate([[0], np.cumsum(units)])
    first_unit = [int(start[b]) + ITEM_COST for b in range(len(ctx))]
    direct, partial = set(), {}
    served = [np.zeros(t, dtype=np.int32) for t in tiles]
    for g in range(num_groups):
        x0, x1 = g * total // num_groups, (g + 1) * total // num_groups
        if x0 >= x1:
            continue
        # the walk of the kernel: start at the sequence whose units contain x0, go on while sequences start before x1
        b = next(i for i in range(len(ctx)) if units[i] > 0 and start[i] <= x0 < start[i] + units[i])
        while b < len(ctx) and start[b] < x1:
            tb = tiles[b]
            if tb > 0:
                t0 = min(max(x0 - first_unit[b], 0), tb)
                t1 = min(max(x1 - first_unit[b], 0), tb)
                if t0 < t1:
                    served[b][t0:t1] += 1
                    if t0 == 0 and t1 == tb:
                        assert b not in direct
                        direct.add(b)
                    else:
                        slot = 1 if t0 == 0 else 0
                        assert (g, slot) not in partial, "a CTA would overwrite one of its two partial slots"
                        partial[(g, slot)] = (b, t0, t1)
            b += 1
    return direct, partial, served, first_unit, total


def expected_tickets(first, tb, total, num_groups):
    """The kernel's `parts`: tickets a split sequence collects before the last arrival combines its partials."""
    if total >= num_groups:
        return ((first + tb) * num_groups - 1) // total - ((first + 1) * num_groups - 1) // total + 1
    return tb


def merge_model(first, tb, total, num_groups):
    """Slots merge_sequence reads for a sequence whose tiles occupy units [first, first + tb) (None: nothing to combine)."""
    gf = min(((first + 1) * num_groups - 1) // total, num_groups - 1)
    gl = min(((first + tb) * num_groups - 1) // total, num_groups - 1)
    if gf == gl:
        return None
    slots = []
    for g in range(gf, gl + 1):
        if g * total // num_groups >= (g + 1) * total // num_groups:
            continue
        slots.append((g, 1 if g == gf else 0))
    return slots


@settings(max_examples=300, deadline=None)
@given(st.lists(st.integers(min_value=0, max_value=3000), min_size=1, max_size=40),
       st.sampled_from([1, 2, 3, 5, 18, 37, 74, 148, 296]))
def test_every_tile_once_and_merge_reads_what_was_written(ctx, num_groups):
    direct, partial, served, first_unit, total = main_kernel_model(ctx, num_groups)
    for b, sv in enumerate(served):
        assert np.all(sv == 1), "each tile of each sequence is streamed by exactly one CTA"
    by_seq = {}
    for (g, slot), (b, t0, t1) in partial.items():
        by_seq.setdefault(b, []).append((g, slot, t0, t1))
    for b, c in enumerate(ctx):
        tb = tiles_of(c)
        if tb == 0:
            assert b not in direct and b not in by_seq  # zero-filled in the prologue
            continue
        want = merge_model(first_unit[b], tb, total, num_groups)
        if b in direct:
            assert want is None and b not in by_seq, "a directly written row must not be merged again"
        else:
            pieces = sorted(by_seq[b])
            assert want is not None
            assert sorted(want) == [(g, s) for g, s, _, _ in pieces], (ctx, num_groups, b, want, pieces)
            assert expected_tickets(first_unit[b], tb, total, num_groups) == len(pieces)
            # the pieces tile the sequence without gap or overlap
            spans = sorted((t0, t1) for _, _, t0, t1 in pieces)
            assert spans[0][0] == 0 and spans[-1][1] == tb
            assert all(a[1] == n[0] for a, n in zip(spans, spans[1:]))


def test_cost_weights_even_out_ranges_with_many_short_sequences():
    """64 one-tile sequences followed by one of 640 tiles, two groups: by tiles alone the first group would take all the
    short sequences plus 288 tiles; with the boundary cost it takes them plus 158 tiles only."""
    direct, partial, served, first_unit, total = main_kernel_model([10] * 64 + [640 * 64], 2)
    assert total == 64 * 5 + 644
    assert partial[(0, 1)] == (64, 0, 158) and partial[(1, 0)] == (64, 158, 640)


def test_known_shapes():
    # one tile, 37 groups: one group works, nothing to merge
    direct, partial, served, first_unit, total = main_kernel_model([1], 37)
    assert direct == {0} and not partial
    # one long sequence over 37 groups: every group but those holding only boundary units serves a piece
    direct, partial, _, first_unit, total = main_kernel_model([32768], 37)
    assert not direct and len(partial) == 37
    assert merge_model(first_unit[0], 512, total, 37) == [(0, 1)] + [(g, 0) for g in range(1, 37)]
