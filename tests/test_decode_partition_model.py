"""CPU model of the integer logic of the paged-decode kernel (csrc/paged_decode.cu): the stream-K cut of the tile
stream into per-CTA ranges, which ranges emit a partial result into which workspace slot, how many tickets a split
sequence expects before it is combined, and which slots the combining CTA reads back.  Property-tested against brute
force: every tile is served exactly once, every output row is written exactly once, the ticket count equals the
number of partials written, and the combine step reads exactly the slots that were written for its sequence."""
import numpy as np
from hypothesis import given, settings, strategies as st

TILE = 64


def tiles_of(ctx):
    return (ctx + TILE - 1) // TILE


def main_kernel_model(ctx, num_groups):
    """Returns (direct, partial): direct = set of sequences written straight to `out`; partial[(group, slot)] = (b, t0, t1)."""
    tiles = [tiles_of(c) for c in ctx]
    total = sum(tiles)
    prefix = np.concatenate([[0], np.cumsum(tiles)])
    direct, partial, served = set(), {}, np.zeros(max(total, 1), dtype=np.int32)
    for g in range(num_groups):
        x0, x1 = g * total // num_groups, (g + 1) * total // num_groups
        if x0 >= x1:
            continue
        # the (b, t) containing global tile x0: the sequence with tiles > 0 and prefix <= x0 < prefix + tiles
        b = next(i for i in range(len(ctx)) if tiles[i] > 0 and prefix[i] <= x0 < prefix[i] + tiles[i])
        t, left = x0 - prefix[b], x1 - x0
        while left > 0:
            if t >= tiles[b]:
                b, t = b + 1, 0
                continue
            n = min(tiles[b] - t, left)
            served[prefix[b] + t: prefix[b] + t + n] += 1
            if t == 0 and t + n == tiles[b]:
                assert b not in direct
                direct.add(b)
            else:
                slot = 1 if t == 0 else 0
                assert (g, slot) not in partial, "a CTA would overwrite one of its two partial slots"
                partial[(g, slot)] = (b, t, t + n)
            left -= n
            t += n
    return direct, partial, served[:total], prefix, total


def expected_tickets(first, tb, total, num_groups):
    """The kernel's `parts`: tickets a split sequence collects before the last arrival combines its partials."""
    if total >= num_groups:
        return ((first + tb) * num_groups - 1) // total - ((first + 1) * num_groups - 1) // total + 1
    return tb


def merge_kernel_model(b, prefix, total, num_groups):
    """Slots merge_sequence reads for sequence b ('zero' if the row is zero-filled, None if nothing is combined)."""
    first, tb = int(prefix[b]), int(prefix[b + 1] - prefix[b])
    if tb == 0:
        return "zero"
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
    direct, partial, served, prefix, total = main_kernel_model(ctx, num_groups)
    assert np.all(served == 1), "each tile of each sequence is streamed by exactly one CTA"
    by_seq = {}
    for (g, slot), (b, t0, t1) in partial.items():
        by_seq.setdefault(b, []).append((g, slot, t0, t1))
    for b, c in enumerate(ctx):
        want = merge_kernel_model(b, prefix, total, num_groups) if total > 0 else "zero"
        if tiles_of(c) == 0:
            assert want == "zero" and b not in direct and b not in by_seq
        elif b in direct:
            assert want is None and b not in by_seq, "a directly written row must not be merged again"
        else:
            pieces = sorted(by_seq[b])
            assert want is not None and want != "zero"
            assert sorted(want) == [(g, s) for g, s, _, _ in pieces], (ctx, num_groups, b, want, pieces)
            assert expected_tickets(int(prefix[b]), tiles_of(c), total, num_groups) == len(pieces)
            # the pieces tile the sequence without gap or overlap
            spans = sorted((t0, t1) for _, _, t0, t1 in pieces)
            assert spans[0][0] == 0 and spans[-1][1] == tiles_of(c)
            assert all(a[1] == n[0] for a, n in zip(spans, spans[1:]))


def test_known_shapes():
    # one tile, 37 groups: only the last group works, nothing to merge
    direct, partial, served, prefix, total = main_kernel_model([1], 37)
    assert direct == {0} and not partial
    # one long sequence over 37 groups: 37 pieces, slot 1 in the first group, slot 0 elsewhere
    direct, partial, _, prefix, total = main_kernel_model([32768], 37)
    assert not direct and len(partial) == 37
    assert merge_kernel_model(0, prefix, total, 37) == [(0, 1)] + [(g, 0) for g in range(1, 37)]
