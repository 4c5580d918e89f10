"""CPU model of the tile bookkeeping of the prefill kernel (csrc/varlen_prefill.cu): which 128-key tiles each 128-row
Q tile of a work item (256 rows of one head, or 128 rows of two heads when the GQA group size is even) visits, and the element mask on its last (diagonal) tile, must cover exactly the causal
region -- key c is used for query position p iff c <= p -- for every sequence length; and the plan kernel's item list
must contain every (sequence, row block) once, longest causal span first."""
import numpy as np
import pytest


def visited(L, q0, x, pair_heads=False):
    """Boolean [rows_of_tile, L_padded]: keys the kernel lets row r of Q tile x (0 = A, 1 = B) of the item at q0 see.
    pair_heads: both tiles are the rows q0 .. q0+127 (of two heads) and visit the same tiles."""
    rows = min(128 if pair_heads else 256, L - q0)
    n_a = q0 // 128 + 1
    n_b = n_a if pair_heads else (q0 // 128 + 2 if rows > 128 else 0)
    n_x = n_a if x == 0 else n_b
    width = (max(n_a, n_b)) * 128
    seen = np.zeros((128, width), dtype=bool)
    for j in range(n_x):
        tile = np.ones((128, 128), dtype=bool)
        if j == n_x - 1:  # diagonal tile: key c visible to row r iff c <= r
            tile = np.arange(128)[None, :] <= np.arange(128)[:, None]
        seen[:, j * 128:(j + 1) * 128] = tile
    return seen, n_x


@pytest.mark.parametrize("L", [1, 5, 127, 128, 129, 255, 256, 257, 300, 511, 512, 513, 1000, 4096])
def test_tiles_and_masks_cover_exactly_the_causal_region(L):
    for q0 in range(0, L, 256):
        for x in (0, 1):
            seen, n_x = visited(L, q0, x)
            for r in range(128):
                p = q0 + 128 * x + r
                if p >= L or n_x == 0:
                    continue  # rows past the sequence are computed on whatever the tile holds and never stored
                want = np.arange(seen.shape[1]) <= p
                assert np.array_equal(seen[r], want), (L, q0, x, r)
        rows = min(256, L - q0)
        assert (rows > 128) == (visited(L, q0, 1)[1] > 0)
    for q0 in range(0, L, 128):  # items of two heads: both tiles hold the same rows
        for x in (0, 1):
            seen, n_x = visited(L, q0, x, pair_heads=True)
            assert n_x == q0 // 128 + 1
            for r in range(min(128, L - q0)):
                assert np.array_equal(seen[r], np.arange(seen.shape[1]) <= q0 + r), (L, q0, x, r)


def test_plan_orders_items_longest_span_first():
    lens = [700, 256, 1, 1300, 0, 257]
    blocks = [(b, l) for b, n in enumerate(lens) for l in range((n + 255) // 256)]
    # the plan kernel: histogram per level, bases assigned from the highest level down, any order inside a level
    max_level = max((n + 255) // 256 for n in lens)
    order = [(b, l) for l in range(max_level - 1, -1, -1) for b, n in enumerate(lens) if (n + 255) // 256 > l]
    assert sorted(order) == sorted(blocks) and len(order) == len(set(order)) == 3 + 1 + 1 + 6 + 0 + 2
    spans = [l for _, l in order]
    assert spans == sorted(spans, reverse=True)
    assert len(order) <= sum(lens) // 256 + len(lens) + 1, "fits the workspace capacity the host computes"
