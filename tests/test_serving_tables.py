"""The serving harness deals its pages by the reference block manager's rule: checked against tables produced by the
reference's own BlockManager / Sequence code (tests/golden/serving_block_tables.npz, made by
tests/golden/make_serving_tables_from_reference.py)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pages_are_dealt_like_the_reference_block_manager():
    sys.path.insert(0, ROOT)
    import bench_serving as bs
    g = np.load(os.path.join(ROOT, "tests", "golden", "serving_block_tables.npz"))
    n, plen, gen, blk = int(g["requests"]), int(g["prompt_len"]), int(g["gen_len"]), int(g["block_size"])
    tables, used = bs.deal_pages(n, plen, gen, blk)
    assert np.array_equal(tables, g["final"])
    assert np.array_equal(tables[:, : g["after_prefill"].shape[1]], g["after_prefill"])
    assert used == int(g["final"].max()) + 1
    # the slot of the token fed at decode step s (engine/model_runner.py:359-361)
    for s in (1, 2, 100, gen - 1):
        pos = plen + s - 1
        assert np.array_equal(tables[:, pos // blk] * blk + pos % blk, g["slots"][s - 1])
