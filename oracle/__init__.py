"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory.  It is imported by the
tests, by ``__graft_entry__.smoke()`` and by the CPU-baseline / reference legs
of ``bench.py`` -- always as the checker or as the timed CPU baseline, never
as the thing shipped.

PARITY UNPINNED: the reference repository holds no golden vectors or
known-answer tests for this path, and JAX (the library whose gather / matmul /
exp / scatter the reference calls) cannot be imported in this image, so the
restatement below is pinned only by (i) following the reference's jnp code line
by line and (ii) cross-checks against independent formulations (torch CPU
``scaled_dot_product_attention`` and a float64 direct evaluation) in the CPU
test-suite.
"""
