"""Block tables of the serving workload as the REFERENCE's own block manager deals them.

    python tests/golden/make_serving_tables_from_reference.py /path/to/nanovllm_jax

Imports ``engine/sequence.py`` and ``engine/block_manager.py`` of the reference checkout (pure Python; the package's
``__init__`` -- which imports JAX -- is bypassed with stub parent packages), runs the allocation sequence of the serving
benchmark (128 requests x 512 prompt tokens, then 255 appended tokens each, block size 256: ``allocate`` per request in
arrival order, ``may_append`` per request per step, engine/scheduler.py:81-125) and stores the resulting tables in
``serving_block_tables.npz``.  ``bench_serving.py`` deals its pages by the same rule without the reference being
present; ``tests/test_serving_tables.py`` holds it to this fixture.
"""
import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_engine(path):
    for name in ("nanovllm_jax", "nanovllm_jax.engine"):
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(path, *name.split(".")[1:])]
        sys.modules[name] = mod
    out = {}
    for name in ("sampling_params", "engine.sequence", "engine.block_manager"):
        full = "nanovllm_jax." + name
        spec = importlib.util.spec_from_file_location(full, os.path.join(path, *name.split(".")) + ".py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        spec.loader.exec_module(mod)
        out[name] = mod
    return out["engine.sequence"].Sequence, out["engine.block_manager"].BlockManager


def main():
    path = os.path.abspath(sys.argv[1])
    Sequence, BlockManager = load_engine(path)
    requests, prompt_len, gen_len, block = 128, 512, 256, 256
    rng = np.random.Generator(np.random.PCG64(5000))
    prompts = rng.integers(0, 151936, size=(requests, prompt_len))
    Sequence.block_size = block
    bm = BlockManager(requests * 3 + 8, block)
    seqs = [Sequence(p.tolist()) for p in prompts]
    for s in seqs:
        assert bm.can_allocate(s)
        bm.allocate(s)
    after_prefill = np.array([s.block_table for s in seqs], dtype=np.int32)
    slots = []
    for step in range(1, gen_len):
        for s in seqs:
            s.append_token(int(step))
            bm.may_append(s)
        # the slot the model runner derives for the token fed at this step (engine/model_runner.py:359-361)
        slots.append([s.block_table[-1] * block + s.last_block_num_tokens - 1 for s in seqs])
    final = np.array([s.block_table for s in seqs], dtype=np.int32)
    np.savez_compressed(os.path.join(HERE, "serving_block_tables.npz"), after_prefill=after_prefill, final=final,
                        slots=np.array(slots, dtype=np.int32), requests=requests, prompt_len=prompt_len, gen_len=gen_len,
                        block_size=block)
    print("after prefill", after_prefill.shape, "final", final.shape, "first rows", final[:3].tolist())


if __name__ == "__main__":
    main()
