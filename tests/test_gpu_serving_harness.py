"""The serving harness (bench_serving.py) on a tiny model: tokens produced through the library's attention
(fused or separate pre-attention step, varlen prefill, paged decode over fixed-shape metadata) must be the ones a dense torch forward over the whole
sequence would pick (teacher-forced: at every step the harness's token must be within a whisker of the dense top logit)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("fused", [True, False])
def test_generated_tokens_agree_with_dense_forward(fused):
    import torch
    import torch.nn.functional as F
    sys.path.insert(0, ROOT)
    import bench_serving as bs

    dev = torch.device("cuda", 0)
    cfg = bs.Qwen3Config(layers=2, hidden=256, heads=4, kv_heads=2, head_dim=128, intermediate=512, vocab=512)
    model = bs.Qwen3(cfg, 1, 0, dev, seed=3, fused=fused)
    # larger weights so that logits are well separated
    for layer in model.layers:
        for name in ("w_qkv", "w_o", "w_gate_up", "w_down"):
            setattr(layer, name, (getattr(layer, name).float() * 4).bfloat16())
    model.lm_head = (model.lm_head.float() * 8).bfloat16()
    rng = np.random.Generator(np.random.PCG64(1))
    n, plen, gen = 3, 300, 6          # prompts cross a 256-token page boundary
    prompts = rng.integers(0, cfg.vocab, size=(n, plen))
    eng = bs.Engine(model, prompts, gen, max_batched_tokens=plen * 2)   # two prefill batches
    first = eng.prefill()
    tokens, _ = eng.decode(first, use_graph=False)
    assert tokens.shape == (n, gen)

    def dense(layer, q, k, v):        # one sequence, causal, GQA by repetition
        g = layer.hq // layer.hk
        qq = q.permute(1, 0, 2).float()
        kk = k.permute(1, 0, 2).repeat_interleave(g, dim=0).float()
        vv = v.permute(1, 0, 2).repeat_interleave(g, dim=0).float()
        o = F.scaled_dot_product_attention(qq, kk, vv, is_causal=True, scale=layer.attn.scale)
        return o.permute(1, 0, 2).to(torch.bfloat16)

    for r in range(n):
        seq = np.concatenate([prompts[r], tokens[r]])
        ids = torch.from_numpy(seq.astype(np.int64)).to(dev)
        hidden = model.forward(ids, torch.arange(len(seq), device=dev), None, dense_attention=dense)
        logits = model.logits(hidden).float()
        for t in range(gen):
            row = logits[plen - 1 + t]
            chosen = int(tokens[r, t])
            assert float(row.max() - row[chosen]) <= 0.05 * max(1.0, float(row.max().abs())), (r, t, float(row.max()), float(row[chosen]))
