"""Chunked prompt processing against the token-by-token walk and against the CPU evaluator."""
import ctypes as C

import pytest
import torch

from oracle import evaluator, generation, qwen3_1_7b as oq
from tests.helpers import assert_close_at_scale, assert_ulps
from tilefoundry_b200.authored import qwen3_1_7b as q
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import DictResource

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


def test_chunk_attention_equals_token_by_token_launches(dev):
    """Seven consecutive tokens of one sequence, starting at position 60 (the chunk crosses a page): the two chunk
    launches (append, then attend) against seven single launches in order."""
    from tilefoundry_b200 import lib
    from tilefoundry_b200.engine import paged_kv
    M, HQ, HKV, D, max_ctx, first = 7, 16, 8, 128, 320, 60
    g = torch.Generator().manual_seed(3)
    cfg = q.Qwen3Config(hidden_size=256, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D,
                        intermediate_size=512, vocab_size=1024, num_hidden_layers=1, max_position_embeddings=512)
    cos, sin = (t.to(dev) for t in q.rope_tables(cfg))
    table = paged_kv.block_table(1, max_ctx, device=dev)
    pool = lambda: (torch.randn(paged_kv.pages_for(max_ctx), 64, HKV, D, generator=g) * 0.5).to(BF).to(dev)
    k_pool, v_pool = pool(), pool()
    qkv = torch.randn(M, (HQ + 2 * HKV) * D, generator=g).to(BF).to(dev)
    gq = (1 + 0.1 * torch.randn(D, generator=g)).to(BF).to(dev)
    gk = (1 + 0.1 * torch.randn(D, generator=g)).to(BF).to(dev)
    pos = torch.arange(first, first + M, dtype=torch.int32, device=dev)
    nsplit = lib.attn_splits(max_ctx)

    def launch(batch, chunk, qkv_t, pos_t, out_t, kp, vp):
        part_o = torch.zeros(batch * HQ * nsplit * D, device=dev, dtype=torch.float32)
        part_ml = torch.zeros(batch * HQ * nsplit * 2, device=dev, dtype=torch.float32)
        counters = torch.zeros(batch * HKV, device=dev, dtype=torch.int32)
        a = lib.AttnGqaArgs(qkv=lib.ptr(qkv_t), gamma_q=lib.ptr(gq), gamma_k=lib.ptr(gk), cos_table=lib.ptr(cos),
                            sin_table=lib.ptr(sin), pos=lib.ptr(pos_t), rope_pos=None, k_pool=lib.ptr(kp),
                            v_pool=lib.ptr(vp), block_table=lib.ptr(table), out=lib.ptr(out_t), k_new_out=None,
                            v_new_out=None, part_o=lib.ptr(part_o), part_ml=lib.ptr(part_ml),
                            counters=lib.ptr(counters), hq=HQ, hkv=HKV, d=D, rotary_dim=D, page_size=64,
                            table_len=table.shape[1], max_ctx=max_ctx, max_pos=cos.shape[0], eps=1e-6,
                            scale=D ** -0.5, norm_mode=lib.NORM_CAST_THEN_GAIN, pdl=0, prefetch=None,
                            prefetch_bytes=0, batch=batch, chunk=chunk)
        lib.check(lib.load().tfb_attn_gqa_decode(C.byref(a), lib.stream()), "tfb_attn_gqa_decode")
        torch.cuda.synchronize()
        assert int(counters.abs().sum()) == 0

    out_c = torch.zeros(M, HQ * D, device=dev, dtype=BF)
    kc, vc = k_pool.clone(), v_pool.clone()
    launch(M, 1, qkv, pos, out_c, kc, vc)
    assert int(out_c.abs().sum()) == 0                       # the append launch writes cache rows only
    launch(M, 2, qkv, pos, out_c, kc, vc)
    out_s = torch.zeros(M, HQ * D, device=dev, dtype=BF)
    ks, vs = k_pool.clone(), v_pool.clone()
    for i in range(M):
        launch(1, 0, qkv[i], pos[i:i + 1], out_s[i], ks, vs)
    assert torch.equal(kc, ks) and torch.equal(vc, vs)
    assert_ulps(out_c.cpu(), out_s.cpu(), 2, "chunk vs token-by-token attention")


@pytest.mark.parametrize("n_prompt", [100, 34, 3])
def test_prefill_matches_walk_and_evaluator(dev, n_prompt):
    from tilefoundry_b200.engine import paged_kv
    from tilefoundry_b200.engine.qwen3 import Qwen3Session
    cfg = q.QWEN3_TINY
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=31, std=0.05))
    res = DictResource({k: v.to(dev) for k, v in weights.items()})
    prompt = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(n_prompt))
    walk = Qwen3Session(cfg, res, max_ctx=160, device=dev, keep_logits=True)
    tok_walk = walk.generate(prompt, 1).tokens
    logits_walk = walk.logits.clone()
    pre = Qwen3Session(cfg, res, max_ctx=160, device=dev, keep_logits=True)
    tok_pre = pre.generate(prompt, 1, prefill=True).tokens
    assert int(pre.pos) == int(walk.pos) == n_prompt
    assert_close_at_scale(pre.logits, logits_walk, "first new token's logits: prefill vs walk")
    for li in range(cfg.num_hidden_layers):
        for name in ("k_pool", "v_pool"):
            a = paged_kv.logical_view(pre.layers[li][name], pre.table[0], n_prompt)
            b = paged_kv.logical_view(walk.layers[li][name], walk.table[0], n_prompt)
            assert_close_at_scale(a, b, f"layer {li} {name}")
    # and against the evaluator's own walk of the same prompt
    ref = evaluator.load(mod, DictResource(weights), oq.make(cfg))
    want = generation.decode_ids(ref, prompt, 1, keep_logits=True, keep_hidden=True)
    ref_logits = want["logits"][n_prompt - 1][0]
    assert_close_at_scale(pre.logits, ref_logits, "first new token's logits: prefill vs evaluator")
    if tok_pre != tok_walk:
        top = torch.topk(ref_logits.float(), 2).values
        assert float(top[0] - top[1]) < 2e-2
    # generation continues from the prefilled cache exactly as from the walked one (same session, both ways)
    more_a = pre.generate(prompt, 24, prefill=True).tokens
    more_b = pre.generate(prompt, 24, prefill=True, use_graph=False).tokens
    assert more_a == more_b and len(more_a) == 24
