"""The several-sequence Qwen3 decode step (tensor-core projections, batched split-KV attention) against the CPU
evaluator run once per sequence on the same seeded weights and prompts."""
import ctypes as C

import pytest
import torch

from oracle import evaluator, generation, qwen3_1_7b as oq
from tests.helpers import assert_close_at_scale, assert_close_bf16, assert_ulps
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


def _cuda(weights, dev):
    return {k: v.to(dev) for k, v in weights.items()}


# ---- the SwiGLU form of the tensor-core projection ---------------------------------------------------

@pytest.mark.parametrize("m", [32, 5, 1])
@pytest.mark.parametrize("n,k", [(6144, 2048), (512, 256), (192, 128)])
def test_swiglu_projection_matches_f32_reference(dev, m, n, k):
    from tilefoundry_b200 import lib
    g = torch.Generator().manual_seed(m * 7 + n + k)
    w = (torch.randn(2 * n, k, generator=g) * k ** -0.5).to(BF)
    x = torch.randn(m, k, generator=g).to(BF)
    gate = (x.float() @ w[:n].float().t()).to(BF)
    up = (x.float() @ w[n:].float().t()).to(BF)
    want = (torch.nn.functional.silu(gate.float()).to(BF).float() * up.float()).to(BF)

    native = lib.load()
    splits = native.tfb_gemm_small_m_swiglu_splits(n, k)
    wd, xd = w.to(dev), x.to(dev)
    y = torch.empty(m, n, device=dev, dtype=BF)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    assert splits in (1, 2, 4, 8)
    a = lib.GemmSmallMArgs(w=lib.ptr(wd), x=lib.ptr(xd), residual=None, y=lib.ptr(y), partial=None,
                           tickets=None, status=lib.ptr(status), m=m, n=n, k=k, pdl=0, swiglu=1)
    for _ in range(2):                                  # twice: nothing carries over between launches
        lib.check(native.tfb_gemm_small_m(C.byref(a), lib.stream()), "tfb_gemm_small_m")
    torch.cuda.synchronize()
    assert int(status) == 0
    assert_close_bf16(y.cpu(), want, f"swiglu {m}x{n}x{k}")
    # exact where the two halves land on the same bf16 values: most elements are bit-equal
    assert (y.cpu() == want).float().mean() > 0.9


def test_swiglu_projection_rejects_bad_shapes(dev):
    from tilefoundry_b200 import lib
    z = torch.zeros(64, device=dev, dtype=BF)
    a = lib.GemmSmallMArgs(w=lib.ptr(z), x=lib.ptr(z), residual=None, y=lib.ptr(z), partial=None,
                           tickets=None, status=lib.ptr(z), m=4, n=100, k=64, pdl=0, swiglu=1)
    assert lib.load().tfb_gemm_small_m(C.byref(a), lib.stream()) != 0      # n not a multiple of 64


# ---- batched attention against one launch per sequence ------------------------------------------------------

def test_batched_attention_equals_per_sequence_launches(dev):
    from tilefoundry_b200 import lib
    from tilefoundry_b200.engine import paged_kv
    B, HQ, HKV, D, max_ctx = 6, 16, 8, 128, 1600
    g = torch.Generator().manual_seed(9)
    cfg = q.Qwen3Config(hidden_size=256, num_attention_heads=HQ, num_key_value_heads=HKV, head_dim=D,
                        intermediate_size=512, vocab_size=1024, num_hidden_layers=1, max_position_embeddings=2048)
    cos, sin = q.rope_tables(cfg)
    cos, sin = cos.to(dev), sin.to(dev)
    table = paged_kv.block_table(B, max_ctx, device=dev)
    k_pool = (torch.randn(B * paged_kv.pages_for(max_ctx), 64, HKV, D, generator=g) * 0.5).to(BF).to(dev)
    v_pool = (torch.randn(B * paged_kv.pages_for(max_ctx), 64, HKV, D, generator=g) * 0.5).to(BF).to(dev)
    qkv = torch.randn(B, (HQ + 2 * HKV) * D, generator=g).to(BF).to(dev)
    gq = (1 + 0.1 * torch.randn(D, generator=g)).to(BF).to(dev)
    gk = (1 + 0.1 * torch.randn(D, generator=g)).to(BF).to(dev)
    # ragged contexts: one tile, a page edge, one chunk of 8 tiles exactly, and two that need the merge of chunks
    pos = torch.tensor([0, 63, 64, 511, 512, 1599], dtype=torch.int32, device=dev)
    nsplit = lib.attn_splits(max_ctx)

    def launch(batch, qkv_t, pos_t, table_t, out_t, kp, vp):
        part_o = torch.zeros(batch * HQ * nsplit * D, device=dev, dtype=torch.float32)
        part_ml = torch.zeros(batch * HQ * nsplit * 2, device=dev, dtype=torch.float32)
        counters = torch.zeros(batch * HKV, device=dev, dtype=torch.int32)
        a = lib.AttnGqaArgs(qkv=lib.ptr(qkv_t), gamma_q=lib.ptr(gq), gamma_k=lib.ptr(gk), cos_table=lib.ptr(cos),
                            sin_table=lib.ptr(sin), pos=lib.ptr(pos_t), rope_pos=None, k_pool=lib.ptr(kp),
                            v_pool=lib.ptr(vp), block_table=lib.ptr(table_t), out=lib.ptr(out_t), k_new_out=None,
                            v_new_out=None, part_o=lib.ptr(part_o), part_ml=lib.ptr(part_ml),
                            counters=lib.ptr(counters), hq=HQ, hkv=HKV, d=D, rotary_dim=D, page_size=64,
                            table_len=table.shape[1], max_ctx=max_ctx, max_pos=cos.shape[0], eps=1e-6,
                            scale=D ** -0.5, norm_mode=lib.NORM_CAST_THEN_GAIN, pdl=0, prefetch=None,
                            prefetch_bytes=0, batch=batch)
        lib.check(lib.load().tfb_attn_gqa_decode(C.byref(a), lib.stream()), "tfb_attn_gqa_decode")
        torch.cuda.synchronize()
        assert int(counters.abs().sum()) == 0

    out_b = torch.zeros(B, HQ * D, device=dev, dtype=BF)
    kb, vb = k_pool.clone(), v_pool.clone()
    launch(B, qkv, pos, table, out_b, kb, vb)
    out_s = torch.zeros(B, HQ * D, device=dev, dtype=BF)
    ks, vs = k_pool.clone(), v_pool.clone()
    for b in range(B):
        launch(1, qkv[b], pos[b:b + 1], table[b:b + 1].contiguous(), out_s[b], ks, vs)
    # the batched kernel groups the softmax partials by 512 positions, the single one by 64: same sums, other order
    assert_ulps(out_b.cpu(), out_s.cpu(), 2, "batched vs per-sequence attention")
    assert torch.equal(kb, ks) and torch.equal(vb, vs)       # every sequence appended to its own pages only
    assert not torch.equal(kb, k_pool)


# ---- the whole step ------------------------------------------------------------------------------------

def _batch_vs_oracle(cfg, dev, batch, n_prompt, n_new, seed, std, use_graph):
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=seed, std=std))
    ref = evaluator.load(mod, DictResource(weights), oq.make(cfg))
    g = torch.Generator().manual_seed(seed + 100)
    prompts = torch.randint(0, cfg.vocab_size, (batch, n_prompt), generator=g)
    want = [generation.decode_ids(ref, prompts[b], n_new, keep_logits=True, keep_hidden=True) for b in range(batch)]
    forced = torch.stack([torch.cat([prompts[b], torch.tensor(want[b]["tokens"], dtype=torch.int64)])
                          for b in range(batch)])
    sess = Qwen3BatchSession(cfg, DictResource(_cuda(weights, dev)), batch=batch, max_ctx=n_prompt + n_new + 5,
                             device=dev, trace_hidden=True)
    sess.reset(forced)
    if use_graph:
        sess.capture()
    got = {"logits": [], "hidden": [], "picked": []}
    for _ in range(n_prompt + n_new - 1):
        sess.run(1, use_graph)
        got["logits"].append(sess.logits.clone())
        got["hidden"].append(sess.trace.clone())
        got["picked"].append(sess.picked.clone())
    torch.cuda.synchronize()
    sess.check_status()
    return want, sess, got


@pytest.mark.parametrize("use_graph,batch", [(False, 3), (True, 3), (True, 32)])
def test_batch_session_matches_evaluator_tiny(dev, use_graph, batch):
    cfg = q.QWEN3_TINY
    n_prompt, n_new = 8, (130 if batch <= 4 else 12)     # the small batch crosses the 64-slot page / split boundary
    want, sess, got = _batch_vs_oracle(cfg, dev, batch, n_prompt, n_new, 17, 0.05, use_graph)
    total = n_prompt + n_new - 1
    assert sess.pos.tolist() == [total] * batch
    excused = 0
    for step in range(total):
        for b in range(batch):
            ref_logits = want[b]["logits"][step][0]
            assert_close_at_scale(got["logits"][step][b], ref_logits, f"logits step {step} seq {b}")
            for li in range(cfg.num_hidden_layers + 1):
                assert_close_at_scale(got["hidden"][step][li][b], want[b]["hidden"][step][li],
                                      f"hidden step {step} layer {li} seq {b}")
            pick, ref_pick = int(got["picked"][step][b]), int(torch.argmax(ref_logits))
            assert pick == int(torch.argmax(got["logits"][step][b].cpu())), f"step {step} seq {b}: pick is not argmax"
            if pick != ref_pick:
                top = torch.topk(ref_logits.float(), 2).values
                noise = (got["logits"][step][b].float().cpu() - ref_logits.float()).abs().max()
                assert float(top[0] - top[1]) <= 2 * float(noise), f"step {step} seq {b}: {pick} vs {ref_pick}"
                excused += 1
    assert excused <= max(8, total * batch // 20), f"{excused} near-tie picks out of {total * batch}"
    # every sequence's cache sits in its own pages and equals the evaluator's appended cache
    from tilefoundry_b200.engine import paged_kv
    assert torch.equal(sess.table.cpu(), paged_kv.block_table(batch, sess.max_ctx))
    for b in range(batch):
        for li, (k_ref, v_ref) in enumerate(want[b]["caches"]):
            k_got = paged_kv.logical_view(sess.layers[li]["k_pool"], sess.table[b], total)
            v_got = paged_kv.logical_view(sess.layers[li]["v_pool"], sess.table[b], total)
            assert_close_at_scale(k_got, k_ref[:, :total], f"seq {b} layer {li} K cache")
            assert_close_at_scale(v_got, v_ref[:, :total], f"seq {b} layer {li} V cache")


def test_batch_generate_graph_equals_eager_and_is_idempotent(dev):
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession
    cfg = q.QWEN3_TINY
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=23, std=0.05))
    sess = Qwen3BatchSession(cfg, DictResource(_cuda(weights, dev)), batch=8, max_ctx=200, device=dev)
    prompts = torch.randint(0, cfg.vocab_size, (8, 16), generator=torch.Generator().manual_seed(1))
    a = sess.generate(prompts, 100, use_graph=True)
    b = sess.generate(prompts, 100, use_graph=False)
    c = sess.generate(prompts, 100, use_graph=True)
    assert a.tokens == b.tokens == c.tokens
    assert len(a.tokens) == 8 and all(len(t) == 100 for t in a.tokens)
    assert a.tokens_per_second > 0
    # sequences are independent: permuting the prompts permutes the continuations
    perm = torch.tensor([3, 0, 7, 1, 6, 2, 5, 4])
    d = sess.generate(prompts[perm], 100, use_graph=True)
    assert [d.tokens[i] for i in range(8)] == [a.tokens[int(perm[i])] for i in range(8)]


def test_batch_step_samples_per_sequence(dev):
    """With a temperature the batch step's pick is the Gumbel-max rule of the head kernel, sequence b keyed by
    seed + b: reproducible (graph or eager), different per sequence and per seed, and the last draw of every sequence
    equals the CPU restatement applied to that sequence's logits."""
    import numpy as np
    from oracle import sampling
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession
    cfg = q.QWEN3_TINY
    weights = q.tie_head(random_weights(q.build(cfg), seed=23, std=0.05))
    res = DictResource(_cuda(weights, dev))
    prompts = torch.randint(0, cfg.vocab_size, (1, 16), generator=torch.Generator().manual_seed(1)).repeat(4, 1)
    sess = Qwen3BatchSession(cfg, res, batch=4, max_ctx=200, device=dev, temperature=0.9, seed=77)
    a = sess.generate(prompts, 40, use_graph=True).tokens
    b = sess.generate(prompts, 40, use_graph=False).tokens
    assert a == b
    assert len({tuple(t) for t in a}) == 4                        # the same prompt four times: four different samples
    step = int(sess.pos[0]) - 1
    logits = sess.logits.float().cpu().numpy()
    for i in range(4):
        scores = sampling.gumbel_scores(logits[i], 0.9, 77 + i, step)
        order = np.argsort(-scores, kind="stable")
        assert a[i][-1] == int(order[0]) or (a[i][-1] == int(order[1]) and scores[order[0]] - scores[order[1]] < 1e-4)
    other = Qwen3BatchSession(cfg, res, batch=4, max_ctx=200, device=dev, temperature=0.9, seed=78).generate(prompts, 40).tokens
    greedy = Qwen3BatchSession(cfg, res, batch=4, max_ctx=200, device=dev).generate(prompts, 40).tokens
    assert other != a and greedy != a
    assert other[0] == a[1]                                      # seed 78 sequence 0 draws as seed 77 sequence 1 did


def test_batch_session_rejects_bad_arguments(dev):
    from tilefoundry_b200.engine.qwen3_batch import Qwen3BatchSession
    cfg = q.QWEN3_TINY
    weights = q.tie_head(random_weights(q.build(cfg), seed=1, std=0.05))
    with pytest.raises(ValueError, match="batch must be"):
        Qwen3BatchSession(cfg, DictResource(_cuda(weights, dev)), batch=33, device=dev)
    sess = Qwen3BatchSession(cfg, DictResource(_cuda(weights, dev)), batch=2, max_ctx=64, device=dev)
    with pytest.raises(ValueError, match="prompts must be"):
        sess.reset(torch.zeros(3, 4, dtype=torch.int64))
    with pytest.raises(ValueError, match="exceed capacity"):
        sess.generate(torch.zeros(2, 4, dtype=torch.int64), 100)
