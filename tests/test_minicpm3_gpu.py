"""Parity of the CUDA path against the CPU oracle -- MiniCPM3 architecture (multi-head latent attention)."""
import pytest
import torch

from oracle import evaluator, minicpm3_4b as om
from tests import parity
from tests.helpers import ATOL, RTOL, assert_close_at_scale
from tilefoundry_b200.authored import minicpm3_4b as m
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import AllClose, DictResource, Equal, NanInf, check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
CLOSE = [AllClose(atol=ATOL, rtol=RTOL), NanInf()]


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


def _sides(cfg, dev, seed=3, std=0.05):
    from tilefoundry_b200.twins.minicpm3_4b import make_twin
    mod = m.build(cfg)
    weights = m.tie_head(random_weights(mod, seed=seed, std=std))
    ref = evaluator.load(mod, DictResource(weights), om.make(cfg))
    twin = make_twin(cfg)()
    twin.load(DictResource(parity.cuda_weights(weights, dev)))
    return ref, twin, weights


def _layer_inputs(cfg, ctx, dev, seed=1):
    g = torch.Generator().manual_seed(seed)
    cos, sin = m.rope_tables(cfg)
    NH = cfg.num_attention_heads
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF)
    kc = torch.randn(1, ctx, NH, cfg.qk_head_dim, generator=g).to(BF)
    vc = torch.randn(1, ctx, NH, cfg.v_head_dim, generator=g).to(BF)
    pos = torch.tensor([ctx], dtype=torch.int32)
    scale = torch.full((1, 1, 1, 1), cfg.qk_head_dim ** -0.5, dtype=BF)
    rs = torch.full((1, 1, 1), cfg.residual_scale, dtype=BF)
    return tuple(t.to(dev) for t in (hidden, cos, sin, pos, kc, vc, scale, rs))


@pytest.mark.parametrize("ctx", [0, 1, 63, 64, 65, 200])
def test_layer_functions_against_evaluator_tiny(dev, ctx):
    cfg = m.MINICPM3_TINY
    ref, twin, _ = _sides(cfg, dev)
    inputs = _layer_inputs(cfg, ctx, dev)
    expect = {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": [Equal()]}
    rep = check(lambda *a: parity.to_cpu(twin.layer0.mla_attention(*a)), parity.on_cpu(ref.layer0.mla_attention),
                inputs[:-1], expect=expect)
    assert rep.passed, f"mla_attention ctx={ctx}\n{rep.render()}"
    rep = check(lambda *a: parity.to_cpu(twin.layer0.decoder_layer(*a)), parity.on_cpu(ref.layer0.decoder_layer),
                inputs, expect=expect)
    assert rep.passed, f"decoder_layer ctx={ctx}\n{rep.render()}"
    for fn in ("mlp", "input_rms_norm"):
        rep = check(lambda *a: parity.to_cpu(getattr(twin.layer0, fn)(*a)), parity.on_cpu(getattr(ref.layer0, fn)),
                    (inputs[0],), expect={"output": CLOSE})
        assert rep.passed, f"{fn}\n{rep.render()}"


def expand_latents(cfg, rows, w_kv_b):
    """Assembled ``(k [1, C, heads, qk], v [1, C, heads, v])`` of latent rows ``[C, kv_lora + rope]`` in the
    authored arithmetic (``examples/minicpm3_4b-cutedsl/model.py:236-247``): one bf16 matmul, the rotary slice
    repeated over the heads."""
    NH, NOPE, R, VD, KVL = (cfg.num_attention_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim,
                            cfg.kv_lora_rank)
    C = rows.shape[0]
    kv = torch.matmul(rows[:, :KVL].reshape(1, C, KVL), w_kv_b.cpu()).reshape(C, NH, NOPE + VD)
    k = torch.cat([kv[:, :, :NOPE], rows[:, None, KVL:].expand(C, NH, R)], dim=-1)
    return k.unsqueeze(0).contiguous(), kv[:, :, NOPE:].unsqueeze(0).contiguous()


@pytest.mark.parametrize("size,ctx", [("tiny", c) for c in (0, 1, 31, 32, 33, 63, 64, 65, 200)]
                         + [("full", c) for c in (0, 1, 63, 64, 65, 200, 1088)])
def test_latent_attention_against_evaluator(dev, size, ctx):
    """The absorbed form over a cache of latents against ``mla_attention`` over the same history assembled: ``out``
    under the bounds of the other functions, and the row it appends re-expanded against ``k_new`` / ``v_new``."""
    cfg = m.MINICPM3_TINY if size == "tiny" else m.MiniCPM3Config(num_hidden_layers=1, vocab_size=4096)
    ref, twin, weights = _sides(cfg, dev, std=0.05 if size == "tiny" else 0.02)
    g = torch.Generator().manual_seed(100 + ctx)
    LAT = cfg.kv_lora_rank + cfg.qk_rope_head_dim
    rows = torch.randn(ctx, LAT, generator=g).to(BF)
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF)
    cos, sin = m.rope_tables(cfg)
    pos = torch.tensor([ctx], dtype=torch.int32)
    scale = torch.full((1, 1, 1, 1), cfg.qk_head_dim ** -0.5, dtype=BF)
    w_kv_b = weights["layer0.w_kv_b"]
    kc, vc = expand_latents(cfg, rows, w_kv_b)
    want_out, want_k, want_v = ref.layer0.mla_attention(hidden, cos, sin, pos, kc, vc, scale)
    got_out, latent_new = twin.layer0.mla_attention_latent(*(t.to(dev) for t in (hidden, cos, sin, pos)),
                                                           rows.reshape(1, ctx, LAT).to(dev), scale.to(dev))
    torch.cuda.synchronize()
    assert_close_at_scale(got_out, want_out, f"out at context {ctx}")
    got_k, got_v = expand_latents(cfg, latent_new.cpu().reshape(1, LAT), w_kv_b)
    assert_close_at_scale(got_k.reshape(want_k.shape), want_k, f"k_new at context {ctx}")
    assert_close_at_scale(got_v.reshape(want_v.shape), want_v, f"v_new at context {ctx}")


def test_full_size_layer_and_root_functions(dev):
    cfg = m.MiniCPM3Config(num_hidden_layers=1, vocab_size=4096)
    ref, twin, _ = _sides(cfg, dev, std=0.02)
    inputs = _layer_inputs(cfg, 333, dev)
    rep = check(lambda *a: parity.to_cpu(twin.layer0.decoder_layer(*a)), parity.on_cpu(ref.layer0.decoder_layer),
                inputs, expect={"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": [Equal()]})
    assert rep.passed, rep.render()
    ids = torch.tensor([17], dtype=torch.int64)
    rep = check(lambda i: twin.embed(i.to(dev)).cpu(), ref.embed, (ids,), expect={"output": [Equal()]})
    assert rep.passed, rep.render()               # scaled by 12 with one bf16 rounding on both sides
    hidden = inputs[0]
    rep = check(lambda h: twin.lm_head(twin.final_rms_norm(h)).cpu(),
                lambda h: ref.lm_head(ref.final_rms_norm(h.cpu())), (hidden,), expect={"output": CLOSE})
    assert rep.passed, rep.render()


@pytest.mark.parametrize("cache", ["latent", "assembled"])
@pytest.mark.parametrize("use_graph", [False, True])
def test_session_matches_evaluator_tiny(dev, use_graph, cache):
    from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session
    cfg = m.MINICPM3_TINY
    mod = m.build(cfg)
    weights = m.tie_head(random_weights(mod, seed=11, std=0.05))
    ref = evaluator.load(mod, DictResource(weights), om.make(cfg))
    make = lambda cap: MiniCPM3Session(cfg, DictResource(parity.cuda_weights(weights, dev)), max_ctx=cap, device=dev,
                                       keep_logits=True, trace_hidden=True, cache=cache)
    n_prompt, n_new = 24, 120
    want, sess, got = parity.teacher_forced(ref, make, cfg.vocab_size, n_prompt, n_new, 11, use_graph)
    excused = parity.compare_run(cfg.num_hidden_layers, want, sess, got, n_prompt, n_new)
    assert excused <= 8
    parity.compare_caches(want, sess, n_prompt + n_new - 1)


@pytest.mark.parametrize("cache", ["latent", "assembled"])
def test_session_matches_evaluator_published_widths(dev, cache):
    """The session walk at the published widths (hidden 2560, 40 heads, q_lora 768 / kv_lora 256, SwiGLU 6400) on a
    stack of two layers and a 4096-token vocabulary: hidden state after every layer, logits, picks and caches of every
    teacher-forced step against the evaluator, graph replay."""
    from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session
    cfg = m.MiniCPM3Config(num_hidden_layers=2, vocab_size=4096, max_position_embeddings=512)
    mod = m.build(cfg)
    weights = m.tie_head(random_weights(mod, seed=13, std=0.02))
    ref = evaluator.load(mod, DictResource(weights), om.make(cfg))
    make = lambda cap: MiniCPM3Session(cfg, DictResource(parity.cuda_weights(weights, dev)), max_ctx=cap, device=dev,
                                       keep_logits=True, trace_hidden=True, cache=cache)
    n_prompt, n_new = 8, 40
    want, sess, got = parity.teacher_forced(ref, make, cfg.vocab_size, n_prompt, n_new, 13, True)
    excused = parity.compare_run(cfg.num_hidden_layers, want, sess, got, n_prompt, n_new)
    assert excused <= 4
    parity.compare_caches(want, sess, n_prompt + n_new - 1)


@pytest.mark.parametrize("size,n_prompt", [("tiny", 100), ("tiny", 34), ("tiny", 3), ("wide", 40)])
def test_prefill_matches_walk_and_evaluator(dev, size, n_prompt):
    """The prompt in chunks of up to 32 tokens (tensor-core projections, token-by-token latent attention) against the
    token-by-token walk of the same session class and against the evaluator: position, latent cache rows, the first
    new token's logits, and the continuation."""
    from oracle import generation
    from tilefoundry_b200.engine import paged_kv
    from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session
    cfg = m.MINICPM3_TINY if size == "tiny" else m.MiniCPM3Config(num_hidden_layers=2, vocab_size=4096,
                                                                  max_position_embeddings=512)
    mod = m.build(cfg)
    weights = m.tie_head(random_weights(mod, seed=31, std=0.05 if size == "tiny" else 0.02))
    res = DictResource(parity.cuda_weights(weights, dev))
    prompt = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(n_prompt))
    walk = MiniCPM3Session(cfg, res, max_ctx=160, device=dev, keep_logits=True)
    tok_walk = walk.generate(prompt, 1).tokens
    logits_walk = walk.logits.clone()
    pre = MiniCPM3Session(cfg, res, max_ctx=160, device=dev, keep_logits=True)
    tok_pre = pre.generate(prompt, 1, prefill=True).tokens
    assert int(pre.pos) == int(walk.pos) == n_prompt
    assert_close_at_scale(pre.logits, logits_walk, "first new token's logits: prefill vs walk")
    for li in range(cfg.num_hidden_layers):
        a = paged_kv.logical_view(pre.layers[li]["k_pool"], pre.table[0], n_prompt)
        b = paged_kv.logical_view(walk.layers[li]["k_pool"], walk.table[0], n_prompt)
        assert_close_at_scale(a, b, f"layer {li} latent rows")
    ref = evaluator.load(mod, DictResource(weights), om.make(cfg))
    want = generation.decode_ids(ref, prompt, 1, keep_logits=True)
    ref_logits = want["logits"][n_prompt - 1][0]
    assert_close_at_scale(pre.logits, ref_logits, "first new token's logits: prefill vs evaluator")
    if tok_pre != tok_walk:
        top = torch.topk(ref_logits.float(), 2).values
        assert float(top[0] - top[1]) < 2e-2
    more_a = pre.generate(prompt, 24, prefill=True).tokens
    more_b = pre.generate(prompt, 24, prefill=True, use_graph=False).tokens
    assert more_a == more_b and len(more_a) == 24
    with pytest.raises(ValueError, match="latent"):
        MiniCPM3Session(cfg, res, max_ctx=160, device=dev, cache="assembled").prefill(4)
