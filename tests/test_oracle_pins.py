"""The CPU oracle against the committed Hugging Face vectors (CPU only).

The reference pins each authored model against a seeded Hugging Face module at
"3 roundings at the output's scale" per fused function
(``tests/models/decode_oracle.py:69-83``).  The same bound is applied per layer
here; logits after the whole (3-layer) stack get a proportionally wider bound.
"""
import torch

from oracle import evaluator, generation, qwen3_1_7b as oq
from tests.helpers import assert_ulps
from tilefoundry_b200.authored import qwen3_1_7b as q
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import DictResource


def _load(golden_dir):
    fx = torch.load(golden_dir / "qwen3_tiny_hf.pt")
    cfg = q.Qwen3Config(**fx["config"])
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=fx["seed_w"], std=fx["std"]))
    chk = int(sum(int(t.view(torch.int16).to(torch.int64).sum()) for t in weights.values()) & 0x7FFFFFFF)
    assert chk == fx["weights_checksum"], "seeded weights differ from the ones the fixture was made with"
    return fx, cfg, evaluator.load(mod, DictResource(weights), oq.make(cfg))


def test_layers_match_hf_hidden_states(golden_dir):
    fx, cfg, loaded = _load(golden_dir)
    hs = fx["hidden_states"]            # [L+1, T, H]; hs[0] = embeddings, hs[L] = after final norm
    T = hs.shape[1]
    cos, sin = q.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, dtype=torch.bfloat16)
    # embedding is an exact gather
    emb = torch.stack([loaded.embed(fx["ids"][t].reshape(1))[0, 0] for t in range(T)])
    assert torch.equal(emb, hs[0])
    for li, layer in enumerate(loaded.modules[:-1]):
        kc = torch.zeros(1, 0, cfg.num_key_value_heads, cfg.head_dim, dtype=torch.bfloat16)
        vc = kc.clone()
        for t in range(T):
            x = hs[li, t].reshape(1, 1, -1)
            out, kn, vn = layer(x, cos, sin, torch.tensor([t], dtype=torch.int32), kc, vc, scale)
            kc, vc = torch.cat([kc, kn], 1), torch.cat([vc, vn], 1)
            assert_ulps(out[0, 0], hs[li + 1, t], 3, f"layer {li} position {t}")


def test_logits_and_greedy_tokens_match_hf(golden_dir):
    fx, cfg, loaded = _load(golden_dir)
    n_new = fx["new_tokens"].numel()
    run = generation.decode_ids(loaded, fx["ids"], n_new, keep_logits=True)
    got = torch.cat(run["logits"][: fx["ids"].numel()])
    assert_ulps(got, fx["logits"], 3 * (cfg.num_hidden_layers + 1), "prompt logits")
    assert run["tokens"] == fx["new_tokens"].tolist()
    full = torch.cat(run["logits"][: fx["final_logits"].shape[0]])
    assert_ulps(full, fx["final_logits"], 3 * (cfg.num_hidden_layers + 1), "continuation logits")


def test_zero_length_context_is_a_first_step(golden_dir):
    # ctx_len admits 0: the step attends only the position it brings itself.
    fx, cfg, loaded = _load(golden_dir)
    caches = loaded.init_caches()
    assert caches[0][0].shape == (1, 0, cfg.num_key_value_heads, cfg.head_dim)
    args = loaded.prepare_inputs_for_generation(fx["ids"][:1], 0, caches)
    logits, fresh = loaded.forward(*args)
    assert logits.shape == (1, cfg.vocab_size) and logits.dtype == torch.bfloat16
    assert_ulps(logits[0], fx["logits"][0], 3 * (cfg.num_hidden_layers + 1), "first step")
    assert fresh[0][0].shape == (1, 1, cfg.num_key_value_heads, cfg.head_dim)


# ---- MiniCPM3: pinned by the reference's own torch statement of its decode path ------------------------

def test_minicpm3_layer_matches_reference_ops_vectors(golden_dir):
    """`tests/golden/minicpm3_tiny_refops.pt` was produced by importing the reference's
    ``examples/minicpm3_4b-cutedsl/kernels/reference_ops.py``.  It rotates in bf16 and keeps the
    attention in f32 where the evaluator rotates in f32 and rounds attention intermediates to bf16,
    so the two agree to a few roundings at the output's scale, not bit for bit."""
    from oracle import minicpm3_4b as om
    from tilefoundry_b200.authored import minicpm3_4b as m

    fx = torch.load(golden_dir / "minicpm3_tiny_refops.pt")
    cfg = m.MiniCPM3Config(**{**fx["config"], "short_factor": tuple(fx["config"]["short_factor"])})
    mod = m.build(cfg)
    weights = m.tie_head(random_weights(mod, seed=fx["seed_w"], std=fx["std"]))
    loaded = evaluator.load(mod, DictResource(weights), om.make(cfg))
    cos, sin = m.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.qk_head_dim ** -0.5, dtype=torch.bfloat16)
    alpha = torch.full((1, 1, 1), cfg.residual_scale, dtype=torch.bfloat16)
    NH = cfg.num_attention_heads
    for case in fx["cases"]:
        pos = torch.tensor([case["ctx"]], dtype=torch.int32)
        out, k_new, v_new = loaded.layer0(case["hidden"], cos, sin, pos, case["k_cache"], case["v_cache"], scale, alpha)
        assert_ulps(out.reshape(-1), case["out"], 3, f"layer out ctx {case['ctx']}")
        assert_ulps(k_new.reshape(-1), case["k_new"], 1, f"k_new ctx {case['ctx']}")
        assert torch.equal(v_new.reshape(-1), case["v_new"])
    assert torch.equal(loaded.embed(torch.tensor([17])).reshape(-1), fx["embed"])
    normed = loaded.final_rms_norm(fx["cases"][-1]["out"].reshape(1, 1, -1))
    assert torch.equal(normed.reshape(-1), fx["final_norm"])
    assert_ulps(loaded.lm_head(normed).reshape(-1), fx["logits"], 1, "logits")


# ---- Qwen3.5: pinned by the reference's own plain-torch statement of every @func ------------------------

def _close_f32(got, want, msg, tol=2e-5):
    """f32 activations: both sides round a matmul's output to bf16 at the same points, so they differ by
    accumulation order inside f32 reductions only -- except where such a difference flips one bf16
    rounding of a matmul output, which the bound below allows at that tensor's scale."""
    err = (got.float().reshape(-1) - want.float().reshape(-1)).abs().max().item()
    scale = want.float().abs().max().item()
    assert err <= tol * scale + 2.0 ** -8 * scale * 1.01, f"{msg}: max err {err:.4g} at scale {scale:.4g}"


def test_qwen3_5_layers_match_reference_torch_ref_vectors(golden_dir):
    """`tests/golden/qwen3_5_tiny_torchref.pt` was produced by importing the reference's
    ``examples/qwen3_5_35b_a3b-tilelang/kernels/torch_ref.py``."""
    from oracle import qwen3_5_35b_a3b as oq5
    from tilefoundry_b200.authored import qwen3_5_35b_a3b as m

    fx = torch.load(golden_dir / "qwen3_5_tiny_torchref.pt")
    cfg = m.Qwen35Config(**fx["config"])
    mod = m.build(cfg)
    weights = random_weights(mod, seed=fx["seed_w"], std=fx["std"], overrides=m.weight_overrides)
    loaded = evaluator.load(mod, DictResource(weights), oq5.make(cfg))
    cos, sin = m.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5)

    for i, case in enumerate(fx["gdn_cases"]):
        rec = (case["rec_a"][:, :, None] * case["rec_b"][:, None, :])[None]
        mixed, entry, updated = loaded.layer0.mixer.linear_attention(case["hidden"], case["conv_state"], rec)
        assert torch.equal(entry, case["entry"]), f"gdn case {i}: conv entry"
        _close_f32(mixed, case["mixed"], f"gdn case {i}: mixer output")
        if case["updated"] is not None:
            _close_f32(updated, case["updated"], f"gdn case {i}: state", tol=1e-4)
        _close_f32((updated[0] * case["probe_k"][None, :, None]).sum(1), case["updated_over_k"], f"gdn case {i}: state over k", tol=1e-4)
        _close_f32((updated[0] * case["probe_v"][None, None, :]).sum(2), case["updated_over_v"], f"gdn case {i}: state over v", tol=1e-4)
        out, _ = loaded.layer0(case["hidden"], (case["conv_state"], rec))
        tokens = loaded.layer0.moe.post_norm(case["hidden"] + case["mixed"])
        rw, idx = loaded.layer0.moe.router.routing(tokens)
        assert torch.equal(idx, case["route_idx"]), f"gdn case {i}: routed experts"
        _close_f32(rw, case["route_w"], f"gdn case {i}: routing weights")
        _close_f32(out, case["out"], f"gdn case {i}: layer output")

    layer = getattr(loaded, f"layer{fx['attn_layer']}")
    for case in fx["attn_cases"]:
        pos = torch.tensor([case["ctx"]], dtype=torch.int32)
        mixed, k_new, v_new = layer.mixer.full_attention(case["hidden"], cos, sin, pos, case["k_cache"], case["v_cache"], scale)
        assert torch.equal(v_new, case["v_new"]), f"ctx {case['ctx']}: v_new"
        _close_f32(k_new, case["k_new"], f"ctx {case['ctx']}: k_new", tol=1e-5)
        _close_f32(mixed, case["mixed"], f"ctx {case['ctx']}: attention output")
        out, _ = layer(case["hidden"], (cos, sin, pos, case["k_cache"], case["v_cache"], scale))
        _close_f32(out, case["out"], f"ctx {case['ctx']}: layer output")

    assert torch.equal(loaded.embed(torch.tensor([17])), fx["embed"])
    normed = loaded.final_rms_norm(fx["attn_cases"][-1]["out"])
    _close_f32(normed, fx["final_norm"], "final norm", tol=1e-5)
    _close_f32(loaded.lm_head(fx["final_norm"]), fx["logits"], "logits", tol=0)


# ---- granite-4.0-h: pinned by Hugging Face GraniteMoeHybridForCausalLM on seeded weights ---------------------

def test_granite_matches_hf_granitemoehybrid(golden_dir):
    """`tests/golden/granite_tiny_hf.pt` holds Hugging Face ``GraniteMoeHybridForCausalLM`` (plain-torch Mamba-2 path)
    on the seeded weights, mapped as the reference's ``examples/granite_4_0_h_small-cuda/hf_alias.py`` maps a
    checkpoint, run over 20 tokens at f32 and at bf16.  The evaluator walks the same tokens step by step (recurrent
    state and KV cache carried), rounding to bf16 after every op; against the f32 run it must stay inside bf16
    noise at every position: logits within 1 % of their scale, every layer's output within 2.5 %, and the same
    greedy token unless the f32 run's own top-2 margin is inside that noise."""
    from oracle import granite_4_0_h_small as og
    from tests import parity
    from tilefoundry_b200.authored import granite_4_0_h_small as gr

    fx = torch.load(golden_dir / "granite_tiny_hf.pt")
    cfg = gr.GraniteConfig(**{**fx["config"], "attention_layers": tuple(fx["config"]["attention_layers"])})
    mod = gr.build(cfg)
    weights = random_weights(mod, seed=fx["seed_w"], std=fx["std"], overrides=gr.weight_overrides)
    ref = evaluator.load(mod, DictResource(weights), og.make(cfg))
    ids, want = fx["ids"], fx["f32"]
    L = cfg.num_hidden_layers
    for step, _, logits, hiddens, _, _, _ in parity.nested_walk(ref, cfg.layer_types, ids, ids.numel()):
        hl = want["logits"][step].float()
        err = (logits[0].float() - hl).abs().max().item()
        assert err <= 1e-2 * hl.abs().max().item(), f"position {step}: logits differ by {err:.4g}"
        for li in range(L - 1):                          # HF's last entry is after the final norm
            hh = want["hidden"][li + 1, step].float()
            eh = (hiddens[li].float() - hh).abs().max().item()
            assert eh <= 2.5e-2 * hh.abs().max().item(), f"position {step} layer {li}: hidden differs by {eh:.4g}"
        if int(logits.argmax()) != int(hl.argmax()):
            top = torch.topk(hl, 2).values
            assert float(top[0] - top[1]) <= 2 * err, f"position {step}: greedy token differs outside the noise"
    # the two Hugging Face runs bracket the evaluator: it is no farther from f32 than HF's own bf16 run is
    hf_gap = (fx["bf16"]["logits"].float() - want["logits"].float()).abs().max().item()
    ours = max((logits[0].float() - want["logits"][step].float()).abs().max().item()
               for step, _, logits, _, _, _, _ in parity.nested_walk(ref, cfg.layer_types, ids, ids.numel()))
    assert ours <= 1.25 * hf_gap + 1e-3, f"evaluator {ours:.4g} vs HF bf16 {hf_gap:.4g} from the f32 run"


# ---- Qwen3 against the reference's OWN torch statements (tests/golden/make_qwen3_refstmt_golden.py) ----------------

def _refstmt_inputs(cfg, ctx, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(torch.bfloat16)
    kc = torch.randn(1, ctx, cfg.num_key_value_heads, cfg.head_dim, generator=g).to(torch.bfloat16)
    vc = torch.randn(1, ctx, cfg.num_key_value_heads, cfg.head_dim, generator=g).to(torch.bfloat16)
    return hidden, kc, vc


def test_qwen3_attention_body_equals_the_reference_f64_statement(golden_dir):
    """``examples/qwen3_1_7b-tilelang/fast/arbitrate.py:22-56`` states the authored attention in float64.  The
    restated function body evaluated at float64 over the same seeded inputs must agree with it to f32 accuracy
    (two handlers compute in f32 whatever they are given) -- the two can then only differ in where they round --
    and the bf16 evaluation must sit within bf16 noise of it."""
    import dataclasses
    fx = torch.load(golden_dir / "qwen3_refstmt.pt")
    cfg = q.QWEN3_TINY
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=fx["seed_w"], std=0.05))
    exact = evaluator.load_as(mod, DictResource(weights), oq.make(dataclasses.replace(cfg, dtype="f64")), torch.float64)
    rounded = evaluator.load(mod, DictResource(weights), oq.make(cfg))
    cos, sin = q.rope_tables(cfg)
    for ctx in fx["f64_contexts"]:
        hidden, kc, vc = _refstmt_inputs(cfg, ctx, fx["seed_x"] + ctx)
        pos = torch.tensor([ctx], dtype=torch.int32)
        want = fx[f"f64_attention_ctx{ctx}"].reshape(-1)
        f64 = lambda t: t.to(torch.float64)
        scale64 = torch.full((1, 1, 1, 1), float(torch.tensor(cfg.head_dim ** -0.5, dtype=torch.bfloat16)), dtype=torch.float64)
        out64, _, _ = exact.layer0.self_attention(f64(hidden), f64(cos), f64(sin), pos, f64(kc), f64(vc), scale64)
        rel = float((out64.reshape(-1) - want).norm() / want.norm())
        # (1e-6, not 1e-12: the RMSNorm and softmax handlers compute in f32 by definition, whatever the operand type)
        assert rel < 1e-6, f"ctx {ctx}: the function body at f64 is {rel:.3g} from the reference's f64 statement"
        scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, dtype=torch.bfloat16)
        out16, _, _ = rounded.layer0.self_attention(hidden, cos, sin, pos, kc, vc, scale)
        rel16 = float((out16.reshape(-1).double() - want).norm() / want.norm())
        assert rel16 < 3e-2, f"ctx {ctx}: the bf16 evaluation is {rel16:.3g} from the f64 statement"


def test_qwen3_layer_matches_the_reference_kernel_statements_at_published_widths(golden_dir):
    """The reference judges its own Qwen3 kernels by torch statements at the published widths
    (``examples/qwen3_1_7b-tilelang/fast/test_kernels.py:32-172``) under max-error-at-scale < 2e-2 and cosine
    > 1 - 2e-2 (``:18-29``).  The restated ``self_attention`` / ``mlp`` / ``input_rms_norm`` are held to those
    statements under the same bound."""
    import dataclasses
    from tests.helpers import assert_close_at_scale
    fx = torch.load(golden_dir / "qwen3_refstmt.pt")
    cfg = dataclasses.replace(q.QWEN3_1_7B, num_hidden_layers=1, vocab_size=1024)
    mod = q.build(cfg)
    weights = q.tie_head(random_weights(mod, seed=fx["seed_w"], std=0.02))
    loaded = evaluator.load(mod, DictResource(weights), oq.make(cfg))
    ctx = fx["wide_ctx"]
    hidden, kc, vc = _refstmt_inputs(cfg, ctx, fx["seed_x"])
    cos, sin = q.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, dtype=torch.bfloat16)
    out, k_new, v_new = loaded.layer0.self_attention(hidden, cos, sin, torch.tensor([ctx], dtype=torch.int32), kc, vc, scale)
    assert_close_at_scale(out, fx["wide_attention_out"], "self_attention out")
    assert_close_at_scale(k_new, fx["wide_k_new"], "k_new")
    assert torch.equal(v_new, fx["wide_v_new"])                       # a projection output, rounded once on both sides
    assert_close_at_scale(loaded.layer0.mlp(hidden), fx["wide_mlp_out"], "mlp")
    assert_ulps(loaded.layer0.input_rms_norm(hidden).reshape(-1), fx["wide_input_norm"], 1, "input_rms_norm")
