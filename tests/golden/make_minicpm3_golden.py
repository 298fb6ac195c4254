"""Generate ``minicpm3_tiny_refops.pt``: one MiniCPM3 decoder layer computed by the REFERENCE's own torch
statement of its decode path, ``examples/minicpm3_4b-cutedsl/kernels/reference_ops.py`` (imported from the
reference checkout; that file depends on torch only), composed exactly as the reference's runtime twin
composes it (``examples/minicpm3_4b-cutedsl/runtime_model.py:148-196``).

transformers 5.5.0 has no MiniCPM3 class, so a Hugging Face pin is not available for this model; this
is the reference-produced pin that is.  Run where the reference checkout is mounted:

    python tests/golden/make_minicpm3_golden.py <path to the reference checkout>
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilefoundry_b200.authored import minicpm3_4b as m          # noqa: E402
from tilefoundry_b200.authored.weights import random_weights    # noqa: E402

SEED_W, SEED_X, STD = 0, 1, 0.05
CONTEXTS = (0, 1, 24, 70)


def load_reference_ops(ref_root: Path):
    path = ref_root / "examples" / "minicpm3_4b-cutedsl" / "kernels" / "reference_ops.py"
    spec = importlib.util.spec_from_file_location("reference_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@torch.no_grad()
def layer(K, cfg, w, hidden, cos, sin, pos, k_cache, v_cache, scale, alpha):
    t = lambda name: w[name][0].t().contiguous()                 # authored (1, in, out) -> (out, in)
    QL, KVL, NH = cfg.q_lora_rank, cfg.kv_lora_rank, cfg.num_attention_heads
    x = hidden.reshape(-1)
    lora = K.rmsnorm_gemv(x, w["gamma_in"], torch.cat([t("w_q_a"), t("w_kv_a")], 0), cfg.rms_norm_eps)
    q_up, kv_up = K.rmsnorm_gemv_pair(lora[:QL], w["gamma_q_a"], t("w_q_b"), lora[QL:QL + KVL], w["gamma_kv_a"],
                                      t("w_kv_b"), cfg.lora_eps)
    ctx = torch.tensor([k_cache.shape[1]])
    attn, k_new, v_new = K.rope_attend(q_up, kv_up, lora[QL + KVL:], cos, sin, pos, k_cache[0], v_cache[0], ctx,
                                       scale, NH, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim)
    h1 = K.gemv_residual(attn, t("w_o"), x, alpha)
    act = K.rmsnorm_gemv_swiglu(h1, w["gamma_post"], t("w_gate"), t("w_up"), cfg.rms_norm_eps)
    out = K.gemv_residual(act, t("w_down"), h1, alpha)
    return out, k_new, v_new


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_minicpm3_golden.py <path to the reference checkout>")
    ref_root = Path(sys.argv[1])
    K = load_reference_ops(ref_root)
    cfg = m.MINICPM3_TINY
    weights = random_weights(m.build(cfg), seed=SEED_W, std=STD)
    w = {k.split(".", 1)[1]: v for k, v in weights.items() if k.startswith("layer0.")}
    cos, sin = m.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.qk_head_dim ** -0.5, dtype=torch.bfloat16)
    alpha = torch.full((1, 1, 1), cfg.residual_scale, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(SEED_X)
    cases = []
    for ctx in CONTEXTS:
        hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(torch.bfloat16)
        kc = (torch.randn(1, ctx, cfg.num_attention_heads, cfg.qk_head_dim, generator=g) * 0.5).to(torch.bfloat16)
        vc = (torch.randn(1, ctx, cfg.num_attention_heads, cfg.v_head_dim, generator=g) * 0.5).to(torch.bfloat16)
        pos = torch.tensor([ctx], dtype=torch.int32)
        out, k_new, v_new = layer(K, cfg, w, hidden, cos, sin, pos, kc, vc, scale, alpha)
        cases.append({"ctx": ctx, "hidden": hidden, "k_cache": kc, "v_cache": vc, "out": out.clone(),
                      "k_new": k_new.clone(), "v_new": v_new.clone()})
    # root-level ops
    table = weights["w_embed"]
    tok = torch.tensor([17])
    emb = K.embed_scaled(table, tok, cfg.scale_emb)
    h = cases[-1]["out"]
    normed = K.rmsnorm(h, weights["gamma_final"], cfg.rms_norm_eps)
    logits = K.lm_head_gemv(normed, table, cfg.logits_scaling)
    torch.save({"config": {k: v for k, v in cfg.__dict__.items()}, "seed_w": SEED_W, "std": STD, "cases": cases,
                "embed": emb, "final_norm": normed, "logits": logits,
                "source": "examples/minicpm3_4b-cutedsl/kernels/reference_ops.py"},
               Path(__file__).parent / "minicpm3_tiny_refops.pt")
    print("cases", [c["ctx"] for c in cases], "out absmax", float(cases[-1]["out"].float().abs().max()))


if __name__ == "__main__":
    main()
