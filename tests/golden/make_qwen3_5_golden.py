"""Generate ``qwen3_5_tiny_torchref.pt``: a Gated-DeltaNet layer, a gated-attention layer, the router/MoE and
the root functions of Qwen3.5 computed by the REFERENCE's own plain-torch statement of its ``@func`` bodies,
``examples/qwen3_5_35b_a3b-tilelang/kernels/torch_ref.py`` (imported from the reference checkout; it depends
on torch and its sibling ``config.py`` only), composed as the authored layer forward composes them
(``examples/qwen3_5_35b_a3b-tilelang/model.py`` ``_layer_forward`` / ``Qwen3_5MoE.forward``).

Run where the reference checkout is mounted:

    python tests/golden/make_qwen3_5_golden.py <path to the reference checkout>
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilefoundry_b200.authored import qwen3_5_35b_a3b as m      # noqa: E402
from tilefoundry_b200.authored.weights import random_weights    # noqa: E402

SEED_W, SEED_X, STD = 0, 1, 0.05
CONTEXTS = (0, 1, 37)
MOE_W = ("w_gate", "w_up", "w_down", "w_shared_gate", "w_shared_up", "w_shared_down", "w_shared_scale")
GDN_W = ("gamma_in", "w_in_qkv", "w_in_z", "w_in_b", "w_in_a", "conv_w", "a_log", "dt_bias")


def load_torch_ref(ref_root: Path):
    base = ref_root / "examples" / "qwen3_5_35b_a3b-tilelang"
    sys.path.insert(0, str(base))
    spec = importlib.util.spec_from_file_location("torch_ref", base / "kernels" / "torch_ref.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def layer_weights(weights, i):
    pre = f"layer{i}."
    return {k[len(pre):].split(".")[-1]: v for k, v in weights.items() if k.startswith(pre)}


@torch.no_grad()
def moe(R, w, hidden):
    tokens = R.post_norm(hidden, w["gamma_post"])
    rw, idx = R.routing(tokens, w["w_router"])
    return R.experts(tokens, rw, idx, *(w[n] for n in MOE_W)), rw, idx


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_qwen3_5_golden.py <path to the reference checkout>")
    ref_root = Path(sys.argv[1])
    R = load_torch_ref(ref_root)
    cfg = m.QWEN3_5_TINY
    R.TOP_K = cfg.top_k
    weights = random_weights(m.build(cfg), seed=SEED_W, std=STD, overrides=m.weight_overrides)
    cos, sin = m.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5)
    g = torch.Generator().manual_seed(SEED_X)
    H = cfg.hidden

    wl = layer_weights(weights, 0)
    gdn_cases = []
    probe_k = torch.randn(cfg.gdn_head_k_dim, generator=g)       # the updated state is kept whole once, then as two projections
    probe_v = torch.randn(cfg.gdn_head_v_dim, generator=g)
    for step in range(3):
        hidden = torch.randn(1, 1, H, generator=g)
        conv_state = torch.randn(1, cfg.conv_dim, cfg.gdn_conv_kernel - 1, generator=g) * (0.0 if step == 0 else 0.5)
        # the state is an outer product of two stored vectors per head, so the fixture stays small
        rec_a = torch.randn(cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, generator=g) * (0.0 if step == 0 else 0.3)
        rec_b = torch.randn(cfg.gdn_n_v_heads, cfg.gdn_head_v_dim, generator=g) * 0.3
        rec = (rec_a[:, :, None] * rec_b[:, None, :])[None]
        mixed, entry, updated = R.linear_attention(hidden, *(wl[n] for n in GDN_W), conv_state, rec, wl["gamma_gdn"], wl["w_out"])
        attended = R.residual_add(hidden, mixed)
        moe_out, rw, idx = moe(R, wl, attended)
        out = R.residual_add(attended, moe_out)
        gdn_cases.append({"hidden": hidden, "conv_state": conv_state, "rec_a": rec_a, "rec_b": rec_b, "mixed": mixed, "entry": entry,
                          "updated": updated if step == 0 else None, "updated_over_k": (updated[0] * probe_k[None, :, None]).sum(1),
                          "updated_over_v": (updated[0] * probe_v[None, None, :]).sum(2), "probe_k": probe_k, "probe_v": probe_v, "route_w": rw, "route_idx": idx, "out": out})

    ai = cfg.full_attention_every - 1
    wa = layer_weights(weights, ai)
    attn_cases = []
    for ctx in CONTEXTS:
        hidden = torch.randn(1, 1, H, generator=g)
        kc = torch.randn(1, ctx, cfg.n_kv_heads, cfg.head_dim, generator=g) * 0.5
        vc = torch.randn(1, ctx, cfg.n_kv_heads, cfg.head_dim, generator=g) * 0.5
        pos = torch.tensor([ctx], dtype=torch.int32)
        mixed, k_new, v_new = R.full_attention(hidden, wa["gamma_in"], wa["w_qg"], wa["w_k"], wa["w_v"], wa["gamma_q"],
                                               wa["gamma_k"], cos, sin, pos, kc, vc, scale, wa["w_o"])
        attended = R.residual_add(hidden, mixed)
        moe_out, _, _ = moe(R, wa, attended)
        attn_cases.append({"ctx": ctx, "hidden": hidden, "k_cache": kc, "v_cache": vc, "mixed": mixed, "k_new": k_new,
                           "v_new": v_new, "out": R.residual_add(attended, moe_out)})

    tok = torch.tensor([17])
    emb = R.embed(weights["table"], tok)
    normed = R.final_rms_norm(attn_cases[-1]["out"], weights["gamma_final"])
    logits = R.lm_head(normed, weights["w_head"])
    torch.save({"config": dict(cfg.__dict__), "seed_w": SEED_W, "std": STD, "attn_layer": ai, "gdn_cases": gdn_cases,
                "attn_cases": attn_cases, "embed": emb, "final_norm": normed, "logits": logits,
                "torch": str(torch.__version__)}, Path(__file__).with_name("qwen3_5_tiny_torchref.pt"))
    print("wrote", Path(__file__).with_name("qwen3_5_tiny_torchref.pt"))


if __name__ == "__main__":
    main()
