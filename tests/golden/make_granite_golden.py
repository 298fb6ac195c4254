"""Generate ``granite_tiny_hf.pt``: Hugging Face ``GraniteMoeHybridForCausalLM`` outputs on seeded weights.

The same kind of pin the reference keeps for its dense models (a Hugging Face module with seeded random
parameters, ``tests/models/decode_oracle.py:126-137``), applied to granite-4.0-h: the authored weights map to
the Hugging Face names exactly as the reference's ``examples/granite_4_0_h_small-cuda/hf_alias.py:44-95`` states
(renames, the depthwise ``Conv1d`` weight with its singleton axis, each layer's experts as one fused
``input_linear`` = gate rows then up rows).  transformers' Mamba-2 layer runs its plain-torch path here (no
``mamba_ssm`` / ``causal_conv1d`` kernels in this image).  Run where ``transformers`` is installed:

    python tests/golden/make_granite_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilefoundry_b200.authored import granite_4_0_h_small as gr  # noqa: E402
from tilefoundry_b200.authored.weights import random_weights     # noqa: E402

T, SEED_W, SEED_X, STD = 20, 0, 1, 0.05


def hf_model(cfg, weights, dtype):
    from transformers.models.granitemoehybrid import GraniteMoeHybridConfig, GraniteMoeHybridForCausalLM

    hf_cfg = GraniteMoeHybridConfig(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
        num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, rms_norm_eps=cfg.rms_norm_eps, tie_word_embeddings=True,
        embedding_multiplier=cfg.embedding_multiplier, logits_scaling=cfg.logits_scaling,
        residual_multiplier=cfg.residual_multiplier, attention_multiplier=cfg.attention_multiplier,
        num_local_experts=cfg.num_local_experts, num_experts_per_tok=cfg.num_experts_per_tok,
        shared_intermediate_size=cfg.shared_intermediate_size, position_embedding_type="nope",
        layer_types=["mamba" if k == "linear_attention" else "attention" for k in cfg.layer_types], mamba_n_heads=cfg.mamba_n_heads, mamba_n_groups=cfg.mamba_n_groups,
        mamba_d_state=cfg.mamba_d_state, mamba_d_head=cfg.mamba_d_head, mamba_d_conv=cfg.mamba_d_conv,
        mamba_expand=cfg.expand // cfg.hidden_size, mamba_chunk_size=8, mamba_conv_bias=True, mamba_proj_bias=False,
        attention_bias=False, attention_dropout=0.0, router_aux_loss_coef=0.0, dtype=dtype, attn_implementation="eager")
    model = GraniteMoeHybridForCausalLM(hf_cfg).to(dtype).eval()
    sd = {"model.embed_tokens.weight": weights["table"], "model.norm.weight": weights["gamma_final"],
          "lm_head.weight": weights["table"]}
    mamba = {"w_in": "in_proj.weight", "conv_b": "conv1d.bias", "a_log": "A_log", "dt_bias": "dt_bias", "d_skip": "D",
             "gamma_ssm": "norm.weight", "w_out": "out_proj.weight"}
    attn = {"w_q": "q_proj.weight", "w_k": "k_proj.weight", "w_v": "v_proj.weight", "w_o": "o_proj.weight"}
    for i, kind in enumerate(cfg.layer_types):
        L, w = f"model.layers.{i}", lambda n: weights[f"layer{i}.{n}"]
        if kind == "linear_attention":
            for ours, theirs in mamba.items():
                sd[f"{L}.mamba.{theirs}"] = w(f"mixer.{ours}")
            sd[f"{L}.mamba.conv1d.weight"] = w("mixer.conv_w").unsqueeze(1)
        else:
            for ours, theirs in attn.items():
                sd[f"{L}.self_attn.{theirs}"] = w(f"mixer.{ours}")
        sd[f"{L}.input_layernorm.weight"] = w("mixer.gamma_in")
        sd[f"{L}.post_attention_layernorm.weight"] = w("moe.gamma_post")
        sd[f"{L}.block_sparse_moe.input_linear.weight"] = torch.cat([w("moe.w_gate"), w("moe.w_up")], dim=1)
        sd[f"{L}.block_sparse_moe.output_linear.weight"] = w("moe.w_down")
        sd[f"{L}.block_sparse_moe.router.layer.weight"] = w("moe.router.w_router")
        sd[f"{L}.shared_mlp.input_linear.weight"] = w("moe.w_shared_in")
        sd[f"{L}.shared_mlp.output_linear.weight"] = w("moe.w_shared_out")
    sd = {k: v.to(dtype) for k, v in sd.items()}
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and not [m for m in missing if "lm_head" not in m], (missing, unexpected)
    return model


@torch.no_grad()
def main():
    cfg = gr.GRANITE_TINY
    weights = random_weights(gr.build(cfg), seed=SEED_W, std=STD, overrides=gr.weight_overrides)
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(SEED_X))
    out = {}
    for name, dtype in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        model = hf_model(cfg, weights, dtype)
        res = model(ids[None], output_hidden_states=True, use_cache=False)
        out[name] = {"logits": res.logits[0].clone(), "hidden": torch.stack([h[0] for h in res.hidden_states]).clone()}
        print(name, "logits", tuple(res.logits.shape), "hidden", tuple(out[name]["hidden"].shape),
              "top tokens", res.logits[0].argmax(-1)[:8].tolist())
    import transformers
    torch.save({"config": dict(cfg.__dict__), "seed_w": SEED_W, "std": STD, "ids": ids, "bf16": out["bf16"], "f32": out["f32"],
                "transformers": transformers.__version__, "torch": str(torch.__version__)},
               Path(__file__).with_name("granite_tiny_hf.pt"))
    print("wrote", Path(__file__).with_name("granite_tiny_hf.pt"))


if __name__ == "__main__":
    main()
