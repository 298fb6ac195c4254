"""Generate ``qwen3_tiny_hf.pt``: Hugging Face Qwen3 outputs on seeded weights.

This is the pin the reference's own tests use for this model: a Hugging Face
module with seeded random parameters, run over the full sequence under a causal
mask with no cache object, last position kept
(reference ``tests/models/decode_oracle.py:126-137,213-233``,
``tests/models/dense_decode.py:40-83``).  Run in a container that has
``transformers``; the output file is committed and read by the CPU tests.

    python tests/golden/make_qwen3_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilefoundry_b200.authored import qwen3_1_7b as q          # noqa: E402
from tilefoundry_b200.authored.weights import random_weights   # noqa: E402

CTX = 24          # the reference's layer tests use ctx_len = 24
N_NEW = 8
SEED_W, SEED_X = 0, 1


def checksum(weights) -> int:
    return int(sum(int(t.view(torch.int16).to(torch.int64).sum()) for t in weights.values()) & 0x7FFFFFFF)


def hf_model(cfg, weights):
    from transformers import Qwen3Config, Qwen3ForCausalLM

    hf_cfg = Qwen3Config(
        hidden_size=cfg.hidden_size, num_attention_heads=cfg.num_attention_heads,
        num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
        intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size,
        num_hidden_layers=cfg.num_hidden_layers, rms_norm_eps=cfg.rms_norm_eps,
        max_position_embeddings=cfg.max_position_embeddings, tie_word_embeddings=True,
        rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta},
        attention_bias=False, dtype=torch.bfloat16, attn_implementation="eager",
    )
    model = Qwen3ForCausalLM(hf_cfg).to(torch.bfloat16).eval()
    sd = {"model.embed_tokens.weight": weights["w_embed"], "model.norm.weight": weights["gamma_final"],
          "lm_head.weight": weights["w_embed"]}
    names = {"gamma_in": "input_layernorm.weight", "gamma_post": "post_attention_layernorm.weight",
             "gamma_q": "self_attn.q_norm.weight", "gamma_k": "self_attn.k_norm.weight"}
    proj = {"w_q": "self_attn.q_proj", "w_k": "self_attn.k_proj", "w_v": "self_attn.v_proj",
            "w_o": "self_attn.o_proj", "w_gate": "mlp.gate_proj", "w_up": "mlp.up_proj",
            "w_down": "mlp.down_proj"}
    for i in range(cfg.num_hidden_layers):
        for ours, theirs in names.items():
            sd[f"model.layers.{i}.{theirs}"] = weights[f"layer{i}.{ours}"]
        for ours, theirs in proj.items():
            # ours is (1, in, out); nn.Linear.weight is (out, in)
            sd[f"model.layers.{i}.{theirs}.weight"] = weights[f"layer{i}.{ours}"][0].t().contiguous()
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not unexpected and all("rotary" in m or "lm_head" in m for m in missing), (missing, unexpected)
    return model


@torch.no_grad()
def main():
    cfg = q.QWEN3_TINY
    mod = q.build(cfg)
    # std 0.05 as the reference's randomised modules draw; gains around 1
    weights = q.tie_head(random_weights(mod, seed=SEED_W, std=0.05))
    model = hf_model(cfg, weights)

    gen = torch.Generator().manual_seed(SEED_X)
    ids = torch.randint(0, cfg.vocab_size, (CTX + 1,), generator=gen)

    # full-sequence forward: logits at every position, hidden states after every layer
    out = model(ids[None], output_hidden_states=True, use_cache=False)
    logits = out.logits[0]                                        # [T, V] bf16
    hidden = torch.stack([h[0] for h in out.hidden_states])      # [L+1, T, H]; last one is post-norm

    # greedy continuation by re-running the whole sequence each step (no cache object)
    seq = ids.clone()
    new_tokens = []
    for _ in range(N_NEW):
        nxt = int(torch.argmax(model(seq[None], use_cache=False).logits[0, -1]))
        new_tokens.append(nxt)
        seq = torch.cat([seq, torch.tensor([nxt])])
    final_logits = model(seq[None], use_cache=False).logits[0]

    torch.save({
        "config": cfg.__dict__, "seed_w": SEED_W, "seed_x": SEED_X, "std": 0.05,
        "weights_checksum": checksum(weights), "ids": ids, "logits": logits,
        "hidden_states": hidden, "new_tokens": torch.tensor(new_tokens),
        "final_logits": final_logits,
        "made_with": {"torch": str(torch.__version__), "transformers": __import__("transformers").__version__},
    }, Path(__file__).parent / "qwen3_tiny_hf.pt")
    print("ids", ids.tolist(), "new", new_tokens, "logits absmax", float(logits.float().abs().max()))


if __name__ == "__main__":
    main()
