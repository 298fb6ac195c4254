"""Qwen3-1.7B decode step: declared signatures and host orchestration.

Mirrors reference ``tests/models/qwen3_1_7b/model.py``: a decoder-layer Module
(functions ``input_rms_norm``, ``self_attention``, ``mlp``, ``decoder_layer``;
entry ``decoder_layer``; ``:124-297`` -- the reference's extra ``placed_mlp`` is a
scheduling experiment over the same arithmetic and is declared too so the name
sets agree) and a root Module with ``embed``, ``final_rms_norm``, ``lm_head`` and
the orchestration methods ``forward / decode_hidden / append_cache / init_caches
/ prepare_inputs_for_generation`` (``:300-418``).  Weight projections are
declared ``(1, in, out)`` exactly as there.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import torch

from ..semantic import DimVar, Module, T, W, func


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int = 2048
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 6144
    vocab_size: int = 151936
    num_hidden_layers: int = 28
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 40960
    dtype: str = "bf16"

    @property
    def q_proj(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_proj(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def gqa(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads


QWEN3_1_7B = Qwen3Config()
#: A small instance of the same architecture for CPU tests and fixtures.
QWEN3_TINY = Qwen3Config(hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=64, intermediate_size=512, vocab_size=1024,
                         num_hidden_layers=3, max_position_embeddings=512)
#: A mid-sized instance with the published head geometry (head_dim 128, two query heads per KV head) and widths
#: that are multiples of 1024, the shapes the one-launch step is built for; small enough for the CPU evaluator.
QWEN3_SMALL = Qwen3Config(hidden_size=1024, num_attention_heads=8, num_key_value_heads=4, head_dim=128,
                          intermediate_size=3072, vocab_size=2048, num_hidden_layers=3,
                          max_position_embeddings=512)


@lru_cache(maxsize=None)
def rope_tables(cfg: Qwen3Config, device="cpu"):
    """cos/sin ``[max_pos, head_dim]`` in the model dtype (reference ``model.py:108-121``)."""
    d = cfg.head_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
    ph = torch.outer(torch.arange(cfg.max_position_embeddings, device=device, dtype=torch.float32), inv)
    ph = torch.cat((ph, ph), dim=-1)
    return ph.cos().to(torch.bfloat16), ph.sin().to(torch.bfloat16)


# --- orchestration methods (host Python; state is the caller's) -----------------

def _forward(self, token_ids, cos_cache, sin_cache, pos_ids, scale, caches):
    hidden = self.embed(token_ids)
    normed, entries = self.decode_hidden(hidden, cos_cache, sin_cache, pos_ids, scale, caches)
    return self.lm_head(normed), entries


def _decode_hidden(self, hidden, cos_cache, sin_cache, pos_ids, scale, caches):
    if len(caches) != len(self.modules):
        raise ValueError(
            f"decoder has {len(self.modules)} layers but was given {len(caches)} caches")
    entries = []
    for layer, (k_cache, v_cache) in zip(self.modules, caches):
        hidden, k_new, v_new = layer(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale)
        entries.append((k_new, v_new))
    return self.final_rms_norm(hidden), tuple(entries)


def _append_cache(self, caches, fresh):
    return tuple((torch.cat([k, kn], dim=1), torch.cat([v, vn], dim=1))
                 for (k, v), (kn, vn) in zip(caches, fresh))


def _make_methods(cfg: Qwen3Config):
    def init_caches(self, device=None):
        device = "cpu" if device is None else device
        shape = (1, 0, cfg.num_key_value_heads, cfg.head_dim)
        return tuple((torch.zeros(shape, device=device, dtype=torch.bfloat16),
                      torch.zeros(shape, device=device, dtype=torch.bfloat16))
                     for _ in range(cfg.num_hidden_layers))

    def prepare_inputs_for_generation(self, input_ids, step, caches, device=None):
        device = "cpu" if device is None else device
        token_ids = input_ids[step].reshape(1).to(device=device, dtype=torch.int64)
        cos, sin = rope_tables(cfg, str(device))
        pos_ids = torch.tensor([step], device=device, dtype=torch.int32)
        scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, device=device, dtype=torch.bfloat16)
        return token_ids, cos, sin, pos_ids, scale, caches

    return {"forward": _forward, "decode_hidden": _decode_hidden, "append_cache": _append_cache,
            "init_caches": init_caches, "prepare_inputs_for_generation": prepare_inputs_for_generation}


@lru_cache(maxsize=None)
def build(cfg: Qwen3Config = QWEN3_1_7B) -> Module:
    """The root Module (children ``layer0..layerN-1``) for *cfg*."""
    H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
    HQ, HKV, QP, KVP = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.q_proj, cfg.kv_proj
    C = DimVar("ctx_len", 0, cfg.max_position_embeddings)
    MP = cfg.max_position_embeddings

    attn_params = dict(
        hidden=T((1, 1, H)), gamma_in=W((H,)),
        w_q=W((1, H, QP)), w_k=W((1, H, KVP)), w_v=W((1, H, KVP)),
        gamma_q=W((D,)), gamma_k=W((D,)),
        cos_cache=T((MP, D)), sin_cache=T((MP, D)), pos_ids=T((1,), "i32"),
        k_cache=T((1, C, HKV, D)), v_cache=T((1, C, HKV, D)), scale=T((1, 1, 1, 1)),
        w_o=W((1, QP, H)),
    )
    mlp_params = dict(hidden=T((1, 1, H)), gamma_post=W((H,)),
                      w_gate=W((1, H, I)), w_up=W((1, H, I)), w_down=W((1, I, H)))
    layer_params = dict(attn_params)
    layer_params.update({k: v for k, v in mlp_params.items() if k != "hidden"})
    layer = Module(
        name="Qwen3_1_7B_DecoderLayer", entry="decoder_layer",
        functions=(
            func("input_rms_norm", hidden=T((1, 1, H)), gamma_in=W((H,))),
            func("self_attention", **attn_params),
            func("mlp", **mlp_params),
            func("placed_mlp", **mlp_params),
            func("decoder_layer", **layer_params),
        ),
    )
    return Module(
        name="Qwen3_1_7B",
        functions=(
            func("embed", w_embed=W((V, H)), token_ids=T((1,), "i64")),
            func("final_rms_norm", hidden=T((1, 1, H)), gamma_final=W((H,))),
            func("lm_head", hidden=T((1, 1, H)), w_head=W((H, V))),
        ),
        modules=tuple(layer.renamed(f"layer{i}") for i in range(cfg.num_hidden_layers)),
        methods=_make_methods(cfg),
        metadata={"config": cfg},
    )


def tie_head(weights: dict) -> dict:
    """Tied embeddings: ``w_head`` is ``w_embed`` transposed (HF ``tie_word_embeddings``)."""
    weights = dict(weights)
    weights["w_head"] = weights["w_embed"].t().contiguous()
    return weights
