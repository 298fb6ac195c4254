"""MiniCPM3-4B (multi-head latent attention) decode step: declared signatures and orchestration.

Mirrors reference ``examples/minicpm3_4b-cutedsl/model.py`` (== ``tests/models/minicpm3_4b/model.py``):
layer functions ``input_rms_norm``, ``mla_attention``, ``mlp``, ``decoder_layer`` (``:188-345``, entry
``decoder_layer``, extra activation ``residual_scale``), root functions ``embed`` (x ``scale_emb``),
``final_rms_norm``, ``lm_head`` (hidden / ``logits_scaling`` before the head) and the orchestration
methods (``:396-498``).  The cache holds assembled keys ``[1, C, heads, nope+rope]`` and values
``[1, C, heads, v]`` as the authored functions state it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from functools import lru_cache

import torch

from ..semantic import DimVar, Module, T, W, func

_SHORT = (1.0591234137867171, 1.1241891283591912, 1.2596935748670968, 1.5380380402321725,
          2.093982484148734, 3.1446935121267696, 4.937952647693647, 7.524541999994549,
          10.475458000005451, 13.062047352306353, 14.85530648787323, 15.906017515851266,
          16.461961959767827, 16.740306425132907, 16.87581087164081, 16.940876586213285)


@dataclass(frozen=True)
class MiniCPM3Config:
    hidden_size: int = 2560
    num_attention_heads: int = 40
    q_lora_rank: int = 768
    kv_lora_rank: int = 256
    qk_nope_head_dim: int = 64
    qk_rope_head_dim: int = 32
    v_head_dim: int = 64
    intermediate_size: int = 6400
    vocab_size: int = 73448
    num_hidden_layers: int = 62
    rms_norm_eps: float = 1e-5
    lora_eps: float = 1e-6          # the two low-rank norms run at the norm class's own default
    rope_theta: float = 10000.0
    short_factor: tuple = _SHORT    # longrope short factors, one per rotary pair
    max_position_embeddings: int = 32768
    scale_emb: float = 12.0
    scale_depth: float = 1.4
    dim_model_base: int = 256
    dtype: str = "bf16"

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    @property
    def logits_scaling(self) -> float:
        return self.hidden_size / self.dim_model_base

    @property
    def residual_scale(self) -> float:
        return self.scale_depth / math.sqrt(self.num_hidden_layers)


MINICPM3_4B = MiniCPM3Config()
MINICPM3_TINY = MiniCPM3Config(hidden_size=256, num_attention_heads=4, q_lora_rank=256, kv_lora_rank=256,
                               intermediate_size=512, vocab_size=1000, num_hidden_layers=3,
                               max_position_embeddings=512, dim_model_base=64)


@lru_cache(maxsize=None)
def rope_tables(cfg: MiniCPM3Config, device="cpu"):
    """cos/sin ``[max_pos, qk_rope_head_dim]`` with the longrope short factors (reference ``model.py:169-185``)."""
    d = cfg.qk_rope_head_dim
    factors = torch.tensor(cfg.short_factor[: d // 2], device=device, dtype=torch.float32)
    inv = 1.0 / (factors * cfg.rope_theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
    ph = torch.outer(torch.arange(cfg.max_position_embeddings, device=device, dtype=torch.float32), inv)
    ph = torch.cat((ph, ph), dim=-1)
    return ph.cos().to(torch.bfloat16), ph.sin().to(torch.bfloat16)


def _forward(self, token_ids, cos_cache, sin_cache, pos_ids, scale, residual_scale, caches):
    hidden = self.embed(token_ids)
    normed, entries = self.decode_hidden(hidden, cos_cache, sin_cache, pos_ids, scale, residual_scale, caches)
    return self.lm_head(normed), entries


def _decode_hidden(self, hidden, cos_cache, sin_cache, pos_ids, scale, residual_scale, caches):
    if len(caches) != len(self.modules):
        raise ValueError(f"decoder has {len(self.modules)} layers but was given {len(caches)} caches")
    entries = []
    for layer, (k_cache, v_cache) in zip(self.modules, caches):
        hidden, k_new, v_new = layer(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale, residual_scale)
        entries.append((k_new, v_new))
    return self.final_rms_norm(hidden), tuple(entries)


def _append_cache(self, caches, fresh):
    return tuple((torch.cat([k, kn], dim=1), torch.cat([v, vn], dim=1))
                 for (k, v), (kn, vn) in zip(caches, fresh))


def _make_methods(cfg: MiniCPM3Config):
    H = cfg.num_attention_heads

    def init_caches(self, device=None):
        device = "cpu" if device is None else device
        return tuple((torch.zeros((1, 0, H, cfg.qk_head_dim), device=device, dtype=torch.bfloat16),
                      torch.zeros((1, 0, H, cfg.v_head_dim), device=device, dtype=torch.bfloat16))
                     for _ in range(cfg.num_hidden_layers))

    def prepare_inputs_for_generation(self, input_ids, step, caches, device=None):
        device = "cpu" if device is None else device
        token_ids = input_ids[step].reshape(1).to(device=device, dtype=torch.int64)
        cos, sin = rope_tables(cfg, str(device))
        pos_ids = torch.tensor([step], device=device, dtype=torch.int32)
        # the assembled 96-wide head sets the scale, not the 32-wide rotary slice
        scale = torch.full((1, 1, 1, 1), cfg.qk_head_dim ** -0.5, device=device, dtype=torch.bfloat16)
        residual_scale = torch.full((1, 1, 1), cfg.residual_scale, device=device, dtype=torch.bfloat16)
        return token_ids, cos, sin, pos_ids, scale, residual_scale, caches

    return {"forward": _forward, "decode_hidden": _decode_hidden, "append_cache": _append_cache,
            "init_caches": init_caches, "prepare_inputs_for_generation": prepare_inputs_for_generation}


@lru_cache(maxsize=None)
def build(cfg: MiniCPM3Config = MINICPM3_4B) -> Module:
    Hd, NH, I, V = cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, cfg.vocab_size
    QK, NOPE, R, VD = cfg.qk_head_dim, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    C = DimVar("ctx_len", 0, cfg.max_position_embeddings)
    MP = cfg.max_position_embeddings
    attn = dict(
        hidden=T((1, 1, Hd)), gamma_in=W((Hd,)),
        w_q_a=W((1, Hd, cfg.q_lora_rank)), gamma_q_a=W((cfg.q_lora_rank,)), w_q_b=W((1, cfg.q_lora_rank, NH * QK)),
        w_kv_a=W((1, Hd, cfg.kv_lora_rank + R)), gamma_kv_a=W((cfg.kv_lora_rank,)),
        w_kv_b=W((1, cfg.kv_lora_rank, NH * (NOPE + VD))),
        cos_cache=T((MP, R)), sin_cache=T((MP, R)), pos_ids=T((1,), "i32"),
        k_cache=T((1, C, NH, QK)), v_cache=T((1, C, NH, VD)), scale=T((1, 1, 1, 1)),
        w_o=W((1, NH * VD, Hd)),
    )
    mlp = dict(hidden=T((1, 1, Hd)), gamma_post=W((Hd,)), w_gate=W((1, Hd, I)), w_up=W((1, Hd, I)),
               w_down=W((1, I, Hd)))
    layer_params = dict(attn)
    layer_params.update({k: v for k, v in mlp.items() if k != "hidden"})
    layer_params["residual_scale"] = T((1, 1, 1))
    layer = Module(
        name="MiniCPM3_4B_DecoderLayer", entry="decoder_layer",
        functions=(func("input_rms_norm", hidden=T((1, 1, Hd)), gamma_in=W((Hd,))),
                   func("mla_attention", **attn), func("mlp", **mlp), func("decoder_layer", **layer_params)))
    return Module(
        name="MiniCPM3_4B",
        functions=(func("embed", w_embed=W((V, Hd)), token_ids=T((1,), "i64")),
                   func("final_rms_norm", hidden=T((1, 1, Hd)), gamma_final=W((Hd,))),
                   func("lm_head", hidden=T((1, 1, Hd)), w_head=W((Hd, V)))),
        modules=tuple(layer.renamed(f"layer{i}") for i in range(cfg.num_hidden_layers)),
        methods=_make_methods(cfg), metadata={"config": cfg})


def tie_head(weights: dict) -> dict:
    weights = dict(weights)
    weights["w_head"] = weights["w_embed"].t().contiguous()
    return weights
