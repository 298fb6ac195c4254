"""Qwen3.5-35B-A3B decode step (Gated DeltaNet / gated attention hybrid + 256-expert MoE): declared
signatures and orchestration.

Mirrors reference ``examples/qwen3_5_35b_a3b-tilelang/model.py`` (the variant with f32 activations and
state and bf16 contracted weights): ``Qwen3_5LinearAttention`` (``conv_step l2_normalise delta_step
linear_attention``, ``:117-228``), ``Qwen3_5FullAttention`` (``partial_rope partial_rope_kv full_attention``,
``:293-417``), ``Qwen3_5Router`` (``routing``, ``:488-499``), ``Qwen3_5MoE`` (``post_norm routed_experts
shared_expert experts`` + ``forward``, ``:502-612``), the two layer Modules (``residual_add`` + ``forward``)
and ``Qwen3_5Decoder`` (``embed final_rms_norm lm_head`` + orchestration, ``:760-892``).  The per-layer
non-state arguments come from ``prepare_inputs_for_generation`` here; the reference's example builds the
same tuples in its runtime (``runtime_model.py:372-385``).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from functools import lru_cache

import torch

from ..semantic import DimVar, Module, T, W, func
from .granite_4_0_h_small import _with_cache

F, BW = "f32", "bf16"


@dataclass(frozen=True)
class Qwen35Config:
    hidden: int = 2048
    vocab: int = 248320
    rms_eps: float = 1e-6
    n_layers: int = 40
    full_attention_every: int = 4          # layers 3, 7, 11, ... are full attention (3 GDN : 1 attention)
    max_ctx: int = 4096
    rope_theta: float = 1.0e7
    n_q_heads: int = 16
    n_kv_heads: int = 2
    head_dim: int = 256
    rotary_dim: int = 64
    gdn_n_k_heads: int = 16
    gdn_n_v_heads: int = 32
    gdn_head_k_dim: int = 128
    gdn_head_v_dim: int = 128
    gdn_conv_kernel: int = 4
    n_experts: int = 256
    top_k: int = 8
    moe_intermediate: int = 512
    shared_intermediate: int = 512

    @property
    def layer_types(self):
        return tuple("full_attention" if (i + 1) % self.full_attention_every == 0 else "linear_attention"
                     for i in range(self.n_layers))
    @property
    def key_dim(self): return self.gdn_n_k_heads * self.gdn_head_k_dim
    @property
    def val_dim(self): return self.gdn_n_v_heads * self.gdn_head_v_dim
    @property
    def conv_dim(self): return 2 * self.key_dim + self.val_dim
    @property
    def num_hidden_layers(self): return self.n_layers
    @property
    def vocab_size(self): return self.vocab


QWEN3_5_35B_A3B = Qwen35Config()
QWEN3_5_TINY = Qwen35Config(hidden=256, vocab=1024, n_layers=4, max_ctx=256, n_q_heads=4, n_kv_heads=2, head_dim=128,
                            rotary_dim=64, gdn_n_k_heads=2, gdn_n_v_heads=4, n_experts=16, top_k=4,
                            moe_intermediate=256, shared_intermediate=256)


def truncated(cfg: Qwen35Config, **changes) -> Qwen35Config:
    """The same widths on a shorter stack / smaller vocabulary (reference ``examples/qwen3_5_35b_a3b-tilelang/
    config.py`` ``truncated``): what the CPU evaluator can hold.  Kernel shapes depend on the widths only."""
    return replace(cfg, **changes)


@lru_cache(maxsize=None)
def rope_tables(cfg: Qwen35Config, device="cpu"):
    """f32 cos/sin ``[max_ctx, rotary_dim]`` (reference ``weights.py`` ``rope_caches``)."""
    half = cfg.rotary_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (2.0 * torch.arange(0, half, dtype=torch.float32, device=device) / cfg.rotary_dim))
    ph = torch.outer(torch.arange(cfg.max_ctx, dtype=torch.float32, device=device), inv)
    ph = torch.cat((ph, ph), dim=-1)
    return ph.cos(), ph.sin()


def _layer_forward(self, hidden, mixer_args):
    mixed, *state = self.mixer(hidden, *mixer_args)
    attended = self.residual_add(hidden, mixed)
    return self.residual_add(attended, self.moe(attended)), tuple(state)


def _moe_forward(self, hidden):
    tokens = self.post_norm(hidden)
    weights, indices = self.router.routing(tokens)
    return self.experts(tokens, weights, indices)


def _make_root_methods(cfg: Qwen35Config):
    kinds = cfg.layer_types
    WIN = cfg.gdn_conv_kernel - 1

    def decode_hidden(self, hidden, layer_args, caches):
        if len(layer_args) != len(self.modules) or len(caches) != len(self.modules):
            raise ValueError(f"decoder has {len(self.modules)} layers but was given {len(layer_args)} argument "
                             f"tuples and {len(caches)} caches")
        states = []
        for layer, mixer_args, cache in zip(self.modules, layer_args, caches):
            hidden, state = layer(hidden, _with_cache(layer.mixer, mixer_args, cache))
            states.append(state)
        return self.final_rms_norm(hidden), tuple(states)

    def forward(self, token_ids, layer_args, caches):
        normed, states = self.decode_hidden(self.embed(token_ids), layer_args, caches)
        return self.lm_head(normed), states

    def init_caches(self, device=None):
        device = "cpu" if device is None else device
        out = []
        for kind in kinds:
            if kind == "linear_attention":
                out.append((torch.zeros(1, cfg.conv_dim, WIN, device=device),
                            torch.zeros(1, cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim, device=device)))
            else:
                empty = torch.zeros(1, 0, cfg.n_kv_heads, cfg.head_dim, device=device)
                out.append((empty, empty))
        return tuple(out)

    def append_cache(self, caches, fresh):
        out = []
        for kind, state, new in zip(kinds, caches, fresh):
            if kind == "linear_attention":
                out.append((torch.cat([state[0], new[0]], dim=2)[:, :, -WIN:], new[1]))
            else:
                out.append(tuple(torch.cat([old, n], dim=1) for old, n in zip(state, new)))
        return tuple(out)

    def prepare_inputs_for_generation(self, input_ids, step, caches, device=None):
        device = "cpu" if device is None else device
        token_ids = input_ids[step].reshape(1).to(device=device, dtype=torch.int64)
        cos, sin = rope_tables(cfg, str(device))
        pos_ids = torch.tensor([step], device=device, dtype=torch.int32)
        scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, device=device, dtype=torch.float32)
        layer_args = tuple(() if kind == "linear_attention" else (cos, sin, pos_ids, scale) for kind in kinds)
        return token_ids, layer_args, caches

    return {"decode_hidden": decode_hidden, "forward": forward, "init_caches": init_caches,
            "append_cache": append_cache, "prepare_inputs_for_generation": prepare_inputs_for_generation}


@lru_cache(maxsize=None)
def build(cfg: Qwen35Config = QWEN3_5_35B_A3B) -> Module:
    H, V = cfg.hidden, cfg.vocab
    HK, HV, DK, DV, KRN = cfg.gdn_n_k_heads, cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim, cfg.gdn_conv_kernel
    CONV, VAL, WIN = cfg.conv_dim, cfg.val_dim, cfg.gdn_conv_kernel - 1
    HQ, HKV, D, ROT, MC = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.rotary_dim, cfg.max_ctx
    E, K, I, IS = cfg.n_experts, cfg.top_k, cfg.moe_intermediate, cfg.shared_intermediate
    C = DimVar("ctx_len", 0, MC)

    gdn = Module(name="Qwen3_5LinearAttention", entry="linear_attention", functions=(
        func("conv_step", conv_state=T((1, CONV, WIN), F), entry=T((1, CONV, 1), F), conv_w=W((CONV, KRN), F)),
        func("l2_normalise", x=T((1, 1, HV, DK), F)),
        func("delta_step", recurrent_state=T((1, HV, DK, DV), F), q=T((1, 1, HV, DK), F), k=T((1, 1, HV, DK), F),
             v=T((1, 1, HV, DV), F), g=T((1, 1, HV), F), beta=T((1, 1, HV), F)),
        func("linear_attention", hidden=T((1, 1, H), F), gamma_in=W((H,), F), w_in_qkv=W((1, H, CONV), BW),
             w_in_z=W((1, H, VAL), BW), w_in_b=W((1, H, HV), BW), w_in_a=W((1, H, HV), BW), conv_w=W((CONV, KRN), F),
             a_log=W((HV,), F), dt_bias=W((HV,), F), conv_state=T((1, CONV, WIN), F),
             recurrent_state=T((1, HV, DK, DV), F), gamma_gdn=W((DV,), F), w_out=W((1, VAL, H), BW))))
    rope_args = dict(cos_cache=T((MC, ROT), F), sin_cache=T((MC, ROT), F), pos_ids=T((1,), "i32"))
    attn = Module(name="Qwen3_5FullAttention", entry="full_attention", functions=(
        func("partial_rope", x=T((1, 1, HQ, D), F), **rope_args),
        func("partial_rope_kv", x=T((1, 1, HKV, D), F), **rope_args),
        func("full_attention", hidden=T((1, 1, H), F), gamma_in=W((H,), F), w_qg=W((1, H, HQ * D * 2), BW),
             w_k=W((1, H, HKV * D), BW), w_v=W((1, H, HKV * D), BW), gamma_q=W((D,), F), gamma_k=W((D,), F),
             **rope_args, k_cache=T((1, C, HKV, D), F), v_cache=T((1, C, HKV, D), F), scale=T((1, 1, 1, 1), F),
             w_o=W((1, HQ * D, H), BW))))
    router = Module(name="Qwen3_5Router", entry="routing",
                    functions=(func("routing", tokens=T((1, H), F), w_router=W((H, E), BW)),))
    exp_w = dict(w_gate=W((E, I, H), BW), w_up=W((E, I, H), BW), w_down=W((E, H, I), BW))
    sh_w = dict(w_shared_gate=W((H, IS), BW), w_shared_up=W((H, IS), BW), w_shared_down=W((IS, H), BW),
                w_shared_scale=W((H, 1), BW))
    moe = Module(name="Qwen3_5MoE", entry="experts", modules=(router.renamed("router"),),
                 methods={"forward": _moe_forward}, functions=(
        func("post_norm", hidden=T((1, 1, H), F), gamma_post=W((H,), F)),
        func("routed_experts", tokens=T((1, H), F), weights=T((1, K), F), indices=T((1, K), "i64"), **exp_w),
        func("shared_expert", tokens=T((1, H), F), **sh_w),
        func("experts", tokens=T((1, H), F), weights=T((1, K), F), indices=T((1, K), "i64"), **exp_w, **sh_w)))
    residual = func("residual_add", a=T((1, 1, H), F), b=T((1, 1, H), F))

    def layer(name, mixer):
        return Module(name=name, entry="residual_add", functions=(residual,),
                      modules=(mixer.renamed("mixer"), moe.renamed("moe")), methods={"forward": _layer_forward})

    kinds = {"linear_attention": layer("Qwen3_5LinearAttnLayer", gdn), "full_attention": layer("Qwen3_5FullAttnLayer", attn)}
    return Module(
        name="Qwen3_5Decoder",
        functions=(func("embed", table=W((V, H), BW), token_ids=T((1,), "i64")),
                   func("final_rms_norm", hidden=T((1, 1, H), F), gamma_final=W((H,), F)),
                   func("lm_head", hidden=T((1, 1, H), F), w_head=W((H, V), BW))),
        modules=tuple(kinds[k].renamed(f"layer{i}") for i, k in enumerate(cfg.layer_types)),
        methods=_make_root_methods(cfg), metadata={"config": cfg})


def weight_overrides(name, ty, gen):
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "a_log":                      # decay rate exp(a_log) in [1, 16]
        return torch.log(1.0 + 15.0 * torch.rand(ty.shape[0], generator=gen))
    if leaf == "dt_bias":
        dt = torch.exp(torch.rand(ty.shape[0], generator=gen) * (torch.log(torch.tensor(0.1)) - torch.log(torch.tensor(1e-3)))
                       + torch.log(torch.tensor(1e-3)))
        return dt + torch.log(-torch.expm1(-dt))
    if leaf == "conv_w":
        return torch.randn(tuple(ty.shape), generator=gen) * 0.3
    return None

