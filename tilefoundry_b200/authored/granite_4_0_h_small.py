"""granite-4.0-h-small decode step (Mamba-2 / attention hybrid + MoE): declared signatures and orchestration.

Mirrors reference ``examples/granite_4_0_h_small-cuda/model.py``: Modules ``GraniteMamba`` (functions
``in_projection conv_step ssm_step gated_out mamba_mixer``, ``:142-274``), ``GraniteAttention`` (``qkv attend
full_attention``, ``:282-373``), ``GraniteRouter`` (``routing``, ``:376-386``), ``GraniteMoE`` (``post_norm
routed_experts shared_mlp experts`` + child ``router`` + ``forward``, ``:389-478``), the two decoder-layer
Modules (``residual_add`` + children ``mixer``/``moe`` + ``forward``, ``:481-530``) and the root
(``embed final_rms_norm lm_head`` + orchestration, ``:601-719``).  Weights are declared ``(out, in)``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from functools import lru_cache

import torch

from ..semantic import Module, T, W, func

MASKED = -1.0e30


@dataclass(frozen=True)
class GraniteConfig:
    hidden_size: int = 4096
    num_hidden_layers: int = 40
    attention_layers: tuple = (5, 15, 25, 35)
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    attention_multiplier: float = 0.0078125
    mamba_n_heads: int = 128
    mamba_d_head: int = 64
    mamba_d_state: int = 128
    mamba_n_groups: int = 1
    mamba_d_conv: int = 4
    num_local_experts: int = 72
    num_experts_per_tok: int = 10
    intermediate_size: int = 768
    shared_intermediate_size: int = 1536
    vocab_size: int = 100352
    rms_norm_eps: float = 1e-5
    embedding_multiplier: float = 12.0
    residual_multiplier: float = 0.22
    logits_scaling: float = 16.0
    max_ctx: int = 4096             # fixed KV capacity of the authored attention functions
    dtype: str = "bf16"

    @property
    def expand(self): return self.mamba_n_heads * self.mamba_d_head
    @property
    def conv_dim(self): return self.expand + 2 * self.mamba_n_groups * self.mamba_d_state
    @property
    def proj(self): return self.expand + self.conv_dim + self.mamba_n_heads
    @property
    def layer_types(self):
        return tuple("full_attention" if i in self.attention_layers else "linear_attention"
                     for i in range(self.num_hidden_layers))


GRANITE_4_0_H_SMALL = GraniteConfig()
GRANITE_TINY = GraniteConfig(hidden_size=256, num_hidden_layers=4, attention_layers=(2,), num_attention_heads=4,
                             num_key_value_heads=2, head_dim=64, mamba_n_heads=8, mamba_d_head=64,
                             num_local_experts=8, num_experts_per_tok=4, intermediate_size=256,
                             shared_intermediate_size=256, vocab_size=1000, max_ctx=256,
                             attention_multiplier=0.015625)


def truncated(cfg: GraniteConfig, **changes) -> GraniteConfig:
    """The same widths on a shorter stack / smaller vocabulary: what a host that cannot hold all 40 layers runs
    the evaluator on (the reference cuts its own large example the same way, ``examples/qwen3_5_35b_a3b-tilelang/
    config.py`` ``truncated``).  Kernel shapes depend on the widths only."""
    return replace(cfg, **changes)


def attention_mask(cfg, step, device="cpu"):
    """Additive mask of a step at position *step*: 0 for positions 0..step, -1e30 beyond (reference ``:584-598``)."""
    row = torch.where(torch.arange(cfg.max_ctx, device=device) <= step,
                      torch.zeros(cfg.max_ctx, device=device, dtype=torch.bfloat16),
                      torch.full((cfg.max_ctx,), MASKED, device=device, dtype=torch.bfloat16))
    return row.reshape(1, 1, cfg.max_ctx)


_CACHE_PARAMS = frozenset({"k_cache", "v_cache", "conv_state", "ssm_state"})


def _with_cache(mixer, mixer_args, cache):
    """*mixer_args* with *cache* spliced in where the mixer's entry declares its state (reference ``:537-551``)."""
    node = getattr(mixer, "module", mixer)
    names = [p.name for p in node.lookup(node.entry).params if not p.is_const][1:]
    at = next(i for i, n in enumerate(names) if n in _CACHE_PARAMS)
    return (*mixer_args[:at], *cache, *mixer_args[at:])


def _layer_forward(self, hidden, mixer_args):
    mixed, *state = self.mixer(hidden, *mixer_args)
    attended = self.residual_add(hidden, mixed)
    return self.residual_add(attended, self.moe(attended)), tuple(state)


def _moe_forward(self, hidden):
    tokens = self.post_norm(hidden)
    weights, indices = self.router.routing(tokens)
    return self.experts(tokens, weights, indices)


def _make_root_methods(cfg: GraniteConfig):
    kinds = cfg.layer_types
    WIN = cfg.mamba_d_conv - 1

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
                out.append((torch.zeros(1, cfg.conv_dim, WIN, dtype=torch.bfloat16, device=device),
                            torch.zeros(1, cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state,
                                        dtype=torch.float32, device=device)))
            else:
                empty = torch.zeros(1, cfg.max_ctx, cfg.num_key_value_heads, cfg.head_dim, dtype=torch.bfloat16,
                                    device=device)
                out.append((empty, empty.clone()))
        return tuple(out)

    def append_cache(self, caches, fresh):
        out = []
        for kind, (a, b), new in zip(kinds, caches, fresh):
            if kind == "linear_attention":
                column, updated = new
                out.append((torch.cat([a, column], dim=2)[:, :, -WIN:], updated))
            else:
                out.append(tuple(new))
        return tuple(out)

    def prepare_inputs_for_generation(self, input_ids, step, caches, device=None):
        device = "cpu" if device is None else device
        token_ids = input_ids[step].reshape(1).to(device=device, dtype=torch.int64)
        cur_pos = torch.full((1,), step, device=device, dtype=torch.int32)
        mask = attention_mask(cfg, step, device)
        layer_args = tuple(() if kind == "linear_attention" else (cur_pos, mask) for kind in kinds)
        return token_ids, layer_args, caches

    return {"decode_hidden": decode_hidden, "forward": forward, "init_caches": init_caches,
            "append_cache": append_cache, "prepare_inputs_for_generation": prepare_inputs_for_generation}


@lru_cache(maxsize=None)
def build(cfg: GraniteConfig = GRANITE_4_0_H_SMALL) -> Module:
    H, V = cfg.hidden_size, cfg.vocab_size
    NH, PD, NS, NG, KRN = cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_n_groups, cfg.mamba_d_conv
    EXP, CONVD, PROJ, WIN = cfg.expand, cfg.conv_dim, cfg.proj, cfg.mamba_d_conv - 1
    HQ, HKV, D, CAP = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx
    E, K, I, IS = cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size, cfg.shared_intermediate_size

    ssm_params = dict(ssm_state=T((1, NH, PD, NS), "f32"), x=T((1, NH, PD)), b_vec=T((1, NG, NS)), c_vec=T((1, NG, NS)),
                      dt_raw=T((1, NH)), a_log=W((NH,)), dt_bias=W((NH,)), d_skip=W((NH,)))
    mamba = Module(name="GraniteMamba", entry="mamba_mixer", functions=(
        func("in_projection", hidden=T((1, 1, H)), gamma_in=W((H,)), w_in=W((PROJ, H))),
        func("conv_step", conv_state=T((1, CONVD, WIN)), entry=T((1, CONVD, 1)), conv_w=W((CONVD, KRN)),
             conv_b=W((CONVD,))),
        func("ssm_step", **ssm_params),
        func("gated_out", y=T((1, NH, PD)), gate=T((1, EXP)), gamma_ssm=W((EXP,)), w_out=W((H, EXP))),
        func("mamba_mixer", hidden=T((1, 1, H)), gamma_in=W((H,)), w_in=W((PROJ, H)), conv_w=W((CONVD, KRN)),
             conv_b=W((CONVD,)), a_log=W((NH,)), dt_bias=W((NH,)), d_skip=W((NH,)),
             conv_state=T((1, CONVD, WIN)), ssm_state=T((1, NH, PD, NS), "f32"), gamma_ssm=W((EXP,)),
             w_out=W((H, EXP)))))
    qkv_w = dict(w_q=W((HQ * D, H)), w_k=W((HKV * D, H)), w_v=W((HKV * D, H)))
    attention = Module(name="GraniteAttention", entry="full_attention", functions=(
        func("qkv", hidden=T((1, 1, H)), gamma_in=W((H,)), **qkv_w),
        func("attend", q=T((1, 1, HQ, D)), k_cache=T((1, CAP, HKV, D)), v_cache=T((1, CAP, HKV, D)),
             cur_pos=T((1,), "i32"), mask=T((1, 1, CAP)), w_o=W((H, HQ * D))),
        func("full_attention", hidden=T((1, 1, H)), gamma_in=W((H,)), **qkv_w, k_cache=T((1, CAP, HKV, D)),
             v_cache=T((1, CAP, HKV, D)), cur_pos=T((1,), "i32"), mask=T((1, 1, CAP)), w_o=W((H, HQ * D)))))
    router = Module(name="GraniteRouter", entry="routing",
                    functions=(func("routing", tokens=T((1, H)), w_router=W((E, H))),))
    exp_w = dict(w_gate=W((E, I, H)), w_up=W((E, I, H)), w_down=W((E, H, I)))
    moe = Module(name="GraniteMoE", entry="experts", modules=(router.renamed("router"),),
                 methods={"forward": _moe_forward}, functions=(
        func("post_norm", hidden=T((1, 1, H)), gamma_post=W((H,))),
        func("routed_experts", tokens=T((1, H)), weights=T((1, K)), indices=T((1, K), "i64"), **exp_w),
        func("shared_mlp", tokens=T((1, H)), w_shared_in=W((2 * IS, H)), w_shared_out=W((H, IS))),
        func("experts", tokens=T((1, H)), weights=T((1, K)), indices=T((1, K), "i64"), **exp_w,
             w_shared_in=W((2 * IS, H)), w_shared_out=W((H, IS)))))
    residual = func("residual_add", a=T((1, 1, H)), b=T((1, 1, H)))

    def layer(name, mixer):
        return Module(name=name, entry="residual_add", functions=(residual,),
                      modules=(mixer.renamed("mixer"), moe.renamed("moe")), methods={"forward": _layer_forward})

    kinds = {"linear_attention": layer("GraniteMambaDecoderLayer", mamba),
             "full_attention": layer("GraniteAttentionDecoderLayer", attention)}
    return Module(
        name="Granite4_0_H_Small",
        functions=(func("embed", table=W((V, H)), token_ids=T((1,), "i64")),
                   func("final_rms_norm", hidden=T((1, 1, H)), gamma_final=W((H,))),
                   func("lm_head", hidden=T((1, 1, H)), table=W((V, H)))),
        modules=tuple(kinds[k].renamed(f"layer{i}") for i, k in enumerate(cfg.layer_types)),
        methods=_make_root_methods(cfg), metadata={"config": cfg})


def weight_overrides(name, ty, gen):
    """Distributions for the parameters N(0, 0.02) would make degenerate: decay rates and biases."""
    leaf = name.rsplit(".", 1)[-1]
    n = ty.shape[0]
    if leaf == "a_log":                      # A = -exp(a_log) in [-16, -1], as Mamba-2 initialises it
        return torch.log(1.0 + 15.0 * torch.rand(n, generator=gen))
    if leaf == "dt_bias":                    # softplus^-1 of dt in [1e-3, 1e-1]
        dt = torch.exp(torch.rand(n, generator=gen) * (torch.log(torch.tensor(0.1)) - torch.log(torch.tensor(1e-3)))
                       + torch.log(torch.tensor(1e-3)))
        return dt + torch.log(-torch.expm1(-dt))
    if leaf == "d_skip":
        return torch.ones(n)
    if leaf == "conv_w":
        return torch.randn(tuple(ty.shape), generator=gen) * 0.3
    return None
