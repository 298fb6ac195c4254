"""Weight preparation for the MiniCPM3, granite and Qwen3.5 sessions: checkpoint names -> authored names -> kernel
layout -> one file, and back.  (``engine/packed.py`` is the same for Qwen3.)

The reference does this in two steps: an alias table maps the authored ``ConstTensor`` names onto a published
checkpoint's keys (``examples/minicpm3_4b-cutedsl/hf_alias.py:25-49``, ``examples/granite_4_0_h_small-cuda/
hf_alias.py:42-88``; lookup rules ``src/tilefoundry/runtime/resource.py:63-85``) and ``Module.prepare`` runs the
converters that fold and repack them (``src/tilefoundry/ir/core/module.py:505-582``).  Here the two steps end in the
layout the kernels read (each engine module's ``pack_model``: projections ``[out, in]`` row-major bf16, the ones
that share an input concatenated, expert slabs as declared), written as ONE safetensors file per model with the
dimensions in its metadata.  A session takes the loaded ``PackedModel`` in place of a resource; for several GPUs it
cuts its shard out of the packed tensors.  The Qwen3.5 checkpoint differs from its authored weights by more than
names (``1 + w`` gains, ``nn.Linear`` layouts, one fused gate/up tensor per layer's experts:
``examples/qwen3_5_35b_a3b-tilelang/model.py:232-287,421-476,501-505,607-652,809-820``); every one of those converters
takes a single raw tensor, so they are read-side transforms of the alias table here (``hf_alias_qwen3_5``).
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path

import torch

from ..runtime.resource import Absolute, Preprocessed

FORMAT = "tfb200-packed-v1"


class PackedModel:
    """Kernel-layout weights of one model: ``root`` = name -> tensor (``None`` for a head tied to the embedding),
    ``layers`` = one name -> tensor dict per layer.  ``key`` names the architecture."""

    def __init__(self, key: str, root: dict, layers: list):
        self.key, self.root, self.layers = key, root, layers

    def to(self, device) -> "PackedModel":
        move = lambda t: None if t is None else t.to(device)
        return PackedModel(self.key, {k: move(v) for k, v in self.root.items()},
                           [{k: move(v) for k, v in layer.items()} for layer in self.layers])


def pack(key: str, cfg, resource) -> PackedModel:
    """Authored names (a dict of seeded weights, an aliased checkpoint, a directory) -> kernel layout."""
    if key == "minicpm3_4b":
        from .minicpm3 import pack_model
    elif key == "granite_4_0_h_small":
        from .granite import pack_model
    elif key == "qwen3_5_35b_a3b":
        from .qwen3_5 import pack_model
    else:
        raise ValueError(f"no packed format for {key!r}")
    return pack_model(cfg, resource)


def _dims(cfg) -> dict:
    return {f.name: getattr(cfg, f.name) for f in dataclasses.fields(cfg)
            if isinstance(getattr(cfg, f.name), (int, float, str, bool, tuple, list))}


def save_packed(path, cfg, packed: PackedModel) -> None:
    from safetensors.torch import save_file
    tensors = {f"root.{k}": v.cpu().contiguous() for k, v in packed.root.items() if v is not None}
    for i, layer in enumerate(packed.layers):
        for k, v in layer.items():
            tensors[f"layers.{i}.{k}"] = v.cpu().contiguous()
    meta = {"format": FORMAT, "model": packed.key, "n_layers": str(len(packed.layers)),
            "absent": json.dumps(sorted(k for k, v in packed.root.items() if v is None)),
            "dims": json.dumps(_dims(cfg), default=list)}
    save_file(tensors, str(Path(path)), metadata=meta)


def load_packed(path, key: str, cfg, device="cpu") -> PackedModel:
    """Read a file written by ``save_packed`` (memory-mapped; tensors land on *device*).  Raises if the file is of
    another format or model, or was packed for other dimensions."""
    from safetensors import safe_open
    with safe_open(str(Path(path)), framework="pt", device=str(device)) as fh:
        meta = fh.metadata() or {}
        if meta.get("format") != FORMAT or meta.get("model") != key:
            raise ValueError(f"{path}: not a {FORMAT} file of {key} (format {meta.get('format')!r}, model {meta.get('model')!r})")
        want = json.loads(json.dumps(_dims(cfg), default=list))
        for k, v in json.loads(meta["dims"]).items():
            if want.get(k) != v:
                raise ValueError(f"{path}: packed for {k}={v}, the configuration has {want.get(k)}")
        root = {k: None for k in json.loads(meta["absent"])}
        layers = [dict() for _ in range(int(meta["n_layers"]))]
        for name in fh.keys():
            if name.startswith("root."):
                root[name[5:]] = fh.get_tensor(name)
            else:
                _, i, k = name.split(".", 2)
                layers[int(i)][k] = fh.get_tensor(name)
    return PackedModel(key, root, layers)


# ---- alias tables: a Hugging Face checkpoint read under the authored names ------------------------------------
def _projection(t: torch.Tensor) -> torch.Tensor:
    """``nn.Linear.weight`` ``(out, in)`` -> the authored ``(1, in, out)``."""
    return t.t().unsqueeze(0).contiguous()


def hf_alias_minicpm3(cfg) -> dict:
    """Authored name -> key of a Hugging Face ``MiniCPM3ForCausalLM`` checkpoint (every projection is an
    ``nn.Linear``; the low-rank a / b projections are separate tensors there too)."""
    alias = {"w_embed": "model.embed_tokens.weight", "gamma_final": "model.norm.weight",
             "w_head": Preprocessed("lm_head.weight", lambda t: t.t().contiguous()),
             "gamma_in": "input_layernorm.weight", "gamma_post": "post_attention_layernorm.weight",
             "gamma_q_a": "self_attn.q_a_layernorm.weight", "gamma_kv_a": "self_attn.kv_a_layernorm.weight"}
    for ours, theirs in (("w_q_a", "self_attn.q_a_proj"), ("w_q_b", "self_attn.q_b_proj"),
                         ("w_kv_a", "self_attn.kv_a_proj_with_mqa"), ("w_kv_b", "self_attn.kv_b_proj"),
                         ("w_o", "self_attn.o_proj"), ("w_gate", "mlp.gate_proj"), ("w_up", "mlp.up_proj"),
                         ("w_down", "mlp.down_proj")):
        alias[ours] = Preprocessed(f"{theirs}.weight", _projection)
    for i in range(cfg.num_hidden_layers):
        alias[f"layer{i}"] = f"model.layers.{i}"
    return alias


def hf_alias_granite(cfg) -> dict:
    """Authored name -> key of a Hugging Face ``GraniteMoeHybridForCausalLM`` checkpoint.  The authored projections
    are declared ``[out, in]`` like ``nn.Linear``; what differs is where things sit: both pre-norms live on the
    layer, one level above the block that uses them; the shared MLP is a sibling of the sparse block; each layer's
    experts are one fused ``input_linear`` (gate rows then up rows); the depthwise convolution carries a singleton
    axis."""
    inter = cfg.intermediate_size
    alias = {"table": "model.embed_tokens.weight", "gamma_final": "model.norm.weight",
             "w_in": "in_proj.weight", "conv_w": Preprocessed("conv1d.weight", lambda t: t.squeeze(1).contiguous()),
             "conv_b": "conv1d.bias", "a_log": "A_log", "dt_bias": "dt_bias", "d_skip": "D", "gamma_ssm": "norm.weight",
             "w_out": "out_proj.weight", "w_q": "q_proj.weight", "w_k": "k_proj.weight", "w_v": "v_proj.weight",
             "w_o": "o_proj.weight",
             "w_gate": Preprocessed("input_linear.weight", lambda t: t[:, :inter].contiguous()),
             "w_up": Preprocessed("input_linear.weight", lambda t: t[:, inter:].contiguous()),
             "w_down": "output_linear.weight", "w_router": "layer.weight"}
    for i, kind in enumerate(cfg.layer_types):
        layer = f"model.layers.{i}"
        mixer = "mamba" if kind == "linear_attention" else "self_attn"
        alias[f"layer{i}"] = layer
        alias[f"{layer}.mixer"] = mixer
        alias[f"{layer}.moe"] = "block_sparse_moe"
        alias[f"{layer}.{mixer}.gamma_in"] = Absolute(f"{layer}.input_layernorm.weight")
        alias[f"{layer}.block_sparse_moe.gamma_post"] = Absolute(f"{layer}.post_attention_layernorm.weight")
        alias[f"{layer}.block_sparse_moe.w_shared_in"] = Absolute(f"{layer}.shared_mlp.input_linear.weight")
        alias[f"{layer}.block_sparse_moe.w_shared_out"] = Absolute(f"{layer}.shared_mlp.output_linear.weight")
    return alias


def hf_alias_qwen3_5(cfg, text_prefix: str = "model.language_model", head: str = "lm_head.weight") -> dict:
    """Authored name -> key of a Hugging Face ``Qwen3_5MoeForConditionalGeneration`` checkpoint, with the read-side
    transform each weight needs (raw names: ``examples/qwen3_5_35b_a3b-tilelang/model.py:931-965``).  What differs:
    the norms of this family multiply by ``1 + w`` where the authored ``rms_norm`` multiplies by ``w`` (all but the
    gated norm of the linear-attention read-out); every ``nn.Linear`` is ``(out, in)`` where the authored matmuls
    take ``(in, out)``; the experts' gate and up projections are the two halves of one ``(experts, 2 * inter,
    hidden)`` tensor, gate first; the depthwise convolution keeps a singleton axis.  Gains, ``A_log``, ``dt_bias`` and
    the convolution kernel are read as f32 (they are added to and exponentiated, not contracted over), the matmul
    weights stay bf16.  A tied head is ``head=`` the embedding's key."""
    inter = cfg.moe_intermediate
    gain = lambda t: t.float() + 1.0
    f32 = lambda t: t.float().contiguous()
    linear = lambda t: t.t().unsqueeze(0).contiguous()            # (out, in) -> (1, in, out)
    flip = lambda t: t.t().contiguous()                            # (a, b) -> (b, a)
    pre = text_prefix
    alias = {"table": Absolute(f"{pre}.embed_tokens.weight"),
             "gamma_final": Preprocessed(Absolute(f"{pre}.norm.weight"), gain),
             "w_head": Preprocessed(Absolute(head), flip)}
    gdn = {"gamma_in": ("input_layernorm.weight", gain), "w_in_qkv": ("linear_attn.in_proj_qkv.weight", linear),
           "w_in_z": ("linear_attn.in_proj_z.weight", linear), "w_in_b": ("linear_attn.in_proj_b.weight", linear),
           "w_in_a": ("linear_attn.in_proj_a.weight", linear),
           "conv_w": ("linear_attn.conv1d.weight", lambda t: t.float().squeeze(1).contiguous()),
           "a_log": ("linear_attn.A_log", f32), "dt_bias": ("linear_attn.dt_bias", f32),
           "gamma_gdn": ("linear_attn.norm.weight", f32), "w_out": ("linear_attn.out_proj.weight", linear)}
    attn = {"gamma_in": ("input_layernorm.weight", gain), "w_qg": ("self_attn.q_proj.weight", linear),
            "w_k": ("self_attn.k_proj.weight", linear), "w_v": ("self_attn.v_proj.weight", linear),
            "gamma_q": ("self_attn.q_norm.weight", gain), "gamma_k": ("self_attn.k_norm.weight", gain),
            "w_o": ("self_attn.o_proj.weight", linear)}
    moe = {"gamma_post": ("post_attention_layernorm.weight", gain),
           "w_gate": ("mlp.experts.gate_up_proj", lambda t: t[:, :inter, :].contiguous()),
           "w_up": ("mlp.experts.gate_up_proj", lambda t: t[:, inter:, :].contiguous()),
           "w_down": ("mlp.experts.down_proj", lambda t: t.contiguous()),
           "w_shared_gate": ("mlp.shared_expert.gate_proj.weight", flip),
           "w_shared_up": ("mlp.shared_expert.up_proj.weight", flip),
           "w_shared_down": ("mlp.shared_expert.down_proj.weight", flip),
           "w_shared_scale": ("mlp.shared_expert_gate.weight", flip)}
    for i, kind in enumerate(cfg.layer_types):
        layer = f"{pre}.layers.{i}"
        for ours, (theirs, read) in (gdn if kind == "linear_attention" else attn).items():
            alias[f"layer{i}.mixer.{ours}"] = Preprocessed(Absolute(f"{layer}.{theirs}"), read)
        for ours, (theirs, read) in moe.items():
            alias[f"layer{i}.moe.{ours}"] = Preprocessed(Absolute(f"{layer}.{theirs}"), read)
        alias[f"layer{i}.moe.router.w_router"] = Preprocessed(Absolute(f"{layer}.mlp.gate.weight"), flip)
    return alias
