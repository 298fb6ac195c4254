"""Weight preparation for the Qwen3 decode sessions: checkpoint names -> authored names -> kernel layout -> one file.

The reference prepares weights in two steps: an alias table maps the authored ``ConstTensor`` names onto a published
checkpoint's keys (``tests/models/qwen3_1_7b/hf_alias.py``; lookup rules ``src/tilefoundry/runtime/resource.py:63-85``)
and ``Module.prepare`` runs the converters that fold and repack them (``src/tilefoundry/ir/core/module.py:505-582``).
Here the same two steps end in the layout the kernels read: every projection ``[out, in]`` row-major bf16 (which is the
checkpoint's own ``nn.Linear`` layout, so packing is concatenation, never a transpose of a large matrix), q|k|v fused,
gate rows followed by up rows.  ``save_packed`` writes that layout as one safetensors file, ``load_packed`` reads it
back (memory-mapped) into what ``Qwen3Session`` / ``Qwen3BatchSession`` take in place of a resource.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

from ..authored.qwen3_1_7b import Qwen3Config
from ..runtime.resource import Preprocessed

FORMAT = "tfb200-qwen3-packed-v1"
LAYER_TENSORS = ("gamma_in", "gamma_post", "gamma_q", "gamma_k", "w_qkv", "w_o", "w_gate_up", "w_down")


def hf_alias(cfg: Qwen3Config, tied_head: bool = True) -> dict:
    """Alias table for a Hugging Face ``Qwen3ForCausalLM`` checkpoint: authored name -> checkpoint key.  Authored
    projections are declared ``(1, in, out)``; ``nn.Linear.weight`` is ``(out, in)``."""
    to_authored = lambda t: t.t().unsqueeze(0)
    alias = {
        "w_embed": "model.embed_tokens.weight",
        "gamma_final": "model.norm.weight",
        "w_head": Preprocessed("model.embed_tokens.weight" if tied_head else "lm_head.weight", lambda t: t.t()),
        "gamma_in": "input_layernorm.weight", "gamma_post": "post_attention_layernorm.weight",
        "gamma_q": "self_attn.q_norm.weight", "gamma_k": "self_attn.k_norm.weight",
    }
    for ours, theirs in (("w_q", "self_attn.q_proj"), ("w_k", "self_attn.k_proj"), ("w_v", "self_attn.v_proj"),
                         ("w_o", "self_attn.o_proj"), ("w_gate", "mlp.gate_proj"), ("w_up", "mlp.up_proj"),
                         ("w_down", "mlp.down_proj")):
        alias[ours] = Preprocessed(f"{theirs}.weight", to_authored)
    for i in range(cfg.num_hidden_layers):
        alias[f"layer{i}"] = f"model.layers.{i}"
    return alias


class PackedQwen3:
    """Kernel-layout weights: ``root`` = {w_embed, w_head (None when tied), gamma_final}, ``layers`` = one dict of
    LAYER_TENSORS per layer (``w_gate`` / ``w_up`` are views of ``w_gate_up``)."""

    def __init__(self, root: dict, layers: list):
        self.root, self.layers = root, layers

    def to(self, device) -> "PackedQwen3":
        move = lambda t: None if t is None else t.to(device)
        layers = []
        for layer in self.layers:
            out = {k: move(layer[k]) for k in LAYER_TENSORS}
            inter = out["w_gate_up"].shape[0] // 2
            out["w_gate"], out["w_up"] = out["w_gate_up"][:inter], out["w_gate_up"][inter:]
            layers.append(out)
        return PackedQwen3({k: move(v) for k, v in self.root.items()}, layers)


def pack(cfg: Qwen3Config, resource) -> PackedQwen3:
    """Authored names (any resource: a dict of seeded weights, an aliased checkpoint) -> kernel layout."""
    from .qwen3 import pack_layer
    names = ("gamma_in", "w_q", "w_k", "w_v", "gamma_q", "gamma_k", "w_o", "gamma_post", "w_gate", "w_up", "w_down")
    embed = resource.load("w_embed").contiguous()
    head = resource.load("w_head").t().contiguous()
    root = {"w_embed": embed, "w_head": None if torch.equal(head, embed) else head,
            "gamma_final": resource.load("gamma_final").contiguous()}
    layers = []
    for i in range(cfg.num_hidden_layers):
        sub = resource.subtree(f"layer{i}")
        layers.append(pack_layer({n: sub.load(n) for n in names}))
    return PackedQwen3(root, layers)


def save_packed(path, cfg: Qwen3Config, packed: PackedQwen3) -> None:
    from safetensors.torch import save_file
    tensors = {k: v.cpu().contiguous() for k, v in packed.root.items() if v is not None}
    for i, layer in enumerate(packed.layers):
        for k in LAYER_TENSORS:
            tensors[f"layers.{i}.{k}"] = layer[k].cpu().contiguous()
    dims = {k: getattr(cfg, k) for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                         "intermediate_size", "vocab_size", "num_hidden_layers")}
    meta = {"format": FORMAT, "tied_head": str(packed.root["w_head"] is None), "dims": json.dumps(dims)}
    save_file(tensors, str(Path(path)), metadata=meta)


def load_packed(path, cfg: Qwen3Config, device="cpu") -> PackedQwen3:
    """Read a file written by save_packed (memory-mapped; tensors land on *device*).  Raises if the file is of
    another format or was packed for other dimensions."""
    from safetensors import safe_open
    with safe_open(str(Path(path)), framework="pt", device=str(device)) as fh:
        meta = fh.metadata() or {}
        if meta.get("format") != FORMAT:
            raise ValueError(f"{path}: not a {FORMAT} file (format {meta.get('format')!r})")
        dims = json.loads(meta["dims"])
        for k, v in dims.items():
            if getattr(cfg, k) != v:
                raise ValueError(f"{path}: packed for {k}={v}, the configuration has {getattr(cfg, k)}")
        keys = set(fh.keys())
        root = {"w_embed": fh.get_tensor("w_embed"), "gamma_final": fh.get_tensor("gamma_final"),
                "w_head": fh.get_tensor("w_head") if "w_head" in keys else None}
        layers = [{k: fh.get_tensor(f"layers.{i}.{k}") for k in LAYER_TENSORS} for i in range(cfg.num_hidden_layers)]
    return PackedQwen3(root, layers).to(device)
