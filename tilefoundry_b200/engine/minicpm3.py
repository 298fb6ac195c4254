"""MiniCPM3-architecture (MLA) decode session: packed weights, paged cache, one captured step.

The cache holds LATENTS by default -- per position the normalised compressed kv vector and the rotated shared
rotary key, 576 bytes per layer -- and the kv up-projection runs absorbed into the query and the output
(``csrc/attn_mla_latent.cu``).  ``cache="assembled"`` keeps per-head keys and values instead (12,800 bytes per
position per layer), the format of the reference's own cache (``examples/minicpm3_4b-cutedsl/model.py:28-38``).
Weights are repacked at load as the reference's fast driver does (``runtime_model.py:248-320``)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored.minicpm3_4b import MiniCPM3Config, rope_tables
from . import paged_kv
from .session import DecodeSession


def split_gate_up(layer: dict) -> dict:
    """``w_gate`` / ``w_up`` as views of the layer's ``w_gate_up`` block (gate rows, then up rows)."""
    inter = layer["w_gate_up"].shape[0] // 2
    layer["w_gate"], layer["w_up"] = layer["w_gate_up"][:inter], layer["w_gate_up"][inter:]
    return layer


def pack_layer(w: dict) -> dict:
    """Authored ``(1, in, out)`` -> ``[out, in]``; q_a and kv_a fused along the output axis, gate and up rows in
    one block (the chunked prompt path runs them as one tensor-core projection; the decode step reads the two
    halves through the ``w_gate`` / ``w_up`` views)."""
    t = lambda name: w[name][0].t().contiguous()
    out = {n: w[n].contiguous() for n in ("gamma_in", "gamma_q_a", "gamma_kv_a", "gamma_post")}
    out.update(w_qkv_a=torch.cat([t("w_q_a"), t("w_kv_a")], dim=0).contiguous(), w_q_b=t("w_q_b"),
               w_kv_b=t("w_kv_b"), w_o=t("w_o"), w_gate_up=torch.cat([t("w_gate"), t("w_up")], dim=0).contiguous(),
               w_down=t("w_down"))
    return split_gate_up(out)


LAYER_WEIGHTS = ("gamma_in", "w_q_a", "gamma_q_a", "w_q_b", "w_kv_a", "gamma_kv_a", "w_kv_b", "w_o",
                 "gamma_post", "w_gate", "w_up", "w_down")


def pack_model(cfg: MiniCPM3Config, resource, device=None):
    """Authored names -> kernel layout (``engine/packed_models.py`` ``PackedModel``): the head is stored only when it
    is not the embedding table."""
    from .packed_models import PackedModel
    to = (lambda t: t) if device is None else (lambda t: t.to(device))
    embed = to(resource.load("w_embed")).contiguous()
    head = to(resource.load("w_head")).t().contiguous()
    root = {"w_embed": embed, "w_head": None if torch.equal(head, embed) else head,
            "gamma_final": to(resource.load("gamma_final")).contiguous()}
    layers = []
    for i in range(cfg.num_hidden_layers):
        sub = resource.subtree(f"layer{i}")
        layer = pack_layer({n: to(sub.load(n)) for n in LAYER_WEIGHTS})
        del layer["w_gate"], layer["w_up"]                      # views of w_gate_up: re-made where the block lands
        layers.append(layer)
    return PackedModel("minicpm3_4b", root, layers)


class MiniCPM3Session(DecodeSession):
    def __init__(self, cfg: MiniCPM3Config, resource, *, max_ctx: int = 2176, device="cuda:0",
                 keep_logits: bool = False, trace_hidden: bool = False, pdl: bool = True,
                 temperature: float = 0.0, seed: int = 0, cache: str = "latent"):
        if not torch.cuda.is_available():
            raise RuntimeError("MiniCPM3Session needs a CUDA device; there is no CPU path")
        if cache not in ("latent", "assembled"):
            raise ValueError(f"cache must be 'latent' or 'assembled', not {cache!r}")
        lib.load()
        self.cache = cache
        latent = cache == "latent"
        self.cfg, self.device, self.max_ctx = cfg, torch.device(device), int(max_ctx)
        dev = self.device
        from .packed_models import PackedModel
        # a resource speaks the authored names and is packed here; a PackedModel is already in the kernels' layout
        # (e.g. read from a file written by engine/packed_models.py save_packed)
        packed = (resource if isinstance(resource, PackedModel) else pack_model(cfg, resource, dev)).to(dev)
        self.w_embed = packed.root["w_embed"]
        self.w_head = self.w_embed if packed.root["w_head"] is None else packed.root["w_head"]
        self.gamma_final = packed.root["gamma_final"]
        self.layers = [split_gate_up(dict(layer)) for layer in packed.layers]

        cos, sin = rope_tables(cfg, "cpu")
        self.max_pos = min(cfg.max_position_embeddings, self.max_ctx)
        self.cos, self.sin = cos[: self.max_pos].contiguous().to(dev), sin[: self.max_pos].contiguous().to(dev)
        NH, QK, VD, H, I, V = (cfg.num_attention_heads, cfg.qk_head_dim, cfg.v_head_dim, cfg.hidden_size,
                               cfg.intermediate_size, cfg.vocab_size)
        self.table = paged_kv.block_table(1, self.max_ctx, device=dev)
        LAT = cfg.kv_lora_rank + cfg.qk_rope_head_dim
        for layer in self.layers:
            if latent:
                layer["k_pool"], layer["v_pool"] = paged_kv.new_pool(1, self.max_ctx, 1, LAT, device=dev), None
            else:
                layer["k_pool"] = paged_kv.new_pool(1, self.max_ctx, NH, QK, device=dev)
                layer["v_pool"] = paged_kv.new_pool(1, self.max_ctx, NH, VD, device=dev)
        bf, f32 = torch.bfloat16, torch.float32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        nsplit = lib.load().tfb_mla_latent_splits(self.max_ctx) if latent else lib.attn_splits(self.max_ctx)
        PD = cfg.kv_lora_rank if latent else VD                 # width of a split's partial output
        self.tokens, self.pos = z(self.max_ctx + 1, dtype=torch.int64), z(1, dtype=torch.int32)
        self.hidden = z(H)
        self.qkv_a = z(cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_head_dim)
        self.q_up, self.kv_up = z(NH * QK), z(NH * (cfg.qk_nope_head_dim + VD))
        self.attn, self.act = z(NH * VD), z(I)
        self.logits = z(V) if keep_logits else None
        self.part_o, self.part_ml = z(NH * nsplit * PD, dtype=f32), z(NH * nsplit * 2, dtype=f32)
        self.q_lat = z(NH * 2 * cfg.kv_lora_rank, dtype=f32) if latent else None
        self.q_rope = z(NH * cfg.qk_rope_head_dim, dtype=f32) if latent else None
        self.counters = z(NH + 1, dtype=torch.int32)
        n_head = lib.lm_head_scratch_entries(V)
        self.head_val, self.head_idx = z(n_head, dtype=f32), z(n_head, dtype=torch.int32)
        self.trace = z(cfg.num_hidden_layers + 1, H) if trace_hidden else None
        self.picked = z(1, dtype=torch.int64)

        self._layer_structs = (lib.MiniCPM3Layer * len(self.layers))()
        for s, layer in zip(self._layer_structs, self.layers):
            for name, _ in lib.MiniCPM3Layer._fields_:
                setattr(s, name, lib.ptr(layer[name]))
        as_bf16 = lambda v: float(torch.tensor(v, dtype=bf))    # the authored step holds these as bf16 tensors
        self.args = lib.MiniCPM3StepArgs(
            temperature=float(temperature), seed=int(seed) & (2 ** 64 - 1),
            layers=self._layer_structs, n_layers=len(self.layers), hidden=H, heads=NH, q_lora=cfg.q_lora_rank,
            kv_lora=cfg.kv_lora_rank, nope=cfg.qk_nope_head_dim, rope=cfg.qk_rope_head_dim, v=VD, inter=I, vocab=V,
            eps=cfg.rms_norm_eps, lora_eps=cfg.lora_eps, scale=as_bf16(QK ** -0.5), embed_scale=cfg.scale_emb,
            residual_scale=as_bf16(cfg.residual_scale), logits_div=cfg.logits_scaling,
            w_embed=lib.ptr(self.w_embed), gamma_final=lib.ptr(self.gamma_final), w_head=lib.ptr(self.w_head),
            cos_table=lib.ptr(self.cos), sin_table=lib.ptr(self.sin), max_pos=self.max_pos,
            page_size=paged_kv.PAGE_SIZE, table_len=self.table.shape[1], max_ctx=self.max_ctx,
            block_table=lib.ptr(self.table), tokens=lib.ptr(self.tokens), pos=lib.ptr(self.pos), n_prompt=0,
            max_tokens=self.max_ctx + 1, hidden_buf=lib.ptr(self.hidden), qkv_a_buf=lib.ptr(self.qkv_a),
            q_up_buf=lib.ptr(self.q_up), kv_up_buf=lib.ptr(self.kv_up), attn_buf=lib.ptr(self.attn),
            act_buf=lib.ptr(self.act), logits=lib.ptr(self.logits), part_o=lib.ptr(self.part_o),
            part_ml=lib.ptr(self.part_ml), counters=lib.ptr(self.counters), head_val=lib.ptr(self.head_val),
            head_idx=lib.ptr(self.head_idx), hidden_trace=lib.ptr(self.trace), picked=lib.ptr(self.picked),
            pdl=int(pdl), cache_layout=lib.MLA_CACHE_LATENT if latent else lib.MLA_CACHE_ASSEMBLED,
            q_lat_buf=lib.ptr(self.q_lat), q_rope_buf=lib.ptr(self.q_rope))
        self.launches_per_step = (2 + (7 if latent else 6) * len(self.layers)
                                  + (len(self.layers) + 1 if trace_hidden else 0))

    def weight_bytes(self) -> int:
        names = ("w_qkv_a", "w_q_b", "w_kv_b", "w_o", "w_gate", "w_up", "w_down")
        return sum(self.layers[0][n].numel() * 2 for n in names) * len(self.layers) + self.w_head.numel() * 2

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        if self.cache == "latent":
            return (c.kv_lora_rank + c.qk_rope_head_dim) * 2 * c.num_hidden_layers
        return c.num_attention_heads * (c.qk_head_dim + c.v_head_dim) * 2 * c.num_hidden_layers

    def assembled_cache(self, layer: int, length: int):
        """``(k [1, length, heads, qk], v [1, length, heads, v])`` of a layer as the authored functions hold them.
        With the latent cache the rows are re-expanded through ``w_kv_b`` in the authored arithmetic (one bf16
        matmul per row, ``examples/minicpm3_4b-cutedsl/model.py:236-247``): a view for checks, not a step of decode."""
        c, L = self.cfg, self.layers[layer]
        if self.cache != "latent":
            return (paged_kv.logical_view(L["k_pool"], self.table[0], length),
                    paged_kv.logical_view(L["v_pool"], self.table[0], length))
        NH, NOPE, R, VD, KVL = (c.num_attention_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim,
                                c.kv_lora_rank)
        rows = paged_kv.logical_view(L["k_pool"], self.table[0], length)[0, :, 0].cpu()       # [length, kvl + rope]
        kv = torch.matmul(rows[:, :KVL], L["w_kv_b"].cpu().t()).reshape(length, NH, NOPE + VD)
        k = torch.cat([kv[:, :, :NOPE], rows[:, None, KVL:].expand(length, NH, R)], dim=-1)
        return k.unsqueeze(0).contiguous(), kv[:, :, NOPE:].unsqueeze(0).contiguous()

    def step(self) -> None:
        lib.check(lib.load().tfb_minicpm3_decode_step(C.byref(self.args), lib.stream()), "tfb_minicpm3_decode_step")

    def prefill(self, n_tokens: int) -> None:
        """Process positions ``pos .. pos + n_tokens - 1`` of the token history in chunks of up to 32 tokens
        (projections once per chunk on the tensor cores, attention token by token over the latent cache) instead of
        one decode step each, and advance the position.  Nothing is picked.  Latent cache only."""
        from .minicpm3_prefill import MiniCPM3Prefill
        if self.cache != "latent":
            raise ValueError("chunked prompt processing is built for the latent cache")
        if getattr(self, "_prefill", None) is None:
            self._prefill = MiniCPM3Prefill(self)
        self._prefill.run(n_tokens)

    def generate(self, prompt_ids, max_new: int, use_graph: bool = True, prefill: bool = False, eos=None):
        """As DecodeSession.generate; with ``prefill`` the prompt (all but its last token) is processed in chunks."""
        if not prefill:
            return super().generate(prompt_ids, max_new, use_graph, eos)
        from .session import Generated
        if eos is not None:
            self.set_eos(eos)
        self.reset(prompt_ids)
        if self.n_prompt + max_new > self.max_ctx + 1:
            raise ValueError(f"{self.n_prompt}+{max_new} tokens exceed capacity {self.max_ctx}")
        if use_graph and self.graph is None:
            self.capture()
        start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        start.record()
        self.prefill(self.n_prompt - 1)
        mid.record()
        self.run(max_new, use_graph)
        end.record()
        torch.cuda.synchronize()
        self._prefill.check_status()
        out = self.tokens[self.n_prompt: self.generated_end(self.n_prompt + max_new)].tolist()
        return Generated(out, mid.elapsed_time(end) / 1e3, start.elapsed_time(mid) / 1e3, self.n_prompt)
