"""Qwen3-architecture decode session: packed weights, paged KV, one captured step.

Where the authored step hands each token's key/value back for the caller to
``torch.cat`` (reference ``tests/models/qwen3_1_7b/model.py:370-383``), a session
keeps a fixed-capacity paged cache, the token history and the position on the
device, so every address a step touches is fixed and the step can be captured once
and replayed -- prompt walk and continuation alike -- with no host round trip
(the same trade the reference's own fast driver makes,
``examples/qwen3_1_7b-tilelang/fast/engine.py:1-21``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import lib
from ..authored.qwen3_1_7b import Qwen3Config, rope_tables
from . import paged_kv


@dataclass
class Generated:
    tokens: list
    seconds: float
    prompt_seconds: float
    prompt_steps: int

    @property
    def tokens_per_second(self) -> float:
        return len(self.tokens) / self.seconds


def pack_layer(w: dict) -> dict:
    """Authored ``(1, in, out)`` projections -> kernel layout ``[out, in]`` with q|k|v fused."""
    t = lambda name: w[name][0].t().contiguous()
    return {
        "gamma_in": w["gamma_in"].contiguous(), "gamma_post": w["gamma_post"].contiguous(),
        "gamma_q": w["gamma_q"].contiguous(), "gamma_k": w["gamma_k"].contiguous(),
        "w_qkv": torch.cat([t("w_q"), t("w_k"), t("w_v")], dim=0).contiguous(),
        "w_o": t("w_o"), "w_gate": t("w_gate"), "w_up": t("w_up"), "w_down": t("w_down"),
    }


class Qwen3Session:
    def __init__(self, cfg: Qwen3Config, resource, *, max_ctx: int = 2176, device="cuda:0",
                 keep_logits: bool = False, trace_hidden: bool = False, pdl: bool = True,
                 l2_prefetch: int = 0, kernel: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("Qwen3Session needs a CUDA device; there is no CPU path")
        lib.load()
        self.cfg, self.device = cfg, torch.device(device)
        self.max_ctx = int(max_ctx)
        dev = self.device
        to = lambda t: t.to(dev)

        root = {n: to(resource.load(n)) for n in ("w_embed", "gamma_final", "w_head")}
        self.w_embed = root["w_embed"].contiguous()
        head = root["w_head"].t().contiguous()
        self.w_head = self.w_embed if torch.equal(head, self.w_embed) else head
        self.gamma_final = root["gamma_final"].contiguous()
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            sub = resource.subtree(f"layer{i}")
            names = ("gamma_in", "w_q", "w_k", "w_v", "gamma_q", "gamma_k", "w_o", "gamma_post",
                     "w_gate", "w_up", "w_down")
            self.layers.append(pack_layer({n: to(sub.load(n)) for n in names}))

        cos, sin = rope_tables(cfg, "cpu")
        self.max_pos = min(cfg.max_position_embeddings, max(self.max_ctx, 1))
        self.cos = cos[: self.max_pos].contiguous().to(dev)
        self.sin = sin[: self.max_pos].contiguous().to(dev)

        HQ, HKV, D, H, I, V = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                               cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size)
        self.table = paged_kv.block_table(1, self.max_ctx, device=dev)
        for layer in self.layers:
            layer["k_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev)
            layer["v_pool"] = paged_kv.new_pool(1, self.max_ctx, HKV, D, device=dev)

        bf, f32 = torch.bfloat16, torch.float32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        nsplit = lib.attn_splits(self.max_ctx)
        self.tokens = z(self.max_ctx + 1, dtype=torch.int64)
        self.pos = z(1, dtype=torch.int32)
        self.hidden = z(H)
        self.qkv = z((HQ + 2 * HKV) * D)
        self.attn = z(HQ * D)
        self.act = z(I)
        self.logits = z(V) if keep_logits else None
        self.part_o = z(HQ * nsplit * D, dtype=f32)
        self.part_ml = z(HQ * nsplit * 2, dtype=f32)
        self.counters = z(HKV + 1, dtype=torch.int32)
        n_head = lib.lm_head_scratch_entries(V)
        self.head_val = z(n_head, dtype=f32)
        self.head_idx = z(n_head, dtype=torch.int32)
        self.trace = z(cfg.num_hidden_layers + 1, H) if trace_hidden else None
        self.picked = z(1, dtype=torch.int64)

        self._layer_structs = (lib.Qwen3Layer * len(self.layers))()
        for s, layer in zip(self._layer_structs, self.layers):
            for name, _ in lib.Qwen3Layer._fields_:
                setattr(s, name, lib.ptr(layer[name]))
        scale = float(torch.tensor(D ** -0.5, dtype=bf))   # the authored step holds it as a bf16 tensor
        self.args = lib.Qwen3StepArgs(
            layers=self._layer_structs, n_layers=len(self.layers), hidden=H, hq=HQ, hkv=HKV, d=D, inter=I,
            vocab=V, eps=cfg.rms_norm_eps, scale=scale,
            w_embed=lib.ptr(self.w_embed), gamma_final=lib.ptr(self.gamma_final), w_head=lib.ptr(self.w_head),
            cos_table=lib.ptr(self.cos), sin_table=lib.ptr(self.sin),
            max_pos=self.max_pos, page_size=paged_kv.PAGE_SIZE, table_len=self.table.shape[1],
            max_ctx=self.max_ctx, block_table=lib.ptr(self.table), tokens=lib.ptr(self.tokens),
            pos=lib.ptr(self.pos), n_prompt=0, max_tokens=self.max_ctx + 1,
            hidden_buf=lib.ptr(self.hidden), qkv_buf=lib.ptr(self.qkv), attn_buf=lib.ptr(self.attn),
            act_buf=lib.ptr(self.act), logits=lib.ptr(self.logits), part_o=lib.ptr(self.part_o),
            part_ml=lib.ptr(self.part_ml), counters=lib.ptr(self.counters), head_val=lib.ptr(self.head_val),
            head_idx=lib.ptr(self.head_idx), hidden_trace=lib.ptr(self.trace),
            pdl=int(pdl), l2_prefetch=int(l2_prefetch), kernel=int(kernel), picked=lib.ptr(self.picked))
        self.graph = None
        self._graph_prompt = None
        #: kernels one step enqueues (embed + 5 per layer + lm_head [+ trace copies and final norm])
        self.launches_per_step = 2 + 5 * len(self.layers) + (
            len(self.layers) + 1 if trace_hidden else 0)

    # weights read once per token, for roofline arithmetic
    def weight_bytes(self) -> int:
        per_layer = sum(self.layers[0][n].numel() * 2 for n in ("w_qkv", "w_o", "w_gate", "w_up", "w_down"))
        return per_layer * len(self.layers) + self.w_head.numel() * 2

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        return 2 * c.num_key_value_heads * c.head_dim * 2 * c.num_hidden_layers

    def reset(self, prompt_ids) -> None:
        """Start a sequence: token history = prompt, position 0.  The cache needs no clearing:
        a step only reads positions below its own."""
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64).reshape(-1)
        if prompt.numel() == 0:
            raise ValueError("decode needs a prompt of at least one token")
        if prompt.numel() > self.max_ctx:
            raise ValueError(f"prompt of {prompt.numel()} tokens exceeds capacity {self.max_ctx}")
        self.tokens.zero_()
        self.tokens[: prompt.numel()] = prompt.to(self.device)
        self.pos.zero_()
        self.counters.zero_()
        if self.args.n_prompt != prompt.numel():
            self.args.n_prompt = int(prompt.numel())
            self.graph = None                         # the prompt length is baked into the capture
        self.n_prompt = int(prompt.numel())

    def step(self) -> None:
        """Enqueue one decode step on the current stream."""
        lib.check(lib.load().tfb_qwen3_decode_step(C.byref(self.args), lib.stream()), "tfb_qwen3_decode_step")

    def capture(self) -> None:
        """Record one step into a CUDA graph (positions and tokens live on the device, so the same
        graph serves every step).  Three eager warm-up steps run first and are rolled back."""
        saved = (self.tokens.clone(), self.pos.clone())
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.tokens.copy_(saved[0]); self.pos.copy_(saved[1])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step()
        torch.cuda.synchronize()
        self.tokens.copy_(saved[0]); self.pos.copy_(saved[1])
        self.graph = graph

    def run(self, steps: int, use_graph: bool = True) -> None:
        if use_graph and self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graph.replay() if use_graph else self.step()

    def generate(self, prompt_ids, max_new: int, use_graph: bool = True) -> Generated:
        """Walk the prompt, then continue greedily for *max_new* tokens; one sync at each end."""
        self.reset(prompt_ids)
        n_prompt = self.n_prompt
        if n_prompt + max_new > self.max_ctx + 1:
            raise ValueError(f"{n_prompt}+{max_new} tokens exceed capacity {self.max_ctx}")
        if use_graph and self.graph is None:
            self.capture()
        start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        start.record()
        self.run(n_prompt - 1, use_graph)          # positions 0 .. n_prompt-2: no sampling needed
        mid.record()
        self.run(max_new, use_graph)               # step at position p writes token p+1
        end.record()
        torch.cuda.synchronize()
        out = self.tokens[n_prompt: n_prompt + max_new].tolist()
        return Generated(out, mid.elapsed_time(end) / 1e3, start.elapsed_time(mid) / 1e3, n_prompt)
