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
import torch

from .. import lib
from ..authored.qwen3_1_7b import Qwen3Config, rope_tables
from . import paged_kv
from .session import DecodeSession, Generated  # noqa: F401

KERNEL_FUSED = 6          # TFB_KERNEL_FUSED: the whole step as one cooperative launch


def fused_step_supported(cfg: Qwen3Config) -> bool:
    """Shapes the one-launch step is built for (the C ABI refuses the others with TFB_EINVAL)."""
    ok_k = lambda k: k >= 1024 and k % 1024 == 0 and k <= 6144
    return (cfg.head_dim == 128 and cfg.num_attention_heads == 2 * cfg.num_key_value_heads
            and ok_k(cfg.hidden_size) and ok_k(cfg.num_attention_heads * cfg.head_dim) and ok_k(cfg.intermediate_size))


def pack_layer(w: dict) -> dict:
    """Authored ``(1, in, out)`` projections -> kernel layout ``[out, in]`` with q|k|v fused."""
    t = lambda name: w[name][0].t().contiguous()
    gate_up = torch.cat([t("w_gate"), t("w_up")], dim=0).contiguous()     # gate rows, then up rows
    inter = gate_up.shape[0] // 2
    return {
        "gamma_in": w["gamma_in"].contiguous(), "gamma_post": w["gamma_post"].contiguous(),
        "gamma_q": w["gamma_q"].contiguous(), "gamma_k": w["gamma_k"].contiguous(),
        "w_qkv": torch.cat([t("w_q"), t("w_k"), t("w_v")], dim=0).contiguous(),
        "w_o": t("w_o"), "w_gate_up": gate_up, "w_gate": gate_up[:inter], "w_up": gate_up[inter:],
        "w_down": t("w_down"),
    }


class Qwen3Session(DecodeSession):
    def __init__(self, cfg: Qwen3Config, resource, *, max_ctx: int = 2176, device="cuda:0",
                 keep_logits: bool = False, trace_hidden: bool = False, pdl: bool = True,
                 l2_prefetch: int = 0, kernel: int | None = None, temperature: float = 0.0, seed: int = 0,
                 top_p: float = 1.0):
        """*kernel*: ``TFB_KERNEL_*`` of the step; ``None`` picks the one-launch step (``KERNEL_FUSED``) where the
        shapes allow it and the pick is greedy, else the step of one launch per kernel (0)."""
        if not torch.cuda.is_available():
            raise RuntimeError("Qwen3Session needs a CUDA device; there is no CPU path")
        lib.load()
        self.cfg, self.device = cfg, torch.device(device)
        self.max_ctx = int(max_ctx)
        dev = self.device
        to = lambda t: t.to(dev)
        if kernel is None:
            kernel = KERNEL_FUSED if fused_step_supported(cfg) else 0

        from .packed import PackedQwen3, pack
        # a resource speaks the authored names and is packed here; a PackedQwen3 (engine/packed.py) is already in
        # the kernels' layout, e.g. read from a file written by save_packed
        packed = (resource if isinstance(resource, PackedQwen3) else pack(cfg, resource)).to(dev)
        self.w_embed = packed.root["w_embed"]
        self.w_head = self.w_embed if packed.root["w_head"] is None else packed.root["w_head"]
        self.gamma_final = packed.root["gamma_final"]
        self.layers = packed.layers

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
        self.fused = int(kernel) == KERNEL_FUSED
        if self.fused:                    # the one-launch step cuts the context into up to (multiprocessors / hkv) splits
            nsplit = max(nsplit, lib.load().tfb_qwen3_step_splits(HKV))
        self.tokens = z(self.max_ctx + 1, dtype=torch.int64)
        self.pos = z(1, dtype=torch.int32)
        self.hidden = z(H)
        self.qkv = z((HQ + 2 * HKV) * D)
        self.attn = z(HQ * D)
        self.act = z(I)
        self.top_p = float(top_p)
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError(f"top_p must be in (0, 1], got {top_p}")
        nucleus = temperature > 0.0 and self.top_p < 1.0        # a second kernel filters the step's own draw
        self.logits = z(V) if keep_logits or nucleus else None
        self.part_o = z(HQ * nsplit * D, dtype=f32)
        self.part_ml = z(HQ * nsplit * 2, dtype=f32)
        self.counters = z(HKV + 1, dtype=torch.int32)
        n_head = max(lib.lm_head_scratch_entries(V), 1024)         # (the one-launch step: one entry per multiprocessor)
        self.head_val = z(n_head, dtype=f32)
        self.head_idx = z(n_head, dtype=torch.int32)
        self.trace = z(cfg.num_hidden_layers + 1, H) if trace_hidden else None
        self.picked = z(1, dtype=torch.int64)

        self._layer_structs = (lib.Qwen3Layer * len(self.layers))()
        for s, layer in zip(self._layer_structs, self.layers):
            for name, _ in lib.Qwen3Layer._fields_:
                setattr(s, name, lib.ptr(layer[name]))
        scale = float(torch.tensor(D ** -0.5, dtype=bf))   # the authored step holds it as a bf16 tensor
        self.chain_sync = torch.zeros(4, device=self.device, dtype=torch.int32)   # grid barrier + status of the chained launch
        # the one-launch step: the layer table on the device (11 pointers per layer, the C struct's field order),
        # its scratch words (merge tickets, launch counter), its tagged activation words and its status word
        self.step_layers = torch.tensor([[layer[name].data_ptr() for name, _ in lib.Qwen3Layer._fields_]
                                         for layer in self.layers], dtype=torch.int64, device=dev)
        self.step_sync = z(max(lib.load().tfb_qwen3_step_sync_words(len(self.layers), HKV), 1), dtype=torch.int32)
        self.step_status = z(1, dtype=torch.int32)
        self.step_xbuf = z(max(int(lib.load().tfb_qwen3_step_xbuf_words(H, HQ, HKV, D, I)), 1), dtype=torch.int32)
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
            pdl=int(pdl), l2_prefetch=int(l2_prefetch), kernel=int(kernel), picked=lib.ptr(self.picked),
            chain_sync=lib.ptr(self.chain_sync), temperature=float(temperature), seed=int(seed) & (2 ** 64 - 1),
            step_layers=lib.ptr(self.step_layers), step_sync=lib.ptr(self.step_sync),
            step_status=lib.ptr(self.step_status), step_xbuf=lib.ptr(self.step_xbuf))
        self.graph = None
        self._graph_prompt = None
        #: kernels one step enqueues (embed + 5 per layer + lm_head [+ trace copies and final norm])
        self.launches_per_step = 1 if self.fused else 2 + 5 * len(self.layers) + (
            len(self.layers) + 1 if trace_hidden else 0)
        self.nucleus = None
        if nucleus:                                   # top-p: tfb_sample_top_p after every step, on the step's own logits
            self.prev_pos = z(1, dtype=torch.int32)
            self.nucleus_hist = z(65664, dtype=torch.int32)
            self.nucleus = lib.SampleTopPArgs(
                logits=lib.ptr(self.logits), pos=lib.ptr(self.pos), prev_pos=lib.ptr(self.prev_pos), tokens=lib.ptr(self.tokens),
                picked=lib.ptr(self.picked), hist=lib.ptr(self.nucleus_hist), vocab=V, n_prompt=0, n_eos=0, pdl=0,
                temperature=float(temperature), top_p=self.top_p, seed=int(seed) & (2 ** 64 - 1))
            self.launches_per_step += 2

    # weights read once per token, for roofline arithmetic
    def weight_bytes(self) -> int:
        per_layer = sum(self.layers[0][n].numel() * 2 for n in ("w_qkv", "w_o", "w_gate", "w_up", "w_down"))
        return per_layer * len(self.layers) + self.w_head.numel() * 2

    def kv_bytes_per_position(self) -> int:
        c = self.cfg
        return 2 * c.num_key_value_heads * c.head_dim * 2 * c.num_hidden_layers

    def step(self) -> None:
        """Enqueue one decode step on the current stream (with ``top_p`` < 1: the step, then the nucleus draw that replaces
        the token it wrote)."""
        if self.nucleus is not None:
            self.prev_pos.copy_(self.pos)
        lib.check(lib.load().tfb_qwen3_decode_step(C.byref(self.args), lib.stream()), "tfb_qwen3_decode_step")
        if self.nucleus is not None:
            self.nucleus.n_prompt = self.args.n_prompt
            lib.check(lib.load().tfb_sample_top_p(C.byref(self.nucleus), lib.stream()), "tfb_sample_top_p")

    def set_eos(self, eos_ids) -> None:
        super().set_eos(eos_ids)
        if self.nucleus is not None:                  # the latch belongs to the kernel that decides the token
            self.nucleus.eos_ids, self.nucleus.n_eos, self.nucleus.stop_at = self.args.eos_ids, self.args.n_eos, self.args.stop_at
            self.args.eos_ids, self.args.n_eos = None, 0      # (the step keeps stop_at: a latched sequence is a no-op)

    def check_status(self) -> None:
        """Raise if a bounded wait of the one-launch step gave up (its results are void then)."""
        code = int(self.step_status)
        if code:
            self.step_status.zero_()
            self.step_sync.zero_()
            self.step_xbuf.zero_()                       # the launch counter restarts: no stale tag may match
            raise RuntimeError(f"tfb_qwen3_decode_step (one launch): a bounded wait gave up (status {code:#x})")

    def prefill(self, n_tokens: int) -> None:
        """Process positions ``pos .. pos + n_tokens - 1`` of the token history in chunks of up to 32 tokens
        (tensor-core projections, chunked attention) instead of one decode step each, and advance the position.
        Nothing is picked: use it for prompt tokens whose successor is already known."""
        from .qwen3_prefill import Qwen3Prefill
        if getattr(self, "_prefill", None) is None:
            self._prefill = Qwen3Prefill(self)
        self._prefill.run(n_tokens)

    def generate(self, prompt_ids, max_new: int, use_graph: bool = True, prefill: bool = False, eos=None):
        """As DecodeSession.generate; with ``prefill`` the prompt (all but its last token) is processed in chunks."""
        if not prefill:
            return super().generate(prompt_ids, max_new, use_graph, eos)
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
