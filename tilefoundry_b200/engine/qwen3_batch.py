"""Qwen3-architecture decode session for several sequences at once (batch <= 32).

The reference's fast driver decodes one sequence (``examples/qwen3_1_7b-tilelang/fast/engine.py:189-271``);
at batch 32 the same weights are streamed once per step for 32 tokens, so every projection becomes a
128 x 32 tensor-core tile product (``tfb_gemm_small_m``) and the KV cache, read once per sequence, becomes the
larger half of a step's bytes.  Each sequence has its own pages in the shared pools (page ``i`` of sequence ``b``
is pool page ``b * pages_per_seq + i``), its own token history row and position word, all on the device, so one
captured step serves every position.
"""
from __future__ import annotations

import ctypes as C
import torch

from .. import lib
from ..authored.qwen3_1_7b import Qwen3Config, rope_tables
from . import paged_kv
from .qwen3 import pack_layer
from .session import Generated

MAX_BATCH = 32


class Qwen3BatchSession:
    def __init__(self, cfg: Qwen3Config, resource, *, batch: int, max_ctx: int = 2176, device="cuda:0",
                 trace_hidden: bool = False, pdl: bool = True, temperature: float = 0.0, seed: int = 0):
        if not torch.cuda.is_available():
            raise RuntimeError("Qwen3BatchSession needs a CUDA device; there is no CPU path")
        if not 1 <= batch <= MAX_BATCH:
            raise ValueError(f"batch must be 1..{MAX_BATCH}, got {batch}")
        lib.load()
        self.cfg, self.device, self.batch = cfg, torch.device(device), int(batch)
        self.max_ctx = int(max_ctx)
        dev, B = self.device, self.batch
        to = lambda t: t.to(dev)

        from .packed import PackedQwen3, pack
        packed = (resource if isinstance(resource, PackedQwen3) else pack(cfg, resource)).to(dev)
        self.w_embed = packed.root["w_embed"]
        self.w_head = self.w_embed if packed.root["w_head"] is None else packed.root["w_head"]
        self.gamma_final = packed.root["gamma_final"]
        self.layers = packed.layers                       # w_gate / w_up are views of w_gate_up, read whole here

        cos, sin = rope_tables(cfg, "cpu")
        self.max_pos = min(cfg.max_position_embeddings, max(self.max_ctx, 1))
        self.cos = cos[: self.max_pos].contiguous().to(dev)
        self.sin = sin[: self.max_pos].contiguous().to(dev)

        HQ, HKV, D, H, I, V = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                               cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size)
        self.table = paged_kv.block_table(B, self.max_ctx, device=dev)
        for layer in self.layers:
            layer["k_pool"] = paged_kv.new_pool(B, self.max_ctx, HKV, D, device=dev)
            layer["v_pool"] = paged_kv.new_pool(B, self.max_ctx, HKV, D, device=dev)

        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        nsplit = lib.attn_splits(self.max_ctx)
        self.max_tokens = self.max_ctx + 1
        self.tokens = z(B, self.max_tokens, dtype=torch.int64)
        self.pos = z(B, dtype=i32)
        self.hidden = z(B, H)
        self.norm = z(B, H)
        self.qkv = z(B, (HQ + 2 * HKV) * D)
        self.attn = z(B, HQ * D)
        self.act = z(B, I)
        self.logits = z(B, V)
        self.part_o = z(B * HQ * nsplit * D, dtype=f32)
        self.part_ml = z(B * HQ * nsplit * 2, dtype=f32)
        self.counters = z(B * HKV + B, dtype=i32)
        self.status = z(1, dtype=i32)
        self.pick_val = z(B * 8, dtype=f32)
        self.pick_idx = z(B * 8, dtype=i32)
        self.picked = z(B, dtype=torch.int64)
        self.trace = z(cfg.num_hidden_layers + 1, B, H) if trace_hidden else None

        self._layer_structs = (lib.Qwen3BatchLayer * len(self.layers))()
        for s, layer in zip(self._layer_structs, self.layers):
            for name, _ in lib.Qwen3BatchLayer._fields_:
                setattr(s, name, lib.ptr(layer[name]))
        scale = float(torch.tensor(D ** -0.5, dtype=bf))   # the authored step holds it as a bf16 tensor
        self.args = lib.Qwen3BatchStepArgs(
            layers=self._layer_structs, n_layers=len(self.layers), batch=B, hidden=H, hq=HQ, hkv=HKV, d=D, inter=I,
            pdl=int(pdl), vocab=V, eps=cfg.rms_norm_eps, scale=scale,
            w_embed=lib.ptr(self.w_embed), gamma_final=lib.ptr(self.gamma_final), w_head=lib.ptr(self.w_head),
            cos_table=lib.ptr(self.cos), sin_table=lib.ptr(self.sin),
            max_pos=self.max_pos, page_size=paged_kv.PAGE_SIZE, table_len=self.table.shape[1],
            max_ctx=self.max_ctx, block_table=lib.ptr(self.table), tokens=lib.ptr(self.tokens),
            pos=lib.ptr(self.pos), n_prompt=0, max_tokens=self.max_tokens,
            hidden_buf=lib.ptr(self.hidden), norm_buf=lib.ptr(self.norm), qkv_buf=lib.ptr(self.qkv),
            attn_buf=lib.ptr(self.attn), act_buf=lib.ptr(self.act), logits=lib.ptr(self.logits),
            part_o=lib.ptr(self.part_o), part_ml=lib.ptr(self.part_ml), counters=lib.ptr(self.counters),
            status=lib.ptr(self.status), pick_val=lib.ptr(self.pick_val), pick_idx=lib.ptr(self.pick_idx),
            picked=lib.ptr(self.picked), hidden_trace=lib.ptr(self.trace),
            temperature=float(temperature), seed=int(seed) & (2 ** 64 - 1))
        self.graph = None
        self.n_prompt = 0
        #: kernels one step enqueues (embed + 7 per layer + final norm + head + pick [+ trace copies])
        self.launches_per_step = 4 + 7 * len(self.layers) + (len(self.layers) + 1 if trace_hidden else 0)

    # bytes one step must move, for roofline arithmetic
    def weight_bytes(self) -> int:
        per_layer = sum(self.layers[0][n].numel() * 2 for n in ("w_qkv", "w_o", "w_gate_up", "w_down"))
        return per_layer * len(self.layers) + self.w_head.numel() * 2

    def kv_bytes_per_position(self) -> int:
        """Per sequence and cached position, all layers."""
        c = self.cfg
        return 2 * c.num_key_value_heads * c.head_dim * 2 * c.num_hidden_layers

    def step(self) -> None:
        """Enqueue one decode step (one token for every sequence) on the current stream."""
        lib.check(lib.load().tfb_qwen3_batch_decode_step(C.byref(self.args), lib.stream()),
                  "tfb_qwen3_batch_decode_step")

    def reset(self, prompts) -> None:
        """Start ``batch`` sequences: *prompts* is ``[batch, n_prompt]`` token ids (equal lengths)."""
        prompts = torch.as_tensor(prompts, dtype=torch.int64)
        if prompts.dim() != 2 or prompts.shape[0] != self.batch or prompts.shape[1] == 0:
            raise ValueError(f"prompts must be [{self.batch}, n >= 1], got {tuple(prompts.shape)}")
        if prompts.shape[1] > self.max_ctx:
            raise ValueError(f"prompt of {prompts.shape[1]} tokens exceeds capacity {self.max_ctx}")
        self.tokens.zero_()
        self.tokens[:, : prompts.shape[1]] = prompts.to(self.device)
        self.pos.zero_()
        self.counters.zero_()
        self.status.zero_()
        if self.args.n_prompt != prompts.shape[1]:
            self.args.n_prompt = int(prompts.shape[1])
            self.graph = None                         # the prompt length is baked into the capture
        self.n_prompt = int(prompts.shape[1])

    def check_status(self) -> None:
        """Raise if a bounded wait inside a tensor-core projection gave up (outputs would be invalid)."""
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"tfb_gemm_small_m: a bounded wait gave up (status {code})")

    def capture(self) -> None:
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
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self.step()
        torch.cuda.synchronize()
        self.tokens.copy_(saved[0]); self.pos.copy_(saved[1])
        self.graph = graph

    def run(self, steps: int, use_graph: bool = True) -> None:
        if use_graph and self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graph.replay() if use_graph else self.step()

    def generate(self, prompts, max_new: int, use_graph: bool = True) -> Generated:
        """Walk the prompts, then continue greedily for *max_new* tokens per sequence; one sync at each end.
        ``Generated.tokens`` is ``[batch][max_new]``; ``tokens_per_second`` counts all sequences."""
        self.reset(prompts)
        n_prompt = self.n_prompt
        if n_prompt + max_new > self.max_tokens:
            raise ValueError(f"{n_prompt}+{max_new} tokens exceed capacity {self.max_ctx}")
        if use_graph and self.graph is None:
            self.capture()
        start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        start.record()
        self.run(n_prompt - 1, use_graph)
        mid.record()
        self.run(max_new, use_graph)
        end.record()
        torch.cuda.synchronize()
        self.check_status()
        out = self.tokens[:, n_prompt: n_prompt + max_new].tolist()
        return BatchGenerated(out, mid.elapsed_time(end) / 1e3, start.elapsed_time(mid) / 1e3, n_prompt)


class BatchGenerated(Generated):
    @property
    def tokens_per_second(self) -> float:
        return sum(len(t) for t in self.tokens) / self.seconds
