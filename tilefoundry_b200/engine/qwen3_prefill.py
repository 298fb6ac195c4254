"""Chunked prompt processing for a Qwen3 decode session.

The reference walks a prompt one token at a time (``tests/models/orchestrator/causal_lm/generation.py:56-61``).
Here up to 32 consecutive prompt tokens go through the layer stack together: every projection streams its weights
once per chunk on the tensor cores, and attention runs in its chunk form (each token attends to the cached rows
before it).  The cache rows and the position the session ends with are those of the token-by-token walk.
"""
from __future__ import annotations

import ctypes as C
import torch

from .. import lib
from . import paged_kv

CHUNK = 32


class Qwen3Prefill:
    def __init__(self, sess):
        cfg, dev = sess.cfg, sess.device
        self.sess = sess
        HQ, HKV, D, H, I = (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.hidden_size,
                            cfg.intermediate_size)
        bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        nsplit = lib.attn_splits(sess.max_ctx)
        self.hidden, self.norm = z(CHUNK, H), z(CHUNK, H)
        self.qkv, self.attn, self.act = z(CHUNK, (HQ + 2 * HKV) * D), z(CHUNK, HQ * D), z(CHUNK, I)
        self.part_o = z(CHUNK * HQ * nsplit * D, dtype=f32)
        self.part_ml = z(CHUNK * HQ * nsplit * 2, dtype=f32)
        self.counters = z(CHUNK * HKV, dtype=i32)
        self.status = z(1, dtype=i32)
        self.pos_rows = z(CHUNK, dtype=i32)
        self._layers = (lib.Qwen3BatchLayer * len(sess.layers))()
        for s, layer in zip(self._layers, sess.layers):
            for name, _ in lib.Qwen3BatchLayer._fields_:
                setattr(s, name, lib.ptr(layer[name]))
        a = sess.args
        self.args = lib.Qwen3PrefillArgs(
            layers=self._layers, n_layers=len(sess.layers), m=CHUNK, hidden=H, hq=HQ, hkv=HKV, d=D, inter=I,
            pdl=a.pdl, eps=a.eps, scale=a.scale, vocab=cfg.vocab_size, w_embed=lib.ptr(sess.w_embed),
            cos_table=lib.ptr(sess.cos), sin_table=lib.ptr(sess.sin), max_pos=sess.max_pos,
            page_size=paged_kv.PAGE_SIZE, table_len=sess.table.shape[1], max_ctx=sess.max_ctx,
            block_table=lib.ptr(sess.table), ids=None, pos_rows=lib.ptr(self.pos_rows),
            hidden_buf=lib.ptr(self.hidden), norm_buf=lib.ptr(self.norm), qkv_buf=lib.ptr(self.qkv),
            attn_buf=lib.ptr(self.attn), act_buf=lib.ptr(self.act), part_o=lib.ptr(self.part_o),
            part_ml=lib.ptr(self.part_ml), counters=lib.ptr(self.counters), status=lib.ptr(self.status))
        #: kernels one chunk enqueues (embed + 8 per layer)
        self.launches_per_chunk = 1 + 8 * len(sess.layers)

    def run(self, n_tokens: int) -> None:
        """Positions ``pos .. pos + n_tokens - 1`` of the session's token history; one host read of the position."""
        sess = self.sess
        first = int(sess.pos.item())
        if n_tokens < 0 or first + n_tokens > sess.max_ctx:
            raise ValueError(f"{first}+{n_tokens} tokens exceed capacity {sess.max_ctx}")
        done = 0
        while n_tokens - done >= 2:
            m = min(CHUNK, n_tokens - done)
            if n_tokens - done - m == 1:                 # never leave a single token: a chunk holds at least two
                m -= 1
            start = first + done
            self.pos_rows[:m] = torch.arange(start, start + m, device=sess.device, dtype=torch.int32)
            self.args.m = m
            self.args.ids = sess.tokens.data_ptr() + 8 * start
            lib.check(lib.load().tfb_qwen3_prefill_chunk(C.byref(self.args), lib.stream()), "tfb_qwen3_prefill_chunk")
            done += m
        sess.pos.fill_(first + done)
        for _ in range(n_tokens - done):                 # a lone leftover token takes the ordinary step
            sess.step()

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"tfb_gemm_small_m: a bounded wait gave up (status {code})")
