"""Chunked prompt processing for a MiniCPM3 decode session (latent cache).

The reference walks a prompt one token at a time (``tests/models/orchestrator/causal_lm/generation.py:56-61``).
Here up to 32 consecutive prompt tokens go through the layer stack together: every projection streams its weights
once per chunk on the tensor cores; the chunk's attention is one launch of each latent-attention kernel with the
token as a grid axis (every token appends its latent row, then each attends to the rows up to its own).  The cache rows and the position the
session ends with are those of the token-by-token walk.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from . import paged_kv

CHUNK = 32


class MiniCPM3Prefill:
    def __init__(self, sess):
        cfg, dev = sess.cfg, sess.device
        self.sess = sess
        H, I, NH, VD = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.v_head_dim
        NA = cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_head_dim
        bf, i32 = torch.bfloat16, torch.int32
        z = lambda *s, dtype=bf: torch.zeros(*s, device=dev, dtype=dtype)
        self.hidden, self.norm = z(CHUNK, H), z(CHUNK, H)
        self.qkv_a, self.attn, self.act = z(CHUNK, NA), z(CHUNK, NH * VD), z(CHUNK, I)
        self.status = z(1, dtype=i32)
        self.pos_rows = z(CHUNK, dtype=i32)
        f32 = torch.float32
        nsplit = lib.load().tfb_mla_latent_splits(sess.max_ctx)
        KVL, R = cfg.kv_lora_rank, cfg.qk_rope_head_dim
        # the chunk's tokens attend in ONE launch of each latent-attention kernel: scratch per token
        self.q_lat, self.q_rope = z(CHUNK, NH * 2 * KVL, dtype=f32), z(CHUNK, NH * R, dtype=f32)
        self.part_o, self.part_ml = z(CHUNK, NH * nsplit * KVL, dtype=f32), z(CHUNK, NH * nsplit * 2, dtype=f32)
        a = sess.args
        self.args = lib.MiniCPM3PrefillArgs(
            layers=sess._layer_structs, n_layers=len(sess.layers), m=CHUNK, hidden=H, heads=NH, q_lora=cfg.q_lora_rank,
            kv_lora=cfg.kv_lora_rank, nope=cfg.qk_nope_head_dim, rope=cfg.qk_rope_head_dim, v=VD, inter=I,
            vocab=cfg.vocab_size, eps=a.eps, lora_eps=a.lora_eps, scale=a.scale, embed_scale=a.embed_scale,
            residual_scale=a.residual_scale, pdl=a.pdl, w_embed=lib.ptr(sess.w_embed), cos_table=lib.ptr(sess.cos),
            sin_table=lib.ptr(sess.sin), max_pos=sess.max_pos, page_size=paged_kv.PAGE_SIZE,
            table_len=sess.table.shape[1], max_ctx=sess.max_ctx, block_table=lib.ptr(sess.table), ids=None,
            pos_rows=lib.ptr(self.pos_rows), hidden_buf=lib.ptr(self.hidden), norm_buf=lib.ptr(self.norm),
            qkv_a_buf=lib.ptr(self.qkv_a), attn_buf=lib.ptr(self.attn), act_buf=lib.ptr(self.act),
            q_lat_buf=lib.ptr(self.q_lat), q_rope_buf=lib.ptr(self.q_rope), part_o=lib.ptr(self.part_o),
            part_ml=lib.ptr(self.part_ml), status=lib.ptr(self.status))

    def launches(self, m: int) -> int:
        """Kernels one chunk enqueues: embed + per layer 2 norms, 4 projections, 3 of the latent attention."""
        return 1 + 9 * len(self.sess.layers)

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
            lib.check(lib.load().tfb_minicpm3_prefill_chunk(C.byref(self.args), lib.stream()), "tfb_minicpm3_prefill_chunk")
            done += m
        sess.pos.fill_(first + done)
        for _ in range(n_tokens - done):                 # a lone leftover token takes the ordinary step
            sess.step()

    def check_status(self) -> None:
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"tfb_gemm_small_m: a bounded wait gave up (status {code})")
