"""Runtime twin of the Qwen3-1.7B Modules: authored signatures, CUDA kernels inside.

Every ``@runtime_func`` keeps the authored contract (reference
``tests/models/qwen3_1_7b/model.py``): prior cache ``[1, C, hkv, d]`` in, this
token's ``(out, k_new, v_new)`` out, nothing mutated, so ``runtime.check`` can put
it beside the evaluator.  Inside, a call stages the prior cache into a scratch
paged pool and runs the same kernels the session runs.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored import qwen3_1_7b as authored
from ..engine import paged_kv
from ..engine.qwen3 import pack_layer
from ..runtime import runtime_func, runtime_module
from ..runtime.decorator import TwinBase

BF = torch.bfloat16


def _new(shape, like, dtype=BF):
    return torch.empty(shape, device=like.device, dtype=dtype)


def make_twin(cfg: authored.Qwen3Config = authored.QWEN3_1_7B):
    """-> the root twin class for *cfg* (children ``layer0..``)."""
    sem = authored.build(cfg)
    layer_sem = sem.modules[0]
    H, D, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
    HQ, HKV, EPS = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.rms_norm_eps

    @runtime_module(layer_sem)
    class Layer:
        def load(self, resource):
            TwinBase.load(self, resource)
            self._packed = pack_layer(self._bound)

        def _attention(self, hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale):
            p = self._packed
            ctx = k_cache.shape[1]
            cap = ctx + 1
            table = paged_kv.block_table(1, cap, device=hidden.device)
            k_pool = paged_kv.new_pool(1, cap, HKV, D, device=hidden.device)
            v_pool = paged_kv.new_pool(1, cap, HKV, D, device=hidden.device)
            paged_kv.fill_from_logical(k_pool, table[0], k_cache)
            paged_kv.fill_from_logical(v_pool, table[0], v_cache)
            qkv = _new((HQ + 2 * HKV) * D, hidden)
            lib.gemv(p["w_qkv"], hidden.reshape(-1), qkv, gamma=p["gamma_in"],
                     prologue=lib.NORM_CAST_THEN_GAIN, eps=EPS)
            nsplit = lib.attn_splits(cap)
            attn, k_new, v_new = _new(HQ * D, hidden), _new((1, 1, HKV, D), hidden), _new((1, 1, HKV, D), hidden)
            part_o = _new(HQ * nsplit * D, hidden, torch.float32)
            part_ml = _new(HQ * nsplit * 2, hidden, torch.float32)
            counters = torch.zeros(HKV, device=hidden.device, dtype=torch.int32)
            # the rope tables are gathered at pos_ids; the cache position is the context length
            pos = torch.tensor([ctx], device=hidden.device, dtype=torch.int32)
            rope_pos = pos_ids.reshape(-1)[:1].to(torch.int32).contiguous()
            a = lib.AttnGqaArgs(
                qkv=lib.ptr(qkv), gamma_q=lib.ptr(p["gamma_q"]), gamma_k=lib.ptr(p["gamma_k"]),
                cos_table=lib.ptr(cos_cache), sin_table=lib.ptr(sin_cache),
                pos=lib.ptr(pos), rope_pos=lib.ptr(rope_pos), k_pool=lib.ptr(k_pool), v_pool=lib.ptr(v_pool),
                block_table=lib.ptr(table), out=lib.ptr(attn), k_new_out=lib.ptr(k_new), v_new_out=lib.ptr(v_new),
                part_o=lib.ptr(part_o), part_ml=lib.ptr(part_ml), counters=lib.ptr(counters),
                hq=HQ, hkv=HKV, d=D, rotary_dim=D, page_size=paged_kv.PAGE_SIZE, table_len=table.shape[1],
                max_ctx=cap, max_pos=cos_cache.shape[0], eps=EPS, scale=float(scale.reshape(-1)[0]),
                norm_mode=lib.NORM_CAST_THEN_GAIN, pdl=0)
            lib.check(lib.load().tfb_attn_gqa_decode(C.byref(a), lib.stream()), "tfb_attn_gqa_decode")
            return attn, k_new, v_new

        @runtime_func
        def input_rms_norm(self, hidden, gamma_in):
            return lib.rmsnorm(hidden, gamma_in, torch.empty_like(hidden), EPS, lib.NORM_CAST_THEN_GAIN)

        @runtime_func
        def self_attention(self, hidden, gamma_in, w_q, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache,
                           pos_ids, k_cache, v_cache, scale, w_o):
            attn, k_new, v_new = self._attention(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale)
            out = lib.gemv(self._packed["w_o"], attn, _new(H, hidden))
            return out.reshape(1, 1, H), k_new, v_new

        def _mlp(self, hidden, residual=None):
            p = self._packed
            act = lib.gemv(p["w_gate"], hidden.reshape(-1), _new(I, hidden), w2=p["w_up"], gamma=p["gamma_post"],
                           prologue=lib.NORM_CAST_THEN_GAIN, epilogue=lib.EPI_SWIGLU, eps=EPS)
            if residual is None:
                return lib.gemv(p["w_down"], act, _new(H, hidden)).reshape(1, 1, H)
            return lib.gemv(p["w_down"], act, _new(H, hidden), residual=residual.reshape(-1),
                            epilogue=lib.EPI_RESIDUAL).reshape(1, 1, H)

        @runtime_func
        def mlp(self, hidden, gamma_post, w_gate, w_up, w_down):
            return self._mlp(hidden)

        @runtime_func
        def placed_mlp(self, hidden, gamma_post, w_gate, w_up, w_down):
            return self._mlp(hidden)

        @runtime_func
        def decoder_layer(self, hidden, gamma_in, w_q, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache,
                          pos_ids, k_cache, v_cache, scale, w_o, gamma_post, w_gate, w_up, w_down):
            attn, k_new, v_new = self._attention(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale)
            h1 = lib.gemv(self._packed["w_o"], attn, _new(H, hidden), residual=hidden.reshape(-1),
                          epilogue=lib.EPI_RESIDUAL)
            return self._mlp(h1, residual=h1), k_new, v_new

    body = {f"layer{i}": Layer for i in range(cfg.num_hidden_layers)}

    def load(self, resource):
        TwinBase.load(self, resource)
        self._head = self._bound["w_head"].t().contiguous()

    @runtime_func
    def embed(self, w_embed, token_ids):
        return lib.embed(w_embed, token_ids.contiguous(), _new((1, 1, H), w_embed))

    @runtime_func
    def final_rms_norm(self, hidden, gamma_final):
        return lib.rmsnorm(hidden, gamma_final, torch.empty_like(hidden), EPS, lib.NORM_CAST_THEN_GAIN)

    @runtime_func
    def lm_head(self, hidden, w_head):
        logits = _new((1, V), hidden)
        n = lib.lm_head_scratch_entries(V)
        token = torch.zeros(1, device=hidden.device, dtype=torch.int64)
        # scratch must stay referenced until the launch is enqueued: two unnamed temporaries
        # would be handed the same block by the caching allocator
        val, idx = _new(n, hidden, torch.float32), _new(n, hidden, torch.int32)
        counter = torch.zeros(1, device=hidden.device, dtype=torch.int32)
        a = lib.LmHeadArgs(w=lib.ptr(self._head), x=lib.ptr(hidden.reshape(-1)), logits=lib.ptr(logits),
                           token_out=lib.ptr(token), scratch_val=lib.ptr(val), scratch_idx=lib.ptr(idx),
                           counter=lib.ptr(counter),
                           n=V, k=H, prologue=lib.NORM_NONE, eps=EPS, x_scale=1.0, out_scale=1.0, pdl=0)
        lib.check(lib.load().tfb_lm_head_argmax(C.byref(a), lib.stream()), "tfb_lm_head_argmax")
        self.last_token = token
        return logits

    body.update(load=load, embed=embed, final_rms_norm=final_rms_norm, lm_head=lm_head)
    return runtime_module(sem)(type("Qwen3_1_7B_Twin", (), body))
