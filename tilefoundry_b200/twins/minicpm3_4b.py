"""Runtime twin of the MiniCPM3-4B Modules (reference ``examples/minicpm3_4b-cutedsl/model.py``):
authored signatures outside, the C-ABI kernels inside; prior assembled cache in, this token's
``(out, k_new, v_new)`` out, nothing mutated."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored import minicpm3_4b as authored
from ..engine import paged_kv
from ..engine.minicpm3 import pack_layer
from ..runtime import runtime_func, runtime_module
from ..runtime.decorator import TwinBase

BF = torch.bfloat16


def _new(shape, like, dtype=BF):
    return torch.empty(shape, device=like.device, dtype=dtype)


def make_twin(cfg: authored.MiniCPM3Config = authored.MINICPM3_4B):
    sem = authored.build(cfg)
    Hd, NH, I, V = cfg.hidden_size, cfg.num_attention_heads, cfg.intermediate_size, cfg.vocab_size
    QK, NOPE, R, VD = cfg.qk_head_dim, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
    QL, KVL, EPS, LEPS = cfg.q_lora_rank, cfg.kv_lora_rank, cfg.rms_norm_eps, cfg.lora_eps
    CAST = lib.NORM_CAST_THEN_GAIN

    @runtime_module(sem.modules[0])
    class Layer:
        def load(self, resource):
            TwinBase.load(self, resource)
            self._packed = pack_layer(self._bound)

        def _attention(self, hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale):
            p = self._packed
            dev = hidden.device
            ctx = k_cache.shape[1]
            cap = ctx + 1
            table = paged_kv.block_table(1, cap, device=dev)
            k_pool = paged_kv.new_pool(1, cap, NH, QK, device=dev)
            v_pool = paged_kv.new_pool(1, cap, NH, VD, device=dev)
            paged_kv.fill_from_logical(k_pool, table[0], k_cache)
            paged_kv.fill_from_logical(v_pool, table[0], v_cache)
            qkv_a = lib.gemv(p["w_qkv_a"], hidden.reshape(-1), _new(QL + KVL + R, hidden), gamma=p["gamma_in"],
                             prologue=CAST, eps=EPS)
            q_up = lib.gemv(p["w_q_b"], qkv_a[:QL], _new(NH * QK, hidden), gamma=p["gamma_q_a"], prologue=CAST, eps=LEPS)
            kv_up = lib.gemv(p["w_kv_b"], qkv_a[QL:QL + KVL], _new(NH * (NOPE + VD), hidden), gamma=p["gamma_kv_a"],
                             prologue=CAST, eps=LEPS)
            nsplit = lib.attn_splits(cap)
            attn = _new(NH * VD, hidden)
            k_new, v_new = _new((1, 1, NH, QK), hidden), _new((1, 1, NH, VD), hidden)
            part_o, part_ml = _new(NH * nsplit * VD, hidden, torch.float32), _new(NH * nsplit * 2, hidden, torch.float32)
            counters = torch.zeros(NH, device=dev, dtype=torch.int32)
            pos = torch.tensor([ctx], device=dev, dtype=torch.int32)
            rope_pos = pos_ids.reshape(-1)[:1].to(torch.int32).contiguous()
            k_rope = qkv_a[QL + KVL:]
            a = lib.AttnMlaArgs(
                q_up=lib.ptr(q_up), kv_up=lib.ptr(kv_up), k_rope=lib.ptr(k_rope), cos_table=lib.ptr(cos_cache),
                sin_table=lib.ptr(sin_cache), pos=lib.ptr(pos), rope_pos=lib.ptr(rope_pos), k_pool=lib.ptr(k_pool),
                v_pool=lib.ptr(v_pool), block_table=lib.ptr(table), out=lib.ptr(attn), k_new_out=lib.ptr(k_new),
                v_new_out=lib.ptr(v_new), part_o=lib.ptr(part_o), part_ml=lib.ptr(part_ml), counters=lib.ptr(counters),
                heads=NH, nope=NOPE, rope=R, v=VD, page_size=paged_kv.PAGE_SIZE, table_len=table.shape[1],
                max_ctx=cap, max_pos=cos_cache.shape[0], scale=float(scale.reshape(-1)[0]), pdl=0)
            lib.check(lib.load().tfb_attn_mla_decode(C.byref(a), lib.stream()), "tfb_attn_mla_decode")
            return attn, k_new, v_new

        def mla_attention_latent(self, hidden, cos_cache, sin_cache, pos_ids, latent_cache, scale):
            """``mla_attention`` over a cache of latents: *latent_cache* is ``[1, C, kv_lora + rope]`` (normalised
            compressed kv vector | rotated shared key per position) instead of the assembled ``k_cache`` /
            ``v_cache``; returns ``(out [1, 1, hidden], latent_new [1, 1, kv_lora + rope])``.  Not an authored
            function (the reference has no latent cache): the decode session's form of it, exposed so a test can hold
            it to ``mla_attention`` on the re-expanded cache."""
            p = self._packed
            dev = hidden.device
            ctx = latent_cache.shape[1]
            cap = ctx + 1
            LAT = KVL + R
            table = paged_kv.block_table(1, cap, device=dev)
            pool = paged_kv.new_pool(1, cap, 1, LAT, device=dev)
            paged_kv.fill_from_logical(pool, table[0], latent_cache.reshape(1, ctx, 1, LAT))
            qkv_a = lib.gemv(p["w_qkv_a"], hidden.reshape(-1), _new(QL + KVL + R, hidden), gamma=p["gamma_in"],
                             prologue=CAST, eps=EPS)
            so = lib.load()
            nsplit = so.tfb_mla_latent_splits(cap)
            f32 = torch.float32
            attn, latent_new = _new(NH * VD, hidden), _new((1, 1, LAT), hidden)
            pos = torch.tensor([ctx], device=dev, dtype=torch.int32)
            rope_pos = pos_ids.reshape(-1)[:1].to(torch.int32).contiguous()
            q_lat, q_rope = _new(NH * 2 * KVL, hidden, f32), _new(NH * R, hidden, f32)
            part_o, part_ml = _new(NH * nsplit * KVL, hidden, f32), _new(NH * nsplit * 2, hidden, f32)
            a = lib.MlaLatentArgs(
                qkv_a=lib.ptr(qkv_a), gamma_q_a=lib.ptr(p["gamma_q_a"]), gamma_kv_a=lib.ptr(p["gamma_kv_a"]),
                w_q_b=lib.ptr(p["w_q_b"]), w_kv_b=lib.ptr(p["w_kv_b"]), cos_table=lib.ptr(cos_cache),
                sin_table=lib.ptr(sin_cache), pos=lib.ptr(pos), rope_pos=lib.ptr(rope_pos), pool=lib.ptr(pool),
                block_table=lib.ptr(table), out=lib.ptr(attn), latent_new_out=lib.ptr(latent_new), q_lat=lib.ptr(q_lat),
                q_rope=lib.ptr(q_rope), part_o=lib.ptr(part_o), part_ml=lib.ptr(part_ml), heads=NH, q_lora=QL,
                kv_lora=KVL, nope=NOPE, rope=R, v=VD, page_size=paged_kv.PAGE_SIZE, table_len=table.shape[1],
                max_ctx=cap, max_pos=cos_cache.shape[0], scale=float(scale.reshape(-1)[0]), lora_eps=LEPS, pdl=0)
            lib.check(so.tfb_mla_latent_decode(C.byref(a), lib.stream()), "tfb_mla_latent_decode")
            return lib.gemv(p["w_o"], attn, _new(Hd, hidden)).reshape(1, 1, Hd), latent_new

        def _mlp(self, hidden, residual=None, res_scale=1.0):
            p = self._packed
            act = lib.gemv(p["w_gate"], hidden.reshape(-1), _new(I, hidden), w2=p["w_up"], gamma=p["gamma_post"],
                           prologue=CAST, epilogue=lib.EPI_SWIGLU, eps=EPS)
            if residual is None:
                return lib.gemv(p["w_down"], act, _new(Hd, hidden)).reshape(1, 1, Hd)
            return lib.gemv(p["w_down"], act, _new(Hd, hidden), residual=residual.reshape(-1),
                            epilogue=lib.EPI_RESIDUAL, res_scale=res_scale).reshape(1, 1, Hd)

        @runtime_func
        def input_rms_norm(self, hidden, gamma_in):
            return lib.rmsnorm(hidden, gamma_in, torch.empty_like(hidden), EPS, CAST)

        @runtime_func
        def mla_attention(self, hidden, gamma_in, w_q_a, gamma_q_a, w_q_b, w_kv_a, gamma_kv_a, w_kv_b, cos_cache,
                          sin_cache, pos_ids, k_cache, v_cache, scale, w_o):
            attn, k_new, v_new = self._attention(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale)
            return lib.gemv(self._packed["w_o"], attn, _new(Hd, hidden)).reshape(1, 1, Hd), k_new, v_new

        @runtime_func
        def mlp(self, hidden, gamma_post, w_gate, w_up, w_down):
            return self._mlp(hidden)

        @runtime_func
        def decoder_layer(self, hidden, gamma_in, w_q_a, gamma_q_a, w_q_b, w_kv_a, gamma_kv_a, w_kv_b, cos_cache,
                          sin_cache, pos_ids, k_cache, v_cache, scale, w_o, gamma_post, w_gate, w_up, w_down,
                          residual_scale):
            rs = float(residual_scale.reshape(-1)[0])
            attn, k_new, v_new = self._attention(hidden, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale)
            h1 = lib.gemv(self._packed["w_o"], attn, _new(Hd, hidden), residual=hidden.reshape(-1),
                          epilogue=lib.EPI_RESIDUAL, res_scale=rs)
            return self._mlp(h1, residual=h1, res_scale=rs), k_new, v_new

    body = {f"layer{i}": Layer for i in range(cfg.num_hidden_layers)}

    def load(self, resource):
        TwinBase.load(self, resource)
        self._head = self._bound["w_head"].t().contiguous()

    @runtime_func
    def embed(self, w_embed, token_ids):
        return lib.embed(w_embed, token_ids.contiguous(), _new((1, 1, Hd), w_embed), scale=cfg.scale_emb)

    @runtime_func
    def final_rms_norm(self, hidden, gamma_final):
        return lib.rmsnorm(hidden, gamma_final, torch.empty_like(hidden), EPS, CAST)

    @runtime_func
    def lm_head(self, hidden, w_head):
        logits = _new((1, V), hidden)
        n = lib.lm_head_scratch_entries(V)
        token = torch.zeros(1, device=hidden.device, dtype=torch.int64)
        val, idx = _new(n, hidden, torch.float32), _new(n, hidden, torch.int32)
        counter = torch.zeros(1, device=hidden.device, dtype=torch.int32)
        a = lib.LmHeadArgs(w=lib.ptr(self._head), x=lib.ptr(hidden.reshape(-1)), logits=lib.ptr(logits),
                           token_out=lib.ptr(token), scratch_val=lib.ptr(val), scratch_idx=lib.ptr(idx),
                           counter=lib.ptr(counter), n=V, k=Hd, prologue=lib.NORM_NONE, eps=EPS,
                           x_scale=-cfg.logits_scaling, out_scale=1.0, pdl=0)
        lib.check(lib.load().tfb_lm_head_argmax(C.byref(a), lib.stream()), "tfb_lm_head_argmax")
        self.last_token = token
        return logits

    body.update(load=load, embed=embed, final_rms_norm=final_rms_norm, lm_head=lm_head)
    return runtime_module(sem)(type("MiniCPM3_4B_Twin", (), body))
