"""TEST INFRASTRUCTURE.  MiniCPM3-4B ``@func`` bodies restated op by op.

Follows reference ``examples/minicpm3_4b-cutedsl/model.py`` line by line (``mla_attention``
``:206-292``, ``mlp`` ``:294-310``, ``decoder_layer`` ``:312-345``, root functions ``:359-394``).
"""
from __future__ import annotations

import torch

from . import ops as tf


def make(cfg):
    EPS, LORA_EPS = cfg.rms_norm_eps, cfg.lora_eps
    NH, QK, NOPE, R, VD = (cfg.num_attention_heads, cfg.qk_head_dim, cfg.qk_nope_head_dim,
                           cfg.qk_rope_head_dim, cfg.v_head_dim)
    Hd, DT, KVL = cfg.hidden_size, cfg.dtype, cfg.kv_lora_rank
    PAIR = NOPE + VD

    def norm(x, gamma, eps):                 # MiniCPMRMSNorm written out: cast, then gain
        x32 = tf.cast(x, "f32")
        var = tf.reduce(x32 * x32, axes=(-1,), keepdim=True, kind="mean")
        return tf.cast(x32 * tf.rsqrt(var + eps), DT) * gamma

    def input_rms_norm(hidden, gamma_in):
        return norm(hidden, gamma_in, EPS)

    def mla_attention(hidden, gamma_in, w_q_a, gamma_q_a, w_q_b, w_kv_a, gamma_kv_a, w_kv_b, cos_cache,
                      sin_cache, pos_ids, k_cache, v_cache, scale, w_o):
        C = k_cache.shape[1]
        x = input_rms_norm(hidden, gamma_in)
        q_n = norm(tf.matmul(x, w_q_a), gamma_q_a, LORA_EPS)
        q = tf.matmul(q_n, w_q_b).reshape(1, 1, NH, QK)
        q_nope, q_rope = q[:, :, :, :NOPE], q[:, :, :, NOPE:QK]
        compressed = tf.matmul(x, w_kv_a)
        kv_c, k_rope_flat = compressed[:, :, :KVL], compressed[:, :, KVL:KVL + R]
        kv_n = norm(kv_c, gamma_kv_a, LORA_EPS)
        kv = tf.matmul(kv_n, w_kv_b).reshape(1, 1, NH, PAIR)
        k_nope, v_new = kv[:, :, :, :NOPE], kv[:, :, :, NOPE:PAIR]
        k_rope = k_rope_flat.reshape(1, 1, 1, R)
        q_rope_e, k_rope_e = tf.rope(q_rope, k_rope, cos_cache, sin_cache, pos_ids)
        k_rope_b = tf.repeat_interleave(k_rope_e, NH, 2)
        query = torch.cat((q_nope, q_rope_e), dim=-1)
        k_new = torch.cat((k_nope, k_rope_b), dim=-1)

        q_s = query * scale
        k_ctx = k_cache.permute(0, 2, 1, 3).reshape(1, 1, NH, C, QK)
        v_ctx = v_cache.permute(0, 2, 1, 3).reshape(1, 1, NH, C, VD)
        q_e = q_s.reshape(1, 1, NH, 1, QK)
        score_ctx = tf.reduce(q_e * k_ctx, axes=(-1,), keepdim=True, kind="sum")
        score_new = tf.reduce(q_s * k_new, axes=(-1,), keepdim=True, kind="sum")
        peak = tf.maximum(tf.reduce(score_ctx, axes=(-2,), keepdim=False, kind="max"), score_new)
        p_ctx = tf.exp(score_ctx - peak.reshape(1, 1, NH, 1, 1))
        p_new = tf.exp(score_new - peak)
        total = tf.reduce(p_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new
        weighted = tf.reduce(p_ctx * v_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new * v_new
        attn = weighted / total
        out = tf.matmul(attn.reshape(1, 1, NH * VD), w_o)
        return out, k_new.contiguous(), v_new.contiguous()

    def mlp(hidden, gamma_post, w_gate, w_up, w_down):
        hn = norm(hidden, gamma_post, EPS)
        return tf.matmul(tf.silu(tf.matmul(hn, w_gate)) * tf.matmul(hn, w_up), w_down)

    def decoder_layer(hidden, gamma_in, w_q_a, gamma_q_a, w_q_b, w_kv_a, gamma_kv_a, w_kv_b, cos_cache,
                      sin_cache, pos_ids, k_cache, v_cache, scale, w_o, gamma_post, w_gate, w_up, w_down,
                      residual_scale):
        attn_out, k_new, v_new = mla_attention(hidden, gamma_in, w_q_a, gamma_q_a, w_q_b, w_kv_a, gamma_kv_a,
                                               w_kv_b, cos_cache, sin_cache, pos_ids, k_cache, v_cache, scale, w_o)
        h1 = hidden + attn_out * residual_scale
        return h1 + mlp(h1, gamma_post, w_gate, w_up, w_down) * residual_scale, k_new, v_new

    def embed(w_embed, token_ids):
        return tf.index_select(w_embed, token_ids, 0).reshape(1, 1, Hd) * cfg.scale_emb

    def final_rms_norm(hidden, gamma_final):
        return norm(hidden, gamma_final, EPS)

    def lm_head(hidden, w_head):
        return tf.matmul(hidden.reshape(1, Hd) / cfg.logits_scaling, w_head)

    layer_impl = {"input_rms_norm": input_rms_norm, "mla_attention": mla_attention, "mlp": mlp,
                  "decoder_layer": decoder_layer}
    root_impl = {"embed": embed, "final_rms_norm": final_rms_norm, "lm_head": lm_head}
    return lambda module: root_impl if module.modules else layer_impl
