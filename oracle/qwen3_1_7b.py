"""TEST INFRASTRUCTURE.  Qwen3-1.7B ``@func`` bodies restated op by op.

Follows reference ``tests/models/qwen3_1_7b/model.py`` line by line; every
intermediate is rounded where the evaluator rounds it (after each op, at the
operand dtype).
"""
from __future__ import annotations

from . import ops as tf


def make(cfg):
    """-> ``impl_for(module)`` for a ``Qwen3Config``."""
    EPS = cfg.rms_norm_eps
    HQ, HKV, D, G = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.gqa
    H, QP = cfg.hidden_size, cfg.q_proj
    DT = cfg.dtype

    def qwen_norm(x, gamma):              # the spelled-out Qwen3RMSNorm, model.py:135-138
        x32 = tf.cast(x, "f32")
        var = tf.reduce(x32 * x32, axes=(-1,), keepdim=True, kind="mean")
        return tf.cast(x32 * tf.rsqrt(var + EPS), DT) * gamma

    def input_rms_norm(hidden, gamma_in):                         # model.py:127-138
        return qwen_norm(hidden, gamma_in)

    def self_attention(hidden, gamma_in, w_q, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache,
                       pos_ids, k_cache, v_cache, scale, w_o):    # model.py:141-217
        C = k_cache.shape[1]
        hn = input_rms_norm(hidden, gamma_in)
        q = tf.matmul(hn, w_q).reshape(1, 1, HQ, D)
        k = tf.matmul(hn, w_k).reshape(1, 1, HKV, D)
        v = tf.matmul(hn, w_v).reshape(1, 1, HKV, D)
        q_n = qwen_norm(q, gamma_q)
        q_rope, _ = tf.rope(q_n, q_n, cos_cache, sin_cache, pos_ids)
        k_n = qwen_norm(k, gamma_k)
        _, k_rope = tf.rope(k_n, k_n, cos_cache, sin_cache, pos_ids)

        q_s = q_rope.reshape(1, 1, HQ, D) * scale
        k_ctx = tf.repeat_interleave(k_cache, G, 2).permute(0, 2, 1, 3).reshape(1, 1, HQ, C, D)
        v_ctx = tf.repeat_interleave(v_cache, G, 2).permute(0, 2, 1, 3).reshape(1, 1, HQ, C, D)
        k_new = tf.repeat_interleave(k_rope, G, 2)
        v_new = tf.repeat_interleave(v, G, 2)

        q_e = q_s.reshape(1, 1, HQ, 1, D)
        score_ctx = tf.reduce(q_e * k_ctx, axes=(-1,), keepdim=True, kind="sum")
        score_new = tf.reduce(q_s * k_new, axes=(-1,), keepdim=True, kind="sum")

        peak = tf.maximum(tf.reduce(score_ctx, axes=(-2,), keepdim=False, kind="max"), score_new)
        peak_e = peak.reshape(1, 1, HQ, 1, 1)
        p_ctx = tf.exp(score_ctx - peak_e)
        p_new = tf.exp(score_new - peak)
        total = tf.reduce(p_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new
        weighted = tf.reduce(p_ctx * v_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new * v_new
        attn = weighted / total
        out = tf.matmul(attn.reshape(1, 1, QP), w_o)
        return out, k_rope, v

    def mlp(hidden, gamma_post, w_gate, w_up, w_down):            # model.py:220-235
        hn = qwen_norm(hidden, gamma_post)
        gate = tf.matmul(hn, w_gate)
        up = tf.matmul(hn, w_up)
        return tf.matmul(tf.silu(gate) * up, w_down)

    def decoder_layer(hidden, gamma_in, w_q, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache,
                      pos_ids, k_cache, v_cache, scale, w_o, gamma_post, w_gate, w_up, w_down):
        attn_out, k_new, v_new = self_attention(                  # model.py:268-297
            hidden, gamma_in, w_q, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache, pos_ids,
            k_cache, v_cache, scale, w_o)
        h1 = hidden + attn_out
        return h1 + mlp(h1, gamma_post, w_gate, w_up, w_down), k_new, v_new

    def embed(w_embed, token_ids):                                # model.py:311-318
        return tf.index_select(w_embed, token_ids, 0).reshape(1, 1, H)

    def final_rms_norm(hidden, gamma_final):                      # model.py:321-329
        return qwen_norm(hidden, gamma_final)

    def lm_head(hidden, w_head):                                  # model.py:332-336
        return tf.matmul(hidden.reshape(1, H), w_head)

    layer_impl = {"input_rms_norm": input_rms_norm, "self_attention": self_attention, "mlp": mlp,
                  "placed_mlp": mlp, "decoder_layer": decoder_layer}
    root_impl = {"embed": embed, "final_rms_norm": final_rms_norm, "lm_head": lm_head}

    def impl_for(module):
        return root_impl if module.modules else layer_impl

    return impl_for
