"""TEST INFRASTRUCTURE.  Qwen3.5-35B-A3B ``@func`` bodies restated op by op (f32 activations and state, bf16
contracted weights).  Follows reference ``examples/qwen3_5_35b_a3b-tilelang/model.py``; a matmul casts its
activation to the weight's dtype, runs at bf16 and casts the result back to f32 (``:189,214-225``)."""
from __future__ import annotations

import math

import torch

from . import ops as tf


def make(cfg):
    H, EPS = cfg.hidden, cfg.rms_eps
    HK, HV, DK, DV = cfg.gdn_n_k_heads, cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim
    KEY, VAL, CONV, KRN = cfg.key_dim, cfg.val_dim, cfg.conv_dim, cfg.gdn_conv_kernel
    VPK = HV // HK
    HQ, HKV, D, ROT = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.rotary_dim
    G = HQ // HKV
    K, I = cfg.top_k, cfg.moe_intermediate
    QSCALE, L2_EPS = 1.0 / math.sqrt(DK), 1e-6
    bw = torch.bfloat16

    def mm(x, w):                            # cast(matmul(cast(x, bf16), w), f32)
        return tf.matmul(x.to(bw), w).float()

    def rms(x, w, eps=1e-6):                 # tf.rms_norm on f32: f32 throughout
        return tf.rms_norm(x, w, eps)

    # ---- Qwen3_5LinearAttention ----
    def conv_step(conv_state, entry, conv_w):
        window = torch.cat((conv_state, entry), dim=2)
        summed = tf.reduce(window * conv_w.reshape(1, CONV, KRN), axes=(-1,), keepdim=False, kind="sum")
        return tf.silu(summed)

    def l2_normalise(x):
        ss = tf.reduce(torch.square(x), axes=(-1,), keepdim=True, kind="sum")
        return x * tf.rsqrt(ss + torch.full_like(ss, L2_EPS))

    def delta_step(recurrent_state, q, k, v, g, beta):
        decayed = recurrent_state * tf.exp(g).reshape(1, HV, 1, 1)
        k_col = k.reshape(1, HV, DK, 1)
        recalled = tf.reduce(decayed * k_col, axes=(-2,), keepdim=False, kind="sum")
        delta = (v.reshape(1, HV, DV) - recalled) * beta.reshape(1, HV, 1)
        updated = decayed + k_col * delta.reshape(1, HV, 1, DV)
        q_scaled = q * torch.full_like(q, QSCALE)
        read = tf.reduce(updated * q_scaled.reshape(1, HV, DK, 1), axes=(-2,), keepdim=False, kind="sum")
        return read, updated

    def linear_attention(hidden, gamma_in, w_in_qkv, w_in_z, w_in_b, w_in_a, conv_w, a_log, dt_bias, conv_state,
                         recurrent_state, gamma_gdn, w_out):
        hn = rms(hidden, gamma_in)
        entry = mm(hn, w_in_qkv).permute(0, 2, 1)
        mixed = conv_step(conv_state, entry, conv_w)
        q = l2_normalise(tf.repeat_interleave(mixed[:, :KEY].reshape(1, 1, HK, DK), VPK, 2))
        k = l2_normalise(tf.repeat_interleave(mixed[:, KEY:2 * KEY].reshape(1, 1, HK, DK), VPK, 2))
        v = mixed[:, 2 * KEY:CONV].reshape(1, 1, HV, DV)
        beta = tf.sigmoid(mm(hn, w_in_b))
        g = -tf.exp(a_log) * tf.softplus(mm(hn, w_in_a) + dt_bias)
        read, updated = delta_step(recurrent_state, q, k, v, g, beta)
        z = mm(hn, w_in_z).reshape(1, HV, DV)
        gated = rms(read, gamma_gdn) * tf.silu(z)
        return mm(gated.reshape(1, 1, VAL), w_out), entry, updated

    # ---- Qwen3_5FullAttention ----
    def partial_rope(x, cos_cache, sin_cache, pos_ids):
        turned, _ = tf.rope(x[..., :ROT], x[..., :ROT], cos_cache, sin_cache, pos_ids)
        return torch.cat((turned, x[..., ROT:D]), dim=-1)

    def full_attention(hidden, gamma_in, w_qg, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache, pos_ids, k_cache,
                       v_cache, scale, w_o):
        C = k_cache.shape[1]
        hn = rms(hidden, gamma_in)
        qg = mm(hn, w_qg).reshape(1, 1, HQ, 2 * D)
        q, gate = qg[..., :D], qg[..., D:2 * D]
        q_rope = partial_rope(rms(q, gamma_q), cos_cache, sin_cache, pos_ids)
        k_rope = partial_rope(rms(mm(hn, w_k).reshape(1, 1, HKV, D), gamma_k), cos_cache, sin_cache, pos_ids)
        v = mm(hn, w_v).reshape(1, 1, HKV, D)
        q_s = q_rope * scale
        k_ctx = tf.repeat_interleave(k_cache, G, 2).permute(0, 2, 1, 3).reshape(1, 1, HQ, C, D)
        v_ctx = tf.repeat_interleave(v_cache, G, 2).permute(0, 2, 1, 3).reshape(1, 1, HQ, C, D)
        k_new, v_new = tf.repeat_interleave(k_rope, G, 2), tf.repeat_interleave(v, G, 2)
        q_e = q_s.reshape(1, 1, HQ, 1, D)
        score_ctx = tf.reduce(q_e * k_ctx, axes=(-1,), keepdim=True, kind="sum")
        score_new = tf.reduce(q_s * k_new, axes=(-1,), keepdim=True, kind="sum")
        peak = tf.maximum(tf.reduce(score_ctx, axes=(-2,), keepdim=False, kind="max"), score_new)
        p_ctx = tf.exp(score_ctx - peak.reshape(1, 1, HQ, 1, 1))
        p_new = tf.exp(score_new - peak)
        total = tf.reduce(p_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new
        weighted = tf.reduce(p_ctx * v_ctx, axes=(-2,), keepdim=False, kind="sum") + p_new * v_new
        gated = (weighted / total).reshape(1, 1, HQ * D) * tf.sigmoid(gate.reshape(1, 1, HQ * D))
        return mm(gated, w_o), k_rope, v

    # ---- router / MoE ----
    def routing(tokens, w_router):
        probs = torch.softmax(mm(tokens, w_router), dim=-1)
        top_vals, indices = tf.topk(probs, K, dim=-1)
        return top_vals / tf.reduce(top_vals, axes=(-1,), keepdim=True, kind="sum"), indices

    def post_norm(hidden, gamma_post):
        return rms(hidden, gamma_post).reshape(1, H)

    def routed_experts(tokens, weights, indices, w_gate, w_up, w_down):
        flat = indices.reshape(K)
        col = tokens.reshape(1, 1, H, 1).to(bw)
        gate = tf.matmul(tf.index_select(w_gate, flat, 0).reshape(1, K, I, H), col).float().reshape(1, K, I)
        up = tf.matmul(tf.index_select(w_up, flat, 0).reshape(1, K, I, H), col).float().reshape(1, K, I)
        hid = tf.silu(gate) * up
        down = tf.matmul(tf.index_select(w_down, flat, 0).reshape(1, K, H, I), hid.reshape(1, K, I, 1).to(bw))
        weighted = down.float().reshape(1, K, H) * weights.reshape(1, K, 1)
        return tf.reduce(weighted, axes=(1,), keepdim=False, kind="sum")

    def shared_expert(tokens, w_shared_gate, w_shared_up, w_shared_down, w_shared_scale):
        dense = mm(tf.silu(mm(tokens, w_shared_gate)) * mm(tokens, w_shared_up), w_shared_down)
        return dense * tf.sigmoid(mm(tokens, w_shared_scale))

    def experts(tokens, weights, indices, w_gate, w_up, w_down, w_shared_gate, w_shared_up, w_shared_down,
                w_shared_scale):
        routed = routed_experts(tokens, weights, indices, w_gate, w_up, w_down)
        shared = shared_expert(tokens, w_shared_gate, w_shared_up, w_shared_down, w_shared_scale)
        return (routed + shared).reshape(1, 1, H)

    def residual_add(a, b):
        return a + b

    def embed(table, token_ids):
        return tf.index_select(table, token_ids, 0).float().reshape(1, 1, H)

    def final_rms_norm(hidden, gamma_final):
        return rms(hidden, gamma_final, EPS)

    def lm_head(hidden, w_head):
        return mm(hidden.reshape(1, H), w_head)

    impls = [
        {"conv_step": conv_step, "l2_normalise": l2_normalise, "delta_step": delta_step, "linear_attention": linear_attention},
        {"partial_rope": partial_rope, "partial_rope_kv": partial_rope, "full_attention": full_attention},
        {"routing": routing},
        {"post_norm": post_norm, "routed_experts": routed_experts, "shared_expert": shared_expert, "experts": experts},
        {"residual_add": residual_add},
        {"embed": embed, "final_rms_norm": final_rms_norm, "lm_head": lm_head},
    ]

    def impl_for(module):
        names = {f.name for f in module.functions}
        for table in impls:
            if names == set(table):
                return table
        raise KeyError(f"no restatement for module {module.name!r} with functions {sorted(names)}")

    return impl_for
