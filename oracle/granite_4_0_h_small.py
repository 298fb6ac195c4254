"""TEST INFRASTRUCTURE.  granite-4.0-h-small ``@func`` bodies restated op by op.

Follows reference ``examples/granite_4_0_h_small-cuda/model.py`` line by line; every intermediate is
rounded where the evaluator rounds it.  A Python float in ``tf.full_like(x, value=v)`` becomes a tensor of
x's dtype, so ``0.22`` is the bf16 nearest to it where x is bf16.
"""
from __future__ import annotations

import torch

from . import ops as tf


def make(cfg):
    H, EPS, DT = cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype
    NH, PD, NS, NG = cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_n_groups
    EXP, CONVD, PROJ, KRN = cfg.expand, cfg.conv_dim, cfg.proj, cfg.mamba_d_conv
    HPG = NH // NG
    HQ, HKV, D, CAP = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx
    G = HQ // HKV
    K, I, IS = cfg.num_experts_per_tok, cfg.intermediate_size, cfg.shared_intermediate_size

    def full_like(x, value):
        return torch.full_like(x, value)

    # ---- GraniteMamba (:142-274) ----
    def in_projection(hidden, gamma_in, w_in):
        hn = tf.rms_norm(hidden, gamma_in, EPS)
        return tf.matmul(hn.reshape(1, H), w_in.t())

    def conv_step(conv_state, entry, conv_w, conv_b):
        window = torch.cat((conv_state, entry), dim=2)
        weighted = window * conv_w.reshape(1, CONVD, KRN)
        summed = tf.reduce(weighted, axes=(-1,), keepdim=False, kind="sum")
        return tf.silu(summed + conv_b.reshape(1, CONVD))

    def ssm_step(ssm_state, x, b_vec, c_vec, dt_raw, a_log, dt_bias, d_skip):
        dt = tf.softplus(dt_raw + dt_bias.reshape(1, NH))
        a = -tf.exp(tf.cast(a_log, "f32"))
        decay = tf.exp(tf.cast(dt, "f32") * a.reshape(1, NH))
        dt_e = dt.reshape(1, NH, 1, 1)
        b_e = tf.repeat_interleave(b_vec, HPG, 1).reshape(1, NH, 1, NS)
        c_e = tf.repeat_interleave(c_vec, HPG, 1).reshape(1, NH, 1, NS)
        d_bx = (dt_e * b_e) * x.reshape(1, NH, PD, 1)
        updated = ssm_state * decay.reshape(1, NH, 1, 1) + tf.cast(d_bx, "f32")
        read = tf.reduce(tf.cast(tf.cast(updated, DT), "f32") * tf.cast(c_e, "f32"), axes=(-1,), keepdim=False,
                         kind="sum")
        y = tf.cast(read, DT) + x * d_skip.reshape(1, NH, 1)
        return y, updated

    def gated_out(y, gate, gamma_ssm, w_out):
        gated = tf.cast(y.reshape(1, EXP), "f32") * tf.silu(tf.cast(gate, "f32"))
        normed = tf.cast(tf.rms_norm(gated, gamma_ssm, EPS), DT)
        return tf.matmul(normed, w_out.t()).reshape(1, 1, H)

    def mamba_mixer(hidden, gamma_in, w_in, conv_w, conv_b, a_log, dt_bias, d_skip, conv_state, ssm_state,
                    gamma_ssm, w_out):
        proj = in_projection(hidden, gamma_in, w_in)
        gate = proj[:, :EXP]
        entry = proj[:, EXP:EXP + CONVD].reshape(1, CONVD, 1)
        dt_raw = proj[:, EXP + CONVD:PROJ]
        mixed = conv_step(conv_state, entry, conv_w, conv_b)
        x = mixed[:, :EXP].reshape(1, NH, PD)
        b_vec = mixed[:, EXP:EXP + NG * NS].reshape(1, NG, NS)
        c_vec = mixed[:, EXP + NG * NS:CONVD].reshape(1, NG, NS)
        y, updated = ssm_step(ssm_state, x, b_vec, c_vec, dt_raw, a_log, dt_bias, d_skip)
        return gated_out(y, gate, gamma_ssm, w_out), entry, updated

    # ---- GraniteAttention (:282-373) ----
    def qkv(hidden, gamma_in, w_q, w_k, w_v):
        hn = tf.rms_norm(hidden, gamma_in, EPS).reshape(1, H)
        return (tf.matmul(hn, w_q.t()).reshape(1, 1, HQ, D), tf.matmul(hn, w_k.t()).reshape(1, 1, HKV, D),
                tf.matmul(hn, w_v.t()).reshape(1, 1, HKV, D))

    def attend(q, k_cache, v_cache, cur_pos, mask, w_o):
        k_ctx = tf.repeat_interleave(k_cache.permute(0, 2, 1, 3), G, 1)
        v_ctx = tf.repeat_interleave(v_cache.permute(0, 2, 1, 3), G, 1)
        q_e = q.reshape(1, HQ, 1, D)
        scores = tf.reduce(q_e * k_ctx, axes=(-1,), keepdim=False, kind="sum")
        s32 = tf.cast(scores, "f32")
        scaled = s32 * full_like(s32, cfg.attention_multiplier) + tf.cast(mask, "f32")
        probs = tf.cast(torch.softmax(scaled, dim=-1), DT)
        attn = tf.reduce(probs.reshape(1, HQ, CAP, 1) * v_ctx, axes=(-2,), keepdim=False, kind="sum")
        return tf.matmul(attn.reshape(1, HQ * D), w_o.t()).reshape(1, 1, H)

    def full_attention(hidden, gamma_in, w_q, w_k, w_v, k_cache, v_cache, cur_pos, mask, w_o):
        q, k, v = qkv(hidden, gamma_in, w_q, w_k, w_v)
        k_next = tf.cache_update(k_cache, k, int(cur_pos))
        v_next = tf.cache_update(v_cache, v, int(cur_pos))
        return attend(q, k_next, v_next, cur_pos, mask, w_o), k_next, v_next

    # ---- router / MoE (:376-478) ----
    def routing(tokens, w_router):
        logits = tf.cast(tf.matmul(tokens, w_router.t()), "f32")
        top_vals, indices = tf.topk(logits, K, dim=-1)
        return tf.cast(torch.softmax(top_vals, dim=-1), DT), indices

    def post_norm(hidden, gamma_post):
        return tf.rms_norm(hidden, gamma_post, EPS).reshape(1, H)

    def routed_experts(tokens, weights, indices, w_gate, w_up, w_down):
        flat = indices.reshape(K)
        gate_w = tf.index_select(w_gate, flat, 0).reshape(1, K, I, H)
        up_w = tf.index_select(w_up, flat, 0).reshape(1, K, I, H)
        down_w = tf.index_select(w_down, flat, 0).reshape(1, K, H, I)
        col = tokens.reshape(1, 1, H, 1)
        gate = tf.matmul(gate_w, col).reshape(1, K, I)
        up = tf.matmul(up_w, col).reshape(1, K, I)
        inner = tf.silu(gate) * up
        down = tf.matmul(down_w, inner.reshape(1, K, I, 1)).reshape(1, K, H)
        weighted = down * weights.reshape(1, K, 1)
        return tf.reduce(weighted, axes=(1,), keepdim=False, kind="sum")

    def shared_mlp(tokens, w_shared_in, w_shared_out):
        both = tf.matmul(tokens, w_shared_in.t())
        return tf.matmul(tf.silu(both[:, :IS]) * both[:, IS:2 * IS], w_shared_out.t())

    def experts(tokens, weights, indices, w_gate, w_up, w_down, w_shared_in, w_shared_out):
        routed = routed_experts(tokens, weights, indices, w_gate, w_up, w_down)
        return (routed + shared_mlp(tokens, w_shared_in, w_shared_out)).reshape(1, 1, H)

    def residual_add(a, b):
        return a + b * full_like(b, cfg.residual_multiplier)

    # ---- root (:615-640) ----
    def embed(table, token_ids):
        row = tf.index_select(table, token_ids, 0)
        return (row * full_like(row, cfg.embedding_multiplier)).reshape(1, 1, H)

    def final_rms_norm(hidden, gamma_final):
        return tf.rms_norm(hidden, gamma_final, EPS)

    def lm_head(hidden, table):
        logits = tf.matmul(hidden.reshape(1, H), table.t())
        return logits / full_like(logits, cfg.logits_scaling)

    impls = {
        "GraniteMamba": {"in_projection": in_projection, "conv_step": conv_step, "ssm_step": ssm_step,
                         "gated_out": gated_out, "mamba_mixer": mamba_mixer},
        "GraniteAttention": {"qkv": qkv, "attend": attend, "full_attention": full_attention},
        "GraniteRouter": {"routing": routing},
        "GraniteMoE": {"post_norm": post_norm, "routed_experts": routed_experts, "shared_mlp": shared_mlp,
                       "experts": experts},
        "layer": {"residual_add": residual_add},
        "root": {"embed": embed, "final_rms_norm": final_rms_norm, "lm_head": lm_head},
    }

    def impl_for(module):
        names = {f.name for f in module.functions}
        for table in impls.values():
            if names == set(table):
                return table
        raise KeyError(f"no restatement for module {module.name!r} with functions {sorted(names)}")

    return impl_for
