"""Runtime twin of the granite-4.0-h-small Modules (reference ``examples/granite_4_0_h_small-cuda/model.py``):
the same nesting (root -> layer -> mixer | moe -> router), every function under its authored name and
signature, state in and state out with nothing mutated; the C-ABI kernels inside."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored import granite_4_0_h_small as authored
from ..engine import paged_kv
from ..runtime import runtime_func, runtime_module
from ..runtime.decorator import TwinBase

BF = torch.bfloat16


def _new(shape, like, dtype=BF):
    return torch.empty(shape, device=like.device, dtype=dtype)


def _bf16(v: float) -> float:
    return float(torch.tensor(v, dtype=BF))


def make_twin(cfg: authored.GraniteConfig = authored.GRANITE_4_0_H_SMALL):
    sem = authored.build(cfg)
    H, V, EPS = cfg.hidden_size, cfg.vocab_size, cfg.rms_norm_eps
    NH, PD, NS, NG, KRN = cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_n_groups, cfg.mamba_d_conv
    EXP, CONVD, PROJ = cfg.expand, cfg.conv_dim, cfg.proj
    HQ, HKV, D, CAP = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx
    E, K, I, IS = cfg.num_local_experts, cfg.num_experts_per_tok, cfg.intermediate_size, cfg.shared_intermediate_size
    RES = _bf16(cfg.residual_multiplier)
    L = lib.load
    first = lambda name: next(m for m in sem.modules if m.mixer.name == "mixer" and
                              any(f.name == name for f in m.mixer.functions))
    mamba_sem = first("mamba_mixer").mixer
    attn_layers = [m for m in sem.modules if any(f.name == "full_attention" for f in m.mixer.functions)]
    attn_sem = attn_layers[0].mixer if attn_layers else None
    moe_sem = sem.modules[0].moe

    @runtime_module(mamba_sem)
    class Mamba:
        @runtime_func
        def in_projection(self, hidden, gamma_in, w_in):
            return lib.gemv(w_in, hidden.reshape(-1), _new(PROJ, hidden), gamma=gamma_in, prologue=lib.NORM_F32GAIN,
                            eps=EPS).reshape(1, PROJ)

        @runtime_func
        def conv_step(self, conv_state, entry, conv_w, conv_b):
            mixed, scratch = _new((1, CONVD), entry), torch.empty_like(conv_state)
            lib.check(L().tfb_conv_step(lib.ptr(entry.reshape(-1).contiguous()), lib.ptr(conv_state.contiguous()),
                                        lib.ptr(scratch), lib.ptr(conv_w), lib.ptr(conv_b), lib.ptr(mixed), None,
                                        CONVD, KRN, 0, lib.stream()), "tfb_conv_step")
            return mixed

        @runtime_func
        def ssm_step(self, ssm_state, x, b_vec, c_vec, dt_raw, a_log, dt_bias, d_skip):
            y, updated = _new((1, NH, PD), x), torch.empty_like(ssm_state)
            lib.check(L().tfb_ssm_step(lib.ptr(ssm_state.contiguous()), lib.ptr(updated), lib.ptr(x.contiguous()),
                                       lib.ptr(b_vec.contiguous()), lib.ptr(c_vec.contiguous()),
                                       lib.ptr(dt_raw.contiguous()), lib.ptr(a_log), lib.ptr(dt_bias), lib.ptr(d_skip),
                                       lib.ptr(y), NH, PD, NS, NG, 0, lib.stream()), "tfb_ssm_step")
            return y, updated

        @runtime_func
        def gated_out(self, y, gate, gamma_ssm, w_out):
            return lib.gemv(w_out, y.reshape(-1).contiguous(), _new(H, y), gamma=gamma_ssm, x_gate=gate.reshape(-1).contiguous(),
                            prologue=lib.NORM_GATED, eps=EPS).reshape(1, 1, H)

        @runtime_func
        def mamba_mixer(self, hidden, gamma_in, w_in, conv_w, conv_b, a_log, dt_bias, d_skip, conv_state, ssm_state,
                        gamma_ssm, w_out):
            proj = self.in_projection(hidden)
            gate = proj[:, :EXP]
            entry = proj[:, EXP:EXP + CONVD].reshape(1, CONVD, 1)
            mixed = self.conv_step(conv_state, entry)
            x = mixed[:, :EXP].reshape(1, NH, PD)
            b_vec = mixed[:, EXP:EXP + NG * NS].reshape(1, NG, NS)
            c_vec = mixed[:, EXP + NG * NS:CONVD].reshape(1, NG, NS)
            y, updated = self.ssm_step(ssm_state, x, b_vec, c_vec, proj[:, EXP + CONVD:PROJ])
            return self.gated_out(y, gate), entry.contiguous(), updated

    body_attn = None
    if attn_sem is not None:
        @runtime_module(attn_sem)
        class Attention:
            def load(self, resource):
                TwinBase.load(self, resource)
                b = self._bound
                self._w_qkv = torch.cat([b["w_q"], b["w_k"], b["w_v"]], 0).contiguous()

            def _attend(self, qkv_flat, k_cache, v_cache, cur_pos):
                dev = qkv_flat.device
                table = paged_kv.block_table(1, CAP, device=dev)
                k_pool, v_pool = paged_kv.new_pool(1, CAP, HKV, D, device=dev), paged_kv.new_pool(1, CAP, HKV, D, device=dev)
                paged_kv.fill_from_logical(k_pool, table[0], k_cache)
                paged_kv.fill_from_logical(v_pool, table[0], v_cache)
                nsplit = lib.attn_splits(CAP)
                attn = _new(HQ * D, qkv_flat)
                part_o, part_ml = _new(HQ * nsplit * D, qkv_flat, torch.float32), _new(HQ * nsplit * 2, qkv_flat, torch.float32)
                counters = torch.zeros(HKV, device=dev, dtype=torch.int32)
                pos = cur_pos.reshape(-1)[:1].to(torch.int32).contiguous()
                a = lib.AttnGqaArgs(qkv=lib.ptr(qkv_flat), pos=lib.ptr(pos), k_pool=lib.ptr(k_pool), v_pool=lib.ptr(v_pool),
                                    block_table=lib.ptr(table), out=lib.ptr(attn), part_o=lib.ptr(part_o),
                                    part_ml=lib.ptr(part_ml), counters=lib.ptr(counters), hq=HQ, hkv=HKV, d=D,
                                    rotary_dim=0, page_size=paged_kv.PAGE_SIZE, table_len=table.shape[1], max_ctx=CAP,
                                    max_pos=CAP, eps=EPS, scale=cfg.attention_multiplier, norm_mode=lib.NORM_NONE, pdl=0)
                lib.check(L().tfb_attn_gqa_decode(C.byref(a), lib.stream()), "tfb_attn_gqa_decode")
                return attn, paged_kv.logical_view(k_pool, table[0], CAP), paged_kv.logical_view(v_pool, table[0], CAP)

            def _qkv_flat(self, hidden):
                return lib.gemv(self._w_qkv, hidden.reshape(-1), _new((HQ + 2 * HKV) * D, hidden),
                                gamma=self._bound["gamma_in"], prologue=lib.NORM_F32GAIN, eps=EPS)

            @runtime_func
            def qkv(self, hidden, gamma_in, w_q, w_k, w_v):
                flat = self._qkv_flat(hidden)
                return (flat[:HQ * D].reshape(1, 1, HQ, D), flat[HQ * D:(HQ + HKV) * D].reshape(1, 1, HKV, D),
                        flat[(HQ + HKV) * D:].reshape(1, 1, HKV, D))

            @runtime_func
            def attend(self, q, k_cache, v_cache, cur_pos, mask, w_o):
                # the caches already hold this token's row at cur_pos; the kernel re-writes the same row
                p = int(cur_pos.reshape(-1)[0])
                flat = torch.cat([q.reshape(-1), k_cache[0, p].reshape(-1), v_cache[0, p].reshape(-1)]).contiguous()
                attn, _, _ = self._attend(flat, k_cache, v_cache, cur_pos)
                return lib.gemv(w_o, attn, _new(H, q)).reshape(1, 1, H)

            @runtime_func
            def full_attention(self, hidden, gamma_in, w_q, w_k, w_v, k_cache, v_cache, cur_pos, mask, w_o):
                attn, k_next, v_next = self._attend(self._qkv_flat(hidden), k_cache, v_cache, cur_pos)
                return lib.gemv(w_o, attn, _new(H, hidden)).reshape(1, 1, H), k_next.contiguous(), v_next.contiguous()
        body_attn = Attention

    @runtime_module(moe_sem.router)
    class Router:
        @runtime_func
        def routing(self, tokens, w_router):
            logits = lib.gemv(w_router, tokens.reshape(-1).contiguous(), _new(E, tokens))
            idx, w = _new((1, K), tokens, torch.int64), _new((1, K), tokens)
            lib.check(L().tfb_router_select(lib.ptr(logits), None, lib.ptr(idx), lib.ptr(w), None, E, K, 0, 0,
                                            lib.stream()), "tfb_router_select")
            return w, idx

    @runtime_module(moe_sem)
    class MoE:
        router = Router

        def _inner(self, tokens, indices, w_gate, w_up):
            return lib.gemv(w_gate, tokens.reshape(-1).contiguous(), _new(K * I, tokens), w2=w_up, epilogue=lib.EPI_SWIGLU,
                            expert_idx=indices.reshape(-1).contiguous(), rows_per_expert=I)

        def _down(self, tokens, inner, weights, indices, w_down, shared_act=None, w_shared_out=None):
            out = _new(H, tokens)
            a = lib.MoeDownArgs(w_down=lib.ptr(w_down), w_shared=lib.ptr(w_shared_out), inner=lib.ptr(inner),
                                shared_act=lib.ptr(shared_act), indices=lib.ptr(indices.reshape(-1).contiguous()),
                                weights=lib.ptr(weights.reshape(-1).contiguous()), out=lib.ptr(out), hidden=H, inter=I,
                                shared_inter=IS, top_k=K, res_scale=1.0, pdl=0)
            lib.check(L().tfb_moe_down(C.byref(a), lib.stream()), "tfb_moe_down")
            return out

        def _shared_act(self, tokens, w_shared_in):
            return lib.gemv(w_shared_in[:IS], tokens.reshape(-1).contiguous(), _new(IS, tokens), w2=w_shared_in[IS:],
                            epilogue=lib.EPI_SWIGLU)

        @runtime_func
        def post_norm(self, hidden, gamma_post):
            return lib.rmsnorm(hidden, gamma_post, torch.empty_like(hidden), EPS, lib.NORM_F32GAIN).reshape(1, H)

        @runtime_func
        def routed_experts(self, tokens, weights, indices, w_gate, w_up, w_down):
            inner = self._inner(tokens, indices, w_gate, w_up)
            return self._down(tokens, inner, weights, indices, w_down).reshape(1, H)

        @runtime_func
        def shared_mlp(self, tokens, w_shared_in, w_shared_out):
            return lib.gemv(w_shared_out, self._shared_act(tokens, w_shared_in), _new(H, tokens)).reshape(1, H)

        @runtime_func
        def experts(self, tokens, weights, indices, w_gate, w_up, w_down, w_shared_in, w_shared_out):
            inner = self._inner(tokens, indices, w_gate, w_up)
            shared = self._shared_act(tokens, w_shared_in)
            return self._down(tokens, inner, weights, indices, w_down, shared, w_shared_out).reshape(1, 1, H)

    def layer_cls(layer_sem, mixer_cls):
        @runtime_func
        def residual_add(self, a, b):
            out = torch.empty_like(a)
            lib.check(L().tfb_residual_add(lib.ptr(a.contiguous()), lib.ptr(b.contiguous()), lib.ptr(out), a.numel(), RES,
                                           lib.stream()), "tfb_residual_add")
            return out
        return runtime_module(layer_sem)(type(layer_sem.name + "_Twin", (), {"mixer": mixer_cls, "moe": MoE,
                                                                               "residual_add": residual_add}))

    body = {}
    for layer_sem in sem.modules:
        is_attn = any(f.name == "full_attention" for f in layer_sem.mixer.functions)
        body[layer_sem.name] = layer_cls(layer_sem, body_attn if is_attn else Mamba)

    @runtime_func
    def embed(self, table, token_ids):
        return lib.embed(table, token_ids.contiguous(), _new((1, 1, H), table), scale=_bf16(cfg.embedding_multiplier))

    @runtime_func
    def final_rms_norm(self, hidden, gamma_final):
        return lib.rmsnorm(hidden, gamma_final, torch.empty_like(hidden), EPS, lib.NORM_F32GAIN)

    @runtime_func
    def lm_head(self, hidden, table):
        logits = _new((1, V), hidden)
        n = lib.lm_head_scratch_entries(V)
        token = torch.zeros(1, device=hidden.device, dtype=torch.int64)
        val, idx = _new(n, hidden, torch.float32), _new(n, hidden, torch.int32)
        counter = torch.zeros(1, device=hidden.device, dtype=torch.int32)
        a = lib.LmHeadArgs(w=lib.ptr(table), x=lib.ptr(hidden.reshape(-1).contiguous()), logits=lib.ptr(logits),
                           token_out=lib.ptr(token), scratch_val=lib.ptr(val), scratch_idx=lib.ptr(idx),
                           counter=lib.ptr(counter), n=V, k=H, prologue=lib.NORM_NONE, eps=EPS, x_scale=1.0,
                           out_scale=1.0 / cfg.logits_scaling, pdl=0)
        lib.check(L().tfb_lm_head_argmax(C.byref(a), lib.stream()), "tfb_lm_head_argmax")
        self.last_token = token
        return logits

    body.update(embed=embed, final_rms_norm=final_rms_norm, lm_head=lm_head)
    return runtime_module(sem)(type("Granite4_0_H_Small_Twin", (), body))
