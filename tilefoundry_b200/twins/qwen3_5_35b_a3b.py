"""Runtime twin of the Qwen3.5-35B-A3B Modules (reference ``examples/qwen3_5_35b_a3b-tilelang/model.py``):
the same nesting (root -> layer -> mixer | moe -> router), every function under its authored name and
signature, state in and state out with nothing mutated; the C-ABI kernels inside.  Activations are f32;
the bf16 weights are re-laid as ``[out, in]`` rows once, at ``load``."""
from __future__ import annotations

import ctypes as C

import torch

from .. import lib
from ..authored import qwen3_5_35b_a3b as authored
from ..engine import paged_kv
from ..engine.qwen3_5 import _rows, pack_mixer, pack_moe
from ..runtime import runtime_func, runtime_module
from ..runtime.decorator import TwinBase

F32 = torch.float32


def _new(shape, like, dtype=F32):
    return torch.empty(shape, device=like.device, dtype=dtype)


def _flat(t):
    return t.reshape(-1).contiguous()


def make_twin(cfg: authored.Qwen35Config = authored.QWEN3_5_35B_A3B):
    sem = authored.build(cfg)
    H, V, EPS = cfg.hidden, cfg.vocab, cfg.rms_eps
    HK, HV, DK, DV, KRN = cfg.gdn_n_k_heads, cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim, cfg.gdn_conv_kernel
    KEY, VAL, CONV = cfg.key_dim, cfg.val_dim, cfg.conv_dim
    HQ, HKV, D, ROT, CAP = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.rotary_dim, cfg.max_ctx
    E, K, I, IS = cfg.n_experts, cfg.top_k, cfg.moe_intermediate, cfg.shared_intermediate
    N_GDN, N_ATT = CONV + VAL + 2 * HV, 2 * HQ * D + 2 * HKV * D
    QSCALE = DK ** -0.5
    L = lib.load
    kinds = cfg.layer_types
    gdn_layer = sem.modules[kinds.index("linear_attention")]
    attn_layer = sem.modules[kinds.index("full_attention")]
    moe_sem = sem.modules[0].moe

    def gemv(w, x, n, k, *, like, **kw):
        y = _new(n, like)
        a = lib.GemvF32Args(w=lib.ptr(w), x=lib.ptr(x), y=lib.ptr(y), n=n, k=k, eps=EPS, pdl=0,
                            **{name: (lib.ptr(v) if isinstance(v, torch.Tensor) else v) for name, v in kw.items()})
        lib.check(L().tfb_gemv_f32(C.byref(a), lib.stream()), "tfb_gemv_f32")
        return y

    def gdn(state, read, **kw):
        a = lib.GdnArgs(state=lib.ptr(state), read=lib.ptr(read), hk=HK, hv=HV, dk=DK, dv=DV, kernel_width=KRN,
                        q_scale=QSCALE, pdl=0, **{n: (lib.ptr(v) if isinstance(v, torch.Tensor) else v) for n, v in kw.items()})
        lib.check(L().tfb_gdn_step(C.byref(a), lib.stream()), "tfb_gdn_step")

    @runtime_module(gdn_layer.mixer)
    class LinearAttention:
        def load(self, resource):
            TwinBase.load(self, resource)
            self._p = pack_mixer("linear_attention", self._bound)

        @runtime_func
        def conv_step(self, conv_state, entry, conv_w):
            mixed = _new((1, CONV), entry)
            lib.check(L().tfb_conv_silu_f32(lib.ptr(_flat(conv_state)), lib.ptr(_flat(entry)), lib.ptr(conv_w),
                                            lib.ptr(mixed), CONV, KRN, 0, lib.stream()), "tfb_conv_silu_f32")
            return mixed

        @runtime_func
        def l2_normalise(self, x):
            y = torch.empty_like(x)
            lib.check(L().tfb_l2norm_f32(lib.ptr(_flat(x)), lib.ptr(y), HV, DK, 1e-6, 0, lib.stream()), "tfb_l2norm_f32")
            return y

        @runtime_func
        def delta_step(self, recurrent_state, q, k, v, g, beta):
            updated, read = recurrent_state.clone().contiguous(), _new((1, HV, DV), q)
            gdn(updated, read, direct_q=_flat(q), direct_k=_flat(k), direct_v=_flat(v), direct_g=_flat(g),
                direct_beta=_flat(beta))
            return read, updated

        @runtime_func
        def linear_attention(self, hidden, gamma_in, w_in_qkv, w_in_z, w_in_b, w_in_a, conv_w, a_log, dt_bias, conv_state,
                             recurrent_state, gamma_gdn, w_out):
            p = self._p
            proj = gemv(p["w_in"], _flat(hidden), N_GDN, H, like=hidden, gamma=gamma_in, prologue=lib.NORM_F32GAIN)
            windows = torch.stack([conv_state.reshape(CONV, KRN - 1), torch.zeros_like(conv_state.reshape(CONV, KRN - 1))]).contiguous()
            updated, read = recurrent_state.clone().contiguous(), _new(VAL, hidden)
            gdn(updated, read, proj=proj, conv_state=windows, conv_state_stride=CONV * (KRN - 1), conv_w=conv_w, a_log=a_log,
                dt_bias=dt_bias)
            out = gemv(p["w_out"], read, H, VAL, like=hidden, gamma=gamma_gdn, gate=proj[CONV:CONV + VAL], seg=DV,
                       prologue=lib.NORM_SEGMENT_GATED)
            return out.reshape(1, 1, H), proj[:CONV].reshape(1, CONV, 1).clone(), updated

    @runtime_module(attn_layer.mixer)
    class FullAttention:
        def load(self, resource):
            TwinBase.load(self, resource)
            self._p = pack_mixer("full_attention", self._bound)

        def _rope(self, x, heads, cos_cache, sin_cache, pos_ids):
            out = torch.empty_like(x)
            lib.check(L().tfb_partial_rope_f32(lib.ptr(_flat(x)), lib.ptr(cos_cache), lib.ptr(sin_cache),
                                               lib.ptr(pos_ids.to(torch.int32).contiguous()), lib.ptr(out), heads, D, ROT, 0,
                                               lib.stream()), "tfb_partial_rope_f32")
            return out

        @runtime_func
        def partial_rope(self, x, cos_cache, sin_cache, pos_ids):
            return self._rope(x, HQ, cos_cache, sin_cache, pos_ids)

        @runtime_func
        def partial_rope_kv(self, x, cos_cache, sin_cache, pos_ids):
            return self._rope(x, HKV, cos_cache, sin_cache, pos_ids)

        @runtime_func
        def full_attention(self, hidden, gamma_in, w_qg, w_k, w_v, gamma_q, gamma_k, cos_cache, sin_cache, pos_ids, k_cache,
                           v_cache, scale, w_o):
            p, dev = self._p, hidden.device
            ctx = k_cache.shape[1]
            proj = gemv(p["w_in"], _flat(hidden), N_ATT, H, like=hidden, gamma=gamma_in, prologue=lib.NORM_F32GAIN)
            table = paged_kv.block_table(1, CAP, device=dev)
            k_pool = paged_kv.new_pool(1, CAP, HKV, D, device=dev, dtype=F32)
            v_pool = paged_kv.new_pool(1, CAP, HKV, D, device=dev, dtype=F32)
            paged_kv.fill_from_logical(k_pool, table[0], k_cache)
            paged_kv.fill_from_logical(v_pool, table[0], v_cache)
            nsplit = L().tfb_attn_gated_splits(CAP)
            out, k_new, v_new = _new(HQ * D, hidden), _new((1, 1, HKV, D), hidden), _new((1, 1, HKV, D), hidden)
            part_o, part_ml = _new(HQ * nsplit * D, hidden), _new(HQ * nsplit * 2, hidden)
            counters = torch.zeros(L().tfb_attn_gated_groups(HQ, HKV, D), device=dev, dtype=torch.int32)
            at = torch.tensor([ctx], device=dev, dtype=torch.int32)       # the cache holds ctx rows: append at ctx
            a = lib.AttnGatedArgs(proj=lib.ptr(proj), gamma_q=lib.ptr(gamma_q), gamma_k=lib.ptr(gamma_k),
                                  cos_table=lib.ptr(cos_cache), sin_table=lib.ptr(sin_cache), pos=lib.ptr(at),
                                  rope_pos=lib.ptr(pos_ids.to(torch.int32).contiguous()), k_pool=lib.ptr(k_pool),
                                  v_pool=lib.ptr(v_pool), block_table=lib.ptr(table), out=lib.ptr(out),
                                  k_new_out=lib.ptr(k_new), v_new_out=lib.ptr(v_new), part_o=lib.ptr(part_o),
                                  part_ml=lib.ptr(part_ml), counters=lib.ptr(counters), hq=HQ, hkv=HKV, d=D,
                                  rotary_dim=ROT, page_size=paged_kv.PAGE_SIZE, table_len=table.shape[1], max_ctx=CAP,
                                  max_pos=CAP, eps=EPS, scale=float(scale.reshape(-1)[0]), pdl=0)
            lib.check(L().tfb_attn_gated_decode(C.byref(a), lib.stream()), "tfb_attn_gated_decode")
            mixed = gemv(p["w_out"], out, H, HQ * D, like=hidden)
            return mixed.reshape(1, 1, H), k_new, v_new

    @runtime_module(moe_sem.router)
    class Router:
        def load(self, resource):
            TwinBase.load(self, resource)
            self._w = _rows(self._bound["w_router"])

        @runtime_func
        def routing(self, tokens, w_router):
            logits = gemv(self._w, _flat(tokens), E, H, like=tokens)
            idx, w = _new((1, K), tokens, torch.int64), _new((1, K), tokens)
            lib.check(L().tfb_router_select(None, lib.ptr(logits), lib.ptr(idx), None, lib.ptr(w), E, K, 1, 0, lib.stream()),
                      "tfb_router_select")
            return w, idx

    @runtime_module(moe_sem)
    class MoE:
        router = Router

        def load(self, resource):
            TwinBase.load(self, resource)
            b = self._bound
            self._sg, self._su, self._sd = _rows(b["w_shared_gate"]), _rows(b["w_shared_up"]), _rows(b["w_shared_down"])
            self._scale = _rows(b["w_shared_scale"])

        def _down(self, like, inner, top_k, weights=None, indices=None, w_down=None, shared=False, gate_logit=None):
            out = _new(H, like)
            a = lib.MoeDownF32Args(w_down=lib.ptr(w_down), w_shared=lib.ptr(self._sd) if shared else None,
                                   inner=lib.ptr(inner), indices=lib.ptr(indices), weights=lib.ptr(weights),
                                   shared_gate_logit=lib.ptr(gate_logit), out=lib.ptr(out), hidden=H, inter=I,
                                   shared_inter=IS, top_k=top_k, pdl=0)
            lib.check(L().tfb_moe_down_f32(C.byref(a), lib.stream()), "tfb_moe_down_f32")
            return out

        @runtime_func
        def post_norm(self, hidden, gamma_post):
            y = torch.empty_like(hidden)
            lib.check(L().tfb_rmsnorm_f32(lib.ptr(_flat(hidden)), lib.ptr(gamma_post), lib.ptr(y), 1, H, 1e-6, 0, lib.stream()),
                      "tfb_rmsnorm_f32")
            return y.reshape(1, H)

        @runtime_func
        def routed_experts(self, tokens, weights, indices, w_gate, w_up, w_down):
            idx = _flat(indices)
            inner = gemv(w_gate, _flat(tokens), K * I, H, like=tokens, w2=w_up, epilogue=lib.EPI_SWIGLU, expert_idx=idx,
                         rows_per_expert=I, routed_slots=K)
            return self._down(tokens, inner, K, _flat(weights), idx, w_down).reshape(1, H)

        @runtime_func
        def shared_expert(self, tokens, w_shared_gate, w_shared_up, w_shared_down, w_shared_scale):
            x = _flat(tokens)
            inner = gemv(self._sg, x, IS, H, like=tokens, w2=self._su, epilogue=lib.EPI_SWIGLU)
            logit = gemv(self._scale, x, 1, H, like=tokens)
            return self._down(tokens, inner, 0, shared=True, gate_logit=logit).reshape(1, H)

        @runtime_func
        def experts(self, tokens, weights, indices, w_gate, w_up, w_down, w_shared_gate, w_shared_up, w_shared_down,
                    w_shared_scale):
            x, idx = _flat(tokens), _flat(indices)
            inner = gemv(w_gate, x, K * I + IS, H, like=tokens, w2=w_up, w_extra=self._sg, w2_extra=self._su,
                         epilogue=lib.EPI_SWIGLU, expert_idx=idx, rows_per_expert=I, routed_slots=K)
            logit = gemv(self._scale, x, 1, H, like=tokens)
            return self._down(tokens, inner, K, _flat(weights), idx, w_down, shared=True, gate_logit=logit).reshape(1, 1, H)

        def route_batch(self, tokens):
            """``routing`` and the shared expert's gate logit for a batch: tokens f32 [T, H] (post-norm) -> routing
            weights f32 [T, K], indices int64 [T, K], gate logits f32 [T] (``tfb_moe_batch_route``)."""
            T = tokens.shape[0]
            x = tokens.contiguous()
            dev = x.device
            weights = torch.empty(T, K, device=dev, dtype=torch.float32)
            indices = torch.empty(T, K, device=dev, dtype=torch.int64)
            gate = torch.empty(T, device=dev, dtype=torch.float32)
            logits = torch.empty(T, E + 1, device=dev, dtype=torch.float32)
            a = lib.MoeRouteArgs(x=lib.ptr(x), w_router=lib.ptr(self.router._w), w_shared_scale=lib.ptr(self._scale),
                                 logits=lib.ptr(logits), indices=lib.ptr(indices), weights=lib.ptr(weights),
                                 shared_gate=lib.ptr(gate), tokens=T, hidden=H, experts=E, top_k=K, mode=1, pdl=0)
            lib.check(L().tfb_moe_batch_route(C.byref(a), lib.stream()), "tfb_moe_batch_route")
            return weights, indices, gate

        def forward_batch(self, hidden):
            """The block's forward for a batch: hidden f32 [T, H] -> f32 [T, H] (post-norm, routing, experts), four kernels
            for the routing and the norm plus the four of ``tfb_moe_batch`` whatever the number of tokens."""
            T = hidden.shape[0]
            x = hidden.contiguous()
            tokens = torch.empty_like(x)
            lib.check(L().tfb_rmsnorm_f32(lib.ptr(x), lib.ptr(self._bound["gamma_post"]), lib.ptr(tokens), T, H, 1e-6, 0, lib.stream()),
                      "tfb_rmsnorm_f32")
            weights, indices, gate = self.route_batch(tokens)
            return self.experts_batch(tokens, weights, indices, gate)

        def experts_batch(self, tokens, weights, indices, gate_logits=None):
            """``experts`` for a batch: tokens f32 [T, H], routing weights f32 [T, K] and indices int64 [T, K] -> f32 [T, H].
            Every selected expert is read once for all of its tokens (``tfb_moe_batch``)."""
            b = self._bound
            T = tokens.shape[0]
            x = tokens.contiguous()
            dev = x.device
            logits = gate_logits if gate_logits is not None else \
                torch.cat([gemv(self._scale, x[t], 1, H, like=x[t]) for t in range(T)]).contiguous()
            out = torch.empty(T, H, device=dev, dtype=torch.float32)
            scratch = dict(x_bf16=torch.empty(T, H, device=dev, dtype=torch.bfloat16),
                           inner=torch.empty(T, K + 1, I, device=dev, dtype=torch.bfloat16),
                           y=torch.empty(T, K + 1, H, device=dev, dtype=torch.bfloat16),
                           counts=torch.empty(2 * (E + 1) + 1, device=dev, dtype=torch.int32),
                           lists=torch.empty(E + 1, T, device=dev, dtype=torch.int32))
            status = torch.zeros(1, device=dev, dtype=torch.int32)
            if IS != I:
                raise ValueError("tfb_moe_batch takes a shared expert as wide as the routed ones")
            a = lib.MoeBatchArgs(x=lib.ptr(x), indices=lib.ptr(indices.contiguous()), weights=lib.ptr(weights.contiguous()),
                                 shared_gate=lib.ptr(logits), residual=None, w_gate=lib.ptr(b["w_gate"]), w_up=lib.ptr(b["w_up"]),
                                 w_down=lib.ptr(b["w_down"]), w_shared_gate=lib.ptr(self._sg), w_shared_up=lib.ptr(self._su),
                                 w_shared_down=lib.ptr(self._sd), out=lib.ptr(out), status=lib.ptr(status), tokens=T, hidden=H,
                                 inter=I, experts=E, top_k=K, pdl=0, **{k: lib.ptr(v) for k, v in scratch.items()})
            lib.check(L().tfb_moe_batch(C.byref(a), lib.stream()), "tfb_moe_batch")
            if int(status):
                raise RuntimeError(f"tfb_moe_batch: a bounded wait gave up (status {int(status):#x})")
            return out

    def layer_cls(layer_sem, mixer_cls):
        @runtime_func
        def residual_add(self, a, b):
            out = torch.empty_like(a)
            lib.check(L().tfb_residual_add_f32(lib.ptr(a.contiguous()), lib.ptr(b.contiguous()), lib.ptr(out), a.numel(), 0,
                                               lib.stream()), "tfb_residual_add_f32")
            return out
        return runtime_module(layer_sem)(type(layer_sem.name + "_Twin", (), {"mixer": mixer_cls, "moe": MoE,
                                                                               "residual_add": residual_add}))

    body = {}
    for layer_sem, kind in zip(sem.modules, kinds):
        body[layer_sem.name] = layer_cls(layer_sem, LinearAttention if kind == "linear_attention" else FullAttention)

    def load(self, resource):
        TwinBase.load(self, resource)
        self._head = _rows(self._bound["w_head"])

    @runtime_func
    def embed(self, table, token_ids):
        out = _new((1, 1, H), table)
        lib.check(L().tfb_embed_f32(lib.ptr(table), lib.ptr(token_ids.contiguous()), lib.ptr(out), 1, H, V, 0, lib.stream()),
                  "tfb_embed_f32")
        return out

    @runtime_func
    def final_rms_norm(self, hidden, gamma_final):
        y = torch.empty_like(hidden)
        lib.check(L().tfb_rmsnorm_f32(lib.ptr(_flat(hidden)), lib.ptr(gamma_final), lib.ptr(y), 1, H, EPS, 0, lib.stream()),
                  "tfb_rmsnorm_f32")
        return y

    @runtime_func
    def lm_head(self, hidden, w_head):
        logits = _new((1, V), hidden, torch.bfloat16)
        n = lib.lm_head_scratch_entries(V)
        token = torch.zeros(1, device=hidden.device, dtype=torch.int64)
        val, idx = _new(n, hidden), _new(n, hidden, torch.int32)
        counter = torch.zeros(1, device=hidden.device, dtype=torch.int32)
        a = lib.LmHeadArgs(w=lib.ptr(self._head), x=lib.ptr(_flat(hidden)), logits=lib.ptr(logits), token_out=lib.ptr(token),
                           scratch_val=lib.ptr(val), scratch_idx=lib.ptr(idx), counter=lib.ptr(counter), n=V, k=H,
                           prologue=lib.NORM_F32_INPUT, eps=EPS, x_scale=1.0, out_scale=1.0, pdl=0)
        lib.check(L().tfb_lm_head_argmax(C.byref(a), lib.stream()), "tfb_lm_head_argmax")
        self.last_token = token
        return logits.float()

    body.update(load=load, embed=embed, final_rms_norm=final_rms_norm, lm_head=lm_head)
    return runtime_module(sem)(type("Qwen3_5_35B_A3B_Twin", (), body))
