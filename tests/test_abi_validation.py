"""Argument validation of the C ABI (no GPU needed: every case is refused on the host before anything is launched).
Pointers are made-up, suitably aligned addresses that are never dereferenced."""
import ctypes as C

import pytest

from tilefoundry_b200 import lib

EINVAL, EALIGN, ECAPACITY = 1, 2, 3
P = 0x10000            # a 16-byte aligned non-null "pointer"
ODD = 0x10004          # not 16-byte aligned


@pytest.fixture(scope="module")
def so():
    return lib.load()


def gemv(**kw):
    base = dict(w=P, x=P, y=P, n=512, k=512, prologue=0, epilogue=0, eps=1e-6, x_scale=1.0, res_scale=1.0, out_scale=1.0)
    base.update(kw)
    return lib.GemvArgs(**base)


def test_gemv_rejects_bad_shapes_pointers_and_combinations(so):
    call = lambda a: so.tfb_gemv(C.byref(a), None)
    assert call(gemv(w=None)) == EINVAL and call(gemv(x=None)) == EINVAL and call(gemv(y=None)) == EINVAL
    assert call(gemv(n=0)) == EINVAL and call(gemv(k=0)) == EINVAL
    assert call(gemv(k=100)) == EINVAL                      # k must be a multiple of 256
    assert call(gemv(k=32768)) == EINVAL                    # wider than a CTA can stage
    assert call(gemv(prologue=7)) == EINVAL and call(gemv(epilogue=9)) == EINVAL
    assert call(gemv(prologue=lib.NORM_F32GAIN)) == EINVAL  # norm without gains
    assert call(gemv(epilogue=lib.EPI_RESIDUAL)) == EINVAL  # residual epilogue without a residual
    assert call(gemv(epilogue=lib.EPI_SWIGLU)) == EINVAL    # SwiGLU without the second matrix
    assert call(gemv(prologue=lib.NORM_GATED, gamma=P)) == EINVAL     # gated norm without its gate vector
    assert call(gemv(expert_idx=P, rows_per_expert=0)) == EINVAL
    assert call(gemv(expert_idx=P, rows_per_expert=96, n=500)) == EINVAL
    assert call(gemv(w=ODD)) == EALIGN and call(gemv(x=ODD)) == EALIGN
    assert so.tfb_gemv(None, None) == EINVAL


def test_gemv_f32_rejects_bad_arguments(so):
    def a(**kw):
        base = dict(w=P, x=P, y=P, n=512, k=512, prologue=0, epilogue=0, eps=1e-6)
        base.update(kw)
        return lib.GemvF32Args(**base)
    call = lambda x: so.tfb_gemv_f32(C.byref(x), None)
    assert call(a(k=96)) == EINVAL and call(a(n=0)) == EINVAL and call(a(w=None)) == EINVAL
    assert call(a(prologue=lib.NORM_CAST_THEN_GAIN, gamma=P)) == EINVAL        # a bf16-only convention
    assert call(a(prologue=lib.NORM_F32GAIN)) == EINVAL
    assert call(a(prologue=lib.NORM_SEGMENT_GATED, gamma=P, gate=P, seg=100)) == EINVAL   # not a power of two
    assert call(a(prologue=lib.NORM_SEGMENT_GATED, gamma=P, seg=128)) == EINVAL           # no gate vector
    assert call(a(epilogue=lib.EPI_STORE_F32)) == EINVAL
    assert call(a(epilogue=lib.EPI_SWIGLU)) == EINVAL
    assert call(a(rows_per_expert=128, routed_slots=2, n=512)) == EINVAL                  # routed slots without indices
    assert call(a(rows_per_expert=128, routed_slots=2, expert_idx=P, n=512)) == EINVAL    # extra slots without their rows
    assert call(a(route_counter=P, route_experts=300, route_top_k=8, idx_out=P, w_out=P)) == EINVAL
    assert call(a(x=ODD)) == EALIGN


def test_attention_rejects_bad_geometry(so):
    base = dict(qkv=P, cos_table=P, sin_table=P, pos=P, k_pool=P, v_pool=P, block_table=P, out=P, part_o=P, part_ml=P, counters=P, hq=16, hkv=8, d=128,
                rotary_dim=128, page_size=64, table_len=4, max_ctx=256, max_pos=256, eps=1e-6, scale=0.1, norm_mode=0, pdl=0)
    call = lambda **kw: so.tfb_attn_gqa_decode(C.byref(lib.AttnGqaArgs(**{**base, **kw})), None)
    assert call(hq=15) == EINVAL                            # heads must divide
    assert call(table_len=2) == ECAPACITY                   # the block table does not cover max_ctx
    assert call(out=None) == EINVAL
    # the allocation-free form validates the same way before it touches its stream: more KV heads than query heads
    # (a ticket clear of 128 words would run past its 64-word region) is refused with nothing queued
    noalloc = lambda **kw: so.tfb_attn_gqa_decode_noalloc(
        C.byref(lib.AttnGqaArgs(**{**base, "part_o": None, "part_ml": None, "counters": None, **kw})), None)
    assert noalloc(hq=64, hkv=128) == EINVAL
    assert noalloc(hq=15) == EINVAL and noalloc(out=None) == EINVAL and noalloc(table_len=2) == ECAPACITY
    assert noalloc(batch=2) == ECAPACITY                    # the built-in scratch holds one sequence
    gated = dict(proj=P, gamma_q=P, gamma_k=P, cos_table=P, sin_table=P, pos=P, k_pool=P, v_pool=P, block_table=P, out=P,
                 part_o=P, part_ml=P, counters=P, hq=16, hkv=2, d=256, rotary_dim=64, page_size=64, table_len=64, max_ctx=4096,
                 max_pos=4096, eps=1e-6, scale=0.0625, pdl=0)
    gcall = lambda **kw: so.tfb_attn_gated_decode(C.byref(lib.AttnGatedArgs(**{**gated, **kw})), None)
    assert gcall(rotary_dim=48) == EINVAL and gcall(rotary_dim=512) == EINVAL
    assert gcall(page_size=48) == EINVAL                    # a split must not straddle a page
    assert gcall(table_len=8) == ECAPACITY
    assert gcall(d=96) == EINVAL and gcall(hq=6) == EINVAL
    assert so.tfb_attn_gated_groups(16, 2, 256) == 8 and so.tfb_attn_gated_groups(16, 3, 256) == 0


def test_small_batch_projection_chain_and_collectives_reject_bad_arguments(so):
    tc = dict(w=P, x=P, y=P, partial=P, tickets=P, status=P, m=32, n=4096, k=2048, pdl=0)
    call = lambda **kw: so.tfb_gemm_small_m(C.byref(lib.GemmSmallMArgs(**{**tc, **kw})), None)
    assert call(m=0) == EINVAL and call(m=33) == EINVAL     # 1..32 tokens
    assert call(k=100) == EINVAL and call(n=0) == EINVAL
    assert call(status=None) == EINVAL and call(w=ODD) == EALIGN
    assert so.tfb_gemm_small_m_splits(0, 2048) == 0
    ch = lib.GemvChainArgs(n_phases=0, pdl=0, sync=P)
    assert so.tfb_gemv_chain(C.byref(ch), None) == EINVAL
    ch = lib.GemvChainArgs(n_phases=5, pdl=0, sync=P)
    assert so.tfb_gemv_chain(C.byref(ch), None) == EINVAL
    ch = lib.GemvChainArgs(n_phases=1, pdl=0, sync=None)
    ch.phase[0] = gemv()
    assert so.tfb_gemv_chain(C.byref(ch), None) == EINVAL
    ch = lib.GemvChainArgs(n_phases=1, pdl=0, sync=P)
    ch.phase[0] = gemv(expert_idx=P, rows_per_expert=64)    # gathered rows are not a chain phase
    assert so.tfb_gemv_chain(C.byref(ch), None) == EINVAL
    red = lib.MoeAllreduceArgs(partial=P, epoch=P, status=P, out=P, hidden=4096, rank=0, world=1, has_shared=1, res_scale=1.0)
    assert so.tfb_moe_allreduce_finalize(C.byref(red), None) == EINVAL          # an exchange needs at least two ranks
    red = lib.MoeAllreduceArgs(partial=P, epoch=P, status=P, out=P, hidden=4096, rank=2, world=2, has_shared=1, res_scale=1.0)
    assert so.tfb_moe_allreduce_finalize(C.byref(red), None) == EINVAL          # rank outside the world
    red = lib.MoeAllreduceArgs(partial=P, epoch=P, status=P, out=P, hidden=4096, rank=0, world=2, has_shared=1, res_scale=1.0)
    assert so.tfb_moe_allreduce_finalize(C.byref(red), None) == EINVAL          # peers' inboxes missing


def test_recurrent_and_moe_entry_points_reject_bad_arguments(so):
    gdn = dict(proj=P, conv_state=P, conv_state_stride=8192 * 3, conv_w=P, a_log=P, dt_bias=P, state=P, read=P, hk=16, hv=32,
               dk=128, dv=128, kernel_width=4, q_scale=0.088, pdl=0)
    call = lambda **kw: so.tfb_gdn_step(C.byref(lib.GdnArgs(**{**gdn, **kw})), None)
    assert call(dk=64) == EINVAL and call(kernel_width=3) == EINVAL and call(hv=30) == EINVAL
    assert call(conv_state_stride=100) == EINVAL            # the two window buffers would overlap
    assert call(state=None) == EINVAL and call(proj=None) == EINVAL
    assert call(direct_q=P) == EINVAL                       # the direct form needs all five vectors
    down = dict(w_down=P, inner=P, indices=P, weights=P, out=P, hidden=2048, inter=512, shared_inter=512, top_k=8, pdl=0)
    dcall = lambda **kw: so.tfb_moe_down_f32(C.byref(lib.MoeDownF32Args(**{**down, **kw})), None)
    assert dcall(top_k=40) == EINVAL and dcall(inter=100) == EINVAL and dcall(out=None) == EINVAL
    assert dcall(top_k=0) == EINVAL                         # nothing to compute without routed or shared rows
    assert dcall(top_k=32, inter=1024) == ECAPACITY         # the gathered activations must fit shared memory
    assert so.tfb_router_select(None, None, P, None, P, 256, 8, 1, 0, None) == EINVAL
    assert so.tfb_router_select(None, P, P, None, P, 300, 8, 1, 0, None) == EINVAL      # more experts than a warp holds
    assert so.tfb_router_select(None, P, P, None, P, 256, 8, 2, 0, None) == EINVAL      # unknown mode
    assert so.tfb_status_string(EINVAL) and so.tfb_status_string(ECAPACITY)


def test_several_sequence_step_rejects_bad_arguments(so):
    tc = dict(w=P, x=P, y=P, status=P, m=32, n=6144, k=2048, pdl=0, swiglu=1)
    call = lambda **kw: so.tfb_gemm_small_m(C.byref(lib.GemmSmallMArgs(**{**tc, **kw})), None)
    assert call(n=100) == EINVAL                            # the SwiGLU form pairs 64 gate rows with 64 up rows
    assert call(residual=P) == EINVAL                       # and has no residual
    assert so.tfb_gemm_small_m_swiglu_splits(6144, 2048) in (1, 2, 4, 8)
    assert so.tfb_gemm_small_m_splits(2048, 2048) in (1, 2, 4, 8)
    assert so.tfb_gemm_small_m_swiglu_splits(0, 2048) == 0

    attn = dict(qkv=P, cos_table=P, sin_table=P, pos=P, k_pool=P, v_pool=P, block_table=P, out=P, part_o=P, part_ml=P,
                counters=P, hq=16, hkv=8, d=128, rotary_dim=128, page_size=64, table_len=4, max_ctx=256, max_pos=256,
                eps=1e-6, scale=0.1, norm_mode=0, pdl=0, batch=4)
    assert so.tfb_attn_gqa_decode_noalloc(C.byref(lib.AttnGqaArgs(**attn)), None) == ECAPACITY   # built-in scratch: one sequence
    assert so.tfb_attn_gqa_decode(C.byref(lib.AttnGqaArgs(**{**attn, "batch": 70000})), None) == EINVAL

    layers = (lib.Qwen3BatchLayer * 1)()
    step = dict(layers=layers, n_layers=1, batch=32, hidden=2048, hq=16, hkv=8, d=128, inter=6144, pdl=1, vocab=151936,
                eps=1e-6, scale=0.088, w_embed=P, gamma_final=P, w_head=P, cos_table=P, sin_table=P, max_pos=2176,
                page_size=64, table_len=34, max_ctx=2176, block_table=P, tokens=P, pos=P, n_prompt=64, max_tokens=2177,
                hidden_buf=P, norm_buf=P, qkv_buf=P, attn_buf=P, act_buf=P, logits=P, part_o=P, part_ml=P, counters=P,
                status=P, pick_val=P, pick_idx=P)
    scall = lambda **kw: so.tfb_qwen3_batch_decode_step(C.byref(lib.Qwen3BatchStepArgs(**{**step, **kw})), None)
    assert scall(batch=0) == EINVAL and scall(batch=33) == EINVAL        # 1..32 sequences
    assert scall(logits=None) == EINVAL                                  # the pick reads the logits
    assert scall(status=None) == EINVAL and scall(norm_buf=None) == EINVAL
    assert scall(inter=6100) == EINVAL                                   # tile shapes
    assert scall(table_len=8) == ECAPACITY                               # the block table does not cover max_ctx
    assert scall(max_tokens=4000) == ECAPACITY
    assert so.tfb_qwen3_batch_decode_step(None, None) == EINVAL


def test_moe_batch_and_its_routing_reject_bad_arguments(so):
    def a(**kw):
        base = dict(x=P, indices=P, weights=P, w_gate=P, w_up=P, w_down=P, out=P, x_bf16=P, inner=P, y=P, counts=P, lists=P,
                    status=P, tokens=64, hidden=2048, inter=512, experts=256, top_k=8)
        base.update(kw)
        return lib.MoeBatchArgs(**base)
    call = lambda x: so.tfb_moe_batch(C.byref(x), None)
    assert so.tfb_moe_batch(None, None) == EINVAL
    assert call(a(x=None)) == EINVAL and call(a(out=None)) == EINVAL and call(a(counts=None)) == EINVAL
    assert call(a(w_gate=ODD)) == EALIGN and call(a(inner=ODD)) == EALIGN
    assert call(a(tokens=0)) == EINVAL and call(a(top_k=0)) == EINVAL and call(a(experts=600)) == EINVAL
    assert call(a(hidden=2000)) == EINVAL                  # the reduction lengths are multiples of 128
    assert call(a(inter=100)) == EINVAL
    assert call(a(hidden=8192)) == EINVAL                  # 24 rows of it do not fit a CTA's shared memory
    assert call(a(w_shared_gate=P)) == EINVAL              # a shared expert comes with all three matrices

    def r(**kw):
        base = dict(x=P, w_router=P, logits=P, indices=P, weights=P, tokens=64, hidden=2048, experts=256, top_k=8, mode=1)
        base.update(kw)
        return lib.MoeRouteArgs(**base)
    route = lambda x: so.tfb_moe_batch_route(C.byref(x), None)
    assert so.tfb_moe_batch_route(None, None) == EINVAL
    assert route(r(logits=None)) == EINVAL and route(r(mode=2)) == EINVAL and route(r(w_router=ODD)) == EALIGN
    assert route(r(experts=300)) == EINVAL and route(r(top_k=40)) == EINVAL and route(r(hidden=1000)) == EINVAL


def test_host_driven_step_rejects_null_arguments(so):
    assert so.tfb_graph_step_host(None, P, P, P, P, None) == EINVAL
    assert so.tfb_graph_step_host(P, None, P, P, P, None) == EINVAL
    assert so.tfb_graph_generate_host(P, P, -1, 4, P, None, None) == EINVAL
    assert so.tfb_graph_generate_host(None, P, 0, 4, P, None, None) == EINVAL
    assert so.tfb_graph_generate_host(P, P, 0, 0, P, None, None) == 0          # no steps: nothing is touched


def test_nucleus_sampling_rejects_bad_arguments(so):
    def a(**kw):
        base = dict(logits=P, pos=P, prev_pos=P, tokens=P, hist=P, vocab=1024, temperature=0.8, top_p=0.9)
        base.update(kw)
        return lib.SampleTopPArgs(**base)
    call = lambda x: so.tfb_sample_top_p(C.byref(x), None)
    assert so.tfb_sample_top_p(None, None) == EINVAL
    assert call(a(logits=None)) == EINVAL and call(a(prev_pos=None)) == EINVAL and call(a(hist=None)) == EINVAL
    assert call(a(temperature=0.0)) == EINVAL and call(a(top_p=0.0)) == EINVAL and call(a(top_p=1.5)) == EINVAL
    assert call(a(vocab=0)) == EINVAL
    assert call(a(n_eos=2)) == EINVAL and call(a(n_eos=2, eos_ids=P)) == EINVAL      # end ids come with their latch
    assert call(a(n_eos=17, eos_ids=P, stop_at=P)) == EINVAL
