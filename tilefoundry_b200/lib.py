"""ctypes binding of ``libtfb200.so`` (declarations: ``include/tfb200.h``).

There is no CPU or PyTorch fallback: if the library is missing or a call returns a
non-zero status, a ``RuntimeError`` is raised.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

import torch

import os

LIB_PATH = Path(os.environ.get("TFB200_LIB") or Path(__file__).resolve().parent / "csrc" / "libtfb200.so")

NORM_NONE, NORM_F32GAIN, NORM_CAST_THEN_GAIN, NORM_GATED = 0, 1, 2, 3
NORM_SEGMENT_GATED, NORM_F32_INPUT = 4, 5
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU, EPI_STORE_F32 = 0, 1, 2, 3

_vp, _i32, _i64, _u64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float


class GemvArgs(C.Structure):
    _fields_ = [("w", _vp), ("w2", _vp), ("x", _vp), ("gamma", _vp), ("residual", _vp), ("y", _vp),
                ("n", _i32), ("k", _i32), ("prologue", _i32), ("epilogue", _i32),
                ("eps", _f32), ("x_scale", _f32), ("res_scale", _f32), ("out_scale", _f32),
                ("prefetch", _vp), ("prefetch_bytes", _u64), ("pdl", _i32), ("kernel", _i32), ("self_prefetch", _i32), ("rows_per_expert", _i32), ("expert_idx", _vp), ("x_gate", _vp), ("expert_rank", _i32), ("expert_world", _i32)]


class LmHeadArgs(C.Structure):
    _fields_ = [("w", _vp), ("x", _vp), ("gamma", _vp), ("logits", _vp), ("token_out", _vp),
                ("scratch_val", _vp), ("scratch_idx", _vp), ("counter", _vp),
                ("n", _i32), ("k", _i32), ("prologue", _i32),
                ("eps", _f32), ("x_scale", _f32), ("out_scale", _f32), ("pdl", _i32),
                ("tokens", _vp), ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32), ("kernel", _i32), ("self_prefetch", _i32), ("index_offset", _i32), ("pair_out", _vp),
                ("temperature", _f32), ("seed", _u64),
                ("eos_ids", _vp), ("stop_at", _vp), ("n_eos", _i32), ("reserved_eos", _i32)]


class AttnGqaArgs(C.Structure):
    _fields_ = [("qkv", _vp), ("gamma_q", _vp), ("gamma_k", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("pos", _vp), ("rope_pos", _vp), ("k_pool", _vp), ("v_pool", _vp), ("block_table", _vp), ("out", _vp),
                ("k_new_out", _vp), ("v_new_out", _vp), ("part_o", _vp), ("part_ml", _vp), ("counters", _vp),
                ("hq", _i32), ("hkv", _i32), ("d", _i32), ("rotary_dim", _i32),
                ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32), ("max_pos", _i32),
                ("eps", _f32), ("scale", _f32), ("norm_mode", _i32), ("pdl", _i32),
                ("prefetch", _vp), ("prefetch_bytes", _u64), ("batch", _i32), ("chunk", _i32)]


class Qwen3Layer(C.Structure):
    _fields_ = [(n, _vp) for n in ("gamma_in", "w_qkv", "gamma_q", "gamma_k", "w_o", "gamma_post",
                                   "w_gate", "w_up", "w_down", "k_pool", "v_pool")]


class Qwen3StepArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(Qwen3Layer)),
                ("n_layers", _i32), ("hidden", _i32), ("hq", _i32), ("hkv", _i32), ("d", _i32), ("inter", _i32),
                ("vocab", _i64), ("eps", _f32), ("scale", _f32),
                ("w_embed", _vp), ("gamma_final", _vp), ("w_head", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("max_pos", _i32), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("tokens", _vp), ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32),
                ("hidden_buf", _vp), ("qkv_buf", _vp), ("attn_buf", _vp), ("act_buf", _vp), ("logits", _vp),
                ("part_o", _vp), ("part_ml", _vp), ("counters", _vp), ("head_val", _vp), ("head_idx", _vp),
                ("hidden_trace", _vp), ("pdl", _i32), ("l2_prefetch", _i32), ("kernel", _i32), ("picked", _vp),
                ("chain_sync", _vp), ("temperature", _f32), ("seed", _u64),
                ("step_layers", _vp), ("step_sync", _vp), ("step_status", _vp),
                ("eos_ids", _vp), ("stop_at", _vp), ("n_eos", _i32), ("reserved_eos", _i32), ("step_xbuf", _vp)]


class GemvChainArgs(C.Structure):
    _fields_ = [("phase", GemvArgs * 4), ("n_phases", _i32), ("pdl", _i32), ("sync", _vp)]


class GemmSmallMArgs(C.Structure):
    _fields_ = [("w", _vp), ("x", _vp), ("residual", _vp), ("y", _vp), ("partial", _vp), ("tickets", _vp), ("status", _vp),
                ("m", _i32), ("n", _i32), ("k", _i32), ("pdl", _i32), ("swiglu", _i32), ("res_scale", _f32)]


class Qwen3BatchLayer(C.Structure):
    _fields_ = [(n, _vp) for n in ("gamma_in", "w_qkv", "gamma_q", "gamma_k", "w_o", "gamma_post", "w_gate_up",
                                   "w_down", "k_pool", "v_pool")]


class Qwen3BatchStepArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(Qwen3BatchLayer)),
                ("n_layers", _i32), ("batch", _i32), ("hidden", _i32), ("hq", _i32), ("hkv", _i32), ("d", _i32),
                ("inter", _i32), ("pdl", _i32), ("vocab", _i64), ("eps", _f32), ("scale", _f32),
                ("w_embed", _vp), ("gamma_final", _vp), ("w_head", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("max_pos", _i32), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("tokens", _vp), ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32),
                ("hidden_buf", _vp), ("norm_buf", _vp), ("qkv_buf", _vp), ("attn_buf", _vp), ("act_buf", _vp),
                ("logits", _vp), ("part_o", _vp), ("part_ml", _vp), ("counters", _vp),
                ("status", _vp), ("pick_val", _vp), ("pick_idx", _vp), ("picked", _vp),
                ("hidden_trace", _vp), ("temperature", _f32), ("reserved", _i32), ("seed", C.c_uint64)]


class Qwen3PrefillArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(Qwen3BatchLayer)),
                ("n_layers", _i32), ("m", _i32), ("hidden", _i32), ("hq", _i32), ("hkv", _i32), ("d", _i32),
                ("inter", _i32), ("pdl", _i32), ("eps", _f32), ("scale", _f32), ("vocab", _i64),
                ("w_embed", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("max_pos", _i32), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("ids", _vp), ("pos_rows", _vp),
                ("hidden_buf", _vp), ("norm_buf", _vp), ("qkv_buf", _vp), ("attn_buf", _vp), ("act_buf", _vp),
                ("part_o", _vp), ("part_ml", _vp), ("counters", _vp), ("status", _vp)]


class SampleTopPArgs(C.Structure):
    _fields_ = [("logits", _vp), ("pos", _vp), ("prev_pos", _vp), ("tokens", _vp), ("picked", _vp), ("threshold_out", _vp),
                ("eos_ids", _vp), ("stop_at", _vp), ("hist", _vp), ("vocab", _i32), ("n_prompt", _i32), ("n_eos", _i32),
                ("pdl", _i32), ("temperature", _f32), ("top_p", _f32), ("seed", C.c_uint64)]


class MoeRouteArgs(C.Structure):
    _fields_ = [("x", _vp), ("w_router", _vp), ("w_shared_scale", _vp), ("logits", _vp), ("indices", _vp), ("weights", _vp),
                ("shared_gate", _vp), ("tokens", _i32), ("hidden", _i32), ("experts", _i32), ("top_k", _i32), ("mode", _i32),
                ("pdl", _i32)]


class MoeBatchArgs(C.Structure):
    _fields_ = [("x", _vp), ("indices", _vp), ("weights", _vp), ("shared_gate", _vp), ("residual", _vp),
                ("w_gate", _vp), ("w_up", _vp), ("w_down", _vp), ("w_shared_gate", _vp), ("w_shared_up", _vp),
                ("w_shared_down", _vp), ("out", _vp), ("x_bf16", _vp), ("inner", _vp), ("y", _vp), ("counts", _vp),
                ("lists", _vp), ("status", _vp), ("tokens", _i32), ("hidden", _i32), ("inter", _i32), ("experts", _i32),
                ("top_k", _i32), ("pdl", _i32)]


class MoeAllreduceArgs(C.Structure):
    _fields_ = [("partial", _vp), ("inbox", _vp * 8), ("flags", _vp * 8), ("epoch", _vp), ("status", _vp),
                ("residual", _vp), ("out", _vp), ("hidden", _i32), ("rank", _i32), ("world", _i32), ("has_shared", _i32),
                ("res_scale", _f32), ("pdl", _i32), ("residual_f32", _vp), ("out_f32", _vp), ("gate_logit", _vp)]


class PickAllgatherArgs(C.Structure):
    _fields_ = [("pair", _vp), ("inbox", _vp * 8), ("flags", _vp * 8), ("epoch", _vp), ("status", _vp), ("tokens", _vp),
                ("pos", _vp), ("picked", _vp), ("n_prompt", _i32), ("max_tokens", _i32), ("rank", _i32), ("world", _i32),
                ("pdl", _i32), ("reserved", _i32)]


class AttnMlaArgs(C.Structure):
    _fields_ = [("q_up", _vp), ("kv_up", _vp), ("k_rope", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("pos", _vp), ("rope_pos", _vp), ("k_pool", _vp), ("v_pool", _vp), ("block_table", _vp),
                ("out", _vp), ("k_new_out", _vp), ("v_new_out", _vp), ("part_o", _vp), ("part_ml", _vp),
                ("counters", _vp), ("heads", _i32), ("nope", _i32), ("rope", _i32), ("v", _i32),
                ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32), ("max_pos", _i32),
                ("scale", _f32), ("pdl", _i32)]


class MiniCPM3Layer(C.Structure):
    _fields_ = [(n, _vp) for n in ("gamma_in", "w_qkv_a", "gamma_q_a", "w_q_b", "gamma_kv_a", "w_kv_b", "w_o",
                                   "gamma_post", "w_gate", "w_up", "w_down", "k_pool", "v_pool")]


class MiniCPM3StepArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(MiniCPM3Layer)),
                ("n_layers", _i32), ("hidden", _i32), ("heads", _i32), ("q_lora", _i32), ("kv_lora", _i32),
                ("nope", _i32), ("rope", _i32), ("v", _i32), ("inter", _i32), ("vocab", _i64),
                ("eps", _f32), ("lora_eps", _f32), ("scale", _f32), ("embed_scale", _f32),
                ("residual_scale", _f32), ("logits_div", _f32),
                ("w_embed", _vp), ("gamma_final", _vp), ("w_head", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("max_pos", _i32), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("tokens", _vp), ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32),
                ("hidden_buf", _vp), ("qkv_a_buf", _vp), ("q_up_buf", _vp), ("kv_up_buf", _vp), ("attn_buf", _vp),
                ("act_buf", _vp), ("logits", _vp), ("part_o", _vp), ("part_ml", _vp), ("counters", _vp),
                ("head_val", _vp), ("head_idx", _vp), ("hidden_trace", _vp), ("picked", _vp), ("pdl", _i32),
                ("temperature", _f32), ("seed", _u64),
                ("eos_ids", _vp), ("stop_at", _vp), ("n_eos", _i32), ("reserved_eos", _i32),
                ("cache_layout", _i32), ("reserved_layout", _i32), ("q_lat_buf", _vp), ("q_rope_buf", _vp)]


class MiniCPM3PrefillArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(MiniCPM3Layer)),
                ("n_layers", _i32), ("m", _i32), ("hidden", _i32), ("heads", _i32), ("q_lora", _i32), ("kv_lora", _i32),
                ("nope", _i32), ("rope", _i32), ("v", _i32), ("inter", _i32), ("vocab", _i64),
                ("eps", _f32), ("lora_eps", _f32), ("scale", _f32), ("embed_scale", _f32), ("residual_scale", _f32),
                ("pdl", _i32), ("w_embed", _vp), ("cos_table", _vp), ("sin_table", _vp),
                ("max_pos", _i32), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("ids", _vp), ("pos_rows", _vp),
                ("hidden_buf", _vp), ("norm_buf", _vp), ("qkv_a_buf", _vp), ("attn_buf", _vp), ("act_buf", _vp),
                ("q_lat_buf", _vp), ("q_rope_buf", _vp), ("part_o", _vp), ("part_ml", _vp), ("status", _vp)]


class MlaLatentArgs(C.Structure):
    _fields_ = [("qkv_a", _vp), ("gamma_q_a", _vp), ("gamma_kv_a", _vp), ("w_q_b", _vp), ("w_kv_b", _vp),
                ("cos_table", _vp), ("sin_table", _vp), ("pos", _vp), ("rope_pos", _vp), ("pool", _vp),
                ("block_table", _vp), ("out", _vp), ("latent_new_out", _vp), ("q_lat", _vp), ("q_rope", _vp),
                ("part_o", _vp), ("part_ml", _vp), ("heads", _i32), ("q_lora", _i32), ("kv_lora", _i32),
                ("nope", _i32), ("rope", _i32), ("v", _i32), ("page_size", _i32), ("table_len", _i32),
                ("max_ctx", _i32), ("max_pos", _i32), ("scale", _f32), ("lora_eps", _f32), ("pdl", _i32),
                ("no_early_rows", _i32), ("tokens", _i32), ("reserved", _i32)]


MLA_CACHE_ASSEMBLED, MLA_CACHE_LATENT = 0, 1


class MoeDownArgs(C.Structure):
    _fields_ = [("w_down", _vp), ("w_shared", _vp), ("inner", _vp), ("shared_act", _vp), ("indices", _vp),
                ("weights", _vp), ("shared_gate", _vp), ("residual", _vp), ("out", _vp),
                ("hidden", _i32), ("inter", _i32), ("shared_inter", _i32), ("top_k", _i32),
                ("res_scale", _f32), ("pdl", _i32), ("expert_rank", _i32), ("expert_world", _i32), ("partial", _vp)]


class GraniteLayer(C.Structure):
    _fields_ = [("kind", _i32), ("pad", _i32)] + [(n, _vp) for n in (
        "gamma_in", "w_in", "conv_w", "conv_b", "a_log", "dt_bias", "d_skip", "gamma_ssm", "w_out", "conv_state",
        "ssm_state", "k_pool", "v_pool", "gamma_post", "w_router", "w_gate", "w_up", "w_down", "w_shared_in",
        "w_shared_out")]


class GraniteStepArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(GraniteLayer)), ("n_layers", _i32), ("hidden", _i32),
                ("nh", _i32), ("pd", _i32), ("ns", _i32), ("ng", _i32), ("conv_width", _i32),
                ("hq", _i32), ("hkv", _i32), ("d", _i32),
                ("experts", _i32), ("top_k", _i32), ("inter", _i32), ("shared_inter", _i32), ("vocab", _i64),
                ("eps", _f32), ("attn_scale", _f32), ("embed_scale", _f32), ("res_scale", _f32), ("logits_scale", _f32),
                ("table", _vp), ("gamma_final", _vp), ("page_size", _i32), ("table_len", _i32), ("max_ctx", _i32),
                ("block_table", _vp), ("tokens", _vp), ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32),
                ("hidden_buf", _vp), ("proj_buf", _vp), ("mixed_buf", _vp), ("y_buf", _vp), ("router_logits", _vp),
                ("router_idx", _vp), ("router_w", _vp), ("inner_buf", _vp), ("shared_buf", _vp), ("logits", _vp),
                ("part_o", _vp), ("part_ml", _vp), ("counters", _vp), ("head_val", _vp), ("head_idx", _vp),
                ("hidden_trace", _vp), ("idx_trace", _vp), ("picked", _vp), ("pdl", _i32),
                ("ep_rank", _i32), ("ep_world", _i32), ("partial", _vp), ("pair", _vp), ("gathered", _vp),
                ("temperature", _f32), ("seed", _u64),
                ("eos_ids", _vp), ("stop_at", _vp), ("n_eos", _i32), ("reserved_eos", _i32)]


#: every symbol ``include/tfb200.h`` declares: name -> (restype, argtypes)
class GemvF32Args(C.Structure):
    _fields_ = [("w", _vp), ("w2", _vp), ("w_extra", _vp), ("w2_extra", _vp), ("x", _vp), ("gamma", _vp), ("gate", _vp),
                ("residual", _vp), ("y", _vp), ("n", _i32), ("k", _i32), ("seg", _i32), ("prologue", _i32),
                ("epilogue", _i32), ("eps", _f32), ("expert_idx", _vp), ("rows_per_expert", _i32),
                ("routed_slots", _i32), ("pdl", _i32), ("reserved", _i32), ("route_counter", _vp), ("route_experts", _i32),
                ("route_top_k", _i32), ("idx_out", _vp), ("w_out", _vp), ("expert_rank", _i32), ("expert_world", _i32)]


class GdnArgs(C.Structure):
    _fields_ = [("proj", _vp), ("conv_state", _vp), ("conv_state_stride", _u64), ("pos", _vp), ("conv_w", _vp),
                ("a_log", _vp), ("dt_bias", _vp), ("state", _vp), ("read", _vp), ("hk", _i32), ("hv", _i32), ("dk", _i32),
                ("dv", _i32), ("kernel_width", _i32), ("q_scale", _f32), ("pdl", _i32), ("reserved", _i32),
                ("direct_q", _vp), ("direct_k", _vp), ("direct_v", _vp), ("direct_g", _vp), ("direct_beta", _vp)]


class AttnGatedArgs(C.Structure):
    _fields_ = [("proj", _vp), ("gamma_q", _vp), ("gamma_k", _vp), ("cos_table", _vp), ("sin_table", _vp), ("pos", _vp),
                ("rope_pos", _vp), ("k_pool", _vp), ("v_pool", _vp), ("block_table", _vp), ("out", _vp),
                ("k_new_out", _vp), ("v_new_out", _vp), ("part_o", _vp), ("part_ml", _vp), ("counters", _vp),
                ("hq", _i32), ("hkv", _i32), ("d", _i32), ("rotary_dim", _i32), ("page_size", _i32), ("table_len", _i32),
                ("max_ctx", _i32), ("max_pos", _i32), ("eps", _f32), ("scale", _f32), ("pdl", _i32), ("reserved", _i32)]


class MoeDownF32Args(C.Structure):
    _fields_ = [("w_down", _vp), ("w_shared", _vp), ("inner", _vp), ("indices", _vp), ("weights", _vp),
                ("shared_gate_logit", _vp), ("residual", _vp), ("out", _vp), ("hidden", _i32), ("inter", _i32),
                ("shared_inter", _i32), ("top_k", _i32), ("pdl", _i32), ("reserved", _i32), ("expert_rank", _i32),
                ("expert_world", _i32), ("partial", _vp)]


class Qwen35Layer(C.Structure):
    _fields_ = [("kind", _i32), ("reserved", _i32), ("gamma_in", _vp), ("w_in", _vp), ("w_out", _vp), ("conv_w", _vp),
                ("a_log", _vp), ("dt_bias", _vp), ("gamma_gdn", _vp), ("conv_state", _vp), ("state", _vp),
                ("gamma_q", _vp), ("gamma_k", _vp), ("k_pool", _vp), ("v_pool", _vp), ("gamma_post", _vp),
                ("w_router", _vp), ("w_gate", _vp), ("w_up", _vp), ("w_down", _vp), ("w_shared_gate", _vp),
                ("w_shared_up", _vp), ("w_shared_down", _vp)]


class Qwen35StepArgs(C.Structure):
    _fields_ = [("layers", C.POINTER(Qwen35Layer)), ("n_layers", _i32), ("pdl", _i32), ("table", _vp),
                ("gamma_final", _vp), ("w_head", _vp), ("cos_table", _vp), ("sin_table", _vp), ("tokens", _vp),
                ("pos", _vp), ("n_prompt", _i32), ("max_tokens", _i32), ("block_table", _vp), ("page_size", _i32),
                ("table_len", _i32), ("max_ctx", _i32), ("hidden", _i32), ("vocab", _i64), ("hk", _i32), ("hv", _i32),
                ("dk", _i32), ("dv", _i32), ("conv_width", _i32), ("hq", _i32), ("hkv", _i32), ("d", _i32),
                ("rotary_dim", _i32), ("experts", _i32), ("top_k", _i32), ("inter", _i32), ("shared_inter", _i32),
                ("conv_state_stride", _u64), ("eps", _f32), ("attn_scale", _f32), ("q_scale", _f32),
                ("hidden_buf", _vp), ("attended_buf", _vp), ("proj_buf", _vp), ("mixed_buf", _vp),
                ("router_logits", _vp), ("router_idx", _vp), ("router_w", _vp), ("inner_buf", _vp), ("part_o", _vp),
                ("part_ml", _vp), ("counters", _vp), ("head_val", _vp), ("head_idx", _vp), ("logits", _vp),
                ("picked", _vp), ("hidden_trace", _vp), ("idx_trace", _vp), ("ep_rank", _i32), ("ep_world", _i32),
                ("partial", _vp), ("pair", _vp), ("expert_prefetch", _i32), ("reserved", _i32),
                ("temperature", _f32), ("seed", _u64),
                ("eos_ids", _vp), ("stop_at", _vp), ("n_eos", _i32), ("reserved_eos", _i32)]


class RouterSelectArgs(C.Structure):
    _fields_ = [("logits_bf16", _vp), ("logits_f32", _vp), ("indices", _vp), ("weights_bf16", _vp), ("weights_f32", _vp),
                ("experts", _i32), ("top_k", _i32), ("mode", _i32), ("pdl", _i32), ("slab", _vp * 4), ("slab_bytes", _u64 * 4),
                ("n_slabs", _i32), ("expert_rank", _i32), ("expert_world", _i32), ("reserved", _i32)]


SYMBOLS = {
    "tfb_version": (_i32, []),
    "tfb_status_string": (C.c_char_p, [_i32]),
    "tfb_last_error": (C.c_char_p, []),
    "tfb_debug_trace": (_i32, [_vp, _i32]),
    "tfb_sample_top_p": (_i32, [C.POINTER(SampleTopPArgs), _vp]),
    "tfb_moe_batch": (_i32, [C.POINTER(MoeBatchArgs), _vp]),
    "tfb_moe_batch_route": (_i32, [C.POINTER(MoeRouteArgs), _vp]),
    "tfb_graph_step_host": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "tfb_graph_generate_host": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp, _vp]),
    "tfb_embed": (_i32, [_vp, _vp, _vp, _i32, _i32, _i64, _f32, _vp]),
    "tfb_rmsnorm": (_i32, [_vp, _vp, _vp, _i32, _i32, _f32, _i32, _vp]),
    "tfb_gemv": (_i32, [C.POINTER(GemvArgs), _vp]),
    "tfb_gemv_pair": (_i32, [C.POINTER(GemvArgs), C.POINTER(GemvArgs), _vp]),
    "tfb_gemv_chain": (_i32, [C.POINTER(GemvChainArgs), _vp]),
    "tfb_gemm_small_m_splits": (_i32, [_i32, _i32]),
    "tfb_gemm_small_m_swiglu_splits": (_i32, [_i32, _i32]),
    "tfb_gemm_small_m": (_i32, [C.POINTER(GemmSmallMArgs), _vp]),
    "tfb_qwen3_batch_decode_step": (_i32, [C.POINTER(Qwen3BatchStepArgs), _vp]),
    "tfb_qwen3_prefill_chunk": (_i32, [C.POINTER(Qwen3PrefillArgs), _vp]),
    "tfb_lm_head_scratch_entries": (_i32, [_i32]),
    "tfb_lm_head_argmax": (_i32, [C.POINTER(LmHeadArgs), _vp]),
    "tfb_attn_splits": (_i32, [_i32]),
    "tfb_attn_gqa_decode": (_i32, [C.POINTER(AttnGqaArgs), _vp]),
    "tfb_attn_gqa_decode_noalloc": (_i32, [C.POINTER(AttnGqaArgs), _vp]),
    "tfb_qwen3_decode_step": (_i32, [C.POINTER(Qwen3StepArgs), _vp]),
    "tfb_qwen3_step_sync_words": (_i32, [_i32, _i32]),
    "tfb_qwen3_step_splits": (_i32, [_i32]),
    "tfb_qwen3_step_xbuf_words": (_i64, [_i32, _i32, _i32, _i32, _i32]),
    "tfb_attn_mla_decode": (_i32, [C.POINTER(AttnMlaArgs), _vp]),
    "tfb_mla_latent_decode": (_i32, [C.POINTER(MlaLatentArgs), _vp]),
    "tfb_minicpm3_prefill_chunk": (_i32, [C.POINTER(MiniCPM3PrefillArgs), _vp]),
    "tfb_mla_latent_splits": (_i32, [_i32]),
    "tfb_minicpm3_decode_step": (_i32, [C.POINTER(MiniCPM3StepArgs), _vp]),
    "tfb_residual_add": (_i32, [_vp, _vp, _vp, _i32, _f32, _vp]),
    "tfb_conv_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "tfb_ssm_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp]),
    "tfb_router_select_prefetch": (_i32, [C.POINTER(RouterSelectArgs), _vp]),
    "tfb_router_select": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "tfb_moe_down": (_i32, [C.POINTER(MoeDownArgs), _vp]),
    "tfb_granite_decode_step": (_i32, [C.POINTER(GraniteStepArgs), _vp]),
    "tfb_granite_step_part": (_i32, [C.POINTER(GraniteStepArgs), _i32, _i32, _vp]),
    "tfb_moe_finalize": (_i32, [_vp, _vp, _vp, _i32, _f32, _i32, _i32, _vp]),
    "tfb_gemv_f32": (_i32, [C.POINTER(GemvF32Args), _vp]),
    "tfb_gdn_step": (_i32, [C.POINTER(GdnArgs), _vp]),
    "tfb_conv_silu_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "tfb_l2norm_f32": (_i32, [_vp, _vp, _i32, _i32, _f32, _i32, _vp]),
    "tfb_partial_rope_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "tfb_attn_gated_splits": (_i32, [_i32]),
    "tfb_attn_gated_groups": (_i32, [_i32, _i32, _i32]),
    "tfb_attn_gated_decode": (_i32, [C.POINTER(AttnGatedArgs), _vp]),
    "tfb_moe_down_f32": (_i32, [C.POINTER(MoeDownF32Args), _vp]),
    "tfb_embed_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _i64, _i32, _vp]),
    "tfb_rmsnorm_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _f32, _i32, _vp]),
    "tfb_residual_add_f32": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp]),
    "tfb_qwen35_decode_step": (_i32, [C.POINTER(Qwen35StepArgs), _vp]),
    "tfb_qwen35_step_part": (_i32, [C.POINTER(Qwen35StepArgs), _i32, _i32, _vp]),
    "tfb_moe_allreduce_finalize": (_i32, [C.POINTER(MoeAllreduceArgs), _vp]),
    "tfb_pick_allgather": (_i32, [C.POINTER(PickAllgatherArgs), _vp]),
    "tfb_pick_finalize": (_i32, [_vp, _i32, _vp, _vp, _i32, _i32, _vp, _i32, _vp]),
}


@lru_cache(maxsize=1)
def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m tilefoundry_b200.build` "
            "(needs nvcc). There is no fallback path."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        msg = lib.tfb_status_string(status).decode()
        detail = lib.tfb_last_error().decode()
        raise RuntimeError(f"{what}: status {status} ({msg})" + (f" [{detail}]" if detail else ""))


def ptr(t: "torch.Tensor | None") -> int | None:
    """Device address of a contiguous CUDA tensor (``None`` stays NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("kernel arguments must be CUDA tensors; there is no CPU path")
    if not t.is_contiguous():
        raise ValueError("kernel arguments must be contiguous")
    return t.data_ptr()


def stream() -> int:
    """torch's current stream, so launches order with the caller's work and can be graph-captured."""
    return torch.cuda.current_stream().cuda_stream


# ---- thin per-op helpers (all enqueue on the current stream) ----------------------

def embed(table, ids, out, scale=1.0):
    check(load().tfb_embed(ptr(table), ptr(ids), ptr(out), ids.numel(), table.shape[1], table.shape[0],
                           scale, stream()), "tfb_embed")
    return out


def rmsnorm(x, gamma, out, eps, mode):
    width = x.shape[-1]
    check(load().tfb_rmsnorm(ptr(x), ptr(gamma), ptr(out), x.numel() // width, width, eps, mode, stream()),
          "tfb_rmsnorm")
    return out


def gemv(w, x, y, *, w2=None, gamma=None, residual=None, prologue=NORM_NONE, epilogue=EPI_STORE,
         eps=0.0, x_scale=1.0, res_scale=1.0, out_scale=1.0, prefetch=None, pdl=False, kernel=0, self_prefetch=False, x_gate=None, expert_idx=None,
         rows_per_expert=0):
    n, k = w.shape[-2:]
    if expert_idx is not None:
        n = expert_idx.numel() * rows_per_expert
    a = GemvArgs(w=ptr(w), w2=ptr(w2), x=ptr(x), gamma=ptr(gamma), residual=ptr(residual), y=ptr(y),
                 n=n, k=k, prologue=prologue, epilogue=epilogue, eps=eps, x_scale=x_scale,
                 res_scale=res_scale, out_scale=out_scale,
                 prefetch=ptr(prefetch), prefetch_bytes=0 if prefetch is None else prefetch.numel() * prefetch.element_size(),
                 pdl=int(pdl), kernel=kernel, self_prefetch=int(self_prefetch), rows_per_expert=rows_per_expert,
                 expert_idx=ptr(expert_idx), x_gate=ptr(x_gate))
    check(load().tfb_gemv(C.byref(a), stream()), "tfb_gemv")
    return y


def attn_splits(max_ctx: int) -> int:
    return load().tfb_attn_splits(max_ctx)


def lm_head_scratch_entries(n: int) -> int:
    return load().tfb_lm_head_scratch_entries(n)
