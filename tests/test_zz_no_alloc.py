"""The allocation-free attention entry point against the ordinary one, through the C ABI.

`tfb_attn_gqa_decode_noalloc` is for callers that cannot allocate device memory: a compiled entry
that receives only the tensors its ABI declares, or a serving loop that must not pay cudaMalloc's
device-wide synchronisation.  It keeps its split-KV scratch in an array inside the library instead of
taking it from the caller.  Both entry points launch the same kernel, so their outputs must be equal
bit for bit; the check is made on two calls in a row because the built-in array is shared and keeps
what the previous call left in it.  This file is collected last on purpose: if it fails, a run that
stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _args(lib, dev, ctx, seed, hq=16, hkv=8, d=128, max_ctx=700):
    from tilefoundry_b200.engine import paged_kv
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g).to(BF).to(dev)
    nsplit = lib.attn_splits(max_ctx)
    t = {
        "qkv": rnd((hq + 2 * hkv) * d), "gq": (1 + 0.1 * torch.randn(d, generator=g)).to(BF).to(dev),
        "gk": (1 + 0.1 * torch.randn(d, generator=g)).to(BF).to(dev),
        "cos": torch.cos(torch.rand(max_ctx, d, generator=g) * 6.28).to(BF).to(dev),
        "sin": torch.sin(torch.rand(max_ctx, d, generator=g) * 6.28).to(BF).to(dev),
        "pos": torch.tensor([ctx], dtype=torch.int32, device=dev),
        "table": paged_kv.block_table(1, max_ctx, device=dev),
        "k_pool": paged_kv.new_pool(1, max_ctx, hkv, d, device=dev),
        "v_pool": paged_kv.new_pool(1, max_ctx, hkv, d, device=dev),
        "out": torch.zeros(hq * d, dtype=BF, device=dev),
        "part_o": torch.zeros(hq * nsplit * d, dtype=torch.float32, device=dev),
        "part_ml": torch.zeros(hq * nsplit * 2, dtype=torch.float32, device=dev),
        "counters": torch.zeros(hkv, dtype=torch.int32, device=dev),
    }
    t["k_pool"].view(-1, hkv, d)[:ctx] = rnd(ctx, hkv, d)
    t["v_pool"].view(-1, hkv, d)[:ctx] = rnd(ctx, hkv, d)
    a = lib.AttnGqaArgs(
        qkv=lib.ptr(t["qkv"]), gamma_q=lib.ptr(t["gq"]), gamma_k=lib.ptr(t["gk"]), cos_table=lib.ptr(t["cos"]),
        sin_table=lib.ptr(t["sin"]), pos=lib.ptr(t["pos"]), k_pool=lib.ptr(t["k_pool"]), v_pool=lib.ptr(t["v_pool"]),
        block_table=lib.ptr(t["table"]), out=lib.ptr(t["out"]), part_o=lib.ptr(t["part_o"]),
        part_ml=lib.ptr(t["part_ml"]), counters=lib.ptr(t["counters"]), hq=hq, hkv=hkv, d=d, rotary_dim=d,
        page_size=paged_kv.PAGE_SIZE, table_len=t["table"].shape[1], max_ctx=max_ctx, max_pos=max_ctx, eps=1e-6,
        scale=d ** -0.5, norm_mode=lib.NORM_CAST_THEN_GAIN, pdl=0)
    return a, t


def test_noalloc_attention_equals_caller_scratch_attention_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    handle = lib.load()
    dev = torch.device("cuda:0")
    for call, (ctx, seed) in enumerate([(500, 1), (131, 2), (64, 3)]):   # calls in a row, different shapes of work
        a, t = _args(lib, dev, ctx, seed)
        lib.check(handle.tfb_attn_gqa_decode(C.byref(a), lib.stream()), "tfb_attn_gqa_decode")
        torch.cuda.synchronize()
        want = t["out"].clone()
        k_row = t["k_pool"].view(-1, 8, 128)[ctx].clone()
        b, u = _args(lib, dev, ctx, seed)                          # same inputs, fresh buffers
        b.part_o = b.part_ml = b.counters = None                   # the entry point must not need them
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(dev), torch.cuda.mem_get_info(dev)[0]
        lib.check(handle.tfb_attn_gqa_decode_noalloc(C.byref(b), lib.stream()), "tfb_attn_gqa_decode_noalloc")
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        # the driver's own count of free device memory: a raw cudaMalloc inside the library would show here,
        # where torch's allocator statistics cannot see it
        # (judged from the second call on: the first may load the library's module and symbol lazily)
        assert call == 0 or torch.cuda.mem_get_info(dev)[0] == free_before, f"call {call}: device memory was allocated"
        assert torch.equal(u["out"], want), f"call {call}: outputs differ"
        assert torch.equal(u["k_pool"].view(-1, 8, 128)[ctx], k_row), f"call {call}: appended key differs"
        assert float(want.float().abs().sum()) > 0


def test_noalloc_rejects_shapes_beyond_the_built_in_scratch():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    handle = lib.load()
    a, _ = _args(lib, torch.device("cuda:0"), 10, 3, max_ctx=5000)  # 79 splits > 64
    status = handle.tfb_attn_gqa_decode_noalloc(C.byref(a), lib.stream())
    assert status == 3                                              # TFB_ECAPACITY
    assert b"exceeds the built-in scratch" in handle.tfb_last_error()
