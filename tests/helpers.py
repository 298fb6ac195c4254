"""Shared test helpers: tolerances the reference's own tests use."""
import torch


def one_ulp_at(reference: torch.Tensor) -> float:
    """One representable step at the tensor's largest magnitude
    (reference ``tests/models/decode_oracle.py:42-54``)."""
    scale = reference.abs().max()
    up = torch.nextafter(scale, torch.full_like(scale, float("inf")))
    down = torch.nextafter(scale, torch.full_like(scale, float("-inf")))
    return max(abs((up - scale).item()), abs((scale - down).item()))


def assert_ulps(got, want, ulps, msg=""):
    assert got.dtype == want.dtype and got.shape == want.shape, (got.dtype, want.dtype, got.shape, want.shape)
    err = (got.float() - want.float()).abs().max().item()
    bound = ulps * one_ulp_at(want)
    assert err <= bound, f"{msg}: max err {err:.4g} > {ulps} ulp-at-scale = {bound:.4g}"


# the stated tolerance for bf16 hidden states and logits
RTOL = 2e-2
ATOL = 2e-2


def assert_close_at_scale(got, want, msg="", rtol=RTOL, atol=ATOL, min_cosine=1 - 2e-2):
    """End-to-end form of the same bound, as the reference's own kernel tests state it
    (``examples/qwen3_1_7b-tilelang/fast/test_kernels.py:18-29``): the largest error relative to
    the tensor's scale stays under rtol (plus atol), and the cosine stays above 1 - 2e-2.
    After a whole layer stack both sides carry bf16 rounding noise of a few ulp-at-scale on
    every element, including the ones near zero that a per-element rtol cannot excuse."""
    g, w = got.float().cpu().flatten(), want.float().cpu().flatten()
    err = (g - w).abs().max().item()
    bound = atol + rtol * w.abs().max().item()
    cos = torch.nn.functional.cosine_similarity(g, w, dim=0).item()
    assert err <= bound, f"{msg}: max err {err:.4g} > {bound:.4g} (atol + rtol*scale)"
    assert cos >= min_cosine, f"{msg}: cosine {cos:.6f} < {min_cosine}"


def assert_close_bf16(got, want, msg="", rtol=RTOL, atol=ATOL):
    g, w = got.float().cpu(), want.float().cpu()
    viol = ((g - w).abs() - (atol + rtol * w.abs())).max().item()
    assert viol <= 0, f"{msg}: allclose(rtol={rtol}, atol={atol}) violated by {viol:.4g}"


def assert_rel_l2(got, want, msg="", max_rel=2e-2, min_cosine=0.9995):
    """Aggregate bound for tensors that went through a deep stack: both implementations round to
    bf16 after every operation, so per-element differences random-walk with depth (a few
    ulp-at-scale after 28 layers) while the relative L2 distance and the direction stay tight."""
    g, w = got.float().cpu().flatten(), want.float().cpu().flatten()
    rel = ((g - w).norm() / w.norm().clamp_min(1e-12)).item()
    cos = torch.nn.functional.cosine_similarity(g, w, dim=0).item()
    assert rel <= max_rel, f"{msg}: rel_l2 {rel:.4g} > {max_rel}"
    assert cos >= min_cosine, f"{msg}: cosine {cos:.6f} < {min_cosine}"
