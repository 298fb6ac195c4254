"""The batch-32 projection on the tensor cores (tcgen05 / TMEM / TMA) against a plain f32 reference of the same
product (torch, CPU): bf16 inputs, f32 accumulation, one rounding of the output."""
import ctypes as C

import pytest
import torch

from tests.helpers import assert_ulps

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


def _run(dev, w, x, residual=None, reps=1):
    from tilefoundry_b200 import lib
    m, k = x.shape
    n = w.shape[0]
    splits = lib.load().tfb_gemm_small_m_splits(n, k)
    y = torch.empty(m, n, device=dev, dtype=BF)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    assert splits in (1, 2, 4, 8)
    a = lib.GemmSmallMArgs(w=lib.ptr(w), x=lib.ptr(x), residual=lib.ptr(residual), y=lib.ptr(y), partial=None,
                           tickets=None, status=lib.ptr(status), m=m, n=n, k=k, pdl=0)
    for _ in range(reps):
        lib.check(lib.load().tfb_gemm_small_m(C.byref(a), lib.stream()), "tfb_gemm_small_m")
    torch.cuda.synchronize()
    assert int(status) == 0, f"a bounded wait gave up (role {int(status)})"
    return y


@pytest.mark.parametrize("m", [32, 17, 1])
@pytest.mark.parametrize("n,k", [(6144, 2048), (2048, 6144), (4096, 2048), (1000, 768), (128, 64)])
def test_small_batch_projection_matches_f32_reference(dev, m, n, k):
    g = torch.Generator().manual_seed(m * 131 + n + k)
    w = (torch.randn(n, k, generator=g) * k ** -0.5).to(BF)
    x = torch.randn(m, k, generator=g).to(BF)
    want = (x.float() @ w.float().t())
    got = _run(dev, w.to(dev), x.to(dev), reps=2)                 # twice: nothing carries over between launches
    assert_ulps(got.cpu(), want.to(BF), 1, f"y {m}x{n}x{k}")
    res = torch.randn(m, n, generator=g).to(BF)
    got = _run(dev, w.to(dev), x.to(dev), residual=res.to(dev))
    assert_ulps(got.cpu(), (res.float() + want.to(BF).float()).to(BF), 1, f"y + residual {m}x{n}x{k}")


def test_rows_agree_with_the_batch_1_projection(dev):
    """Row m of the batched product is the batch-1 projection of token m (same weights, same rounding point)."""
    from tilefoundry_b200 import lib
    g = torch.Generator().manual_seed(5)
    n, k, m = 4096, 2048, 32
    w = (torch.randn(n, k, generator=g) * k ** -0.5).to(BF).to(dev)
    x = torch.randn(m, k, generator=g).to(BF).to(dev)
    y = _run(dev, w, x)
    for row in (0, 13, 31):
        one = lib.gemv(w, x[row].contiguous(), torch.empty(n, device=dev, dtype=BF))
        assert_ulps(y[row], one, 1, f"token {row}")
