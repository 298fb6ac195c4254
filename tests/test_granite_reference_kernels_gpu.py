"""The granite evaluator restatement (``oracle/granite_4_0_h_small.py``) against the REFERENCE's own CUDA C kernels
(``examples/granite_4_0_h_small-cuda/kernels/granite.cu``, built unmodified for sm_100a by ``oracle/build_ref.py``
into ``oracle/_ref``), at the published widths, on the GPU: every ``@func`` the kernels implement is run by both and
compared under the bounds of the other parity tests (2e-2 of the tensor's scale, f32 state 1e-3, routing indices
exact).  This is the pin that makes the granite oracle reference-held; it also prints what the reference's kernels
take on this GPU for the shapes its README quotes (``README.md:233-244``)."""
import pytest
import torch

from oracle import build_ref, granite_4_0_h_small as og
from tests.helpers import assert_close_at_scale
from tilefoundry_b200.authored import granite_4_0_h_small as gr

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
CFG = gr.truncated(gr.GRANITE_4_0_H_SMALL, num_hidden_layers=2, attention_layers=(0,), vocab_size=1024, max_ctx=512)


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    mod = build_ref.load_built()
    if mod is None:
        pytest.skip("oracle/_ref/granite/granite_ref_kernels.so is not built (python -m oracle.build_ref, where the "
                    "reference checkout is mounted)")
    return mod


@pytest.fixture(scope="module")
def F():
    """The restated function bodies by name, gathered over one layer of each kind."""
    impl_for, table = og.make(CFG), {}

    def gather(module):
        table.update(impl_for(module))
        for child in module.modules:
            gather(child)

    gather(gr.build(CFG))
    return table


def _r(g, *shape, scale=1.0, dtype=BF):
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def _time(fn, reps=20):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def test_in_projection_and_gated_out(K, F):
    dev, g = torch.device("cuda:0"), torch.Generator().manual_seed(1)
    H, PROJ, EXP, EPS = CFG.hidden_size, CFG.proj, CFG.expand, CFG.rms_norm_eps
    hidden, gamma, w_in = _r(g, 1, 1, H), (1 + _r(g, H, scale=0.02).float()).to(BF), _r(g, PROJ, H, scale=0.02)
    xn, proj = torch.empty(H, dtype=BF, device=dev), torch.empty(PROJ, dtype=BF, device=dev)
    K.rms_norm(hidden.reshape(-1).to(dev), gamma.to(dev), xn, EPS)
    K.gemv(w_in.to(dev), xn, proj)
    assert_close_at_scale(proj, F["in_projection"](hidden, gamma, w_in).reshape(-1), "in_projection")
    y, gate = _r(g, 1, CFG.mamba_n_heads, CFG.mamba_d_head), _r(g, 1, EXP)
    gamma_s, w_out = (1 + _r(g, EXP, scale=0.02).float()).to(BF), _r(g, H, EXP, scale=0.02)
    yn, out = torch.empty(EXP, dtype=BF, device=dev), torch.empty(H, dtype=BF, device=dev)
    K.rms_norm_gated(y.reshape(-1).to(dev), gate.reshape(-1).to(dev), gamma_s.to(dev), yn, EPS)
    K.gemv(w_out.to(dev), yn, out)
    assert_close_at_scale(out, F["gated_out"](y, gate, gamma_s, w_out).reshape(-1), "gated_out")
    w_dev = w_in.to(dev)
    print(f"\nreference gemv, in_projection {PROJ}x{H}: {_time(lambda: K.gemv(w_dev, xn, proj)):.1f} us (L2-warm)")


def test_conv_and_ssm_steps(K, F):
    dev, g = torch.device("cuda:0"), torch.Generator().manual_seed(2)
    NH, PD, NS, CONVD = CFG.mamba_n_heads, CFG.mamba_d_head, CFG.mamba_d_state, CFG.conv_dim
    state, entry = _r(g, 1, CONVD, 3), _r(g, 1, CONVD, 1)
    conv_w, conv_b = _r(g, CONVD, 4, scale=0.3), _r(g, CONVD, scale=0.1)
    st_dev, out = state[0].contiguous().to(dev), torch.empty(CONVD, dtype=BF, device=dev)
    K.mamba_conv(st_dev, entry.reshape(-1).to(dev), conv_w.to(dev), conv_b.to(dev), out)
    assert_close_at_scale(out, F["conv_step"](state, entry, conv_w, conv_b).reshape(-1), "conv_step")
    assert torch.equal(st_dev.cpu(), torch.cat([state, entry], 2)[0, :, -3:])          # the window slid in place
    ssm = _r(g, 1, NH, PD, NS, scale=0.5, dtype=torch.float32)
    x, b_vec, c_vec, dt_raw = _r(g, 1, NH, PD), _r(g, 1, 1, NS), _r(g, 1, 1, NS), _r(g, 1, NH)
    a_log = torch.log(1 + 15 * torch.rand(NH, generator=g)).to(BF)
    dt_bias, d_skip = _r(g, NH, scale=0.5), torch.ones(NH, dtype=BF)
    ssm_dev, y = ssm[0].contiguous().to(dev), torch.empty(NH * PD, dtype=BF, device=dev)
    K.mamba_ssm(ssm_dev, x.reshape(-1).to(dev), b_vec.reshape(-1).to(dev), c_vec.reshape(-1).to(dev),
                dt_raw.reshape(-1).to(dev), a_log.to(dev), dt_bias.to(dev), d_skip.to(dev), y)
    want_y, want_state = F["ssm_step"](ssm, x, b_vec, c_vec, dt_raw, a_log, dt_bias, d_skip)
    assert_close_at_scale(y, want_y.reshape(-1), "ssm_step y")
    torch.testing.assert_close(ssm_dev.cpu(), want_state[0], rtol=1e-3, atol=1e-3)     # the f32 recurrent state


def test_routing_and_experts(K, F):
    dev, g = torch.device("cuda:0"), torch.Generator().manual_seed(3)
    H, E, TOPK, I = CFG.hidden_size, CFG.num_local_experts, CFG.num_experts_per_tok, CFG.intermediate_size
    w_router = _r(g, E, H, scale=0.02)
    for trial in range(6):
        tokens = _r(g, 1, H)
        logits = torch.empty(E, dtype=torch.float32, device=dev)
        K.gemv_f32(w_router.to(dev), tokens.reshape(-1).to(dev), logits, 1.0)
        wts, idx = torch.empty(TOPK, dtype=BF, device=dev), torch.empty(TOPK, dtype=torch.int64, device=dev)
        K.topk_softmax(logits, wts, idx)
        want_w, want_idx = F["routing"](tokens, w_router)
        ref_logits = torch.matmul(tokens, w_router.t()).float().reshape(-1)
        diff = (idx.cpu() != want_idx.reshape(-1)).nonzero().flatten().tolist()
        for i in diff:                                     # a different expert only where the two logits are equal
            assert float(ref_logits[idx[i]]) == float(ref_logits[want_idx.reshape(-1)[i]]), (trial, idx.tolist(), want_idx.tolist())
        assert_close_at_scale(wts, want_w.reshape(-1), f"routing weights, trial {trial}")
    w_gate, w_up, w_down = _r(g, E, I, H, scale=0.02), _r(g, E, I, H, scale=0.02), _r(g, E, H, I, scale=0.02)
    both, h = torch.empty(TOPK * 2 * I, dtype=BF, device=dev), torch.empty(TOPK * I, dtype=BF, device=dev)
    wg, wu, wd, tok = w_gate.to(dev), w_up.to(dev), w_down.to(dev), tokens.reshape(-1).to(dev)
    K.experts_gate_up(wg, wu, tok, idx, both, h)
    partial, out = torch.empty(TOPK * H, dtype=torch.float32, device=dev), torch.empty(H, dtype=BF, device=dev)
    K.experts_down(wd, h, idx, wts, partial, out)
    want = F["routed_experts"](tokens, wts.cpu().reshape(1, TOPK), idx.cpu().reshape(1, TOPK), w_gate, w_up, w_down)
    assert_close_at_scale(out, want.reshape(-1), "routed_experts")
    print(f"\nreference experts_gate_up ({TOPK} of {E} experts, {2 * I}x{H} each): "
          f"{_time(lambda: K.experts_gate_up(wg, wu, tok, idx, both, h)):.1f} us (L2-warm)")


@pytest.mark.parametrize("step", [7, 15, 63, 64, 300])
def test_attention(K, F, step):
    """Lengths at which every one of the reference kernel's eight position stripes holds a position.  With an empty
    stripe (7 * ceil(len / 8) >= len, which only lengths below 50 can meet) its partial is exp(-inf - -inf) and the
    combine's ``gs > 0`` test then writes zeros for the head, so those lengths say nothing about the oracle."""
    dev, g = torch.device("cuda:0"), torch.Generator().manual_seed(step)
    cfg = CFG
    HQ, HKV, D, CAP, H = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx, cfg.hidden_size
    q = _r(g, 1, 1, HQ, D)
    kc, vc = torch.zeros(1, CAP, HKV, D, dtype=BF), torch.zeros(1, CAP, HKV, D, dtype=BF)
    kc[:, :step + 1], vc[:, :step + 1] = _r(g, 1, step + 1, HKV, D), _r(g, 1, step + 1, HKV, D)
    w_o = _r(g, H, HQ * D, scale=0.02)
    cur = torch.tensor([step], dtype=torch.int32)
    part_acc = torch.empty(HQ * 8 * D, dtype=torch.float32, device=dev)
    part_ms = torch.empty(HQ * 8 * 2, dtype=torch.float32, device=dev)
    attn, out = torch.empty(HQ * D, dtype=BF, device=dev), torch.empty(H, dtype=BF, device=dev)
    K.attn_decode(q.reshape(-1).to(dev), kc[0].reshape(CAP, -1).to(dev), vc[0].reshape(CAP, -1).to(dev), cur.to(dev),
                  part_acc, part_ms, attn, HQ, HKV, cfg.attention_multiplier)
    K.gemv(w_o.to(dev), attn, out)
    want = F["attend"](q, kc, vc, cur, gr.attention_mask(cfg, step), w_o)
    assert_close_at_scale(out, want.reshape(-1), f"attend at position {step}")
