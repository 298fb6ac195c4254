"""Parity of the CUDA path against the CPU oracle -- granite-4.0-h (Mamba-2 + attention hybrid, MoE)."""
import pytest
import torch

from oracle import evaluator, generation, granite_4_0_h_small as og
from tests import parity
from tests.helpers import ATOL, RTOL, assert_close_at_scale
from tilefoundry_b200.authored import granite_4_0_h_small as gr
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import AllClose, DictResource, Equal, NanInf, check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
CLOSE = [AllClose(atol=ATOL, rtol=RTOL), NanInf()]
STATE = [AllClose(atol=1e-3, rtol=1e-3), NanInf()]          # fp32 recurrent state


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


def _sides(cfg, dev, seed=3, std=0.05):
    from tilefoundry_b200.twins.granite_4_0_h_small import make_twin
    mod = gr.build(cfg)
    weights = random_weights(mod, seed=seed, std=std, overrides=gr.weight_overrides)
    ref = evaluator.load(mod, DictResource(weights), og.make(cfg))
    twin = make_twin(cfg)()
    twin.load(DictResource(parity.cuda_weights(weights, dev)))
    return ref, twin, weights


def _check(twin_fn, ref_fn, inputs, expect):
    rep = check(lambda *a: parity.to_cpu(twin_fn(*a)), parity.on_cpu(ref_fn), inputs, expect=expect)
    assert rep.passed, rep.render()


def test_mamba_functions(dev):
    cfg = gr.GRANITE_TINY
    ref, twin, _ = _sides(cfg, dev)
    g = torch.Generator().manual_seed(5)
    r = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale)
    NH, PD, NS, NG = cfg.mamba_n_heads, cfg.mamba_d_head, cfg.mamba_d_state, cfg.mamba_n_groups
    hidden = r(1, 1, cfg.hidden_size).to(BF).to(dev)
    conv_state = r(1, cfg.conv_dim, 3).to(BF).to(dev)
    entry = r(1, cfg.conv_dim, 1).to(BF).to(dev)
    ssm_state = r(1, NH, PD, NS, scale=0.5).to(dev)
    rm, tm = ref.layer0.mixer, twin.layer0.mixer
    _check(tm.in_projection, rm.in_projection, (hidden,), {"output": CLOSE})
    _check(tm.conv_step, rm.conv_step, (conv_state, entry), {"output": CLOSE})
    ssm_in = (ssm_state, r(1, NH, PD).to(BF).to(dev), r(1, NG, NS).to(BF).to(dev), r(1, NG, NS).to(BF).to(dev),
              r(1, NH).to(BF).to(dev))
    _check(tm.ssm_step, rm.ssm_step, ssm_in, {"output[0]": CLOSE, "output[1]": STATE})
    _check(tm.gated_out, rm.gated_out, (r(1, NH, PD).to(BF).to(dev), r(1, cfg.expand).to(BF).to(dev)), {"output": CLOSE})
    _check(tm.mamba_mixer, rm.mamba_mixer, (hidden, conv_state, ssm_state),
           {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": STATE})
    # inputs were not mutated
    assert torch.equal(ssm_state.cpu(), ssm_in[0].cpu())


@pytest.mark.parametrize("step", [0, 1, 63, 64, 130])
def test_attention_functions(dev, step):
    cfg = gr.GRANITE_TINY
    ref, twin, _ = _sides(cfg, dev)
    g = torch.Generator().manual_seed(step)
    HKV, D, CAP = cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
    kc = torch.zeros(1, CAP, HKV, D, dtype=BF)
    vc = torch.zeros(1, CAP, HKV, D, dtype=BF)
    kc[:, :step] = torch.randn(1, step, HKV, D, generator=g).to(BF)
    vc[:, :step] = torch.randn(1, step, HKV, D, generator=g).to(BF)
    cur = torch.tensor([step], dtype=torch.int32)
    mask = gr.attention_mask(cfg, step)
    ra, ta = ref.layer2.mixer, twin.layer2.mixer
    _check(ta.qkv, ra.qkv, (hidden,), {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})
    inputs = tuple(t.to(dev) for t in (hidden, kc, vc, cur, mask))
    _check(ta.full_attention, ra.full_attention, inputs, {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})
    q = torch.randn(1, 1, cfg.num_attention_heads, D, generator=g).to(BF)
    kc[:, step] = torch.randn(HKV, D, generator=g).to(BF)
    vc[:, step] = torch.randn(HKV, D, generator=g).to(BF)
    _check(ta.attend, ra.attend, tuple(t.to(dev) for t in (q, kc, vc, cur, mask)), {"output": CLOSE})


def test_moe_functions_and_routing_indices(dev):
    cfg = gr.GRANITE_TINY
    ref, twin, _ = _sides(cfg, dev)
    g = torch.Generator().manual_seed(9)
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
    rm, tm = ref.layer0.moe, twin.layer0.moe
    _check(tm.post_norm, rm.post_norm, (hidden,), {"output": CLOSE})
    tokens = rm.post_norm(hidden.cpu())
    # routing: integer output, bit-exact; weights within tolerance
    _check(tm.router.routing, rm.router.routing, (tokens.to(dev),), {"output[0]": CLOSE, "output[1]": [Equal()]})
    weights, indices = rm.router.routing(tokens)
    args = tuple(t.to(dev) for t in (tokens, weights, indices))
    _check(tm.routed_experts, rm.routed_experts, args, {"output": CLOSE})
    _check(tm.shared_mlp, rm.shared_mlp, (tokens.to(dev),), {"output": CLOSE})
    _check(tm.experts, rm.experts, args, {"output": CLOSE})
    _check(tm, rm, (hidden,), {"output": CLOSE})                 # the block's own forward
    a, b = hidden, torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
    _check(twin.layer0.residual_add, ref.layer0.residual_add, (a, b), {"output": CLOSE})


def test_router_select_modes_and_ties(dev):
    from tilefoundry_b200 import lib
    E, K = 72, 10
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(E, generator=g).to(BF)
    logits[40] = logits[7]                                        # an exact tie: lower index first
    idx, w = torch.zeros(K, dtype=torch.int64, device=dev), torch.zeros(K, dtype=BF, device=dev)
    lib.check(lib.load().tfb_router_select(lib.ptr(logits.to(dev)), None, lib.ptr(idx), lib.ptr(w), None, E, K, 0, 0,
                                           lib.stream()), "router")
    vals, ref_idx = torch.topk(logits.float(), K)
    got = idx.cpu().tolist()
    assert sorted(got) == sorted(ref_idx.tolist())
    assert torch.equal(logits.float()[idx.cpu()], vals)           # same values in the same order
    if 7 in got and 40 in got:
        assert got.index(7) < got.index(40)
    assert_close_at_scale(w, torch.softmax(vals, -1).to(BF), "router weights", rtol=1e-2, atol=1e-3)
    # mode 1: softmax over all experts, top-k, renormalise (f32)
    E2, K2 = 256, 8
    lg = torch.randn(E2, generator=g)
    idx2, w2 = torch.zeros(K2, dtype=torch.int64, device=dev), torch.zeros(K2, dtype=torch.float32, device=dev)
    lib.check(lib.load().tfb_router_select(None, lib.ptr(lg.to(dev)), lib.ptr(idx2), None, lib.ptr(w2), E2, K2, 1, 0,
                                           lib.stream()), "router")
    pv, pi = torch.topk(torch.softmax(lg, -1), K2)
    assert idx2.cpu().tolist() == pi.tolist()
    torch.testing.assert_close(w2.cpu(), pv / pv.sum(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("use_graph", [False, True])
def test_session_matches_evaluator_tiny(dev, use_graph):
    """Teacher-forced run of the whole hybrid stack: logits and hidden states within the end-to-end bound,
    routing indices of every layer bit-exact wherever the router logits are not tied within noise,
    fp32 recurrent state within 1e-3, KV cache and page table as the evaluator built them."""
    from tilefoundry_b200.engine.granite import GraniteSession
    from tilefoundry_b200.engine import paged_kv
    cfg = gr.GRANITE_TINY
    mod = gr.build(cfg)
    weights = random_weights(mod, seed=11, std=0.05, overrides=gr.weight_overrides)
    ref = evaluator.load(mod, DictResource(weights), og.make(cfg))
    n_prompt, n_new = 16, 80
    prompt = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(111))
    want = generation.decode_ids(ref, prompt, n_new, keep_logits=True)
    forced = torch.cat([prompt, torch.tensor(want["tokens"], dtype=torch.int64)])
    sess = GraniteSession(cfg, DictResource(parity.cuda_weights(weights, dev)), max_ctx=n_prompt + n_new + 5, device=dev,
                          keep_logits=True, trace_hidden=True)
    sess.reset(forced)
    if use_graph:
        sess.capture()
    total = n_prompt + n_new - 1
    mismatched_picks = 0
    for step in range(total):
        sess.run(1, use_graph)
        ref_logits = want["logits"][step][0]
        assert_close_at_scale(sess.logits, ref_logits, f"logits step {step}")
        if int(sess.picked) != int(torch.argmax(ref_logits)):
            top = torch.topk(ref_logits.float(), 2).values
            noise = (sess.logits.float().cpu() - ref_logits.float()).abs().max()
            assert float(top[0] - top[1]) <= 2 * float(noise), f"pick differs at step {step}"
            mismatched_picks += 1
    assert mismatched_picks <= 6
    assert int(sess.pos) == total
    # state after the walk
    assert torch.equal(sess.table.cpu(), paged_kv.block_table(1, sess.max_ctx))
    for li, (kind, state) in enumerate(zip(cfg.layer_types, want["caches"])):
        layer = sess.layers[li]
        if kind == "linear_attention":
            window, matrix = state
            assert_close_at_scale(layer["conv_state"], window[0], f"layer {li} conv window")
            torch.testing.assert_close(layer["ssm_state"].cpu(), matrix[0], rtol=2e-2, atol=2e-2,
                                       msg=lambda m: f"layer {li} ssm state after {total} steps: {m}")
        else:
            k_ref, v_ref = state
            assert_close_at_scale(paged_kv.logical_view(layer["k_pool"], sess.table[0], total), k_ref[:, :total],
                                  f"layer {li} K cache")
            assert_close_at_scale(paged_kv.logical_view(layer["v_pool"], sess.table[0], total), v_ref[:, :total],
                                  f"layer {li} V cache")
