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

# The published widths on a stack cut to two Mamba-2 layers and one attention layer and a 4096-entry vocabulary:
# hidden 4096, 128 heads x 64 with d_state 128, 72 experts top-10 of 768, shared 1536, 32 q / 8 kv heads x 128.
# Every kernel is instantiated by these widths, not by the depth, so this is the configuration the benchmark runs.
WIDE = gr.truncated(gr.GRANITE_4_0_H_SMALL, num_hidden_layers=3, attention_layers=(2,), vocab_size=4096, max_ctx=256)
CONFIGS = {"tiny": (gr.GRANITE_TINY, 0.05), "wide": (WIDE, 0.02)}


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


@pytest.fixture(scope="module", params=["tiny", "wide"])
def sides(request, dev):
    """(config, evaluator side, twin, host weights, device weights); pytest groups the tests by configuration, so
    each configuration's weights are drawn once and dropped before the next is built."""
    from tilefoundry_b200.twins.granite_4_0_h_small import make_twin
    cfg, std = CONFIGS[request.param]
    mod = gr.build(cfg)
    weights = random_weights(mod, seed=3, std=std, overrides=gr.weight_overrides)
    on_dev = parity.cuda_weights(weights, dev)
    ref = evaluator.load(mod, DictResource(weights), og.make(cfg))
    twin = make_twin(cfg)()
    twin.load(DictResource(on_dev))
    yield cfg, ref, twin, weights, on_dev
    del ref, twin, weights, on_dev
    torch.cuda.empty_cache()


def _check(twin_fn, ref_fn, inputs, expect):
    rep = check(lambda *a: parity.to_cpu(twin_fn(*a)), parity.on_cpu(ref_fn), inputs, expect=expect)
    assert rep.passed, rep.render()


def test_mamba_functions(dev, sides):
    cfg, ref, twin = sides[:3]
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
    # the f32 state carried over several tokens, each step from the evaluator's own state: 1e-3 at every step
    state = ssm_state
    for _ in range(6):
        step_in = (state, r(1, NH, PD).to(BF).to(dev), r(1, NG, NS).to(BF).to(dev), r(1, NG, NS).to(BF).to(dev),
                   r(1, NH).to(BF).to(dev))
        _check(tm.ssm_step, rm.ssm_step, step_in, {"output[0]": CLOSE, "output[1]": STATE})
        state = rm.ssm_step(*[t.cpu() for t in step_in])[1].to(dev)
    _check(tm.gated_out, rm.gated_out, (r(1, NH, PD).to(BF).to(dev), r(1, cfg.expand).to(BF).to(dev)), {"output": CLOSE})
    _check(tm.mamba_mixer, rm.mamba_mixer, (hidden, conv_state, ssm_state),
           {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": STATE})
    # inputs were not mutated
    assert torch.equal(ssm_state.cpu(), ssm_in[0].cpu())


@pytest.mark.parametrize("step", [0, 1, 63, 64, 130])
def test_attention_functions(dev, sides, step):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(step)
    HKV, D, CAP = cfg.num_key_value_heads, cfg.head_dim, cfg.max_ctx
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
    kc = torch.zeros(1, CAP, HKV, D, dtype=BF)
    vc = torch.zeros(1, CAP, HKV, D, dtype=BF)
    kc[:, :step] = torch.randn(1, step, HKV, D, generator=g).to(BF)
    vc[:, :step] = torch.randn(1, step, HKV, D, generator=g).to(BF)
    cur = torch.tensor([step], dtype=torch.int32)
    mask = gr.attention_mask(cfg, step)
    ai = cfg.attention_layers[0]
    ra, ta = getattr(ref, f"layer{ai}").mixer, getattr(twin, f"layer{ai}").mixer
    _check(ta.qkv, ra.qkv, (hidden,), {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})
    inputs = tuple(t.to(dev) for t in (hidden, kc, vc, cur, mask))
    _check(ta.full_attention, ra.full_attention, inputs, {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})
    q = torch.randn(1, 1, cfg.num_attention_heads, D, generator=g).to(BF)
    kc[:, step] = torch.randn(HKV, D, generator=g).to(BF)
    vc[:, step] = torch.randn(HKV, D, generator=g).to(BF)
    _check(ta.attend, ra.attend, tuple(t.to(dev) for t in (q, kc, vc, cur, mask)), {"output": CLOSE})


def test_moe_functions_and_routing_indices(dev, sides):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(9)
    rm, tm = ref.layer0.moe, twin.layer0.moe
    for trial in range(4):                                       # routing is an integer output: several token vectors
        hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
        _check(tm.post_norm, rm.post_norm, (hidden,), {"output": CLOSE})
        tokens = rm.post_norm(hidden.cpu())
        # routing: an integer output -- the experts bit-exact, slot by slot, except where two router logits are
        # exactly equal (their order is not determined); weights within tolerance
        got_w, got_idx = tm.router.routing(tokens.to(dev))
        want_w, want_idx = rm.router.routing(tokens)
        w_r = rm.router.constants["w_router"]
        w_r = w_r if w_r.shape[0] == tokens.shape[-1] else w_r.t()
        parity.assert_same_routing(got_idx, want_idx, torch.matmul(tokens.to(w_r.dtype), w_r), f"trial {trial}")
        assert got_idx.dtype == want_idx.dtype and got_w.dtype == want_w.dtype and got_w.shape == want_w.shape
        assert_close_at_scale(got_w, want_w, f"routing weights, trial {trial}")
    weights, indices = rm.router.routing(tokens)
    args = tuple(t.to(dev) for t in (tokens, weights, indices))
    _check(tm.routed_experts, rm.routed_experts, args, {"output": CLOSE})
    _check(tm.shared_mlp, rm.shared_mlp, (tokens.to(dev),), {"output": CLOSE})
    _check(tm.experts, rm.experts, args, {"output": CLOSE})
    _check(tm, rm, (hidden,), {"output": CLOSE})                 # the block's own forward
    a, b = hidden, torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF).to(dev)
    _check(twin.layer0.residual_add, ref.layer0.residual_add, (a, b), {"output": CLOSE})


def test_root_functions(dev, sides):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(2)
    ids = torch.tensor([cfg.vocab_size - 1])
    assert torch.equal(twin.embed(ids.to(dev)).cpu(), ref.embed(ids))
    hidden = torch.randn(1, 1, cfg.hidden_size, generator=g).to(BF)
    _check(twin.final_rms_norm, ref.final_rms_norm, (hidden.to(dev),), {"output": CLOSE})
    normed = ref.final_rms_norm(hidden)
    _check(twin.lm_head, ref.lm_head, (normed.to(dev),), {"output": CLOSE})


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


# A routing pick is decided by bf16 router logits computed from inputs that already differ by the arithmetic noise
# of the layers below: two logits closer than this (two bf16 steps at the logits' magnitude) may legitimately
# come out in the other order.
TIE_MARGIN = 3e-2


def cfg_is_tiny(cfg):
    return cfg.hidden_size < 1024


def _session(cfg, on_dev, dev, cap):
    from tilefoundry_b200.engine.granite import GraniteSession
    return GraniteSession(cfg, DictResource(on_dev), max_ctx=cap, device=dev, keep_logits=True, trace_hidden=True)


def _walk_lengths(cfg):
    return (16, 80) if cfg_is_tiny(cfg) else (64, 32)      # the wide stack: 64 prompt ids + 32 new tokens


def _forced_tokens(cfg, ref, seed=111):
    n_prompt, n_new = _walk_lengths(cfg)
    prompt = torch.randint(0, cfg.vocab_size, (n_prompt,), generator=torch.Generator().manual_seed(seed))
    want = generation.decode_ids(ref, prompt, n_new, keep_logits=True)
    return want, torch.cat([prompt, torch.tensor(want["tokens"], dtype=torch.int64)]), n_prompt + n_new - 1


def _load_state(sess, cfg, caches, step):
    """Put the evaluator's caches into the session (the state the step at position *step* reads)."""
    from tilefoundry_b200.engine import paged_kv
    sess.pos.fill_(step)
    for layer, kind, state in zip(sess.layers, cfg.layer_types, caches):
        if kind == "linear_attention":
            layer["conv_state"].copy_(state[0][0])
            layer["ssm_state"].copy_(state[1][0])
        else:
            paged_kv.fill_from_logical(layer["k_pool"], sess.table[0], state[0][:, :step])
            paged_kv.fill_from_logical(layer["v_pool"], sess.table[0], state[1][:, :step])


def _same_experts(sess, picks):
    got = sess.idx_trace.cpu()
    return [sorted(got[li].tolist()) == sorted(p.tolist()) for li, p in enumerate(picks)]


@pytest.mark.parametrize("use_graph", [False, True])
def test_step_matches_evaluator_from_its_own_state(dev, sides, use_graph):
    """Every step starts from the evaluator's caches, so one step of the whole hybrid stack is judged at a time:
    the routed experts of every layer (bit-exact as a set; a differing pick is accepted only where the evaluator's
    own margin between the last expert taken and the first left out is a near-tie), per-layer hidden states and
    logits within the end-to-end bound, and the state the step leaves behind: convolution window, Mamba-2 state
    (within 2e-2 of its scale here, because the step's own bf16 inputs already differ in their last bit; the 1e-3
    bound on the f32 update itself is held by ``test_mamba_functions`` on identical inputs), new K/V rows."""
    from tilefoundry_b200.engine import paged_kv
    cfg, ref, twin, _, on_dev = sides
    _, forced, total = _forced_tokens(cfg, ref)
    sess = _session(cfg, on_dev, dev, total + 6)
    sess.reset(forced)
    if use_graph:
        sess.capture()
    excused = 0
    for walk in parity.nested_walk(ref, cfg.layer_types, forced, total):
        step, before, logits, hiddens, picks, margins, after = walk
        if not use_graph:                            # routing on the evaluator's own router inputs: exact
            parity.routing_on_evaluator_inputs(twin, walk, f"step {step}")
        _load_state(sess, cfg, before, step)
        sess.run(1, use_graph)
        same = _same_experts(sess, picks)
        if not all(same):
            first = same.index(False)                # layers above it see a different input: only the first is judged
            assert margins[first] <= TIE_MARGIN, f"step {step}: experts differ at layer {first}, margins {margins}"
            for li in range(first):
                assert_close_at_scale(sess.trace[li], hiddens[li], f"step {step} layer {li} hidden")
            excused += 1
            continue
        for li, h in enumerate(hiddens):
            assert_close_at_scale(sess.trace[li], h, f"step {step} layer {li} hidden")
        assert_close_at_scale(sess.logits, logits[0], f"logits step {step}")
        assert int(sess.picked) == int(torch.argmax(sess.logits.float())), f"step {step}: pick is not argmax"
        assert int(sess.pos) == step + 1
        for li, (kind, state) in enumerate(zip(cfg.layer_types, after)):
            layer = sess.layers[li]
            if kind == "linear_attention":
                assert_close_at_scale(layer["conv_state"], state[0][0], f"step {step} layer {li} conv window")
                assert_close_at_scale(layer["ssm_state"], state[1][0], f"step {step} layer {li} ssm state")
            else:
                n = step + 1
                for name, want_cache in (("k_pool", state[0]), ("v_pool", state[1])):
                    got = paged_kv.logical_view(layer[name], sess.table[0], n)
                    assert_close_at_scale(got[:, -1], want_cache[:, n - 1], f"step {step} layer {li} new {name} row")
    # tiny: 4-8 well separated experts, near-ties are rare; wide: the gap between the last expert taken and the
    # first left out is within two bf16 steps of the logits in about one layer-step in five
    allowed = total // 5 if cfg_is_tiny(cfg) else total // 2
    assert excused <= allowed, f"{excused} of {total} steps had a routing near-tie"


@pytest.mark.parametrize("use_graph", [False, True])
def test_free_running_session_tracks_evaluator(dev, sides, use_graph):
    """The session keeps its own state over the whole teacher-forced walk.  Until the first routing near-tie
    resolves the other way the comparison is the strict one (logits and every layer's hidden state within the
    end-to-end bound, greedy picks equal except inside the logit noise); after it the two trajectories are
    different, equally valid roundings of one sequence -- the differing expert lives on in the recurrent state --
    and must stay close in direction.  The page table is exact throughout."""
    from tilefoundry_b200.engine import paged_kv
    cfg, ref, _, _, on_dev = sides
    _, forced, total = _forced_tokens(cfg, ref)
    sess = _session(cfg, on_dev, dev, total + 6)
    sess.reset(forced)
    if use_graph:
        sess.capture()
    diverged_at, mismatched_picks = None, 0
    for step, _, logits, hiddens, picks, margins, _ in parity.nested_walk(ref, cfg.layer_types, forced, total):
        sess.run(1, use_graph)
        same = _same_experts(sess, picks)
        if diverged_at is None and not all(same):
            assert margins[same.index(False)] <= TIE_MARGIN, f"step {step}: experts differ, margins {margins}"
            diverged_at = step
        ref_logits = logits[0]
        if diverged_at is None:
            assert_close_at_scale(sess.logits, ref_logits, f"logits step {step}")
            for li, h in enumerate(hiddens):
                assert_close_at_scale(sess.trace[li], h, f"step {step} layer {li} hidden")
            if int(sess.picked) != int(torch.argmax(ref_logits)):
                top = torch.topk(ref_logits.float(), 2).values
                noise = (sess.logits.float().cpu() - ref_logits.float()).abs().max()
                assert float(top[0] - top[1]) <= 2 * float(noise), f"pick differs at step {step}"
                mismatched_picks += 1
        else:
            cos = torch.nn.functional.cosine_similarity(sess.logits.float().cpu().flatten(), ref_logits.float().flatten(), dim=0)
            assert float(cos) >= 0.97, f"step {step} (routing diverged at {diverged_at}): logits cosine {float(cos):.4f}"
    assert mismatched_picks <= 6
    # with a handful of well separated experts a near-tie in the first steps would be a bug; at the published
    # widths the gap at the selection's edge is under two bf16 steps in about one layer-step in five
    assert diverged_at is None or diverged_at >= 5 or not cfg_is_tiny(cfg), f"routing diverged at step {diverged_at}"
    assert int(sess.pos) == total
    assert torch.equal(sess.table.cpu(), paged_kv.block_table(1, sess.max_ctx))
