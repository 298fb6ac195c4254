"""Parity of the CUDA path against the CPU oracle -- Qwen3.5-35B-A3B (Gated DeltaNet + gated attention hybrid,
256-expert MoE; f32 activations and state, bf16 contracted weights)."""
import pytest
import torch

from oracle import evaluator, generation, qwen3_5_35b_a3b as oq
from tests import parity
from tests.helpers import ATOL, RTOL, assert_close_at_scale
from tilefoundry_b200.authored import qwen3_5_35b_a3b as qa
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import AllClose, DictResource, Equal, NanInf, check

pytestmark = pytest.mark.gpu
CLOSE = [AllClose(atol=ATOL, rtol=RTOL), NanInf()]          # through a bf16 product
F32 = [AllClose(atol=1e-3, rtol=1e-3), NanInf()]            # pure f32 arithmetic


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


# The published widths on a stack cut to three Gated DeltaNet layers and one gated-attention layer and a
# 4096-entry vocabulary: hidden 2048, 16 k / 32 v heads x 128, 16 q / 2 kv heads x 256 with 64 rotary dims, 256
# experts top-8 of 512 + the shared expert.  Every kernel is instantiated by these widths, not by the depth, so
# this is the configuration the benchmark runs.
WIDE = qa.truncated(qa.QWEN3_5_35B_A3B, n_layers=4, vocab=4096, max_ctx=256)
CONFIGS = {"tiny": (qa.QWEN3_5_TINY, 0.05), "wide": (WIDE, 0.02)}


@pytest.fixture(scope="module", params=["tiny", "wide"])
def sides(request, dev):
    """(config, evaluator side, twin, device weights); pytest groups the tests by configuration, so each
    configuration's weights are drawn once and dropped before the next is built."""
    from tilefoundry_b200.twins.qwen3_5_35b_a3b import make_twin
    cfg, std = CONFIGS[request.param]
    mod = qa.build(cfg)
    weights = random_weights(mod, seed=3, std=std, overrides=qa.weight_overrides)
    on_dev = parity.cuda_weights(weights, dev)
    ref = evaluator.load(mod, DictResource(weights), oq.make(cfg))
    twin = make_twin(cfg)()
    twin.load(DictResource(on_dev))
    yield cfg, ref, twin, on_dev
    del ref, twin, weights, on_dev
    torch.cuda.empty_cache()


def _check(twin_fn, ref_fn, inputs, expect):
    rep = check(lambda *a: parity.to_cpu(twin_fn(*a)), parity.on_cpu(ref_fn), inputs, expect=expect)
    assert rep.passed, rep.render()


def test_linear_attention_functions(dev, sides):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(5)
    r = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(dev)
    HV, DK, DV, CONV = cfg.gdn_n_v_heads, cfg.gdn_head_k_dim, cfg.gdn_head_v_dim, cfg.conv_dim
    rm, tm = ref.layer0.mixer, twin.layer0.mixer
    conv_state, entry = r(1, CONV, 3, scale=0.5), r(1, CONV, 1)
    _check(tm.conv_step, rm.conv_step, (conv_state, entry), {"output": F32})
    _check(tm.l2_normalise, rm.l2_normalise, (r(1, 1, HV, DK),), {"output": F32})
    state = r(1, HV, DK, DV, scale=0.1)
    unit = lambda t: t / t.norm(dim=-1, keepdim=True)
    step_in = (state, unit(r(1, 1, HV, DK)), unit(r(1, 1, HV, DK)), r(1, 1, HV, DV), -torch.rand(1, 1, HV, generator=g).to(dev),
               torch.rand(1, 1, HV, generator=g).to(dev))
    _check(tm.delta_step, rm.delta_step, step_in, {"output[0]": F32, "output[1]": F32})
    hidden = r(1, 1, cfg.hidden)
    _check(tm.linear_attention, rm.linear_attention, (hidden, conv_state, state),
           {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})
    assert torch.equal(state.cpu(), step_in[0].cpu())              # inputs were not mutated


@pytest.mark.parametrize("ctx", [0, 1, 63, 64, 130])
def test_full_attention_functions(dev, sides, ctx):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(ctx)
    HQ, HKV, D = cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim
    ai = cfg.full_attention_every - 1
    ra, ta = getattr(ref, f"layer{ai}").mixer, getattr(twin, f"layer{ai}").mixer
    cos, sin = qa.rope_tables(cfg)
    pos = torch.tensor([ctx], dtype=torch.int32)
    on = lambda *ts: tuple(t.to(dev) for t in ts)
    _check(ta.partial_rope, ra.partial_rope, on(torch.randn(1, 1, HQ, D, generator=g), cos, sin, pos), {"output": F32})
    _check(ta.partial_rope_kv, ra.partial_rope_kv, on(torch.randn(1, 1, HKV, D, generator=g), cos, sin, pos), {"output": F32})
    hidden = torch.randn(1, 1, cfg.hidden, generator=g)
    kc = torch.randn(1, ctx, HKV, D, generator=g) * 0.5
    vc = torch.randn(1, ctx, HKV, D, generator=g) * 0.5
    scale = torch.full((1, 1, 1, 1), D ** -0.5)
    _check(ta.full_attention, ra.full_attention, on(hidden, cos, sin, pos, kc, vc, scale),
           {"output[0]": CLOSE, "output[1]": CLOSE, "output[2]": CLOSE})


def test_moe_functions_and_routing_indices(dev, sides):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(9)
    rm, tm = ref.layer0.moe, twin.layer0.moe
    for trial in range(4):                                       # routing is an integer output: several token vectors
        hidden = torch.randn(1, 1, cfg.hidden, generator=g).to(dev)
        _check(tm.post_norm, rm.post_norm, (hidden,), {"output": F32})
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
    _check(tm.shared_expert, rm.shared_expert, (tokens.to(dev),), {"output": CLOSE})
    _check(tm.experts, rm.experts, args, {"output": CLOSE})
    _check(tm, rm, (hidden,), {"output": CLOSE})                 # the block's own forward
    b = torch.randn(1, 1, cfg.hidden, generator=g).to(dev)
    _check(twin.layer0.residual_add, ref.layer0.residual_add, (hidden, b), {"output": F32})


@pytest.mark.parametrize("n_tokens", [1, 5, 64])
def test_experts_for_a_batch_of_tokens(dev, sides, n_tokens):
    """``tfb_moe_batch``: the block's ``experts`` for several tokens at once -- every selected expert read once, its rows
    against all of its tokens on the tensor cores -- equals the evaluator's ``experts`` token by token (the evaluator's
    own routing is handed to both sides, so no near-tie can make them differ).  64 tokens with 8 of 256 experts each is
    the batch the grouped form is for; 1 and 5 tokens leave most experts without a token."""
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(40 + n_tokens)
    rm, tm = ref.layer0.moe, twin.layer0.moe
    hidden = torch.randn(n_tokens, 1, 1, cfg.hidden, generator=g)
    tokens = torch.cat([rm.post_norm(h) for h in hidden])                       # [T, H] f32
    routed = [rm.router.routing(tokens[t:t + 1]) for t in range(n_tokens)]
    weights = torch.cat([w.reshape(1, -1) for w, _ in routed])
    indices = torch.cat([i.reshape(1, -1) for _, i in routed])
    want = torch.cat([rm.experts(tokens[t:t + 1], *routed[t]).reshape(1, -1) for t in range(n_tokens)])
    got = tm.experts_batch(tokens.to(dev), weights.to(dev), indices.to(dev)).cpu()
    assert_close_at_scale(got, want, f"experts of {n_tokens} tokens")
    # and the one-token path of the twin agrees with it on its own routing inputs
    one = tm.experts(tokens[:1].to(dev), weights[:1].to(dev), indices[:1].to(dev)).reshape(1, -1).cpu()
    assert_close_at_scale(got[:1], one, "batch form against the one-token kernels")


def test_block_forward_for_a_batch_of_tokens(dev, sides):
    """Post-norm, routing and experts for 48 tokens in eight launches: the routing of every token equals the evaluator's
    (experts bit-exact except across exactly equal or near-equal probabilities), the gate logits and weights are
    close, and the block's output equals the evaluator's forward for every token whose routing agrees."""
    cfg, ref, twin = sides[:3]
    T = 48
    g = torch.Generator().manual_seed(77)
    rm, tm = ref.layer0.moe, twin.layer0.moe
    hidden = torch.randn(T, 1, 1, cfg.hidden, generator=g)
    tokens = torch.cat([rm.post_norm(h) for h in hidden])
    got_w, got_idx, got_gate = (v.cpu() for v in tm.route_batch(tokens.to(dev)))
    w_r = rm.router.constants["w_router"]
    w_r = w_r if w_r.shape[0] == tokens.shape[-1] else w_r.t()
    same, flips = [], []
    for t in range(T):
        want_w, want_idx = rm.router.routing(tokens[t:t + 1])
        same.append(torch.equal(got_idx[t], want_idx.reshape(-1)))
        if same[-1]:
            assert_close_at_scale(got_w[t], want_w.reshape(-1), f"routing weights, token {t}")
            continue
        try:                                                   # an exact tie of bf16 logits may be taken in either order
            parity.assert_same_routing(got_idx[t:t + 1], want_idx.reshape(1, -1), torch.matmul(tokens[t:t + 1].to(w_r.dtype), w_r), f"token {t}")
        except AssertionError:                                 # a logit one bf16 step apart (the sums run in another order)
            flips.append(t)
    assert len(flips) <= 2, f"routing differs beyond exact ties on tokens {flips}"
    assert sum(same) >= T // 2, f"routing differs on {T - sum(same)} of {T} tokens"      # (exact ties of bf16 logits are common)
    got = tm.forward_batch(hidden.reshape(T, cfg.hidden).to(dev)).cpu()
    for t in range(T):
        if same[t]:
            assert_close_at_scale(got[t], rm(hidden[t]).reshape(-1), f"block forward, token {t}")


def test_root_functions(dev, sides):
    cfg, ref, twin = sides[:3]
    g = torch.Generator().manual_seed(2)
    ids = torch.tensor([cfg.vocab - 1])
    assert torch.equal(twin.embed(ids.to(dev)).cpu(), ref.embed(ids))
    hidden = torch.randn(1, 1, cfg.hidden, generator=g)
    _check(twin.final_rms_norm, ref.final_rms_norm, (hidden.to(dev),), {"output": F32})
    normed = ref.final_rms_norm(hidden)
    _check(twin.lm_head, ref.lm_head, (normed.to(dev),), {"output": CLOSE})
    assert int(twin.last_token) == int(torch.argmax(twin.lm_head(normed.to(dev))))


def cfg_is_tiny(cfg):
    return cfg.hidden < 1024


def _setup(dev, sides):
    from tilefoundry_b200.engine.qwen3_5 import Qwen35Session
    cfg, ref, _, on_dev = sides
    n_prompt, max_new = (16, 60) if cfg_is_tiny(cfg) else (64, 32)   # the wide stack: 64 prompt ids + 32 new tokens
    prompt = torch.randint(0, cfg.vocab, (n_prompt,), generator=torch.Generator().manual_seed(111))
    want = generation.decode_ids(ref, prompt, max_new)
    forced = torch.cat([prompt, torch.tensor(want["tokens"], dtype=torch.int64)])
    sess = Qwen35Session(cfg, DictResource(on_dev), max_ctx=n_prompt + max_new + 5, device=dev,
                         keep_logits=True, trace_hidden=True)
    sess.reset(forced)
    return cfg, ref, sess, forced, n_prompt + max_new - 1


def _load_state(sess, cfg, caches, step):
    """Put the evaluator's caches into the session (the state the step at position *step* reads)."""
    from tilefoundry_b200.engine import paged_kv
    sess.pos.fill_(step)
    for layer, kind, state in zip(sess.layers, cfg.layer_types, caches):
        if kind == "linear_attention":
            layer["conv_state"][step & 1].copy_(state[0][0])
            layer["state"].copy_(state[1][0])
        else:
            paged_kv.fill_from_logical(layer["k_pool"], sess.table[0], state[0])
            paged_kv.fill_from_logical(layer["v_pool"], sess.table[0], state[1])


def _same_experts(sess, picks):
    got = sess.idx_trace.cpu()
    return [sorted(got[li].tolist()) == sorted(p.tolist()) for li, p in enumerate(picks)]


# A routing pick is decided by bf16 router logits computed from inputs that already differ by the arithmetic
# noise of the layers below: two logits closer than this may legitimately come out in the other order.
TIE_MARGIN = 3e-2


@pytest.mark.parametrize("use_graph", [False, True])
def test_step_matches_evaluator_from_its_own_state(dev, sides, use_graph):
    """Every step starts from the evaluator's caches, so one step of the whole hybrid stack is judged at a
    time: per-layer hidden states, logits, routed experts, and the state the step leaves behind.  A step in
    which a router pick differs is accepted only if the evaluator's own margin for that pick is a near-tie."""
    from tilefoundry_b200.engine import paged_kv
    cfg, ref, sess, forced, total = _setup(dev, sides)
    twin = sides[2]
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
                assert_close_at_scale(sess.conv_window(layer), state[0][0], f"step {step} layer {li} conv window")
                assert_close_at_scale(layer["state"], state[1][0], f"step {step} layer {li} recurrent state")
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
    """The session keeps its own state over the whole walk.  Until the first routing near-tie resolves the
    other way the comparison is the strict one; after it the two trajectories are different (equally valid)
    roundings of one sequence and must stay close in direction."""
    from tilefoundry_b200.engine import paged_kv
    cfg, ref, sess, forced, total = _setup(dev, sides)
    if use_graph:
        sess.capture()
    diverged_at = None
    for step, _, logits, hiddens, picks, margins, _ in parity.nested_walk(ref, cfg.layer_types, forced, total):
        sess.run(1, use_graph)
        if diverged_at is None and not all(_same_experts(sess, picks)):
            diverged_at = step
        if diverged_at is None:
            assert_close_at_scale(sess.logits, logits[0], f"logits step {step}")
            for li, h in enumerate(hiddens):
                assert_close_at_scale(sess.trace[li], h, f"step {step} layer {li} hidden")
        else:
            cos = torch.nn.functional.cosine_similarity(sess.logits.float().cpu().flatten(), logits[0].flatten(), dim=0)
            assert float(cos) >= 0.97, f"step {step} (routing diverged at {diverged_at}): logits cosine {float(cos):.4f}"
    # with a handful of well separated experts a near-tie in the first steps would be a bug; at the published
    # widths the gap at the selection's edge is under two bf16 steps in about one layer-step in five
    assert diverged_at is None or diverged_at >= 5 or not cfg_is_tiny(cfg), f"routing diverged at step {diverged_at}"
    assert int(sess.pos) == total
    assert torch.equal(sess.table.cpu(), paged_kv.block_table(1, sess.max_ctx))


def test_generate_equals_stepwise_and_replays(dev):
    """generate() (one captured graph, device-resident token history) returns the tokens a step-by-step eager
    walk returns, and a second sequence through the same graph starts from zeroed recurrent state."""
    from tilefoundry_b200.engine.qwen3_5 import Qwen35Session
    cfg = qa.QWEN3_5_TINY
    weights = random_weights(qa.build(cfg), seed=4, std=0.05, overrides=qa.weight_overrides)
    sess = Qwen35Session(cfg, DictResource(parity.cuda_weights(weights, dev)), max_ctx=96, device=dev)
    prompt = torch.randint(0, cfg.vocab, (9,), generator=torch.Generator().manual_seed(8))
    a = sess.generate(prompt, 40, use_graph=True).tokens
    b = sess.generate(prompt, 40, use_graph=False).tokens
    c = sess.generate(prompt, 40, use_graph=True).tokens
    assert a == b == c


def test_router_projection_selects_experts_in_its_last_cta(dev):
    """The router projection can select the top-k itself (last CTA to finish); that must give the very experts
    and weights the stand-alone selection gives from the same logits, and leave its ticket at zero."""
    import ctypes as C
    from tilefoundry_b200 import lib
    E, K, H = 256, 8, 2048
    g = torch.Generator().manual_seed(21)
    w_r = (torch.randn(E + 1, H, generator=g) * H ** -0.5).to(torch.bfloat16).to(dev)
    w_r[200] = w_r[17]                                             # an exact tie resolves to the lower index
    x, gamma = torch.randn(H, generator=g).to(dev), (1 + 0.1 * torch.randn(H, generator=g)).to(dev)
    logits = torch.empty(E + 1, device=dev)
    idx, w = torch.zeros(K, dtype=torch.int64, device=dev), torch.zeros(K, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    a = lib.GemvF32Args(w=lib.ptr(w_r), x=lib.ptr(x), gamma=lib.ptr(gamma), y=lib.ptr(logits), n=E + 1, k=H,
                        prologue=lib.NORM_F32GAIN, epilogue=lib.EPI_STORE, eps=1e-6, pdl=0, route_counter=lib.ptr(counter),
                        route_experts=E, route_top_k=K, idx_out=lib.ptr(idx), w_out=lib.ptr(w))
    for _ in range(2):
        lib.check(lib.load().tfb_gemv_f32(C.byref(a), lib.stream()), "tfb_gemv_f32")
    idx2, w2 = torch.zeros(K, dtype=torch.int64, device=dev), torch.zeros(K, device=dev)
    lib.check(lib.load().tfb_router_select(None, lib.ptr(logits), lib.ptr(idx2), None, lib.ptr(w2), E, K, 1, 0, lib.stream()), "select")
    assert torch.equal(idx.cpu(), idx2.cpu())
    torch.testing.assert_close(w.cpu(), w2.cpu(), rtol=1e-5, atol=1e-7)   # two summation orders of the same sums
    assert int(counter) == 0
    probs = torch.softmax(logits[:E].cpu(), -1)
    pv, _ = torch.topk(probs, K)
    assert torch.equal(probs[idx.cpu()], pv)                       # same values in the same order (equal values: any order in torch)
    got = idx.cpu().tolist()
    assert (17 not in got and 200 not in got) or (17 in got and (200 not in got or got.index(17) < got.index(200)))


def test_select_with_expert_prefetch_selects_the_same(dev):
    """The selection that also asks L2 for the chosen experts' weights returns what the plain selection returns
    (the prefetch has no architectural effect), with and without an expert-parallel split."""
    import ctypes as C
    from tilefoundry_b200 import lib
    E, K, I, H = 64, 8, 128, 256
    g = torch.Generator().manual_seed(31)
    logits = torch.randn(E, generator=g).to(dev)
    slabs = [torch.zeros(E, I, H, dtype=torch.bfloat16, device=dev) for _ in range(3)]
    idx, w = torch.zeros(K, dtype=torch.int64, device=dev), torch.zeros(K, device=dev)
    lib.check(lib.load().tfb_router_select(None, lib.ptr(logits), lib.ptr(idx), None, lib.ptr(w), E, K, 1, 0, lib.stream()), "select")
    for world, rank in ((1, 0), (2, 1)):
        idx2, w2 = torch.zeros(K, dtype=torch.int64, device=dev), torch.zeros(K, device=dev)
        local = [s[rank::world].contiguous() for s in slabs]
        a = lib.RouterSelectArgs(logits_f32=lib.ptr(logits), indices=lib.ptr(idx2), weights_f32=lib.ptr(w2), experts=E, top_k=K,
                                 mode=1, pdl=0, n_slabs=3, expert_rank=rank, expert_world=world)
        for i, s in enumerate(local):
            a.slab[i], a.slab_bytes[i] = s.data_ptr(), I * H * 2
        lib.check(lib.load().tfb_router_select_prefetch(C.byref(a), lib.stream()), "tfb_router_select_prefetch")
        torch.cuda.synchronize()
        assert torch.equal(idx2.cpu(), idx.cpu()) and torch.equal(w2.cpu(), w.cpu())
