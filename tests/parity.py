"""Shared parity drivers: a session walking the evaluator's own token sequence, compared step by step."""
import torch

from oracle import generation
from tests.helpers import assert_close_at_scale


def cuda_weights(weights, dev):
    return {k: v.to(dev) for k, v in weights.items()}


def on_cpu(fn):
    return lambda *args: fn(*[a.cpu() if isinstance(a, torch.Tensor) else a for a in args])


def to_cpu(x):
    return tuple(to_cpu(i) for i in x) if isinstance(x, tuple) else x.cpu()


def teacher_forced(ref, make_session, vocab, n_prompt, n_new, seed, use_graph):
    """The evaluator decodes greedily on the CPU; the session then walks the very same token sequence
    (given to it as its prompt), so a near-tie in one step cannot make the two sides diverge."""
    g = torch.Generator().manual_seed(seed + 100)
    prompt = torch.randint(0, vocab, (n_prompt,), generator=g)
    want = generation.decode_ids(ref, prompt, n_new, keep_logits=True, keep_hidden=True)
    forced = torch.cat([prompt, torch.tensor(want["tokens"], dtype=torch.int64)])
    sess = make_session(n_prompt + n_new + 5)
    sess.reset(forced)
    if use_graph:
        sess.capture()
    got = {"logits": [], "hidden": [], "picked": []}
    for _ in range(n_prompt + n_new - 1):
        sess.run(1, use_graph)
        got["logits"].append(sess.logits.clone())
        got["hidden"].append(sess.trace.clone())
        got["picked"].append(sess.picked.clone())
    torch.cuda.synchronize()
    return want, sess, got


def compare_run(n_layers, want, sess, got, n_prompt, n_new):
    """Logits and hidden states within the end-to-end bound at every step; greedy picks bit-exact
    except where the evaluator's top-2 margin is inside twice the measured logit difference."""
    total = n_prompt + n_new - 1
    assert int(sess.pos) == total
    excused = 0
    for step in range(total):
        ref_logits = want["logits"][step][0]
        assert_close_at_scale(got["logits"][step], ref_logits, f"logits step {step}")
        for li in range(n_layers + 1):
            assert_close_at_scale(got["hidden"][step][li], want["hidden"][step][li], f"hidden step {step} layer {li}")
        pick, ref_pick = int(got["picked"][step]), int(torch.argmax(ref_logits))
        assert pick == int(torch.argmax(got["logits"][step].cpu())), f"step {step}: pick is not argmax"
        if pick != ref_pick:
            top = torch.topk(ref_logits.float(), 2).values
            noise = (got["logits"][step].float().cpu() - ref_logits.float()).abs().max()
            assert float(top[0] - top[1]) <= 2 * float(noise), (
                f"step {step}: picked {pick}, evaluator {ref_pick}, margin {float(top[0] - top[1]):.4g}, "
                f"noise {float(noise):.4g}")
            excused += 1
    return excused


def compare_caches(want, sess, total):
    from tilefoundry_b200.engine import paged_kv
    assert torch.equal(sess.table.cpu(), paged_kv.block_table(1, sess.max_ctx))
    for li, (k_ref, v_ref) in enumerate(want["caches"]):
        if hasattr(sess, "assembled_cache"):                  # a latent cache is compared re-expanded
            k_got, v_got = sess.assembled_cache(li, total)
        else:
            k_got = paged_kv.logical_view(sess.layers[li]["k_pool"], sess.table[0], total)
            v_got = paged_kv.logical_view(sess.layers[li]["v_pool"], sess.table[0], total)
        assert_close_at_scale(k_got, k_ref[:, :total], f"layer {li} K cache")
        assert_close_at_scale(v_got, v_ref[:, :total], f"layer {li} V cache")


class WalkStep:
    """One teacher-forced evaluator step of a root -> layer -> (mixer | moe -> router) model."""
    __slots__ = ("step", "before", "logits", "hiddens", "picks", "margins", "after", "router_inputs")

    def __init__(self, **kw):
        for k, v in kw.items():
            setattr(self, k, v)

    def __iter__(self):                       # (step, caches before, logits, hiddens, picks, margins, caches after)
        return iter((self.step, self.before, self.logits, self.hiddens, self.picks, self.margins, self.after))


def nested_walk(ref, cfg_kinds, forced, steps):
    """Teacher-forced oracle walk of a root -> layer -> (mixer | moe -> router) model, one step at a time.
    Yields a ``WalkStep``: the caches before and after, logits, hidden state after every layer, routing indices
    per layer, the routing margin per layer and the router's own input per layer.  The margin is the gap
    between the router logit of the last selected expert and the best one left out -- a routing pick inside
    the arithmetic noise shows as a margin near zero, an exact tie as zero."""
    from tilefoundry_b200.authored.granite_4_0_h_small import _with_cache
    caches = ref.init_caches()
    for step in range(steps):
        token_ids, layer_args, caches_in = ref.prepare_inputs_for_generation(forced[: step + 1], step, caches)
        hidden = ref.embed(token_ids)
        fresh, hiddens, picks, margins, router_inputs = [], [], [], [], []
        for layer, margs, cache in zip(ref.modules, layer_args, caches_in):
            mixed, *state = layer.mixer(hidden, *_with_cache(layer.mixer, margs, cache))
            attended = layer.residual_add(hidden, mixed)
            tokens = layer.moe.post_norm(attended)
            rw, idx = layer.moe.router.routing(tokens)
            hidden = layer.residual_add(attended, layer.moe.experts(tokens, rw, idx))
            fresh.append(tuple(state))
            hiddens.append(hidden.reshape(-1))
            picks.append(idx.reshape(-1))
            router_inputs.append(tokens)
            w_r = layer.moe.router.constants["w_router"]
            w_r = w_r if w_r.shape[0] == tokens.shape[-1] else w_r.t()          # authored as (in, out) or (out, in)
            logits = torch.matmul(tokens.to(w_r.dtype), w_r).float().reshape(-1)
            top = torch.topk(logits, idx.numel() + 1).values
            margins.append(float(top[-2] - top[-1]))
        after = ref.append_cache(caches, tuple(fresh))
        yield WalkStep(step=step, before=caches, logits=ref.lm_head(ref.final_rms_norm(hidden)), hiddens=hiddens,
                       picks=picks, margins=margins, after=after, router_inputs=router_inputs)
        caches = after


def routing_on_evaluator_inputs(twin, walk_step, where):
    """Every layer's router run through the twin on the very vector the evaluator's router saw: the selected
    experts must be the evaluator's, bit for bit; a different set is admissible only on an exact tie between
    the last expert taken and the first left out (margin 0), where the order is not determined."""
    for li, (tokens, want, margin) in enumerate(zip(walk_step.router_inputs, walk_step.picks, walk_step.margins)):
        router = getattr(twin, f"layer{li}").moe.router
        _, got = router.routing(tokens.to(next(iter(router._bound.values())).device))
        got = got.reshape(-1).cpu()
        if sorted(got.tolist()) != sorted(want.tolist()):
            assert margin == 0.0, f"{where} layer {li}: experts {got.tolist()} != {want.tolist()}, margin {margin:.4g}"


def assert_same_routing(got_idx, want_idx, router_logits, where=""):
    """Routing indices, position by position.  Where the two sides name different experts their router logits must
    be EQUAL: an exact tie, inside the selection (the order of equal values is not determined) or at its edge
    (which of two equal experts is the last one taken is not determined either).  Anything else is an error."""
    got, want = got_idx.reshape(-1).cpu(), want_idx.reshape(-1).cpu()
    logits = router_logits.reshape(-1).float().cpu()
    assert got.numel() == want.numel() and len(set(got.tolist())) == got.numel(), f"{where}: {got.tolist()}"
    diff = (got != want).nonzero().flatten().tolist()
    for i in diff:
        assert float(logits[got[i]]) == float(logits[want[i]]), (
            f"{where}: slot {i} holds expert {int(got[i])} (logit {float(logits[got[i]]):.6g}), the evaluator's holds "
            f"{int(want[i])} (logit {float(logits[want[i]]):.6g})")
    return len(diff)
