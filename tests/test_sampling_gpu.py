"""On-device sampling (Gumbel-max inside the head kernel) against the CPU restatement of the same generator and pick,
fed with the kernel's own bf16 logits."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import sampling
from tilefoundry_b200.authored import qwen3_1_7b as q
from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import DictResource

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tilefoundry_b200 import lib
    lib.load()
    return torch.device("cuda:0")


class Head:
    """One head matrix and activation on the device, and everything a tfb_lm_head_argmax call needs."""

    def __init__(self, dev, n, k, seed=0):
        from tilefoundry_b200 import lib
        g = torch.Generator().manual_seed(seed)
        self.n, self.k, self.dev = n, k, dev
        self.w = (torch.randn(n, k, generator=g) * k ** -0.5 * 3).to(BF).to(dev)
        self.x = torch.randn(k, generator=g).to(BF).to(dev)
        entries = lib.lm_head_scratch_entries(n)
        self.val = torch.zeros(entries, device=dev, dtype=torch.float32)
        self.idx = torch.zeros(entries, device=dev, dtype=torch.int32)
        self.counter = torch.zeros(1, device=dev, dtype=torch.int32)
        self.logits = torch.zeros(n, device=dev, dtype=BF)
        self.token = torch.zeros(1, device=dev, dtype=torch.int64)
        self.pos = torch.zeros(1, device=dev, dtype=torch.int32)
        self.pair = torch.zeros(2, device=dev, dtype=torch.float32)

    def run(self, temperature, seed, step, rows=None, pair=False):
        from tilefoundry_b200 import lib
        lo, hi = rows if rows else (0, self.n)
        self.pos.fill_(step)
        w = self.w[lo:hi]
        # pos alone (no token history): the kernel reads it as the step of the draw and leaves it unchanged
        a = lib.LmHeadArgs(w=lib.ptr(w), x=lib.ptr(self.x), gamma=None, logits=lib.ptr(self.logits[lo:hi]),
                           token_out=lib.ptr(self.token), scratch_val=lib.ptr(self.val), scratch_idx=lib.ptr(self.idx),
                           counter=lib.ptr(self.counter), n=hi - lo, k=self.k, prologue=lib.NORM_NONE, eps=0.0,
                           x_scale=1.0, out_scale=1.0, pdl=0, tokens=None, pos=lib.ptr(self.pos), n_prompt=0,
                           max_tokens=0, kernel=0, self_prefetch=0, index_offset=lo,
                           pair_out=lib.ptr(self.pair) if pair else None, temperature=temperature, seed=seed)
        lib.check(lib.load().tfb_lm_head_argmax(C.byref(a), lib.stream()), "tfb_lm_head_argmax")
        torch.cuda.synchronize()
        assert int(self.counter) == 0 and int(self.pos) == step
        return int(self.token)


def _expect(logits_f32, temperature, seed, step, got):
    """The oracle's pick, or -- where its two best perturbed scores are closer than the log() rounding between the two
    sides -- whichever of the two the kernel chose."""
    scores = sampling.gumbel_scores(logits_f32, temperature, seed, step)
    order = np.argsort(-scores, kind="stable")[:2]
    if got != int(order[0]):
        assert got == int(order[1]) and scores[order[0]] - scores[order[1]] < 1e-4, (got, order, scores[order])


@pytest.mark.parametrize("n,k", [(5000, 512), (151936, 256), (37, 256)])
def test_sample_equals_oracle_pick_on_the_kernels_own_logits(dev, n, k):
    head = Head(dev, n, k, seed=n)
    greedy = head.run(0.0, 123, 5)
    logits = head.logits.float().cpu().numpy()
    assert greedy == int(np.argmax(logits))                      # temperature 0: the lowest-index maximum
    picks = set()
    for seed, step, temperature in [(1, 0, 1.0), (1, 1, 1.0), (2, 1, 1.0), (99, 700, 0.7), (2 ** 63 + 5, 3, 1.5),
                                    (7, 2047, 0.3), (7, 2048, 0.3), (8, 2048, 2.0)]:
        got = head.run(temperature, seed, step)
        assert np.array_equal(head.logits.float().cpu().numpy(), logits)       # the logits are not perturbed
        _expect(logits, temperature, seed, step, got)
        picks.add(got)
    assert len(picks) > 1                                        # seeds and steps do change the draw


def test_draws_follow_softmax_of_logits_over_temperature(dev):
    head = Head(dev, 48, 256, seed=4)
    head.run(0.0, 0, 0)
    logits = head.logits.float().cpu().numpy()
    temperature, steps = 0.8, 6000
    counts = np.zeros(48)
    for step in range(steps):
        counts[head.run(temperature, 31337, step)] += 1
    want = np.exp((logits - logits.max()) / temperature)
    want /= want.sum()
    total_variation = 0.5 * np.abs(counts / steps - want).sum()
    assert total_variation < 0.05, total_variation


def test_vocabulary_shards_draw_the_same_token(dev):
    """Two half-vocabulary launches (index_offset, pair output) agree with the whole-vocabulary draw."""
    head = Head(dev, 6000, 512, seed=8)
    for seed, step in [(5, 0), (5, 1), (6, 9), (77, 300)]:
        whole = head.run(0.9, seed, step)
        pairs = []
        for rows in [(0, 3008), (3008, 6000)]:
            head.run(0.9, seed, step, rows=rows, pair=True)
            pairs.append(head.pair.cpu().tolist())
        best = max(pairs, key=lambda p: (p[0], -p[1]))
        assert int(best[1]) == whole


def test_session_sampling_is_reproducible_and_seeded(dev):
    from tilefoundry_b200.engine.qwen3 import Qwen3Session
    cfg = q.QWEN3_TINY
    weights = q.tie_head(random_weights(q.build(cfg), seed=5, std=0.05))
    res = DictResource({k: v.to(dev) for k, v in weights.items()})
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    a = Qwen3Session(cfg, res, max_ctx=128, device=dev, keep_logits=True, temperature=1.0, seed=42)
    one = a.generate(prompt, 60, use_graph=True).tokens
    two = a.generate(prompt, 60, use_graph=False).tokens
    assert one == two                                            # same seed, graph or eager: same transcript
    b = Qwen3Session(cfg, res, max_ctx=128, device=dev, temperature=1.0, seed=43)
    other = b.generate(prompt, 60).tokens
    assert other != one
    greedy = Qwen3Session(cfg, res, max_ctx=128, device=dev).generate(prompt, 60).tokens
    assert greedy != one
    # the last step's draw, re-derived on the CPU from the logits the session kept
    step = int(a.pos) - 1
    logits = a.logits.float().cpu().numpy()
    _expect(logits, 1.0, 42, step, one[-1])


def test_one_launch_step_samples_with_the_same_rule(dev):
    """The one-launch Qwen3 step draws inside its head phase: reproducible (graph or eager), keyed by the seed, and
    every checked draw equals the CPU restatement applied to the logits the step itself wrote."""
    from tilefoundry_b200.engine.qwen3 import KERNEL_FUSED, Qwen3Session
    cfg = q.QWEN3_SMALL
    weights = q.tie_head(random_weights(q.build(cfg), seed=5, std=0.05))
    res = DictResource({k: v.to(dev) for k, v in weights.items()})
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    a = Qwen3Session(cfg, res, max_ctx=128, device=dev, keep_logits=True, temperature=0.8, seed=42, kernel=KERNEL_FUSED)
    assert a.launches_per_step == 1
    one = a.generate(prompt, 60, use_graph=True).tokens
    two = a.generate(prompt, 60, use_graph=False).tokens
    a.check_status()
    assert one == two
    step = int(a.pos) - 1
    _expect(a.logits.float().cpu().numpy(), 0.8, 42, step, one[-1])
    for n_new in (1, 7, 23):                                     # a few more draws, each against the step's own logits
        t = a.generate(prompt, n_new, use_graph=False).tokens
        assert t == one[:len(t)]
        _expect(a.logits.float().cpu().numpy(), 0.8, 42, int(a.pos) - 1, t[-1])
    other = Qwen3Session(cfg, res, max_ctx=128, device=dev, temperature=0.8, seed=43, kernel=KERNEL_FUSED).generate(prompt, 60).tokens
    greedy = Qwen3Session(cfg, res, max_ctx=128, device=dev, kernel=KERNEL_FUSED).generate(prompt, 60).tokens
    assert other != one and greedy != one


def test_nucleus_sampling_after_the_step(dev):
    """``top_p`` < 1: every new token is the nucleus draw of the CPU restatement on the step's own logits, for the
    one-launch step and the step of separate launches; reproducible; ``top_p`` close to 0 draws among the top value's tokens; an end
    id picked by the nucleus draw latches the sequence."""
    from tilefoundry_b200.engine.qwen3 import KERNEL_FUSED, Qwen3Session
    cfg = q.QWEN3_SMALL
    weights = q.tie_head(random_weights(q.build(cfg), seed=5, std=0.05))
    res = DictResource({k: v.to(dev) for k, v in weights.items()})
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(2))
    for kernel in (KERNEL_FUSED, 0):
        a = Qwen3Session(cfg, res, max_ctx=128, device=dev, temperature=0.8, seed=42, top_p=0.6, kernel=kernel)
        one = a.generate(prompt, 40, use_graph=True).tokens
        two = a.generate(prompt, 40, use_graph=False).tokens
        if kernel == KERNEL_FUSED:
            a.check_status()
        assert one == two
        for n_new in (1, 9, 40):                                   # draws against the step's own logits
            t = a.generate(prompt, n_new, use_graph=False).tokens
            assert t == one[:n_new]
            want = sampling.sample_top_p(a.logits.float().cpu().numpy(), 0.8, 0.6, 42, int(a.pos) - 1)
            assert t[-1] == want, (kernel, n_new, t[-1], want)
        plain = Qwen3Session(cfg, res, max_ctx=128, device=dev, temperature=0.8, seed=42, kernel=kernel).generate(prompt, 40).tokens
        assert plain != one                                        # the filter changes the draws
        tight = Qwen3Session(cfg, res, max_ctx=128, device=dev, temperature=0.8, seed=42, top_p=1e-6, kernel=kernel)
        for n_new in (1, 7, 25):                                   # a nucleus of the top VALUE alone (several tokens may share it)
            last = tight.generate(prompt, n_new, use_graph=False).tokens[-1]
            assert float(tight.logits[last]) == float(tight.logits.max())
        stop = one[5]
        cut = a.generate(prompt, 40, eos=[stop]).tokens
        assert cut == one[:one.index(stop)]


@pytest.mark.parametrize("model", ["minicpm3", "granite", "qwen3_5"])
def test_other_sessions_sample_too(dev, model):
    """The other three decode steps hand temperature and seed to the same head kernel."""
    from tests import parity
    if model == "minicpm3":
        from tilefoundry_b200.authored import minicpm3_4b as a
        from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session as S
        cfg = a.MINICPM3_TINY
        weights = a.tie_head(random_weights(a.build(cfg), seed=9, std=0.05))
    elif model == "granite":
        from tilefoundry_b200.authored import granite_4_0_h_small as a
        from tilefoundry_b200.engine.granite import GraniteSession as S
        cfg = a.GRANITE_TINY
        weights = random_weights(a.build(cfg), seed=9, std=0.05, overrides=a.weight_overrides)
    else:
        from tilefoundry_b200.authored import qwen3_5_35b_a3b as a
        from tilefoundry_b200.engine.qwen3_5 import Qwen35Session as S
        cfg = a.QWEN3_5_TINY
        weights = random_weights(a.build(cfg), seed=9, std=0.05, overrides=a.weight_overrides)
    res = DictResource(parity.cuda_weights(weights, dev))
    prompt = torch.randint(0, cfg.vocab_size, (10,), generator=torch.Generator().manual_seed(3))
    sess = S(cfg, res, max_ctx=96, device=dev, keep_logits=True, temperature=0.9, seed=77)
    one = sess.generate(prompt, 40, use_graph=True).tokens
    two = sess.generate(prompt, 40, use_graph=False).tokens
    assert one == two
    step = int(sess.pos) - 1
    _expect(sess.logits.float().cpu().numpy().reshape(-1), 0.9, 77, step, one[-1])
    greedy = S(cfg, res, max_ctx=96, device=dev).generate(prompt, 40).tokens
    other = S(cfg, res, max_ctx=96, device=dev, temperature=0.9, seed=78).generate(prompt, 40).tokens
    assert one != greedy and one != other
