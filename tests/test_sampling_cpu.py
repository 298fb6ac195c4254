"""The CPU restatement of on-device sampling: generator range and pinned values, and that Gumbel-max over it draws
from softmax(logits / temperature)."""
import numpy as np

from oracle import sampling


def test_uniforms_are_open_interval_seeded_and_pinned():
    u = sampling.uniforms(7, 3, 200000)
    assert u.dtype == np.float64 and 0.0 < u.min() and u.max() < 1.0
    assert abs(u.mean() - 0.5) < 5e-3 and abs(np.corrcoef(u[:-1], u[1:])[0, 1]) < 1e-2
    assert not np.array_equal(u[:100], sampling.uniforms(8, 3, 100))
    assert not np.array_equal(u[:100], sampling.uniforms(7, 4, 100))
    # a shard draws what the whole vocabulary draws for the same indices
    assert np.array_equal(sampling.uniforms(7, 3, 50, index_offset=1000), u[1000:1050])
    # the generator itself, pinned: splitmix64 finaliser of seed + golden * (index + 1) + 0xD1B5.. * (step + 1)
    z = (0 + 0x9E3779B97F4A7C15 * 1 + 0xD1B54A32D192ED03 * 1) & (2 ** 64 - 1)
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & (2 ** 64 - 1)
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & (2 ** 64 - 1)
    z ^= z >> 31
    assert sampling.uniforms(0, 0, 1)[0] == ((z >> 41) + 0.5) / 8388608.0


def test_gumbel_max_draws_from_softmax():
    logits = np.array([2.0, 1.0, 0.0, -1.0, 0.5, -30.0], dtype=np.float32)
    for temperature in (0.7, 1.0, 2.5):
        counts = np.zeros(6)
        for step in range(20000):
            counts[sampling.sample(logits, temperature, 11, step)] += 1
        want = np.exp(logits / temperature)
        want /= want.sum()
        assert 0.5 * np.abs(counts / counts.sum() - want).sum() < 0.02
    # temperature -> 0 approaches the greedy pick
    assert all(sampling.sample(logits, 1e-3, 5, s) == 0 for s in range(50))


def test_nucleus_threshold_and_pick():
    rng = np.random.default_rng(3)
    import torch
    logits = (torch.from_numpy(rng.standard_normal(4000).astype(np.float32)) * 2).to(torch.bfloat16).float().numpy()
    for temperature in (0.7, 1.0):
        p = np.exp((logits.astype(np.float64) - logits.max()) / temperature)
        p /= p.sum()
        for top_p in (0.05, 0.5, 0.9):
            tau = sampling.nucleus_threshold(logits, temperature, top_p)
            assert p[logits >= tau].sum() >= top_p - 1e-12           # the nucleus holds the mass asked for ...
            assert p[logits > tau].sum() < top_p + 1e-12             # ... and would not without the threshold's own tokens
            picks = {sampling.sample_top_p(logits, temperature, top_p, 5, s) for s in range(300)}
            assert all(logits[i] >= tau for i in picks) and (len(picks) > 1 or (logits >= tau).sum() == 1)
        # the whole distribution: the plain draw
        assert all(sampling.sample_top_p(logits, temperature, 1.0, 5, s) == sampling.sample(logits, temperature, 5, s) for s in range(50))
    # a nucleus of one value: always the (lowest-index) maximum when it alone carries the mass
    spike = np.full(100, -20.0, dtype=np.float32)
    spike[17] = 10.0
    assert all(sampling.sample_top_p(spike, 1.0, 0.9, 1, s) == 17 for s in range(20))
