"""TEST INFRASTRUCTURE ONLY -- CPU restatement of on-device token sampling.

The reference samples on the device with the Gumbel-max rule: the argmax of ``logit / temperature + G`` with
``G = -log(-log(u))`` is a draw from ``softmax(logits / temperature)``
(``examples/granite_4_0_h_small-cuda/kernels/granite.cu:712-797``).  The reference draws ``u`` from cuRAND's Philox
stream keyed by its launch geometry; this build keys ``u`` by ``(seed, step, vocabulary index)`` through the
splitmix64 finaliser so that the draw does not depend on how the vocabulary is tiled or sharded.  This file restates
that generator and the pick with numpy integers, for the tests to compare the kernel against.  The product never
imports it.
"""
import numpy as np

_M64 = (1 << 64) - 1


def uniforms(seed: int, step: int, n: int, index_offset: int = 0) -> np.ndarray:
    """u_i in (0, 1), f64 (23 random bits), for vocabulary indices index_offset .. index_offset + n - 1."""
    with np.errstate(over="ignore"):
        idx = (np.arange(n, dtype=np.uint64) + np.uint64(index_offset) + np.uint64(1)) & np.uint64(0xFFFFFFFF)
        z = (np.uint64(seed & _M64) + np.uint64(0x9E3779B97F4A7C15) * idx
             + np.uint64(0xD1B54A32D192ED03) * np.uint64((step + 1) & 0xFFFFFFFF))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return ((z >> np.uint64(41)).astype(np.float64) + 0.5) * (1.0 / 8388608.0)


def gumbel_scores(logits: np.ndarray, temperature: float, seed: int, step: int, index_offset: int = 0) -> np.ndarray:
    """logit / T + Gumbel variate, f32 (logits: the bf16 logits as f32)."""
    u = uniforms(seed, step, logits.shape[0], index_offset)
    g = (-np.log(-np.log(u))).astype(np.float32)         # both logarithms in double, rounded once
    return (logits.astype(np.float32) / np.float32(temperature)).astype(np.float32) + g


def sample(logits: np.ndarray, temperature: float, seed: int, step: int, index_offset: int = 0) -> int:
    """Lowest index of the largest perturbed score."""
    return int(np.argmax(gumbel_scores(logits, temperature, seed, step, index_offset)))


def _bf16_keys(logits: np.ndarray) -> np.ndarray:
    """Order-preserving 16-bit keys of bf16 values given as f32 (the kernel's histogram index)."""
    bits = (logits.astype(np.float32).view(np.uint32) >> np.uint32(16)).astype(np.uint32)
    neg = (bits & np.uint32(0x8000)) != 0
    return np.where(neg, ~bits & np.uint32(0xFFFF), bits | np.uint32(0x8000)).astype(np.int64)


def nucleus_threshold(logits: np.ndarray, temperature: float, top_p: float) -> float:
    """The smallest logit value inside the nucleus: distinct values from the largest down, mass count * exp((value - max)
    / T) in f64, the first value at which the running mass reaches top_p * total."""
    keys = _bf16_keys(logits)
    counts = np.bincount(keys, minlength=65536)
    present = np.nonzero(counts)[0][::-1]                          # descending keys
    bits = np.where(present & 0x8000, present & 0x7FFF, ~present & 0xFFFF).astype(np.uint32) << np.uint32(16)
    values = bits.view(np.float32).astype(np.float64)
    mass = counts[present] * np.exp((values - values[0]) / np.float64(np.float32(temperature)))
    run = np.cumsum(mass)
    k = int(np.searchsorted(run, np.float64(np.float32(top_p)) * run[-1], side="left"))
    return float(values[min(k, len(values) - 1)])


def sample_top_p(logits: np.ndarray, temperature: float, top_p: float, seed: int, step: int) -> int:
    """Gumbel-max pick among the tokens whose logit is at least the nucleus threshold (lowest index on ties)."""
    tau = nucleus_threshold(logits, temperature, top_p)
    scores = gumbel_scores(logits, temperature, seed, step)
    scores = np.where(logits.astype(np.float32) >= np.float32(tau), scores, -np.inf)
    return int(np.argmax(scores))
