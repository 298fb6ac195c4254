"""The four decode steps at their PUBLISHED sizes (every layer, every expert, the whole vocabulary), where the CPU
evaluator cannot follow in test time: properties that do not depend on size.  A greedy run is repeatable; replaying
the captured graph gives the tokens of eager launches; returning to a snapshot and decoding again gives the same
continuation (the recurrent state, the cache rows and the token history all roll back); an end-of-sequence id cuts
the run where that token first appears.  Parity with the evaluator itself is held at these widths on shortened stacks
(``test_granite_gpu.py``, ``test_qwen3_5_gpu.py``, ``test_minicpm3_gpu.py``) and at full depth for Qwen3
(``test_qwen3_gpu.py``)."""
import pytest
import torch

from tilefoundry_b200.runtime import DictResource

pytestmark = pytest.mark.gpu
KEYS = ["qwen3_1_7b", "minicpm3_4b", "granite_4_0_h_small", "qwen3_5_35b_a3b"]


def _workload(key):
    from tilefoundry_b200.authored.weights import random_weights_on
    if key == "qwen3_1_7b":
        from tilefoundry_b200.authored import qwen3_1_7b as a
        from tilefoundry_b200.engine.qwen3 import Qwen3Session as S
        cfg, over = a.QWEN3_1_7B, None
    elif key == "minicpm3_4b":
        from tilefoundry_b200.authored import minicpm3_4b as a
        from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session as S
        cfg, over = a.MINICPM3_4B, None
    elif key == "granite_4_0_h_small":
        from tilefoundry_b200.authored import granite_4_0_h_small as a
        from tilefoundry_b200.engine.granite import GraniteSession as S
        cfg, over = a.GRANITE_4_0_H_SMALL, a.weight_overrides
    else:
        from tilefoundry_b200.authored import qwen3_5_35b_a3b as a
        from tilefoundry_b200.engine.qwen3_5 import Qwen35Session as S
        cfg, over = a.QWEN3_5_35B_A3B, a.weight_overrides
    dev = torch.device("cuda:0")
    tied = hasattr(a, "tie_head")
    w = random_weights_on(a.build(cfg), dev, seed=0, std=0.02, overrides=over, skip=("w_head",) if tied else ())
    if tied:
        w["w_head"] = w["w_embed"].t()
    vocab = cfg.vocab if key == "qwen3_5_35b_a3b" else cfg.vocab_size
    return S(cfg, DictResource(w), max_ctx=256, device=dev), vocab


@pytest.mark.parametrize("key", KEYS)
def test_full_size_step_is_repeatable_and_rolls_back(key):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    free, _ = torch.cuda.mem_get_info()
    if key == "qwen3_5_35b_a3b" and free < 90e9:
        pytest.skip("needs 90 GB of device memory")
    sess, vocab = _workload(key)
    prompt = torch.randint(0, vocab, (24,), generator=torch.Generator().manual_seed(5))
    first = sess.generate(prompt, 40).tokens
    assert len(first) == 40 and all(0 <= t < vocab for t in first)
    assert sess.generate(prompt, 40).tokens == first                        # repeatable
    assert sess.generate(prompt, 40, use_graph=False).tokens == first       # graph replay == eager launches
    # back to the state after 10 generated tokens, then the same continuation
    sess.reset(prompt)
    sess.run(len(prompt) - 1 + 10, True)
    snap = sess.snapshot()
    sess.run(30, True)
    torch.cuda.synchronize()
    assert sess.tokens[len(prompt): len(prompt) + 40].tolist() == first
    sess.restore(snap)
    sess.run(30, False)
    torch.cuda.synchronize()
    assert sess.tokens[len(prompt): len(prompt) + 40].tolist() == first
    # an end id stops the run where that token first appears
    j = max(i for i in range(40) if first[i] not in first[:i])
    assert sess.generate(prompt, 40, eos=[first[j]]).tokens == first[:j]
    if hasattr(sess, "check_status"):
        sess.check_status()
    del sess
    torch.cuda.empty_cache()
