"""The end-of-sequence latch: a graph-replayed ``generate`` stops where the reference loop would
(``tests/models/orchestrator/causal_lm/generation.py:70-72``: the end token is not part of the output) without
asking the host after every token."""
import pytest
import torch

from tilefoundry_b200.authored.weights import random_weights
from tilefoundry_b200.runtime import DictResource




@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def _sessions(dev):
    from tilefoundry_b200.authored import granite_4_0_h_small as gr, minicpm3_4b as m, qwen3_1_7b as q
    from tilefoundry_b200.engine.granite import GraniteSession
    from tilefoundry_b200.engine.minicpm3 import MiniCPM3Session
    from tilefoundry_b200.engine.qwen3 import KERNEL_FUSED, Qwen3Session
    cuda = lambda w: {k: v.to(dev) for k, v in w.items()}
    wq = cuda(q.tie_head(random_weights(q.build(q.QWEN3_SMALL), seed=5, std=0.05)))
    yield "qwen3 one launch", Qwen3Session(q.QWEN3_SMALL, DictResource(wq), max_ctx=128, device=dev, kernel=KERNEL_FUSED), q.QWEN3_SMALL.vocab_size
    yield "qwen3 launch per kernel", Qwen3Session(q.QWEN3_SMALL, DictResource(wq), max_ctx=128, device=dev, kernel=0), q.QWEN3_SMALL.vocab_size
    wm = cuda(m.tie_head(random_weights(m.build(m.MINICPM3_TINY), seed=5, std=0.05)))
    yield "minicpm3", MiniCPM3Session(m.MINICPM3_TINY, DictResource(wm), max_ctx=128, device=dev), m.MINICPM3_TINY.vocab_size
    wg = cuda(random_weights(gr.build(gr.GRANITE_TINY), seed=5, std=0.05, overrides=gr.weight_overrides))
    yield "granite", GraniteSession(gr.GRANITE_TINY, DictResource(wg), max_ctx=128, device=dev), gr.GRANITE_TINY.vocab_size


@pytest.mark.gpu
def test_generate_stops_at_the_first_end_token(dev):
    for name, sess, vocab in _sessions(dev):
        prompt = torch.randint(0, vocab, (9,), generator=torch.Generator().manual_seed(3))
        free = sess.generate(prompt, 60).tokens
        assert len(free) == 60
        # an end token whose FIRST appearance is as late in the run as this run offers (random small models soon
        # repeat themselves), and one that never appears
        j = max(i for i in range(60) if free[i] not in free[:i])
        absent = next(t for t in range(vocab) if t not in free)
        for use_graph in (True, False):
            got = sess.generate(prompt, 60, use_graph=use_graph, eos=[free[j], absent]).tokens
            assert got == free[:j], f"{name} (graph={use_graph}): stopped after {len(got)} tokens, expected {j}"
            assert int(sess.stop_at) == 9 + j and int(sess.pos) == 9 + j, name
            assert int(sess.tokens[9 + j]) == free[j], name                # the end token itself sits in its slot
        # an end id inside the PROMPT does not stop anything: only picked tokens count
        if int(prompt[3]) not in free[:20]:
            assert sess.generate(prompt, 20, eos=[int(prompt[3])]).tokens == free[:20], name
        # without end ids the latch is off again
        assert sess.generate(prompt, 60, eos=[]).tokens == free, name


def test_latch_arguments_are_validated():
    import ctypes as C
    from tilefoundry_b200 import lib
    P = 0x10000
    a = lib.LmHeadArgs(w=P, x=P, token_out=P, scratch_val=P, scratch_idx=P, counter=P, n=1024, k=256, prologue=0, eps=1e-6,
                       x_scale=1.0, out_scale=1.0, eos_ids=P, n_eos=3, stop_at=None)
    assert lib.load().tfb_lm_head_argmax(C.byref(a), None) == 1          # end ids without a latch word: TFB_EINVAL
    a.stop_at, a.n_eos = P, 17
    assert lib.load().tfb_lm_head_argmax(C.byref(a), None) == 1          # more than 16 ids
