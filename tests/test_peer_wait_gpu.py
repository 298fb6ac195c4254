"""The exchange kernels' waits are bounded: a peer that never publishes its flag makes the kernel give up after
about a second, report which peer it waited for in ``*status`` and return, and the context stays usable.

The absent peer is a pair of buffers on the same GPU that nothing writes (no second process, no second kernel): the
kernel under test is the only launch in flight, so nothing here waits on another launch.  A healthy exchange over
real peers is covered by ``tests/multi_gpu_granite.py`` and ``tests/multi_gpu_qwen35.py``."""
import ctypes as C
import time

import pytest
import torch

from tilefoundry_b200 import lib

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_pick_allgather_gives_up_on_an_absent_peer():
    so, dev = lib.load(), torch.device("cuda:0")
    pair = torch.tensor([1.5, 7.0], device=dev)
    inbox = [torch.zeros(2 * 2 * 2, device=dev) for _ in range(2)]
    flags = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(2)]
    epoch, status = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    picked = torch.full((1,), -1, dtype=torch.int64, device=dev)
    a = lib.PickAllgatherArgs(pair=_ptr(pair), epoch=_ptr(epoch), status=_ptr(status), picked=_ptr(picked),
                              n_prompt=0, max_tokens=0, rank=0, world=2, pdl=0)
    for r in range(2):
        a.inbox[r], a.flags[r] = inbox[r].data_ptr(), flags[r].data_ptr()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    lib.check(so.tfb_pick_allgather(C.byref(a), lib.stream()), "tfb_pick_allgather")
    torch.cuda.synchronize()                                   # returns: the wait ran out, nothing faulted
    took = time.perf_counter() - t0
    assert int(status.item()) == 0x300 + 1, hex(int(status.item()))         # "gave up waiting for rank 1's pick"
    assert 0.5 < took < 10.0, took
    assert int(flags[1][0].item()) == 1                        # this rank's own flag for the epoch was published
    assert int(epoch.item()) == 1
    # the context is intact: an ordinary kernel of the library still runs and is right
    x = torch.arange(8, device=dev, dtype=torch.float32)
    assert float((x * 2).sum().item()) == 56.0


def test_moe_allreduce_gives_up_on_an_absent_peer():
    so, dev, H = lib.load(), torch.device("cuda:0"), 256
    partial = torch.ones(2 * H, device=dev)
    inbox = [torch.zeros(2 * 2 * 2 * H, device=dev) for _ in range(2)]
    flags = [torch.zeros(2 * 1, dtype=torch.int32, device=dev) for _ in range(2)]
    epoch, status = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    out = torch.zeros(H, dtype=torch.bfloat16, device=dev)
    a = lib.MoeAllreduceArgs(partial=_ptr(partial), epoch=_ptr(epoch), status=_ptr(status), out=_ptr(out), hidden=H,
                             rank=0, world=2, has_shared=1, res_scale=1.0, pdl=0)
    for r in range(2):
        a.inbox[r], a.flags[r] = inbox[r].data_ptr(), flags[r].data_ptr()
    lib.check(so.tfb_moe_allreduce_finalize(C.byref(a), lib.stream()), "tfb_moe_allreduce_finalize")
    torch.cuda.synchronize()
    assert int(status.item()) == 0x200 + 1, hex(int(status.item()))         # "gave up waiting for rank 1's slice"
    # this rank's slice did land in the peer's inbox before the wait (epoch 1 -> parity 1, slot of rank 0)
    assert torch.equal(inbox[1][(1 * 2 + 0) * 2 * H:(1 * 2 + 0) * 2 * H + 2 * H], partial)
    # a second call on the same buffers, with the "peer" now answering (flag and inbox written by the host), succeeds
    status.zero_()
    inbox[0][(0 * 2 + 1) * 2 * H:(0 * 2 + 1) * 2 * H + 2 * H] = 2.0          # epoch 2 -> parity 0, slot of rank 1
    flags[0][1 * 1 + 0] = 2
    torch.cuda.synchronize()
    lib.check(so.tfb_moe_allreduce_finalize(C.byref(a), lib.stream()), "tfb_moe_allreduce_finalize")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(out.float().cpu(), torch.full((H,), 6.0))            # (1 + 2) routed + (1 + 2) shared
