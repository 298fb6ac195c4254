"""Symmetric buffers for the exchange kernels of a sharded step (``csrc/collective.cu``): every rank's inboxes and
flags, mapped into every process through ``torch.distributed._symmetric_memory``."""
from __future__ import annotations

import torch


class PeerBuffers:
    """``mode`` is ``"peer"`` when the buffers are mapped, else ``"nccl"`` (the caller then keeps to NCCL collectives).
    ``reduce_inbox[r]``, ``reduce_flags[r]``, ``pick_inbox[r]``, ``pick_flags[r]`` are addresses of rank r's regions as
    mapped in this process; ``reduce_epoch``, ``pick_epoch``, ``status`` are this rank's local counters."""

    def __init__(self, group, rank: int, world: int, hidden: int, device, want: str | None):
        import torch.distributed as dist
        self.mode = "nccl"
        if want == "nccl":
            return
        n_cta = (hidden + 255) // 256
        words = [2 * world * 2 * hidden, world * n_cta, 2 * world * 2, world]   # reduce inbox / flags, pick inbox / flags
        words = [(w + 63) // 64 * 64 for w in words]                             # keep every region 256-byte aligned
        ok = torch.ones(1, device=device)
        try:
            import os
            # the exchange kernels use plain peer loads and stores; keep the buffer off any NVLink multicast object
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            self._sym = symm.empty(sum(words), dtype=torch.float32, device=device)
            self._sym.zero_()
            self._handle = symm.rendezvous(self._sym, group)
            ptrs = [int(p) for p in self._handle.buffer_ptrs]
            why = "another rank could not map symmetric memory"
        except Exception as exc:                                                 # noqa: BLE001 -- "not available here"
            why, ptrs = repr(exc), None
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)                   # all ranks agree on the mode
        if float(ok) == 0.0:
            if want == "peer":
                raise RuntimeError(f"peer-memory collectives were requested but are unavailable: {why}")
            return
        torch.cuda.synchronize()
        dist.barrier(group=group)                                                # every inbox and flag is zero before any push
        off = [0, words[0] * 4, (words[0] + words[1]) * 4, (words[0] + words[1] + words[2]) * 4]
        self.reduce_inbox = [p + off[0] for p in ptrs]
        self.reduce_flags = [p + off[1] for p in ptrs]
        self.pick_inbox = [p + off[2] for p in ptrs]
        self.pick_flags = [p + off[3] for p in ptrs]
        z = lambda n: torch.zeros(n, device=device, dtype=torch.int32)
        self.reduce_epoch, self.pick_epoch, self.status = z(n_cta), z(1), z(1)
        self.mode = "peer"


def leave_together(sessions=(), bound_s: float = 30.0) -> None:
    """End of a multi-rank run: every rank drops its captured graphs, finishes its GPU work, meets the others at a
    barrier and only then tears the process group down, so no rank is gone while a peer still pushes into its
    buffers.  A CUDA graph that recorded NCCL kernels holds a reference on the communicator, and the
    communicator's teardown waits until that reference is released -- destroying the process group while such a
    graph is alive therefore never returns; the graphs go first.  The teardown is bounded all the same: if it has
    not returned after *bound_s* seconds the process exits (its work is done and synchronised by then)."""
    import gc
    import os
    import sys
    import threading

    import torch.distributed as dist

    for s in sessions:
        s.graph = None
    gc.collect()
    torch.cuda.synchronize()
    if not dist.is_initialized():
        return
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    bound = threading.Timer(bound_s, lambda: os._exit(0))
    bound.daemon = True
    bound.start()
    dist.destroy_process_group()
    bound.cancel()
