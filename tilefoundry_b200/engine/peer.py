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
