"""What every fixed-address decode session shares: token history and position on the device,
one captured step, and the generate loop."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import lib


@dataclass
class Generated:
    tokens: list
    seconds: float
    prompt_seconds: float
    prompt_steps: int

    @property
    def tokens_per_second(self) -> float:
        return len(self.tokens) / self.seconds


class DecodeSession:
    """Subclasses set ``device, max_ctx, tokens, pos, counters, args`` (a ctypes step-args struct with
    an ``n_prompt`` field) and implement ``step()``."""

    graph = None
    n_prompt = 0
    eos_ids = None
    stop_at = None

    def step(self) -> None:
        raise NotImplementedError

    def reset(self, prompt_ids) -> None:
        """Start a sequence: token history = prompt, position 0.  The cache needs no clearing: a step
        only reads positions below its own."""
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64).reshape(-1)
        if prompt.numel() == 0:
            raise ValueError("decode needs a prompt of at least one token")
        if prompt.numel() > self.max_ctx:
            raise ValueError(f"prompt of {prompt.numel()} tokens exceeds capacity {self.max_ctx}")
        self.tokens.zero_()
        self.tokens[: prompt.numel()] = prompt.to(self.device)
        self.pos.zero_()
        self.counters.zero_()
        if self.stop_at is not None:
            self.stop_at.zero_()
        if self.args.n_prompt != prompt.numel():
            self.args.n_prompt = int(prompt.numel())
            self.graph = None                         # the prompt length is baked into the capture
        self.n_prompt = int(prompt.numel())

    def set_eos(self, eos_ids) -> None:
        """End-of-sequence token ids (at most 16; empty: none).  Once a step picks one of them as a NEW token the
        sequence is over: the head kernel latches the slot in ``stop_at`` on the device and every later step leaves
        the token history and the position alone, so ``generate`` can replay its fixed number of steps without a
        host round trip and read where the sequence ended once, at the end (the reference loop asks the host every
        token: ``tests/models/orchestrator/causal_lm/generation.py:70-72``)."""
        from .. import lib
        ids = [int(t) for t in eos_ids]
        if len(ids) > 16:
            raise ValueError("at most 16 end-of-sequence ids")
        if not hasattr(self.args, "eos_ids"):
            raise NotImplementedError(f"{type(self).__name__} has no end-of-sequence latch")
        if getattr(self, "world", 1) > 1 and ids:
            raise NotImplementedError("the sharded step's pick exchange has no end-of-sequence latch")
        self.eos_ids = torch.tensor(ids, dtype=torch.int64, device=self.device) if ids else None
        if self.stop_at is None:
            self.stop_at = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.args.eos_ids = lib.ptr(self.eos_ids)
        self.args.n_eos = len(ids)
        self.args.stop_at = lib.ptr(self.stop_at) if ids else None
        self.graph = None                             # the pointers are baked into a capture

    def state_tensors(self) -> list:
        """Device tensors, besides the token history and the position, that a step updates in place and a later
        step reads again (recurrent state, convolution windows).  Cache rows are not listed: a step only reads
        rows below its own position, so rows written by later steps need no rolling back."""
        return []

    def snapshot(self) -> dict:
        """Copy of everything needed to return to the current position later with ``restore``."""
        return {"tokens": self.tokens.clone(), "pos": self.pos.clone(), "state": [t.clone() for t in self.state_tensors()],
                "stop_at": None if self.stop_at is None else self.stop_at.clone()}

    def restore(self, snap: dict) -> None:
        self.tokens.copy_(snap["tokens"]); self.pos.copy_(snap["pos"])
        if self.stop_at is not None and snap.get("stop_at") is not None:
            self.stop_at.copy_(snap["stop_at"])
        for dst, src in zip(self.state_tensors(), snap["state"]):
            dst.copy_(src)

    def capture(self) -> None:
        """Record one step into a CUDA graph (positions and tokens live on the device, so the same
        graph serves every step).  Three eager warm-up steps run first and are rolled back."""
        saved = self.snapshot()                       # the warm-up steps advance position and recurrent state
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                self.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.restore(saved)
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: a process group's watchdog thread may query CUDA events meanwhile
        with torch.cuda.graph(graph, capture_error_mode="thread_local"):
            self.step()
        torch.cuda.synchronize()
        self.restore(saved)
        self.graph = graph

    def step_host(self, pos: int, token_in: torch.Tensor, token_out: torch.Tensor) -> None:
        """One iteration of a host-driven generation loop (the reference's ``generation.decode``): the token id in
        ``token_in`` (pinned int64[1]) goes to ``tokens[pos]``, the captured step runs, its pick comes back in
        ``token_out`` (pinned int64[1]); returns when the stream has finished.  One C call: two 8-byte copies, one
        graph launch, one wait."""
        if self.graph is None:
            self.capture()
        if not (0 <= pos and pos + 1 < self.tokens.numel()):
            raise ValueError(f"position {pos} has no successor slot in a history of {self.tokens.numel()}")
        for t in (token_in, token_out):
            if t.is_cuda or not t.is_pinned() or t.dtype != torch.int64 or t.numel() != 1:
                raise ValueError("token_in / token_out must be pinned host int64 tensors of one element")
        base = self.tokens.data_ptr()
        lib.check(lib.load().tfb_graph_step_host(int(self.graph.raw_cuda_graph_exec()), base + 8 * pos, token_in.data_ptr(),
                                                 base + 8 * (pos + 1), token_out.data_ptr(), lib.stream()),
                  "tfb_graph_step_host")

    def generate_host(self, pos: int, steps: int, token_io: torch.Tensor) -> list:
        """*steps* iterations of ``step_host`` from position *pos* in one C call: ``token_io`` (pinned int64[1]) holds the
        token fed to the next step and receives each pick; the picks are returned."""
        if self.graph is None:
            self.capture()
        if not (0 <= pos and pos + steps < self.tokens.numel()):
            raise ValueError(f"positions {pos}..{pos + steps} exceed a history of {self.tokens.numel()}")
        if token_io.is_cuda or not token_io.is_pinned() or token_io.dtype != torch.int64 or token_io.numel() != 1:
            raise ValueError("token_io must be a pinned host int64 tensor of one element")
        out = torch.empty(max(steps, 1), dtype=torch.int64)
        lib.check(lib.load().tfb_graph_generate_host(int(self.graph.raw_cuda_graph_exec()), self.tokens.data_ptr(), pos, steps,
                                                     token_io.data_ptr(), out.data_ptr(), lib.stream()),
                  "tfb_graph_generate_host")
        return out[:steps].tolist()

    def run(self, steps: int, use_graph: bool = True) -> None:
        if use_graph and self.graph is None:
            self.capture()
        for _ in range(steps):
            self.graph.replay() if use_graph else self.step()

    def generate(self, prompt_ids, max_new: int, use_graph: bool = True, eos=None) -> Generated:
        """Walk the prompt, then continue greedily for *max_new* tokens; one sync at each end.  *eos*: token ids
        that end the sequence; the tokens before the first of them are returned (``set_eos``)."""
        if eos is not None:
            self.set_eos(eos)
        self.reset(prompt_ids)
        n_prompt = self.n_prompt
        if n_prompt + max_new > self.max_ctx + 1:
            raise ValueError(f"{n_prompt}+{max_new} tokens exceed capacity {self.max_ctx}")
        if use_graph and self.graph is None:
            self.capture()
        start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        start.record()
        self.run(n_prompt - 1, use_graph)          # positions 0 .. n_prompt-2: no sampling needed
        mid.record()
        self.run(max_new, use_graph)               # step at position p writes token p+1
        end.record()
        torch.cuda.synchronize()
        out = self.tokens[n_prompt: self.generated_end(n_prompt + max_new)].tolist()
        return Generated(out, mid.elapsed_time(end) / 1e3, start.elapsed_time(mid) / 1e3, n_prompt)

    def generated_end(self, limit: int) -> int:
        """Index in the token history one past the last generated token that counts: the slot of the end-of-sequence
        token if one was picked (it is not part of the output), else *limit*."""
        stop = int(self.stop_at) if self.stop_at is not None and self.eos_ids is not None else 0
        return min(stop, limit) if stop else limit
