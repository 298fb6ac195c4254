"""How a MoE decode step is split over the GPUs of one node (one process per GPU).

The reference is single-GPU throughout, so none of this has a counterpart there.  The split follows
what each piece is bound by at batch 1:

* routed experts -- expert ``e`` lives on rank ``e % n`` as local expert ``e // n``.  The router is
  replicated, so every rank sees the same indices (integer parity is untouched) and computes only the
  selected experts it owns;
* shared expert -- gate/up rows and the matching down columns are sliced ``1/n`` each;
* both leave an un-rounded f32 partial per rank; ONE all-reduce per MoE block sums them before any
  rounding is applied, so the only difference from one GPU is f32 summation order;
* lm_head -- vocabulary rows sliced ``1/n``; each rank reduces its slice to (best logit, global index)
  and an all-gather of ``n`` pairs feeds the final pick (lowest index on ties);
* the mixers (Mamba-2 / attention) and their state are replicated.
"""
from __future__ import annotations

import torch


def expert_owner(e: int, world: int) -> int:
    return e % world


def local_experts(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """``[experts, ...]`` slab -> the experts this rank owns, in local order (``e // world``)."""
    if w.shape[0] % world:
        raise ValueError(f"{w.shape[0]} experts do not divide over {world} ranks")
    return w[rank::world].contiguous()


def shared_slices(w_in: torch.Tensor, w_out: torch.Tensor, rank: int, world: int):
    """``w_shared_in [2*IS, H]`` (gate rows then up rows), ``w_shared_out [H, IS]`` -> this rank's
    ``[2*IS/n, H]`` (its gate rows then its up rows) and ``[H, IS/n]``."""
    two_is = w_in.shape[0]
    inter = two_is // 2
    if inter % world or (inter // world) % 8:
        raise ValueError(f"shared intermediate size {inter} does not slice over {world} ranks in multiples of 8")
    per = inter // world
    lo, hi = rank * per, (rank + 1) * per
    local_in = torch.cat([w_in[lo:hi], w_in[inter + lo: inter + hi]], dim=0).contiguous()
    return local_in, w_out[:, lo:hi].contiguous()


def vocab_slice(vocab: int, rank: int, world: int) -> tuple[int, int]:
    if vocab % world:
        raise ValueError(f"vocabulary {vocab} does not divide over {world} ranks")
    per = vocab // world
    return rank * per, (rank + 1) * per


def pick_from_pairs(pairs: torch.Tensor) -> int:
    """Host statement of the final pick: pairs ``[world, 2]`` of (logit, index); highest logit, then lowest index."""
    best_v, best_i = float("-inf"), 2 ** 31
    for v, i in pairs.tolist():
        if v > best_v or (v == best_v and int(i) < best_i):
            best_v, best_i = v, int(i)
    return best_i
