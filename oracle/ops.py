"""TEST INFRASTRUCTURE.  The evaluator's op handlers as torch calls.

Each function cites the ``@register_eval`` handler it restates (paths under the
reference's ``src/tilefoundry/ir/hir/``).  Elementwise and reduce ops run at the
operand dtype (torch on CPU accumulates a bf16 reduction in f32 and rounds once);
a Python float literal takes its tensor partner's dtype (``parser/base.py:282-306``),
which is what torch's scalar promotion does too.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "f64": torch.float64,
      "i32": torch.int32, "i64": torch.int64}


def cast(x, dtype):                       # tensor/cast.py
    return x.to(DT[dtype])


def matmul(a, b):                         # nn/matmul.py:188-192
    return torch.matmul(a, b)


def rms_norm(x, w, eps):                  # nn/rms_norm.py:103-110 (f32 throughout, one rounding)
    xf, wf = x.float(), w.float()
    ms = xf.pow(2).mean(dim=-1, keepdim=True)
    return (xf * torch.rsqrt(ms + eps) * wf).to(x.dtype)


def rope(q, k, cos_cache, sin_cache, pos_ids):   # nn/rope.py:147-172 (rotate-half, f32 math)
    qf, kf = q.float(), k.float()
    pos = pos_ids.reshape(-1).long()
    cos = cos_cache[pos].float()[None, :, None, :]
    sin = sin_cache[pos].float()[None, :, None, :]

    def rot(x):
        h = x.shape[-1] // 2
        return torch.cat((-x[..., h:], x[..., :h]), dim=-1)

    return (qf * cos + rot(qf) * sin).to(q.dtype), (kf * cos + rot(kf) * sin).to(k.dtype)


def softmax(x, axis=-1):                  # nn/softmax.py:65-69
    return torch.softmax(x.float(), dim=axis).to(x.dtype)


def silu(x):                              # nn/silu.py:39
    return F.silu(x)


def sigmoid(x):                           # nn/sigmoid.py:36
    return torch.sigmoid(x)


def softplus(x):                          # math/softplus.py:38
    return F.softplus(x)


def rsqrt(x):                             # math/unary.py:73-91
    return torch.rsqrt(x)


def exp(x):
    return torch.exp(x)


def reduce(x, axes, keepdim, kind):       # tensor/reduce.py:124-147
    axes = tuple(axes)
    if kind == "max" and any(x.shape[a] == 0 for a in axes):
        # empty-axis max is the least representable value, -inf where the dtype holds it
        shape = list(x.shape)
        for a in axes:
            shape[a] = 1
        out = torch.full(shape, float("-inf"), dtype=x.dtype)
        return out if keepdim else out.squeeze(dim=axes)
    if kind == "mean":
        return x.mean(dim=axes, keepdim=keepdim)
    if kind == "sum":
        return x.sum(dim=axes, keepdim=keepdim)
    if kind == "max":
        return x.amax(dim=axes, keepdim=keepdim)
    if kind == "abs_max":
        return x.abs().amax(dim=axes, keepdim=keepdim)
    raise ValueError(kind)


def maximum(a, b):                        # math/binary.py:192-214
    return torch.maximum(a, b)


def topk(x, k, dim=-1, largest=True, sorted=True):   # tensor/topk.py:269-291 (indices i64)
    return torch.topk(x, k, dim=dim, largest=largest, sorted=sorted)


def argmax(x, dim=None, keepdim=False):   # tensor/argmax.py:99-102 (lowest index on ties)
    return torch.argmax(x, dim=dim, keepdim=keepdim)


def index_select(x, idx, dim):            # tensor/index_select.py:141-149
    return torch.index_select(x, dim, idx.long())


def repeat_interleave(x, repeats, axis):  # tensor/repeat_interleave.py
    return torch.repeat_interleave(x, repeats, dim=axis)


def cache_update(cache, new, pos):        # tensor/cache_update.py:228-245 (value semantics)
    s = new.shape[1]
    p = int(pos)
    if p + s > cache.shape[1]:
        raise ValueError(f"cache_update: position {p}+{s} exceeds capacity {cache.shape[1]}")
    out = cache.clone()
    out[:, p:p + s] = new[:, :s]
    return out
