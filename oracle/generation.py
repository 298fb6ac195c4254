"""TEST INFRASTRUCTURE.  The reference's greedy decode loop over token ids.

Restates ``tests/models/orchestrator/causal_lm/generation.py:41-85`` without the
tokenizer: walk the prompt one token per step, then sample greedily
(``torch.argmax``, lowest index on ties) ``max_new`` times.  Returns the token ids,
per-step logits if asked, and the decode-only seconds.
"""
from __future__ import annotations

from time import perf_counter

import torch


def greedy(logits) -> int:
    return int(torch.argmax(logits).item())


def _forward_traced(loaded, trace, token_ids, cos, sin, pos_ids, *rest):
    """``forward`` with the residual stream after every layer recorded (same calls, same order).
    Covers the attention-cache models, whose step takes ``(token, cos, sin, pos, *scalars, caches)``
    and whose layers take ``(hidden, cos, sin, pos, k_cache, v_cache, *scalars)``."""
    *scalars, caches = rest
    hidden = loaded.embed(token_ids)
    entries, rows = [], []
    for layer, (k_cache, v_cache) in zip(loaded.modules, caches):
        hidden, k_new, v_new = layer(hidden, cos, sin, pos_ids, k_cache, v_cache, *scalars)
        entries.append((k_new, v_new))
        rows.append(hidden.reshape(-1))
    normed = loaded.final_rms_norm(hidden)
    rows.append(normed.reshape(-1))
    trace.append(torch.stack(rows))
    return loaded.lm_head(normed), tuple(entries)


def decode_ids(loaded, prompt_ids, max_new, device="cpu", keep_logits=False, keep_hidden=False, caches=None,
               logits=None):
    """*caches* / *logits*: continue a run whose ``prompt_ids`` have all been walked already (the ``caches`` and
    ``last_logits`` an earlier call returned for exactly these ids); the prompt loop is then skipped."""
    prompt_ids = torch.as_tensor(prompt_ids, dtype=torch.int64)
    n_prompt = prompt_ids.numel()
    input_ids = torch.empty(n_prompt + max_new, dtype=torch.int64)
    input_ids[:n_prompt] = prompt_ids
    resumed = caches is not None
    if not resumed:
        caches = loaded.init_caches(device=device)
    kept, trace = [], []
    t_prompt = perf_counter()
    for step in range(0 if resumed else n_prompt):
        args = loaded.prepare_inputs_for_generation(input_ids[: step + 1], step, caches, device=device)
        logits, fresh = _forward_traced(loaded, trace, *args) if keep_hidden else loaded.forward(*args)
        caches = loaded.append_cache(caches, fresh)
        if keep_logits:
            kept.append(logits)
    t_prompt = perf_counter() - t_prompt
    out = []
    started = perf_counter()
    for step in range(max_new):
        token = greedy(logits)
        out.append(token)
        input_ids[n_prompt + step] = token
        pos = n_prompt + step
        args = loaded.prepare_inputs_for_generation(input_ids[: pos + 1], pos, caches, device=device)
        logits, fresh = _forward_traced(loaded, trace, *args) if keep_hidden else loaded.forward(*args)
        caches = loaded.append_cache(caches, fresh)
        if keep_logits:
            kept.append(logits)
    seconds = perf_counter() - started
    return {"tokens": out, "seconds": seconds, "prompt_seconds": t_prompt, "logits": kept,
            "caches": caches, "hidden": trace, "last_logits": logits}
