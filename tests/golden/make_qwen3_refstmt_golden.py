"""Generate ``qwen3_refstmt.pt``: outputs of the REFERENCE's own torch statements of the Qwen3 decode arithmetic,
for ``tests/test_oracle_pins.py`` to hold ``oracle/qwen3_1_7b.py`` to.

Two sources in the reference checkout, both plain torch; they are lifted from their files with ``ast`` at
generation time (the files import the example's kernel library at module level, which this image cannot) and
executed unchanged -- none of their text is stored here:

* ``examples/qwen3_1_7b-tilelang/fast/arbitrate.py:22-56`` ``f64_attention``: the authored attention function in
  float64, nothing rounded anywhere;
* ``examples/qwen3_1_7b-tilelang/fast/test_kernels.py``: the per-kernel statements the reference judges its own
  kernels by, at the published widths -- ``rms_norm`` (``:32-39``), the per-head norm ``nrm`` and ``_rope_ref``
  (``:96-130``), ``_attn_ref`` (``:133-140``), ``silu_mul`` (``:165-172``) -- composed here in the order the
  authored ``self_attention`` / ``mlp`` compose them, projections as ``x.float() @ w.float()`` rounded to bf16,
  the way ``t_gemv`` states a projection (``:57-66``).

Inputs are seeded, so only the outputs are stored.  Run where the reference checkout is mounted:

    python tests/golden/make_qwen3_refstmt_golden.py <path to the reference checkout>
"""
from __future__ import annotations

import ast
import dataclasses
import math
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tilefoundry_b200.authored import qwen3_1_7b as q            # noqa: E402
from tilefoundry_b200.authored.weights import random_weights    # noqa: E402

OUT = Path(__file__).with_name("qwen3_refstmt.pt")
SEED_W, SEED_X = 0, 1
F64_CONTEXTS = (0, 1, 37)
WIDE_CTX = 37
#: one layer at the published widths (small vocabulary: the head is not part of these statements)
WIDE = dataclasses.replace(q.QWEN3_1_7B, num_hidden_layers=1, vocab_size=1024)


def lift(path: Path, functions=(), nested=(), expressions=()):
    """Definitions and expressions of *path*, by name, executed in a namespace that holds torch only.
    *nested*: ``(outer function, inner function)``; *expressions*: ``(function, assigned name)`` -> the
    right-hand side of that assignment as a callable of a namespace dict."""
    tree = ast.parse(path.read_text())
    ns = {"torch": torch, "math": math}
    outer = {n.name: n for n in tree.body if isinstance(n, ast.FunctionDef)}
    for name in functions:
        exec(compile(ast.Module([outer[name]], []), str(path), "exec"), ns)
    for fn, inner in nested:
        node = next(n for n in ast.walk(outer[fn]) if isinstance(n, ast.FunctionDef) and n.name == inner)
        exec(compile(ast.Module([node], []), str(path), "exec"), ns)
    exprs = {}
    for fn, target in expressions:
        node = next(n for n in ast.walk(outer[fn]) if isinstance(n, ast.Assign)
                    and isinstance(n.targets[0], ast.Name) and n.targets[0].id == target)
        code = compile(ast.Expression(node.value), str(path), "eval")
        exprs[(fn, target)] = lambda env, code=code: eval(code, {**ns, **env})
    return ns, exprs


def layer0(weights):
    return {k.split(".", 1)[1]: v for k, v in weights.items() if k.startswith("layer0.")}


def inputs(cfg, ctx, seed):
    g = torch.Generator().manual_seed(seed)
    hidden = (torch.randn(1, 1, cfg.hidden_size, generator=g)).to(torch.bfloat16)
    kc = torch.randn(1, ctx, cfg.num_key_value_heads, cfg.head_dim, generator=g).to(torch.bfloat16)
    vc = torch.randn(1, ctx, cfg.num_key_value_heads, cfg.head_dim, generator=g).to(torch.bfloat16)
    return hidden, kc, vc


@torch.no_grad()
def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_qwen3_refstmt_golden.py <path to the reference checkout>")
    fast = Path(sys.argv[1]) / "examples" / "qwen3_1_7b-tilelang" / "fast"
    out = {"seed_w": SEED_W, "seed_x": SEED_X, "f64_contexts": F64_CONTEXTS, "wide_ctx": WIDE_CTX}

    # ---- the authored attention in float64 (arbitrate.py), small instance, three contexts --------------------
    arb, _ = lift(fast / "arbitrate.py", functions=("f64_attention",))
    cfg = q.QWEN3_TINY
    w = layer0(q.tie_head(random_weights(q.build(cfg), seed=SEED_W, std=0.05)))
    cos, sin = q.rope_tables(cfg)
    scale = torch.full((1, 1, 1, 1), cfg.head_dim ** -0.5, dtype=torch.bfloat16)
    for ctx in F64_CONTEXTS:
        hidden, kc, vc = inputs(cfg, ctx, SEED_X + ctx)
        out[f"f64_attention_ctx{ctx}"] = arb["f64_attention"](hidden, w, cos, sin, ctx, kc, vc, scale, cfg)

    # ---- the per-kernel statements (test_kernels.py) at the published widths, composed as the authored layer ----
    D, H, I = WIDE.head_dim, WIDE.hidden_size, WIDE.intermediate_size
    HQ, HKV, EPS = WIDE.num_attention_heads, WIDE.num_key_value_heads, WIDE.rms_norm_eps
    T, E = lift(fast / "test_kernels.py", functions=("_rope_ref", "_attn_ref"), nested=(("t_qk_rope_cache", "nrm"),),
                expressions=(("t_rms_norm", "ref"),))
    T.update(D=D, H=H, HQ=HQ, HKV=HKV, EPS=EPS, I=I)
    # (silu_mul's statement is the argument of report(...) in t_silu_mul, not an assignment: lifted separately)
    tk = ast.parse((fast / "test_kernels.py").read_text())
    silu_fn = next(n for n in tk.body if isinstance(n, ast.FunctionDef) and n.name == "t_silu_mul")
    call = next(n for n in ast.walk(silu_fn) if isinstance(n, ast.Call) and getattr(n.func, "id", "") == "report")
    silu_code = compile(ast.Expression(call.args[2]), "test_kernels.py", "eval")
    silu_mul = lambda g, u: eval(silu_code, {"torch": torch, "g": g, "u": u})
    rms = lambda x, g: E[("t_rms_norm", "ref")]({"x32": x.float(), "g": g, "EPS": EPS})
    proj = lambda x, wm: (x.float() @ wm.float()).to(torch.bfloat16)          # t_gemv's statement of a projection

    w = layer0(q.tie_head(random_weights(q.build(WIDE), seed=SEED_W, std=0.02)))
    cos, sin = q.rope_tables(WIDE)
    hidden, kc, vc = inputs(WIDE, WIDE_CTX, SEED_X)
    x = rms(hidden.reshape(H), w["gamma_in"])
    qr, kr, vr = (proj(x, w[n][0]) for n in ("w_q", "w_k", "w_v"))
    q_rot = T["_rope_ref"](T["nrm"](qr.float().view(HQ, D), w["gamma_q"]), cos, sin, WIDE_CTX)
    k_rot = T["_rope_ref"](T["nrm"](kr.float().view(HKV, D), w["gamma_k"]), cos, sin, WIDE_CTX)
    k_all = torch.cat([kc[0], k_rot.view(1, HKV, D)], 0)
    v_all = torch.cat([vc[0], vr.view(1, HKV, D)], 0)
    attn = T["_attn_ref"](q_rot, k_all, v_all, WIDE_CTX + 1)
    out["wide_attention_out"] = proj(attn, w["w_o"][0])
    out["wide_k_new"], out["wide_v_new"] = k_rot.view(1, 1, HKV, D), vr.view(1, 1, HKV, D)
    xn = rms(hidden.reshape(H), w["gamma_post"])
    out["wide_mlp_out"] = proj(silu_mul(proj(xn, w["w_gate"][0]), proj(xn, w["w_up"][0])), w["w_down"][0])
    out["wide_input_norm"] = x
    torch.save(out, OUT)
    print(f"wrote {OUT} ({OUT.stat().st_size} bytes): {sorted(k for k in out if isinstance(out[k], torch.Tensor))}")


if __name__ == "__main__":
    main()
