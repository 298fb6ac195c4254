"""A ``tilefoundry check``-compatible command for the twins of this repository.

    python -m tests.check_cli FILE.py:Selector[.child][.fn] --inputs random \\
        --out output[0] --fn allclose --atol 2e-2 --rtol 2e-2 [--out output[1] --fn equal] [--dim ctx_len=24] [--json]

Takes the arguments the reference's own command takes (``src/tilefoundry/cli/check.py:52-88``): the
subject as ``FILE.py:Selector``, ``--inputs random``, and the comparison as an ordered run of ``--out`` /
``--fn`` / bounds, where every ``--fn`` applies to the ``--out`` before it and every bound to the ``--fn``
before it (``:30-49``).  As there (``:303-368``) activations are one seeded draw (seed 0) from the declared
types and weights are drawn the first time either side asks for them and cached, so both sides are handed
the same tensors; the two sides are the twin loaded from that resource and the evaluator loaded from it
(``:498-523``); the verdict is ``runtime.check``'s, printed as the reference prints it -- one block per
output with every measured value, ``PASS`` / ``FAIL`` last -- or as one JSON object with ``--json``
(``:697-770``).  Exit status 0 on PASS, 1 on FAIL, 2 on a usage error.

What differs, and why: the reference resolves its subject through its parser and IR, which need packages
this image does not have; here ``FILE.py`` is one of ``tilefoundry_b200/twins/*.py``, ``Selector`` names a
twin factory or class in it (``make_twin``), followed by child and function names, and the evaluator side
is the CPU restatement under ``oracle/`` -- which only test code may import, hence this file's place under
``tests/``.  ``--config NAME`` picks one of the file's named configurations (default: the smallest).
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from tilefoundry_b200.runtime import measure                      # noqa: E402
from tilefoundry_b200.semantic import DimVar, to_torch_dtype      # noqa: E402

SEED = 0
#: twins file stem -> (authored module, oracle module, {config name: attribute}, default config)
MODELS = {
    "qwen3_1_7b": ("qwen3_1_7b", "qwen3_1_7b", {"tiny": "QWEN3_TINY", "small": "QWEN3_SMALL", "full": "QWEN3_1_7B"}),
    "minicpm3_4b": ("minicpm3_4b", "minicpm3_4b", {"tiny": "MINICPM3_TINY", "full": "MINICPM3_4B"}),
    "granite_4_0_h_small": ("granite_4_0_h_small", "granite_4_0_h_small",
                            {"tiny": "GRANITE_TINY", "full": "GRANITE_4_0_H_SMALL"}),
    "qwen3_5_35b_a3b": ("qwen3_5_35b_a3b", "qwen3_5_35b_a3b", {"tiny": "QWEN3_5_TINY", "full": "QWEN3_5_35B_A3B"}),
}
BOUNDS = sorted({b for p in measure.PREDICATES.values() for b in p.bounds})


class Ordered(argparse.Action):
    """Keeps ``--out`` / ``--fn`` / bounds in the order they were written (reference ``cli/check.py:30-49``)."""

    def __call__(self, parser, namespace, values, option_string=None):
        stated = getattr(namespace, "comparison", None)
        if stated is None:
            stated = []
            setattr(namespace, "comparison", stated)
        stated.append((self.dest, values))


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="check", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("source", metavar="SOURCE", help="FILE.py:Selector -- a twin, one of its children, or a function")
    ap.add_argument("--inputs", choices=("random",), default="random",
                    help="how activations and weights are made (no checkpoint is present here: random only)")
    ap.add_argument("--out", action=Ordered, metavar="OUTPUT",
                    help="which output the following --fn apply to: `output`, or `output[0]` `output[1]` ... in return order")
    ap.add_argument("--fn", action=Ordered, metavar="F", choices=sorted(measure.PREDICATES), help="a comparison to make")
    for bound in BOUNDS:
        ap.add_argument(f"--{bound}", action=Ordered, type=float, help=argparse.SUPPRESS)
    ap.add_argument("--dim", action="append", metavar="NAME=V", help="bind a dimension declared as a range")
    ap.add_argument("--config", default=None, help="named configuration of the model file (default: its smallest)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--json", action="store_true", help="machine-readable report")
    return ap


def expectations(comparison) -> dict:
    """``{output path: [Predicate, ...]}`` from the ordered options (reference ``cli/check.py`` ``expectations``)."""
    if not comparison:
        raise ValueError("no comparison requested: every output needs at least one --fn (there is no default bound)")
    expect: dict[str, list] = {}
    out = fn = None
    bounds: dict[str, float] = {}

    def close():
        nonlocal fn, bounds
        if fn is None:
            return
        cls = measure.PREDICATES[fn]
        missing = [b for b in cls.bounds if b not in bounds]
        if missing:
            raise ValueError(f"--fn {fn} needs {' '.join('--' + b for b in cls.bounds)}; missing {missing}")
        extra = [b for b in bounds if b not in cls.bounds]
        if extra:
            raise ValueError(f"--fn {fn} takes no --{extra[0]}")
        expect.setdefault(out, []).append(cls(**{b: bounds[b] for b in cls.bounds}))
        fn, bounds = None, {}

    for key, value in comparison:
        if key == "out":
            close()
            out = value
        elif key == "fn":
            close()
            if out is None:
                raise ValueError("--fn before any --out: say which output it applies to")
            fn = value
        else:
            if fn is None:
                raise ValueError(f"--{key} before any --fn")
            bounds[key] = value
    close()
    return expect


def draw(shape, dtype, generator, device="cpu") -> torch.Tensor:
    """One tensor of *dtype* from *generator* (reference ``cli/check.py:303-312``)."""
    td = to_torch_dtype(dtype)
    if td.is_floating_point:
        return torch.randn(tuple(shape), generator=generator, device=device).to(td)
    if td == torch.bool:
        return torch.randint(0, 2, tuple(shape), generator=generator, device=device).to(td)
    return torch.randint(0, 8, tuple(shape), generator=generator, device=device).to(td)


def extents(type_, dims) -> tuple:
    shape = []
    for extent in type_.shape:
        if isinstance(extent, DimVar):
            if extent.name not in dims:
                raise ValueError(f"shape {type_.shape} still states {extent.name} as a range; bind it with --dim")
            if not extent.admits(dims[extent.name]):
                raise ValueError(f"--dim {extent.name}={dims[extent.name]} is outside its declared range")
            extent = dims[extent.name]
        shape.append(int(extent))
    return tuple(shape)


class RandomWeights:
    """Each weight drawn the first time it is asked for, from its declared type, and cached, so the two sides of a
    comparison are handed the same draw (reference ``cli/check.py:335-368``)."""

    def __init__(self, module, generator, dims, drawn=None, prefix=""):
        self._module, self._generator, self._dims = module, generator, dims
        self._drawn = {} if drawn is None else drawn
        self._prefix = prefix

    def load(self, name):
        key = f"{self._prefix}{name}"
        if key not in self._drawn:
            declared = self._module.weights[name]
            value = draw(extents(declared, self._dims), declared.dtype, self._generator)
            if value.is_floating_point():
                value = value * 0.05 + (1.0 if name.rsplit(".", 1)[-1].startswith("gamma") else 0.0)
                value = value.to(to_torch_dtype(declared.dtype))
            self._drawn[key] = value
        return self._drawn[key]

    def load_group(self, name):
        return None

    def subtree(self, seg):
        for child in self._module.modules:
            if child.name == seg:
                return RandomWeights(child, self._generator, self._dims, self._drawn, f"{self._prefix}{seg}.")
        raise KeyError(seg)


class OnDevice:
    """The same resource with every tensor moved to the twin's device."""

    def __init__(self, inner, device):
        self._inner, self._device = inner, device

    def load(self, name):
        return self._inner.load(name).to(self._device)

    def load_group(self, name):
        return None

    def subtree(self, seg):
        return OnDevice(self._inner.subtree(seg), self._device)


def resolve(source: str, config: str | None):
    """``(label, twin class, oracle impl_for, remaining selector parts)`` of ``FILE.py:Selector``."""
    if ":" not in source:
        raise ValueError("SOURCE is FILE.py:Selector")
    path_s, selector = source.split(":", 1)
    path = Path(path_s)
    if not path.is_absolute():
        path = ROOT / path
    if not path.exists():
        raise ValueError(f"{path} does not exist")
    stem = path.stem
    if stem not in MODELS:
        raise ValueError(f"{path.name}: no evaluator restatement is known for this file; known: {sorted(MODELS)}")
    authored_name, oracle_name, configs = MODELS[stem]
    authored = importlib.import_module(f"tilefoundry_b200.authored.{authored_name}")
    name = config or next(iter(configs))
    if name not in configs:
        raise ValueError(f"--config {name}: {path.name} has {sorted(configs)}")
    cfg = getattr(authored, configs[name])
    try:                                          # a file of this repository is imported under its package name
        dotted = ".".join(path.resolve().relative_to(ROOT).with_suffix("").parts)
        mod = importlib.import_module(dotted)
    except ValueError:
        spec = importlib.util.spec_from_file_location(f"_check_subject_{stem}", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    parts = selector.split(".")
    if not hasattr(mod, parts[0]):
        raise ValueError(f"{path.name} has no {parts[0]!r}")
    subject = getattr(mod, parts[0])
    twin_cls = subject if isinstance(subject, type) else subject(cfg)
    oracle = importlib.import_module(f"oracle.{oracle_name}")
    return f"{path.name}:{selector}", twin_cls, oracle.make(cfg), parts[1:], name


def run(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        expect = expectations(getattr(args, "comparison", None))
        dims = {}
        for item in args.dim or []:
            k, _, v = item.partition("=")
            dims[k] = int(v)
        label, twin_cls, impl_for, rest, cfg_name = resolve(args.source, args.config)
        from oracle import evaluator
        twin = twin_cls()
        sem = twin.module
        generator = torch.Generator().manual_seed(SEED)
        # walk children, then the function (default: the Module's entry)
        node_sem, node_twin, path_res = sem, twin, []
        while rest and any(c.name == rest[0] for c in node_sem.modules):
            seg = rest.pop(0)
            node_sem = next(c for c in node_sem.modules if c.name == seg)
            node_twin = getattr(node_twin, seg)
            path_res.append(seg)
        fn_name = rest.pop(0) if rest else node_sem.entry
        if rest:
            raise ValueError(f"{'.'.join(rest)!r}: nothing of that name under {node_sem.name}")
        if fn_name is None or not any(f.name == fn_name for f in node_sem.functions):
            raise ValueError(f"{node_sem.name} has no function {fn_name!r}; it has {[f.name for f in node_sem.functions]}")
        function = node_sem.lookup(fn_name)
        activations = tuple(draw(extents(p.type, dims), p.type.dtype, generator) for p in function.activations)
        resource = RandomWeights(sem, generator, dims)
        reference_root = evaluator.load(sem, resource, impl_for)
        twin.load(OnDevice(resource, torch.device(args.device)))
        ref_node = reference_root
        for seg in path_res:
            ref_node = getattr(ref_node, seg)
        dev = torch.device(args.device)

        def to_cpu(x):
            return tuple(to_cpu(i) for i in x) if isinstance(x, tuple) else x.cpu()

        candidate = lambda *a: to_cpu(getattr(node_twin, fn_name)(*[t.to(dev) for t in a]))
        reference = getattr(ref_node, fn_name)
        report = measure.check(candidate, reference, activations, expect=expect)
    except (ValueError, KeyError, TypeError) as exc:
        print(f"check: {exc}", file=sys.stderr)
        return 2

    outputs = [{"path": o.path, "dtype": o.dtype, "shape": list(o.shape), "ref_norm": o.ref_norm, "passed": o.passed,
                "fns": [{"fn": r.predicate.name, **{b: getattr(r.predicate, b) for b in r.predicate.bounds},
                         **{k: float(v) for k, v in r.values.items()}, "passed": r.passed,
                         **({"note": r.note} if r.note else {})} for r in o.results]} for o in report.outputs]
    record = {"source": label, "config": cfg_name, "function": fn_name, "reference": "evaluator (CPU restatement)",
              "inputs": {"activations": {"source": f"random, seed {SEED}", "dtypes": [str(a.dtype) for a in activations]},
                         "weights": {"source": f"random, seed {SEED}, drawn on first use"}},
              "dims": dims, "outputs": outputs, "passed": report.passed}
    if args.json:
        print(json.dumps(record))
        return 0 if report.passed else 1
    lines = [label, f"  reference: {record['reference']}",
             f"  inputs:    activations {record['inputs']['activations']['source']} "
             f"{record['inputs']['activations']['dtypes']}; weights {record['inputs']['weights']['source']}", ""]
    for o in outputs:
        shape = ",".join(str(e) for e in o["shape"])
        norm = "" if o["ref_norm"] is None else f"   ref_norm {o['ref_norm']:.6g}"
        lines.append(f"  {o['path']}   {o['dtype']}[{shape}]{norm}")
        for m in o["fns"]:
            cls = measure.PREDICATES[m["fn"]]
            bounds = " ".join(f"{b}={m[b]:g}" for b in cls.bounds)
            values = " ".join(f"{k} {v:g}" for k, v in m.items() if k not in ("fn", "passed", "note", *cls.bounds))
            stated = f"{m['fn']}({bounds})" if bounds else m["fn"]
            lines.append(f"    {stated:<34} {values:<26} {'PASS' if m['passed'] else 'FAIL'}")
            if "note" in m:
                lines.append(f"      {m['note']}")
        lines.append("")
    lines.append("PASS" if report.passed else "FAIL")
    print("\n".join(lines))
    return 0 if report.passed else 1


if __name__ == "__main__":
    sys.exit(run())
