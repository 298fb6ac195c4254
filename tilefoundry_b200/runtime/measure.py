"""``check``: run a candidate and a reference on the same inputs and compare.

Follows reference ``src/tilefoundry/runtime/measure.py``: results may be a tensor
or nested tuples of tensors, addressed ``output``, ``output[0]``, ``output[1][2]``
(``:264-277``); both sides must flatten to the same paths, shapes and dtypes
(``:350-362``); every output must state at least one predicate, there is no
default bound (``:295-322``); an integer output admits only ``equal``
(``:280-292``).  Predicates: ``allclose rel_l2 cosine equal ulp max_abs max_rel
nan_inf`` (``:62-216``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, ClassVar, Mapping, Sequence

import torch

from ..semantic import dtype_name

__all__ = [
    "PREDICATES", "AllClose", "Cosine", "Equal", "MaxAbs", "MaxRel", "NanInf",
    "OutputCheck", "Predicate", "PredicateResult", "RelL2", "Report", "Ulp", "check",
]

_TINY = 1e-12


@dataclass(frozen=True)
class PredicateResult:
    predicate: "Predicate"
    values: Mapping[str, float]
    passed: bool
    note: str | None = None


@dataclass(frozen=True)
class Predicate:
    name: ClassVar[str] = ""
    bounds: ClassVar[tuple[str, ...]] = ()
    needs_reference: ClassVar[bool] = True
    discrete: ClassVar[bool] = True      # meaningful on integer outputs?
    guidance: ClassVar[str] = ""

    def measure(self, candidate: torch.Tensor, reference: torch.Tensor | None) -> PredicateResult:
        raise NotImplementedError

    def _out(self, values, passed, note=None) -> PredicateResult:
        return PredicateResult(self, dict(values), bool(passed), note)


@dataclass(frozen=True)
class AllClose(Predicate):
    atol: float
    rtol: float
    name = "allclose"
    bounds = ("atol", "rtol")
    discrete = False
    guidance = "per element: |got - want| <= atol + rtol*|want|"

    def measure(self, candidate, reference):
        got, want = candidate.float(), reference.float()
        over = ((got - want).abs() - (self.atol + self.rtol * want.abs())).max().item()
        shown = over if over != over else max(over, 0.0)   # keep NaN visible
        return self._out({"max_violation": shown}, over <= 0.0)


@dataclass(frozen=True)
class RelL2(Predicate):
    max: float
    name = "rel_l2"
    bounds = ("max",)
    discrete = False
    guidance = "||got - want|| / ||want||"

    def measure(self, candidate, reference):
        got, want = candidate.float(), reference.float()
        dist, ref = (got - want).norm().item(), want.norm().item()
        if ref <= _TINY:
            return self._out({"absolute_l2": dist}, dist <= self.max,
                             "reference norm is zero; distance reported as absolute")
        return self._out({"rel_l2": dist / ref}, dist / ref <= self.max)


@dataclass(frozen=True)
class Cosine(Predicate):
    min: float
    name = "cosine"
    bounds = ("min",)
    discrete = False
    guidance = "direction of the flattened outputs; exposes a systematic bias"

    def measure(self, candidate, reference):
        a, b = candidate.float().flatten(), reference.float().flatten()
        na, nb = a.norm().item(), b.norm().item()
        if na <= _TINY and nb <= _TINY:
            return self._out({"cosine": 1.0}, 1.0 >= self.min, "both sides are all zero")
        if na <= _TINY or nb <= _TINY:
            return self._out({"cosine": 0.0}, False, "one side is all zero, the other is not")
        value = (torch.dot(a, b) / (a.norm() * b.norm())).item()
        return self._out({"cosine": value}, value >= self.min)


@dataclass(frozen=True)
class Equal(Predicate):
    name = "equal"
    guidance = "bitwise; the only predicate for discrete outputs"

    def measure(self, candidate, reference):
        bad = int((candidate != reference).sum().item())
        return self._out({"mismatched": float(bad), "elements": float(candidate.numel())}, bad == 0)


_INT_VIEW = {torch.bfloat16: torch.int16, torch.float16: torch.int16,
             torch.float32: torch.int32, torch.float64: torch.int64}


def _monotone_bits(t: torch.Tensor) -> torch.Tensor:
    """Float bits mapped to integers that sort like the floats do."""
    view = _INT_VIEW.get(t.dtype)
    if view is None:
        raise ValueError(f"check: ulp is defined on a float output, not on {t.dtype}")
    bits = t.view(view).to(torch.int64)
    top = 1 << (t.element_size() * 8 - 1)
    return torch.where(bits >= 0, bits, -(bits + top))


@dataclass(frozen=True)
class Ulp(Predicate):
    max: float
    name = "ulp"
    bounds = ("max",)
    discrete = False
    guidance = "count of representable values between got and want"

    def measure(self, candidate, reference):
        d = (_monotone_bits(candidate) - _monotone_bits(reference)).abs().max().item()
        return self._out({"max_ulp": float(d)}, d <= self.max)


@dataclass(frozen=True)
class MaxAbs(Predicate):
    max: float
    name = "max_abs"
    bounds = ("max",)
    discrete = False
    guidance = "largest absolute difference"

    def measure(self, candidate, reference):
        v = (candidate.float() - reference.float()).abs().max().item()
        return self._out({"max_abs": v}, v <= self.max)


@dataclass(frozen=True)
class MaxRel(Predicate):
    max: float
    name = "max_rel"
    bounds = ("max",)
    discrete = False
    guidance = "largest relative difference; a nonzero miss against an exact zero is infinite"

    def measure(self, candidate, reference):
        got, want = candidate.float(), reference.float()
        diff, mag = (got - want).abs(), want.abs()
        rel = torch.where(mag > 0, diff / mag.clamp_min(_TINY),
                          torch.where(diff == 0, torch.zeros_like(diff),
                                      torch.full_like(diff, float("inf"))))
        v = rel.max().item()
        return self._out({"max_rel": v}, v <= self.max)


@dataclass(frozen=True)
class NanInf(Predicate):
    name = "nan_inf"
    needs_reference = False
    discrete = False
    guidance = "no NaN, no Inf; needs no reference"

    def measure(self, candidate, reference=None):
        nan = int(torch.isnan(candidate).sum().item())
        inf = int(torch.isinf(candidate).sum().item())
        return self._out({"nan": float(nan), "inf": float(inf)}, nan == 0 and inf == 0)


PREDICATES: Mapping[str, type] = {
    p.name: p for p in (AllClose, RelL2, Cosine, Equal, Ulp, MaxAbs, MaxRel, NanInf)
}


@dataclass(frozen=True)
class OutputCheck:
    path: str
    shape: tuple[int, ...]
    dtype: str
    ref_norm: float | None
    results: tuple[PredicateResult, ...]

    @property
    def passed(self) -> bool:
        return all(r.passed for r in self.results)


@dataclass(frozen=True)
class Report:
    outputs: tuple[OutputCheck, ...]

    @property
    def passed(self) -> bool:
        return all(o.passed for o in self.outputs)

    def render(self) -> str:
        lines = []
        for o in self.outputs:
            for r in o.results:
                vals = " ".join(f"{k}={v:.4g}" for k, v in r.values.items())
                lines.append(f"{'ok  ' if r.passed else 'FAIL'} {o.path:<16} {o.dtype:<5} "
                             f"{r.predicate.name:<8} {vals}")
        return "\n".join(lines)


def _leaves(x, path="output"):
    if isinstance(x, torch.Tensor):
        return [(path, x)]
    if isinstance(x, tuple):
        out = []
        for i, item in enumerate(x):
            out += _leaves(item, f"{path}[{i}]")
        return out
    raise TypeError(f"check: {path} must be a torch.Tensor or a tuple of them, got {type(x).__name__}")


def check(candidate: Callable, reference: Callable | None, inputs: tuple, *,
          expect: Mapping[str, Sequence[Predicate]]) -> Report:
    got = _leaves(candidate(*inputs))
    if not got:
        raise ValueError("check: the candidate produced no tensor, so nothing was compared")
    paths = [p for p, _ in got]

    unknown = sorted(set(expect) - set(paths))
    if unknown:
        raise ValueError(f"check: {unknown} name no output; this run produced {paths}")
    for p in paths:
        stated = tuple(expect.get(p) or ())
        if not stated:
            raise ValueError(
                f"check: no comparison requested for output {p!r}. Every output needs at "
                "least one predicate and there is no default bound."
            )
        if reference is None:
            two_sided = sorted({q.name for q in stated if q.needs_reference})
            if two_sided:
                free = sorted(n for n, q in PREDICATES.items() if not q.needs_reference)
                raise ValueError(
                    f"check: {p!r} asks for {two_sided} but there is no reference; "
                    f"without one only {free} can be measured"
                )

    want: dict[str, torch.Tensor] = {}
    if reference is not None:
        ref = _leaves(reference(*inputs))
        if [p for p, _ in ref] != paths:
            raise ValueError(
                f"check: candidate/reference output structures differ: {paths} vs {[p for p, _ in ref]}"
            )
        for (p, a), (_, b) in zip(got, ref):
            if a.shape != b.shape or a.dtype != b.dtype:
                raise ValueError(
                    f"check: {p} shape/dtype mismatch: candidate {tuple(a.shape)}/{a.dtype} "
                    f"vs reference {tuple(b.shape)}/{b.dtype}"
                )
            want[p] = b.to(a.device)

    outs = []
    for p, a in got:
        preds = tuple(expect[p])
        if not a.dtype.is_floating_point:
            for q in preds:
                if not q.discrete:
                    raise ValueError(
                        f"check: {p} is {dtype_name(a.dtype)}; {q.name} is not meaningful on a "
                        "discrete output, where one wrong value is a wrong result. Use equal."
                    )
        b = want.get(p)
        outs.append(OutputCheck(p, tuple(a.shape), dtype_name(a.dtype),
                                None if b is None else b.float().norm().item(),
                                tuple(q.measure(a, b) for q in preds)))
    return Report(tuple(outs))
