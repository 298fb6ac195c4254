"""Declarative record of an authored TileFoundry ``Module``.

TileFoundry authors a model's decode step as ``@module`` classes whose ``@func``
methods are parsed into HIR (reference ``src/tilefoundry/ir/core/module.py:197``).
A runtime twin only ever reads a small part of that object: the function names,
each function's ordered parameters with their ``is_const`` flag and declared
shape / dtype, the child modules, the ``entry`` name and the plain-Python
orchestration ``methods``.  This file re-provides exactly that part as plain
dataclasses, so a twin can be validated one-to-one against a declaration
without the reference's parser.  The attribute names are the reference's, so the
same twin decorates a real ``tilefoundry.ir.core.module.Module`` unchanged.

Nothing here evaluates a function body: a declaration has none.
"""
from __future__ import annotations

import types
from dataclasses import dataclass, field, replace
from typing import Callable, Mapping, Sequence

import torch

DTYPES: Mapping[str, torch.dtype] = {
    "bf16": torch.bfloat16,
    "f16": torch.float16,
    "f32": torch.float32,
    "f64": torch.float64,
    "i32": torch.int32,
    "i64": torch.int64,
    "i8": torch.int8,
    "u8": torch.uint8,
    "bool": torch.bool,
}
_NAMES = {v: k for k, v in DTYPES.items()}


def to_torch_dtype(name: str) -> torch.dtype:
    """Torch dtype for a DSL dtype name (reference ``evaluator/value.py:21-44``)."""
    try:
        return DTYPES[name]
    except KeyError:
        raise ValueError(f"unknown dtype name {name!r}; known: {sorted(DTYPES)}") from None


def dtype_name(dtype: torch.dtype) -> str:
    try:
        return _NAMES[dtype]
    except KeyError:
        raise ValueError(f"torch dtype {dtype} has no DSL name") from None


@dataclass(frozen=True)
class DimVar:
    """A ranged dimension, e.g. ``ctx_len`` in ``[lo, hi)`` (reference ``ir/types/dim.py``)."""

    name: str
    lo: int
    hi: int

    def admits(self, extent: int) -> bool:
        return self.lo <= extent < self.hi


@dataclass(frozen=True)
class TensorType:
    """Declared shape (ints or ``DimVar``) and dtype name of one parameter."""

    shape: tuple
    dtype: str

    def matches_shape(self, shape: Sequence[int]) -> bool:
        if len(shape) != len(self.shape):
            return False
        for want, got in zip(self.shape, shape):
            if isinstance(want, DimVar):
                if not want.admits(int(got)):
                    return False
            elif int(want) != int(got):
                return False
        return True


@dataclass(frozen=True)
class Param:
    name: str
    type: TensorType
    is_const: bool = False


@dataclass(frozen=True)
class Function:
    """Signature of one ``@func``: name plus parameters in declared order."""

    name: str
    params: tuple[Param, ...]

    @property
    def activations(self) -> tuple[Param, ...]:
        return tuple(p for p in self.params if not p.is_const)

    @property
    def constants(self) -> tuple[Param, ...]:
        return tuple(p for p in self.params if p.is_const)


def T(shape, dtype: str = "bf16") -> tuple[TensorType, bool]:
    """An activation parameter (the DSL's ``Tensor[shape, dtype]``)."""
    return TensorType(tuple(shape), dtype), False


def W(shape, dtype: str = "bf16") -> tuple[TensorType, bool]:
    """A weight parameter (the DSL's ``ConstTensor[shape, dtype]``)."""
    return TensorType(tuple(shape), dtype), True


def func(name: str, **params: tuple[TensorType, bool]) -> Function:
    """``func("mlp", hidden=T(...), w=W(...))`` -> ``Function`` (keyword order = declared order)."""
    return Function(name, tuple(Param(n, ty, const) for n, (ty, const) in params.items()))


def validate_declared(owner: str, what: str, value: torch.Tensor, decl: TensorType) -> None:
    """Strict shape + dtype check of a bound tensor (reference ``module.py:144-159``)."""
    if not decl.matches_shape(tuple(value.shape)):
        raise ValueError(
            f"Module {owner!r}: {what} has shape {tuple(value.shape)}, declared {decl.shape}"
        )
    want = to_torch_dtype(decl.dtype)
    if value.dtype != want:
        raise ValueError(
            f"Module {owner!r}: {what} has dtype {value.dtype}, declared {decl.dtype}; "
            "convert the weight when preparing the checkpoint, not when reading it"
        )


@dataclass(frozen=True)
class Module:
    """The fields of an authored ``Module`` a runtime twin reads."""

    name: str
    functions: tuple[Function, ...]
    entry: str | None = None
    modules: tuple["Module", ...] = ()
    methods: Mapping[str, Callable] = field(default_factory=dict)
    metadata: Mapping[str, object] = field(default_factory=dict)

    def __post_init__(self) -> None:
        fn_names = [f.name for f in self.functions]
        child_names = [m.name for m in self.modules]
        for label, names in (("function", fn_names), ("child module", child_names)):
            dup = sorted({n for n in names if names.count(n) > 1})
            if dup:
                raise ValueError(f"Module {self.name!r}: duplicate {label} name(s) {dup}")
        clash = sorted(
            (set(fn_names) & set(child_names))
            | (set(self.methods) & (set(fn_names) | set(child_names)))
        )
        if clash:
            raise ValueError(
                f"Module {self.name!r}: name(s) {clash} are used twice among functions, "
                "child modules and methods; the three sets must be disjoint"
            )
        if self.entry is not None and self.entry not in fn_names:
            raise ValueError(f"Module {self.name!r}: entry {self.entry!r} not in functions")

    def renamed(self, name: str) -> "Module":
        return replace(self, name=name)

    @property
    def weights(self) -> Mapping[str, TensorType]:
        """Every ``is_const`` parameter once, in (function, parameter) order."""
        out: dict[str, TensorType] = {}
        for fn in self.functions:
            for p in fn.params:
                if not p.is_const:
                    continue
                seen = out.get(p.name)
                if seen is not None and seen != p.type:
                    raise ValueError(
                        f"Module {self.name!r}: weight {p.name!r} declared with two types "
                        f"({seen} and {p.type})"
                    )
                out[p.name] = p.type
        return out

    def lookup(self, name: str) -> Function:
        hits = [f for f in self.functions if f.name == name]
        if len(hits) != 1:
            raise ValueError(
                f"Module {self.name!r}: {name!r} must resolve to exactly one function, "
                f"found {len(hits)}"
            )
        return hits[0]

    def all_weight_names(self, prefix: str = "") -> list[str]:
        """Dotted names of every declared weight in this subtree, in draw order."""
        names = [f"{prefix}{n}" for n in self.weights]
        for child in self.modules:
            names.extend(child.all_weight_names(f"{prefix}{child.name}."))
        return names

    def all_weights(self, prefix: str = "") -> list[tuple[str, TensorType]]:
        out = [(f"{prefix}{n}", ty) for n, ty in self.weights.items()]
        for child in self.modules:
            out.extend(child.all_weights(f"{prefix}{child.name}."))
        return out

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        for child in self.__dict__.get("modules", ()):
            if child.name == name:
                return child
        method = self.__dict__.get("methods", {}).get(name)
        if method is not None:
            return types.MethodType(method, self)
        raise AttributeError(f"Module {self.__dict__.get('name')!r} has no child or method {name!r}")


def refuse_bare_call(module: Module, kind: str) -> None:
    """A bare call needs a ``forward`` method or an entry (reference ``module.py:162-177``)."""
    if module.entry is not None:
        return
    named = sorted({f.name for f in module.functions} | set(module.methods))
    raise TypeError(
        f"{kind} {module.name!r} has neither a forward method nor an entry; "
        "call a function by name" + (f": {', '.join(named)}" if named else "")
    )


__all__ = [
    "DTYPES", "DimVar", "Function", "Module", "Param", "T", "TensorType", "W",
    "dtype_name", "func", "refuse_bare_call", "to_torch_dtype", "validate_declared",
]
