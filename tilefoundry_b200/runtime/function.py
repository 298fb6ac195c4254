"""Entry ABI records and the ``RuntimeFunction`` base.

Same surface as reference ``src/tilefoundry/runtime/function.py:14-91``.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..semantic import TensorType

__all__ = ["EntryABI", "ParamABI", "RuntimeFunction", "entry_abi_of", "param_abi_of"]


@dataclass(frozen=True)
class ParamABI:
    name: str
    type: TensorType


@dataclass(frozen=True)
class EntryABI:
    """All parameters in declared order; the last ``output_count`` are outputs."""

    name: str
    params: tuple[ParamABI, ...]
    output_count: int = 0

    @property
    def input_count(self) -> int:
        return len(self.params) - self.output_count

    @property
    def input_params(self) -> tuple[ParamABI, ...]:
        return self.params[: self.input_count]

    @property
    def output_params(self) -> tuple[ParamABI, ...]:
        return self.params[self.input_count:]


class RuntimeFunction:
    """A kernel object that may stand in for a ``@runtime_func`` method."""

    def __init__(self, type: EntryABI) -> None:
        self.type = type

    def __call__(self, *args):
        raise NotImplementedError(f"RuntimeFunction {self.type.name!r}: __call__ is not implemented")


def param_abi_of(param) -> ParamABI:
    if not isinstance(param.type, TensorType):
        raise TypeError(f"param {param.name!r} must carry a TensorType")
    return ParamABI(param.name, param.type)


def entry_abi_of(fn) -> EntryABI:
    """Value-returning ABI of a declared function: every param an input."""
    return EntryABI(fn.name, tuple(param_abi_of(p) for p in fn.params), 0)
