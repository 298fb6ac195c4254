"""``RuntimeModule`` and ``CompiledModule``: the objects a caller steps.

Mirrors reference ``src/tilefoundry/runtime/module.py:16-102``: a runtime module
has a ``name``, an optional ``entry``, ordered child ``modules``; ``load`` walks
the children with ``resource.subtree(child.name)``; calling the module runs
``forward``.
"""
from __future__ import annotations

from typing import Callable

import torch

from ..semantic import to_torch_dtype
from .function import EntryABI

__all__ = ["CompiledModule", "RuntimeModule"]


class RuntimeModule:
    def __init__(self, name: str, entry: str | None = None, modules=()) -> None:
        self.name = name
        self.entry = entry
        self.modules = tuple(modules)

    @property
    def module(self):
        """The authored Module this stands for; ``None`` for a hand-written subclass."""
        return None

    def forward(self, *args):
        raise NotImplementedError(f"RuntimeModule {self.name!r}: forward() is not implemented")

    def __call__(self, *args):
        return self.forward(*args)

    def load(self, resource) -> None:
        for child in self.modules:
            child.load(resource.subtree(child.name))


class CompiledModule(RuntimeModule):
    """One out-parameter entry wrapped as a module (reference ``module.py:59-102``).

    ``m(*inputs)`` allocates the trailing ``output_count`` tensors from the ABI and
    returns them; ``m(*inputs, *outputs)`` writes into the tensors given.
    """

    def __init__(self, type: EntryABI, fn: Callable) -> None:
        super().__init__(name=type.name, entry=type.name)
        self.type = type
        self.fn = fn

    def forward(self, *args):
        abi = self.type
        if len(args) == len(abi.params):
            outs = tuple(args[abi.input_count:])
            self.fn(*args)
        elif len(args) == abi.input_count:
            device = next((a.device for a in args if isinstance(a, torch.Tensor)), None)
            if device is None:
                raise TypeError(f"{abi.name}: no tensor among the inputs to take a device from")
            outs = tuple(
                torch.empty(p.type.shape, dtype=to_torch_dtype(p.type.dtype), device=device)
                for p in abi.output_params
            )
            self.fn(*args, *outs)
        else:
            raise TypeError(
                f"{abi.name}: takes {abi.input_count} inputs, or {len(abi.params)} inputs "
                f"and outputs; got {len(args)}"
            )
        return outs[0] if len(outs) == 1 else outs
