"""Seeded synthetic checkpoints.

Real checkpoints are not assumed to be present; a model is exercised with bf16
weights drawn ~N(0, std) from one ``torch.Generator`` in the Module's declared
weight order (root functions first, then each child in order), so any two sides
that bind by name see identical tensors.  Norm gains can be drawn as ``1 + N(0,
std)`` to keep activations at a realistic scale.
"""
from __future__ import annotations

import torch

from ..semantic import Module, to_torch_dtype


def random_weights(module: Module, seed: int = 0, std: float = 0.02, *,
                   gain_prefix: str = "gamma", unit_gains: bool = True,
                   overrides=None, device="cpu") -> dict[str, torch.Tensor]:
    """Flat ``{dotted name: tensor}`` for ``DictResource``.

    ``overrides(name, type, generator) -> tensor | None`` lets a model give
    specific parameters (decay rates, biases) their own distribution.
    """
    gen = torch.Generator(device="cpu").manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, ty in module.all_weights():
        leaf = name.rsplit(".", 1)[-1]
        value = overrides(name, ty, gen) if overrides is not None else None
        if value is None:
            value = torch.randn(tuple(ty.shape), generator=gen, dtype=torch.float32) * std
            if unit_gains and leaf.startswith(gain_prefix):
                value = value + 1.0
        out[name] = value.to(to_torch_dtype(ty.dtype)).to(device)
    return out


def random_weights_on(module: Module, device, seed: int = 0, std: float = 0.02, *, gain_prefix: str = "gamma",
                      overrides=None, skip=()) -> dict[str, torch.Tensor]:
    """Same distributions as ``random_weights`` but drawn directly on *device* (a 32B-parameter model
    takes minutes to draw on the host).  The values differ from the host generator's: use it where only
    the shapes and distributions matter (benchmarks), not where two sides must bind the same tensors."""
    gen = torch.Generator(device=device).manual_seed(seed)
    cpu_gen = torch.Generator(device="cpu").manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for name, ty in module.all_weights():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in skip:
            continue
        value = overrides(name, ty, cpu_gen) if overrides is not None else None
        if value is not None:
            out[name] = value.to(to_torch_dtype(ty.dtype)).to(device)
            continue
        value = torch.randn(tuple(ty.shape), generator=gen, device=device, dtype=torch.float32) * std
        if leaf.startswith(gain_prefix):
            value += 1.0
        out[name] = value.to(to_torch_dtype(ty.dtype))
        del value
    return out
