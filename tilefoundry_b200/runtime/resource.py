"""Checkpoint access: ``load(name)``, ``load_group(name)``, ``subtree(segment)``.

Same protocol and alias rules as reference ``src/tilefoundry/runtime/resource.py``:
an alias map is consulted first under the qualified name (``prefix + name``),
then under the bare name, else the name stands for itself (``:63-85``).  An alias
value is a string (relative rename), a tuple of strings (a group, only readable
through ``load_group``), ``Absolute(key)`` (ignores the prefix) or
``Preprocessed(name, read)`` (rename plus a one-tensor transform such as a
transpose).  ``DictResource`` is the in-memory double; ``SafetensorsResource``
reads a checkpoint directory (sharded with an index file, or one
``model.safetensors``).
"""
from __future__ import annotations

import dataclasses
import json
from pathlib import Path
from typing import Callable, Mapping, Protocol, Union

import torch

__all__ = ["Absolute", "DictResource", "Preprocessed", "RuntimeResource", "SafetensorsResource"]


@dataclasses.dataclass(frozen=True)
class Absolute:
    name: str


@dataclasses.dataclass(frozen=True)
class Preprocessed:
    name: "str | Absolute"
    read: Callable[[torch.Tensor], torch.Tensor]

    def __post_init__(self) -> None:
        if isinstance(self.name, tuple):
            raise TypeError(
                f"Preprocessed: {self.name!r} is a group of raw tensors; combining several "
                "tensors is a weight converter's job, not a read-side transform"
            )


AliasValue = Union[str, tuple, Absolute, Preprocessed]


class RuntimeResource(Protocol):
    def load(self, name: str) -> torch.Tensor: ...
    def load_group(self, name: str) -> "tuple[torch.Tensor, ...] | None": ...
    def subtree(self, seg: str) -> "RuntimeResource": ...


class _Aliased:
    """Name resolution shared by both resources."""

    _kind = "RuntimeResource"

    def __init__(self, prefix: str, alias: Mapping[str, AliasValue] | None) -> None:
        self._prefix = prefix
        self._alias = alias or {}

    def _hit(self, name: str):
        for key in (self._prefix + name, name):
            if key in self._alias:
                return self._alias[key]
        return None

    def _keys(self, name: str):
        """-> (raw key | tuple of raw keys, transform | None)"""
        hit, read = self._hit(name), None
        if isinstance(hit, Preprocessed):
            hit, read = hit.name, hit.read
        if hit is None:
            return self._prefix + name, read
        if isinstance(hit, Absolute):
            return hit.name, read
        if isinstance(hit, tuple):
            return tuple(self._prefix + one for one in hit), read
        return self._prefix + hit, read

    def _segment(self, seg: str) -> str:
        hit = self._hit(seg)
        if hit is None:
            return seg
        if not isinstance(hit, str):
            raise TypeError(
                f"{self._kind}.subtree: segment {seg!r} resolves to {hit!r}; a subtree "
                "segment must resolve to one relative name"
            )
        return hit

    def _fetch(self, raw_key: str) -> torch.Tensor:
        raise NotImplementedError

    def load(self, name: str) -> torch.Tensor:
        keys, read = self._keys(name)
        if isinstance(keys, tuple):
            raise TypeError(
                f"{self._kind}.load: {name!r} resolves to the group {keys!r} "
                f"({len(keys)} raw names); use load_group"
            )
        try:
            value = self._fetch(keys)
        except KeyError:
            raise KeyError(f"{self._kind}: no tensor named {name!r} (raw key {keys!r})") from None
        return value if read is None else read(value)

    def load_group(self, name: str):
        keys, _ = self._keys(name)
        if not isinstance(keys, tuple):
            return None
        out = []
        for raw in keys:
            try:
                out.append(self._fetch(raw))
            except KeyError:
                raise KeyError(f"{self._kind}: no tensor named {name!r} (raw key {raw!r})") from None
        return tuple(out)


class DictResource(_Aliased):
    """Flat dot-prefixed dict shared by every scoped view (``{"layer0.w_q": t}``)."""

    _kind = "DictResource"

    def __init__(self, data: Mapping[str, torch.Tensor], prefix: str = "", alias=None) -> None:
        super().__init__(prefix, alias)
        self._data = data

    def _fetch(self, raw_key: str) -> torch.Tensor:
        return self._data[raw_key]

    def subtree(self, seg: str) -> "DictResource":
        return DictResource(self._data, f"{self._prefix}{self._segment(seg)}.", self._alias)


def _pinned_device(device: str) -> str:
    # safetensors reads a bare "cuda" as index 0 while torch means the current
    # device; make the word mean what torch means (reference resource.py:45-60).
    if device == "cuda" and torch.cuda.is_available():
        return f"cuda:{torch.cuda.current_device()}"
    return device


class SafetensorsResource(_Aliased):
    _kind = "SafetensorsResource"

    def __init__(self, ckpt_dir: str, prefix: str = "", device: str = "cuda", alias=None) -> None:
        super().__init__(prefix, alias)
        self._dir = Path(ckpt_dir)
        self._device = device
        self._shared = {"map": None, "handles": {}}

    def _weight_map(self) -> dict:
        if self._shared["map"] is None:
            index = self._dir / "model.safetensors.index.json"
            if index.is_file():
                self._shared["map"] = dict(json.loads(index.read_text(encoding="utf-8"))["weight_map"])
            else:
                from safetensors import safe_open

                single = self._dir / "model.safetensors"
                if not single.is_file():
                    raise FileNotFoundError(
                        f"SafetensorsResource: {self._dir} holds neither "
                        "model.safetensors.index.json nor model.safetensors"
                    )
                with safe_open(str(single), framework="pt", device="cpu") as fh:
                    self._shared["map"] = dict.fromkeys(fh.keys(), single.name)
        return self._shared["map"]

    def _fetch(self, raw_key: str) -> torch.Tensor:
        from safetensors import safe_open

        shard = self._weight_map()[raw_key]
        handle = self._shared["handles"].get(shard)
        if handle is None:
            handle = safe_open(str(self._dir / shard), framework="pt",
                               device=_pinned_device(self._device))
            self._shared["handles"][shard] = handle
        return handle.get_tensor(raw_key)

    def subtree(self, seg: str) -> "SafetensorsResource":
        child = SafetensorsResource(str(self._dir), f"{self._prefix}{self._segment(seg)}.",
                                    self._device, self._alias)
        child._shared = self._shared
        return child
