"""``@runtime_module`` / ``@runtime_func``: authoring a twin of an authored Module.

Contract (reference ``src/tilefoundry/runtime/decorator.py:24-232``):

* the set of ``@runtime_func`` method names (or ``RuntimeFunction`` attributes) of
  the decorated class equals the Module's function-name set, and the set of
  attributes that are ``RuntimeModule`` subclasses equals its child-name set;
  either mismatch is a ``TypeError`` at decoration time that lists what is
  missing and what is extra;
* ``module`` is reserved on the twin;
* a kernel body is written ``def fn(self, *every declared param)``; callers pass
  activations only and ``is_const`` parameters are filled by name from the
  weights ``load`` bound (``KeyError`` naming the weight when unbound);
* ``load(resource)`` reads each declared weight by name, checks shape and dtype
  strictly, then recurses with ``resource.subtree(child.name)``;
* ``forward`` and any other orchestration method come from the Module's
  ``methods`` unless the twin class defines its own.

``sem`` may be a ``tilefoundry_b200.semantic.Module`` or a real TileFoundry
``Module``: only ``name / functions / modules / methods / entry / weights`` and
``param.name / param.is_const / param.type`` are read.
"""
from __future__ import annotations

import inspect
import types
from typing import Callable

from ..semantic import refuse_bare_call, validate_declared
from .function import RuntimeFunction
from .module import RuntimeModule

__all__ = ["runtime_func", "runtime_module"]

_MARK = "_tilefoundry_runtime_func"
_RESERVED = frozenset({"module"})


def runtime_func(fn: Callable) -> Callable:
    if not inspect.isfunction(fn):
        raise TypeError(f"runtime_func: expected a plain function, got {type(fn).__name__}")
    setattr(fn, _MARK, True)
    return fn


def _is_kernel(value) -> bool:
    if isinstance(value, RuntimeFunction):
        return True
    return inspect.isfunction(value) and getattr(value, _MARK, False)


def _is_child_class(value) -> bool:
    return isinstance(value, type) and issubclass(value, RuntimeModule)


def _same_names(cls_name: str, what: str, found: set, against: str, expected: set) -> None:
    if found != expected:
        raise TypeError(
            f"@runtime_module {cls_name!r}: {what} {sorted(found)} must equal {against} "
            f"{sorted(expected)}; missing {sorted(expected - found)}, extra {sorted(found - expected)}"
        )


def _bind_kernel(twin: "TwinBase", ir_fn, body) -> Callable:
    as_object = isinstance(body, RuntimeFunction)
    n_acts = sum(1 for p in ir_fn.params if not p.is_const)

    def call(*acts):
        if len(acts) != n_acts:
            raise TypeError(
                f"{twin.name}.{ir_fn.name}: takes {n_acts} activation(s) "
                f"({', '.join(p.name for p in ir_fn.params if not p.is_const)}), got {len(acts)}"
            )
        it = iter(acts)
        full = []
        for p in ir_fn.params:
            if p.is_const:
                if p.name not in twin._bound:
                    raise KeyError(
                        f"RuntimeModule {twin.name!r}: weight {p.name!r} of {ir_fn.name!r} "
                        "is not bound; call load(resource) first"
                    )
                full.append(twin._bound[p.name])
            else:
                full.append(next(it))
        return body(*full) if as_object else body(twin, *full)

    call.__name__ = ir_fn.name
    return call


class TwinBase(RuntimeModule):
    """Behaviour shared by every generated twin class."""

    _ir = None

    @property
    def module(self):
        return self._ir

    def load(self, resource) -> None:
        for name, decl in self._ir.weights.items():
            try:
                value = resource.load(name)
            except KeyError as exc:
                raise KeyError(f"RuntimeModule {self.name!r}: missing weight {name!r}") from exc
            validate_declared(self.name, f"weight {name!r}", value, decl)
            self._bound[name] = value
        for child in self.modules:
            child.load(resource.subtree(child.name))

    def forward(self, *acts):
        method = self._ir.methods.get("forward")
        if method is not None:
            return method(self, *acts)
        refuse_bare_call(self._ir, "RuntimeModule")
        return getattr(self, self._ir.entry)(*acts)

    def __getattr__(self, name: str):
        # Only reached when normal lookup fails: orchestration methods of the
        # authored Module are served bound to the twin.
        if name.startswith("_"):
            raise AttributeError(name)
        ir = self.__dict__.get("_ir")
        method = None if ir is None else ir.methods.get(name)
        if method is None:
            raise AttributeError(
                f"RuntimeModule {self.__dict__.get('name')!r} has no runtime function, "
                f"child module or method {name!r}"
            )
        return types.MethodType(method, self)


def runtime_module(sem) -> Callable[[type], type]:
    fn_names = {f.name for f in sem.functions}
    child_names = {m.name for m in sem.modules}

    def decorate(cls: type) -> type:
        taken = sorted((fn_names | child_names | set(sem.methods)) & _RESERVED)
        if taken:
            raise TypeError(
                f"@runtime_module {cls.__name__!r}: Module {sem.name!r} declares {taken}, "
                "a name every twin reserves; rename it in the authored Module"
            )
        body = {k: v for k, v in vars(cls).items() if not (k.startswith("__") and k.endswith("__"))}
        written = sorted(set(body) & _RESERVED)
        if written:
            raise TypeError(
                f"@runtime_module {cls.__name__!r} defines {written}, which the generated "
                "twin answers itself (it names the authored Module)"
            )
        _same_names(cls.__name__, "@runtime_func names",
                    {k for k, v in body.items() if _is_kernel(v)},
                    "semantic function names", fn_names)
        _same_names(cls.__name__, "child module names",
                    {k for k, v in body.items() if _is_child_class(v)},
                    "semantic child module names", child_names)

        def __init__(self, ir=None) -> None:
            ir = sem if ir is None else ir
            self._ir = ir
            self._bound = {}
            children = []
            for child_ir in ir.modules:
                child_cls = body.get(child_ir.name)
                if child_cls is None:
                    raise TypeError(
                        f"{cls.__name__}: ir {ir.name!r} has child {child_ir.name!r} "
                        "with no runtime child class of that name"
                    )
                child = child_cls(ir=child_ir)
                setattr(self, child_ir.name, child)
                children.append(child)
            RuntimeModule.__init__(self, name=ir.name, entry=ir.entry, modules=tuple(children))
            for fn in ir.functions:
                impl = body.get(fn.name)
                if impl is None:
                    raise TypeError(
                        f"{cls.__name__}: ir {ir.name!r} has function {fn.name!r} "
                        "with no @runtime_func of that name"
                    )
                setattr(self, fn.name, _bind_kernel(self, fn, impl))
            post = body.get("_post_init")
            if post is not None:
                post(self)

        ns = dict(body)
        ns["__init__"] = __init__
        ns["__module__"] = cls.__module__
        if cls.__dict__.get("__doc__") is not None:
            ns["__doc__"] = cls.__dict__["__doc__"]
        return type(cls.__name__, (TwinBase,), ns)

    return decorate
