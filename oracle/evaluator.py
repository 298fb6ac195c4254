"""TEST INFRASTRUCTURE.  ``load(module, resource, impl)`` -> the evaluator side of ``check``.

Plays the part of the reference's ``Module.load -> LoadedModule``
(``src/tilefoundry/ir/core/module.py:444-466,699-794``): constants are read by
declared name with strict shape/dtype validation, children load from
``resource.subtree(child.name)``, a function attribute is a callable over
activations only, and ``forward`` / the other orchestration methods are the
authored Module's own, bound to the loaded object.  The function bodies come
from an ``impl`` namespace of torch restatements keyed by function name.
"""
from __future__ import annotations

import types

from tilefoundry_b200.semantic import refuse_bare_call, validate_declared


class Loaded:
    def __init__(self, module, constants, children, impl):
        self.module = module
        self.name = module.name
        self.constants = constants
        self.modules = tuple(children)
        self._impl = impl
        for child in self.modules:
            setattr(self, child.name, child)
        for fn in module.functions:
            setattr(self, fn.name, self._runner(fn))

    def _runner(self, fn):
        body = self._impl[fn.name]
        n_acts = len(fn.activations)

        def run(*acts):
            if len(acts) != n_acts:
                raise TypeError(f"{self.name}.{fn.name}: takes {n_acts} activations, got {len(acts)}")
            it = iter(acts)
            full = [self.constants[p.name] if p.is_const else next(it) for p in fn.params]
            return body(*full)

        return run

    def forward(self, *acts):
        method = self.module.methods.get("forward")
        if method is not None:
            return method(self, *acts)
        refuse_bare_call(self.module, "LoadedModule")
        return getattr(self, self.module.entry)(*acts)

    def __call__(self, *acts):
        return self.forward(*acts)

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        method = self.__dict__["module"].methods.get(name)
        if method is None:
            raise AttributeError(f"LoadedModule {self.__dict__['name']!r} has no {name!r}")
        return types.MethodType(method, self)


def load(module, resource, impl_for):
    """*impl_for(module)* -> ``{function name: torch callable}`` for that (sub)module."""
    consts = {}
    for name, decl in module.weights.items():
        try:
            value = resource.load(name)
        except KeyError as exc:
            raise KeyError(f"Module {module.name!r}: missing declared weight {name!r}") from exc
        validate_declared(module.name, f"weight {name!r}", value, decl)
        consts[name] = value
    kids = [load(c, resource.subtree(c.name), impl_for) for c in module.modules]
    return Loaded(module, consts, kids, impl_for(module))


def load_as(module, resource, impl_for, dtype):
    """Like ``load`` but with every floating weight cast to *dtype* and no dtype validation: used to
    run the same function bodies at f32/f64 as an arbiter between two bf16 implementations (the
    reference keeps such an arbiter too, ``examples/qwen3_1_7b-tilelang/fast/arbitrate.py``)."""
    consts = {}
    for name in module.weights:
        value = resource.load(name)
        consts[name] = value.to(dtype) if value.is_floating_point() else value
    kids = [load_as(c, resource.subtree(c.name), impl_for, dtype) for c in module.modules]
    return Loaded(module, consts, kids, impl_for(module))
