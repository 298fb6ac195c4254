"""Host-side boundary: twin decoration rules, resources, `check`, and the C-ABI export list (CPU only).

Mirrors the reference's boundary doubles (``tests/fixtures/logical/*_twin.py``,
``tests/runtime/``): a tiny authored Module, a matching torch twin, and deliberate negatives.
"""
import re
from pathlib import Path

import pytest
import torch

from tilefoundry_b200 import semantic as sem
from tilefoundry_b200.runtime import (AllClose, Absolute, Cosine, DictResource, Equal, NanInf, Preprocessed,
                                      RuntimeModule, Ulp, check, runtime_func, runtime_module)
from tilefoundry_b200.semantic import T, W, func

ROOT = Path(__file__).resolve().parents[1]


def _square():
    child = sem.Module("scale", (func("apply", x=T((4,), "f32"), w=W((4,), "f32")),), entry="apply")
    return sem.Module("Square", (func("square", x=T((4,), "f32")),), modules=(child,),
                      methods={"forward": lambda self, x: self.scale(self.square(x))})


def _twin_cls(module):
    @runtime_module(module.modules[0])
    class Scale:
        @runtime_func
        def apply(self, x, w):
            return x * w

    @runtime_module(module)
    class Twin:
        scale = Scale

        @runtime_func
        def square(self, x):
            return x * x
    return Twin


def test_twin_runs_orchestration_and_binds_weights_by_name():
    mod = _square()
    twin = _twin_cls(mod)()
    assert twin.module is mod and twin.scale.module is mod.modules[0]
    with pytest.raises(KeyError, match="not bound"):
        twin.scale.apply(torch.ones(4))
    twin.load(DictResource({"scale.w": torch.full((4,), 3.0)}))
    out = twin(torch.arange(4.0))
    assert torch.equal(out, torch.arange(4.0) ** 2 * 3)
    with pytest.raises(TypeError, match="takes 1 activation"):
        twin.scale.apply(torch.ones(4), torch.ones(4))


def test_load_validates_shape_and_dtype_strictly():
    twin = _twin_cls(_square())()
    with pytest.raises(ValueError, match="shape"):
        twin.load(DictResource({"scale.w": torch.ones(5)}))
    with pytest.raises(ValueError, match="dtype"):
        twin.load(DictResource({"scale.w": torch.ones(4, dtype=torch.bfloat16)}))
    with pytest.raises(KeyError, match="missing weight"):
        twin.load(DictResource({}))


def test_decoration_requires_one_to_one_names():
    mod = _square()
    with pytest.raises(TypeError, match="missing \\['square'\\]"):
        @runtime_module(mod)
        class NoKernel:
            scale = type("S", (RuntimeModule,), {})
    with pytest.raises(TypeError, match="extra \\['cube'\\]"):
        @runtime_module(mod.modules[0])
        class Extra:
            @runtime_func
            def apply(self, x, w):
                return x

            @runtime_func
            def cube(self, x):
                return x
    with pytest.raises(TypeError, match="child module names"):
        @runtime_module(mod)
        class NoChild:
            @runtime_func
            def square(self, x):
                return x
    with pytest.raises(TypeError, match="answers itself"):
        @runtime_module(mod.modules[0])
        class Reserved:
            module = 1

            @runtime_func
            def apply(self, x, w):
                return x


def test_resource_alias_rules():
    data = {"model.layers.0.q.weight": torch.arange(6.0).reshape(2, 3), "tok": torch.ones(2)}
    alias = {"layer0": "model.layers.0", "w_q": Preprocessed("q.weight", lambda t: t.t().contiguous()),
             "w_embed": Absolute("tok"), "pair": ("q.weight", "q.weight")}
    res = DictResource(data, alias=alias)
    sub = res.subtree("layer0")
    assert sub.load("w_q").shape == (3, 2)
    assert torch.equal(sub.load("w_embed"), data["tok"])          # absolute ignores the prefix
    assert len(sub.load_group("pair")) == 2 and sub.load_group("w_q") is None
    with pytest.raises(TypeError, match="load_group"):
        sub.load("pair")
    with pytest.raises(KeyError, match="no tensor named"):
        sub.load("absent")
    with pytest.raises(TypeError, match="one relative name"):
        res.subtree("w_embed")


def test_check_contract():
    ref = lambda x: (x * 2, (x.to(torch.int64),))
    good = lambda x: (x * 2 + 1e-4, (x.to(torch.int64),))
    x = torch.arange(4.0)
    expect = {"output[0]": [AllClose(atol=1e-3, rtol=0), Cosine(min=0.999), NanInf()], "output[1][0]": [Equal()]}
    assert check(good, ref, (x,), expect=expect).passed
    drifted = lambda x: (x * 2 + 1, (x.to(torch.int64),))
    assert not check(drifted, ref, (x,), expect=expect).passed
    with pytest.raises(ValueError, match="no comparison requested"):
        check(good, ref, (x,), expect={"output[0]": [NanInf()]})
    with pytest.raises(ValueError, match="Use equal"):
        check(good, ref, (x,), expect={"output[0]": [NanInf()], "output[1][0]": [AllClose(atol=1, rtol=0)]})
    with pytest.raises(ValueError, match="name no output"):
        check(good, ref, (x,), expect={**expect, "output[7]": [Equal()]})
    with pytest.raises(ValueError, match="no reference"):
        check(good, None, (x,), expect=expect)
    with pytest.raises(ValueError, match="structures differ"):
        check(lambda x: x, ref, (x,), expect={"output": [NanInf()]})
    a = torch.tensor([1.0], dtype=torch.bfloat16)
    b = torch.nextafter(a.float(), torch.tensor([2.0])).to(torch.bfloat16)
    assert Ulp(max=1).measure(a, a).passed


def test_library_exports_every_declared_symbol():
    """The C-ABI library loads and exports each function include/tfb200.h declares (no GPU needed)."""
    from tilefoundry_b200 import build, lib
    build.build()
    header = (ROOT / "include" / "tfb200.h").read_text()
    declared = set(re.findall(r"TFB_API\s+[\w\s\*]+?\b(tfb_\w+)\s*\(", header))
    assert declared and declared == set(lib.SYMBOLS), (declared ^ set(lib.SYMBOLS))
    handle = lib.load()
    for name in declared:
        assert getattr(handle, name) is not None
    assert handle.tfb_version() >= 100
    assert handle.tfb_status_string(1).decode().startswith("invalid argument")
    assert handle.tfb_attn_splits(130) == 3 and handle.tfb_attn_splits(0) == 0


def test_kernels_refuse_cpu_tensors():
    from tilefoundry_b200 import lib
    with pytest.raises(ValueError, match="no CPU path"):
        lib.ptr(torch.zeros(4))


def test_paged_kv_table_and_views():
    from tilefoundry_b200.engine import paged_kv
    table = paged_kv.block_table(2, 130)
    assert table.tolist() == [[0, 1, 2], [3, 4, 5]] and table.dtype == torch.int32
    pool = torch.zeros(6, 64, 2, 8)
    cache = torch.randn(1, 70, 2, 8)
    paged_kv.fill_from_logical(pool, table[1], cache)
    assert torch.equal(paged_kv.logical_view(pool, table[1], 70), cache)
    assert float(pool[:3].abs().sum()) == 0                       # sequence 0's pages untouched
    paged_kv.fill_from_logical(pool, table[0], cache[:, :0])      # empty cache: nothing to do
