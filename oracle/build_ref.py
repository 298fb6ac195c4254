"""TEST INFRASTRUCTURE.  Builds the reference's own CUDA C kernels for the granite example, unmodified, from
where they lie in the reference tree, for sm_100a:

    python -m oracle.build_ref [--force]

Source: ``examples/granite_4_0_h_small-cuda/kernels/granite.cu`` of the reference checkout (path in
``TILEFOUNDRY_REFERENCE``, default: a ``reference`` directory beside this repository); recipe: the flags of the reference's own
``kernels/__init__.py:24-41`` with the architecture switched the way its ``GRANITE_CUDA_ARCH`` switch does
(``:14``).  Output: ``oracle/_ref/granite/granite_ref_kernels.so`` only -- no reference source is copied.
The library is used by ``tests/test_granite_reference_kernels_gpu.py`` to hold the evaluator restatement
(``oracle/granite_4_0_h_small.py``) to the reference's kernels on a B200; nothing under ``tilefoundry_b200/``
loads it."""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "granite"
NAME = "granite_ref_kernels"


def reference_source() -> Path:
    root = Path(os.environ.get("TILEFOUNDRY_REFERENCE") or HERE.parents[1] / "reference")
    return root / "examples" / "granite_4_0_h_small-cuda" / "kernels" / "granite.cu"


def built() -> Path | None:
    so = OUT / f"{NAME}.so"
    return so if so.exists() else None


def build(force: bool = False, verbose: bool = False) -> Path | None:
    """The built library, or None when the reference tree is not present (then whatever was built earlier stays)."""
    src = reference_source()
    if not src.exists():
        return built()
    if built() and not force and built().stat().st_mtime >= src.stat().st_mtime:
        return built()
    from torch.utils.cpp_extension import load

    OUT.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(name=NAME, sources=[str(src)], build_directory=str(OUT), is_python_module=False,
         extra_cuda_cflags=["-O3", "--use_fast_math", "-lineinfo", "-gencode=arch=compute_100a,code=sm_100a",
                            "--expt-relaxed-constexpr"],
         extra_cflags=["-O3"], verbose=verbose)
    return built()


def load_built():
    """The built extension as a Python module (its functions are the reference's ``m.def`` list), or None."""
    so = built()
    if so is None:
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
