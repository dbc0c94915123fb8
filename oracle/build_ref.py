"""Builds the reference project's cuBLASLt submission as a loadable extension.  TEST INFRASTRUCTURE ONLY.

The reference has no CPU code for this path; the one implementation in it that is a plain
library call with no hand-written device waits is ``sub_cub.py`` (``cuda_nvfp4_gemm_cublaslt``,
sub_cub.py:48-143, bound by ``custom_kernel`` at sub_cub.py:165-169).  This recipe compiles that
file's own C++/CUDA source -- taken from the file where it lies in the reference checkout, with
the very flags it passes to ``load_inline`` (sub_cub.py:146-162) -- into

    oracle/_ref/nvfp4_tcgen05_gemm_tma_all.so

Nothing of the reference is copied into this repository: the sources are handed to the compiler
from a temporary directory and only the built module is kept (``oracle/_ref/`` is git-ignored).
On a machine with a B200 the tests load that module to pin the CPU oracle against outputs the
reference itself produces (``tests/test_reference_pin_gpu.py``,
``tests/golden/make_ref_golden.py``).  The product never loads it.

    python oracle/build_ref.py            # needs the reference checkout (NVFP4_REFERENCE_DIR)
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import sys
import tempfile
import types
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
MODULE_NAME = "nvfp4_tcgen05_gemm_tma_all"      # the extension name sub_cub.py:147 gives it
MODULE_PATH = OUT_DIR / f"{MODULE_NAME}.so"


def reference_dir() -> Path:
    return Path(os.environ.get("NVFP4_REFERENCE_DIR", "/root/reference"))


def available() -> bool:
    return MODULE_PATH.exists()


def _capture_load_inline_arguments(ref: Path) -> dict:
    """Runs sub_cub.py's module body with ``load_inline`` replaced by a recorder, so that the
    sources and flags are exactly the ones the file would have compiled itself."""
    import torch.utils.cpp_extension as cpp_ext

    captured: dict = {}

    def recorder(**kwargs):
        captured.update(kwargs)
        return types.SimpleNamespace()

    real = cpp_ext.load_inline
    sys.path.insert(0, str(ref))          # sub_cub.py imports the reference's own task.py
    saved_task = sys.modules.pop("task", None)
    cpp_ext.load_inline = recorder
    try:
        code = compile((ref / "sub_cub.py").read_text(), str(ref / "sub_cub.py"), "exec")
        exec(code, {"__name__": "reference_sub_cub"})
    finally:
        cpp_ext.load_inline = real
        sys.path.remove(str(ref))
        sys.modules.pop("task", None)
        if saved_task is not None:
            sys.modules["task"] = saved_task
    if "cuda_sources" not in captured:
        raise RuntimeError("sub_cub.py did not call load_inline as expected")
    return captured


def build(force: bool = False) -> Path:
    ref = reference_dir()
    if not (ref / "sub_cub.py").exists():
        raise FileNotFoundError(f"no reference checkout at {ref} (set NVFP4_REFERENCE_DIR)")
    if MODULE_PATH.exists() and not force and MODULE_PATH.stat().st_mtime >= (ref / "sub_cub.py").stat().st_mtime:
        return MODULE_PATH
    import torch.utils.cpp_extension as cpp_ext

    kwargs = _capture_load_inline_arguments(ref)
    OUT_DIR.mkdir(exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="nvfp4_ref_build_") as tmp:
        kwargs = dict(kwargs, build_directory=tmp, verbose=False)
        # the link step names libcuda (sub_cub.py:160); without a driver on this machine the
        # toolkit's stub directory supplies it, and importing the finished module fails for the
        # same reason -- which is fine, it only has to load where there is a GPU
        stubs = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64" / "stubs"
        kwargs["extra_ldflags"] = list(kwargs.get("extra_ldflags", [])) + ([f"-L{stubs}"] if stubs.exists() else [])
        try:
            cpp_ext.load_inline(**kwargs)
        except ImportError:
            pass
        built = Path(tmp) / f"{MODULE_NAME}.so"
        if not built.exists():
            raise RuntimeError("the reference extension did not build")
        shutil.copyfile(built, MODULE_PATH)
    return MODULE_PATH


def load():
    """Imports the built module (needs a CUDA driver) and returns the reference's operator entry:
    ``custom_kernel(data)`` with the body of sub_cub.py:165-169."""
    import ctypes
    import glob

    import torch  # noqa: F401  (the extension links against torch)

    if not MODULE_PATH.exists():
        raise FileNotFoundError(f"{MODULE_PATH} is missing: run oracle/build_ref.py where the reference checkout is")
    # The module leaves its cuBLASLt symbols to be resolved from the process (the way a
    # load_inline build does): make torch's own cuBLASLt visible to it.
    site = Path(torch.__file__).resolve().parent.parent
    for lib in sorted(glob.glob(str(site / "nvidia" / "cublas" / "lib" / "libcublasLt.so.*"))):
        ctypes.CDLL(lib, mode=ctypes.RTLD_GLOBAL)
    spec = importlib.util.spec_from_file_location(MODULE_NAME, MODULE_PATH)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)

    def custom_kernel(data):
        a, b, sfa, sfb, sfa_perm, sfb_perm, c = data
        return module.cuda_nvfp4_gemm_cublaslt(a, b, sfa, sfb, sfa_perm, sfb_perm, c)

    return custom_kernel


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
