"""Build the reference's own ``mixed_cache_ops`` extension, unmodified, for the
checker (TEST INFRASTRUCTURE ONLY).

The reference ships one native source, ``additional_designs/mixed_cache_kernels/
mixed_cache.cu`` (a torch pybind extension, built by its ``mixed_cache_setup.py``
with no arch flags).  This recipe compiles that file where it lies, for sm_100a,
and writes the module into ``oracle/_ref/``; no reference source is copied.  The
GPU test ``tests/test_gpu_reference_ext.py`` loads it and compares its three ops
with the CPU oracle and with this package's kernels.

Run: ``python -m oracle.build_ref``  (needs the reference checkout; the GPU box
only uses the prebuilt module).
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
# where the reference checkout lies: $APTSERVE_REFERENCE, else a directory named "reference"
# beside this repository
REFERENCE_ROOT = Path(os.environ.get("APTSERVE_REFERENCE") or HERE.parent.parent / "reference")
SOURCE = REFERENCE_ROOT / "additional_designs" / "mixed_cache_kernels" / "mixed_cache.cu"
MODULE = "mixed_cache_ops"


def module_path() -> Path:
    return OUT_DIR / f"{MODULE}{sysconfig.get_config_var('EXT_SUFFIX')}"


def build() -> Path:
    import torch
    from torch.utils import cpp_extension as ce
    if not SOURCE.exists():
        raise FileNotFoundError(f"reference source not found: {SOURCE}")
    OUT_DIR.mkdir(exist_ok=True)
    out = module_path()
    if out.exists() and out.stat().st_mtime >= SOURCE.stat().st_mtime:
        return out
    includes = [f"-I{p}" for p in ce.include_paths("cuda")]
    includes.append(f"-I{sysconfig.get_paths()['include']}")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
           "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
           f"-DTORCH_EXTENSION_NAME={MODULE}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *includes, str(SOURCE), "-o", str(out),
           f"-L{libdir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
           "-ltorch_python", f"-Xlinker=-rpath,{libdir}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on the reference source:\n{r.stdout[-4000:]}")
    return out


def build_if_possible():
    if module_path().exists() and not SOURCE.exists():
        return module_path()
    return build()


def load():
    """Import the prebuilt module (after ``import torch``)."""
    import importlib.util
    import torch  # noqa: F401  (its shared libraries must be loaded first)
    path = module_path()
    if not path.exists():
        raise FileNotFoundError(f"{path} not built; run python -m oracle.build_ref")
    spec = importlib.util.spec_from_file_location(MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build())
