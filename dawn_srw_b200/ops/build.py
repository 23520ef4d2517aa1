"""In-tree build of the CUDA extension ``dawn_srw_b200/ops/_dsb_cuda*.so``.

Every ``.cu`` under ``csrc/`` is compiled by ``nvcc`` for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``), the pybind11 bindings by ``g++``
against the torch headers, and everything is linked into one shared object that
sits beside this file (so it travels with the source tree; nothing is
installed into site-packages).  Objects are rebuilt only when their source (or
a header) is newer.  ``nvcc`` cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import List

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "_build"
EXT_NAME = "_dsb_cuda"
SO_PATH = HERE / f"{EXT_NAME}.so"
PLAIN_SO_PATH = HERE / "libdsb_kernels.so"     # kernels + C ABI only (no torch / python)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newer(src: Path, dst: Path, extra: List[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *extra])


def _run(cmd, log=None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r


def build(verbose: bool = False, force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension as ce
    BUILD.mkdir(exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
    objs = []
    for cu in sorted(CSRC.glob("*.cu")):
        obj = BUILD / (cu.stem + ".o")
        if force or _newer(cu, obj, headers):
            if verbose:
                print(f"[build] nvcc {cu.name}", flush=True)
            _run([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(cu), "-o", str(obj)],
                 log=BUILD / (cu.stem + ".ptxas.txt"))
        objs.append(obj)
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", str(CSRC)]
    cxx_objs = []
    for cpp in sorted(CSRC.glob("*.cpp")):
        obj = BUILD / (cpp.stem + ".cpp.o")
        if force or _newer(cpp, obj, headers):
            if verbose:
                print(f"[build] g++ {cpp.name}", flush=True)
            abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
            _run(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                  f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                  *inc, "-c", str(cpp), "-o", str(obj)])
        cxx_objs.append(obj)
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_lib = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64"
    stamp = max(o.stat().st_mtime for o in objs + cxx_objs)
    if force or not SO_PATH.exists() or SO_PATH.stat().st_mtime < stamp:
        # the allocation-free entry point (and its 64 MiB device array) belongs to the plain
        # C library only
        ext_objs = [o for o in objs if o.stem != "srw_forward_static"]
        # link beside the target and rename: a reader never sees a half-written library
        tmp = SO_PATH.with_suffix(".so.tmp")
        _run(["g++", "-shared", "-o", str(tmp), *map(str, ext_objs + cxx_objs),
              f"-L{torch_lib}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
              "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
              f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{cuda_lib}"])
        os.replace(tmp, SO_PATH)
    if force or not PLAIN_SO_PATH.exists() or PLAIN_SO_PATH.stat().st_mtime < stamp:
        tmp = PLAIN_SO_PATH.with_suffix(".so.tmp")
        _run(["g++", "-shared", "-o", str(tmp), *map(str, objs),
              f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{cuda_lib}"])
        os.replace(tmp, PLAIN_SO_PATH)
    return SO_PATH


def load():
    """Import the built extension (building it first if it is missing)."""
    import importlib.util
    import torch  # noqa: F401  (must be imported before the extension)
    if not SO_PATH.exists():
        build()
    spec = importlib.util.spec_from_file_location(EXT_NAME, str(SO_PATH))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
