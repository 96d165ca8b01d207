"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``libxpool_kernels.so`` — every ``csrc/kernels/*.cu`` compiled for ``sm_100a`` only
  (``-gencode arch=compute_100a,code=sm_100a``); nvcc cross-compiles without a GPU.
* ``libxpool_runtime.so`` — the host-only C++ runtime in ``csrc/runtime/*.cpp`` (protocol
  state machines, scheduler, shared-memory channels); it has no CUDA dependency, so CPU-only
  tests load it.

The reference builds one static core plus a pybind module with CMake for five architectures
(src/cext/CMakeLists.txt, cmake/XpoolCudaArchitectures.cmake:3-6); here the ABI is plain C and is
loaded with ctypes, which keeps a rebuild to seconds per file.

Run ``python -m crosspool_b200.native.build`` to (re)build; ``--force`` rebuilds everything.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
OBJ = HERE / "build"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-Wall",
    f"-I{CSRC / 'include'}",
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-Wall", "-Wextra", "-Werror", f"-I{CSRC / 'include'}", "-pthread"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return exe


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted((CSRC / "include").rglob("*")):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _needs(obj: Path, src: Path, stamp: str) -> bool:
    tag = obj.with_suffix(obj.suffix + ".stamp")
    want = hashlib.sha256(src.read_bytes()).hexdigest()[:16] + stamp
    if obj.exists() and tag.exists() and tag.read_text() == want:
        return False
    return True


def _mark(obj: Path, src: Path, stamp: str) -> None:
    tag = obj.with_suffix(obj.suffix + ".stamp")
    tag.write_text(hashlib.sha256(src.read_bytes()).hexdigest()[:16] + stamp)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    out = HERE / "libxpool_kernels.so"
    stamp = _headers_digest()
    sources = sorted((CSRC / "kernels").glob("*.cu"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _needs(obj, src, stamp):
            cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append((cmd, obj, src))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            for fut, (cmd, obj, src) in [(ex.submit(_run, j[0]), j) for j in jobs]:
                fut.result()
                _mark(obj, src, stamp)
    if jobs or not out.exists():
        _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


def build_runtime(force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    out = HERE / "libxpool_runtime.so"
    stamp = _headers_digest()
    sources = sorted((CSRC / "runtime").glob("*.cpp"))
    cxx = shutil.which("g++") or "g++"
    objs = []
    rebuilt = False
    for src in sources:
        obj = OBJ / ("rt_" + src.stem + ".o")
        objs.append(obj)
        if force or _needs(obj, src, stamp):
            _run([cxx, *CXX_FLAGS, "-c", str(src), "-o", str(obj)])
            _mark(obj, src, stamp)
            rebuilt = True
    if rebuilt or not out.exists():
        _run([cxx, "-shared", "-o", str(out), *map(str, objs), "-pthread", "-lrt"])
    return out


def build_torch_ops(force: bool = False) -> Path:
    """``libxpool_torch_ops.so``: the ``xpool::ffn_shim`` operator (``csrc/bindings/torch_ops.cpp``) compiled against
    this interpreter's PyTorch headers and linked to ``libxpool_kernels.so`` beside it."""
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(exist_ok=True)
    out = HERE / "libxpool_torch_ops.so"
    src = CSRC / "bindings" / "torch_ops.cpp"
    import torch

    stamp = _headers_digest() + torch.__version__
    obj = OBJ / "torch_ops.o"
    if force or _needs(obj, src, stamp) or not out.exists():
        cxx = shutil.which("g++") or "g++"
        inc = [f"-I{p}" for p in ce.include_paths("cuda")]
        cuda_inc = Path(_nvcc()).resolve().parent.parent / "include"
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-Wall", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-I{CSRC / 'include'}", f"-I{cuda_inc}",
              *inc, "-c", str(src), "-o", str(obj)])
        libdir = Path(torch.__file__).resolve().parent / "lib"
        _run([cxx, "-shared", "-o", str(out), str(obj), f"-L{HERE}", "-lxpool_kernels", f"-L{libdir}", "-ltorch", "-ltorch_cpu",
              "-lc10", "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{libdir}"])
        _mark(obj, src, stamp)
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    out = {"runtime": build_runtime(force), "kernels": build_kernels(force, verbose)}
    out["torch_ops"] = build_torch_ops(force)
    return out


if __name__ == "__main__":
    paths = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in paths.items():
        print(f"{k}: {v}")
