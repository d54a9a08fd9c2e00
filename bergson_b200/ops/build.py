"""In-tree build of the sm_100a extension.

``python -m bergson_b200.ops.build`` compiles ``csrc/*.cu`` with
``-gencode arch=compute_100a,code=sm_100a`` and links them with the pybind bindings
into ``bergson_b200/ops/_build/bergson_b200_C.so``.  nvcc cross-compiles, so no GPU is
needed to build.  A hash of the sources and flags is stored beside the library; the
build is skipped when it matches.
"""

from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "_build"
NAME = "bergson_b200_C"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=" + NAME, "-D_GLIBCXX_USE_CXX11_ABI=1"]


def _sources() -> tuple[list[Path], list[Path]]:
    return sorted(CSRC.glob("*.cu")), sorted(CSRC.glob("*.cpp"))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.iterdir()):
        if p.suffix in {".cu", ".cuh", ".h", ".cpp"}:
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    import torch

    h.update(torch.__version__.encode())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    print(" ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True)


def build(force: bool = False, verbose_ptxas: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    OUT.mkdir(exist_ok=True)
    so = OUT / f"{NAME}.so"
    stamp = OUT / "build.sha256"
    digest = _digest()
    if not force and so.exists() and stamp.exists() and stamp.read_text() == digest:
        return so

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = Path(cuda_home) / "bin" / "nvcc"
    cus, cpps = _sources()
    objs = []
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    for src in cus:
        obj = OUT / (src.stem + ".o")
        _run([nvcc, *NVCC_FLAGS, *extra, "-I", CSRC, "-c", src, "-o", obj])
        objs.append(obj)
    includes = []
    for inc in cpp_extension.include_paths("cuda"):
        includes += ["-I", inc]
    includes += ["-I", sysconfig.get_paths()["include"], "-I", CSRC]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cxx_flags = [f for f in CXX_FLAGS if not f.startswith("-D_GLIBCXX")] + [f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
    for src in cpps:
        obj = OUT / (src.stem + ".o")
        _run(["g++", *cxx_flags, *includes, "-c", src, "-o", obj])
        objs.append(obj)
    lib_dirs = []
    for d in cpp_extension.library_paths("cuda"):
        lib_dirs += ["-L", d, f"-Wl,-rpath,{d}"]
    _run([
        "g++", "-shared", *objs, "-o", so, *lib_dirs,
        "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart",
    ])
    stamp.write_text(digest)
    return so


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose_ptxas="--ptxas-v" in sys.argv)
    print(f"built {path}")
