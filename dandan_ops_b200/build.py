"""Compile the CUDA sources of this package into lib/libb2w4a16.so for sm_100a.

The library is a plain C-ABI shared object (no torch headers), so one nvcc call
builds it in a few seconds, with or without a GPU in the machine.
"""
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libb2w4a16.so"
STAMP = LIB_DIR / "libb2w4a16.stamp"
SHIM_SRC = CSRC / "torch_shim" / "shim.cpp"
SHIM_PATH = LIB_DIR / "dandan_ops_b200_C.so"
SHIM_STAMP = LIB_DIR / "dandan_ops_b200_C.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")))


def source_digest():
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for path in _sources():
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


def nvcc_path():
    for cand in (os.environ.get("B2_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise RuntimeError("nvcc not found; set B2_NVCC")


def is_current():
    return LIB_PATH.is_file() and STAMP.is_file() and STAMP.read_text().strip() == source_digest()


def build(force=False, verbose=False):
    """Build the library if its sources changed (or `force`).  Returns the .so path."""
    if not force and is_current():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    units = sorted(str(p) for p in CSRC.glob("*.cu"))
    cmd = [nvcc_path(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []),
           "-I", str(INCLUDE), "-o", str(LIB_PATH), *units]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    STAMP.write_text(source_digest() + "\n")
    return LIB_PATH


def shim_digest():
    import torch

    h = hashlib.sha256(torch.__version__.encode())
    h.update(SHIM_SRC.read_bytes())
    h.update((INCLUDE / "b2_w4a16.h").read_bytes())
    return h.hexdigest()


def build_shim(force=False):
    """Compile the torch operator library (csrc/torch_shim/shim.cpp): `torch.ops.load_library`-loadable,
    linked against lib/libb2w4a16.so (found next to it through its run path).  One g++ call; needs the
    headers of the installed torch and the CUDA runtime headers, no GPU."""
    import torch
    from torch.utils import cpp_extension

    build()
    if not force and SHIM_PATH.is_file() and SHIM_STAMP.is_file() and SHIM_STAMP.read_text().strip() == shim_digest():
        return SHIM_PATH
    cuda_home = Path(nvcc_path()).resolve().parent.parent
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-w", str(SHIM_SRC), "-o", str(SHIM_PATH),
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-I", str(cuda_home / "include")]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    cmd += ["-L", str(torch_lib), "-L", str(LIB_DIR), "-lb2w4a16", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
            "-L", str(cuda_home / "lib64"), "-lcudart", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("g++ failed on the torch shim:\n" + proc.stdout + proc.stderr)
    SHIM_STAMP.write_text(shim_digest() + "\n")
    return SHIM_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_shim(force="--force" in sys.argv))
