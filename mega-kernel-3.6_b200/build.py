"""In-tree build of the native code: libmk36.so (CUDA kernels + C ABI, no torch) and the PyTorch
extension mega_kernel_qwen36/_C*.so (thin shim over the C ABI).

    python build.py            # build what is out of date
    python build.py --force    # rebuild everything

Counterpart of the reference's setup.py (CUDAExtension, TORCH_CUDA_ARCH_LIST 9.0;12.0,
setup.py:14-39); here the only target is sm_100a and the kernels live in a torch-free library.
nvcc cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
CSRC = HERE / "csrc"
PKG = HERE / "mega_kernel_qwen36"
OBJ = HERE / "build"
INCLUDE = ROOT / "include"

CUDA_SOURCES = [
    "mk36_api.cu",
    "mk36_comm.cu",
    "moe_decode.cu",
    "moe_decode_ring.cu",
    "moe_decode_stream.cu",
    "moe_decode_batch.cu",
    "dense_ffn_decode.cu",
    "dense_ffn_mma.cu",
    "dense_ffn_stream.cu",
    "attention_decode.cu",
    "attention_decode_mma.cu",
    "attention_decode_stream.cu",
    "attention_decode_static.cu",
    "linear_attention_decode.cu",
    "linear_decode.cu",
]
LIB_NAME = "libmk36.so"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, quiet=False):
    if not quiet:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(str(c) for c in cmd)}")
    return proc.stdout + proc.stderr


def lib_path() -> Path:
    return PKG / LIB_NAME


def ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return PKG / f"_C{suffix}"


def build_library(force: bool = False, verbose_ptxas: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    nvcc = _nvcc()
    jobs = []
    objects = []
    for src in CUDA_SOURCES:
        s = CSRC / src
        o = OBJ / (s.stem + ".o")
        objects.append(o)
        if force or not _newer(o, [s] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", s, "-o", o]
            if verbose_ptxas:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for out in pool.map(_run, jobs):
                if verbose_ptxas:
                    print(out)
    lib = lib_path()
    if force or jobs or not _newer(lib, objects):
        _run([nvcc, "-shared", "-o", lib, *objects, "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a"])
    return lib


def build_extension(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    ext = ext_path()
    src = CSRC / "torch_shim.cpp"
    lib = lib_path()
    if not force and _newer(ext, [src, INCLUDE / "mk36.h", lib]):
        return ext
    includes = cpp_extension.include_paths("cuda")
    cuda_inc = Path(_nvcc()).resolve().parent.parent / "include"
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        os.environ.get("CXX", "g++"),
        "-O2",
        "-std=c++17",
        "-fPIC",
        "-shared",
        "-DTORCH_EXTENSION_NAME=_C",
        "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
        "-I",
        INCLUDE,
        "-I",
        sysconfig.get_paths()["include"],
        "-I",
        cuda_inc,
    ]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [
        src,
        "-o",
        ext,
        f"-L{PKG}",
        "-l:" + LIB_NAME,
        # the C++ runtime as a shared library, named before the driver's own -lstdc++: a toolchain that only
        # ships libstdc++.a would otherwise put a second, uninitialised copy of the iostream machinery into the
        # extension, and formatting a number into an error message would crash instead of raising
        "-l:libstdc++.so.6",
        f"-L{torch_lib}",
        "-lc10",
        "-lc10_cuda",
        "-ltorch_cpu",
        "-ltorch_cuda",
        "-ltorch",
        "-ltorch_python",
        "-Wl,-rpath,$ORIGIN",
        f"-Wl,-rpath,{torch_lib}",
    ]
    _run(cmd)
    return ext


def build_all(force: bool = False, verbose_ptxas: bool = False):
    lib = build_library(force=force, verbose_ptxas=verbose_ptxas)
    ext = build_extension(force=force)
    return lib, ext


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-verbose", action="store_true", help="print registers / spills per kernel")
    ap.add_argument("--library-only", action="store_true")
    ns = ap.parse_args()
    if ns.library_only:
        print(build_library(force=ns.force, verbose_ptxas=ns.ptxas_verbose))
    else:
        for p in build_all(force=ns.force, verbose_ptxas=ns.ptxas_verbose):
            print(p)
