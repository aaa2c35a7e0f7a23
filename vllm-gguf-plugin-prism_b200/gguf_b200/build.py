"""In-tree build of the native libraries (explicit nvcc / g++ commands, sm_100a only).

Outputs, next to the Python package they serve (git-ignored, shipped with the tree):
  vllm_gguf_plugin/libgguf_b200.so   the C-ABI kernel library (include/gguf_b200.h)
  vllm_gguf_plugin/_C_gguf.abi3.so   torch stable-ABI library `_C_gguf` calling the C-ABI

quantize_q8_1.cu and gemv1.cu (the decode GEMV that quantizes its activations itself) are
compiled with --use_fast_math: the two fp32 divisions of the q8_1 quantization must be the same
approximate instructions the reference emits (the reference builds everything with that flag,
setup.py:34-42).  The other files contain no expression the flag would change in a way that
matters, and stay with IEEE defaults.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent.parent           # .../vllm-gguf-plugin-prism_b200
CSRC = PKG / "csrc"
OUT = PKG / "vllm_gguf_plugin"
OBJ = PKG / "build"
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CU_FILES = ["capi.cu", "quantize_q8_1.cu", "dequantize.cu", "gemv.cu", "gemv1.cu", "mmq.cu", "noalloc.cu", "tp.cu", "moe_fused.cu"]
FAST_MATH = {"quantize_q8_1.cu", "gemv1.cu"}


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))


def _nvcc(src: Path, obj: Path, verbose: bool):
    cmd = [f"{CUDA}/bin/nvcc", "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", *ARCH, "-c", str(src), "-o", str(obj)]
    if src.name in FAST_MATH:
        cmd.insert(1, "--use_fast_math")
    if verbose:
        cmd += ["-Xptxas", "-v"]
    subprocess.check_call(cmd)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    so = OUT / "libgguf_b200.so"
    hdrs = _headers()
    srcs = [CSRC / f for f in CU_FILES if (CSRC / f).exists()]
    jobs = []
    for src in srcs:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *hdrs]):
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _nvcc(j[0], j[1], verbose), jobs))
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if force or jobs or _stale(so, objs):
        subprocess.check_call([f"{CUDA}/bin/nvcc", "-shared", *ARCH, "-o", str(so), *map(str, objs), "-lcudart"])
    return so


def build_torch_shim(force: bool = False) -> Path:
    import torch

    troot = Path(torch.__file__).parent
    so = OUT / "_C_gguf.abi3.so"
    src = CSRC / "torch_shim.cpp"
    if not force and not _stale(so, [src, PKG.parent / "include" / "gguf_b200.h"]):
        return so
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DUSE_CUDA", str(src), "-o", str(so),
           f"-I{troot / 'include'}", f"-I{sysconfig.get_paths()['include']}", f"-I{CUDA}/include",
           f"-L{OUT}", "-lgguf_b200", f"-L{troot / 'lib'}", "-ltorch", "-ltorch_cpu", "-lc10",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{troot / 'lib'}"]
    subprocess.check_call(cmd)
    return so


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force, verbose), build_torch_shim(force)


if __name__ == "__main__":
    print(*build_all(force="--force" in sys.argv, verbose="-v" in sys.argv), sep="\n")
