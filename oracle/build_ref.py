"""Build the reference plugin's own CUDA extension into oracle/_ref/ (test infrastructure).

The reference's native path is two translation units
(vllm_gguf_plugin/csrc/torch_bindings.cpp and csrc/gguf/gguf_kernel.cu, built by
setup.py:34-61 with -O3 -std=c++17 --use_fast_math -DUSE_CUDA).  This recipe compiles
them from where they lie, for sm_100a, with two additions that do not touch the sources:

* ``-D_C_gguf=_C_gguf_ref`` renames only the *string* of the torch library namespace
  (the registration macros stringize their argument after macro expansion), so the
  reference ops load as ``torch.ops._C_gguf_ref.*`` next to the product's ``_C_gguf``
  in one process;
* ``ref_harness.cu`` includes gguf_kernel.cu and exports the internal q8_1 quantizer.

Output: oracle/_ref/_C_gguf_ref.so (git-ignored).  Needs the reference checkout; when it
is absent the already-built file is used as is.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

def _ref_root():
    sys.path.insert(0, str(HERE.parent))
    from oracle import reference_root

    return reference_root()



def _torch_paths():
    import torch

    root = Path(torch.__file__).parent
    return root / "include", root / "lib"


def build(force: bool = False) -> Path | None:
    so = OUT / "_C_gguf_ref.so"
    ref = _ref_root()
    if ref is None:
        return so if so.exists() else None
    csrc = ref / "vllm_gguf_plugin" / "csrc"
    srcs = [csrc / "torch_bindings.cpp", csrc / "gguf" / "gguf_kernel.cu", HERE / "ref_harness.cu"]
    hdrs = list((csrc / "gguf").glob("*")) + [Path(__file__)]
    if so.exists() and not force:
        newest = max(p.stat().st_mtime for p in srcs + hdrs)
        if so.stat().st_mtime >= newest:
            return so
    OUT.mkdir(exist_ok=True)
    tinc, tlib = _torch_paths()
    pyinc = sysconfig.get_paths()["include"]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    common = ["-O3", "-std=c++17", "-DUSE_CUDA", "-D_C_gguf=_C_gguf_ref",
              f"-I{csrc}", f"-I{csrc / 'gguf'}", f"-I{tinc}", f"-I{pyinc}", f"-I{cuda}/include"]
    obj_b = Path("/tmp") / "gguf_ref_torch_bindings.o"
    obj_k = Path("/tmp") / "gguf_ref_harness.o"
    subprocess.check_call(["g++", "-fPIC", "-c", str(srcs[0]), "-o", str(obj_b)] + common)
    # ref_harness.cu textually includes gguf_kernel.cu, so one nvcc call builds both.
    subprocess.check_call([f"{cuda}/bin/nvcc", "-Xcompiler", "-fPIC", "--use_fast_math",
                           "-gencode", "arch=compute_100a,code=sm_100a",
                           "-c", str(srcs[2]), "-o", str(obj_k)] + common)
    subprocess.check_call(["g++", "-shared", "-o", str(so), str(obj_b), str(obj_k),
                           f"-L{tlib}", "-ltorch", "-ltorch_cuda", "-ltorch_cpu", "-lc10", "-lc10_cuda",
                           f"-L{cuda}/lib64", "-lcudart", f"-Wl,-rpath,{tlib}"])
    return so


if __name__ == "__main__":
    p = build(force="--force" in sys.argv)
    print(p if p else "reference checkout absent and no prebuilt oracle/_ref/_C_gguf_ref.so")
