"""In-tree build of the sm_100a extension ``onecat_vllm.ops._C``.

Kernels are plain CUDA translation units compiled by nvcc for ``sm_100a`` only; ``bindings.cpp`` is the single file
that sees PyTorch headers. Objects are cached by modification time under ``csrc/build/``; the shared object lands next
to this file so that it travels with the source tree."""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
OUT = os.path.join(HERE, "_C.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + (["-DONECAT_GEMM_TRACE"] if os.environ.get("ONECAT_GEMM_TRACE") else [])
# --use_fast_math only affects __expf/exp2f-style intrinsics used in softmax/SiLU epilogues; accumulation stays fp32


def _sources() -> tuple[list[str], list[str]]:
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = ["bindings.cpp"]
    return cu, cpp


def _newer(src: str, obj: str, deps: list[str]) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in [src] + deps)


def build(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    bdir = os.path.join(CSRC, "build")
    os.makedirs(bdir, exist_ok=True)
    cu, cpp = _sources()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    jobs, objs = [], []
    for f in cu:
        src, obj = os.path.join(CSRC, f), os.path.join(bdir, f + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj])
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for f in cpp:
        src, obj = os.path.join(CSRC, f), os.path.join(bdir, f + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
                         "-DTORCH_API_INCLUDE_EXTENSION_H", "-I/usr/local/cuda/include"] + inc + ["-c", src, "-o", obj])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        if verbose:
            sys.stderr.write(r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(OUT) or force:
        libdirs = ce.library_paths(device_type="cuda")
        link = ["g++", "-shared", "-o", OUT] + objs + [f"-L{d}" for d in libdirs] + [f"-Wl,-rpath,{d}" for d in libdirs] + \
               ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        run(link)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
