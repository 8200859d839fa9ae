"""Builds ``onecat_vllm/utils/_cumem.so``: the sleep-mode device allocator (plain C++; the CUDA driver is loaded at run time)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(os.path.dirname(HERE)), "utils", "_cumem.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "cumem_allocator.cpp")
    if not force and os.path.exists(OUT) and os.path.getmtime(src) < os.path.getmtime(OUT):
        return OUT
    inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", f"-I{inc}", src, "-o", OUT, "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("cumem allocator build failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
