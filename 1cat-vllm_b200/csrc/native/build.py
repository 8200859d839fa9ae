"""Builds the host-side native module ``onecat_vllm.utils._native`` (C++17 + pybind11, no CUDA, no PyTorch)."""
from __future__ import annotations

import os
import subprocess
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(os.path.dirname(HERE)), "utils", "_native.so")


def build(force: bool = False) -> str:
    import pybind11
    srcs = [os.path.join(HERE, f) for f in sorted(os.listdir(HERE)) if f.endswith(".cpp")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(s) < os.path.getmtime(OUT) for s in srcs):
        return OUT
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", f"-I{pybind11.get_include()}",
           f"-I{sysconfig.get_paths()['include']}"] + srcs + ["-o", OUT, "-lrt", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("native build failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
