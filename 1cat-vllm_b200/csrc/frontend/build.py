"""Builds the native front end (``onecat_vllm/entrypoints/onecat_frontend``): plain C++17, no third-party headers; libzmq is
loaded at run time."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(os.path.dirname(HERE)), "entrypoints", "onecat_frontend")


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, f) for f in ("server.cpp", "tokenizer.h", "value.h", "zmq_dyn.h", "unicode_tables.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(s) < os.path.getmtime(OUT) for s in srcs):
        return OUT
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", "-Wno-unused-result", os.path.join(HERE, "server.cpp"), "-o", OUT, "-ldl", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("front end build failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
