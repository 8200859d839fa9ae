"""Launcher of the native (C++) front end: builds the binary when its sources are newer, finds the libzmq that ships inside pyzmq
and starts ``onecat_frontend`` with an engine-core command line made from the usual engine arguments.

    python -m onecat_vllm.entrypoints.native_frontend /path/to/checkpoint --port 8000 --tensor-parallel-size 2

The front end itself is ``csrc/frontend/server.cpp`` (HTTP server, tokenizer, ZMQ/msgpack client of the engine core).
(reference: the ``vllm-rs`` launcher in rust/src/main.rs)"""
from __future__ import annotations

import glob
import importlib.util
import os
import shlex
import sys


def binary_path() -> str:
    here = os.path.dirname(os.path.abspath(__file__))
    spec = importlib.util.spec_from_file_location("_onecat_frontend_build", os.path.join(os.path.dirname(here), "csrc", "frontend", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


def find_libzmq() -> str:
    import zmq
    root = os.path.dirname(os.path.dirname(zmq.__file__))
    hits = sorted(glob.glob(os.path.join(root, "pyzmq.libs", "libzmq*.so*"))) + sorted(glob.glob(os.path.join(os.path.dirname(zmq.__file__), "**", "libzmq*.so*"), recursive=True))
    return hits[0] if hits else "libzmq.so.5"


def command(engine_args: list[str], host: str = "127.0.0.1", port: int = 8000, tokenizer: str = "byte", served_model_name: str = "model",
            handshake_timeout: int = 600) -> list[str]:
    engine = [sys.executable, "-m", "onecat_vllm.engine.core_proc", "--input-addr", "{input}", "--output-addr", "{output}"] + list(engine_args)
    return [binary_path(), "--host", host, "--port", str(port), "--tokenizer", tokenizer, "--served-model-name", served_model_name,
            "--zmq-lib", find_libzmq(), "--handshake-timeout", str(handshake_timeout), "--engine-cmd", " ".join(shlex.quote(a) for a in engine)]


def main(argv=None) -> None:
    import argparse
    ap = argparse.ArgumentParser("native-frontend", description="HTTP front end in C++; unknown arguments go to the engine core")
    ap.add_argument("model")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tokenizer", default=None, help="directory with tokenizer.json / tekken.json, or 'byte' (default: the model directory)")
    ap.add_argument("--served-model-name", default=None)
    a, rest = ap.parse_known_args(argv)
    tok = a.tokenizer or (a.model if os.path.isdir(a.model) else "byte")
    cmd = command([a.model] + rest, a.host, a.port, tok, a.served_model_name or a.model)
    os.execv(cmd[0], cmd)


if __name__ == "__main__":
    main()
