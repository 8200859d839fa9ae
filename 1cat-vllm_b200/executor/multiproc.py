"""Multi-process executor: one worker process per GPU, RPCs broadcast to all workers, replies from rank 0
(reference: vllm/v1/executor/multiproc_executor.py:103 class, :268 worker monitor, :340 ``collective_rpc``, :542
``WorkerProc``, :769-792 death pipe, :950 ``worker_busy_loop``).

Transport: a shared-memory ring (``onecat_vllm.utils.shm_ring``, native spin-wait helper) carries the broadcast when the
native module is built; pipes are the fallback and always carry replies. A monitor thread watches worker sentinels and
marks the executor failed (→ ``EngineDeadError`` upstream); workers watch a death pipe and exit when the parent goes away."""
from __future__ import annotations

import multiprocessing as mp
import os
import pickle
import signal
import threading
import time
import traceback
from multiprocessing.connection import wait as mp_wait
from typing import Optional

from onecat_vllm import envs
from onecat_vllm.config import VllmConfig
from onecat_vllm.executor.uniproc import Executor
from onecat_vllm.logger import decorate_logs, init_logger

log = init_logger(__name__)


def _free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _load_native():
    try:
        from onecat_vllm.utils import _native
        return _native
    except ImportError:
        return None


_VIA_PIPE = b"\x00PIPE"


def _worker_main(cfg: VllmConfig, rank: int, local_rank: int, init_method: str, rpc_conn, death_conn, ready_conn, ring_spec=None) -> None:
    decorate_logs(f"Worker_{rank}")
    signal.signal(signal.SIGINT, signal.SIG_IGN)

    def watch_parent():
        try:
            death_conn.recv()  # EOF when the parent dies
        except EOFError:
            pass
        os._exit(1)

    threading.Thread(target=watch_parent, daemon=True).start()
    try:
        from onecat_vllm.worker.worker import Worker
        w = Worker(cfg, rank, local_rank, init_method=init_method)
        w.init_device()
        w.load_model()
        ready_conn.send(("READY", None))
    except Exception:
        ready_conn.send(("FAILED", traceback.format_exc()))
        return
    ring = None
    if ring_spec is not None:
        name, n, chunks, chunk_bytes = ring_spec
        ring = _load_native().ShmRing(name, n, chunks, chunk_bytes, False)
    while True:
        try:
            if ring is None:
                msg = rpc_conn.recv()
            else:  # broadcast arrives on the shared-memory ring; oversized messages fall back to the pipe
                raw = ring.read(rank, 500.0)
                if raw is None:
                    continue
                msg = rpc_conn.recv() if raw == _VIA_PIPE else pickle.loads(raw)
        except EOFError:
            break
        if msg is None:
            break
        method, args, kwargs, want_reply = msg
        try:
            fn = getattr(w, method) if isinstance(method, str) else None
            res = fn(*args, **kwargs) if fn else pickle.loads(method)(w, *args, **kwargs)
            if want_reply:
                rpc_conn.send(("OK", res))
        except Exception as e:
            rpc_conn.send(("ERR", f"{e!r}\n{traceback.format_exc()}"))
    try:
        w.shutdown()
    except Exception:
        pass


class MultiprocExecutor(Executor):
    uses_processes = True

    def _init_executor(self) -> None:
        cfg = self.cfg
        ws = cfg.parallel_config.world_size
        ctx = mp.get_context(envs.ONECAT_WORKER_MULTIPROC_METHOD)
        init_method = f"tcp://127.0.0.1:{_free_port()}"
        self.procs, self.conns, self._death = [], [], []
        readies = []
        self.ring, ring_spec = None, None
        native = _load_native()
        if native is not None:
            ring_spec = (f"/onecat-rpc-{os.getpid()}-{id(self) & 0xffff:x}", ws, envs.ONECAT_RPC_RING_CHUNKS, envs.ONECAT_RPC_RING_CHUNK_BYTES)
            self.ring = native.ShmRing(ring_spec[0], ws, ring_spec[2], ring_spec[3], True)
        for r in range(ws):
            parent, child = ctx.Pipe()
            d_r, d_w = ctx.Pipe(duplex=False)
            rd_r, rd_w = ctx.Pipe(duplex=False)
            p = ctx.Process(target=_worker_main, args=(cfg, r, r, init_method, child, d_r, rd_w, ring_spec), daemon=True, name=f"onecat-worker-{r}")
            p.start()
            child.close()
            d_r.close()
            rd_w.close()
            self.procs.append(p)
            self.conns.append(parent)
            self._death.append(d_w)
            readies.append(rd_r)
        deadline = time.time() + envs.ONECAT_HANDSHAKE_TIMEOUT_SECONDS * 5
        for r, c in enumerate(readies):
            while not c.poll(0.2):
                if not self.procs[r].is_alive():
                    self.shutdown()
                    raise RuntimeError(f"worker {r} died during start-up (exit code {self.procs[r].exitcode})")
                if time.time() > deadline:
                    self.shutdown()
                    raise TimeoutError("workers did not become ready in time")
            status, err = c.recv()
            if status != "READY":
                self.shutdown()
                raise RuntimeError(f"worker {r} failed to start:\n{err}")
        self._stop = False
        self._monitor = threading.Thread(target=self._watch_workers, daemon=True, name="onecat-worker-monitor")
        self._monitor.start()

    def _watch_workers(self) -> None:
        sentinels = [p.sentinel for p in self.procs]
        import sys
        try:
            mp_wait(sentinels)   # a sentinel fires when its process has exited
            dead = [p.name for p in self.procs if not p.is_alive()]
        except (OSError, ValueError):
            return   # the process objects were closed under us: the executor is being torn down
        if self._stop or sys.is_finalizing():
            return
        self.is_failed = True
        log.error(f"worker process(es) {dead} exited unexpectedly")
        cb = self.failure_callback
        if cb is not None:
            self.failure_callback = None
            cb()

    def collective_rpc(self, method, args=(), kwargs=None, timeout: Optional[float] = None) -> list:
        if self.is_failed:
            raise RuntimeError("executor failed")
        if not isinstance(method, str):
            import cloudpickle
            method = cloudpickle.dumps(method)
        timeout = timeout or envs.ONECAT_EXECUTE_MODEL_TIMEOUT_SECONDS
        self._broadcast((method, args, kwargs or {}, True))
        out = []
        deadline = time.time() + timeout
        for r, c in enumerate(self.conns):
            while not c.poll(0.05):
                if self.is_failed or not self.procs[r].is_alive():
                    self.is_failed = True
                    raise RuntimeError(f"worker {r} died during {method if isinstance(method, str) else 'rpc'}")
                if time.time() > deadline:
                    raise TimeoutError(f"RPC {method if isinstance(method, str) else 'fn'} timed out after {timeout}s")
            status, res = c.recv()
            if status != "OK":
                raise RuntimeError(f"worker {r} raised: {res}")
            out.append(res)
        return out

    def _broadcast(self, msg) -> None:
        if self.ring is None:
            for c in self.conns:
                c.send(msg)
            return
        raw = pickle.dumps(msg, protocol=pickle.HIGHEST_PROTOCOL)
        if len(raw) <= self.ring.chunk_bytes:
            if not self.ring.write(raw, 30000.0):
                self.is_failed = True
                raise RuntimeError("a worker stopped consuming the RPC ring")
            return
        if not self.ring.write(_VIA_PIPE, 30000.0):
            self.is_failed = True
            raise RuntimeError("a worker stopped consuming the RPC ring")
        for c in self.conns:
            c.send(msg)

    def shutdown(self) -> None:
        self._stop = True
        try:
            if getattr(self, "procs", None):
                self._broadcast(None)
        except Exception:
            pass
        for p in getattr(self, "procs", []):
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()  # exact process we started
                p.join(timeout=2)
        for d in getattr(self, "_death", []):
            try:
                d.close()
            except Exception:
                pass
        self.procs, self.conns = [], []
        self.ring = None
