"""Data-parallel coordinator: one small process between the engine replicas and any number of front ends
(reference: vllm/v1/engine/coordinator.py ``DPCoordinator`` / ``DPCoordinatorProc``).

* Every engine pushes its queue lengths (waiting, running) after each step, and a ``wave_complete`` note when it runs out of work.
* The coordinator publishes the table of all engines' queue lengths, the current wave number and whether the engines are running,
  at most every ``publish_interval_s`` and only when something changed; front ends subscribe and balance new requests on it, so that
  several API-server processes see one another's load.
* Waves: the engines of a data-parallel group are either all running or all idle. A front end that routes a request while the group
  is idle sends ``first_req``; the coordinator then marks the group running and broadcasts ``start_wave`` to the engines. When every
  engine has reported ``wave_complete`` for the current wave the group goes idle and the wave number advances. A ``first_req`` that
  carries an old wave number raced with the end of that wave and starts the next one, which is what keeps a request from being
  stranded on a replica whose peers have gone to sleep.

Wire format: msgpack maps over ZMQ (PUSH/PULL towards the coordinator, PUB/SUB away from it)."""
from __future__ import annotations

import multiprocessing as mp
import threading
import time
from typing import Callable, Optional

import msgpack
import zmq


class CoordinatorState:
    """The bookkeeping itself, free of sockets (driven by ``run_coordinator`` and by the tests)."""

    def __init__(self, num_engines: int):
        self.n = num_engines
        self.counts = [[0, 0] for _ in range(num_engines)]
        self.wave = 0
        self.running = False
        self._idle: set = set()
        self.dirty = True

    def on_engine(self, msg: dict) -> Optional[dict]:
        """An engine's report; returns a broadcast for the engines when one is due."""
        e = int(msg["engine"])
        if "stats" in msg:
            c = [int(msg["stats"][0]), int(msg["stats"][1])]
            if c != self.counts[e]:
                self.counts[e] = c
                self.dirty = True
        if "wave_complete" in msg and int(msg["wave_complete"]) == self.wave and self.running:
            self._idle.add(e)
            if len(self._idle) == self.n:       # every replica ran dry: the wave is over
                self.running = False
                self.wave += 1
                self._idle.clear()
                self.dirty = True
        if msg.get("start_wave") is not None:   # an engine got work while the group was idle (a request sent past the front ends)
            return self.on_first_req({"wave": int(msg["start_wave"]), "engine": e})
        return None

    def on_first_req(self, msg: dict) -> Optional[dict]:
        """A front end routed a request while it believed the group idle; returns the ``start_wave`` broadcast when the group was."""
        if self.running:
            return None        # the wave it belongs to is under way (or a newer one is): nothing to wake
        self.running = True
        self._idle.clear()
        self.dirty = True
        return {"start_wave": self.wave, "exclude": int(msg.get("engine", -1))}

    def snapshot(self) -> dict:
        self.dirty = False
        return {"counts": [list(c) for c in self.counts], "wave": self.wave, "running": self.running}


def run_coordinator(num_engines: int, engine_in: str, front_in: str, front_pub: str, engine_pub: str, ready=None, stop=None,
                    publish_interval_s: float = 0.1) -> None:
    ctx = zmq.Context()
    s_eng, s_front = ctx.socket(zmq.PULL), ctx.socket(zmq.PULL)
    p_front, p_eng = ctx.socket(zmq.PUB), ctx.socket(zmq.PUB)
    for s, a in ((s_eng, engine_in), (s_front, front_in), (p_front, front_pub), (p_eng, engine_pub)):
        s.setsockopt(zmq.LINGER, 0)
        s.bind(a)
    if ready is not None:
        ready.set()
    st = CoordinatorState(num_engines)
    poller = zmq.Poller()
    poller.register(s_eng, zmq.POLLIN)
    poller.register(s_front, zmq.POLLIN)
    last = 0.0
    try:
        while stop is None or not stop.is_set():
            for sock, _ in poller.poll(50):
                msg = msgpack.unpackb(sock.recv(), raw=False)
                if msg.get("shutdown"):
                    return
                out = st.on_engine(msg) if sock is s_eng else st.on_first_req(msg)
                if out is not None:
                    p_eng.send(msgpack.packb(out))
            now = time.monotonic()
            if st.dirty and now - last >= publish_interval_s:
                p_front.send(msgpack.packb(st.snapshot()))
                last = now
    finally:
        for s in (s_eng, s_front, p_front, p_eng):
            s.close()
        ctx.term()


class DPCoordinator:
    """Owner of the coordinator process. ``addresses`` names the four endpoints (``engine_in``, ``front_in``, ``front_pub``,
    ``engine_pub``) to hand to engines and front ends."""

    def __init__(self, num_engines: int, addresses: Optional[dict] = None):
        import os
        import tempfile
        if addresses is None:
            d = tempfile.mkdtemp(prefix="onecat-dpc-")
            addresses = {k: f"ipc://{os.path.join(d, k)}" for k in ("engine_in", "front_in", "front_pub", "engine_pub")}
        self.addresses = addresses
        ctx = mp.get_context("spawn")
        self._ready = ctx.Event()
        self.proc = ctx.Process(target=run_coordinator, args=(num_engines, addresses["engine_in"], addresses["front_in"], addresses["front_pub"],
                                                              addresses["engine_pub"], self._ready), daemon=True, name="DPCoordinator")
        self.proc.start()
        if not self._ready.wait(30):
            raise RuntimeError("the data-parallel coordinator did not start")

    def close(self) -> None:
        if self.proc.is_alive():
            try:
                ctx = zmq.Context.instance()
                s = ctx.socket(zmq.PUSH)
                s.setsockopt(zmq.LINGER, 200)
                s.connect(self.addresses["front_in"])
                s.send(msgpack.packb({"shutdown": True}))
                s.close()
            except Exception:
                pass
            self.proc.join(3)
            if self.proc.is_alive():
                self.proc.terminate()


class EngineReporter:
    """Engine side: push queue lengths and wave notes; listen for ``start_wave``."""

    def __init__(self, engine_index: int, addresses: dict):
        self.e = engine_index
        self.ctx = zmq.Context.instance()
        self.push = self.ctx.socket(zmq.PUSH)
        self.push.setsockopt(zmq.LINGER, 0)
        self.push.connect(addresses["engine_in"])
        self.sub = self.ctx.socket(zmq.SUB)
        self.sub.setsockopt(zmq.SUBSCRIBE, b"")
        self.sub.connect(addresses["engine_pub"])
        self.wave = 0
        self.running = False
        self._last = None

    def report(self, waiting: int, running: int) -> None:
        if (waiting, running) != self._last:
            self._last = (waiting, running)
            self.push.send(msgpack.packb({"engine": self.e, "stats": [waiting, running]}))

    def became_busy(self) -> None:
        """Work arrived while this engine thought the group idle."""
        if not self.running:
            self.running = True
            self.push.send(msgpack.packb({"engine": self.e, "start_wave": self.wave}))

    def became_idle(self) -> None:
        if self.running:
            self.running = False
            self.push.send(msgpack.packb({"engine": self.e, "wave_complete": self.wave}))
            self.wave += 1

    def poll_start_wave(self) -> Optional[int]:
        """The wave a broadcast asks this engine to join (None when there is none pending)."""
        got = None
        while self.sub.poll(0):
            m = msgpack.unpackb(self.sub.recv(), raw=False)
            if "start_wave" in m and m.get("exclude") != self.e:
                self.wave = max(self.wave, int(m["start_wave"]))
                self.running = True
                got = self.wave
        return got

    def close(self) -> None:
        self.push.close()
        self.sub.close()


class FrontendSubscriber:
    """Front-end side: a thread keeps the latest table; ``first_req`` is sent when a request is routed while the group is idle."""

    def __init__(self, addresses: dict, on_update: Optional[Callable[[dict], None]] = None):
        self.ctx = zmq.Context.instance()
        self.sub = self.ctx.socket(zmq.SUB)
        self.sub.setsockopt(zmq.SUBSCRIBE, b"")
        self.sub.connect(addresses["front_pub"])
        self.push = self.ctx.socket(zmq.PUSH)
        self.push.setsockopt(zmq.LINGER, 0)
        self.push.connect(addresses["front_in"])
        self.state: dict = {"counts": [], "wave": 0, "running": False}
        self.on_update = on_update
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self.thread = threading.Thread(target=self._loop, daemon=True, name="dp-coordinator-sub")
        self.thread.start()

    def _loop(self) -> None:
        while not self._stop.is_set():
            if self.sub.poll(100):
                m = msgpack.unpackb(self.sub.recv(), raw=False)
                with self._lock:
                    self.state = m
                if self.on_update is not None:
                    self.on_update(m)

    def counts(self) -> list:
        with self._lock:
            return [list(c) for c in self.state.get("counts", [])]

    def request_routed(self, engine: int) -> None:
        with self._lock:
            running, wave = self.state.get("running", False), self.state.get("wave", 0)
        if not running:
            self.push.send(msgpack.packb({"first_req": True, "engine": engine, "wave": wave}))

    def close(self) -> None:
        self._stop.set()
        self.thread.join(1)
        self.sub.close()
        self.push.close()
