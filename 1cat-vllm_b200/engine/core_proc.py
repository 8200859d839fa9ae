"""Engine core in its own process behind ZMQ, and the clients that talk to it
(reference: vllm/v1/engine/core.py:1018 ``EngineCoreProc``, :1134-1273 handshake, :1376 busy loop, :1491 utility calls,
:1569-1581 ``ENGINE_CORE_DEAD``; clients vllm/v1/engine/core_client.py:461 ``MPClient``, :748 sync, :919 asyncio).

Sockets: the client binds a ROUTER for inputs and a PULL for outputs; the engine connects a DEALER (identity = engine index)
and a PUSH. First input frame = 1-byte request type (ADD / ABORT / UTILITY), the rest is the msgpack body (+ buffers).
Handshake: engine → ``HELLO``; client → config acknowledgement; engine → ``READY`` with ``num_gpu_blocks``/``max_model_len``.
If the core dies it sends ``ENGINE_CORE_DEAD`` (when it still can) and the client raises ``EngineDeadError``; a monitor thread
also watches the process sentinel."""
from __future__ import annotations

import multiprocessing as mp
import os
import pickle
import queue
import signal
import threading
import time
import traceback
from typing import Any, Optional

import zmq
import zmq.asyncio

from onecat_vllm import envs
from onecat_vllm.config import VllmConfig
from onecat_vllm.engine import serial
from onecat_vllm.engine.core import EngineDeadError
from onecat_vllm.logger import decorate_logs, init_logger
from onecat_vllm.request import EngineCoreOutput, EngineCoreOutputs, EngineCoreRequest

log = init_logger(__name__)
ENGINE_CORE_DEAD = b"ENGINE_CORE_DEAD"


def _ipc_path(tag: str) -> str:
    import tempfile
    import uuid
    return f"ipc://{tempfile.gettempdir()}/onecat-{tag}-{uuid.uuid4().hex[:12]}"


# ----------------------------------------------------------------------------- engine side
def run_engine_core(cfg: VllmConfig, input_addr: str, output_addr: str, engine_index: int, log_stats: bool, death_conn,
                    coord_addrs: Optional[dict] = None) -> None:
    decorate_logs(f"EngineCore_{engine_index}")
    signal.signal(signal.SIGINT, signal.SIG_IGN)
    if death_conn is not None:
        def watch():
            try:
                death_conn.recv()
            except EOFError:
                pass
            os._exit(1)
        threading.Thread(target=watch, daemon=True).start()
    pc = cfg.parallel_config
    if pc.data_parallel_size > 1 and cfg.device == "cuda":
        # replica i owns GPUs [i * world, (i + 1) * world) of those visible to the frontend; set before CUDA initialises here
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids = vis.split(",") if vis else [str(i) for i in range(pc.data_parallel_size * pc.world_size)]
        os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(ids[engine_index * pc.world_size:(engine_index + 1) * pc.world_size])
    ctx = zmq.Context()
    inp = ctx.socket(zmq.DEALER)
    inp.setsockopt(zmq.IDENTITY, engine_index.to_bytes(2, "little"))
    inp.connect(input_addr)
    out = ctx.socket(zmq.PUSH)
    out.connect(output_addr)
    core = None
    try:
        inp.send_multipart(serial.encode({"status": "HELLO", "local": True, "headless": False}))
        if not inp.poll(envs.ONECAT_HANDSHAKE_TIMEOUT_SECONDS * 1000):
            raise TimeoutError("no handshake reply from the frontend")
        serial.decode(inp.recv_multipart())
        from onecat_vllm.engine.core import EngineCore
        core = EngineCore(cfg, log_stats=log_stats)
        inp.send_multipart(serial.encode({"status": "READY", "num_gpu_blocks": cfg.cache_config.num_gpu_blocks,
                                          "max_model_len": cfg.model_config.max_model_len, "dtype": str(cfg.model_config.dtype)}))
        reporter = None
        if coord_addrs is not None:
            from onecat_vllm.engine.coordinator import EngineReporter
            reporter = EngineReporter(engine_index, coord_addrs)
        _busy_loop(core, inp, out, engine_index, reporter)
    except Exception:
        log.error("engine core failed:\n" + traceback.format_exc())
        try:
            out.send_multipart([ENGINE_CORE_DEAD], flags=zmq.NOBLOCK)
        except Exception:
            pass
    finally:
        if core is not None:
            core.shutdown()
        inp.close(linger=200)
        out.close(linger=200)
        ctx.term()


def _busy_loop(core, inp, out, engine_index: int, reporter=None) -> None:
    """Drain inputs, step while there is work, block on the socket when idle (reference: core.py:1376-1440). With a data-parallel
    coordinator the engine reports its queue lengths after every step and the edges between having work and having none."""
    while True:
        if reporter is not None:
            reporter.poll_start_wave()
            if core.scheduler.has_requests():
                reporter.became_busy()
            else:
                reporter.became_idle()
        timeout = 0 if core.scheduler.has_requests() else 200
        while inp.poll(timeout):
            frames = inp.recv_multipart()
            kind, body = frames[0], frames[1:]
            if kind == serial.REQ_ADD:
                try:
                    core.add_request(EngineCoreRequest.from_wire(serial.decode(body)))
                except Exception as e:  # bad request: report as an aborted output instead of killing the engine
                    d = serial.decode(body)
                    o = EngineCoreOutputs([EngineCoreOutput(d.get("request_id", "?"), [], finish_reason=3, stop_reason=repr(e))])
                    out.send_multipart(serial.encode(_outs_wire(o, engine_index)))
            elif kind == serial.REQ_ABORT:
                core.abort_requests(serial.decode(body))
            elif kind == serial.REQ_UTILITY:
                call_id, method, args = serial.decode(body)
                if method == "shutdown":
                    return
                try:
                    res = getattr(core, method)(*args)
                    try:
                        serial.encode(res)
                    except TypeError:
                        res = repr(res)
                    reply = {"call_id": call_id, "result": res}
                except Exception as e:
                    reply = {"call_id": call_id, "error": f"{e!r}"}
                out.send_multipart(serial.encode({"utility_output": reply, "engine_index": engine_index}))
            timeout = 0
        if core.scheduler.has_requests():
            if reporter is not None:
                reporter.became_busy()
            outs, _ = core.step()
            for client, o in outs.items():
                out.send_multipart(serial.encode(_outs_wire(o, engine_index)))
            if reporter is not None:
                reporter.report(len(core.scheduler.waiting), len(core.scheduler.running))


def _outs_wire(o: EngineCoreOutputs, engine_index: int) -> dict:
    st = o.scheduler_stats
    return {"engine_index": engine_index, "outputs": [x.to_wire() for x in o.outputs], "timestamp": o.timestamp,
            "scheduler_stats": dict(st.__dict__) if st is not None else None}


# ----------------------------------------------------------------------------- client side
class _MPClientBase:
    def __init__(self, cfg: VllmConfig, log_stats: bool, asyncio_mode: bool):
        self.cfg = cfg
        self.sync_ctx = zmq.Context()
        self.input_addr, self.output_addr = _ipc_path("in"), _ipc_path("out")
        hs = self.sync_ctx.socket(zmq.ROUTER)
        hs.bind(self.input_addr)
        pull = self.sync_ctx.socket(zmq.PULL)
        pull.bind(self.output_addr)
        mctx = mp.get_context("spawn")
        # data parallelism: one engine core (scheduler + executor over tp*pp GPUs) per replica, all on the same socket pair;
        # the ROUTER addresses a replica by its identity (reference: v1/engine/core_client.py:1169 DPAsyncMPClient, :1349 DPLBAsyncMPClient)
        self.num_engines = max(1, cfg.parallel_config.data_parallel_size)
        self.procs, self._death_ws = [], []
        # opt-in coordinator process: the replicas' queue lengths reach every front end that subscribes, and idle / running waves
        # are kept for the group (reference: v1/engine/coordinator.py)
        self.coordinator = self._coord_sub = None
        coord_addrs = None
        if self.num_engines > 1 and envs.ONECAT_DP_COORDINATOR:
            from onecat_vllm.engine.coordinator import DPCoordinator
            self.coordinator = DPCoordinator(self.num_engines)
            coord_addrs = self.coordinator.addresses
        for i in range(self.num_engines):
            d_r, d_w = mctx.Pipe(duplex=False)
            pr = mctx.Process(target=run_engine_core, args=(cfg, self.input_addr, self.output_addr, i, log_stats, d_r, coord_addrs), daemon=True,
                              name=f"onecat-engine-core-{i}")
            pr.start()
            d_r.close()
            self.procs.append(pr)
            self._death_ws.append(d_w)
        self.proc, self._death_w = self.procs[0], self._death_ws[0]
        self.engine_ids = [i.to_bytes(2, "little") for i in range(self.num_engines)]
        self.engine_id = self.engine_ids[0]
        self._owner: dict = {}                      # request id -> replica
        self._inflight = [0] * self.num_engines     # requests sent and not yet finished
        self._lb = [(0, 0)] * self.num_engines      # last reported (waiting, running) per replica
        if coord_addrs is not None:
            from onecat_vllm.engine.coordinator import FrontendSubscriber

            def _table(m: dict) -> None:
                for i, c in enumerate(m.get("counts", [])[: self.num_engines]):
                    self._lb[i] = (int(c[0]), int(c[1]))
            self._coord_sub = FrontendSubscriber(coord_addrs, on_update=_table)
        self.dead = False
        try:
            self._handshake(hs)
        except Exception:
            self._kill()
            raise
        if asyncio_mode:
            # same underlying sockets, awaitable API: the engine's connections (and the ROUTER's routing table) survive
            self.inp, self.outp = zmq.asyncio.Socket.shadow(hs), zmq.asyncio.Socket.shadow(pull)
            self._keep = (hs, pull)
        else:
            self.inp, self.outp = hs, pull
        self._call_id = 0
        self._mon = threading.Thread(target=self._monitor, daemon=True)
        self._mon.start()

    def _handshake(self, hs) -> None:
        deadline = time.time() + envs.ONECAT_HANDSHAKE_TIMEOUT_SECONDS * 5
        ready = 0
        while ready < self.num_engines:
            if not hs.poll(200):
                for pr in self.procs:
                    if not pr.is_alive():
                        raise RuntimeError(f"engine core exited during start-up (code {pr.exitcode})")
                if time.time() > deadline:
                    raise TimeoutError("engine core handshake timed out")
                continue
            ident, *frames = hs.recv_multipart()
            msg = serial.decode(frames)
            if msg["status"] == "HELLO":
                hs.send_multipart([ident] + serial.encode({"ack": True}))
            elif msg["status"] == "READY":
                self.cfg.cache_config.num_gpu_blocks = msg["num_gpu_blocks"]
                ready += 1

    def _monitor(self) -> None:
        while not getattr(self, "_closing", False):
            if any(not pr.is_alive() for pr in self.procs):
                if not getattr(self, "_closing", False):
                    self.dead = True
                return
            time.sleep(0.1)

    # ---- replica choice and bookkeeping
    def _route(self, req: EngineCoreRequest) -> bytes:
        """Replica for a new request: the one asked for, else the least loaded by (4 x waiting + running) as last reported,
        plus what was sent since (reference: core_client.py:1400-1430 ``get_core_engine_for_request``)."""
        n = self.num_engines
        if n == 1:
            return self.engine_id
        e = req.data_parallel_rank
        if e is None or not 0 <= e < n:
            e = min(range(n), key=lambda i: (4 * self._lb[i][0] + self._lb[i][1] + self._inflight[i], i))
        self._owner[req.request_id] = e
        self._inflight[e] += 1
        if self._coord_sub is not None:
            self._coord_sub.request_routed(e)
        return self.engine_ids[e]

    def _abort_targets(self, ids: list) -> dict:
        by: dict = {}
        for rid in ids:
            e = self._owner.pop(rid, 0)
            if self.num_engines > 1:
                self._inflight[e] = max(0, self._inflight[e] - 1)
            by.setdefault(e, []).append(rid)
        return by

    def _account(self, o: EngineCoreOutputs) -> None:
        if self.num_engines == 1:
            return
        e = o.engine_index
        if o.scheduler_stats is not None:
            self._lb[e] = (o.scheduler_stats.num_waiting_reqs, o.scheduler_stats.num_running_reqs)
        for x in o.outputs:
            if x.finished and self._owner.pop(x.request_id, None) is not None:
                self._inflight[e] = max(0, self._inflight[e] - 1)

    def _check(self) -> None:
        if self.dead:
            raise EngineDeadError("the engine core process died")

    def _close_coordinator(self) -> None:
        if getattr(self, "_coord_sub", None) is not None:
            self._coord_sub.close()
            self._coord_sub = None
        if getattr(self, "coordinator", None) is not None:
            self.coordinator.close()
            self.coordinator = None

    def _kill(self) -> None:
        self._closing = True
        self._close_coordinator()
        for pr in self.procs:
            if pr.is_alive():
                pr.terminate()  # exact children we started
                pr.join(5)

    @staticmethod
    def _parse(frames) -> EngineCoreOutputs:
        if frames[0] == ENGINE_CORE_DEAD:
            raise EngineDeadError("the engine core reported a fatal error")
        d = serial.decode(frames)
        if "utility_output" in d:
            return EngineCoreOutputs(utility_output=d["utility_output"])
        from onecat_vllm.core.scheduler import SchedulerStats
        st = SchedulerStats(**d["scheduler_stats"]) if d.get("scheduler_stats") else None
        return EngineCoreOutputs([EngineCoreOutput.from_wire(x) for x in d["outputs"]], st, d.get("timestamp", 0.0), d.get("engine_index", 0))


class SyncMPClient(_MPClientBase):
    def __init__(self, cfg: VllmConfig, log_stats: bool = False):
        super().__init__(cfg, log_stats, asyncio_mode=False)
        self._util: dict = {}

    def add_request(self, req: EngineCoreRequest) -> None:
        self._check()
        self.inp.send_multipart([self._route(req), serial.REQ_ADD] + serial.encode(req.to_wire()))

    def abort_requests(self, ids: list) -> None:
        if ids and not self.dead:
            for e, rids in self._abort_targets(list(ids)).items():
                self.inp.send_multipart([self.engine_ids[e], serial.REQ_ABORT] + serial.encode(rids))

    def get_output(self, timeout_s: float = 300.0) -> EngineCoreOutputs:
        deadline = time.time() + timeout_s
        while True:
            self._check()
            if self.outp.poll(100):
                o = self._parse(self.outp.recv_multipart())
                if o.utility_output is not None:
                    self._util.setdefault(o.utility_output["call_id"], []).append(o.utility_output)
                    continue
                self._account(o)
                return o
            if time.time() > deadline:
                raise TimeoutError("no output from the engine core")

    def call_utility(self, method: str, *args):
        self._check()
        self._call_id += 1
        cid = self._call_id
        for eid in self.engine_ids:  # utility calls go to every replica
            self.inp.send_multipart([eid, serial.REQ_UTILITY] + serial.encode([cid, method, list(args)]))
        deadline = time.time() + envs.ONECAT_EXECUTE_MODEL_TIMEOUT_SECONDS
        while len(self._util.get(cid, ())) < self.num_engines:
            self._check()
            if self.outp.poll(100):
                o = self._parse(self.outp.recv_multipart())
                if o.utility_output is not None:
                    self._util.setdefault(o.utility_output["call_id"], []).append(o.utility_output)
            if time.time() > deadline:
                raise TimeoutError(f"utility call {method} timed out")
        rs = self._util.pop(cid)
        for r in rs:
            if "error" in r:
                raise RuntimeError(r["error"])
        return rs[0]["result"] if self.num_engines == 1 else [r["result"] for r in rs]

    def shutdown(self) -> None:
        self._closing = True
        try:
            if not self.dead:
                for eid, pr in zip(self.engine_ids, self.procs):
                    if pr.is_alive():
                        self.inp.send_multipart([eid, serial.REQ_UTILITY] + serial.encode([0, "shutdown", []]))
                for pr in self.procs:
                    pr.join(10)
        except Exception:
            pass
        self._kill()
        for s in (getattr(self, "inp", None), getattr(self, "outp", None)):
            if s is not None:
                s.close(linger=0)
        for w in self._death_ws:
            try:
                w.close()
            except Exception:
                pass


class AsyncMPClient(_MPClientBase):
    def __init__(self, cfg: VllmConfig, log_stats: bool = False):
        super().__init__(cfg, log_stats, asyncio_mode=True)
        self._util_futs: dict = {}

    async def add_request_async(self, req: EngineCoreRequest) -> None:
        self._check()
        await self.inp.send_multipart([self._route(req), serial.REQ_ADD] + serial.encode(req.to_wire()))

    async def abort_requests_async(self, ids: list) -> None:
        if ids and not self.dead:
            for e, rids in self._abort_targets(list(ids)).items():
                await self.inp.send_multipart([self.engine_ids[e], serial.REQ_ABORT] + serial.encode(rids))

    async def get_output_async(self) -> EngineCoreOutputs:
        while True:
            self._check()
            if await self.outp.poll(200):
                o = self._parse(await self.outp.recv_multipart())
                if o.utility_output is not None:
                    cid = o.utility_output["call_id"]
                    ent = self._util_futs.get(cid)
                    if ent is not None:
                        ent[1].append(o.utility_output)
                        if len(ent[1]) == self.num_engines:
                            self._util_futs.pop(cid)
                            if not ent[0].done():
                                ent[0].set_result(ent[1])
                    continue
                self._account(o)
                return o

    async def call_utility_async(self, method: str, *args):
        import asyncio
        self._check()
        self._call_id += 1
        cid = self._call_id
        fut = asyncio.get_running_loop().create_future()
        self._util_futs[cid] = (fut, [])
        for eid in self.engine_ids:
            await self.inp.send_multipart([eid, serial.REQ_UTILITY] + serial.encode([cid, method, list(args)]))
        rs = await asyncio.wait_for(fut, envs.ONECAT_EXECUTE_MODEL_TIMEOUT_SECONDS)
        for r in rs:
            if "error" in r:
                raise RuntimeError(r["error"])
        return rs[0]["result"] if self.num_engines == 1 else [r["result"] for r in rs]

    def shutdown(self) -> None:
        self._closing = True
        self._kill()
        for s in (getattr(self, "inp", None), getattr(self, "outp", None)):
            if s is not None:
                s.close(linger=0)
        for w in self._death_ws:
            try:
                w.close()
            except Exception:
                pass


# ----------------------------------------------------------------------------- stand-alone engine core
def main_headless(argv=None) -> None:
    """``python -m onecat_vllm.engine.core_proc --input-addr A --output-addr B <engine args>``: an engine core that connects to
    a front end which already listens on the two addresses (the native front end starts it this way). It speaks the same
    handshake and frames as the engine processes the Python clients spawn, and exits when its parent does."""
    import argparse
    from onecat_vllm.config import EngineArgs
    ap = argparse.ArgumentParser("engine-core")
    ap.add_argument("--input-addr", required=True)
    ap.add_argument("--output-addr", required=True)
    ap.add_argument("--engine-index", type=int, default=0)
    ap.add_argument("model_tag", nargs="?", default=None)
    EngineArgs.add_cli_args(ap)
    a = ap.parse_args(argv)
    if a.model_tag:
        a.model = a.model_tag
    ea = EngineArgs.from_cli_args(a)
    parent = os.getppid()

    def watch_parent():
        while os.getppid() == parent:
            time.sleep(0.5)
        os._exit(1)
    threading.Thread(target=watch_parent, daemon=True).start()
    run_engine_core(ea.create_engine_config(), a.input_addr, a.output_addr, a.engine_index, not ea.disable_log_stats, None)


if __name__ == "__main__":
    main_headless()
