"""Parameter sweeps over the serving benchmark: start a server once per server-parameter set, run the client once per
client-parameter set (``--num-runs`` repeats), keep one result file per run so an interrupted sweep resumes, and write a summary
table with the Pareto front of throughput against latency. ``bench sweep workload`` finds the useful range of one load variable
(request rate or concurrency) by measuring the serial and the saturated operating points first and spacing the rest between them
(reference: vllm/benchmarks/sweep/serve.py ``run_combs``/``--resume``/``--dry-run``; param_sweep.py ``ParameterSweep``;
server.py ``ServerProcess``; serve_workload.py:87 ``explore_comb_workloads``; plot_pareto.py)."""
from __future__ import annotations

import argparse
import csv
import itertools
import json
import math
import os
import shlex
import signal
import subprocess
import sys
import time
import urllib.request
from pathlib import Path
from typing import Callable, Optional


# ---------------------------------------------------------------------------------------------------------------- parameter sets


def load_param_sets(spec: Optional[str]) -> list[dict]:
    """A file path or inline JSON. A list of objects is taken as is; an object of lists is expanded to its cartesian product;
    an object of objects names each set (the name is kept under ``_name``)."""
    if not spec:
        return [{}]
    text = Path(spec).read_text() if os.path.exists(spec) else spec
    data = json.loads(text)
    if isinstance(data, list):
        return [dict(d) for d in data] or [{}]
    if all(isinstance(v, dict) for v in data.values()) and data:
        return [dict(v, _name=k) for k, v in data.items()]
    keys = list(data)
    vals = [v if isinstance(v, list) else [v] for v in data.values()]
    return [dict(zip(keys, c)) for c in itertools.product(*vals)] or [{}]


def set_name(params: dict) -> str:
    if "_name" in params:
        return str(params["_name"])
    if not params:
        return "default"
    return "-".join(f"{k}={v}" for k, v in sorted(params.items())).replace("/", "_").replace(" ", "")


def apply_params(cmd: list[str], params: dict) -> list[str]:
    """Override or append ``--key value`` pairs; ``true`` becomes a bare flag, ``false``/``None`` removes the flag. Keys may be
    written with underscores or dashes; ``--key=value`` forms already in the command are replaced too."""
    out = list(cmd)
    for k, v in params.items():
        if k.startswith("_"):
            continue
        flag = "--" + k.replace("_", "-")
        alt = "--" + k
        i = 0
        while i < len(out):
            tok = out[i]
            if tok in (flag, alt):
                has_val = i + 1 < len(out) and not out[i + 1].startswith("--")
                del out[i:i + (2 if has_val else 1)]
                continue
            if tok.startswith(flag + "=") or tok.startswith(alt + "="):
                del out[i]
                continue
            i += 1
        if v is True:
            out.append(flag)
        elif v is False or v is None:
            continue
        elif isinstance(v, (dict, list)):
            out += [flag, json.dumps(v)]
        else:
            out += [flag, str(v)]
    return out


# ------------------------------------------------------------------------------------------------------------------------ server


class ServerProcess:
    """The server command in its own process group, so that stopping it also stops its engine-core and worker children."""

    def __init__(self, cmd: list[str], ready_timeout: float = 600.0, show_stdout: bool = False, after_bench_cmd: Optional[list[str]] = None):
        self.cmd, self.ready_timeout, self.show_stdout, self.after_bench_cmd = cmd, ready_timeout, show_stdout, after_bench_cmd
        self.proc: Optional[subprocess.Popen] = None

    def address(self) -> str:
        host, port = "127.0.0.1", "8000"
        for i, t in enumerate(self.cmd):
            if t == "--port" and i + 1 < len(self.cmd):
                port = self.cmd[i + 1]
            elif t.startswith("--port="):
                port = t.split("=", 1)[1]
            elif t == "--host" and i + 1 < len(self.cmd) and self.cmd[i + 1] not in ("0.0.0.0", "::"):
                host = self.cmd[i + 1]
        return f"http://{host}:{port}"

    def __enter__(self):
        out = None if self.show_stdout else subprocess.DEVNULL
        self.proc = subprocess.Popen(self.cmd, stdout=out, stderr=out, start_new_session=True)
        self.wait_ready()
        return self

    def wait_ready(self) -> None:
        t0 = time.monotonic()
        url = self.address() + "/health"
        while time.monotonic() - t0 < self.ready_timeout:
            if self.proc.poll() is not None:
                raise RuntimeError(f"server exited with code {self.proc.returncode} before it became ready")
            try:
                with urllib.request.urlopen(url, timeout=2) as r:
                    if r.status == 200:
                        return
            except Exception:
                time.sleep(1.0)
        raise TimeoutError(f"server not ready after {self.ready_timeout:.0f}s")

    def reset_caches(self) -> None:
        """Between runs the prefix cache is emptied so one run's prompts are not the next run's hits."""
        try:
            urllib.request.urlopen(urllib.request.Request(self.address() + "/reset_prefix_cache", method="POST"), timeout=10).close()
        except Exception:
            pass
        if self.after_bench_cmd:
            subprocess.run(self.after_bench_cmd, check=False)

    def __exit__(self, *exc):
        if self.proc and self.proc.poll() is None:
            # the exact process group this object created
            os.killpg(self.proc.pid, signal.SIGINT)
            try:
                self.proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                os.killpg(self.proc.pid, signal.SIGKILL)
                self.proc.wait()
        return False


# --------------------------------------------------------------------------------------------------------------------------- runs


def _run_client(cmd: list[str], result_path: Path, show_stdout: bool) -> dict:
    out = None if show_stdout else subprocess.DEVNULL
    subprocess.run(cmd + ["--save-result", str(result_path)], check=True, stdout=out, stderr=out)
    return json.loads(result_path.read_text())


def run_set(bench_cmd: list[str], serve_params: dict, bench_params: dict, out_dir: Path, num_runs: int, *, resume: bool = False,
            dry_run: bool = False, show_stdout: bool = False, run_client: Callable = _run_client, server: Optional[ServerProcess] = None,
            label: Optional[str] = None) -> list[dict]:
    """The ``num_runs`` repeats of one (server set, client set) pair. Each run's metrics land in
    ``<out>/<server set>/<client set>/run=<i>.json`` with both parameter sets merged in; with ``resume`` a file that exists is read
    back instead of run again."""
    d = out_dir / set_name(serve_params) / (label or set_name(bench_params))
    cmd = apply_params(bench_cmd, bench_params)
    rows = []
    for i in range(num_runs):
        path = d / f"run={i}.json"
        if dry_run:
            print("[dry-run] " + shlex.join(cmd + ["--save-result", str(path)]))
            continue
        if resume and path.exists():
            rows.append(json.loads(path.read_text()))
            continue
        d.mkdir(parents=True, exist_ok=True)
        res = run_client(cmd, path, show_stdout)
        row = {**{k: v for k, v in serve_params.items()}, **{k: v for k, v in bench_params.items()}, "run": i, **res}
        path.write_text(json.dumps(row))
        rows.append(row)
        if server is not None:
            server.reset_caches()
    return rows


def run_grid(serve_cmd: Optional[list[str]], bench_cmd: list[str], serve_sets: list[dict], bench_sets: list[dict], out_dir: Path,
             num_runs: int = 1, *, resume=False, dry_run=False, show_stdout=False, ready_timeout=600.0, after_bench_cmd=None,
             run_client: Callable = _run_client, server_factory: Callable = ServerProcess, per_set: Optional[Callable] = None) -> list[dict]:
    """Every server set × every client set. ``serve_cmd`` None means a server is already running. ``per_set(server, serve_params,
    bench_params)`` replaces the plain repeat loop (the workload explorer uses it)."""
    rows: list[dict] = []
    for sp in serve_sets:
        todo = bench_sets
        if resume and not dry_run and per_set is None:
            # a server is not started for a set whose runs are all on disk already
            done = all((out_dir / set_name(sp) / set_name(bp) / f"run={i}.json").exists() for bp in bench_sets for i in range(num_runs))
            if done:
                for bp in bench_sets:
                    rows += run_set(bench_cmd, sp, bp, out_dir, num_runs, resume=True)
                continue
        if dry_run or serve_cmd is None:
            if dry_run and serve_cmd is not None:
                print("[dry-run] " + shlex.join(apply_params(serve_cmd, sp)))
            for bp in todo:
                rows += (per_set(None, sp, bp) if per_set else run_set(bench_cmd, sp, bp, out_dir, num_runs, resume=resume, dry_run=dry_run,
                                                                       show_stdout=show_stdout, run_client=run_client))
            continue
        with server_factory(apply_params(serve_cmd, sp), ready_timeout, show_stdout, after_bench_cmd) as srv:
            for bp in todo:
                rows += (per_set(srv, sp, bp) if per_set else run_set(bench_cmd, sp, bp, out_dir, num_runs, resume=resume, show_stdout=show_stdout,
                                                                      run_client=run_client, server=srv))
    return rows


# --------------------------------------------------------------------------------------------------------------- workload explorer


def _operating_point(row: dict, var: str) -> float:
    """Where a finished run actually sat on the load axis: its achieved request rate, or (Little's law) rate × mean latency for
    the number of requests in flight."""
    rate = float(row["request_throughput"])
    return rate if var == "request_rate" else rate * float(row["mean_e2el_ms"]) / 1e3


def explore_workload(bench_cmd, serve_params, bench_params, out_dir, num_runs, var: str, iters: int, dataset_size: int, **kw) -> list[dict]:
    """Run the serial point (one request at a time) and the saturated point (everything at once), read the load each reached,
    then run ``iters − 2`` values spaced evenly between them."""
    if iters < 2:
        raise ValueError("workload iterations must be at least 2")
    if var not in ("request_rate", "max_concurrency"):
        raise ValueError(f"unknown workload variable {var!r}")
    dry = kw.get("dry_run", False)

    def at(value, extra=None):
        bp = dict(bench_params, **(extra or {var: value}))
        return run_set(bench_cmd, serve_params, bp, out_dir, num_runs, label=f"{set_name(bench_params)}/{var}={value}", **kw)

    serial = at(1, {"max_concurrency": 1})
    batch = at(dataset_size, {"max_concurrency": dataset_size})
    if dry or not serial or not batch:
        return serial + batch
    lo = math.ceil(sum(_operating_point(r, var) for r in serial) / len(serial))
    hi = math.floor(sum(_operating_point(r, var) for r in batch) / len(batch))
    mids: list[dict] = []
    if iters > 2 and hi > lo:
        step = (hi - lo) / (iters - 1)
        for v in sorted({round(lo + step * i) for i in range(1, iters - 1)} - {lo, hi}):
            if v > 0:
                mids += at(v)
    return serial + mids + batch


# ------------------------------------------------------------------------------------------------------------------------ summary


def pareto_front(rows: list[dict], x: str = "p50_tpot_ms", y: str = "output_throughput") -> list[dict]:
    """Rows that no other row beats on both axes (lower ``x``, higher ``y``), by rising ``x``."""
    pts = sorted((r for r in rows if r.get(x) is not None and r.get(y) is not None), key=lambda r: (r[x], -r[y]))
    front, best = [], -math.inf
    for r in pts:
        if r[y] > best:
            front.append(r)
            best = r[y]
    return front


def write_summary(rows: list[dict], out_dir: Path, x: str = "p50_tpot_ms", y: str = "output_throughput") -> dict:
    out_dir.mkdir(parents=True, exist_ok=True)
    keys: list[str] = []
    for r in rows:
        for k in r:
            if k not in keys:
                keys.append(k)
    with open(out_dir / "summary.csv", "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys)
        w.writeheader()
        for r in rows:
            w.writerow({k: (json.dumps(v) if isinstance(v, (dict, list)) else v) for k, v in r.items()})
    front = pareto_front(rows, x, y)
    summ = {"runs": len(rows), "pareto_x": x, "pareto_y": y, "pareto": front}
    (out_dir / "summary.json").write_text(json.dumps(summ, indent=1))
    return summ


# ---------------------------------------------------------------------------------------------------------------------------- CLI


def add_cli(sub) -> None:
    sw = sub.add_parser("sweep", help="parameter sweeps over `bench serve`")
    sw.add_argument("kind", choices=["serve", "workload", "summary"])
    sw.add_argument("--serve-cmd", default=None, help="server command line; omit to use a server that is already up")
    sw.add_argument("--bench-cmd", default=None, help="client command line; default: this package's `bench serve`")
    sw.add_argument("--after-bench-cmd", default=None)
    sw.add_argument("--serve-params", default=None, help="JSON (or a file of it): list of sets, or object of lists to cross")
    sw.add_argument("--bench-params", default=None)
    sw.add_argument("--output-dir", "-o", default="bench_results")
    sw.add_argument("--experiment-name", default=None)
    sw.add_argument("--num-runs", type=int, default=1)
    sw.add_argument("--server-ready-timeout", type=float, default=600.0)
    sw.add_argument("--show-stdout", action="store_true")
    sw.add_argument("--dry-run", action="store_true")
    sw.add_argument("--resume", action="store_true")
    sw.add_argument("--workload-var", default="request_rate", choices=["request_rate", "max_concurrency"])
    sw.add_argument("--workload-iters", type=int, default=8)
    sw.add_argument("--pareto-x", default="p50_tpot_ms")
    sw.add_argument("--pareto-y", default="output_throughput")


def _dataset_size(cmd: list[str], bp: dict, default: int = 64) -> int:
    if "num_prompts" in bp or "num-prompts" in bp:
        return int(bp.get("num_prompts", bp.get("num-prompts")))
    for i, t in enumerate(cmd):
        if t == "--num-prompts" and i + 1 < len(cmd):
            return int(cmd[i + 1])
        if t.startswith("--num-prompts="):
            return int(t.split("=", 1)[1])
    return default


def main(a: argparse.Namespace) -> None:
    out = Path(a.output_dir) / (a.experiment_name or "sweep")
    if a.kind == "summary":
        rows = [json.loads(p.read_text()) for p in sorted(out.rglob("run=*.json"))]
        print(json.dumps(write_summary(rows, out, a.pareto_x, a.pareto_y), indent=1))
        return
    serve_cmd = shlex.split(a.serve_cmd) if a.serve_cmd else None
    bench_cmd = shlex.split(a.bench_cmd) if a.bench_cmd else [sys.executable, "-m", "onecat_vllm.entrypoints.bench", "serve"]
    if serve_cmd and not a.bench_cmd:
        bench_cmd += ["--base-url", ServerProcess(serve_cmd).address()]  # the default client talks to the server this sweep starts
    serve_sets, bench_sets = load_param_sets(a.serve_params), load_param_sets(a.bench_params)
    kw = dict(resume=a.resume, dry_run=a.dry_run, show_stdout=a.show_stdout)
    per_set = None
    if a.kind == "workload":
        def per_set(srv, sp, bp):
            return explore_workload(bench_cmd, sp, bp, out, a.num_runs, a.workload_var, a.workload_iters, _dataset_size(bench_cmd, bp), server=srv, **kw)
    rows = run_grid(serve_cmd, bench_cmd, serve_sets, bench_sets, out, a.num_runs, ready_timeout=a.server_ready_timeout,
                    after_bench_cmd=shlex.split(a.after_bench_cmd) if a.after_bench_cmd else None, per_set=per_set, **kw)
    if not a.dry_run:
        print(json.dumps(write_summary(rows, out, a.pareto_x, a.pareto_y), indent=1))
