"""Benchmark harness: ``bench throughput`` (offline), ``bench latency`` (offline, fixed batch), ``bench serve`` (HTTP client with
TTFT / TPOT / ITL / E2EL percentiles and goodput), over random-token datasets
(reference: vllm/benchmarks/throughput.py, latency.py, serve.py:407 ``calculate_metrics`` with TPOT = (latency − ttft)/(out_len − 1))."""
from __future__ import annotations

import argparse
import asyncio
import json
import random
import statistics
import time
from dataclasses import dataclass, field
from typing import Optional


def _pct(xs: list, p: float) -> Optional[float]:
    if not xs:
        return None
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(round(p / 100.0 * (len(xs) - 1))))]


@dataclass
class RequestRecord:
    prompt_len: int
    output_len: int = 0
    ttft: Optional[float] = None
    latency: float = 0.0
    itl: list = field(default_factory=list)
    ok: bool = True


def calculate_metrics(records: list[RequestRecord], duration: float, goodput_slo: Optional[dict] = None) -> dict:
    good = [r for r in records if r.ok and r.output_len > 0]
    tpots = [(r.latency - r.ttft) / (r.output_len - 1) for r in good if r.output_len > 1 and r.ttft is not None]
    ttfts = [r.ttft for r in good if r.ttft is not None]
    itls = [x for r in good for x in r.itl]
    out = {"completed": len(good), "failed": len(records) - len(good), "duration_s": duration,
           "total_input_tokens": sum(r.prompt_len for r in good), "total_output_tokens": sum(r.output_len for r in good),
           "request_throughput": len(good) / duration if duration else 0.0,
           "output_throughput": sum(r.output_len for r in good) / duration if duration else 0.0,
           "total_token_throughput": sum(r.prompt_len + r.output_len for r in good) / duration if duration else 0.0}
    for name, xs in (("ttft", ttfts), ("tpot", tpots), ("itl", itls), ("e2el", [r.latency for r in good])):
        out[f"mean_{name}_ms"] = 1e3 * statistics.fmean(xs) if xs else None
        for p in (50, 90, 99):
            v = _pct(xs, p)
            out[f"p{p}_{name}_ms"] = 1e3 * v if v is not None else None
    if goodput_slo:
        ok = 0
        for r in good:
            tp = (r.latency - r.ttft) / (r.output_len - 1) if r.output_len > 1 and r.ttft is not None else 0.0
            if (r.ttft or 0) * 1e3 <= goodput_slo.get("ttft", 1e18) and tp * 1e3 <= goodput_slo.get("tpot", 1e18) and \
                    r.latency * 1e3 <= goodput_slo.get("e2el", 1e18):
                ok += 1
        out["request_goodput"] = ok / duration if duration else 0.0
    return out


def random_prompts(n: int, input_len: int, vocab: int, seed: int = 0, range_ratio: float = 0.0) -> list[list[int]]:
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        l = input_len if range_ratio <= 0 else rng.randint(int(input_len * (1 - range_ratio)), int(input_len * (1 + range_ratio)))
        out.append([rng.randrange(vocab) for _ in range(max(l, 1))])
    return out


def _engine_args(a):
    from onecat_vllm.config import EngineArgs
    return EngineArgs.from_cli_args(a)


def bench_throughput(a) -> dict:
    from onecat_vllm import LLM, SamplingParams
    ea = _engine_args(a)
    llm = LLM(**ea.__dict__)
    vocab = llm.llm_engine.cfg.model_config.vocab_size
    from onecat_vllm.entrypoints.bench_datasets import build_dataset
    rows = build_dataset(a, vocab, llm.get_tokenizer() if a.dataset_name not in ("random", "prefix_repetition") else None)
    prompts = [r.prompt for r in rows]
    sps = [SamplingParams(temperature=0.0, max_tokens=r.expected_output_len, ignore_eos=True, detokenize=False) for r in rows]
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sps)
    dt = time.perf_counter() - t0
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    n_in = sum(len(o.prompt_token_ids or []) for o in outs) or sum(r.prompt_len for r in rows)
    llm.shutdown()
    return {"elapsed_s": dt, "requests_per_s": len(outs) / dt, "output_tokens_per_s": n_out / dt,
            "total_tokens_per_s": (n_out + n_in) / dt, "dataset": a.dataset_name}


def bench_latency(a) -> dict:
    from onecat_vllm import LLM, SamplingParams
    ea = _engine_args(a)
    llm = LLM(**ea.__dict__)
    vocab = llm.llm_engine.cfg.model_config.vocab_size
    sp = SamplingParams(temperature=0.0, max_tokens=a.output_len, ignore_eos=True, detokenize=False)
    lats = []
    for it in range(a.num_iters_warmup + a.num_iters):
        prompts = random_prompts(a.batch_size, a.input_len, vocab, a.seed + it)
        t0 = time.perf_counter()
        llm.generate(prompts, sp)
        if it >= a.num_iters_warmup:
            lats.append(time.perf_counter() - t0)
    llm.shutdown()
    return {"avg_latency_s": statistics.fmean(lats), "p50_s": _pct(lats, 50), "p90_s": _pct(lats, 90), "p99_s": _pct(lats, 99)}


async def _serve_one(client, url, model, prompt, output_len, rec: RequestRecord, api_key):
    body = {"model": model, "prompt": prompt, "max_tokens": output_len, "temperature": 0.0, "ignore_eos": True, "stream": True}
    headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
    t0 = time.perf_counter()
    last = t0
    try:
        async with client.stream("POST", url + "/v1/completions", json=body, headers=headers) as resp:
            if resp.status_code != 200:
                rec.ok = False
                return
            async for line in resp.aiter_lines():
                if not line.startswith("data: ") or line == "data: [DONE]":
                    continue
                d = json.loads(line[6:])
                if not d.get("choices"):
                    continue
                now = time.perf_counter()
                if rec.ttft is None:
                    rec.ttft = now - t0
                else:
                    rec.itl.append(now - last)
                last = now
                rec.output_len += 1
        rec.latency = last - t0
    except Exception:
        rec.ok = False


async def _bench_serve_async(a) -> dict:
    import httpx
    async with httpx.AsyncClient(timeout=None) as client:
        model = a.model_name or (await client.get(a.base_url + "/v1/models")).json()["data"][0]["id"]
        vocab = a.vocab_size
        from onecat_vllm.entrypoints.bench_datasets import build_dataset
        rows = build_dataset(a, vocab)
        prompts = [r.prompt for r in rows]
        recs = [RequestRecord(r.prompt_len) for r in rows]
        sem = asyncio.Semaphore(a.max_concurrency) if a.max_concurrency else None
        rng = random.Random(a.seed)

        async def run(p, r, n_out):
            if sem is None:
                await _serve_one(client, a.base_url, model, p, n_out, r, a.api_key)
            else:
                async with sem:
                    await _serve_one(client, a.base_url, model, p, n_out, r, a.api_key)

        t0 = time.perf_counter()
        tasks = []
        replay = getattr(a, "replay_arrivals", False)
        for row, r in zip(rows, recs):
            if replay and row.arrival_s is not None:
                # a trace row is sent at its logged offset from the start of the run
                await asyncio.sleep(max(row.arrival_s - (time.perf_counter() - t0), 0.0))
            tasks.append(asyncio.create_task(run(row.prompt, r, row.expected_output_len)))
            if not replay and a.request_rate and a.request_rate != float("inf"):
                await asyncio.sleep(rng.expovariate(a.request_rate))
        await asyncio.gather(*tasks)
        dur = time.perf_counter() - t0
    slo = dict(kv.split(":") for kv in a.goodput) if a.goodput else None
    if slo:
        slo = {k: float(v) for k, v in slo.items()}
    return calculate_metrics(recs, dur, slo)


def bench_startup(a) -> dict:
    """Cold-start cost: engine construction (weights, KV cache, warm-up, graph capture) and the first generated token
    (reference: vllm/benchmarks/startup.py)."""
    from onecat_vllm import LLM, SamplingParams
    ea = _engine_args(a)
    t0 = time.perf_counter()
    llm = LLM(**ea.__dict__)
    t1 = time.perf_counter()
    vocab = llm.llm_engine.cfg.model_config.vocab_size
    llm.generate(random_prompts(1, a.input_len, vocab, a.seed), SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, detokenize=False))
    t2 = time.perf_counter()
    llm.shutdown()
    return {"engine_init_s": t1 - t0, "first_token_s": t2 - t1, "total_s": t2 - t0}


def main(argv=None) -> None:
    p = argparse.ArgumentParser("bench")
    sub = p.add_subparsers(dest="mode", required=True)
    from onecat_vllm.config import EngineArgs
    from onecat_vllm.entrypoints.bench_datasets import add_dataset_args
    for name in ("throughput", "latency", "startup"):
        sp = sub.add_parser(name)
        EngineArgs.add_cli_args(sp)
        sp.add_argument("--input-len", type=int, default=1024)
        sp.add_argument("--output-len", type=int, default=128)
        sp.add_argument("--num-prompts", type=int, default=64)
        sp.add_argument("--batch-size", type=int, default=8)
        sp.add_argument("--num-iters", type=int, default=5)
        sp.add_argument("--num-iters-warmup", type=int, default=2)
        add_dataset_args(sp)
    sv = sub.add_parser("serve")
    sv.add_argument("--base-url", default="http://127.0.0.1:8000")
    sv.add_argument("--model-name", default=None)
    sv.add_argument("--api-key", default=None)
    sv.add_argument("--vocab-size", type=int, default=32000)
    sv.add_argument("--input-len", type=int, default=1024)
    sv.add_argument("--output-len", type=int, default=128)
    sv.add_argument("--num-prompts", type=int, default=64)
    sv.add_argument("--max-concurrency", type=int, default=0)
    sv.add_argument("--request-rate", type=float, default=float("inf"))
    sv.add_argument("--goodput", nargs="*", default=None, help="SLOs as ttft:MS tpot:MS e2el:MS")
    sv.add_argument("--seed", type=int, default=0)
    sv.add_argument("--save-result", default=None, help="also write the metrics to this JSON file")
    add_dataset_args(sv)
    from onecat_vllm.entrypoints import bench_sweep
    bench_sweep.add_cli(sub)
    a = p.parse_args(argv)
    if a.mode == "sweep":
        return bench_sweep.main(a)
    if a.mode == "throughput":
        res = bench_throughput(a)
    elif a.mode == "latency":
        res = bench_latency(a)
    elif a.mode == "startup":
        res = bench_startup(a)
    else:
        res = asyncio.run(_bench_serve_async(a))
    if getattr(a, "save_result", None):
        with open(a.save_result, "w") as f:
            json.dump(res, f)
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
