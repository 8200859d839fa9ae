#!/usr/bin/env python
"""Headline benchmark: output tokens/s of the dense 27B-class AWQ W4A16 decoder (64 layers, hidden 5120, 40 q / 8 kv heads
of 128, SwiGLU 17408, vocab 151936) serving 1024-in / 256-out requests at concurrency 64, tensor-parallel over N GPUs.

A "step" is one engine iteration (schedule → forward → sample) of the continuous-batching steady state of that
workload: 64 running requests whose progress is spread evenly over their 256 output tokens, a finished request being
replaced at once by a fresh 1024-token prompt (so one step in four also carries a 1024-token prefill chunk).
Weights are random (AWQ codes uniform, fp16 scales |N(0, 0.01)|), prompts are random token ids.

``value`` is device-timed (CUDA events around each step's H2D copy, forward and sampling; max over ranks); ``e2e`` is
the same steps timed by the wall clock through ``LLMEngine.add_request/step`` including scheduling, the pinned
host→device input copy and the device→host read of the sampled ids.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG_27B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=5120, intermediate_size=17408, num_hidden_layers=64,
               num_attention_heads=40, num_key_value_heads=8, head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=4096, tie_word_embeddings=False,
               quantization_config=dict(quant_method="awq", bits=4, group_size=128, zero_point=True))
# The other configurations of the benchmark plan (selected with --config; the default stays the dense AWQ model above).
_GDN = dict(linear_num_key_heads=16, linear_num_value_heads=48, linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4,
            full_attention_interval=4, attn_output_gate=True, partial_rotary_factor=0.25)
CFG_HYBRID_27B = dict(architectures=["Qwen3_5ForCausalLM"], hidden_size=5120, intermediate_size=17408, num_hidden_layers=64,
                      num_attention_heads=24, num_key_value_heads=4, head_dim=256, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                      max_position_embeddings=262144, tie_word_embeddings=False, **_GDN)
CFG_MOE_35B = dict(architectures=["Qwen3_5MoeForCausalLM"], hidden_size=2048, intermediate_size=5632, num_hidden_layers=40,
                   num_attention_heads=16, num_key_value_heads=2, head_dim=256, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                   max_position_embeddings=8192, tie_word_embeddings=False, num_experts=256, num_experts_per_tok=8, moe_intermediate_size=512,
                   shared_expert_intermediate_size=512, norm_topk_prob=True,
                   quantization_config=dict(quant_method="fp8", weight_block_size=[128, 128], modules_to_not_convert=["self_attn", "linear_attn", "shared_expert", "lm_head"]),
                   **dict(_GDN, linear_num_value_heads=32))
CFG_DSV3 = dict(architectures=["DeepseekV3ForCausalLM"], hidden_size=7168, intermediate_size=18432, num_hidden_layers=61, num_attention_heads=128,
                num_key_value_heads=128, vocab_size=129280, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=8192,
                tie_word_embeddings=False, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                n_routed_experts=256, n_shared_experts=1, num_experts_per_tok=8, moe_intermediate_size=2048, n_group=8, topk_group=4,
                routed_scaling_factor=2.5, norm_topk_prob=True, first_k_dense_replace=3, scoring_func="sigmoid",
                quantization_config=dict(quant_method="fp8", weight_block_size=[128, 128], expert_method="mxfp4"))
CONFIGS = {
    # name: (hf config, description, concurrency, input len, output len, speculative config, dtype string)
    "dense27b": (CFG_27B, "dense 27B-class AWQ W4A16 (64L, h5120, 40q/8kv x128, ffn 17408, vocab 151936)", 64, 1024, 256, None,
                 "bf16 activations/KV, int4 AWQ weights (W4A16)"),
    "hybrid27b": (CFG_HYBRID_27B, "hybrid 27B-class bf16 (64L, 3:1 Gated-DeltaNet : gated attention 24q/4kv x256) + MTP(3), Bernoulli(0.7) acceptance", 8,
                  131072, 512, dict(method="mtp", num_speculative_tokens=3, synthetic_acceptance_rate=0.7), "bf16"),
    "moe35b": (CFG_MOE_35B, "MoE 35B-A3B-class (40L, h2048, 3:1 GDN : attention, 256 experts top-8 + shared, FP8 128x128 experts)", 256, 2048, 512, None,
               "bf16 activations/KV, FP8 e4m3 block-scaled expert weights (weight-only)"),
    "dsv3": (CFG_DSV3, "DeepSeek-V3-class MLA + MoE (h7168, 128 heads, 256 experts top-8 grouped sigmoid, MXFP4 experts, FP8 dense)", 128, 4096, 1024, None,
             "bf16 activations/KV, MXFP4 expert weights, FP8 block-scaled dense weights (weight-only)"),
}
QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def reference_arm(args) -> None:
    """``--impl reference``: drive the reference's own unmodified Python tree (``baseline/_ref/vllm``, laid out by
    ``baseline/prepare_reference.py`` beside the compiled extension modules of the vLLM wheel in the image) through its ``LLM.generate``
    on the same model and workload, in a subprocess that never imports this repository's package. Whatever stops it (the tree is
    missing, an import fails, a kernel is absent from the stock binaries, the run raises) is reported at run time as ``unavailable``
    with the exception text. Under ``torch.distributed.run`` only rank 0 runs it (the reference spawns its own tensor-parallel
    workers); the other ranks leave at once."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    label = "reference-python+stock-0.22-binaries"
    base_cfg, desc, c0, in0, out0, _spec, dtype_desc = CONFIGS["dense27b"]
    C, IN, OUT = args.concurrency or c0, args.input_len or in0, args.output_len or out0
    if not os.path.isdir(os.path.join(ref_root, "vllm")) and os.path.exists(os.path.join(ref_root, "WITHDRAWN.txt")):
        print(json.dumps({"impl": "reference", "unavailable": open(os.path.join(ref_root, "WITHDRAWN.txt")).read().strip()}))
        return
    if not os.path.isdir(os.path.join(ref_root, "vllm")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/vllm is missing: run python baseline/prepare_reference.py (pip install of the "
                          "reference fails offline: setup.py imports setuptools_rust, CMake fetches CUTLASS/FlashMLA/DeepGEMM)"}))
        return
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "GROUP_RANK",
                                                             "ROLE_RANK", "LOCAL_WORLD_SIZE", "ROLE_WORLD_SIZE", "TORCHELASTIC_RUN_ID",
                                                             "TORCHELASTIC_RESTART_COUNT", "TORCHELASTIC_MAX_RESTARTS", "OMP_NUM_THREADS")}
    env["PYTHONPATH"] = ref_root
    env.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "run_reference.py"), "--gpus", str(args.gpus), "--concurrency", str(C),
           "--input-len", str(IN), "--output-len", str(OUT), "--cfg", json.dumps(base_cfg)]
    sampler = ClockSampler(0)
    try:
        r = subprocess.run(cmd, env=env, cwd=tempfile.gettempdir(), capture_output=True, text=True, timeout=1500)
        line = next((l for l in reversed(r.stdout.strip().splitlines()) if l.startswith("{")), None)
        res = json.loads(line) if line else {"ok": False, "error": f"no result line (exit {r.returncode}): {r.stderr.strip()[-400:]}"}
    except subprocess.TimeoutExpired:
        res = {"ok": False, "error": "the reference run did not finish within 1500 s"}
    clocks = sampler.stop()
    if not res.get("ok"):
        print(json.dumps({"impl": "reference", "unavailable": f"{label}: {res.get('error')}", "where": res.get("where")}))
        return
    v = res["tokens_per_s"]
    print(json.dumps({
        "impl": "reference", "impl_detail": label, "metric": "output tokens/s (box, max over ranks)", "value": v, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": dtype_desc, "data": "synthetic: random token ids, dummy-loader weights of the named architecture",
        "same_config": True,
        "config": {"model": desc, "name": "dense27b", "global_batch": C, "seq_len": IN + OUT, "parallelism": f"tp{args.gpus}",
                   "workload": f"{res['requests']} requests, {IN} in / {OUT} out, at most {C} running; wall clock of LLM.generate (ramp-up and tail included)",
                   "layers": base_cfg["num_hidden_layers"], "output_tokens": res["output_tokens"], "vllm_file": res.get("vllm_file")},
        "clocks": clocks,
        "e2e": {"value": v, "unit": "tokens/s", "note": "LLM.generate takes host token ids and returns host token ids: the wall-clock number is end to end"},
        "timing": "wall clock around LLM.generate with torch.cuda.synchronize on both sides (the reference exposes no per-step device timer)"}))


class ClockSampler:
    def __init__(self, index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(index)],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, pw, reasons = [], [], [], set()
        for line in self.f:
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2])); pw.append(float(c[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


def stock_vllm_arm(args) -> None:
    """Context only, never the reference arm: the same dense AWQ workload through the stock ``vllm`` wheel of the image (library code:
    its own kernels and scheduler), random weights via ``load_format="dummy"``. 256 requests of 1024 random tokens in / 256 out with
    at most 64 running; the number is output tokens over the wall time of ``LLM.generate``."""
    import json as _json
    try:
        import torch
        from vllm import LLM as VLLM
        from vllm import SamplingParams as VSP
        d = tempfile.mkdtemp(prefix="onecat_stock_")
        cfg = dict(CFG_27B, model_type="qwen3", hidden_act="silu", torch_dtype="bfloat16", attention_bias=False, use_cache=True,
                   initializer_range=0.02, bos_token_id=1, eos_token_id=2)
        cfg["quantization_config"] = dict(cfg["quantization_config"], version="gemm")
        with open(os.path.join(d, "config.json"), "w") as f:
            _json.dump(cfg, f)
        C, IN, OUT = args.concurrency or 64, args.input_len or 1024, args.output_len or 256
        llm = VLLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", max_model_len=IN + OUT + 16, max_num_seqs=C,
                   max_num_batched_tokens=8192, tensor_parallel_size=args.gpus, gpu_memory_utilization=0.85, enable_prefix_caching=False, seed=0)
        g = torch.Generator().manual_seed(0)
        n_req = 4 * C
        prompts = [{"prompt_token_ids": torch.randint(0, cfg["vocab_size"], (IN,), generator=g).tolist()} for _ in range(n_req)]
        sp = VSP(temperature=0.0, max_tokens=OUT, ignore_eos=True, detokenize=False)
        llm.generate(prompts[:C], VSP(temperature=0.0, max_tokens=8, ignore_eos=True, detokenize=False))  # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        toks = sum(len(o.outputs[0].token_ids) for o in outs)
        import vllm
        print(_json.dumps({"impl": "stock-vllm", "vllm_version": vllm.__version__, "metric": "output tokens/s (wall clock of LLM.generate)",
                           "value": toks / wall, "unit": "tokens/s", "n_gpus": args.gpus, "wall_s": wall, "output_tokens": toks,
                           "config": {"model": CONFIGS["dense27b"][1], "workload": f"{n_req} requests, {IN} in / {OUT} out, at most {C} running"}}))
    except Exception as e:  # context only: never fail the caller
        print(_json.dumps({"impl": "stock-vllm", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}))


def ours_offline_arm(args) -> None:
    """The workload of ``stock_vllm_arm`` measured the same way through this engine's ``LLM.generate`` (wall clock, ramp-up and tail
    included), for a like-for-like context comparison on one GPU."""
    import json as _json
    import torch
    from onecat_vllm import LLM, SamplingParams
    cfg = dict(CFG_27B)
    C, IN, OUT = args.concurrency or 64, args.input_len or 1024, args.output_len or 256
    llm = LLM(hf_config=cfg, dtype="bfloat16", device="cuda", max_model_len=IN + OUT + 16, max_num_seqs=C, max_num_batched_tokens=8192,
              enable_prefix_caching=False, gpu_memory_utilization=0.85, kv_cache_memory_bytes=_kv_bytes(cfg, C, IN + OUT + 32, 1))
    g = torch.Generator().manual_seed(0)
    n_req = 4 * C
    prompts = [{"prompt_token_ids": torch.randint(0, cfg["vocab_size"], (IN,), generator=g).tolist()} for _ in range(n_req)]
    llm.generate(prompts[:C], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, detokenize=False))  # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=OUT, ignore_eos=True, detokenize=False))
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    toks = sum(len(o.outputs[0].token_ids) for o in outs)
    print(_json.dumps({"impl": "ours-offline", "metric": "output tokens/s (wall clock of LLM.generate)", "value": toks / wall, "unit": "tokens/s",
                       "n_gpus": 1, "wall_s": wall, "output_tokens": toks,
                       "config": {"model": CONFIGS["dense27b"][1], "workload": f"{n_req} requests, {IN} in / {OUT} out, at most {C} running"}}))


def _kv_bytes(cfg: dict, C: int, seq: int, gpus: int) -> int:
    """KV-cache bytes per GPU for C sequences of `seq` tokens (bf16): attention layers only; MLA keeps one 576-wide latent."""
    L = cfg["num_hidden_layers"]
    if cfg.get("kv_lora_rank"):
        per_tok = L * (cfg["kv_lora_rank"] + cfg["qk_rope_head_dim"]) * 2
    else:
        attn_layers = L // cfg["full_attention_interval"] if cfg.get("full_attention_interval") else L
        kvh = max(cfg["num_key_value_heads"] // gpus, 1)
        per_tok = attn_layers * 2 * kvh * cfg["head_dim"] * 2
    state = 0
    if cfg.get("full_attention_interval"):  # Gated-DeltaNet layers keep a recurrent state and a conv window per sequence
        hv, hk = cfg["linear_num_value_heads"] // gpus, cfg["linear_num_key_heads"] // gpus
        k, v = cfg["linear_key_head_dim"], cfg["linear_value_head_dim"]
        per_seq = hv * k * v * 4 + (2 * hk * k + hv * v) * (cfg["linear_conv_kernel_dim"] - 1) * 2
        state = (L - L // cfg["full_attention_interval"]) * per_seq * (C + 2)
    return int((C + 2) * seq * per_tok * 1.02 + state * 1.05)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="dense27b", choices=sorted(CONFIGS), help="benchmark configuration; the default is the headline one")
    ap.add_argument("--concurrency", type=int, default=0, help="0 = the configuration's own value")
    ap.add_argument("--input-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: a value other than 0 makes the run invalid as a headline number")
    ap.add_argument("--tp-comm", default=os.environ.get("ONECAT_TP_COMM", "fused"))
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--no-full", action="store_true", help="skip the full-workload pass (4 x concurrency requests, ramp-up and tail) after the timed steps")
    ap.add_argument("--no-async", action="store_true", help="plain schedule-run-update order instead of async scheduling (one step kept in flight)")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.impl == "stock-vllm":
        stock_vllm_arm(args)
        return
    if args.impl == "ours-offline":
        ours_offline_arm(args)
        return
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
        raise SystemExit(f"WORLD_SIZE={world} but --gpus={args.gpus}")
    if args.warmup < 3:
        args.warmup = 3
    torch.cuda.set_device(local)
    from onecat_vllm.config import EngineArgs
    from onecat_vllm.engine.llm_engine import LLMEngine
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.sampling_params import RequestOutputKind, SamplingParams

    base_cfg, desc, c0, in0, out0, spec, dtype_desc = CONFIGS[args.config]
    cfg = dict(base_cfg)
    if args.config == "dsv3" and not args.layers and args.gpus < 8:
        cfg["num_hidden_layers"] = max(4, 61 * args.gpus // 8)  # the plan's 1/2/4-GPU points: same layer shapes, 61*n/8 layers
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    C, IN, OUT = args.concurrency or c0, args.input_len or in0, args.output_len or out0
    ea = EngineArgs(hf_config=cfg, dtype="bfloat16", device="cuda", max_model_len=IN + OUT + 16, max_num_seqs=C, max_num_batched_tokens=8192,
                    tensor_parallel_size=args.gpus, distributed_executor_backend="external_launcher" if args.gpus > 1 else None,
                    tp_comm=args.tp_comm, enable_prefix_caching=False, gpu_memory_utilization=0.85, disable_log_stats=False,
                    enforce_eager=args.eager, speculative_config=spec, async_scheduling=not args.no_async,
                    enable_expert_parallel=args.config in ("moe35b", "dsv3") and args.gpus > 1,
                    kv_cache_memory_bytes=_kv_bytes(cfg, C, IN + OUT + 32, args.gpus))
    eng = LLMEngine.from_engine_args(ea)
    runner = eng.engine_core.core.executor.worker.runner
    g = torch.Generator().manual_seed(0)
    counter = [0]
    timing = [False]
    arrivals: dict = {}

    def add(prompt_len: int, max_tokens: int) -> None:
        ids = torch.randint(0, cfg["vocab_size"], (prompt_len,), generator=g).tolist()
        sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True, output_kind=RequestOutputKind.DELTA, detokenize=False)
        eng.add_request(f"r{counter[0]}", ids, sp)
        if timing[0]:
            arrivals[f"r{counter[0]}"] = time.perf_counter()
        counter[0] += 1

    # steady state: request i has already produced i*OUT/C of its OUT tokens (same KV footprint as a prompt that long)
    stride = max(OUT // C, 1)
    for i in range(C):
        done = min(i * stride, OUT - 1)
        add(IN + done, OUT - done)

    def one_step():
        outs = eng.step()
        new = fin = 0
        for o in outs:
            new += sum(len(c.token_ids) for c in o.outputs)
            if o.finished:
                fin += 1
        for _ in range(fin):
            add(IN, OUT)  # closed loop at fixed concurrency
        st = getattr(eng, "last_scheduler_stats", None)
        return new, (st.step_device_ms if st is not None else 0.0), (st.num_scheduled_tokens if st else 0), outs

    # untimed: initial prefill of the staggered population, then W warm-up steps
    initial = {f"r{i}" for i in range(C)}
    reqs = eng.engine_core.core.scheduler.requests
    for _ in range(100000):  # bounded: the closed loop keeps adding requests, only the initial population has to be prefilled
        if not any(rid in reqs and reqs[rid].num_computed_tokens < reqs[rid].num_prompt_tokens for rid in initial):
            break
        one_step()
    core = eng.engine_core
    for i in range(args.warmup):
        if i == args.warmup - 1:
            core.call_utility("set_overlap", False)  # the last warm-up step leaves nothing in flight: the timed steps start from a drained engine
        one_step()
    core.call_utility("set_overlap", True)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    K.reset_launches()
    runner.graph_launches = 0
    sampler = ClockSampler(local)
    time.sleep(0.25)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    timing[0] = True
    tokens, dev_ms, sched_tokens, ttfts, step_ms = 0, 0.0, 0, [], []
    dev_steps: list = []
    h2d = d2h = 0
    for i in range(args.steps):
        if i == args.steps - 1:
            core.call_utility("set_overlap", False)  # the K-th step launches nothing behind itself: exactly K steps run inside the timed region
        ts = time.perf_counter()
        n, ms, st_tok, outs = one_step()
        step_ms.append((time.perf_counter() - ts) * 1e3)
        dev_steps.append(ms)
        tokens += n
        dev_ms += ms
        sched_tokens += st_tok
        h2d += runner.h2d_bytes
        d2h += runner.d2h_bytes
        now = time.perf_counter()
        for o in outs:
            if o.request_id in arrivals and o.outputs and o.outputs[0].token_ids:
                ttfts.append((now - arrivals.pop(o.request_id)) * 1e3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    wall = time.perf_counter() - t0
    core.call_utility("set_overlap", True)
    clocks = sampler.stop()
    if os.environ.get("ONECAT_BENCH_DUMP") and rank == 0:   # per-step wall and device times, for looking at where host time goes
        with open(os.environ["ONECAT_BENCH_DUMP"], "w") as f:
            json.dump({"wall_ms": step_ms, "device_ms": dev_steps}, f)
    launches = K.launches() + getattr(runner, "graph_launches", 0)
    status = K.check_status()
    # ---- the whole workload the configuration names (4 x concurrency requests from an empty engine, ramp-up and tail included),
    # through the same public add_request / step calls, by the wall clock; reported beside the steady-state figure
    full = None
    if not args.no_full and args.config == "dense27b":
        timing[0] = False
        eng.abort_request([rid for rid in list(reqs)])
        while eng.has_unfinished_requests():
            eng.step()
        n_req, done_tokens, ttft_full, first_seen = 4 * C, 0, [], {}
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        tf0 = time.perf_counter()
        base = counter[0]
        for _ in range(n_req):
            add(IN, OUT)
        while eng.has_unfinished_requests():
            for o in eng.step():
                n_new = sum(len(c.token_ids) for c in o.outputs)
                done_tokens += n_new
                if n_new and o.request_id not in first_seen:
                    first_seen[o.request_id] = time.perf_counter() - tf0
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        wall_full = time.perf_counter() - tf0
        tw = torch.tensor([wall_full], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        full = {"value": done_tokens / float(tw[0]), "unit": "tokens/s", "wall_s": float(tw[0]), "requests": n_req, "output_tokens": done_tokens,
                "note": f"{n_req} requests of {IN} in / {OUT} out submitted at once to an empty engine, at most {C} running; wall clock, max over ranks"}
        status |= K.check_status()
    t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms = float(t[0]), float(t[1])
    if rank == 0:
        decode_ms = sorted(step_ms)[len(step_ms) // 2]
        res = {
            "metric": "output tokens/s (box, max over ranks)", "value": tokens / (dev_ms / 1e3) if dev_ms > 0 else None, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype_desc,
            "data": "synthetic: random token ids, random-init weights of the named architecture",
            "config": {"model": desc, "name": args.config,
                       "global_batch": C, "seq_len": IN + OUT, "parallelism": f"tp{args.gpus}", "workload": f"{IN} in / {OUT} out, concurrency {C}, closed loop steady state",
                       "layers": cfg["num_hidden_layers"], "l2": "inputs larger than L2 (each step streams >10 GB of weights and KV)",
                       "tp_comm": args.tp_comm if args.gpus > 1 else "none", "cuda_graphs": not args.eager,
                       "scheduled_tokens_per_step": sched_tokens / args.steps, "output_tokens": tokens},
            "clocks": clocks,
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d // args.steps, "d2h_bytes_per_step": d2h // args.steps,
                    "ms_per_step": wall_ms / args.steps, "p50_tpot_ms": decode_ms,
                    "p50_ttft_ms": (sorted(ttfts)[len(ttfts) // 2] if ttfts else None)},
            "e2e_full_workload": full,
            "gpu_launches": launches, "device_status": status,
            "torch_standins": sorted(K.TORCH_STANDINS),
        }
        if args.layers:
            res["invalid"] = "reduced layer count (debug run)"
        print(json.dumps(res))
    sys.stdout.flush()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    eng.shutdown()


if __name__ == "__main__":
    main()
