"""Reference arm of the benchmark: the dense 27B-class AWQ workload through the reference's own ``vllm.LLM.generate``.

Runs in a subprocess of ``bench.py --impl reference`` with ``PYTHONPATH`` pointing at ``baseline/_ref`` (see
``prepare_reference.py``), so that ``import vllm`` resolves to the reference's unmodified Python tree; nothing of this repository's
engine, models or kernels is imported here. Random weights come from the reference's dummy loader, prompts are random token ids.
Two measurements, both in output tokens per second over the whole job:
* ``value``: the full workload (4 x concurrency requests, 1024 in / 256 out, at most ``concurrency`` running) over the wall time of
  ``LLM.generate`` bracketed by device synchronisation;
* the prompts live in host memory and the sampled ids are read back by the engine every step, so the same number is the end-to-end one.
Prints ONE JSON line; on any failure the line carries ``unavailable`` with the exception text.
"""
import argparse
import json
import os
import sys
import tempfile
import time
import traceback


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--cfg", required=True, help="JSON of the HF config of the benchmark model")
    a = ap.parse_args()
    try:
        import torch
        import vllm
        here = os.path.realpath(os.path.dirname(vllm.__file__))
        if "baseline" not in here or "_ref" not in here:
            raise RuntimeError(f"import vllm resolved to {here}, not to the reference tree under baseline/_ref")
        from vllm import LLM, SamplingParams
        cfg = json.loads(a.cfg)
        cfg.update(model_type="qwen3", hidden_act="silu", torch_dtype="bfloat16", attention_bias=False, use_cache=True, initializer_range=0.02,
                   bos_token_id=1, eos_token_id=2)
        cfg["quantization_config"] = dict(cfg["quantization_config"], version="gemm")
        d = tempfile.mkdtemp(prefix="onecat_ref_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        C, IN, OUT = a.concurrency, a.input_len, a.output_len
        llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", max_model_len=IN + OUT + 16, max_num_seqs=C,
                  max_num_batched_tokens=8192, tensor_parallel_size=a.gpus, gpu_memory_utilization=0.85, enable_prefix_caching=False, seed=0)
        g = torch.Generator().manual_seed(0)
        n_req = a.requests or 4 * C
        prompts = [{"prompt_token_ids": torch.randint(0, cfg["vocab_size"], (IN,), generator=g).tolist()} for _ in range(n_req)]
        llm.generate(prompts[:C], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True, detokenize=False))  # warm-up
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=OUT, ignore_eos=True, detokenize=False))
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        toks = sum(len(o.outputs[0].token_ids) for o in outs)
        print(json.dumps({"ok": True, "tokens_per_s": toks / wall, "wall_s": wall, "output_tokens": toks, "requests": n_req,
                          "vllm_file": here, "vllm_version": getattr(vllm, "__version__", "?")}))
        return 0
    except BaseException as e:  # noqa: BLE001 - the caller wants the reason as data, whatever it is
        tb = traceback.format_exc().strip().splitlines()
        print(json.dumps({"ok": False, "error": f"{type(e).__name__}: {str(e)[:400]}", "where": tb[-3:] if len(tb) >= 3 else tb}))
        return 0


if __name__ == "__main__":
    sys.exit(main())
