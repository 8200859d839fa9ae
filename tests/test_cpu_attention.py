"""The C++ paged attention of the CPU backend against the PyTorch oracle (decode rows, prefill chunks over a cached prefix, sliding
window, soft cap, sinks, fp32 and bf16 caches, strided queries), and an engine run that takes it."""
import pytest
import torch

from onecat_vllm import ops
from onecat_vllm.ops import ref


def _case(dtype, D, Hq, Hkv, bs, lens, ctxs, seed=0):
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    T = sum(lens)
    S = [c + l for c, l in zip(ctxs, lens)]
    nb = [-(-s // bs) for s in S]
    total = sum(nb) + 1
    cache = (torch.randn(total, 2, Hkv, bs, D, generator=g) * 0.5).to(dtype)
    perm = torch.randperm(total - 1, generator=g) + 1          # pages in no particular order
    bt = torch.zeros(R, max(nb), dtype=torch.int32)
    o = 0
    for r in range(R):
        bt[r, : nb[r]] = perm[o:o + nb[r]].to(torch.int32)
        o += nb[r]
    wide = (torch.randn(T, Hq, 2 * D, generator=g) * 0.5).to(dtype)
    q = wide[..., :D]                                          # rows of a wider buffer, as the fused projection gives them
    qsl = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32)
    sl = torch.tensor(S, dtype=torch.int32)
    return q, cache, bt, qsl, sl


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opts", [dict(), dict(window=9), dict(softcap=3.0), dict(sinks=True), dict(window=5, softcap=2.0, sinks=True)])
def test_native_cpu_attention_matches_the_oracle(dtype, opts):
    D, Hq, Hkv, bs = 32, 6, 2, 16
    q, cache, bt, qsl, sl = _case(dtype, D, Hq, Hkv, bs, lens=[1, 7, 1, 33, 16], ctxs=[40, 0, 0, 21, 64])
    kw = dict(window=opts.get("window", 0), softcap=opts.get("softcap", 0.0))
    sinks = torch.linspace(-1.0, 1.0, Hq) if opts.get("sinks") else None
    want, want_lse = ref.paged_attention(q, cache, bt, qsl, sl, D ** -0.5, return_lse=True, sinks=sinks, **kw)
    got, got_lse = ops.cpu_paged_attention(q, cache, bt, qsl, sl, D ** -0.5, return_lse=True, sinks=sinks, threads=3, **kw)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got.float(), want.float(), atol=tol, rtol=tol), float((got.float() - want.float()).abs().max())
    assert torch.allclose(got_lse, want_lse, atol=1e-4, rtol=1e-4)
    one = ops.cpu_paged_attention(q, cache, bt, qsl, sl, D ** -0.5, sinks=sinks, threads=1, **kw)
    assert torch.equal(one, got)                                # the thread count does not change the result


def test_engine_runs_on_the_native_cpu_attention(monkeypatch):
    from onecat_vllm import LLM, SamplingParams, envs
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=500, max_position_embeddings=256)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 40, 70)]
    sp = SamplingParams(temperature=0, max_tokens=12, ignore_eos=True)

    def run():
        llm = LLM(hf_config=cfg, max_model_len=256, dtype="float32", device="cpu", max_num_batched_tokens=48)
        out = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        llm.shutdown()
        return out
    want = run()
    monkeypatch.setenv("ONECAT_CPU_ATTENTION", "native")
    calls = []
    orig = ops.cpu_paged_attention
    monkeypatch.setattr(ops, "cpu_paged_attention", lambda *a, **k: (calls.append(1), orig(*a, **k))[1])
    assert envs.ONECAT_CPU_ATTENTION == "native"
    assert run() == want and calls
