"""Multi-GPU checks (2 ranks as child processes over NCCL + CUDA-IPC peer memory): the fused reduce + residual + RMSNorm
kernels against an fp32 reference built from NCCL, and a TP2 engine against TP1."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _need2():
    _need(2)


def _fused_worker(rank, world, port, q, oneshot="lamport"):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ONECAT_TP_ONESHOT=oneshot, NCCL_NVLS_ENABLE="0", ONECAT_TP_NVLS="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    from onecat_vllm.parallel.fused import LAMPORT, ONE_SHOT, TWO_SHOT, FusedTP
    dev = torch.device("cuda", rank)
    H, tmax = 5120, 1024
    f = FusedTP(world, rank, dev, tmax, H)
    ok = True
    msgs = []

    def check(it, T, mode, gemma, pushed_gemm=False):
        nonlocal ok
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        g2 = torch.Generator(device=dev).manual_seed(7 + it)
        res = torch.randn(T, H, device=dev, generator=g2).bfloat16()
        w = (torch.randn(H, device=dev, generator=g2) * 0.1 + (0 if gemma else 1)).bfloat16()
        if pushed_gemm:
            # row-parallel GEMM whose epilogue stores its tiles into the peers' slabs: this rank holds a K-slice of the weight
            Kd = 256
            xa = torch.randn(T, Kd, device=dev, generator=g).bfloat16()
            wa = (torch.randn(H, Kd, device=dev, generator=g) * 0.05).bfloat16()
            part = (xa.float() @ wa.float().t()).bfloat16()  # what the kernel computes, up to accumulation order
            out = f.partial_buffer(T, H, torch.bfloat16)
            y = K.gemm_bf16(xa, wa, out=out) if not f.use_push(T) else K._gemm(xa, wa, None, None, out, None, H, H, H, 0, 0, 1, push=f.push_spec(T))
            x, r = f.reduce_add_norm(y, res, w, 1e-6, gemma, pushed=f.use_push(T))
            tol = 0.08
        else:
            part = torch.randn(T, H, device=dev, generator=g).bfloat16()
            part[0, :16] = -0.0  # the arrival marker of the flag-free path is a legal value of the data
            part[T - 1, H - 8:] = 0.0
            buf = f.partial_buffer(T, H, torch.bfloat16)
            buf.copy_(part)
            x, r = f.reduce_add_norm(buf, res, w, 1e-6, gemma, mode=mode)
            tol = 0.05
        torch.cuda.synchronize()
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        tot = sum(p.float() for p in parts)  # the kernel sums bf16 partials in fp32 in rank order
        new_res = (tot + res.float()).bfloat16()
        xe, _ = ref.rms_norm(new_res, w, 1e-6, None, gemma)
        eff = f.mode_for(T) if (mode is None or pushed_gemm) else (LAMPORT if (mode == ONE_SHOT and f.mode_for(T) == LAMPORT) else mode)
        if eff == TWO_SHOT:
            per = -(-T // world)
            lo, hi = min(rank * per, T), min(rank * per + per, T)
            r_ok = torch.equal(r[lo:hi], new_res[lo:hi]) if not pushed_gemm else bool(((r[lo:hi].float() - new_res[lo:hi].float()).abs() < 0.1).all())
        else:
            r_ok = torch.equal(r, new_res) if not pushed_gemm else bool(((r.float() - new_res.float()).abs() < 0.1).all())
        err = (x.float() - xe.float()).abs().max().item()
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x.contiguous())
        same = all(torch.equal(xs[0], t) for t in xs)  # all ranks must hold bit-identical outputs
        if not (r_ok and err < tol and same):
            ok = False
            msgs.append(f"it={it} T={T} mode={mode} eff={eff} pushed={pushed_gemm} r_ok={r_ok} err={err} same={same}")

    try:
        cases = [(1, ONE_SHOT, False), (64, ONE_SHOT, True), (333, TWO_SHOT, False), (1024, TWO_SHOT, True), (5, TWO_SHOT, False),
                 (64, ONE_SHOT, False), (64, ONE_SHOT, False), (7, None, True), (200, None, False), (33, None, False), (64, None, True),
                 (1, None, False), (256, None, False), (2, None, True)]
        for it, (T, mode, gemma) in enumerate(cases):
            check(it, T, mode, gemma)
        for it, T in enumerate((1, 48, 64, 130, 300, 16, 16, 16, 600, 1024)):  # GEMM + reduction; large batches push from the epilogue
            check(50 + it, T, None, it % 2 == 0, pushed_gemm=True)
        os.environ["ONECAT_TP_PUSH"] = "always"   # decode-sized batches too: the epilogue stores into the peers' arrival buffers
        for it, T in enumerate((1, 48, 64, 130, 16, 16, 16)):
            check(70 + it, T, None, it % 2 == 0, pushed_gemm=True)
        os.environ["ONECAT_TP_PUSH"] = "auto"
        # a captured reduction replayed back to back: the buffer rotation lives in device memory, so replays need no host state
        T = 8
        part = torch.full((T, H), float(rank + 1), device=dev).bfloat16()
        buf = f.partial_buffer(T, H, torch.bfloat16)
        buf.copy_(part)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                f.all_reduce(buf)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        dist.barrier()
        if f.mode_for(T) == LAMPORT:  # the flag path alternates host-side slots and is not replayed here
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                y1 = f.all_reduce(buf)
                y2 = f.all_reduce(y1)
            for _ in range(25):
                gr.replay()
            torch.cuda.synchronize()
            tot = float(sum(range(1, world + 1)))
            if not (torch.equal(y1, torch.full_like(y1, tot)) and torch.equal(y2, torch.full_like(y2, tot * world))):
                ok = False
                msgs.append(f"graph replay mismatch {y1[0, 0].item()} {y2[0, 0].item()}")
        ar = f.all_reduce(torch.full((3, H), float(rank + 1), device=dev).bfloat16())
        torch.cuda.synchronize()
        if not torch.equal(ar, torch.full((3, H), float(sum(range(1, world + 1))), device=dev).bfloat16()):
            ok = False
            msgs.append("all_reduce mismatch")
        st = K.check_status()
        if st:
            ok = False
            msgs.append(f"status {st}")
    finally:
        dist.barrier()
        f.close()
        dist.destroy_process_group()
    q.put((rank, ok, msgs))


def _spawn(fn, world, *args):
    import torch.multiprocessing as mp
    from onecat_vllm.executor.multiproc import _free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port, q) + args) for r in range(world)]
    for p in procs:
        p.start()
    res = []
    for p in procs:
        p.join(240)
    while not q.empty():
        res.append(q.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert len(res) == world, f"only {len(res)} of {world} ranks reported (exit codes {[p.exitcode for p in procs]})"
    for rank, ok, msgs in res:
        assert ok, f"rank {rank}: {msgs}"


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("oneshot", ["lamport", "flags"])
def test_fused_reduce_norm(world, oneshot):
    """Reduce + residual + RMSNorm over peer memory (flag-free and flag-based one-shot, two-shot), the GEMM epilogue push, and a
    captured reduction replayed 25 times, against a CPU-rank simulation (gather every rank's bf16 partial, sum in fp32, add, normalise)."""
    _need(world)
    _spawn(_fused_worker, world, oneshot)


def _nvls_worker(rank, world, port, q):
    """The reduction that adds inside the switch: sums, residual and normalised rows against a simulation from gathered partials,
    bit-identical outputs on all ranks, results that stay valid over the next reductions, and a captured pair replayed 25 times."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), ONECAT_TP_NVLS="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    from onecat_vllm.parallel.fused import NVLS, FusedTP
    dev = torch.device("cuda", rank)
    H, tmax = 5120, 1024
    f = FusedTP(world, rank, dev, tmax, H)
    ok, msgs = True, []
    try:
        if f.nv is None:
            msgs.append("no multicast support on this machine: nothing to check")
        else:
            kept = []
            for it, (T, gemma, with_res) in enumerate([(1, False, True), (64, True, True), (7, False, True), (333, False, True), (1024, True, True),
                                                        (64, False, False), (16, False, True), (5, True, True)]):
                assert f.mode_for(T) == NVLS
                g = torch.Generator(device=dev).manual_seed(100 * it + rank)
                g2 = torch.Generator(device=dev).manual_seed(7 + it)
                part = torch.randn(T, H, device=dev, generator=g).bfloat16()
                res = torch.randn(T, H, device=dev, generator=g2).bfloat16() if with_res else None
                w = (torch.randn(H, device=dev, generator=g2) * 0.1 + (0 if gemma else 1)).bfloat16()
                buf = f.partial_buffer(T, H, torch.bfloat16)
                buf.copy_(part)
                x, r = f.reduce_add_norm(buf, res, w, 1e-6, gemma)
                torch.cuda.synchronize()
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                tot = sum(p.float() for p in parts).bfloat16()          # the switch accumulates in fp32 and returns bf16
                new_res = (tot.float() + res.float()).bfloat16() if with_res else tot
                xe, _ = ref.rms_norm(new_res, w, 1e-6, None, gemma)
                # the switch rounds intermediate sums to bf16 on its way: up to an ulp of the largest partial sum
                r_ok = True if not with_res else bool(((r.float() - new_res.float()).abs() <= 0.14).all())
                err = (x.float() - xe.float()).abs().max().item()
                both = torch.cat([x, r]) if with_res else x
                xs = [torch.empty_like(both) for _ in range(world)]
                dist.all_gather(xs, both.contiguous())
                same = all(torch.equal(xs[0], t) for t in xs)
                kept.append((x, x.clone()))
                if not (r_ok and err < 0.08 and same):
                    ok = False
                    msgs.append(f"it={it} T={T} r_ok={r_ok} err={err} same={same}")
            # a result stays where it is for the next three reductions
            for (view, copy) in kept[-3:]:
                if not torch.equal(view, copy):
                    ok = False
                    msgs.append("a result was overwritten within three reductions")
            T = 8
            buf = f.partial_buffer(T, H, torch.bfloat16)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(4):
                    f.partial_buffer(T, H, torch.bfloat16).fill_(float(rank + 1))
                    f.all_reduce(f.partial_buffer(T, H, torch.bfloat16))
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            dist.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                b1 = f.partial_buffer(T, H, torch.bfloat16)
                b1.fill_(float(rank + 1))
                y1 = f.all_reduce(b1)
                b2 = f.partial_buffer(T, H, torch.bfloat16)
                b2.copy_(y1)
                y2 = f.all_reduce(b2)
            for _ in range(25):
                gr.replay()
            torch.cuda.synchronize()
            tot = float(sum(range(1, world + 1)))
            if not (torch.equal(y1, torch.full_like(y1, tot)) and torch.equal(y2, torch.full_like(y2, tot * world))):
                ok = False
                msgs.append(f"graph replay mismatch {y1[0, 0].item()} {y2[0, 0].item()}")
            st = K.check_status()
            if st:
                ok = False
                msgs.append(f"status {st}")
    finally:
        dist.barrier()
        f.close()
        dist.destroy_process_group()
    q.put((rank, ok, msgs))


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_switch_reduce_norm(world):
    _need(world)
    _spawn(_nvls_worker, world)


def _a2a_worker(rank, world, port, q, qmethod="none"):
    """Expert-parallel MoE by token exchange over peer memory: every rank routes a slice of the batch; the gathered result must
    match the single-process expert oracle over all experts, eagerly and when a captured exchange is replayed."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    from onecat_vllm.parallel.all2all import PeerAll2All, TorchAll2All, token_slice
    dev = torch.device("cuda", rank)
    E, k, H, I, tmax = 8 * world, 4, 256, 128, 512
    El = E // world
    g = torch.Generator().manual_seed(1)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16()

    class Layer:
        pass
    layer = Layer()
    layer.qmethod, layer.block, layer.E_local, layer.e_off, layer._dq, layer.kernel_state = "none", None, El, rank * El, None, None
    layer.w13 = torch.nn.Parameter(w13[rank * El:(rank + 1) * El].to(dev), requires_grad=False)
    layer.w2 = torch.nn.Parameter(w2[rank * El:(rank + 1) * El].to(dev), requires_grad=False)
    layer.dequantized = lambda: (layer.w13, layer.w2)
    K.prepare_moe(layer)
    mgr = PeerAll2All(world, rank, dev, tmax, H, E, k)
    ok, msgs = True, []
    w13d, w2d = w13.to(dev), w2.to(dev)

    def batch(T, seed):
        gg = torch.Generator().manual_seed(seed)
        x = (torch.randn(T, H, generator=gg)).bfloat16().to(dev)
        if seed % 3 == 0:   # skewed routing: most pairs go to the experts of one rank
            logits = torch.randn(T, E, generator=gg) + torch.cat([torch.full((El,), 4.0), torch.zeros(E - El)])
        else:
            logits = torch.randn(T, E, generator=gg)
        w, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
        return x, (w / w.sum(-1, keepdim=True)).to(dev), ids.to(torch.int32).to(dev)

    for it, T in enumerate((1, 3, 64, 200, 512, 64)):
        x, w, ids = batch(T, it)
        want = ref.fused_experts(x, w13d, w2d, w, ids.long())
        lo, hi = token_slice(T, world, rank)
        got = mgr.moe(layer, x[lo:hi], w[lo:hi], ids[lo:hi], t_off=lo, T_total=T, gather=True).clone()
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        scale = want.float().abs().max().item() + 1e-6
        if err > 0.03 * scale + 0.02:
            ok = False
            msgs.append(f"T={T} err={err} scale={scale}")
        all_got = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(all_got, got)
        if any(not torch.equal(all_got[0], t) for t in all_got):
            ok = False
            msgs.append(f"T={T}: ranks hold different gathered rows")
    # a captured exchange replayed on fresh inputs: sequence numbers live on the device, so the graph needs no reset
    T = 48
    lo, hi = token_slice(T, world, rank)
    xs, ws, idss = torch.zeros(hi - lo, H, device=dev, dtype=torch.bfloat16), torch.zeros(hi - lo, k, device=dev), torch.zeros(hi - lo, k, device=dev, dtype=torch.int32)
    x, w, ids = batch(T, 100)
    xs.copy_(x[lo:hi]); ws.copy_(w[lo:hi]); idss.copy_(ids[lo:hi])
    mgr.moe(layer, xs, ws, idss, t_off=lo, T_total=T, gather=True)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = mgr.moe(layer, xs, ws, idss, t_off=lo, T_total=T, gather=True)
    for rep in range(6):
        x, w, ids = batch(T, 200 + rep)
        xs.copy_(x[lo:hi]); ws.copy_(w[lo:hi]); idss.copy_(ids[lo:hi])
        graph.replay()
        torch.cuda.synchronize()
        want = ref.fused_experts(x, w13d, w2d, w, ids.long())
        err = (out.float() - want.float()).abs().max().item()
        if err > 0.03 * want.float().abs().max().item() + 0.02:
            ok = False
            msgs.append(f"replay {rep} err={err}")
        dist.barrier()
    st = K.check_status()
    if st != 0:
        ok = False
        msgs.append(f"device status {st}")
    del graph
    torch.cuda.synchronize()
    dist.barrier()
    mgr.close()
    q.put((rank, ok, msgs))
    dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_exchange_over_peer_memory(world):
    _need(world)
    _spawn(_a2a_worker, world)


CFG = dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=2048, num_hidden_layers=3, num_attention_heads=8,
           num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
           tie_word_embeddings=False)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("tp_comm", ["fused", "nccl"])
def test_engine_tp2_matches_tp1(tmp_path, tp_comm):
    _need2()
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.bfloat16), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 300, 64)]
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    kw = dict(model=str(tmp_path), device="cuda", dtype="bfloat16", max_model_len=1024, max_num_batched_tokens=512, max_num_seqs=8, gpu_memory_utilization=0.2)
    one = LLM(**kw)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    one.shutdown()
    two = LLM(tensor_parallel_size=2, distributed_executor_backend="mp", tp_comm=tp_comm, **kw)
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp)]
    two.shutdown()
    agree = sum(next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), len(x)) for x, y in zip(got, ref))
    # random weights give near-tied logits, so bf16 summation order flips a greedy choice now and then and everything after it
    # differs: the first token of every prompt must agree, and most of the prefix overall
    assert all(x[0] == y[0] for x, y in zip(got, ref)), f"TP2 ({tp_comm}) first tokens differ: {got} vs {ref}"
    assert agree / (16 * len(prompts)) > 0.4, f"TP2 ({tp_comm}) diverges from TP1 too early: {got} vs {ref}"


@pytest.mark.timeout(600)
def test_lora_tp2_matches_tp1_on_gpus(tmp_path):
    """A LoRA adapter served by two tensor-parallel GPU ranks (sharded A / B, delta added before the fused reduction) against one GPU."""
    _need2()
    import json
    from safetensors.torch import save_file
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.lora import LoRARequest
    from onecat_vllm.models import build_model
    base = tmp_path / "base"
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.bfloat16), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG, str(base))
    ad = tmp_path / "ad"
    ad.mkdir()
    g = torch.Generator().manual_seed(3)
    r, H, I = 8, CFG["hidden_size"], CFG["intermediate_size"]
    dims = {"q_proj": (H, CFG["num_attention_heads"] * 128), "v_proj": (H, CFG["num_key_value_heads"] * 128), "o_proj": (CFG["num_attention_heads"] * 128, H),
            "gate_proj": (H, I), "down_proj": (I, H)}
    sd = {}
    for layer in range(CFG["num_hidden_layers"]):
        for name, (din, dout) in dims.items():
            blk = "self_attn" if name in ("q_proj", "v_proj", "o_proj") else "mlp"
            pre = f"base_model.model.model.layers.{layer}.{blk}.{name}"
            sd[pre + ".lora_A.weight"] = (torch.randn(r, din, generator=g) * 0.05).bfloat16()
            sd[pre + ".lora_B.weight"] = (torch.randn(dout, r, generator=g) * 0.05).bfloat16()
    save_file(sd, str(ad / "adapter_model.safetensors"))
    (ad / "adapter_config.json").write_text(json.dumps({"r": r, "lora_alpha": 16, "target_modules": list(dims)}))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 130)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    req = LoRARequest("ad", 1, str(ad))
    kw = dict(model=str(base), device="cuda", dtype="bfloat16", max_model_len=512, max_num_seqs=8, gpu_memory_utilization=0.2, enable_lora=True)
    one = LLM(**kw)
    plain = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp, lora_request=req)]
    one.shutdown()
    two = LLM(tensor_parallel_size=2, distributed_executor_backend="mp", **kw)
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp, lora_request=req)]
    two.shutdown()
    assert ref != plain, "the adapter must change the output"
    assert all(x[0] == y[0] for x, y in zip(got, ref)), f"TP2 LoRA first tokens differ: {got} vs {ref}"
    agree = sum(next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), len(x)) for x, y in zip(got, ref))
    assert agree / (12 * len(prompts)) > 0.4, f"TP2 LoRA diverges from one GPU too early: {got} vs {ref}"


CFG_MOE = dict(architectures=["Qwen3MoeForCausalLM"], hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
               num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
               tie_word_embeddings=False, num_experts=32, num_experts_per_tok=4, moe_intermediate_size=256, norm_topk_prob=True)


@pytest.mark.timeout(600)
@pytest.mark.parametrize("ep_comm", ["reduce", "a2a"])
def test_engine_expert_parallel_two_gpus(tmp_path, monkeypatch, ep_comm):
    """A Qwen-MoE engine with its experts split over two GPUs: partial sums through the fused reduction, or token exchange over
    peer memory (each rank routes half of every batch, decode graphs included), against one GPU."""
    _need2()
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    m = build_model(ModelConfig.from_hf_dict(CFG_MOE, dtype=torch.bfloat16), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, CFG_MOE, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 300, 64)]
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    kw = dict(model=str(tmp_path), device="cuda", dtype="bfloat16", max_model_len=1024, max_num_batched_tokens=512, max_num_seqs=8, gpu_memory_utilization=0.2)
    one = LLM(**kw)
    ref = [o.outputs[0].token_ids for o in one.generate(prompts, sp)]
    one.shutdown()
    monkeypatch.setenv("ONECAT_EP_COMM", ep_comm)
    two = LLM(tensor_parallel_size=2, distributed_executor_backend="mp", enable_expert_parallel=True, **kw)
    got = [o.outputs[0].token_ids for o in two.generate(prompts, sp)]
    two.shutdown()
    agree = sum(next((i for i, (a, b) in enumerate(zip(x, y)) if a != b), len(x)) for x, y in zip(got, ref))
    assert all(x[0] == y[0] for x, y in zip(got, ref)), f"EP2 ({ep_comm}) first tokens differ: {got} vs {ref}"
    assert agree / (16 * len(prompts)) > 0.4, f"EP2 ({ep_comm}) diverges from one GPU too early: {got} vs {ref}"
