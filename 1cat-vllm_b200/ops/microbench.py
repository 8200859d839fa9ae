"""Kernel micro-benchmarks with roofline fractions against the measured peaks of the box.

``python -m onecat_vllm.ops.microbench [--only gemm|w4|wq|attn|attn_prefill|norm|gdn|gdn_prefill|moe|sample|mla|rope|reject|w4tp] [--small] [--json PATH]``
Timing: CUDA events on the launching stream, 3 warm-up launches, an L2 flush (a 256 MB write) before every timed
launch, median of ``--iters`` launches. ``--small`` runs one launch of one case per kernel (for ncu captures)."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks() -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    for up in (3, 2):
        p = os.path.join(*([here] + [".."] * up + ["MEASURED_PEAKS.json"]))
        if os.path.exists(p):
            d = json.load(open(p))
            return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


_FLUSH = None


def timeit(fn, iters: int = 10, warmup: int = 3, flush: bool = True) -> float:
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


class _L:
    def __init__(self, fuse=False):
        self.fuse_silu_mul, self.bias, self.kernel_state = fuse, None, None


def bench_gemm(rows: list, small: bool, iters: int, pk: dict) -> None:
    from onecat_vllm.ops import cuda as K
    shapes = [(8192, 7168, 5120), (8192, 34816, 5120), (8192, 5120, 17408), (1088, 34816, 5120), (64, 5120, 5120), (64, 151936, 5120)]
    if small:
        shapes = [(2048, 8192, 5120)]
    for T, N, Kd in shapes:
        x = torch.randn(T, Kd, device="cuda").bfloat16()
        w = (torch.randn(N, Kd, device="cuda") * 0.02).bfloat16()
        out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: K.gemm_bf16(x, w, out=out), 1 if small else iters, 1 if small else 3)
        tf = 2.0 * T * N * Kd / ms / 1e9
        lib = timeit(lambda: torch.matmul(x, w.t()), 1 if small else iters, 1 if small else 3)
        rows.append(dict(kernel="gemm_bf16", T=T, N=N, K=Kd, ms=ms, tflops=tf, frac_of_peak=tf / pk["bf16_tflops"], cublas_ms=lib,
                         cublas_tflops=2.0 * T * N * Kd / lib / 1e9))
        del x, w, out


def bench_w4(rows: list, small: bool, iters: int, pk: dict) -> None:
    from onecat_vllm.ops import cuda as K
    cases = [(64, 7168, 5120, False), (64, 34816, 5120, True), (64, 5120, 17408, False), (64, 5120, 5120, False), (1, 34816, 5120, True),
             (256, 34816, 5120, True), (1088, 34816, 5120, True), (1088, 7168, 5120, False), (1088, 5120, 5120, False), (1088, 5120, 17408, False),
             (8192, 34816, 5120, True), (8192, 5120, 17408, False)]
    if small:
        cases = [(64, 34816, 5120, True), (64, 7168, 5120, False)]
    for T, N, Kd, fuse in cases:
        q = torch.randint(0, 16, (N, Kd), device="cuda", dtype=torch.uint8)
        z = torch.randint(0, 16, (N, Kd // 128), device="cuda", dtype=torch.uint8)
        s = (torch.rand(N, Kd // 128, device="cuda") * 0.01 + 1e-3).half()
        layer = _L(fuse)
        K.prepare_w4(layer, q, z, s, 128)
        del q, z, s
        x = torch.randn(T, Kd, device="cuda").bfloat16()
        out = torch.empty(T, layer.kernel_state["n_out"], device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: K.linear(layer, x, out=out), 1 if small else iters, 1 if small else 3)
        wbytes = N * Kd / 2 + N * (Kd // 128) * 4
        bytes_ = wbytes + T * Kd * 2 + out.numel() * 2
        tf = 2.0 * T * N * Kd / ms / 1e9
        rows.append(dict(kernel="gemm_w4a16", T=T, N=N, K=Kd, fused_silu=fuse, ms=ms, gbs=bytes_ / ms / 1e6, frac_of_hbm=bytes_ / ms / 1e6 / pk["hbm_gbs"],
                         tflops=tf, frac_of_peak=tf / pk["bf16_tflops"]))
        del layer, x, out


def bench_w4_tp(rows: list, small: bool, iters: int, pk: dict) -> None:
    """The four packed GEMMs of one dense-27B decoder layer at the slices a tensor-parallel rank holds (qkv and gate|up split by
    output rows, o and down by k), decode-sized batches: flushed single launches and back-to-back launches inside a CUDA graph."""
    from onecat_vllm.ops import cuda as K

    def graph_us(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n * 1e3
    for tp in ((8,) if small else (1, 2, 4, 8)):
        for T in ((64,) if small else (64, 16)):
            tot_cold = tot_graph = 0.0
            for name, N, Kd, fuse in (("qkv", 7168 // tp, 5120, False), ("o", 5120, 5120 // tp, False), ("gate|up", 34816 // tp, 5120, True),
                                      ("down", 5120, 17408 // tp, False)):
                q = torch.randint(0, 16, (N, Kd), device="cuda", dtype=torch.uint8)
                z = torch.randint(0, 16, (N, Kd // 128), device="cuda", dtype=torch.uint8)
                s_ = (torch.rand(N, Kd // 128, device="cuda") * 0.01 + 1e-3).half()
                layer = _L(fuse)
                K.prepare_w4(layer, q, z, s_, 128)
                del q, z, s_
                x = torch.randn(T, Kd, device="cuda").bfloat16()
                out = torch.empty(T, layer.kernel_state["n_out"], device="cuda", dtype=torch.bfloat16)
                cold = timeit(lambda: K.linear(layer, x, out=out), 1 if small else iters, 1 if small else 3) * 1e3
                warm = cold if small else graph_us(lambda: K.linear(layer, x, out=out))
                tot_cold += cold
                tot_graph += warm
                rows.append(dict(kernel="gemm_w4a16_tp_slice", tp=tp, proj=name, T=T, N=N, K=Kd, us_flushed=cold, us_in_graph=warm,
                                 gbs=(N * Kd / 2) / cold / 1e3))
                del layer, x, out
            rows.append(dict(kernel="gemm_w4a16_tp_slice", tp=tp, proj="layer total", T=T, us_flushed=tot_cold, us_in_graph=tot_graph))


def bench_attn(rows: list, small: bool, iters: int, pk: dict, prefill_only: bool = False) -> None:
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    cases = [("decode", 64, 1, 1150, 40, 8, 128), ("decode", 8, 1, 32768, 40, 8, 128), ("decode-d256", 64, 1, 2048, 24, 4, 256),
             ("prefill", 8, 1024, 0, 40, 8, 128), ("prefill", 1, 8192, 0, 40, 8, 128), ("prefill-d256", 1, 4096, 0, 24, 4, 256),
             ("decode-fp8kv", 64, 1, 1150, 40, 8, 128), ("decode-fp8kv", 8, 1, 32768, 40, 8, 128), ("decode-window128", 64, 1, 1150, 40, 8, 128)]
    if small:
        cases = [("decode", 64, 1, 1150, 40, 8, 128)]
    if prefill_only:
        cases = [("prefill", 2, 2048, 0, 40, 8, 128)] if small else [c for c in cases if c[0].startswith("prefill")]
    for name, R, ql, ctx, Hq, Hkv, D in cases:
        S = ctx + ql
        nb = -(-S // 16)
        total = R * nb + 1
        cache = (torch.randn(total, 2, Hkv, 16, D, device="cuda") * 0.3).bfloat16()
        if "fp8kv" in name:
            cache = cache.to(torch.float8_e4m3fn)
        window = 128 if "window" in name else 0
        bt = (torch.arange(R * nb, device="cuda", dtype=torch.int32) + 1).view(R, nb)
        T = R * ql
        q = (torch.randn(T, Hq, D, device="cuda") * 0.3).bfloat16()
        qsl = (torch.arange(R + 1, device="cuda", dtype=torch.int32) * ql)
        sl = torch.full((R,), S, device="cuda", dtype=torch.int32)
        md = AttentionMetadata(R, T, qsl, sl, bt, None, None, ql, S, query_lens_cpu=[ql] * R, seq_lens_cpu=[S] * R)
        out = torch.empty(T, Hq, D, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: K.paged_attention(q, cache, md, D ** -0.5, out=out, window=window), 1 if small else iters, 1 if small else 3)
        kv_bytes = R * (min(S, window) if window else S) * 2 * Hkv * D * cache.element_size()
        flops = 4.0 * R * Hq * D * (ql * ctx + ql * (ql + 1) / 2)
        rows.append(dict(kernel="paged_attention", case=name, R=R, q_len=ql, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, ms=ms, kv_gbs=kv_bytes / ms / 1e6,
                         frac_of_hbm=kv_bytes / ms / 1e6 / pk["hbm_gbs"], tflops=flops / ms / 1e9, plan=md.attn_plan[1]))
        del cache, q, out


def bench_norm(rows: list, small: bool, iters: int, pk: dict) -> None:
    from onecat_vllm.ops import cuda as K
    for T, H in ([(8192, 5120)] if small else [(8192, 5120), (64, 5120), (8192, 7168)]):
        x = torch.randn(T, H, device="cuda").bfloat16()
        r = torch.randn(T, H, device="cuda").bfloat16()
        w = torch.ones(H, device="cuda").bfloat16()
        ms = timeit(lambda: K.rms_norm(x, w, 1e-6, r, False), 1 if small else iters, 1 if small else 3)
        b = 4 * T * H * 2
        rows.append(dict(kernel="rms_norm_residual", T=T, H=H, ms=ms, gbs=b / ms / 1e6, frac_of_hbm=b / ms / 1e6 / pk["hbm_gbs"]))


def bench_gdn(rows: list, small: bool, iters: int, pk: dict, prefill_only: bool = False) -> None:
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    Hk, Hv, Kd, Vd, kw = 16, 48, 128, 128, 4
    C = 2 * Hk * Kd + Hv * Vd
    cases = [("decode", 64, 1)] if small else [("decode", 64, 1), ("decode", 8, 1), ("verify4", 8, 4), ("prefill", 4, 2048), ("prefill", 1, 8192)]
    if prefill_only:
        cases = [("prefill", 1, 2048)] if small else [("prefill", 1, 2048), ("prefill", 1, 8192), ("prefill", 4, 2048)]
    for name, R, ql in cases:
        T = R * ql
        mixed = (torch.randn(T, C, device="cuda") * 0.5).bfloat16()
        ba = torch.randn(T, 2 * Hv, device="cuda").bfloat16()
        conv_w = (torch.randn(C, kw, device="cuda") * 0.3).bfloat16()
        A_log, dtb = torch.rand(Hv, device="cuda"), torch.rand(Hv, device="cuda")
        conv_state = torch.zeros(R, C, kw - 1, device="cuda", dtype=torch.bfloat16)
        ssm = torch.zeros(R, Hv, Kd, Vd, device="cuda")
        qsl = torch.arange(R + 1, device="cuda", dtype=torch.int32) * ql
        state_bytes = 2 * R * Hv * Kd * Vd * 4
        for mode in (("chunked", "recurrent") if name == "prefill" else ("recurrent",)):
            os.environ["ONECAT_GDN_PREFILL"] = mode
            md = AttentionMetadata(R, T, qsl, None, None, None, None, ql, 0, state_slots=torch.arange(R, device="cuda", dtype=torch.int32),
                                   has_initial_state=torch.ones(R, device="cuda", dtype=torch.int32), query_lens_cpu=[ql] * R)
            ms = timeit(lambda: K.gdn_forward(mixed, ba[:, :Hv], ba[:, Hv:], conv_w, A_log, dtb, conv_state, ssm, md, Hk, Hv, Kd, Vd), 1 if small else iters,
                        1 if small else 3)
            # chunked form: ~11.5 MFLOP per 64-token chunk and value head (K K^T, Q K^T, T W/U, and the three products against the state)
            flops = (T / 64.0) * Hv * 11.5e6 if mode == "chunked" else 0.0
            rows.append(dict(kernel="gdn_conv+" + ("chunked_prefill" if (mode == "chunked" and name == "prefill") else "recurrence"), case=name, R=R, q_len=ql, ms=ms,
                             state_gbs=state_bytes / ms / 1e6, frac_of_hbm=state_bytes / ms / 1e6 / pk["hbm_gbs"], tokens_per_s=T / ms * 1e3,
                             us_per_token=ms * 1e3 / ql, tflops=flops / ms / 1e9))
        os.environ.pop("ONECAT_GDN_PREFILL", None)


def bench_moe(rows: list, small: bool, iters: int, pk: dict) -> None:
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    cases = [(256, 256, 8, 2048, 512)] if small else [(256, 256, 8, 2048, 512), (8192, 256, 8, 2048, 512), (64, 256, 8, 2048, 512)]
    for kind in (("none",) if small else ("none", "fp8", "mxfp4")):
        for T, E, k, H, I in cases:
            x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()

            class M:
                pass
            m = M()
            m.qmethod, m.E_local, m.e_off, m._dq, m.block = kind, E, 0, None, (128, 128)
            if kind == "none":
                m.w13 = (torch.randn(E, 2 * I, H, device="cuda") * 0.03).bfloat16()
                m.w2 = (torch.randn(E, H, I, device="cuda") * 0.03).bfloat16()
                m.dequantized = lambda: (m.w13, m.w2)
                wb = 2.0
            elif kind == "fp8":
                m.w13 = (torch.randn(E, 2 * I, H, device="cuda")).to(torch.float8_e4m3fn)
                m.w2 = (torch.randn(E, H, I, device="cuda")).to(torch.float8_e4m3fn)
                m.w13_scale = torch.full((E, 2 * I // 128, H // 128), 0.03, device="cuda")
                m.w2_scale = torch.full((E, H // 128, I // 128), 0.03, device="cuda")
                wb = 1.0
            else:
                m.w13 = torch.randint(0, 256, (E, 2 * I, H // 2), device="cuda", dtype=torch.uint8)
                m.w2 = torch.randint(0, 256, (E, H, I // 2), device="cuda", dtype=torch.uint8)
                m.w13_scale = torch.full((E, 2 * I, H // 32), 120, device="cuda", dtype=torch.uint8)
                m.w2_scale = torch.full((E, H, I // 32), 120, device="cuda", dtype=torch.uint8)
                wb = 0.5 + 1.0 / 32
            K.prepare_moe(m)
            tw, ti = ref.topk_softmax(torch.randn(T, E, device="cuda"), k, True)
            ms = timeit(lambda: K.fused_moe(m, x, tw, ti), 1 if small else iters, 1 if small else 3)
            flops = 2.0 * T * k * 3 * H * I
            wbytes = min(E, T * k) * 3 * H * I * wb
            rows.append(dict(kernel=f"fused_moe({'bf16' if kind == 'none' else kind} experts)", T=T, E=E, k=k, H=H, I=I, ms=ms, tflops=flops / ms / 1e9,
                             frac_of_peak=flops / ms / 1e9 / pk["bf16_tflops"], weight_gbs=wbytes / ms / 1e6))
            del m


def bench_wq(rows: list, small: bool, iters: int, pk: dict) -> None:
    """Weight-only FP8 (128x128 block scales) and MXFP4 linears: DeepSeek-V3-class shapes (hidden 7168)."""
    from onecat_vllm.ops import cuda as K
    cases = [(64, 7168, 7168), (64, 36864, 7168), (8192, 7168, 7168)]
    if small:
        cases = cases[:1]
    for kind in ("fp8", "mxfp4"):
        for T, N, Kd in cases:
            layer = _L(False)
            if kind == "fp8":
                layer.weight = torch.nn.Parameter(torch.randn(N, Kd, device="cuda").to(torch.float8_e4m3fn), requires_grad=False)
                layer.weight_scale_inv = torch.nn.Parameter(torch.full((N // 128, Kd // 128), 0.02, device="cuda"), requires_grad=False)
                K.prepare_fp8(layer, (128, 128))
                wbytes = N * Kd + N * (Kd // 128) * 4
            else:
                layer.weight = torch.nn.Parameter(torch.randint(0, 256, (N, Kd // 2), device="cuda", dtype=torch.uint8), requires_grad=False)
                layer.weight_scale = torch.nn.Parameter(torch.full((N, Kd // 32), 120, device="cuda", dtype=torch.uint8), requires_grad=False)
                K.prepare_fp4(layer, "mxfp4")
                wbytes = N * Kd / 2 + N * (Kd // 64) * 4
            x = torch.randn(T, Kd, device="cuda").bfloat16()
            out = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            ms = timeit(lambda: K.linear(layer, x, out=out), 1 if small else iters, 1 if small else 3)
            bytes_ = wbytes + T * Kd * 2 + out.numel() * 2
            tf = 2.0 * T * N * Kd / ms / 1e9
            rows.append(dict(kernel=f"gemm_{kind}_weight_only", T=T, N=N, K=Kd, ms=ms, gbs=bytes_ / ms / 1e6, frac_of_hbm=bytes_ / ms / 1e6 / pk["hbm_gbs"],
                             tflops=tf, frac_of_peak=tf / pk["bf16_tflops"]))
            del layer, x, out


def bench_mla(rows: list, small: bool, iters: int, pk: dict) -> None:
    """Absorbed MLA decode over a paged latent cache (576-wide rows): 128 heads, one query token per request."""
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    lora, rope, bs, H = 512, 64, 16, 128
    for R, ctx in ([(32, 4096)] if small else [(32, 4096), (128, 5120), (8, 32768)]):
        nb = -(-ctx // bs)
        cache = (torch.randn(R * nb + 1, bs, lora + rope, device="cuda") * 0.3).bfloat16()
        bt = (torch.arange(R * nb, device="cuda", dtype=torch.int32) + 1).view(R, nb)
        q_abs = (torch.randn(R, H, lora, device="cuda") * 0.3).bfloat16()
        q_pe = (torch.randn(R, H, rope, device="cuda") * 0.3).bfloat16()
        qsl = torch.arange(R + 1, device="cuda", dtype=torch.int32)
        sl = torch.full((R,), ctx, device="cuda", dtype=torch.int32)
        md = AttentionMetadata(R, R, qsl, sl, bt, None, None, 1, ctx, query_lens_cpu=[1] * R, seq_lens_cpu=[ctx] * R)
        ms = timeit(lambda: K.mla_decode(q_abs, q_pe, cache, md, 192 ** -0.5, lora), 1 if small else iters, 1 if small else 3)
        b = R * ctx * (lora + rope) * 2
        rows.append(dict(kernel="mla_decode", R=R, ctx=ctx, heads=H, ms=ms, latent_gbs=b / ms / 1e6, frac_of_hbm=b / ms / 1e6 / pk["hbm_gbs"],
                         tflops=2.0 * R * H * ctx * (2 * lora + rope) / ms / 1e9))


def bench_rope(rows: list, small: bool, iters: int, pk: dict) -> None:
    """q/k RMSNorm + rotary embedding in place + K/V insert into the paged cache (one kernel), 40 q / 8 kv heads of 128."""
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    Hq, Hkv, D, bs = 40, 8, 128, 16
    cs = ref.build_cos_sin_cache(D, 40960, 1e6, "cuda")
    for T in ([8192] if small else [64, 1088, 8192]):
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
        q, k, v = qkv[:, :Hq * D].view(T, Hq, D), qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D), qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
        nb = T // bs + 2
        cache = torch.zeros(nb, 2, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
        pos = torch.arange(T, device="cuda", dtype=torch.int32)
        slots = torch.randperm(T, device="cuda").to(torch.int32) + bs
        qn, kn = torch.ones(D, device="cuda").bfloat16(), torch.ones(D, device="cuda").bfloat16()
        ms = timeit(lambda: K.rope_and_cache(q, k, v, pos, cs, cache, slots, D, qn, kn, 1e-6, False), 1 if small else iters, 1 if small else 3)
        b = T * D * 2 * (2 * (Hq + Hkv) + Hkv + 2 * Hkv)   # q, k read and written; v read; k, v written to the cache
        rows.append(dict(kernel="rope_qknorm_cache_insert", T=T, ms=ms, gbs=b / ms / 1e6, frac_of_hbm=b / ms / 1e6 / pk["hbm_gbs"]))


def bench_reject(rows: list, small: bool, iters: int, pk: dict) -> None:
    """Rejection sampler over [B, k+1, V] target logits (greedy and stochastic), vocabulary 151936, three drafts."""
    from onecat_vllm.sample.metadata import SamplingMetadata
    from onecat_vllm.sample.rejection_sampler import RejectionSampler
    V, k = 151936, 3
    for B in ([64] if small else [8, 64, 256]):
        tl = torch.randn(B, k + 1, V, device="cuda").bfloat16()
        draft = tl.float().argmax(-1)[:, :k].contiguous()
        nd = torch.full((B,), k, device="cuda")
        bonus = torch.full((B,), 7, device="cuda")
        for greedy in ((True,) if small else (True, False)):
            md = SamplingMetadata(temperature=None if greedy else torch.ones(B, device="cuda"), all_greedy=greedy, all_random=not greedy, top_p=None,
                                  top_k=None, min_p=None, generators={}, max_num_logprobs=None, no_penalties=True)
            rs = RejectionSampler(seed=1)
            ms = timeit(lambda: rs(draft, nd, tl, bonus, md), 1 if small else iters, 1 if small else 3)
            b = B * (k + 1) * V * 2
            rows.append(dict(kernel="rejection_sample", B=B, drafts=k, V=V, greedy=greedy, ms=ms, logits_gbs=b / ms / 1e6,
                             frac_of_hbm=b / ms / 1e6 / pk["hbm_gbs"]))


def bench_sample(rows: list, small: bool, iters: int, pk: dict) -> None:
    """The fused sampler against the sort-based PyTorch formulation on the same device (vocabulary 151936)."""
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.ops import ref
    V = 151936
    for B in ([64] if small else [1, 64, 256]):
        lg = torch.randn(B, V, device="cuda") * 2.0
        t = torch.full((B,), 0.8, device="cuda")
        k = torch.full((B,), 50, device="cuda", dtype=torch.int64)
        pp = torch.full((B,), 0.9, device="cuda")
        seeds = torch.randint(0, 1 << 62, (B,), dtype=torch.int64, device="cuda")
        from onecat_vllm.ops import _C
        k32 = k.to(torch.int32)
        ms = timeit(lambda: _C.sample(lg, t, k32, pp, None, seeds, None), 1 if small else iters, 1 if small else 3)

        def torch_way():
            x = ref.top_k_top_p_min_p(lg / t.unsqueeze(-1), k, pp, None)
            return ref.random_sample(torch.softmax(x, -1), {})
        ms_t = timeit(torch_way, 1 if small else iters, 1 if small else 3)
        rows.append(dict(kernel="sample_topk_topp", B=B, V=V, top_k=50, top_p=0.9, ms=ms, torch_sort_ms=ms_t, speedup=ms_t / ms,
                         l2_gbs=10 * B * V * 4 / ms / 1e6))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    pk = _peaks()
    rows: list = []
    for name, fn in (("gemm", bench_gemm), ("w4", bench_w4), ("attn", bench_attn), ("norm", bench_norm), ("gdn", bench_gdn), ("moe", bench_moe), ("wq", bench_wq), ("sample", bench_sample), ("mla", bench_mla), ("w4tp", bench_w4_tp),
                     ("rope", bench_rope), ("reject", bench_reject),
                     ("attn_prefill", lambda r, s_, i, p_: bench_attn(r, s_, i, p_, prefill_only=True)),
                     ("gdn_prefill", lambda r, s_, i, p_: bench_gdn(r, s_, i, p_, prefill_only=True))):
        if not a.only and name in ("attn_prefill", "gdn_prefill", "w4tp"):
            continue
        if a.only and a.only != name:
            continue
        fn(rows, a.small, a.iters, pk)
    from onecat_vllm.ops import cuda as K
    res = {"peaks": pk, "rows": rows, "device_status": K.check_status()}
    for r in rows:
        print(json.dumps(r))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(res, f, indent=1)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
    main()
