"""Numerics of the sm_100a kernels against the fp32 PyTorch restatements in ``onecat_vllm.ops.ref``."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from onecat_vllm.ops import ref


def K():
    from onecat_vllm.ops import cuda
    return cuda


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, rtol, atol, what=""):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} mismatches, max err {float(err.max()):.4g} at {int(err.argmax())}"


@pytest.mark.parametrize("T,H", [(1, 2048), (5, 5120), (127, 7168), (300, 512)])
@pytest.mark.parametrize("gemma", [False, True])
def test_rms_norm(T, H, gemma):
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    r = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    w = (torch.randn(H, device="cuda", generator=g) * 0.1 + (0 if gemma else 1)).bfloat16()
    y, ro = K().rms_norm(x, w, 1e-6, r, gemma)
    ye, re = ref.rms_norm(x.cpu(), w.cpu(), 1e-6, r.cpu(), gemma)
    _close(ro, re, 0, 0, "residual")
    _close(y, ye, 2e-2, 2e-2, "normed")
    y2, none = K().rms_norm(x, w, 1e-6, None, gemma)
    assert none is None
    _close(y2, ref.rms_norm(x.cpu(), w.cpu(), 1e-6, None, gemma)[0], 2e-2, 2e-2)
    assert K().check_status() == 0


def test_silu_and_mul_and_argmax():
    x = torch.randn(33, 2 * 1408, device="cuda").bfloat16()
    _close(K().silu_and_mul(x), ref.silu_and_mul(x.cpu()), 1e-2, 1e-2)
    lg = torch.randn(7, 151936, device="cuda").bfloat16()
    lg[3, 777] = 100.0
    assert K().argmax(lg).tolist() == lg.float().argmax(-1).tolist()
    lf = torch.randn(5, 32000, device="cuda")
    assert K().argmax(lf).tolist() == lf.argmax(-1).tolist()


@pytest.mark.parametrize("D,rot,qk_norm,gated", [(128, 128, False, False), (256, 64, True, True), (128, 64, True, False)])
def test_rope_and_cache(D, rot, qk_norm, gated):
    T, Hq, Hkv, bs, nb = 37, 6, 2, 16, 12
    g = torch.Generator(device="cuda").manual_seed(1)
    width = Hq * D * (2 if gated else 1) + 2 * Hkv * D
    qkv = torch.randn(T, width, device="cuda", generator=g).bfloat16()
    qw = Hq * D * (2 if gated else 1)
    q = qkv[:, :qw].view(T, Hq, 2 * D)[..., :D] if gated else qkv[:, :qw].view(T, Hq, D)
    k = qkv[:, qw:qw + Hkv * D].view(T, Hkv, D)
    v = qkv[:, qw + Hkv * D:].view(T, Hkv, D)
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cs = ref.build_cos_sin_cache(rot, 512, 1e6, "cuda")
    cache = torch.zeros(nb, 2, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
    slots[5] = -1
    qn = (torch.randn(D, device="cuda") * 0.1).bfloat16() if qk_norm else None
    kn = (torch.randn(D, device="cuda") * 0.1).bfloat16() if qk_norm else None
    qkv_c = qkv.cpu().clone()
    q_c = qkv_c[:, :qw].view(T, Hq, 2 * D)[..., :D] if gated else qkv_c[:, :qw].view(T, Hq, D)
    k_c = qkv_c[:, qw:qw + Hkv * D].view(T, Hkv, D)
    v_c = qkv_c[:, qw + Hkv * D:].view(T, Hkv, D)
    cache_c = cache.cpu().clone()
    ref.rope_and_cache(q_c, k_c, v_c, pos.cpu(), cs.cpu(), cache_c, slots.cpu(), rot, qn.cpu() if qk_norm else None,
                       kn.cpu() if qk_norm else None, 1e-6, True)
    K().rope_and_cache(q, k, v, pos, cs, cache, slots, rot, qn, kn, 1e-6, True)
    _close(qkv, qkv_c, 2e-2, 2e-2, "q/k in place")
    _close(cache, cache_c, 2e-2, 2e-2, "cache")
    assert K().check_status() == 0


def test_rope_with_rotary_sections():
    """Positions [3, T] (temporal, height, width) with the frequencies split into sections, rows of a wider buffer."""
    T, Hq, Hkv, D, bs, nb = 45, 4, 2, 128, 16, 8
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(T, Hq, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(T, Hkv, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(T, Hkv, D, device="cuda", generator=g).bfloat16()
    wide = torch.randint(0, 500, (3, 64), device="cuda", dtype=torch.int32, generator=g)
    pos3 = wide[:, :T]                                  # row stride 64, as the runner's staging buffer gives it
    cs = ref.build_cos_sin_cache(D, 512, 1e4, "cuda")
    cache = torch.zeros(nb, 2, Hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
    qc, kc, vc, cache_c = q.cpu().clone(), k.cpu().clone(), v.cpu().clone(), cache.cpu().clone()
    sec = (16, 24, 24)
    ref.rope_and_cache(qc, kc, vc, pos3.cpu(), cs.cpu(), cache_c, slots.cpu(), D, None, None, 1e-6, False, sec)
    K().rope_and_cache(q, k, v, pos3, cs, cache, slots, D, None, None, 1e-6, False, sec)
    _close(q, qc, 2e-2, 2e-2, "q")
    _close(cache, cache_c, 2e-2, 2e-2, "cache")
    # the sections matter: the temporal row alone gives another rotation
    q1 = qc.clone()
    assert K().check_status() == 0
    q2 = torch.randn(T, Hq, D, generator=torch.Generator().manual_seed(4)).bfloat16()
    ref.rope_and_cache(q2, kc.clone(), vc.clone(), pos3[0].cpu(), cs.cpu(), None, slots.cpu(), D)
    assert not torch.equal(q1, q2)


def _ref_gemm(x, w):
    return x.float().cpu() @ w.float().cpu().t()


@pytest.mark.parametrize("T", [1, 5, 64, 127, 129, 300, 1000])
@pytest.mark.parametrize("N,Kd", [(128, 64), (384, 256), (5120, 5120)])
def test_gemm_bf16(T, N, Kd):
    g = torch.Generator(device="cuda").manual_seed(T * 7 + N)
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, Kd, device="cuda", generator=g) * 0.05).bfloat16()
    y = K().gemm_bf16(x, w)
    torch.cuda.synchronize()
    assert K().check_status() == 0, "a bounded device wait expired"
    _close(y, _ref_gemm(x, w), 2e-2, 2e-2 * math.sqrt(Kd) * 0.05, f"gemm {T}x{N}x{Kd}")


@pytest.mark.parametrize("splits,tn", [(2, 0), (5, 0), (1, 32), (3, 128)])
def test_gemm_bf16_splitk_and_tiles(splits, tn):
    T, N, Kd = 70, 640, 1280
    x = torch.randn(T, Kd, device="cuda").bfloat16()
    w = (torch.randn(N, Kd, device="cuda") * 0.05).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    if tn and tn < T:
        tn = 0
    y = K().gemm_bf16(x, w, bias=b, force_splits=splits, force_tn=tn)
    y2 = K().gemm_bf16(x, w, bias=b, force_splits=splits, force_tn=tn)  # counters must be back to zero
    torch.cuda.synchronize()
    assert K().check_status() == 0
    e = _ref_gemm(x, w) + b.float().cpu()
    _close(y, e, 2e-2, 5e-2, "split-k")
    assert torch.equal(y, y2), "split-K reduction must be bit-stable across launches"


class _FakeLayer:
    def __init__(self, fuse):
        self.fuse_silu_mul = fuse
        self.bias = None
        self.kernel_state = None


@pytest.mark.parametrize("T", [1, 8, 64, 200, 700])
@pytest.mark.parametrize("fuse", [False, True])
def test_gemm_w4(T, fuse):
    N, Kd, grp = 1024, 768 if not fuse else 640, 128
    if Kd % grp:
        Kd = 768
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randint(0, 16, (N, Kd), device="cuda", generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (N, Kd // grp), device="cuda", generator=g, dtype=torch.uint8)
    s = (torch.randn(N, Kd // grp, device="cuda", generator=g).abs() * 0.01 + 1e-3).half()
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    layer = _FakeLayer(fuse)
    K().prepare_w4(layer, q, z, s, grp)
    y = K().linear(layer, x)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    wd = (q.float() - z.float().repeat_interleave(grp, 1)) * s.float().bfloat16().float().repeat_interleave(grp, 1)
    wd = wd.bfloat16().float().cpu()
    e = x.float().cpu() @ wd.t()
    if fuse:
        e = torch.nn.functional.silu(e[:, : N // 2]) * e[:, N // 2:]
    _close(y, e, 3e-2, 3e-2, f"w4 T={T} fuse={fuse}")


@pytest.mark.parametrize("T", [1, 16, 33, 64])
@pytest.mark.parametrize("N,Kd,fuse", [(896, 5120, False), (5120, 640, False), (256, 1024, False), (4352, 5120, True), (1024, 384, True)])
def test_gemm_w4_cluster_splitk(T, N, Kd, fuse):
    """Decode-sized 4-bit GEMMs whose k range is split over a thread-block cluster (2 to 8 CTAs per tile, partials summed through
    distributed shared memory): against the fp32 oracle, bit-identical across launches, status word clean."""
    grp = 128
    g = torch.Generator(device="cuda").manual_seed(N + Kd + T)
    q = torch.randint(0, 16, (N, Kd), device="cuda", generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (N, Kd // grp), device="cuda", generator=g, dtype=torch.uint8)
    s = (torch.randn(N, Kd // grp, device="cuda", generator=g).abs() * 0.01 + 1e-3).half()
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    layer = _FakeLayer(fuse)
    K().prepare_w4(layer, q, z, s, grp)
    y = K().linear(layer, x).clone()
    y2 = K().linear(layer, x).clone()
    torch.cuda.synchronize()
    assert K().check_status() == 0
    wd = (q.float() - z.float().repeat_interleave(grp, 1)) * s.float().bfloat16().float().repeat_interleave(grp, 1)
    e = x.float().cpu() @ wd.bfloat16().float().cpu().t()
    if fuse:
        e = torch.nn.functional.silu(e[:, : N // 2]) * e[:, N // 2:]
    _close(y, e, 3e-2, 3e-2 * math.sqrt(Kd / 768), f"w4 cluster T={T} N={N} K={Kd}")
    assert torch.equal(y, y2), "the cluster reduction sums in split order: launches must agree bit for bit"


class _Fp8Layer(_FakeLayer):
    pass


@pytest.mark.parametrize("T", [1, 64, 200, 700])
@pytest.mark.parametrize("fuse,block", [(False, (128, 128)), (True, (128, 128)), (False, None)])
def test_gemm_fp8_weight_only(T, fuse, block):
    """FP8 e4m3 weights (block-scaled 128x128, or one scale per merged output) dequantised inside the GEMM, against the fp32
    product with the dequantised weights. All 256 byte patterns except NaN occur, e4m3 subnormals included."""
    N, Kd = 1024, 768
    g = torch.Generator(device="cuda").manual_seed(5)
    codes = torch.randint(0, 256, (N, Kd), device="cuda", generator=g, dtype=torch.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x3C  # no NaN patterns
    w8 = codes.view(torch.float8_e4m3fn)
    layer = _Fp8Layer(fuse)
    layer.weight = torch.nn.Parameter(w8.clone(), requires_grad=False)
    if block:
        sc = torch.rand(N // 128, Kd // 128, device="cuda", generator=g) * 2e-4 + 1e-5
        layer.weight_scale_inv = torch.nn.Parameter(sc, requires_grad=False)
        wd = ref.fp8_block_dequantize(w8, sc, block)
    else:
        layer.local_output_sizes = [N // 2, N // 2]
        sc = torch.tensor([3e-4, 1e-4], device="cuda")
        layer.weight_scale = torch.nn.Parameter(sc, requires_grad=False)
        wd = torch.cat([w8[: N // 2].float() * sc[0], w8[N // 2:].float() * sc[1]])
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    K().prepare_fp8(layer, block)
    assert layer.kernel_state["wkind"] == 2 and not hasattr(layer, "weight")
    y = K().linear(layer, x)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    sb = (sc if block else sc.view(2, 1)).float() * 2.0 ** 120
    # the kernel multiplies by the bf16-rounded scale and rounds the weight to bf16
    rs = (sb.bfloat16().float() / 2.0 ** 120)
    if block:
        wk = ref.fp8_block_dequantize(w8, rs, block)
    else:
        wk = torch.cat([w8[: N // 2].float() * rs[0], w8[N // 2:].float() * rs[1]])
    e = x.float().cpu() @ wk.bfloat16().float().cpu().t()
    if fuse:
        e = torch.nn.functional.silu(e[:, : N // 2]) * e[:, N // 2:]
    _close(y, e, 3e-2, 3e-2, f"fp8 T={T} fuse={fuse} block={block}")
    # and stays close to the exact-scale product
    e2 = x.float().cpu() @ wd.float().cpu().t()
    if fuse:
        e2 = torch.nn.functional.silu(e2[:, : N // 2]) * e2[:, N // 2:]
    _close(y, e2, 5e-2, 5e-2, "fp8 vs exact scales")


@pytest.mark.parametrize("T", [1, 64, 300])
@pytest.mark.parametrize("fuse", [False, True])
def test_gemm_mxfp4_weight_only(T, fuse):
    """MXFP4 (e2m1 nibbles, one ue8m0 scale per 32 k) dequantised inside the GEMM: every nibble value, 0.5 included, and scales
    over a range of exponents; exact in bf16, so only accumulation order differs from the fp32 product."""
    N, Kd = 512, 640
    g = torch.Generator(device="cuda").manual_seed(6)
    packed = torch.randint(0, 256, (N, Kd // 2), device="cuda", generator=g, dtype=torch.uint8)
    sc = torch.randint(110, 124, (N, Kd // 32), device="cuda", generator=g, dtype=torch.uint8)
    layer = _FakeLayer(fuse)
    layer.weight = torch.nn.Parameter(packed.clone(), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(sc.clone(), requires_grad=False)
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    K().prepare_fp4(layer, "mxfp4")
    assert layer.kernel_state["wkind"] == 3
    y = K().linear(layer, x)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    wd = ref.mxfp4_dequantize(packed, sc)
    e = x.float().cpu() @ wd.float().cpu().t()
    if fuse:
        e = torch.nn.functional.silu(e[:, : N // 2]) * e[:, N // 2:]
    _close(y, e, 2e-2, 2e-2, f"mxfp4 T={T} fuse={fuse}")


@pytest.mark.parametrize("T", [1, 64, 300])
@pytest.mark.parametrize("fuse", [False, True])
def test_gemm_nvfp4_weight_only(T, fuse):
    """NVFP4 (e2m1 nibbles, one e4m3 scale per 16 k, one fp32 global scale) dequantised inside the GEMM."""
    N, Kd = 512, 640
    g = torch.Generator(device="cuda").manual_seed(7)
    packed = torch.randint(0, 256, (N, Kd // 2), device="cuda", generator=g, dtype=torch.uint8)
    sc = (torch.rand(N, Kd // 16, device="cuda", generator=g) * 3 + 0.25).to(torch.float8_e4m3fn)
    gs = torch.tensor([0.0123], device="cuda")
    layer = _FakeLayer(fuse)
    layer.weight = torch.nn.Parameter(packed.clone(), requires_grad=False)
    layer.weight_scale = torch.nn.Parameter(sc.clone(), requires_grad=False)
    layer.weight_scale_2 = torch.nn.Parameter(gs.clone(), requires_grad=False)
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    K().prepare_fp4(layer, "nvfp4")
    assert layer.kernel_state["wkind"] == 4 and not hasattr(layer, "weight")
    y = K().linear(layer, x)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    # the kernel multiplies by bf16(scale * global): dequantise with that rounding for the tight comparison
    sr = ((sc.float() * gs) * 2.0 ** 126).bfloat16().float() / 2.0 ** 126
    wd = ref.fp4_unpack(packed) * sr.repeat_interleave(16, dim=-1)
    e = x.float().cpu() @ wd.bfloat16().float().cpu().t()
    if fuse:
        e = torch.nn.functional.silu(e[:, : N // 2]) * e[:, N // 2:]
    _close(y, e, 3e-2, 3e-2 * float(e.abs().max()) / 10, f"nvfp4 T={T} fuse={fuse}")
    e2 = x.float().cpu() @ ref.nvfp4_dequantize(packed, sc, gs).float().cpu().t()
    if fuse:
        e2 = torch.nn.functional.silu(e2[:, : N // 2]) * e2[:, N // 2:]
    assert float((y.float().cpu() - e2).abs().max()) < 2e-2 * float(e2.abs().max()), "nvfp4 vs exact scales"


@pytest.mark.parametrize("kind", ["fp8", "mxfp4"])
@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (40, 32, 8), (300, 8, 2)])
def test_fused_moe_packed_experts(kind, T, E, k):
    """Grouped GEMMs over packed FP8 (128x128 block scales) / MXFP4 expert weights against per-expert fp32 FFNs on the
    dequantised weights."""
    H, I = 256, 128
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.5).bfloat16()
    logits = torch.randn(T, E, device="cuda", generator=g)
    tw, ti = ref.topk_softmax(logits, k, True)

    class M:
        pass
    m = M()
    m.qmethod, m.E_local, m.e_off, m._dq, m.block = kind, E, 0, None, (128, 128)
    if kind == "fp8":
        c13 = torch.randint(0, 256, (E, 2 * I, H), device="cuda", generator=g, dtype=torch.uint8)
        c2 = torch.randint(0, 256, (E, H, I), device="cuda", generator=g, dtype=torch.uint8)
        for c in (c13, c2):
            c[(c & 0x7F) == 0x7F] = 0x30
            c &= 0xBF  # keep |w| < 2 so the FFN output stays in a sane range
        m.w13, m.w2 = c13.view(torch.float8_e4m3fn), c2.view(torch.float8_e4m3fn)
        m.w13_scale = torch.rand(E, 2 * I // 128, H // 128, device="cuda", generator=g) * 0.05 + 0.01
        m.w2_scale = torch.rand(E, H // 128, I // 128, device="cuda", generator=g) * 0.05 + 0.01
        w13 = ref.fp8_block_dequantize(m.w13, m.w13_scale, m.block)
        w2 = ref.fp8_block_dequantize(m.w2, m.w2_scale, m.block)
    else:
        m.w13 = torch.randint(0, 256, (E, 2 * I, H // 2), device="cuda", generator=g, dtype=torch.uint8)
        m.w2 = torch.randint(0, 256, (E, H, I // 2), device="cuda", generator=g, dtype=torch.uint8)
        m.w13_scale = torch.randint(118, 122, (E, 2 * I, H // 32), device="cuda", generator=g, dtype=torch.uint8)
        m.w2_scale = torch.randint(118, 122, (E, H, I // 32), device="cuda", generator=g, dtype=torch.uint8)
        w13, w2 = ref.mxfp4_dequantize(m.w13, m.w13_scale), ref.mxfp4_dequantize(m.w2, m.w2_scale)
    K().prepare_moe(m)
    assert m.kernel_state is not None and m.kernel_state["wkind"] == (2 if kind == "fp8" else 3) and not hasattr(m, "w13")
    y = K().fused_moe(m, x, tw, ti)
    torch.cuda.synchronize()
    assert K().check_status() == 0 and "fused_moe" not in K().TORCH_STANDINS
    e = ref.fused_experts(x.cpu(), w13.float().cpu(), w2.float().cpu(), tw.cpu(), ti.cpu(), 0)
    _close(y, e, 4e-2, 1e-2, f"moe {kind} T={T} E={E}")


def test_awq_layer_matches_reference_dequant():
    """AWQ checkpoint layout (int32 [K, N/8], nibble order 0,4,1,5,2,6,3,7) through the layer's repacking."""
    from onecat_vllm.config import QuantConfig
    from onecat_vllm.layers.linear import MergedColumnParallelLinear
    Kd, I = 512, 256
    with torch.device("cuda"):
        layer = MergedColumnParallelLinear(Kd, [I, I], quant=QuantConfig("awq"), prefix="mlp.gate_up_proj", dtype=torch.bfloat16, fuse_silu_mul=True)
    g = torch.Generator(device="cuda").manual_seed(5)
    layer.qweight.data = torch.randint(-2 ** 31, 2 ** 31 - 1, layer.qweight.shape, device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    layer.qzeros.data = torch.randint(-2 ** 31, 2 ** 31 - 1, layer.qzeros.shape, device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
    layer.scales.data = (torch.randn(layer.scales.shape, device="cuda", generator=g).abs() * 0.01 + 1e-3).half()
    wd = ref.awq_dequantize(layer.qweight.cpu(), layer.qzeros.cpu(), layer.scales.cpu().float().bfloat16().float(), 128).t()
    layer.process_weights_after_loading()
    x = torch.randn(19, Kd, device="cuda", generator=g).bfloat16()
    y = layer(x)
    e = x.float().cpu() @ wd.float().bfloat16().float().t()
    e = torch.nn.functional.silu(e[:, :I]) * e[:, I:]
    _close(y, e, 3e-2, 3e-2, "awq layer")


def _attn_case(qlens, ctxs, Hq, Hkv, D, bs=16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    R = len(qlens)
    seq = [c + q for q, c in zip(qlens, ctxs)]
    nb_per = [-(-s // bs) for s in seq]
    total = sum(nb_per) + 3
    perm = torch.randperm(total, device="cuda", generator=g).to(torch.int32)
    bt = torch.zeros(R, max(nb_per) + 2, dtype=torch.int32, device="cuda")
    o = 0
    for r, n in enumerate(nb_per):
        bt[r, :n] = perm[o:o + n]
        o += n
    cache = (torch.randn(total, 2, Hkv, bs, D, device="cuda", generator=g) * 0.5).bfloat16()
    T = sum(qlens)
    q = (torch.randn(T, Hq, D, device="cuda", generator=g) * 0.5).bfloat16()
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
    sl = torch.tensor(seq, dtype=torch.int32, device="cuda")
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    md = AttentionMetadata(R, T, qsl, sl, bt, torch.zeros(T, dtype=torch.int32, device="cuda"), torch.zeros(T, dtype=torch.int32, device="cuda"),
                           max(qlens), max(seq), query_lens_cpu=list(qlens), seq_lens_cpu=seq)
    return q, cache, md


@pytest.mark.parametrize("name,qlens,ctxs,Hq,Hkv,D", [
    ("decode", [1] * 9, [0, 15, 16, 63, 64, 300, 1000, 2047, 5], 40, 8, 128),
    ("verify4", [4] * 5, [10, 100, 777, 64, 60], 40, 8, 128),
    ("prefill", [1, 17, 200, 64], [0, 0, 0, 0], 8, 2, 128),
    ("chunked-prefix", [130, 33], [256, 1000], 10, 2, 128),
    ("mixed", [1, 1, 300, 1, 2], [500, 20, 100, 0, 77], 40, 8, 128),
    ("prefill-long", [700, 129, 128], [0, 300, 1], 40, 8, 128),
    ("decode-d256", [1] * 4, [0, 100, 1025, 31], 24, 4, 256),
    ("decode-d64", [1] * 5, [0, 100, 1025, 31, 4000], 32, 8, 64),
    ("verify-d64", [4] * 3, [10, 600, 2000], 16, 4, 64),
    ("prefill-d64", [300, 70, 513, 1], [0, 200, 64, 77], 32, 8, 64),
    ("prefill-d256", [77, 5, 140], [0, 200, 64], 16, 2, 256),
    ("verify-d256", [4, 4], [100, 3], 24, 4, 256),
])
def test_paged_attention(name, qlens, ctxs, Hq, Hkv, D):
    q, cache, md = _attn_case(qlens, ctxs, Hq, Hkv, D)
    scale = D ** -0.5
    out = K().paged_attention(q, cache, md, scale)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    e = ref.paged_attention(q.cpu(), cache.cpu(), md.block_table.cpu(), md.query_start_loc.cpu(), md.seq_lens.cpu(), scale)
    _close(out, e, 2e-2, 1e-2, name)


def test_prefill_attention_tcgen05_matches_mma_path_and_lse(monkeypatch):
    """Head size 128 prefill runs on the tcgen05 kernel by default; it must agree with the mma.sync kernel and return the
    same log-sum-exp."""
    import onecat_vllm.ops.cuda as KC
    q, cache, md = _attn_case([300, 70, 513], [0, 200, 64], 16, 4, 128, seed=3)
    T = q.shape[0]
    lse_tc = torch.zeros(T, 16, device="cuda")
    lse_mma = torch.zeros(T, 16, device="cuda")
    out_tc = KC.paged_attention(q, cache, md, 128 ** -0.5, lse=lse_tc)
    monkeypatch.setattr(KC, "_ATTN_PREFILL_TC", False)
    out_mma = KC.paged_attention(q, cache, md, 128 ** -0.5, lse=lse_mma)
    torch.cuda.synchronize()
    assert KC.check_status() == 0
    assert (out_tc.float() - out_mma.float()).abs().max() < 2e-2
    assert (lse_tc - lse_mma).abs().max() < 2e-2


@pytest.mark.parametrize("name,qlens,ctxs,Hq,Hkv,D,window,softcap,use_sinks", [
    ("window-decode", [1] * 6, [0, 100, 127, 128, 1000, 4000], 16, 4, 128, 128, 0.0, False),
    ("window-prefill", [300, 70, 513, 1], [0, 200, 64, 700], 16, 4, 128, 64, 0.0, False),
    ("window-verify-d256", [4] * 3, [10, 600, 2000], 8, 2, 256, 512, 0.0, False),
    ("softcap", [1, 1, 200, 3], [500, 20, 100, 77], 16, 4, 256, 0, 50.0, False),
    ("sinks", [1, 1, 300, 1, 2], [5000, 20, 100, 0, 77], 64, 8, 128, 0, 0.0, True),
    ("window+sinks", [1, 1, 300, 1], [5000, 130, 100, 0], 64, 8, 128, 128, 0.0, True),
])
def test_paged_attention_window_softcap_sinks(name, qlens, ctxs, Hq, Hkv, D, window, softcap, use_sinks):
    """Sliding window, tanh soft-capping and attention sinks (Gemma / GPT-OSS / Mistral families) against the fp32 oracle, over the
    decode (split-KV + combine), verify and prefill forms of the kernel."""
    q, cache, md = _attn_case(qlens, ctxs, Hq, Hkv, D, seed=7)
    sinks = torch.randn(Hq, device="cuda") * 2.0 if use_sinks else None
    scale = D ** -0.5 * 4.0   # larger scores so that capping and sinks move the result
    out = K().paged_attention(q, cache, md, scale, window=window, softcap=softcap, sinks=sinks)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    e = ref.paged_attention(q.cpu(), cache.cpu(), md.block_table.cpu(), md.query_start_loc.cpu(), md.seq_lens.cpu(), scale,
                            window=window, softcap=softcap, sinks=None if sinks is None else sinks.cpu())
    _close(out, e, 2e-2, 1e-2, name)
    if window:
        full = ref.paged_attention(q.cpu(), cache.cpu(), md.block_table.cpu(), md.query_start_loc.cpu(), md.seq_lens.cpu(), scale)
        assert (full.float() - e.float()).abs().max() > 1e-2   # the window changes the answer in these cases


def test_fp8_kv_cache_store_and_attention():
    """An e4m3 KV cache: the rope + insert kernel stores saturated e4m3 bytes equal to the oracle's, and decode, verify and prefill
    attention over such a cache match the fp32 oracle reading the same bytes."""
    T, Hq, Hkv, D, bs, nb = 50, 8, 2, 128, 16, 10
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(T, Hq, D, device="cuda", generator=g).bfloat16()
    k = (torch.randn(T, Hkv, D, device="cuda", generator=g) * 3).bfloat16()
    v = (torch.randn(T, Hkv, D, device="cuda", generator=g) * 300).bfloat16()   # some values saturate at 448
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    cs = ref.build_cos_sin_cache(D, 512, 1e6, "cuda")
    cache = torch.zeros(nb, 2, Hkv, bs, D, device="cuda", dtype=torch.float8_e4m3fn)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
    qc, kc, vc, cache_c = q.cpu().clone(), k.cpu().clone(), v.cpu().clone(), cache.cpu().clone()
    ref.rope_and_cache(qc, kc, vc, pos.cpu(), cs.cpu(), cache_c, slots.cpu(), D)
    K().rope_and_cache(q, k, v, pos, cs, cache, slots, D, None, None, 1e-6, False)
    torch.cuda.synchronize()
    a, b = cache.cpu().view(torch.uint8).int(), cache_c.view(torch.uint8).int()
    # k goes through a bf16 rotation on both sides: allow the last e4m3 step on a handful of values
    assert ((a - b).abs() <= 1).all() and (a != b).float().mean() < 0.01
    assert (a[:, 1] == b[:, 1]).all()
    for name, qlens, ctxs, hq, hkv, d in [("decode", [1] * 5, [0, 100, 1000, 3000, 63], 40, 8, 128), ("verify", [4] * 3, [10, 600, 2000], 8, 2, 256),
                                          ("prefill", [300, 70, 513], [0, 200, 64], 16, 4, 128), ("prefill-d256", [200, 3], [100, 77], 8, 2, 256),
                                          ("mixed-d64", [1, 200, 3], [900, 100, 77], 16, 4, 64)]:
        qq, cache_bf, md = _attn_case(qlens, ctxs, hq, hkv, d, seed=5)
        c8 = cache_bf.to(torch.float8_e4m3fn)
        out = K().paged_attention(qq, c8, md, d ** -0.5)
        torch.cuda.synchronize()
        assert K().check_status() == 0
        e = ref.paged_attention(qq.cpu(), c8.cpu(), md.block_table.cpu(), md.query_start_loc.cpu(), md.seq_lens.cpu(), d ** -0.5)
        _close(out, e, 2e-2, 1e-2, name)


def test_fp8_kv_cache_values_are_read_exactly():
    """With a single key the attention output is that key's value row: every finite e4m3 code (subnormals included) must come back
    as exactly its value."""
    D, bs = 128, 16
    codes = torch.tensor([c for c in range(256) if c & 0x7f != 0x7f], dtype=torch.uint8)   # 0x7f / 0xff are NaN
    rows = -(-codes.numel() // D)
    pad = torch.zeros(rows * D, dtype=torch.uint8)
    pad[: codes.numel()] = codes
    cache = torch.zeros(rows, 2, 1, bs, D, dtype=torch.uint8, device="cuda")
    cache[:, 1, 0, 0, :] = pad.view(rows, D).cuda()
    c8 = cache.view(torch.float8_e4m3fn)
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    q = torch.randn(rows, 1, D, device="cuda").bfloat16()
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    sl = torch.ones(rows, dtype=torch.int32, device="cuda")
    bt = torch.arange(rows, dtype=torch.int32, device="cuda").view(rows, 1)
    md = AttentionMetadata(rows, rows, qsl, sl, bt, None, None, 1, 1, query_lens_cpu=[1] * rows, seq_lens_cpu=[1] * rows)
    out = K().paged_attention(q, c8, md, D ** -0.5)
    torch.cuda.synchronize()
    want = pad.view(torch.float8_e4m3fn).float().view(rows, D)
    assert torch.equal(out.float().cpu().view(rows, D), want)


def test_sampler_kernel_filters_and_draws():
    """The fused sampler: the set of tokens kept by min-p / top-k / top-p equals the sort-based oracle's, draws follow the
    filtered softmax, temperature ~ 0 rows take the arg-max and a seeded generator repeats its draw."""
    B, V = 12, 5000
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = torch.randn(B, V, device="cuda", generator=g) * 3.0
    temp = torch.tensor([1.0, 0.7, 1.3, 1.0, 0.5, 1.0, 2.0, 1.0, 0.0, 1.0, 0.9, 1.0], device="cuda")
    top_k = torch.tensor([0, 50, 0, 7, 0, 1000, 3, 0, 5, V + 5, 20, 1], device="cuda")
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 1.0, 0.8, 1.0, 0.3, 0.9, 0.99, 0.6, 1.0], device="cuda")
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.05, 0.0, 0.0, 0.01, 0.0, 0.0, 0.02, 0.0], device="cuda")
    kept = torch.zeros(B, V, dtype=torch.uint8, device="cuda")
    out = K().sample(logits, temp, top_k, top_p, min_p, None, kept)
    torch.cuda.synchronize()
    scaled = (logits / torch.where(temp < 1e-5, torch.ones_like(temp), temp).unsqueeze(-1)).cpu()
    want = ref.top_k_top_p_min_p(scaled, top_k.cpu(), top_p.cpu(), min_p.cpu())
    want_kept = torch.isfinite(want)
    for r in range(B):
        if temp[r] < 1e-5:
            assert out[r].item() == logits[r].argmax().item()
            continue
        diff = (kept[r].cpu().bool() != want_kept[r]).sum().item()
        # a token whose cumulative mass sits within rounding of the nucleus boundary may fall on either side
        assert diff <= 1, (r, diff, int(kept[r].sum()), int(want_kept[r].sum()))
        assert kept[r, out[r]].item() == 1
    assert out[11].item() == logits[11].argmax().item()        # top_k = 1
    # distribution: many draws of one filtered row against its softmax
    row = logits[3:4].expand(4000, V).contiguous()
    draws = K().sample(row, torch.ones(4000, device="cuda"), torch.full((4000,), 7, device="cuda"), None, None, None, None)
    probs = torch.softmax(ref.top_k_top_p_min_p(scaled[3:4], torch.tensor([7]), None, None)[0], -1)
    freq = torch.bincount(draws.cpu(), minlength=V).float() / 4000
    assert (freq > 0).sum() <= 7 and (freq - probs).abs().max() < 0.04
    # a seeded request repeats; an unseeded one (almost surely) does not give the same 64 draws twice
    flat = torch.zeros(64, V, device="cuda")
    g1, g2 = torch.Generator(device="cuda").manual_seed(9), torch.Generator(device="cuda").manual_seed(9)
    a1 = K().sample(flat[:1], torch.ones(1, device="cuda"), None, None, None, {0: g1}, None)
    a2 = K().sample(flat[:1], torch.ones(1, device="cuda"), None, None, None, {0: g2}, None)
    assert a1.item() == a2.item()
    u1 = K().sample(flat, torch.ones(64, device="cuda"), None, None, None, None, None)
    u2 = K().sample(flat, torch.ones(64, device="cuda"), None, None, None, None, None)
    assert not torch.equal(u1, u2) and u1.unique().numel() > 32
    # bf16 logits take the same path
    ob = K().sample(logits.bfloat16(), torch.zeros(B, device="cuda"), None, None, None, None, None)
    assert torch.equal(ob.cpu(), logits.bfloat16().float().argmax(-1).cpu())


@pytest.mark.parametrize("scheme", ["ct_w4", "fp8-channel"])
def test_compressed_tensors_linear_layers(scheme):
    """compressed-tensors layers on the packed-weight GEMM: symmetric int4 (pack-quantized) and FP8 with one scale per output
    channel, against the fp32 product with the layer's own dequantised weights."""
    from onecat_vllm.config import QuantConfig
    from onecat_vllm.layers.linear import ColumnParallelLinear
    N, Kd, T = 1024, 768, 40
    g = torch.Generator(device="cuda").manual_seed(8)
    if scheme == "ct_w4":
        layer = ColumnParallelLinear(Kd, N, quant=QuantConfig(method="ct_w4", bits=4, group_size=128, zero_point=False, sym=True,
                                                              modules_to_not_convert=[]), prefix="l.proj", dtype=torch.bfloat16).cuda()
        layer.weight_packed.data = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, Kd // 8), device="cuda", generator=g, dtype=torch.int64).to(torch.int32)
        layer.weight_scale.data = (torch.rand(N, Kd // 128, device="cuda", generator=g) * 0.02 + 0.001).half()
    else:
        layer = ColumnParallelLinear(Kd, N, quant=QuantConfig(method="fp8", bits=8, group_size=0, zero_point=False, strategy="channel",
                                                              modules_to_not_convert=[]), prefix="l.proj", dtype=torch.bfloat16).cuda()
        codes = torch.randint(0, 256, (N, Kd), device="cuda", generator=g, dtype=torch.uint8)
        codes[(codes & 0x7F) == 0x7F] = 0x3C
        layer.weight.data = codes.view(torch.float8_e4m3fn)
        layer.weight_scale.data = torch.rand(N, 1, device="cuda", generator=g) * 3e-4 + 1e-5
    wd = layer.method.dequantized_weight(layer).float().cpu()
    layer.process_weights_after_loading()
    assert layer.kernel_state["kind"] == "w4"
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    y = layer(x)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    _close(y, x.float().cpu() @ wd.t(), 3e-2, 2e-2, scheme)


def test_paged_attention_forced_splits():
    q, cache, md = _attn_case([1] * 3, [5000, 130, 0], 40, 8, 128, seed=4)
    from onecat_vllm.ops.cuda import plan_attention
    for s in (2, 7, 32):
        md.attn_plan = ((40, 8, 128), plan_attention(md.query_lens_cpu, md.seq_lens_cpu, 40, 8, 128, 148, force_splits=s))
        out = K().paged_attention(q, cache, md, 128 ** -0.5)
        e = ref.paged_attention(q.cpu(), cache.cpu(), md.block_table.cpu(), md.query_start_loc.cpu(), md.seq_lens.cpu(), 128 ** -0.5)
        _close(out, e, 2e-2, 1e-2, f"splits={s}")


def test_rms_norm_gated():
    T, Hh, D = 21, 6, 128
    x = torch.randn(T, Hh * D, device="cuda").bfloat16()
    zz = torch.randn(T, 3 * Hh * D, device="cuda").bfloat16()
    z = zz[:, Hh * D: 2 * Hh * D]
    w = torch.randn(D, device="cuda").bfloat16()
    y = K().rms_norm_gated(x, z, w, 1e-6, Hh)
    e = ref.rms_norm_gated(x.cpu().reshape(T * Hh, D), z.cpu().reshape(T * Hh, D), w.cpu(), 1e-6).reshape(T, Hh * D)
    _close(y, e, 2e-2, 2e-2)


def test_peer_wait_is_bounded_and_reports_status():
    """A reduction waits on a peer flag that nothing ever sets: the kernel must give up after its limit, raise the
    status word and leave the context usable (no trap, no hang)."""
    from onecat_vllm.ops import _C
    T, H, tp = 4, 512, 2
    part = [torch.randn(T, H, device="cuda").bfloat16() for _ in range(tp)]
    flags = [torch.zeros(2 * 2 * tp * 1024, dtype=torch.int32, device="cuda") for _ in range(tp)]
    seq = torch.zeros(1024, dtype=torch.int32, device="cuda")
    x = torch.zeros(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    K().check_status()
    _C.tp_reduce_norm([t.data_ptr() for t in part], [f.data_ptr() for f in flags], seq, [x.data_ptr(), 0], None, None, w, T, H, 0, 0, False, 0,
                      1e-6, 2_000_000, T, [], 0, 0, 0, False)  # 2 ms limit; the flag of "rank 1" is never written
    torch.cuda.synchronize()
    assert K().check_status() & 2, "the expired wait must be reported"
    assert K().check_status() == 0, "status is cleared after reading"
    assert float(x.abs().sum()) == 0.0, "no output may be produced after a failed wait"
    # the context still works
    y, _ = K().rms_norm(part[0], w, 1e-6, None, False)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()


def test_expert_exchange_waits_are_bounded():
    """The expert-parallel exchange with a peer that never takes part (its slab is a second buffer on this GPU that nothing writes):
    every stage gives up after its limit, the status word reports it, nothing is written out of bounds and the context lives on."""
    from onecat_vllm.ops import _C
    n, El, k, H, I, T = 2, 32, 2, 256, 128, 8
    E = n * El
    cap, ret_rows = 64, 32

    def up(v):
        return -(-v // 256) * 256
    off = [0, up(n * E * 4)]
    off.append(off[1] + 256)
    off.append(off[2] + up(cap * H * 2))
    off.append(off[3] + up(cap * 4))
    off.append(off[4] + up(ret_rows * H * 2))
    total = off[5] + up(64 * H * 2)
    slabs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(n)]
    w13 = (torch.randn(El * 2 * I, H, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(El * H, I, device="cuda") * 0.05).bfloat16()
    x = torch.randn(T, H, device="cuda").bfloat16()
    ids = torch.randint(0, E, (T, k), device="cuda", dtype=torch.int32)
    w = torch.rand(T, k, device="cuda")
    state = torch.zeros(8 + 2 * E, dtype=torch.int32, device="cuda")
    K().check_status()
    ws = K().workspace(x.device)
    y = _C.fused_moe_a2a(x, w13, w2, w, ids, El, ws.counters, 0, None, None, 0, 1, [s.data_ptr() for s in slabs], off, state, 0, cap, ret_rows,
                         64, 0, True, 1_000_000)   # 1 ms per wait
    torch.cuda.synchronize()
    assert K().check_status() & 2, "the expired waits must be reported"
    assert int(slabs[1][off[2]:].view(torch.int16).abs().sum()) == 0, "nothing may be dispatched after the count exchange failed"
    z, _ = K().rms_norm(x, torch.ones(H, device="cuda", dtype=torch.bfloat16), 1e-6, None, False)
    torch.cuda.synchronize()
    assert torch.isfinite(z.float()).all() and y.shape == (T, H)


def test_gdn_kernels_match_sequential_oracle():
    """conv + gating + gated delta rule: prefill chunk with and without an initial state, then single-token decode."""
    Hk, Hv, Kd, Vd, kw = 2, 6, 128, 128, 4
    C = 2 * Hk * Kd + Hv * Vd
    g = torch.Generator(device="cuda").manual_seed(0)
    conv_w = (torch.randn(C, kw, device="cuda", generator=g) * 0.3).bfloat16()
    A_log = torch.rand(Hv, device="cuda", generator=g)
    dt_bias = torch.rand(Hv, device="cuda", generator=g)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device="cuda")
    conv_state = (torch.randn(4, C, kw - 1, device="cuda", generator=g) * 0.5).bfloat16()
    ssm = torch.randn(4, Hv, Kd, Vd, device="cuda", generator=g) * 0.1
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    for qlens, init in (([37, 5, 1], [1, 0, 1]), ([1, 1, 1], [1, 1, 1])):
        T = sum(qlens)
        mixed = (torch.randn(T, C, device="cuda", generator=g) * 0.5).bfloat16()
        ba = torch.randn(T, 2 * Hv, device="cuda", generator=g).bfloat16()
        qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
        hi = torch.tensor(init, dtype=torch.int32, device="cuda")
        md = AttentionMetadata(3, T, qsl, None, None, None, None, max(qlens), 0, state_slots=slots, has_initial_state=hi)
        cs_c, ssm_c = conv_state.cpu().clone(), ssm.cpu().clone()
        o = K().gdn_forward(mixed, ba[:, :Hv], ba[:, Hv:], conv_w, A_log, dt_bias, conv_state, ssm, md, Hk, Hv, Kd, Vd)
        torch.cuda.synchronize()
        mc = ref.causal_conv1d(mixed.cpu(), conv_w.cpu(), None, cs_c, qsl.cpu(), slots.cpu(), hi.cpu())
        qq, kk, vv = mc[:, : Hk * Kd].reshape(T, Hk, Kd), mc[:, Hk * Kd: 2 * Hk * Kd].reshape(T, Hk, Kd), mc[:, 2 * Hk * Kd:].reshape(T, Hv, Vd)
        gg, beta = ref.gdn_gating(ba[:, Hv:].cpu(), ba[:, :Hv].cpu(), A_log.cpu(), dt_bias.cpu())
        oe = ref.gated_delta_rule(qq, kk, vv, gg, beta, ssm_c, qsl.cpu(), slots.cpu(), hi.cpu())
        _close(o.view(T, Hv, Vd), oe, 3e-2, 3e-2, f"gdn out {qlens}")
        _close(conv_state, cs_c, 1e-2, 1e-2, "conv state")
        _close(ssm[slots.long()], ssm_c[slots.long().cpu()], 3e-2, 3e-2, "recurrent state")
    assert K().check_status() == 0


@pytest.mark.parametrize("qlens,init", [([200, 5, 1], [0, 0, 1]), ([64, 130, 333], [1, 0, 1]), ([1024], [0]), ([700, 1, 65], [1, 1, 0])])
def test_gdn_chunked_prefill_matches_sequential_oracle(qlens, init):
    """Sequences of 64 tokens or more take the chunked tensor-core kernels (whole and ragged chunks, with and without an initial
    state), shorter ones the recurrent kernel in the same call; outputs and the state handed to the next step are checked against
    the token-by-token recurrence in fp32, and against the recurrent kernel itself."""
    import os
    Hk, Hv, Kd, Vd, kw = 2, 6, 128, 128, 4
    C = 2 * Hk * Kd + Hv * Vd
    R = len(qlens)
    g = torch.Generator(device="cuda").manual_seed(5)
    conv_w = (torch.randn(C, kw, device="cuda", generator=g) * 0.3).bfloat16()
    A_log = torch.rand(Hv, device="cuda", generator=g) - 1.0
    dt_bias = torch.rand(Hv, device="cuda", generator=g)
    slots = torch.tensor([2, 0, 3][:R], dtype=torch.int32, device="cuda")
    conv_state = (torch.randn(4, C, kw - 1, device="cuda", generator=g) * 0.5).bfloat16()
    ssm = torch.randn(4, Hv, Kd, Vd, device="cuda", generator=g) * 0.1
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    T = sum(qlens)
    mixed = (torch.randn(T, C, device="cuda", generator=g) * 0.5).bfloat16()
    ba = torch.randn(T, 2 * Hv, device="cuda", generator=g).bfloat16()
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
    hi = torch.tensor(init, dtype=torch.int32, device="cuda")

    def run(mode):
        os.environ["ONECAT_GDN_PREFILL"] = mode
        md = AttentionMetadata(R, T, qsl, None, None, None, None, max(qlens), 0, state_slots=slots, has_initial_state=hi, query_lens_cpu=list(qlens))
        cs, st = conv_state.clone(), ssm.clone()
        o = K().gdn_forward(mixed, ba[:, :Hv], ba[:, Hv:], conv_w, A_log, dt_bias, cs, st, md, Hk, Hv, Kd, Vd)
        torch.cuda.synchronize()
        return o, cs, st

    try:
        o_c, cs_c, st_c = run("chunked")
        o_r, cs_r, st_r = run("recurrent")
    finally:
        os.environ.pop("ONECAT_GDN_PREFILL", None)
    cs_e, st_e = conv_state.cpu().clone(), ssm.cpu().clone()
    mc = ref.causal_conv1d(mixed.cpu(), conv_w.cpu(), None, cs_e, qsl.cpu(), slots.cpu(), hi.cpu())
    qq, kk, vv = mc[:, : Hk * Kd].reshape(T, Hk, Kd), mc[:, Hk * Kd: 2 * Hk * Kd].reshape(T, Hk, Kd), mc[:, 2 * Hk * Kd:].reshape(T, Hv, Vd)
    gg, beta = ref.gdn_gating(ba[:, Hv:].cpu(), ba[:, :Hv].cpu(), A_log.cpu(), dt_bias.cpu())
    oe = ref.gated_delta_rule(qq, kk, vv, gg, beta, st_e, qsl.cpu(), slots.cpu(), hi.cpu())
    _close(o_r.view(T, Hv, Vd), oe, 3e-2, 3e-2, f"recurrent kernel {qlens}")
    _close(o_c.view(T, Hv, Vd), oe, 4e-2, 4e-2, f"chunked kernels {qlens}")
    _close(st_c[slots.long()], st_e[slots.long().cpu()], 4e-2, 4e-2, "state after the chunked prefill")
    _close(cs_c, cs_e, 1e-2, 1e-2, "conv state")
    # hand-over: one decode token per sequence on top of the chunked prefill's state must match the oracle continuing from its own
    T2 = R
    mixed2 = (torch.randn(T2, C, device="cuda", generator=g) * 0.5).bfloat16()
    ba2 = torch.randn(T2, 2 * Hv, device="cuda", generator=g).bfloat16()
    qsl2 = torch.arange(R + 1, dtype=torch.int32, device="cuda")
    one = torch.ones(R, dtype=torch.int32, device="cuda")
    md2 = AttentionMetadata(R, T2, qsl2, None, None, None, None, 1, 0, state_slots=slots, has_initial_state=one, query_lens_cpu=[1] * R)
    o2 = K().gdn_forward(mixed2, ba2[:, :Hv], ba2[:, Hv:], conv_w, A_log, dt_bias, cs_c, st_c, md2, Hk, Hv, Kd, Vd)
    torch.cuda.synchronize()
    mc2 = ref.causal_conv1d(mixed2.cpu(), conv_w.cpu(), None, cs_e, qsl2.cpu(), slots.cpu(), one.cpu())
    g2, b2 = ref.gdn_gating(ba2[:, Hv:].cpu(), ba2[:, :Hv].cpu(), A_log.cpu(), dt_bias.cpu())
    oe2 = ref.gated_delta_rule(mc2[:, : Hk * Kd].reshape(T2, Hk, Kd), mc2[:, Hk * Kd: 2 * Hk * Kd].reshape(T2, Hk, Kd), mc2[:, 2 * Hk * Kd:].reshape(T2, Hv, Vd),
                               g2, b2, st_e, qsl2.cpu(), slots.cpu(), one.cpu())
    _close(o2.view(T2, Hv, Vd), oe2, 4e-2, 4e-2, "decode after chunked prefill")
    assert K().check_status() == 0


@pytest.mark.parametrize("D", [64, 128, 256, 512])
def test_merge_attn_states_kernel(D):
    g = torch.Generator(device="cuda").manual_seed(D)
    T, H = 37, 5
    o1, o2 = torch.randn(T, H, D, device="cuda", generator=g).bfloat16(), torch.randn(T, H, D, device="cuda", generator=g).bfloat16()
    l1, l2 = torch.randn(T, H, device="cuda", generator=g) * 5, torch.randn(T, H, device="cuda", generator=g) * 5
    l1[0, 0] = float("-inf")            # an empty side contributes nothing
    l1[1, 1] = l2[1, 1] = float("-inf")  # both empty: zeros, lse -inf-like is not required, only finiteness of the output
    o, lse = K().merge_attn_states(o1, l1, o2, l2)
    oe, le = ref.merge_attn_states(o1.cpu(), l1.cpu(), o2.cpu(), l2.cpu())
    _close(o, oe, 2e-2, 2e-2, "merged output")
    ok = torch.isfinite(le)
    _close(lse.cpu()[ok], le[ok], 1e-3, 1e-3, "merged lse")
    assert torch.equal(o[0, 0], o2[0, 0])


@pytest.mark.parametrize("deepseek", [False, True])
def test_router_matches_reference(deepseek):
    T, E, k = 77, 256, 8
    logits = torch.randn(T, E, device="cuda").bfloat16()
    from types import SimpleNamespace
    if deepseek:
        bias = torch.randn(E, device="cuda") * 0.1
        cfg = SimpleNamespace(num_experts_per_tok=k, n_group=8, topk_group=4, scoring_func="sigmoid", norm_topk_prob=True, routed_scaling_factor=2.5)
        w, ids = K().route(logits, cfg, bias)
        we, ie = ref.grouped_topk(logits.float().cpu(), k, 8, 4, bias.cpu(), "sigmoid", True, 2.5)
    else:
        cfg = SimpleNamespace(num_experts_per_tok=k, n_group=1, topk_group=1, scoring_func="softmax", norm_topk_prob=True, routed_scaling_factor=1.0)
        w, ids = K().route(logits, cfg, None)
        we, ie = ref.topk_softmax(logits.float().cpu(), k, True)
    assert "route" not in K().TORCH_STANDINS
    # bf16 logits contain exact ties, and torch.topk does not promise which tied expert it returns: compare the selected
    # weights as multisets everywhere, and the expert ids on the rows where both picked the same set
    _close(w.cpu().sort(-1)[0], we.sort(-1)[0], 2e-2, 1e-3, "sorted routing weights")
    rows = (ids.cpu().sort(-1)[0] == ie.sort(-1)[0]).all(-1)
    assert rows.float().mean() > 0.85
    wd = torch.zeros(T, E).scatter_(1, ids.cpu().long(), w.cpu())
    wed = torch.zeros(T, E).scatter_(1, ie.long(), we)
    _close(wd[rows], wed[rows], 2e-2, 1e-3, "routing weights")
    assert (ids >= 0).all() and (ids < E).all() and all(len(set(r)) == k for r in ids.cpu().tolist())


def test_rejection_sampler_kernel():
    from onecat_vllm.sample.metadata import SamplingMetadata
    from onecat_vllm.sample.rejection_sampler import RejectionSampler
    B, k, V = 64, 3, 4096

    def md(greedy):
        m = SamplingMetadata(temperature=None if greedy else torch.ones(B, device="cuda"), all_greedy=greedy, all_random=not greedy, top_p=None, top_k=None,
                             min_p=None, generators={}, max_num_logprobs=None, no_penalties=True)
        return m
    tl = torch.randn(B, k + 1, V, device="cuda").bfloat16()
    am = tl.float().argmax(-1)
    draft = am[:, :k].clone()
    draft[::2, 1] = (draft[::2, 1] + 1) % V  # every other request: second draft wrong
    bonus = torch.full((B,), 7, device="cuda")
    out = RejectionSampler()(draft, torch.full((B,), k, device="cuda"), tl, bonus, md(True))
    parsed = RejectionSampler.parse_output(out)
    for b in range(B):
        exp = [int(am[b, 0]), int(am[b, 1])] if b % 2 == 0 else [int(am[b, 0]), int(am[b, 1]), int(am[b, 2]), 7]
        assert parsed[b] == exp, (b, parsed[b], exp)
    assert "rejection_sample" not in K().TORCH_STANDINS
    # random mode: acceptance probability of a point-mass draft equals its target probability
    p = torch.tensor([0.6, 0.3, 0.1] + [0.0] * (V - 3), device="cuda").clamp_min(1e-9)
    tl2 = torch.log(p).view(1, 1, V).repeat(4096, 2, 1).float()
    d2 = torch.zeros(4096, 1, dtype=torch.long, device="cuda")
    m2 = SamplingMetadata(temperature=torch.ones(4096, device="cuda"), all_greedy=False, all_random=True, top_p=None, top_k=None, min_p=None, generators={},
                          max_num_logprobs=None, no_penalties=True)
    o2 = RejectionSampler(seed=5)(d2, torch.ones(4096, dtype=torch.long, device="cuda"), tl2, torch.full((4096,), 2, device="cuda"), m2)
    first = o2[:, 0].cpu()
    freq = torch.bincount(first, minlength=3)[:3].float() / 4096
    assert torch.allclose(freq, torch.tensor([0.6, 0.3, 0.1]), atol=0.04), freq
    # synthetic acceptance
    rs = RejectionSampler(synthetic_rates=[0.7, 0.7, 0.7], seed=3)
    o3 = rs(draft, torch.full((B,), k, device="cuda"), tl, bonus, md(True))
    lens = torch.tensor([len(r) for r in RejectionSampler.parse_output(o3)]).float()
    assert 1.8 < lens.mean() < 3.3


@pytest.mark.parametrize("T,E,k,e_off,E_local", [(1, 16, 2, 0, 16), (37, 16, 4, 0, 16), (300, 64, 8, 16, 32), (5, 256, 8, 0, 256)])
def test_fused_moe_grouped_gemm(T, E, k, e_off, E_local):
    """Grouped tcgen05 GEMMs over device-built work lists against per-expert fp32 FFNs; with e_off/E_local only a slice of the
    experts is local and the rest of each token's routing contributes nothing (expert parallelism)."""
    H, I = 256, 128
    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = (torch.randn(T, H, device="cuda", generator=g) * 0.5).bfloat16()
    w13 = (torch.randn(E_local, 2 * I, H, device="cuda", generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(E_local, H, I, device="cuda", generator=g) * 0.05).bfloat16()
    logits = torch.randn(T, E, device="cuda", generator=g)
    tw, ti = ref.topk_softmax(logits, k, True)

    class M:
        pass
    m = M()
    m.qmethod, m.E_local, m.e_off, m._dq = "none", E_local, e_off, None
    m.w13, m.w2 = w13.clone(), w2.clone()
    m.dequantized = lambda: (m.w13, m.w2)
    K().prepare_moe(m)
    assert m.kernel_state is not None
    y = K().fused_moe(m, x, tw, ti)
    torch.cuda.synchronize()
    assert K().check_status() == 0 and "fused_moe" not in K().TORCH_STANDINS
    e = ref.fused_experts(x.cpu(), w13.cpu(), w2.cpu(), tw.cpu(), ti.cpu(), e_off)
    _close(y, e, 3e-2, 3e-3, f"moe T={T} E={E}")
    y2 = K().fused_moe(m, x, tw, ti)
    assert torch.equal(y, y2), "slot order varies between runs but the output must not"


@pytest.mark.parametrize("name,qlens,ctxs,H", [("decode", [1, 1, 1, 1], [0, 70, 1000, 4100], 16), ("decode-128h", [1, 1], [300, 65], 128),
                                               ("verify+prefill", [4, 37], [100, 0], 16)])
def test_mla_decode(name, qlens, ctxs, H):
    lora, rope, bs = 512, 64, 16
    g = torch.Generator(device="cuda").manual_seed(2)
    R = len(qlens)
    seq = [c + q for q, c in zip(qlens, ctxs)]
    nbp = [-(-s // bs) for s in seq]
    total = sum(nbp) + 2
    perm = torch.randperm(total, device="cuda", generator=g).to(torch.int32)
    bt = torch.zeros(R, max(nbp) + 1, dtype=torch.int32, device="cuda")
    o = 0
    for r, n in enumerate(nbp):
        bt[r, :n] = perm[o:o + n]
        o += n
    cache = (torch.randn(total, bs, lora + rope, device="cuda", generator=g) * 0.3).bfloat16()
    T = sum(qlens)
    q_abs = (torch.randn(T, H, lora, device="cuda", generator=g) * 0.3).bfloat16()
    q_pe = (torch.randn(T, H, rope, device="cuda", generator=g) * 0.3).bfloat16()
    from onecat_vllm.worker.attn_metadata import AttentionMetadata
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device="cuda")
    sl = torch.tensor(seq, dtype=torch.int32, device="cuda")
    md = AttentionMetadata(R, T, qsl, sl, bt, None, None, max(qlens), max(seq), query_lens_cpu=list(qlens), seq_lens_cpu=seq)
    scale = (128 + 64) ** -0.5
    out = K().mla_decode(q_abs, q_pe, cache, md, scale, lora)
    torch.cuda.synchronize()
    assert K().check_status() == 0 and "mla_decode" not in K().TORCH_STANDINS
    e = ref.mla_decode(q_abs.cpu(), q_pe.cpu(), cache.cpu(), bt.cpu(), qsl.cpu(), sl.cpu(), scale, lora)
    _close(out, e, 2e-2, 5e-3, name)
