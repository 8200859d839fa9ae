"""Out-of-bounds detection without a sanitizer: outputs sit inside larger buffers filled with a sentinel (a write one element too far
changes it), scratch areas are NaN-poisoned before the launch (a partial that is read without having been written shows up as NaN),
and the shapes straddle every tile edge of the kernels. Nothing here feeds a kernel an index that could fault."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
SENT = 12288.0   # exactly representable in bf16


def K():
    from onecat_vllm.ops import cuda
    return cuda


def _framed(T, N, col_off):
    buf = torch.full((T + 2, N + 32), SENT, device="cuda", dtype=torch.bfloat16)
    return buf, buf[1:T + 1, col_off:col_off + N]


def _frame_intact(buf, T, N, col_off):
    m = torch.ones_like(buf, dtype=torch.bool)
    m[1:T + 1, col_off:col_off + N] = False
    return bool((buf[m].float() == SENT).all())


@pytest.mark.parametrize("T", [1, 31, 33, 64, 65, 127, 129, 257])
@pytest.mark.parametrize("N,Kd", [(136, 192), (640, 1280), (5000, 320)])
@pytest.mark.parametrize("col_off", [8, 4])   # 16-byte aligned rows (vector stores) and rows that are not (scalar stores)
def test_bf16_gemm_writes_only_its_output(T, N, Kd, col_off):
    g = torch.Generator(device="cuda").manual_seed(T + N)
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    w = (torch.randn(N, Kd, device="cuda", generator=g) * 0.05).bfloat16()
    K().workspace(x.device).splitk.view(torch.int16).fill_(0x7FC0)      # bf16 / fp32 NaN pattern over the split-K scratch
    buf, out = _framed(T, N, col_off)
    K().gemm_bf16(x, w, out=out)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    assert _frame_intact(buf, T, N, col_off), "a store landed outside the output"
    e = x.float() @ w.float().t()
    assert torch.isfinite(out.float()).all() and (out.float() - e).abs().max() <= 3e-2 * math.sqrt(Kd) * 0.05 + 2e-2 * e.abs().max()


class _Layer:
    def __init__(self, fuse):
        self.fuse_silu_mul, self.bias, self.kernel_state = fuse, None, None


@pytest.mark.parametrize("T", [1, 17, 64, 65, 193, 400])
@pytest.mark.parametrize("N,Kd,fuse", [(384, 256, False), (896, 5120, False), (512, 640, True)])
def test_w4_gemm_writes_only_its_output(T, N, Kd, fuse):
    grp = 128
    g = torch.Generator(device="cuda").manual_seed(T * 3 + N)
    q = torch.randint(0, 16, (N, Kd), device="cuda", generator=g, dtype=torch.uint8)
    z = torch.randint(0, 16, (N, Kd // grp), device="cuda", generator=g, dtype=torch.uint8)
    s = (torch.randn(N, Kd // grp, device="cuda", generator=g).abs() * 0.01 + 1e-3).half()
    x = torch.randn(T, Kd, device="cuda", generator=g).bfloat16()
    layer = _Layer(fuse)
    K().prepare_w4(layer, q, z, s, grp)
    n_out = layer.kernel_state["n_out"]
    K().workspace(x.device).splitk.view(torch.int16).fill_(0x7FC0)
    buf, out = _framed(T, n_out, 8)
    K().linear(layer, x, out=out)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    assert _frame_intact(buf, T, n_out, 8), "a store landed outside the output"
    assert torch.isfinite(out.float()).all()


def test_cache_insert_touches_only_the_mapped_slots():
    from onecat_vllm.ops import ref
    T, Hq, Hkv, D, bs, nb = 70, 8, 2, 128, 16, 12
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    q, k, v = qkv[:, :Hq * D].view(T, Hq, D), qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D), qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cache = torch.full((nb, 2, Hkv, bs, D), SENT, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
    slots[3] = -1      # a padded token: writes nothing
    cs = ref.build_cos_sin_cache(D, 512, 1e6, "cuda")
    K().rope_and_cache(q, k, v, torch.arange(T, device="cuda", dtype=torch.int32), cs, cache, slots, D, None, None, 1e-6, False)
    torch.cuda.synchronize()
    assert K().check_status() == 0
    used = torch.zeros(nb * bs, dtype=torch.bool, device="cuda")
    used[slots[slots >= 0].long()] = True
    flat = cache.permute(0, 3, 1, 2, 4).reshape(nb * bs, 2, Hkv, D)     # [slot][k|v][head][D]
    assert bool((flat[~used].float() == SENT).all()), "a slot that no token maps to was written"
    assert bool((flat[used].float() != SENT).any(dim=-1).all()), "a mapped slot was left unwritten"
