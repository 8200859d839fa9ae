"""Python side of the sm_100a kernels: weight repacking, workspaces, launch planning.

Importing this module loads the in-tree extension ``onecat_vllm.ops._C`` and fails loudly when it is missing: on a
CUDA device there is no eager fallback for the ops implemented here. Ops whose kernels are not written yet
(listed in ``TORCH_STANDINS``) run the PyTorch restatement on the device and are reported as such."""
from __future__ import annotations

import os
from typing import Optional

import torch

from onecat_vllm.ops import ref

try:
    from onecat_vllm.ops import _C
except ImportError as e:  # pragma: no cover
    raise ImportError("the CUDA extension onecat_vllm.ops._C is not built; run `python -c 'import __graft_entry__ as g; g.build()'` "
                      f"or `python 1cat-vllm_b200/ops/build.py` ({e})") from e

EPI_STORE, EPI_SILU_MUL = 0, 1
TORCH_STANDINS: set = set()  # names of ops that ran as device-side PyTorch code in this process
_LAUNCHES = 0  # launches of our own kernels (for bench accounting)
_LIB_GEMM = os.environ.get("ONECAT_GEMM_BACKEND", "tcgen05") == "library"  # debug switch only
_ATTN_PREFILL_TC = os.environ.get("ONECAT_ATTN_PREFILL", "tcgen05") != "mma"  # head size 128 prefill: tcgen05 kernel unless "mma"


def launches() -> int:
    return _LAUNCHES


def reset_launches() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


class _Workspace:
    """Per-device scratch: split-K partials + tile counters, split-KV partials."""

    def __init__(self, device):
        self.device = device
        self.splitk = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        self.counters = torch.zeros(8192, dtype=torch.int32, device=device)  # upper half: scratch
        self.attn_o = None
        self.attn_ml = None

    def attn_static(self, n_o: int, n_ml: int):
        """Buffers whose addresses are baked into CUDA graphs: sized once per engine for its largest graph."""
        if getattr(self, "s_o", None) is None or self.s_o.numel() < n_o or self.s_ml.numel() < n_ml:
            # a later engine in the same process may need more; graphs captured earlier keep their (retired) buffers alive
            if getattr(self, "s_o", None) is not None:
                self._retired = getattr(self, "_retired", []) + [(self.s_o, self.s_ml)]
            self.s_o = torch.empty(n_o, dtype=torch.float32, device=self.device)
            self.s_ml = torch.empty(n_ml, dtype=torch.float32, device=self.device)
        return self.s_o, self.s_ml

    def attn(self, n_o: int, n_ml: int):
        if self.attn_o is None or self.attn_o.numel() < n_o:
            self.attn_o = torch.empty(n_o, dtype=torch.float32, device=self.device)
        if self.attn_ml is None or self.attn_ml.numel() < n_ml:
            self.attn_ml = torch.empty(n_ml, dtype=torch.float32, device=self.device)
        return self.attn_o, self.attn_ml


_WS: dict = {}


def workspace(device) -> _Workspace:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _WS:
        _WS[key] = _Workspace(torch.device("cuda", key))
    return _WS[key]


def check_status(clear: bool = True) -> int:
    return int(_C.read_status(clear))


# ----------------------------------------------------------------------------- weight repacking
_NIB_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # nibble i of a packed word holds k offset _NIB_ORDER[i]


def interleave_gate_up(n_inter: int, device) -> torch.Tensor:
    """Row permutation putting 16 gate rows next to the matching 16 up rows, so that one warp of the GEMM epilogue
    holds both halves of SiLU(gate)*up."""
    assert n_inter % 16 == 0, "the intermediate size must be a multiple of 16"
    b = torch.arange(n_inter // 16, device=device).view(-1, 1, 1) * 16
    j = torch.arange(16, device=device).view(1, 1, 16)
    half = torch.tensor([0, n_inter], device=device).view(1, 2, 1)
    return (b + j + half).reshape(-1)


def pack_w4(q: torch.Tensor, z: torch.Tensor, s: torch.Tensor, group: int):
    """q ``[N,K]`` uint8 codes, z ``[N,K/g]`` uint8 zeros, s ``[N,K/g]`` scales → (tiles uint8 ``[N/128, K/64, 4096]``,
    sz int32 ``[K/g, Npad]``). A tile holds 128 rows × 64 k as two halves of ``[128 rows][4 words]``; each 32-bit word is
    8 consecutive k of one row in ``_NIB_ORDER``."""
    N, K = q.shape
    assert K % 64 == 0 and group % 64 == 0, "K and the group size must be multiples of 64"
    npad = -(-N // 128) * 128
    if npad != N:
        q = torch.cat([q, q.new_zeros(npad - N, K)])
        z = torch.cat([z, z.new_zeros(npad - N, z.shape[1])])
        s = torch.cat([s, s.new_zeros(npad - N, s.shape[1])])
    nt, kt = npad // 128, K // 64
    qq = q.view(nt, 128, kt, 8, 8).to(torch.int32)
    words = torch.zeros(nt, 128, kt, 8, dtype=torch.int32, device=q.device)
    for i, k in enumerate(_NIB_ORDER):
        words |= qq[..., k] << (4 * i)
    tiles = words.view(nt, 128, kt, 2, 4).permute(0, 2, 3, 1, 4).contiguous().view(torch.uint8).view(nt, kt, 4096)
    sb = s.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    zb = (z.to(torch.float32) + 128.0).to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    sz = (sb | (zb << 16)).t().contiguous()
    return tiles, sz, npad


def prepare_w4(layer, q: torch.Tensor, z: torch.Tensor, s: torch.Tensor, group: int) -> None:
    """Repack a 4-bit layer for the kernel. ``q/z/s`` are in logical ``[out, in]`` orientation."""
    n_rows = q.shape[0]
    n_out = n_rows
    epi = EPI_STORE
    if layer.fuse_silu_mul:
        perm = interleave_gate_up(n_rows // 2, q.device)
        q, z, s = q[perm], z[perm], s[perm]
        n_out, epi = n_rows // 2, EPI_SILU_MUL
    tiles, sz, npad = pack_w4(q.contiguous(), z.contiguous(), s.contiguous(), group)
    layer.kernel_state = dict(kind="w4", tiles=tiles, sz=sz, n_rows=n_rows, n_out=n_out, n_pad=npad, epi=epi, group_ktiles=group // 64,
                              K=q.shape[1])


def prepare_bf16(layer) -> None:
    w = layer.weight.data
    n_rows, epi, n_out = w.shape[0], EPI_STORE, w.shape[0]
    if layer.fuse_silu_mul:
        w = w[interleave_gate_up(n_rows // 2, w.device)].contiguous()
        layer.weight.data = w
        epi, n_out = EPI_SILU_MUL, n_rows // 2
    layer.kernel_state = dict(kind="bf16", n_rows=n_rows, n_out=n_out, epi=epi, K=w.shape[1])


def _bf16_bits(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF


def pack_fp8(w8: torch.Tensor, row_scale: torch.Tensor, group: int):
    """w8 ``[N,K]`` e4m3 (any 1-byte dtype), row_scale ``[N, K/group]`` fp32 (dequantisation scale of each row over each k group;
    group a multiple of 64) → (tiles uint8 ``[N/128, K/64, 8192]``, sz int32 ``[K/group, Npad]``). A tile is four chunks of
    ``[128 rows][16 bytes]`` (chunk c = k 16c..16c+15); the scale words are ``bf16(scale * 2**120)``: the kernel builds each bf16
    from the fp8 bits with the exponent 120 too small."""
    N, K = w8.shape
    assert K % 64 == 0 and group % 64 == 0 and K % group == 0
    npad = -(-N // 128) * 128
    w8 = w8.contiguous().view(torch.uint8)
    if npad != N:
        w8 = torch.cat([w8, w8.new_zeros(npad - N, K)])
        row_scale = torch.cat([row_scale, row_scale.new_zeros(npad - N, row_scale.shape[1])])
    nt, kt = npad // 128, K // 64
    tiles = w8.view(nt, 128, kt, 4, 16).permute(0, 2, 3, 1, 4).contiguous().view(nt, kt, 8192)
    sc = row_scale.float() * (2.0 ** 120)
    assert bool(torch.isfinite(sc.to(torch.bfloat16)).all()), "fp8 scale too large for the bf16 scale word"
    sz = _bf16_bits(sc).t().contiguous()
    return tiles, sz, npad


def pack_mxfp4(packed: torch.Tensor, scales_ue8m0: torch.Tensor):
    """packed ``[N, K/2]`` uint8 (low nibble = even k), scales ``[N, K/32]`` ue8m0 → (tiles uint8 ``[N/128, K/64, 4096]`` in the
    4-bit tile layout of ``pack_w4``, sz int32 ``[K/64, Npad]`` with the two 32-k groups' ``bf16(2**(e-127) * 2**126)`` in the low
    and high half)."""
    N, K2 = packed.shape
    K = K2 * 2
    assert K % 64 == 0
    npad = -(-N // 128) * 128
    q = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(N, K)
    e = scales_ue8m0.to(torch.int32)
    if npad != N:
        q = torch.cat([q, q.new_zeros(npad - N, K)])
        e = torch.cat([e, e.new_full((npad - N, e.shape[1]), 127)])
    nt, kt = npad // 128, K // 64
    qq = q.view(nt, 128, kt, 8, 8).to(torch.int32)
    words = torch.zeros(nt, 128, kt, 8, dtype=torch.int32, device=q.device)
    for i, k in enumerate(_NIB_ORDER):
        words |= qq[..., k] << (4 * i)
    tiles = words.view(nt, 128, kt, 2, 4).permute(0, 2, 3, 1, 4).contiguous().view(torch.uint8).view(nt, kt, 4096)
    assert int(e.max()) <= 128, "MXFP4 scale above 2.0 does not fit the bf16 scale word"
    sb = _bf16_bits(torch.exp2(e.float() - 1.0)).view(npad, kt, 2)
    sz = (sb[..., 0] | (sb[..., 1] << 16)).t().contiguous()
    return tiles, sz, npad


def pack_nvfp4(packed: torch.Tensor, scales_e4m3: torch.Tensor, global_scale: torch.Tensor):
    """packed ``[N, K/2]`` uint8 (low nibble = even k), scales ``[N, K/16]`` e4m3, one fp32 global scale → (tiles as ``pack_mxfp4``,
    sz int32 ``[K/64, Npad, 2]``: per row and k tile the four 16-k groups' ``bf16(scale * global * 2**126)``, two per word)."""
    N, K2 = packed.shape
    K = K2 * 2
    assert K % 64 == 0
    tiles, _, npad = pack_mxfp4(packed, torch.full((N, K // 32), 127, dtype=torch.uint8, device=packed.device))
    sc = scales_e4m3.float() * global_scale.float().reshape(-1)[0] * (2.0 ** 126)
    assert bool(torch.isfinite(sc.to(torch.bfloat16)).all()), "NVFP4 scale too large for the bf16 scale word"
    if npad != N:
        sc = torch.cat([sc, sc.new_zeros(npad - N, sc.shape[1])])
    sb = _bf16_bits(sc).view(npad, K // 64, 2, 2)
    sz = (sb[..., 0] | (sb[..., 1] << 16)).permute(1, 0, 2).contiguous()
    return tiles, sz, npad


def _fp8_row_scales(layer, block) -> tuple[torch.Tensor, int]:
    """Per-row, per-k-group dequantisation scales of an FP8 linear layer and the k group size."""
    N, K = layer.weight.shape
    if block:
        bn, bk = block
        assert bk % 64 == 0, "fp8 k blocks must be multiples of 64"
        return layer.weight_scale_inv.float().repeat_interleave(bn, dim=0)[:N].contiguous(), bk
    ws = layer.weight_scale.float().reshape(-1)
    if ws.numel() == N and getattr(layer.method, "channel", False):
        return ws.reshape(N, 1).contiguous(), K   # one scale per output channel
    if ws.numel() == 1:
        return ws.expand(N).reshape(N, 1).contiguous(), K
    rows = torch.cat([ws[i].expand(n) for i, n in enumerate(layer.local_output_sizes)])
    return rows.reshape(N, 1).contiguous(), K


def prepare_fp8(layer, block) -> None:
    """FP8 e4m3 weights stay one byte each in HBM: tiles + scale words for the weight-only path of the tcgen05 GEMM
    (dequantised to bf16 on the way into TMEM; activations stay bf16)."""
    N, K = layer.weight.shape
    if K % 64 or (block and (K % block[1] or block[1] % 64)):
        w = layer.method.dequantized_weight(layer).to(torch.bfloat16)
        return _swap_to_dense(layer, w)
    rs, group = _fp8_row_scales(layer, block)
    w8 = layer.weight.data
    n_rows, n_out, epi = N, N, EPI_STORE
    if layer.fuse_silu_mul:
        perm = interleave_gate_up(N // 2, w8.device)
        w8, rs = w8.view(torch.uint8)[perm], rs[perm]
        n_out, epi = N // 2, EPI_SILU_MUL
    tiles, sz, npad = pack_fp8(w8, rs, group)
    layer.kernel_state = dict(kind="w4", wkind=2, tiles=tiles, sz=sz, n_rows=n_rows, n_out=n_out, n_pad=npad, epi=epi, group_ktiles=group // 64, K=K)
    for n in ("weight", "weight_scale", "weight_scale_inv"):
        if hasattr(layer, n):
            delattr(layer, n)


def prepare_fp4(layer, kind: str) -> None:
    """MXFP4 and NVFP4 weights stay packed (tiles + scale words, dequantised to bf16 on the way into TMEM)."""
    N, K2 = layer.weight.shape
    if kind not in ("mxfp4", "nvfp4") or (K2 * 2) % 64:
        w = layer.method.dequantized_weight(layer).to(torch.bfloat16)
        return _swap_to_dense(layer, w)
    pk, sc = layer.weight.data, layer.weight_scale.data
    n_rows, n_out, epi = N, N, EPI_STORE
    if layer.fuse_silu_mul:
        perm = interleave_gate_up(N // 2, pk.device)
        pk, sc = pk[perm], sc[perm]
        n_out, epi = N // 2, EPI_SILU_MUL
    if kind == "nvfp4":
        tiles, sz, npad = pack_nvfp4(pk.contiguous(), sc.contiguous(), layer.weight_scale_2.data)
    else:
        tiles, sz, npad = pack_mxfp4(pk.contiguous(), sc.contiguous())
    layer.kernel_state = dict(kind="w4", wkind=4 if kind == "nvfp4" else 3, tiles=tiles, sz=sz, n_rows=n_rows, n_out=n_out, n_pad=npad, epi=epi,
                              group_ktiles=1, K=K2 * 2)
    for n in ("weight", "weight_scale", "weight_scale_2"):
        if hasattr(layer, n):
            delattr(layer, n)


def _swap_to_dense(layer, w: torch.Tensor) -> None:
    from onecat_vllm.layers.linear import UnquantizedMethod
    for n in ("weight", "weight_scale", "weight_scale_inv", "weight_scale_2"):
        if hasattr(layer, n):
            delattr(layer, n)
    layer.weight = torch.nn.Parameter(w.contiguous(), requires_grad=False)
    layer.method = UnquantizedMethod()
    prepare_bf16(layer)


# ----------------------------------------------------------------------------- GEMM
def _gemm(x, w, w4, sz, out, bias, N, n_rows, n_out, n_pad, epi, gk, force_splits=0, force_tn=0, push=None, wkind=1, trace=0):
    """``push`` = (list of destination addresses, rows per owner[, address of the buffer-select word, buffer stride in elements]):
    tensor-parallel epilogue that stores into peers' slabs (the last two for the flag-free arrival buffers)."""
    global _LAUNCHES
    ws = workspace(x.device)
    _C.gemm(x, w, w4, sz, out, bias, ws.splitk, ws.counters, N, n_rows, n_out, n_pad, epi, gk, force_splits, force_tn,
            push[0] if push else [], push[1] if push else 0, wkind if w4 is not None else 0, trace,
            push[2] if push and len(push) > 2 else 0, push[3] if push and len(push) > 2 else 0)
    _LAUNCHES += 1
    return out


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
              force_splits: int = 0, force_tn: int = 0) -> torch.Tensor:
    """x ``[T,K]`` @ w ``[N,K]``^T → ``[T,N]`` bf16."""
    N = w.shape[0]
    if _LIB_GEMM:
        return torch.nn.functional.linear(x, w, bias)
    if out is None:
        out = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    if x.stride(-1) != 1 or (x.stride(0) * 2) % 16:
        x = x.contiguous()
    return _gemm(x, w, None, None, out, bias, N, N, N, 0, EPI_STORE, 1, force_splits, force_tn)


def linear(layer, x: torch.Tensor, out: Optional[torch.Tensor] = None, push=None) -> torch.Tensor:
    ks = layer.kernel_state
    if ks is None:
        prepare_bf16(layer)
        ks = layer.kernel_state
    T = x.shape[0]
    if x.stride(-1) != 1 or (x.stride(0) * 2) % 16:
        x = x.contiguous()
    if out is None:
        out = torch.empty(T, ks["n_out"], dtype=torch.bfloat16, device=x.device)
    bias = layer.bias
    if ks["kind"] == "w4":
        if _LIB_GEMM:
            raise RuntimeError("the library GEMM debug switch does not cover 4-bit weights")
        return _gemm(x, None, ks["tiles"], ks["sz"], out, bias, ks["n_rows"], ks["n_rows"], ks["n_out"], ks["n_pad"], ks["epi"], ks["group_ktiles"], push=push,
                     wkind=ks.get("wkind", 1))
    if _LIB_GEMM:
        y = torch.nn.functional.linear(x, layer.weight, bias)
        if ks["epi"] == EPI_SILU_MUL:  # rows are interleaved in blocks of 16
            y = y.view(T, -1, 2, 16)
            return (torch.nn.functional.silu(y[:, :, 0].float()) * y[:, :, 1].float()).to(x.dtype).reshape(T, -1)
        return y
    return _gemm(x, layer.weight, None, None, out, bias, ks["n_rows"], ks["n_rows"], ks["n_out"], 0, ks["epi"], 1, push=push)


# ----------------------------------------------------------------------------- elementwise
def rms_norm(x, w, eps, residual=None, gemma=False):
    global _LAUNCHES
    _LAUNCHES += 1
    if w.dtype != torch.bfloat16:
        w = w.to(torch.bfloat16)
    if x.stride(-1) != 1:
        x = x.contiguous()
    y, r = _C.rms_norm(x, w, eps, residual, gemma)
    return y, r


def rms_norm_gated(x, z, w, eps, heads):
    global _LAUNCHES
    _LAUNCHES += 1
    T = x.shape[0]
    if x.stride(-1) != 1:
        x = x.contiguous()
    if z.stride(-1) != 1:
        z = z.contiguous()
    return _C.rms_norm_gated(x, z, w.to(torch.bfloat16), eps, heads).view(T, -1)


def silu_and_mul(x):
    global _LAUNCHES
    _LAUNCHES += 1
    return _C.silu_and_mul(x.contiguous())


def rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim, q_norm_w, k_norm_w, eps, gemma, mrope_section=None):
    global _LAUNCHES
    _LAUNCHES += 1
    s0, s1 = (int(mrope_section[0]), int(mrope_section[0] + mrope_section[1])) if mrope_section is not None and positions.dim() == 2 else (0, 0)
    _C.rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim, q_norm_w, k_norm_w, eps, gemma, 1.0, 1.0, s0, s1)


def sample(logits, temperature, top_k=None, top_p=None, min_p=None, generators=None, kept=None):
    """One kernel per batch: temperature, min-p, top-k, top-p and the random draw (rows with temperature ~ 0 take their arg-max).
    Each row gets a 64-bit word of randomness: from its request's generator when it has one (so seeded requests repeat), else from
    the device's default generator."""
    global _LAUNCHES
    _LAUNCHES += 2
    B = logits.shape[0]
    seeds = torch.randint(0, 1 << 62, (B,), dtype=torch.int64, device=logits.device)
    for i, gen in (generators or {}).items():
        seeds[i] = torch.randint(0, 1 << 62, (1,), dtype=torch.int64, device=logits.device, generator=gen)[0]
    return _C.sample(logits, temperature.float().contiguous(), None if top_k is None else top_k.to(torch.int32).contiguous(),
                     None if top_p is None else top_p.float().contiguous(), None if min_p is None else min_p.float().contiguous(), seeds, kept)


def merge_attn_states(o1, lse1, o2, lse2):
    global _LAUNCHES
    _LAUNCHES += 1
    o, lse = _C.merge_attn_states(o1.contiguous(), lse1.float().contiguous(), o2.contiguous(), lse2.float().contiguous())
    return o, lse


def argmax(logits):
    global _LAUNCHES
    _LAUNCHES += 1
    return _C.argmax(logits)


# ----------------------------------------------------------------------------- attention
_NUM_SMS: dict = {}


def _sms(device) -> int:
    k = device.index or 0
    if k not in _NUM_SMS:
        _NUM_SMS[k] = torch.cuda.get_device_properties(device).multi_processor_count
    return _NUM_SMS[k]


def choose_kv_splits(base_ctas: int, max_seq: int, num_sms: int) -> int:
    """KV splits of the decode kernel: enough CTAs for about two full waves (two CTAs fit per SM), but at least four
    64-key tiles per split so that the copy pipeline fills."""
    want = -(-(4 * num_sms) // max(base_ctas, 1))
    by_ctx = max(1, -(-max_seq // 64) // 4)
    return max(1, min(want, by_ctx, 32))


def choose_decode_splits(base_ctas: int, max_seq: int, num_sms: int) -> int:
    """KV splits of the paged decode kernel from a cost model of its waves. Two CTAs fit per SM; a CTA needs about 1.6 us to start
    and 1.9 us per 64-key tile when the SMs are full, and more than one split adds the combine launch (about 6 us). Measured on
    B200 (64 requests x 8 KV heads x 1150 keys): 71.7 us unsplit against 80.9 us in two splits, whose 1024 CTAs need four waves
    of 296 where 512 need two; 16 requests x 4096 keys: 66 us in two splits (one wave) against 83 us in three (two waves)."""
    nt = max(1, -(-max_seq // 64))
    slots = 2 * num_sms
    best, best_cost = 1, None
    for s in range(1, min(32, nt) + 1):
        per = -(-nt // s)
        if s > 1 and per < 2:
            break
        waves = -(-(max(base_ctas, 1) * s) // slots)
        cost = waves * (1.6 + 1.9 * per) + (6.0 + 0.15 * s if s > 1 else 0.0)  # the combine kernel reads one partial per split
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def plan_attention(query_lens: list, seq_lens: list, Hq: int, Hkv: int, D: int, num_sms: int, force_splits: int = 0):
    """Decide which requests take the decode kernel (rows = q_len * group fit in one 16/32-row tile) and how many KV
    splits it uses. Returns (short_q_len, num_q_tiles for the prefill kernel, splits)."""
    G = Hq // Hkv
    max_rows = 32 if D <= 128 else 16
    short = max_rows // G
    n_short = sum(1 for q in query_lens if 0 < q <= short)
    if n_short:  # the row tile of the decode kernel follows the longest short query actually present (q=1 -> 16 rows)
        short = max(q for q in query_lens if 0 < q <= short)
    TQ = 64 // G
    tiles = sum(-(-q // TQ) for q in query_lens if q > short)
    splits = 1
    if n_short:
        max_s = max((s for q, s in zip(query_lens, seq_lens) if q <= short), default=1)
        splits = choose_decode_splits(n_short * Hkv, max_s, num_sms)
    if force_splits:
        splits = force_splits
    return short, tiles, splits


def paged_attention(q, kv_cache, md, scale, out=None, lse=None, window=0, softcap=0.0, sinks=None):
    """``window`` (tokens, 0 = full), ``softcap`` (0 = off) and ``sinks`` (fp32 ``[Hq]``) select the mma.sync kernels; the tcgen05
    prefill kernel serves plain causal attention with D = 128."""
    global _LAUNCHES
    T, Hq, D = q.shape
    Hkv = kv_cache.shape[2]
    if out is None:
        out = torch.empty(T, Hq, D, dtype=q.dtype, device=q.device)
    plan = getattr(md, "attn_plan", None)
    if plan is None or plan[0] != (Hq, Hkv, D):
        plan = ((Hq, Hkv, D), plan_attention(md.query_lens_cpu, md.seq_lens_cpu, Hq, Hkv, D, _sms(q.device)))
        md.attn_plan = plan
    short, tiles, splits = plan[1]
    n_short = sum(1 for x in md.query_lens_cpu if 0 < x <= short)
    ws_o = ws_ml = None
    if n_short and splits > 1:
        w = workspace(q.device)
        ws_o, ws_ml = (w.attn_static if getattr(md, "static_ws", False) else w.attn)(splits * T * Hq * D, splits * T * Hq * 2)
    if n_short:
        _C.paged_attention(q, kv_cache, out, lse, md.query_start_loc, md.seq_lens, md.block_table, scale, 1, 0, splits,
                           md.max_query_len, short, ws_o, ws_ml, window, softcap, sinks, 1.0, 1.0)
        _LAUNCHES += 2 if splits > 1 else 1
    if tiles:
        if (D == 128 and q.stride(1) == D and _ATTN_PREFILL_TC and not window and not softcap and sinks is None
                and kv_cache.dtype == torch.bfloat16):
            # tcgen05 kernel: 128-token query tiles per (request, head)
            tiles_tc = sum(-(-x // 128) for x in md.query_lens_cpu if x > short)
            _C.paged_attention(q, kv_cache, out, lse, md.query_start_loc, md.seq_lens, md.block_table, scale, 2, tiles_tc, 1,
                               md.max_query_len, short, None, None, 0, 0.0, None, 1.0, 1.0)
        else:
            _C.paged_attention(q, kv_cache, out, lse, md.query_start_loc, md.seq_lens, md.block_table, scale, 0, tiles, 1,
                               md.max_query_len, short, None, None, window, softcap, sinks, 1.0, 1.0)
        _LAUNCHES += 1
    return out


# ----------------------------------------------------------------------------- ops still served by device-side PyTorch
GDN_CHUNK_MIN_LEN = 64  # sequences with at least this many new tokens take the chunked (tensor-core) kernels


def _gdn_chunk_meta(md, device):
    """Chunk list of this step for the chunked Gated-DeltaNet kernels, built once per step from the host-side query lengths:
    int32 ``[chunk_req | chunk_t0 | long_req | long_chunk0]`` on the device (asynchronous copy from pinned memory)."""
    cached = getattr(md, "_gdn_chunks", None)
    if cached is not None:
        return cached
    qlens = getattr(md, "query_lens_cpu", None)
    meta, nc, nl = None, 0, 0
    if qlens and max(qlens) >= GDN_CHUNK_MIN_LEN and not getattr(md, "is_uniform_decode", False):
        creq, ct0, lreq, lc0 = [], [], [], []
        t = 0
        for r, n in enumerate(qlens):
            if n >= GDN_CHUNK_MIN_LEN:
                lreq.append(r)
                lc0.append(len(creq))
                for c in range(0, n, 64):
                    creq.append(r)
                    ct0.append(t + c)
            t += n
        nc, nl = len(creq), len(lreq)
        host = torch.tensor(creq + ct0 + lreq + lc0, dtype=torch.int32).pin_memory()
        meta = host.to(device, non_blocking=True)
        md._gdn_chunks_host = host  # keep the pinned buffer alive until the copy has run
    md._gdn_chunks = (meta, nc, nl)
    return md._gdn_chunks


def gdn_forward(mixed, b, a, conv_w, A_log, dt_bias, conv_state, ssm_state, md, Hk, Hv, K, V):
    """Conv + gating + gated delta rule. Short sequences (decode, verification) run the recurrent kernel; sequences of at least
    ``GDN_CHUNK_MIN_LEN`` new tokens run the chunked tensor-core kernels. Under speculative verification (``md.gdn_record`` set by
    the runner) the slots are left untouched and the state after every token is recorded for the later commit."""
    global _LAUNCHES
    _LAUNCHES += 3
    rec = getattr(md, "gdn_record", None)
    hi = md.has_initial_state if md.has_initial_state.dtype == torch.int32 else md.has_initial_state.to(torch.int32)
    if rec is None:
        meta, nc, nl = _gdn_chunk_meta(md, mixed.device) if os.environ.get("ONECAT_GDN_PREFILL", "chunked") == "chunked" else (None, 0, 0)
        if nl:
            _LAUNCHES += 2
        return _C.gdn_forward(mixed, b, a, conv_w.to(torch.bfloat16), A_log, dt_bias, conv_state, ssm_state, md.query_start_loc, md.state_slots,
                              hi, Hk, Hv, K, V, True, None, meta, nc, nl, GDN_CHUNK_MIN_LEN)
    q = md.spec_q
    spec = torch.empty(md.num_reqs, q, Hv, K, V, dtype=torch.float32, device=mixed.device)
    prev = conv_state[md.state_slots.long()].clone()
    out = _C.gdn_forward(mixed, b, a, conv_w.to(torch.bfloat16), A_log, dt_bias, conv_state, ssm_state, md.query_start_loc, md.state_slots,
                         hi, Hk, Hv, K, V, False, spec, None, 0, 0, 0)
    rec.append(dict(conv_state=conv_state, ssm_state=ssm_state, spec=spec, prev=prev, mixed=mixed, kw=conv_w.shape[1]))
    return out


def gdn_commit(md, rec: list, n_valid: torch.Tensor) -> None:
    """After verification: every Gated-DeltaNet layer takes the state that follows the last accepted token."""
    global _LAUNCHES
    hi = md.has_initial_state if md.has_initial_state.dtype == torch.int32 else md.has_initial_state.to(torch.int32)
    slots = md.state_slots.long()
    ar = torch.arange(md.num_reqs, device=n_valid.device)
    idx = (n_valid.long() - 1).clamp(min=0)
    qlen = md.query_start_loc[1:] - md.query_start_loc[:-1]
    recorded = qlen <= md.spec_q  # longer sequences (prefill chunks) wrote their slot directly
    rs, ridx = slots[recorded], ar[recorded]
    for e in rec:
        e["ssm_state"][rs] = e["spec"][ridx, idx[recorded].clamp(max=e["spec"].shape[1] - 1)]
        _C.gdn_conv_commit(e["mixed"], e["conv_state"], e["prev"], n_valid.to(torch.int32), md.query_start_loc, md.state_slots, hi, e["kw"])
        _LAUNCHES += 2


def prepare_moe(moe) -> None:
    """Stack the local experts for the grouped GEMM. bf16 experts: ``w13`` → ``[E*2I, H]`` with each expert's gate|up rows
    interleaved in blocks of 16 (SiLU·mul happens in the GEMM epilogue), ``w2`` → ``[E*H, I]``. Block-scaled FP8 and MXFP4 experts
    stay packed: tiles + scale words of the stacked matrices, dequantised inside the GEMM."""
    E, I2 = moe.w13.shape[0], moe.w13.shape[1]
    I = I2 // 2
    H = moe.w2.shape[1]
    if I2 % 128 or H % 128 or I % 64:
        moe.kernel_state = None  # odd shapes take the device-side PyTorch path
        return
    perm = interleave_gate_up(I, moe.w13.device)
    q = moe.qmethod
    bn, bk = getattr(moe, "block", None) or (128, 128)
    if q == "fp8" and bk % 64 == 0 and H % bk == 0 and I % bk == 0:
        s13 = moe.w13_scale.float().repeat_interleave(bn, dim=1)[:, :I2][:, perm].reshape(E * I2, -1)
        s2 = moe.w2_scale.float().repeat_interleave(bn, dim=1)[:, :H].reshape(E * H, -1)
        t13, z13, _ = pack_fp8(moe.w13.data.view(torch.uint8)[:, perm].reshape(E * I2, H), s13.contiguous(), bk)
        t2, z2, _ = pack_fp8(moe.w2.data.view(torch.uint8).reshape(E * H, I), s2.contiguous(), bk)
        moe.kernel_state = dict(w13=t13, w2=t2, w13_sz=z13, w2_sz=z2, wkind=2, I2=I2, gk=bk // 64)
    elif q == "mxfp4":
        t13, z13, _ = pack_mxfp4(moe.w13.data[:, perm].reshape(E * I2, H // 2).contiguous(), moe.w13_scale.data[:, perm].reshape(E * I2, -1).contiguous())
        t2, z2, _ = pack_mxfp4(moe.w2.data.reshape(E * H, I // 2).contiguous(), moe.w2_scale.data.reshape(E * H, -1).contiguous())
        moe.kernel_state = dict(w13=t13, w2=t2, w13_sz=z13, w2_sz=z2, wkind=3, I2=I2, gk=1)
    else:
        w13, w2 = moe.dequantized()
        w13s = w13.to(torch.bfloat16)[:, perm, :].reshape(E * I2, H).contiguous()
        w2s = w2.to(torch.bfloat16).reshape(E * H, I).contiguous()
        moe.kernel_state = dict(w13=w13s, w2=w2s, wkind=0)
        if q == "none":  # the stacked copies replace the originals
            moe._dq = None
            moe.w13 = torch.nn.Parameter(w13s.view(E, I2, H), requires_grad=False)
            moe.w2 = torch.nn.Parameter(w2s.view(E, H, I), requires_grad=False)
            moe.kernel_state = dict(w13=moe.w13.view(E * I2, H), w2=moe.w2.view(E * H, I), wkind=0)
            return
    moe._dq = None
    for n in ("w13", "w2", "w13_scale", "w2_scale"):
        if hasattr(moe, n):
            delattr(moe, n)


def route(logits, cfg, bias):
    global _LAUNCHES
    E = logits.shape[1]
    if E % 32 or E > 512 or cfg.num_experts_per_tok > 16:
        TORCH_STANDINS.add("route")
        if cfg.scoring_func == "sigmoid" or cfg.n_group > 1:
            return ref.grouped_topk(logits, cfg.num_experts_per_tok, cfg.n_group, cfg.topk_group, bias, cfg.scoring_func, cfg.norm_topk_prob,
                                    cfg.routed_scaling_factor)
        return ref.topk_softmax(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob)
    _LAUNCHES += 1
    deepseek = cfg.scoring_func == "sigmoid" or cfg.n_group > 1
    return _C.route(logits.to(torch.bfloat16), bias, cfg.num_experts_per_tok, cfg.n_group if deepseek else 1, cfg.topk_group if deepseek else 1,
                    cfg.scoring_func == "sigmoid", cfg.norm_topk_prob, cfg.routed_scaling_factor if deepseek else 1.0)


def fused_moe(moe, x, topk_w, topk_ids):
    global _LAUNCHES
    ks = moe.kernel_state
    if ks is None:
        TORCH_STANDINS.add("fused_moe")
        w13, w2 = moe.dequantized()
        return ref.fused_experts(x, w13, w2, topk_w, topk_ids, moe.e_off)
    ws = workspace(x.device)
    _LAUNCHES += 7
    if x.stride(-1) != 1 or (x.stride(0) * 2) % 16:
        x = x.contiguous()
    return _C.fused_moe(x, ks["w13"], ks["w2"], topk_w.contiguous().float(), topk_ids.contiguous().to(torch.int32), moe.E_local, moe.e_off,
                        ws.splitk, ws.counters, ks.get("wkind", 0), ks.get("w13_sz"), ks.get("w2_sz"), ks.get("I2", 0), ks.get("gk", 1))


def mla_decode(q_abs, q_pe, latent_cache, md, scale, lora):
    global _LAUNCHES
    T, H, _ = q_abs.shape
    if lora != 512 or q_pe.shape[-1] != 64 or q_abs.dtype != torch.bfloat16:
        TORCH_STANDINS.add("mla_decode")
        return ref.mla_decode(q_abs, q_pe, latent_cache, md.block_table, md.query_start_loc, md.seq_lens, scale, lora)
    row_tiles = -(-md.max_query_len * H // 16)
    ws_o = ws_ml = None
    if getattr(md, "static_ws", False) and getattr(md, "attn_plan", None) is not None and md.attn_plan[0][0] == "mla":
        splits = md.attn_plan[1][2]  # captured decode graph: the split count is part of the graph's key, the workspace is static
        if splits > 1:
            so, sm_ = workspace(q_abs.device).s_o, workspace(q_abs.device).s_ml
            assert so.numel() >= splits * T * H * 512 and sm_.numel() >= splits * T * H * 2
            ws_o, ws_ml = so, sm_
    else:
        splits = choose_kv_splits(md.num_reqs * row_tiles, max(md.seq_lens_cpu) if md.seq_lens_cpu else md.max_seq_len, _sms(q_abs.device))
        if splits > 1:
            ws_o, ws_ml = workspace(q_abs.device).attn(splits * T * H * 512, splits * T * H * 2)
    _LAUNCHES += 2 if splits > 1 else 1
    return _C.mla_decode(q_abs.contiguous(), q_pe.contiguous(), latent_cache, md.query_start_loc, md.seq_lens, md.block_table, scale,
                         md.max_query_len, splits, ws_o, ws_ml)


_REJ_STEP = [0]


def rejection_sample(draft_ids, num_draft, target_logits, bonus_ids, md, draft_probs, uniforms, synthetic_rates, gen):
    """Draft probabilities are not used: proposers here emit point-mass (greedy) drafts, for which q(x) = 1."""
    global _LAUNCHES
    _LAUNCHES += 2
    _REJ_STEP[0] += 1
    temp = None if md.all_greedy else md.temperature
    rates = torch.tensor(synthetic_rates, dtype=torch.float32, device=target_logits.device) if synthetic_rates is not None else None
    seed = (gen.initial_seed() if gen is not None else 0) * 1000003 + _REJ_STEP[0]
    return _C.rejection_sample(draft_ids.contiguous(), num_draft, target_logits, bonus_ids, uniforms.contiguous(), temp, rates, seed, not md.all_greedy)
