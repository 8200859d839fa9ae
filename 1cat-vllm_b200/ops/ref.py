"""Plain PyTorch restatements of every op.

They serve three roles: the CPU execution path (the tiny-model plumbing run), the fp32 oracle that every CUDA
kernel is tested against, and the timed CPU baseline. Math follows the reference's native/CPU code:
RMSNorm (reference: model_executor/layers/layernorm.py:201 ``forward_native``, Gemma :252-420), NeoX RoPE
(csrc/libtorch_stable/pos_encoding_kernels.cu:77), paged attention (v1/attention/backends/flash_attn_v100.py:2216
``_torch_attention_reference``), AWQ dequant (layers/quantization/awq.py:59-97), gated delta rule
(flash_qla/ops/gated_delta_rule/chunk/sm70/csrc/gdn_forward.cu:131-215), MoE routing
(csrc/moe/topk_softmax_kernels.cu, grouped_topk_kernels.cu), rejection sampling (v1/sample/rejection_sampler.py:896-1026).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms / activations
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None, gemma: bool = False):
    """Returns (normed, new_residual). With ``residual`` the add happens first, in fp32."""
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        new_res = xf.to(x.dtype)
        xf = new_res.float()  # the stored (rounded) residual is what gets normalised
    else:
        new_res = None
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps)
    y = y * (1.0 + w.float()) if gemma else y * w.float()
    return y.to(x.dtype), new_res


def rms_norm_gated(x: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm(x) * w * silu(z) per head (reference: layers/layernorm.py:422 ``RMSNormGated``)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return (y * F.silu(z.float())).to(x.dtype)


def gelu_tanh_and_mul(x: torch.Tensor) -> torch.Tensor:
    """GeGLU: gelu_tanh(gate) * up (reference: layers/activation.py ``GeluAndMul``)."""
    d = x.shape[-1] // 2
    return (F.gelu(x[..., :d].float(), approximate="tanh") * x[..., d:].float()).to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.silu(x[..., :d].float()) * x[..., d:].float()).to(x.dtype)


# ----------------------------------------------------------------------------- rope + kv insert
def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def scaled_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict], device=None):
    """Rotary inverse frequencies under a context-extension rule, and the factor that multiplies cos / sin
    (reference: layers/rotary_embedding/ — linear, llama3, yarn and DeepSeek-yarn variants; the formulas are the published ones)."""
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=device) / rotary_dim))
    kind = (scaling or {}).get("rope_type") or (scaling or {}).get("type") or "default"
    if kind in ("default", "mrope"):   # multimodal rotary sections coincide with the plain rule for text-only positions
        return inv, 1.0
    f = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return inv / f, 1.0
    orig = float(scaling.get("original_max_position_embeddings", 8192))
    if kind == "llama3":
        lo_f, hi_f = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        wavelen = 2 * math.pi / inv
        smooth = ((orig / wavelen - lo_f) / (hi_f - lo_f)).clamp(0, 1)
        out = torch.where(wavelen > orig / lo_f, inv / f, inv)
        mid = (wavelen <= orig / lo_f) & (wavelen >= orig / hi_f)
        return torch.where(mid, (1 - smooth) * inv / f + smooth * inv, out), 1.0
    if kind in ("yarn", "deepseek_yarn"):
        bf, bs = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

        def corr(n_rot):
            return rotary_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

        lo, hi = corr(bf), corr(bs)
        if scaling.get("truncate", True):
            lo, hi = math.floor(lo), math.ceil(hi)
        lo, hi = max(lo, 0), min(hi, rotary_dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = ((torch.arange(rotary_dim // 2, dtype=torch.float32, device=device) - lo) / (hi - lo)).clamp(0, 1)
        extrap = 1.0 - ramp
        out = inv / f * (1 - extrap) + inv * extrap
        if scaling.get("attention_factor") is not None:
            att = float(scaling["attention_factor"])
        elif scaling.get("mscale") and scaling.get("mscale_all_dim"):
            att = yarn_mscale(f, float(scaling["mscale"])) / yarn_mscale(f, float(scaling["mscale_all_dim"]))
        else:
            att = yarn_mscale(f)
        return out, att
    if kind in ("longrope", "su"):
        # Phi-3 long context: per-frequency divisors, the long set when the table extends past the original context
        # (``scaling["max_pos"]`` is filled in by the table builder), and a magnitude factor from the extension ratio
        max_pos = float(scaling.get("max_pos", orig))
        ext = scaling["long_factor"] if max_pos > orig else scaling["short_factor"]
        ratio = float(scaling.get("factor") or (float(scaling.get("max_position_embeddings", max_pos)) / orig))
        att = scaling.get("attention_factor")
        att = float(att) if att is not None else (1.0 if ratio <= 1.0 else math.sqrt(1.0 + math.log(ratio) / math.log(orig)))
        return inv / torch.tensor(ext, dtype=torch.float32, device=device), att
    if kind == "dynamic":
        # NTK-aware base change evaluated once for the extended length ``factor * original`` (reference:
        # layers/rotary_embedding/dynamic_ntk_scaling_rope.py computes its table the same way)
        base = theta * ((f * (orig * f) / orig) - (f - 1.0)) ** (rotary_dim / max(rotary_dim - 2, 1))
        return 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=device) / rotary_dim)), 1.0
    raise ValueError(f"rope scaling type {kind!r} is not supported")


def build_cos_sin_cache(rotary_dim: int, max_pos: int, theta: float, device=None, scaling: Optional[dict] = None) -> torch.Tensor:
    if scaling and (scaling.get("rope_type") or scaling.get("type")) in ("longrope", "su"):
        scaling = dict(scaling, max_pos=max_pos)
    inv, att = scaled_inv_freq(rotary_dim, theta, scaling, device)
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    fr = torch.outer(t, inv)
    return torch.cat([fr.cos() * att, fr.sin() * att], dim=-1)  # [max_pos, rotary_dim] fp32


def _rope_neox(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    xr = x[..., :rotary_dim].float()
    h = rotary_dim // 2
    x1, x2 = xr[..., :h], xr[..., h:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    return torch.cat([out, x[..., rotary_dim:].float()], dim=-1)


def _head_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, gemma: bool) -> torch.Tensor:
    if w is None:
        return x.float()
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * (1.0 + w.float()) if gemma else y * w.float()).to(x.dtype).float()


def rope_and_cache(q, k, v, positions, cos_sin, kv_cache, slot_mapping, rotary_dim: int,
                   q_norm_w=None, k_norm_w=None, eps: float = 1e-6, gemma: bool = False, mrope_section=None) -> None:
    """In place: optional per-head RMSNorm on q/k, NeoX RoPE on the first ``rotary_dim`` dims, then K and V
    rows are written into the paged cache ``[blocks, 2, kv_heads, block_size, head]`` at ``slot_mapping``
    (slot = block * block_size + offset; negative = skip)."""
    T, Hq, D = q.shape
    if mrope_section is not None and positions.dim() == 2:
        # frequency i takes the position component of the section it lies in (reference: rotary_embedding/mrope.py)
        h = rotary_dim // 2
        comp = torch.repeat_interleave(torch.arange(3, device=positions.device), torch.tensor(list(mrope_section), device=positions.device))[:h]
        cs3 = cos_sin[positions.long()]                                     # [3, T, rotary_dim]
        pick = comp.view(1, 1, h).expand(1, T, h)
        cos = torch.gather(cs3[..., :h], 0, pick)[0]
        sin = torch.gather(cs3[..., h:], 0, pick)[0]
    else:
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, : rotary_dim // 2], cs[:, rotary_dim // 2:]
    qn = _rope_neox(_head_norm(q, q_norm_w, eps, gemma), cos, sin, rotary_dim)
    kn = _rope_neox(_head_norm(k, k_norm_w, eps, gemma), cos, sin, rotary_dim)
    q.copy_(qn.to(q.dtype))
    k.copy_(kn.to(k.dtype))
    if kv_cache is not None:
        bs = kv_cache.shape[3]
        sm = slot_mapping.long()
        ok = sm >= 0
        blk, off = sm[ok] // bs, sm[ok] % bs
        if kv_cache.dtype == torch.float8_e4m3fn:  # saturating e4m3 store with unit scales, written through a byte view
            c8 = kv_cache.view(torch.uint8)
            c8[blk, 0, :, off, :] = k[ok].float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            c8[blk, 1, :, off, :] = v[ok].float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
        else:
            kv_cache[blk, 0, :, off, :] = k[ok].to(kv_cache.dtype)
            kv_cache[blk, 1, :, off, :] = v[ok].to(kv_cache.dtype)


# ----------------------------------------------------------------------------- paged attention
def paged_attention(q, kv_cache, block_table, query_start_loc, seq_lens, scale: float,
                    out: Optional[torch.Tensor] = None, return_lse: bool = False, window: int = 0, softcap: float = 0.0,
                    sinks: Optional[torch.Tensor] = None):
    """Causal varlen attention over a paged cache. Request r owns query rows
    ``query_start_loc[r]:query_start_loc[r+1]`` which are the LAST rows of its ``seq_lens[r]``-token context
    (so decode, chunked prefill with prefix and multi-token verify are the same call).
    q ``[T, Hq, D]``, kv_cache ``[blocks, 2, Hkv, bs, D]``. fp32 math. ``window`` > 0: query i sees keys i-window+1..i
    (reference: Gemma2/3, GPT-OSS, Mistral sliding attention); ``softcap`` > 0: scores become cap·tanh(score/cap) (Gemma2);
    ``sinks`` ``[Hq]``: one extra logit per head that takes probability mass but contributes no value (GPT-OSS)."""
    T, Hq, D = q.shape
    Hkv, bs = kv_cache.shape[2], kv_cache.shape[3]
    g = Hq // Hkv
    o = torch.empty_like(q) if out is None else out
    lse = torch.full((T, Hq), -float("inf"), dtype=torch.float32, device=q.device)
    qsl = query_start_loc.tolist()
    sl = seq_lens.tolist()
    for r in range(len(sl)):
        q0, q1, S = qsl[r], qsl[r + 1], sl[r]
        nq = q1 - q0
        if nq == 0:
            continue
        nb = -(-S // bs)
        blocks = block_table[r, :nb].long()
        # an fp8 cache is gathered through a byte view (index ops on float8 tensors are not available everywhere)
        pages = kv_cache.view(torch.uint8)[blocks].view(torch.float8_e4m3fn) if kv_cache.dtype == torch.float8_e4m3fn else kv_cache[blocks]
        kk = pages[:, 0].float().permute(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :S]
        vv = pages[:, 1].float().permute(1, 0, 2, 3).reshape(Hkv, nb * bs, D)[:, :S]
        qq = q[q0:q1].float().permute(1, 0, 2).reshape(Hkv, g, nq, D)
        s = torch.einsum("hgqd,hkd->hgqk", qq, kk) * scale
        qpos = torch.arange(S - nq, S, device=q.device).view(1, 1, nq, 1)
        kpos = torch.arange(S, device=q.device).view(1, 1, 1, S)
        if softcap > 0:
            s = torch.tanh(s / softcap) * softcap
        s = s.masked_fill(kpos > qpos, -float("inf"))
        if window > 0:
            s = s.masked_fill(kpos <= qpos - window, -float("inf"))
        l = torch.logsumexp(s, dim=-1)
        if sinks is not None:
            l = torch.logaddexp(l, sinks.float().view(Hkv, g, 1).expand_as(l))
        p = torch.exp(s - l.unsqueeze(-1))
        oo = torch.einsum("hgqk,hkd->hgqd", p, vv).reshape(Hq, nq, D).permute(1, 0, 2)
        o[q0:q1] = oo.to(o.dtype)
        lse[q0:q1] = l.reshape(Hq, nq).t()
    return (o, lse) if return_lse else o


def merge_attn_states(o1, lse1, o2, lse2):
    """LSE-weighted merge of two partial attention results (reference: csrc/attention/merge_attn_states.cu:19;
    distributed form v1/attention/ops/dcp_alltoall.py:39 ``_lse_weighted_combine``)."""
    m = torch.maximum(lse1, lse2)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    den = (w1 + w2).clamp_min(1e-30)
    o = (o1.float() * (w1 / den).unsqueeze(-1) + o2.float() * (w2 / den).unsqueeze(-1)).to(o1.dtype)
    return o, m + torch.log(den)


def mla_decode(q_nope_abs, q_rope, latent_cache, block_table, query_start_loc, seq_lens, scale: float, kv_lora: int):
    """MLA decode as MQA over the latent cache (reference: csrc/cpu/mla_decode.cpp; layers/attention/mla_attention.py
    ``forward_mqa``). q_nope_abs ``[T,H,kv_lora]`` (W_UK absorbed), q_rope ``[T,H,rope]``, cache
    ``[blocks, bs, kv_lora+rope]``. Returns ``[T,H,kv_lora]`` (to be multiplied by W_UV)."""
    T, H, _ = q_nope_abs.shape
    bs = latent_cache.shape[1]
    out = torch.empty(T, H, kv_lora, dtype=q_nope_abs.dtype, device=q_nope_abs.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    qcat = torch.cat([q_nope_abs, q_rope], dim=-1).float()
    for r in range(len(sl)):
        q0, q1, S = qsl[r], qsl[r + 1], sl[r]
        nq = q1 - q0
        if nq == 0:
            continue
        nb = -(-S // bs)
        kv = latent_cache[block_table[r, :nb].long()].reshape(nb * bs, -1)[:S].float()
        s = torch.einsum("qhd,kd->hqk", qcat[q0:q1], kv) * scale
        qpos = torch.arange(S - nq, S, device=kv.device).view(1, nq, 1)
        s = s.masked_fill(torch.arange(S, device=kv.device).view(1, 1, S) > qpos, -float("inf"))
        p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("hqk,kd->qhd", p, kv[:, :kv_lora]).to(out.dtype)
    return out


# ----------------------------------------------------------------------------- quantised weights
AWQ_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)  # nibble i of an int32 holds column AWQ_ORDER[i] of the 8-column group


def awq_unpack(qweight: torch.Tensor) -> torch.Tensor:
    """int32 ``[K, N/8]`` → uint8 ``[K, N]`` values 0..15 in natural column order."""
    K, N8 = qweight.shape
    shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
    nib = (qweight.unsqueeze(-1) >> shifts) & 0xF  # [K, N8, 8] nibble i
    inv = torch.empty(8, dtype=torch.long, device=qweight.device)
    for i, c in enumerate(AWQ_ORDER):
        inv[c] = i
    return nib[..., inv].reshape(K, N8 * 8).to(torch.uint8)


def awq_pack(w: torch.Tensor) -> torch.Tensor:
    """uint8 ``[K, N]`` (0..15) → int32 ``[K, N/8]`` in AWQ nibble order."""
    K, N = w.shape
    w = w.reshape(K, N // 8, 8).to(torch.int64)
    out = torch.zeros(K, N // 8, dtype=torch.int64, device=w.device)
    for i, c in enumerate(AWQ_ORDER):
        out |= w[..., c] << (4 * i)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def awq_dequantize(qweight, qzeros, scales, group_size: int = 128) -> torch.Tensor:
    """W[k,n] = (q[k,n] - z[k/g,n]) * s[k/g,n]; returns ``[K, N]`` in the dtype of ``scales``."""
    q = awq_unpack(qweight).float()
    z = awq_unpack(qzeros).float().repeat_interleave(group_size, dim=0)
    s = scales.float().repeat_interleave(group_size, dim=0)
    return ((q - z) * s).to(scales.dtype)


def gptq_dequantize(qweight, qzeros, scales, g_idx=None, bits: int = 4, sym: bool = True) -> torch.Tensor:
    """GPTQ: int32 ``[K/8, N]`` packed along K, zeros ``[K/g, N/8]`` packed along N storing ``z-1``
    (reference: layers/quantization/auto_gptq.py:304-520)."""
    K8, N = qweight.shape
    shifts = torch.arange(0, 32, 4, device=qweight.device, dtype=torch.int32)
    q = ((qweight.unsqueeze(1) >> shifts.view(1, 8, 1)) & 0xF).reshape(K8 * 8, N).float()
    z = ((qzeros.unsqueeze(-1) >> shifts) & 0xF).reshape(qzeros.shape[0], -1).float() + 1.0
    K = K8 * 8
    g = g_idx.long() if g_idx is not None else torch.arange(K, device=q.device) // (K // scales.shape[0])
    return ((q - z[g]) * scales.float()[g]).to(scales.dtype)


_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def fp4_unpack(packed: torch.Tensor) -> torch.Tensor:
    """uint8 ``[..., K/2]`` (low nibble first) → fp32 ``[..., K]`` e2m1 values."""
    lut = _E2M1.to(packed.device)
    lo, hi = (packed & 0xF).long(), (packed >> 4).long()
    return torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)


def mxfp4_dequantize(packed: torch.Tensor, scales_ue8m0: torch.Tensor) -> torch.Tensor:
    """e2m1 + one ue8m0 (2^(e-127)) scale per 32 elements (reference: layers/quantization/mxfp4.py:470-803)."""
    v = fp4_unpack(packed)
    s = torch.exp2(scales_ue8m0.float() - 127.0).repeat_interleave(32, dim=-1)
    return v * s


def nvfp4_dequantize(packed: torch.Tensor, scales_e4m3: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """e2m1 + e4m3 scale per 16 elements + fp32 global scale (reference: utils/nvfp4_emulation_utils.py)."""
    v = fp4_unpack(packed)
    s = scales_e4m3.float().repeat_interleave(16, dim=-1)
    return v * s * global_scale.float()


def fp8_block_dequantize(w_fp8: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    """e4m3 ``[N, K]`` with one fp32 scale per ``block`` (reference: layers/quantization/utils/fp8_utils.py)."""
    N, K = w_fp8.shape[-2:]
    s = scale_inv.float().repeat_interleave(block[0], dim=-2)[..., :N, :].repeat_interleave(block[1], dim=-1)[..., :K]
    return w_fp8.float() * s


def fp8_per_token_group_quant(x: torch.Tensor, group: int = 128):
    """Dynamic 1×128 activation quantisation → (e4m3 values, fp32 scales)."""
    T, K = x.shape
    xg = x.float().reshape(T, K // group, group)
    amax = xg.abs().amax(-1, keepdim=True).clamp_min(1e-10)
    s = amax / 448.0
    q = (xg / s).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.reshape(T, K), s.squeeze(-1)


# ----------------------------------------------------------------------------- gated delta net
def causal_conv1d(x, weight, bias, conv_state, query_start_loc, state_slots, has_initial_state, activation: bool = True):
    """Depthwise causal conv (kernel k) over varlen sequences with a rolling state of the last k-1 inputs.
    x ``[T, C]``, weight ``[C, k]``, conv_state ``[slots, C, k-1]`` updated in place
    (reference: layers/mamba/ops/causal_conv1d.py:16,746)."""
    T, C = x.shape
    kw = weight.shape[1]
    out = torch.empty_like(x)
    qsl = query_start_loc.tolist()
    for r in range(len(qsl) - 1):
        a, b = qsl[r], qsl[r + 1]
        if a == b:
            continue
        slot = int(state_slots[r])
        prev = conv_state[slot].float() if bool(has_initial_state[r]) else torch.zeros(C, kw - 1, device=x.device)
        seq = torch.cat([prev.t(), x[a:b].float()], dim=0)  # [k-1+L, C]
        win = seq.unfold(0, kw, 1)  # [L, C, k]
        y = (win * weight.float().unsqueeze(0)).sum(-1)
        if bias is not None:
            y = y + bias.float()
        out[a:b] = (F.silu(y) if activation else y).to(x.dtype)
        conv_state[slot] = seq[-(kw - 1):].t().to(conv_state.dtype)
    return out


def conv_state_after(prev: torch.Tensor, x_chunk: torch.Tensor, n: int) -> torch.Tensor:
    """Conv state ``[C, k-1]`` after consuming the first ``n`` rows of ``x_chunk`` ``[L, C]`` starting from ``prev``."""
    m = prev.shape[1]
    seq = torch.cat([prev.t().float(), x_chunk[:n].float()], dim=0)
    return seq[-m:].t().to(prev.dtype)


def gdn_gating(a, b, A_log, dt_bias):
    """g = -exp(A_log) * softplus(a + dt_bias) (log-space decay), beta = sigmoid(b)
    (reference: layers/mamba/gdn/qwen_gdn_linear_attn.py:6945-7013)."""
    g = -torch.exp(A_log.float()) * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def _l2norm(x, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).sum(-1, keepdim=True) + eps)


def gated_delta_rule(q, k, v, g, beta, state, query_start_loc, state_slots, has_initial_state, scale: Optional[float] = None,
                     use_qk_l2norm: bool = True, token_states: Optional[torch.Tensor] = None):
    """Sequential gated delta rule, fp32 state ``[slots, Hv, K, V]`` updated in place:
    ``S <- e^g S + k (x) ((v - (e^g S)^T k) beta)``, ``o = S^T q * scale``. q,k ``[T,Hk,K]``, v ``[T,Hv,V]``,
    g,beta ``[T,Hv]``. This token-by-token form is the oracle for both the chunked prefill and the
    recurrent decode kernels."""
    T, Hk, K = q.shape
    Hv, V = v.shape[1], v.shape[2]
    rep = Hv // Hk
    scale = K ** -0.5 if scale is None else scale
    qf, kf = q.float(), k.float()
    if use_qk_l2norm:
        qf, kf = _l2norm(qf), _l2norm(kf)
    qf = qf.repeat_interleave(rep, dim=1) * scale
    kf = kf.repeat_interleave(rep, dim=1)
    out = torch.empty(T, Hv, V, dtype=v.dtype, device=v.device)
    qsl = query_start_loc.tolist()
    for r in range(len(qsl) - 1):
        a, b = qsl[r], qsl[r + 1]
        if a == b:
            continue
        slot = int(state_slots[r])
        S = state[slot].float().clone() if bool(has_initial_state[r]) else torch.zeros(Hv, K, V, device=v.device)
        for t in range(a, b):
            S = S * torch.exp(g[t].float()).view(Hv, 1, 1)
            kv = torch.einsum("hk,hkv->hv", kf[t], S)
            delta = (v[t].float() - kv) * beta[t].float().view(Hv, 1)
            S = S + torch.einsum("hk,hv->hkv", kf[t], delta)
            out[t] = torch.einsum("hk,hkv->hv", qf[t], S).to(out.dtype)
            if token_states is not None and (b - a) <= token_states.shape[1]:
                token_states[r, t - a] = S
        if token_states is None or (b - a) > token_states.shape[1]:
            state[slot] = S.to(state.dtype)
    return out


# ----------------------------------------------------------------------------- MoE
def topk_softmax(logits: torch.Tensor, k: int, renormalize: bool):
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def grouped_topk(logits, k: int, n_group: int, topk_group: int, bias=None, scoring: str = "sigmoid",
                 renormalize: bool = True, scaling: float = 1.0):
    """DeepSeek-V3 routing: score, pick ``topk_group`` groups by the sum of their top-2 biased scores, then
    top-k inside them; weights come from the un-biased scores (reference: models/deepseek_v2.py:245-388,
    csrc/moe/grouped_topk_kernels.cu:516)."""
    s = torch.sigmoid(logits.float()) if scoring == "sigmoid" else torch.softmax(logits.float(), -1)
    sb = s + bias.float() if bias is not None else s
    T, E = s.shape
    gs = sb.view(T, n_group, E // n_group)
    group_score = gs.topk(2, dim=-1)[0].sum(-1) if bias is not None else gs.max(-1)[0]
    gi = group_score.topk(topk_group, dim=-1)[1]
    mask = torch.zeros(T, n_group, device=s.device, dtype=torch.bool).scatter_(1, gi, True)
    masked = sb.masked_fill(~mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E), -float("inf"))
    ids = masked.topk(k, dim=-1)[1]
    w = s.gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * scaling, ids.to(torch.int32)


def swiglu_oai(h: torch.Tensor, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
    """GPT-OSS gated activation on ``[gate | up]``: ``(up + 1) * gate * sigmoid(alpha * gate)`` with gate clamped from above and up
    clamped on both sides (reference: layers/activation.py ``SwigluOAIAndMul``)."""
    d = h.shape[-1] // 2
    gate, up = h[..., :d].float().clamp(max=limit), h[..., d:].float().clamp(-limit, limit)
    return ((up + 1.0) * gate * torch.sigmoid(gate * alpha)).to(h.dtype)


def fused_experts(x, w13, w2, topk_w, topk_ids, expert_offset: int = 0, b13=None, b2=None, act: str = "silu", mm=None):
    """Per-expert SwiGLU FFNs, weighted sum over each token's top-k. ``w13`` ``[E_local, 2I, H]``,
    ``w2`` ``[E_local, H, I]`` hold experts ``expert_offset .. expert_offset+E_local``; tokens routed elsewhere
    contribute nothing (reference: csrc/cpu/cpu_fused_moe.cpp)."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w13.shape[0]
    for e in range(E):
        sel = (topk_ids == e + expert_offset)
        tok = sel.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        wt = (topk_w * sel).sum(-1)[tok]
        if mm is not None:   # device path: ``mm(x, w)`` = x @ w^T in the model dtype
            h = mm(x[tok].contiguous(), w13[e]).float()
        else:
            h = F.linear(x[tok].float(), w13[e].float())
        if b13 is not None:
            h = h + b13[e].float()
        h = silu_and_mul(h) if act == "silu" else swiglu_oai(h)
        o = mm(h.to(x.dtype).contiguous(), w2[e]).float() if mm is not None else F.linear(h, w2[e].float())
        if b2 is not None:
            o = o + b2[e].float()
        out[tok] += o * wt.unsqueeze(-1)
    return out.to(x.dtype)


# ----------------------------------------------------------------------------- sampling
def apply_penalties(logits, prompt_mask, output_counts, presence, frequency, repetition):
    """logits ``[B,V]`` fp32; ``prompt_mask`` bool ``[B,V]``; ``output_counts`` ``[B,V]``
    (reference: csrc/libtorch_stable/sampler.cu:14; v1/sample/ops/penalties.py)."""
    seen = prompt_mask | (output_counts > 0)
    rp = repetition.view(-1, 1)
    logits = torch.where(seen, torch.where(logits > 0, logits / rp, logits * rp), logits)
    logits = logits - frequency.view(-1, 1) * output_counts.float()
    logits = logits - presence.view(-1, 1) * (output_counts > 0).float()
    return logits


def top_k_top_p_min_p(logits, top_k, top_p, min_p):
    """Mask logits outside top-k / nucleus / min-p (reference: v1/sample/ops/topk_topp_sampler.py:323)."""
    B, V = logits.shape
    if min_p is not None and bool((min_p > 0).any()):
        p = torch.softmax(logits, -1)
        thr = p.max(-1, keepdim=True)[0] * min_p.view(-1, 1)
        logits = logits.masked_fill(p < thr, -float("inf"))
    srt, idx = logits.sort(dim=-1, descending=False)
    if top_k is not None:
        kk = torch.where(top_k <= 0, torch.full_like(top_k, V), top_k).clamp(max=V).long()
        thr = srt.gather(1, (V - kk).view(-1, 1))
        srt = srt.masked_fill(srt < thr, -float("inf"))
    if top_p is not None:
        pr = torch.softmax(srt, -1)
        cum = pr.cumsum(-1)
        mask = cum <= (1 - top_p.view(-1, 1))
        mask[:, -1] = False
        srt = srt.masked_fill(mask, -float("inf"))
    return torch.empty_like(logits).scatter_(1, idx, srt)


def random_sample(probs: torch.Tensor, generators: dict, default_gen: Optional[torch.Generator] = None) -> torch.Tensor:
    """argmax(p / Exp(1)) with per-request generators (reference: v1/sample/ops/topk_topp_sampler.py:417-438)."""
    q = torch.empty_like(probs)
    if len(generators) != probs.shape[0]:
        q.exponential_(generator=default_gen)
    for i, gen in generators.items():
        q[i].exponential_(generator=gen)
    return (probs / q).argmax(-1)


def rejection_sample(draft_ids, num_draft, target_logits_or_probs, bonus_ids, draft_probs=None, uniforms=None,
                     greedy: Optional[torch.Tensor] = None, synthetic_rates: Optional[list[float]] = None,
                     exp_noise: Optional[torch.Tensor] = None, pad: int = -1):
    """Sequential verification of ``k`` drafts per request.
    draft_ids ``[B,k]``; target probs ``[B,k,V]`` (argmax is used when ``greedy[b]``); bonus_ids ``[B]``;
    uniforms ``[B,k]`` float64. Returns ``[B,k+1]`` padded with ``pad``.
    greedy: accept while draft == argmax(target); on the first mismatch emit the argmax.
    random: accept iff p_t(x)/p_d(x) >= u (p_d = 1 without draft probs); on reject emit the recovered token
    argmax(max(p_t - p_d, 0) / Exp). synthetic: accept iff u < rate[pos]; the emitted token on reject is the
    same recovered token. All accepted → append the bonus token."""
    B, k = draft_ids.shape
    out = torch.full((B, k + 1), pad, dtype=torch.long, device=draft_ids.device)
    tp = target_logits_or_probs
    for b in range(B):
        n = int(num_draft[b])
        is_greedy = bool(greedy[b]) if greedy is not None else False
        rejected = False
        for i in range(n):
            d = int(draft_ids[b, i])
            if synthetic_rates is not None:
                accept = float(uniforms[b, i]) < synthetic_rates[i]
            elif is_greedy:
                accept = d == int(tp[b, i].argmax())
            else:
                pd = float(draft_probs[b, i, d]) if draft_probs is not None else 1.0
                accept = pd > 0 and float(tp[b, i, d]) / pd >= float(uniforms[b, i])
            if accept:
                out[b, i] = d
                continue
            if is_greedy:
                out[b, i] = int(tp[b, i].argmax())
            else:
                resid = tp[b, i].float().clone()
                if draft_probs is not None:
                    resid = (resid - draft_probs[b, i].float()).clamp_min(0)
                else:
                    resid[d] = 0.0
                noise = exp_noise[b, i] if exp_noise is not None else torch.ones_like(resid)
                out[b, i] = int((resid / noise).argmax())
            rejected = True
            break
        if not rejected:
            out[b, n] = int(bonus_ids[b])
    return out


# ----------------------------------------------------------------------------- Mamba-2 (state-space duality) scan
def mamba2_scan(x, dt, A, B, C, D, ssm_state, query_start_loc, state_slots, has_initial_state, chunk: int = 64):
    """Selective state-space recurrence of Mamba-2 over varlen sequences, state per (sequence, head) kept in ``ssm_state``
    ``[slots, H, P, N]`` fp32 and updated in place:  ``h_t = exp(dt_t A) h_{t-1} + dt_t x_t ⊗ B_t``,  ``y_t = h_t C_t + D x_t``.
    x ``[T, H, P]``, dt ``[T, H]`` (after softplus), A ``[H]`` (negative), B / C ``[T, G, N]`` with H a multiple of G, D ``[H]``.
    Sequences longer than one token run the chunked form (quadratic inside a chunk of ``chunk`` tokens, a recurrence over chunk
    states between them), single tokens the recurrence itself
    (reference: layers/mamba/ops/ssd_combined.py ``mamba_chunk_scan_combined``; layers/mamba/ops/mamba_ssm.py ``selective_state_update``)."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    y = torch.empty(T, H, P, dtype=torch.float32, device=x.device)
    qsl = query_start_loc.tolist()
    Af, Df = A.float(), D.float()
    for r in range(len(qsl) - 1):
        a, b = qsl[r], qsl[r + 1]
        L = b - a
        if L == 0:
            continue
        slot = int(state_slots[r])
        h = ssm_state[slot].float() if bool(has_initial_state[r]) else torch.zeros(H, P, N, device=x.device)
        xs, dts = x[a:b].float(), dt[a:b].float()
        Bs = B[a:b].float().repeat_interleave(rep, dim=1)       # [L, H, N]
        Cs = C[a:b].float().repeat_interleave(rep, dim=1)
        if L == 1:
            h = h * torch.exp(dts[0] * Af).view(H, 1, 1) + (dts[0].view(H, 1) * xs[0]).unsqueeze(-1) * Bs[0].unsqueeze(1)
            y[a] = torch.einsum("hpn,hn->hp", h, Cs[0]) + Df.view(H, 1) * xs[0]
            ssm_state[slot] = h
            continue
        for c0 in range(0, L, chunk):
            c1 = min(c0 + chunk, L)
            xc, dtc, Bc, Cc = xs[c0:c1], dts[c0:c1], Bs[c0:c1], Cs[c0:c1]
            cum = torch.cumsum(dtc * Af, dim=0)                  # [Q, H] log-decay from the chunk start up to and including t
            # inside the chunk: y_i += sum_{j <= i} exp(cum_i - cum_j) (C_i . B_j) dt_j x_j
            decay = torch.exp((cum.unsqueeze(1) - cum.unsqueeze(0)).permute(2, 0, 1))            # [H, Q(i), Q(j)]
            decay = torch.tril(decay)
            cb = torch.einsum("ihn,jhn->hij", Cc, Bc)
            yc = torch.einsum("hij,jh,jhp->ihp", cb * decay, dtc, xc)
            # the state carried into the chunk
            yc = yc + torch.einsum("ihn,hpn,ih->ihp", Cc, h, torch.exp(cum))
            y[a + c0:a + c1] = yc + Df.view(1, H, 1) * xc
            # state after the chunk
            tail = torch.exp(cum[-1].unsqueeze(0) - cum)         # [Q, H] decay from t to the chunk end
            h = h * torch.exp(cum[-1]).view(H, 1, 1) + torch.einsum("jh,jh,jhp,jhn->hpn", tail, dtc, xc, Bc)
        ssm_state[slot] = h
    return y


def mamba1_scan(x, dt, A, B, C, D, ssm_state, query_start_loc, state_slots, has_initial_state):
    """Selective scan of Mamba-1 over varlen sequences: one state ``[d_inner, N]`` per sequence in ``ssm_state`` ``[slots, 1, d_inner, N]``
    fp32, updated in place:  ``h_t = exp(dt_t ⊗ A) h_{t-1} + (dt_t x_t) ⊗ B_t``,  ``y_t = h_t C_t + D x_t``.
    x, dt ``[T, d_inner]`` (dt after softplus), A ``[d_inner, N]`` (negative), B / C ``[T, N]``, D ``[d_inner]``. The decay differs per
    channel and state index, so the recurrence runs token by token, vectorised over channels
    (reference: layers/mamba/ops/mamba_ssm.py ``selective_scan_fn`` / ``selective_state_update``)."""
    T, Di = x.shape
    y = torch.empty(T, Di, dtype=torch.float32, device=x.device)
    qsl = query_start_loc.tolist()
    Af, Df = A.float(), D.float()
    for r in range(len(qsl) - 1):
        a, b = qsl[r], qsl[r + 1]
        if a == b:
            continue
        slot = int(state_slots[r])
        h = ssm_state[slot, 0].float() if bool(has_initial_state[r]) else torch.zeros(Di, Af.shape[1], device=x.device)
        xs, dts, Bs, Cs = x[a:b].float(), dt[a:b].float(), B[a:b].float(), C[a:b].float()
        dA = torch.exp(dts.unsqueeze(-1) * Af.unsqueeze(0))                  # [L, d_inner, N]
        dBx = (dts * xs).unsqueeze(-1) * Bs.unsqueeze(1)                     # [L, d_inner, N]
        for t in range(b - a):
            h = dA[t] * h + dBx[t]
            y[a + t] = h @ Cs[t] + Df * xs[t]
        ssm_state[slot, 0] = h
    return y
