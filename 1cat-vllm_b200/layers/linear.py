"""Tensor-parallel linear layers with pluggable quantisation methods.

Layer family and sharding rules follow the reference (reference: model_executor/layers/linear.py:449
``ReplicatedLinear``, :630 ``ColumnParallelLinear``, :829 ``MergedColumnParallelLinear``, :1207
``QKVParallelLinear``, :1624 ``RowParallelLinear``); checkpoint layouts follow its quantisation methods
(AWQ layers/quantization/awq.py:59-97,391-432; GPTQ auto_gptq.py:304; FP8 fp8.py:349; NVFP4 modelopt.py:1162;
MXFP4 mxfp4.py:470). A row-parallel layer returns this rank's *partial* sums; the cross-rank reduction is
fused with the following residual-add + RMSNorm (``onecat_vllm.parallel.tp_ops``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from onecat_vllm.config import QuantConfig
from onecat_vllm.ops import ref
from onecat_vllm.parallel.state import get_state


def _p(t: torch.Tensor) -> nn.Parameter:
    return nn.Parameter(t, requires_grad=False)


# ----------------------------------------------------------------------------- quantisation methods
class LinearMethod:
    """``layout(name)`` → (out_axis, out_div, in_axis, in_div) describing how a checkpoint tensor maps to the
    logical [out, in] weight, so one generic loader can shard every format."""

    name = "none"

    def create_weights(self, layer: "LinearBase", in_f: int, out_f: int, dtype: torch.dtype) -> None:
        raise NotImplementedError

    def layout(self, layer, pname: str):
        raise NotImplementedError

    def process_weights_after_loading(self, layer: "LinearBase") -> None:
        pass

    def dequantized_weight(self, layer: "LinearBase") -> torch.Tensor:
        """[out, in] weight in the compute dtype (CPU path and oracle)."""
        raise NotImplementedError

    def apply(self, layer: "LinearBase", x: torch.Tensor) -> torch.Tensor:
        if x.is_cuda:
            from onecat_vllm.ops import cuda as K
            return K.linear(layer, x)
        w = layer._dq_cache
        if w is None:
            w = layer._dq_cache = self.dequantized_weight(layer).detach().to(x.dtype)
        y = F.linear(x, w, layer.bias if hasattr(layer, "bias") and layer.bias is not None else None)
        if layer.fuse_silu_mul:
            y = ref.silu_and_mul(y)
        return y


class UnquantizedMethod(LinearMethod):
    def create_weights(self, layer, in_f, out_f, dtype):
        layer.weight = _p(torch.empty(out_f, in_f, dtype=dtype))

    def layout(self, layer, pname):
        return (0, 1, 1, 1) if pname == "weight" else (0, 1, None, 1)

    def dequantized_weight(self, layer):
        return layer.weight

    def process_weights_after_loading(self, layer):
        if layer.weight.is_cuda and layer.weight.dtype == torch.bfloat16:
            from onecat_vllm.ops import cuda as K
            K.prepare_bf16(layer)


class AWQMethod(LinearMethod):
    name = "awq"

    def __init__(self, q: QuantConfig):
        self.g = q.group_size
        assert q.bits == 4, "AWQ: only 4-bit checkpoints are supported"

    def create_weights(self, layer, in_f, out_f, dtype):
        g = self.g
        assert in_f % g == 0 and out_f % 8 == 0, f"AWQ shapes must divide group/pack size ({in_f}, {out_f})"
        layer.qweight = _p(torch.zeros(in_f, out_f // 8, dtype=torch.int32))
        layer.qzeros = _p(torch.zeros(in_f // g, out_f // 8, dtype=torch.int32))
        layer.scales = _p(torch.zeros(in_f // g, out_f, dtype=torch.float16))

    def layout(self, layer, pname):
        return {"qweight": (1, 8, 0, 1), "qzeros": (1, 8, 0, self.g), "scales": (1, 1, 0, self.g)}.get(pname, (0, 1, None, 1))

    def dequantized_weight(self, layer):
        return ref.awq_dequantize(layer.qweight, layer.qzeros, layer.scales, self.g).t().contiguous()

    def process_weights_after_loading(self, layer):
        if layer.qweight.is_cuda:
            from onecat_vllm.ops import cuda as K
            K.prepare_w4(layer, ref.awq_unpack(layer.qweight).t().contiguous(), ref.awq_unpack(layer.qzeros).t().contiguous(),
                         layer.scales.t().contiguous(), self.g)
            del layer.qweight, layer.qzeros, layer.scales


class GPTQMethod(LinearMethod):
    name = "gptq"

    def __init__(self, q: QuantConfig):
        self.g, self.sym, self.desc_act = q.group_size, q.sym, q.desc_act

    def create_weights(self, layer, in_f, out_f, dtype):
        g = self.g if self.g > 0 else in_f
        layer.qweight = _p(torch.zeros(in_f // 8, out_f, dtype=torch.int32))
        layer.qzeros = _p(torch.zeros(in_f // g, out_f // 8, dtype=torch.int32))
        layer.scales = _p(torch.zeros(in_f // g, out_f, dtype=torch.float16))
        layer.g_idx = _p(torch.arange(in_f, dtype=torch.int32) // g)

    def layout(self, layer, pname):
        g = self.g if self.g > 0 else layer.in_features
        return {"qweight": (1, 1, 0, 8), "qzeros": (1, 8, 0, g), "scales": (1, 1, 0, g), "g_idx": (None, 1, 0, 1)}.get(pname, (0, 1, None, 1))

    def dequantized_weight(self, layer):
        gi = layer.g_idx if self.desc_act else None
        if gi is not None:
            gi = gi - gi.min()
        return ref.gptq_dequantize(layer.qweight, layer.qzeros, layer.scales, gi).t().contiguous()

    def process_weights_after_loading(self, layer):
        if layer.qweight.is_cuda:
            from onecat_vllm.ops import cuda as K
            if self.desc_act:  # act-order permutes K per group: serve through the dense kernel
                layer.weight = _p(self.dequantized_weight(layer).to(layer.compute_dtype))
                layer.method = UnquantizedMethod()
            else:
                K8, N = layer.qweight.shape
                sh = torch.arange(0, 32, 4, device=layer.qweight.device, dtype=torch.int32)
                q = ((layer.qweight.unsqueeze(1) >> sh.view(1, 8, 1)) & 0xF).reshape(K8 * 8, N).to(torch.uint8)
                z = (((layer.qzeros.unsqueeze(-1) >> sh) & 0xF).reshape(layer.qzeros.shape[0], -1) + 1).to(torch.uint8)
                K.prepare_w4(layer, q.t().contiguous(), z.t().contiguous(), layer.scales.t().contiguous(), self.g if self.g > 0 else K8 * 8)
            del layer.qweight, layer.qzeros, layer.scales, layer.g_idx


class FP8Method(LinearMethod):
    """e4m3 weights, per-tensor ``weight_scale`` or 128×128 ``weight_scale_inv`` blocks."""

    name = "fp8"

    def __init__(self, q: QuantConfig):
        self.block = q.weight_block_size
        self.channel = not self.block and q.strategy == "channel"

    def create_weights(self, layer, in_f, out_f, dtype):
        layer.weight = _p(torch.zeros(out_f, in_f, dtype=torch.float8_e4m3fn))
        if self.block:
            bn, bk = self.block
            layer.weight_scale_inv = _p(torch.ones(-(-out_f // bn), -(-in_f // bk), dtype=torch.float32))
        elif self.channel:
            layer.weight_scale = _p(torch.ones(out_f, 1, dtype=torch.float32))   # one scale per output channel, as stored
        else:
            layer.weight_scale = _p(torch.ones(max(len(layer.output_sizes), 1), dtype=torch.float32))

    def layout(self, layer, pname):
        if pname == "weight":
            return (0, 1, 1, 1)
        if pname == "weight_scale_inv":
            return (0, self.block[0], 1, self.block[1])
        if pname == "weight_scale" and self.channel:
            return (0, 1, None, 1)
        return (None, 1, None, 1)

    def dequantized_weight(self, layer):
        if self.block:
            return ref.fp8_block_dequantize(layer.weight, layer.weight_scale_inv, self.block)
        w = layer.weight.float()
        if self.channel:
            return w * layer.weight_scale.float()
        if layer.weight_scale.numel() == 1:
            return w * layer.weight_scale.float()
        outs, o = [], 0
        for i, n in enumerate(layer.local_output_sizes):
            outs.append(w[o:o + n] * layer.weight_scale[i].float())
            o += n
        return torch.cat(outs)

    def process_weights_after_loading(self, layer):
        if layer.weight.is_cuda:
            from onecat_vllm.ops import cuda as K
            K.prepare_fp8(layer, self.block)


class CTInt4Method(LinearMethod):
    """compressed-tensors ``pack-quantized`` int4, symmetric: ``weight_packed [out, in/8]`` int32 holding eight codes along the input
    (code = value + 8, element j in bits 4j..4j+3) and ``weight_scale [out, in/group]``
    (reference: layers/quantization/compressed_tensors/schemes/compressed_tensors_wNa16.py)."""

    name = "ct_w4"

    def __init__(self, q: QuantConfig):
        self.g = q.group_size

    def create_weights(self, layer, in_f, out_f, dtype):
        g = self.g if self.g > 0 else in_f
        layer.weight_packed = _p(torch.zeros(out_f, in_f // 8, dtype=torch.int32))
        layer.weight_scale = _p(torch.ones(out_f, in_f // g, dtype=torch.float16))
        layer.weight_shape = _p(torch.tensor([out_f, in_f], dtype=torch.int64))

    def layout(self, layer, pname):
        g = self.g if self.g > 0 else layer.in_features
        return {"weight_packed": (0, 1, 1, 8), "weight_scale": (0, 1, 1, g)}.get(pname, (None, 1, None, 1))

    def _codes(self, layer):
        sh = torch.arange(0, 32, 4, device=layer.weight_packed.device, dtype=torch.int32)
        return ((layer.weight_packed.unsqueeze(-1) >> sh) & 0xF).reshape(layer.weight_packed.shape[0], -1)

    def dequantized_weight(self, layer):
        q = self._codes(layer).float() - 8.0
        g = q.shape[1] // layer.weight_scale.shape[1]
        return q * layer.weight_scale.float().repeat_interleave(g, dim=1)

    def process_weights_after_loading(self, layer):
        if layer.weight_packed.is_cuda:
            from onecat_vllm.ops import cuda as K
            q = self._codes(layer).to(torch.uint8)
            g = q.shape[1] // layer.weight_scale.shape[1]
            z = torch.full(layer.weight_scale.shape, 8, dtype=torch.uint8, device=q.device)
            K.prepare_w4(layer, q.contiguous(), z, layer.weight_scale.to(torch.float16).contiguous(), g)
            del layer.weight_packed, layer.weight_scale, layer.weight_shape


class FP4Method(LinearMethod):
    """NVFP4 (e2m1 + e4m3 scale /16 + fp32 global scale) and MXFP4 (e2m1 + ue8m0 scale /32)."""

    def __init__(self, q: QuantConfig):
        self.name = q.method
        self.g = 16 if q.method == "nvfp4" else 32

    def create_weights(self, layer, in_f, out_f, dtype):
        layer.weight = _p(torch.zeros(out_f, in_f // 2, dtype=torch.uint8))
        if self.name == "nvfp4":
            layer.weight_scale = _p(torch.ones(out_f, in_f // 16, dtype=torch.float8_e4m3fn))
            layer.weight_scale_2 = _p(torch.ones(1, dtype=torch.float32))
        else:
            layer.weight_scale = _p(torch.full((out_f, in_f // 32), 127, dtype=torch.uint8))

    def layout(self, layer, pname):
        return {"weight": (0, 1, 1, 2), "weight_scale": (0, 1, 1, self.g)}.get(pname, (None, 1, None, 1))

    def dequantized_weight(self, layer):
        if self.name == "nvfp4":
            return ref.nvfp4_dequantize(layer.weight, layer.weight_scale, layer.weight_scale_2)
        return ref.mxfp4_dequantize(layer.weight, layer.weight_scale)

    def process_weights_after_loading(self, layer):
        if layer.weight.is_cuda:
            from onecat_vllm.ops import cuda as K
            K.prepare_fp4(layer, self.name)


def get_linear_method(q: Optional[QuantConfig], prefix: str) -> LinearMethod:
    if q is None or q.method == "none" or any(m in prefix for m in q.modules_to_not_convert):
        return UnquantizedMethod()
    return {"awq": AWQMethod, "gptq": GPTQMethod, "fp8": FP8Method, "nvfp4": FP4Method, "mxfp4": FP4Method, "ct_w4": CTInt4Method}[q.method](q)


# ----------------------------------------------------------------------------- layers
class LinearBase(nn.Module):
    """``output_sizes`` are the *global* logical segments stacked along the output (e.g. q, k, v).
    ``parallel``: "column" shards each segment over TP ranks, "row" shards the input, "replicated" neither."""

    def __init__(self, in_features: int, output_sizes: list[int], parallel: str = "replicated", bias: bool = False,
                 quant: Optional[QuantConfig] = None, prefix: str = "", dtype: torch.dtype = torch.float32,
                 fuse_silu_mul: bool = False, segment_tp: Optional[list[int]] = None) -> None:
        super().__init__()
        st = get_state()
        self.tp, self.tp_rank = st.tp_size, st.tp_rank
        self.parallel, self.prefix, self.compute_dtype = parallel, prefix, dtype
        self.fuse_silu_mul = fuse_silu_mul
        self.in_features_global, self.output_sizes = in_features, list(output_sizes)
        # segment_tp[i]: over how many ranks segment i is split (kv heads may be replicated)
        self.segment_tp = segment_tp or [self.tp if parallel == "column" else 1] * len(output_sizes)
        self.local_output_sizes = [s // t for s, t in zip(self.output_sizes, self.segment_tp)]
        self.in_features = in_features // self.tp if parallel == "row" else in_features
        self.out_features = sum(self.local_output_sizes)
        self.method = get_linear_method(quant, prefix)
        self.method.create_weights(self, self.in_features, self.out_features, dtype)
        # a row-parallel bias is added once, by rank 0
        self.bias = _p(torch.zeros(self.out_features, dtype=dtype)) if bias else None
        self._dq_cache = None
        self.kernel_state = None  # filled by ops.cuda.prepare_*
        self.lora_slots: Optional[dict] = None  # adapter slot -> list of (A, B, first output column); filled by lora.LoRAManager

    def _segment_rank(self, seg: int) -> int:
        t = self.segment_tp[seg]
        return self.tp_rank // (self.tp // t) if t > 0 else 0

    def load_weight(self, pname: str, loaded: torch.Tensor, shard_id: Optional[int] = None) -> None:
        """Copy (the right shard of) a checkpoint tensor into parameter ``pname``.
        ``shard_id`` selects the stacked segment the tensor belongs to; ``None`` = the tensor spans all segments."""
        if pname in ("input_scale", "input_zero_point", "output_scale", "weight_g_idx") and not hasattr(self, pname):
            return  # static activation scales of W8A8 checkpoints: activations stay bf16 here (weight-only use of the weights)
        if pname == "bias" and self.parallel == "row" and self.tp > 1 and self.tp_rank != 0:
            return  # the ranks' outputs are summed: the bias joins once, on rank 0 (the others keep zeros)
        param = getattr(self, pname)
        oa, od, ia, idv = self.method.layout(self, pname) if pname != "bias" else (0, 1, None, 1)
        if loaded.dim() == 0 or (oa is None and loaded.numel() == 1):   # per-tensor scalars arrive as 0-d or one-element tensors
            loaded = loaded.reshape(())
            if shard_id is not None and param.numel() > 1:
                param.data[shard_id] = loaded
            else:
                param.data.fill_(loaded.item())
            return
        if ia is not None and self.parallel == "row" and self.tp > 1:
            n = self.in_features // idv if self.in_features % idv == 0 else -(-self.in_features // idv)
            loaded = loaded.narrow(ia, self.tp_rank * n, n)
        if oa is None:
            param.data.copy_(loaded.reshape(param.shape))
            return
        segs = range(len(self.output_sizes)) if shard_id is None else [shard_id]
        src_off = 0
        for s in segs:
            loc, t = self.local_output_sizes[s], self.segment_tp[s]
            n = -(-loc // od)
            dst_off = sum(self.local_output_sizes[:s]) // od
            if self.parallel == "column" and t > 1:
                a = src_off + self._segment_rank(s) * n
            else:
                a = src_off
            param.data.narrow(oa, dst_off, n).copy_(loaded.narrow(oa, a, n))
            src_off += -(-self.output_sizes[s] // od) if shard_id is None else 0

    def process_weights_after_loading(self) -> None:
        self.method.process_weights_after_loading(self)
        self._dq_cache = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.method.apply(self, x)
        if self.lora_slots:
            from onecat_vllm.lora import apply_lora
            y = apply_lora(self, x, y)
        return y


class ReplicatedLinear(LinearBase):
    def __init__(self, in_f, out_f, **kw):
        super().__init__(in_f, [out_f], "replicated", **kw)


class ColumnParallelLinear(LinearBase):
    def __init__(self, in_f, out_f, **kw):
        super().__init__(in_f, [out_f], "column", **kw)


class MergedColumnParallelLinear(LinearBase):
    def __init__(self, in_f, out_sizes, **kw):
        super().__init__(in_f, list(out_sizes), "column", **kw)


class QKVParallelLinear(LinearBase):
    """q|k|v stacked along the output; KV heads are replicated when there are fewer of them than TP ranks."""

    def __init__(self, hidden, head_dim, num_heads, num_kv_heads, q_mult: int = 1, **kw):
        tp = get_state().tp_size
        kv_tp = min(tp, num_kv_heads)
        self.num_heads, self.num_kv_heads = num_heads // tp, max(num_kv_heads // tp, 1)
        super().__init__(hidden, [num_heads * head_dim * q_mult, num_kv_heads * head_dim, num_kv_heads * head_dim], "column",
                         segment_tp=[tp, kv_tp, kv_tp], **kw)


class RowParallelLinear(LinearBase):
    """Returns partial sums when TP > 1; the caller owns the reduction."""

    def __init__(self, in_f, out_f, **kw):
        super().__init__(in_f, [out_f], "row", **kw)

    def forward(self, x):
        if x.is_cuda and self.tp > 1 and not self.lora_slots:
            from onecat_vllm.ops import cuda as K
            from onecat_vllm.parallel.tp_ops import row_parallel_out
            out = row_parallel_out(x.shape[0], self.out_features, x.dtype, x.device)
            if out is not None and not K._LIB_GEMM:
                # the GEMM epilogue stores its tiles straight into the peers' slabs (reduce-scatter fused into the GEMM)
                fused = get_state().fused
                if fused.use_push(x.shape[0]):
                    y = K.linear(self, x, out=out, push=fused.push_spec(x.shape[0]))
                    y._tp_pushed = True
                    return y
                return K.linear(self, x, out=out)  # partial sums stay in this rank's slot; the reduction pulls them
        return super().forward(x)
