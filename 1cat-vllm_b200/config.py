"""Engine configuration: ``EngineArgs`` → ``VllmConfig`` composed of typed sub-configs.

Mirrors the reference's configuration surface at a much smaller scale
(reference: vllm/engine/arg_utils.py, vllm/config/vllm.py, config/model.py,
config/cache.py, config/parallel.py, config/scheduler.py, config/speculative.py).
Each sub-config validates itself in ``__post_init__`` and exposes ``compute_hash``.
"""
from __future__ import annotations

import argparse
import dataclasses
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional, Union

import torch

_DTYPES = {
    "auto": None, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
    "half": torch.float16, "fp16": torch.float16, "float32": torch.float32, "float": torch.float32, "fp32": torch.float32,
}


def _hash(obj: Any) -> str:
    return hashlib.sha256(json.dumps(obj, sort_keys=True, default=str).encode()).hexdigest()[:16]


# ----------------------------------------------------------------------------- model
@dataclass
class QuantConfig:
    """Checkpoint quantisation layout (reference: model_executor/layers/quantization/__init__.py:12-45)."""

    method: str = "none"  # none | awq | gptq | fp8 | nvfp4 | mxfp4 | ct_w4 (compressed-tensors pack-quantized int4)
    bits: int = 4
    group_size: int = 128
    zero_point: bool = True  # AWQ asymmetric
    desc_act: bool = False  # GPTQ act-order
    sym: bool = True  # GPTQ symmetric uint4b8
    weight_block_size: Optional[tuple[int, int]] = None  # fp8 128x128
    activation_scheme: str = "dynamic"
    modules_to_not_convert: list[str] = field(default_factory=lambda: ["lm_head", "embed_tokens"])
    expert_method: Optional[str] = None  # mixed precision: quant method of routed experts (e.g. mxfp4)
    strategy: str = "tensor"  # fp8 without blocks: one scale per tensor or per output channel

    @classmethod
    def from_hf(cls, q: Optional[dict]) -> "QuantConfig":
        if not q:
            return cls()
        m = (q.get("quant_method") or q.get("quant_algo") or "none").lower()
        if m in ("awq", "awq_marlin"):
            return cls("awq", q.get("bits", q.get("w_bit", 4)), q.get("group_size", q.get("q_group_size", 128)),
                       q.get("zero_point", True), modules_to_not_convert=q.get("modules_to_not_convert") or ["lm_head", "embed_tokens"])
        if m in ("gptq", "gptq_marlin", "auto_gptq"):
            return cls("gptq", q.get("bits", 4), q.get("group_size", 128), zero_point=not q.get("sym", True),
                       desc_act=q.get("desc_act", False), sym=q.get("sym", True))
        if m == "fp8":
            wbs = q.get("weight_block_size")
            return cls("fp8", 8, 0, False, weight_block_size=tuple(wbs) if wbs else None,
                       activation_scheme=q.get("activation_scheme", "dynamic"), expert_method=q.get("expert_method"),
                       modules_to_not_convert=(q.get("modules_to_not_convert") or q.get("ignored_layers") or []) + ["lm_head", "embed_tokens"])
        if m == "compressed-tensors":
            # llm-compressor checkpoints (reference: layers/quantization/compressed_tensors/): the first config group decides
            groups = q.get("config_groups") or {}
            w = (next(iter(groups.values())) if groups else {}).get("weights") or {}
            skip = [x for x in (q.get("ignore") or []) if not x.startswith("re:")] + ["lm_head", "embed_tokens"]
            if w.get("type") == "float" and w.get("num_bits") == 8 and w.get("strategy", "tensor") in ("tensor", "channel"):
                return cls("fp8", 8, 0, False, strategy=w.get("strategy", "tensor"), modules_to_not_convert=skip)
            if w.get("type") == "int" and w.get("num_bits") == 4 and q.get("format", "pack-quantized") == "pack-quantized":
                if not w.get("symmetric", True) or w.get("actorder"):
                    raise ValueError("compressed-tensors int4: only symmetric weights without activation ordering are supported")
                return cls("ct_w4", 4, int(w.get("group_size") or -1), False, sym=True, modules_to_not_convert=skip)
            raise ValueError(f"unsupported compressed-tensors scheme: {w}")
        if m in ("nvfp4", "modelopt_fp4", "modelopt"):
            return cls("nvfp4", 4, 16, False)
        if m in ("mxfp4",):
            return cls("mxfp4", 4, 32, False)
        raise ValueError(f"unsupported quantization method {m!r}")


@dataclass
class ModelConfig:
    """Architecture description, normalised from an HF ``config.json`` (or a dict for synthetic models).

    Covers the architectures of the reference's model zoo that this engine serves:
    dense Llama/Qwen2/Qwen3 (reference: models/llama.py, qwen3.py), Qwen3-Next/Qwen3.5 hybrids with
    Gated-DeltaNet (models/qwen3_next.py:319-1092), Qwen3-MoE, DeepSeek-V2/V3 MLA+MoE (models/deepseek_v2.py).
    """

    model: str = "dummy"
    architecture: str = "LlamaForCausalLM"
    vocab_size: int = 32000
    hidden_size: int = 256
    intermediate_size: int = 688
    num_hidden_layers: int = 4
    num_attention_heads: int = 8
    num_key_value_heads: int = 2
    head_dim: int = 32
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    partial_rotary_factor: float = 1.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False  # per-head RMSNorm on q and k (Qwen3)
    gemma_norm: bool = False  # weight applied as (1 + w) (Qwen3-Next)
    attn_output_gate: bool = False  # gated attention: o * sigmoid(gate)
    # Gemma / GLM / Granite family switches
    hidden_act: str = "silu"  # silu | gelu_tanh (GeGLU)
    embed_scale: float = 1.0  # token embeddings are multiplied by this (Gemma: sqrt(hidden); Granite: embedding_multiplier)
    sandwich_norm: bool = False  # each sub-block's output is normalised before it joins the residual (Gemma2/3, GLM-4)
    attn_scale: Optional[float] = None  # softmax scale when it is not head_dim ** -0.5
    attn_softcap: float = 0.0  # tanh soft-capping of attention scores (Gemma2)
    final_softcap: float = 0.0  # tanh soft-capping of the output logits (Gemma2)
    sliding_window: int = 0  # window of the layers listed in sliding_layers
    sliding_layers: tuple = ()
    rope_local_theta: Optional[float] = None  # rotary base of the sliding layers when it differs (Gemma3)
    rope_scaling: Optional[dict] = None  # {"rope_type": linear | llama3 | yarn | dynamic, ...} of the full-attention layers
    rope_interleaved: bool = False  # checkpoint rotates adjacent pairs (GLM); q/k rows are permuted to the half-split layout at load
    residual_multiplier: float = 1.0  # Granite: sub-block outputs are scaled before the residual add
    logit_scale: float = 1.0  # logits are multiplied by this (Granite: 1 / logits_scaling)
    attn_sinks: bool = False  # one learned sink logit per query head joins the softmax denominator (GPT-OSS)
    attn_o_bias: bool = False  # bias on the attention output projection
    mlp_bias: bool = False  # biases on the dense feed-forward projections (Llama / Granite ``mlp_bias``)
    norm_type: str = "rms"  # rms | layernorm (mean-and-variance normalisation; ``gemma_norm`` then means the weight is stored minus one)
    norm_affine: bool = True  # False: the layer norm has no learned parameters (OLMo)
    norm_bias: bool = False  # the layer norm has a bias
    parallel_block: bool = False  # h += attn(norm(h)) + mlp(norm(h)) with one norm per block (Cohere)
    qkv_clip: Optional[float] = None  # clamp of the q / k / v projections (OLMo ``clip_qkv``)
    mlp_gated: bool = True  # False: down(act(up(x))) without a gate projection (Arcee: squared ReLU)
    router_linear_bias: bool = False  # the router is a linear layer with bias
    expert_bias: bool = False  # every expert projection has a bias
    moe_act: str = "silu"  # silu | swiglu_oai: (up + 1) * gate * sigmoid(1.702 gate) with gate <= 7 and |up| <= 7 (GPT-OSS)
    router_bias: bool = False  # softmax routing whose top-k selection adds a learned per-expert bias (Ernie-4.5-MoE)
    qk_norm_after_rope: bool = False  # per-head q / k RMSNorm applied to the rotated vectors (HunYuan) instead of before the rotation
    nope_layers: tuple = ()  # layers whose attention applies no rotary embedding (SmolLM3)
    pre_norm: bool = True  # False: no norm before a sub-block, its output is normalised and added (OLMo-2 / OLMo-3)
    qk_norm_full: bool = False  # q / k RMSNorm over the whole projection instead of per head (OLMo-2 / OLMo-3)
    num_labels: int = 0  # > 0: a *ForSequenceClassification checkpoint (a ``score`` head on the pooled state instead of an LM head)
    # hybrid (Gated-DeltaNet)
    layer_types: Optional[list[str]] = None  # "full_attention" | "linear_attention" (Gated-DeltaNet) | "mamba2" | "mamba1" | "short_conv"
    # Mamba-2 mixers (Bamba, Mamba2): heads x head size = inner width; B / C groups of the state size; conv kernel
    mamba_n_heads: int = 0
    mamba_d_head: int = 64
    mamba_n_groups: int = 1
    mamba_d_state: int = 128
    mamba_d_conv: int = 4
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    mamba_time_step_limit: tuple = (0.0, float("inf"))
    mamba_norm_groups: int = 1   # groups of the gated RMSNorm over the inner width
    mamba_dt_rank: int = 0       # Mamba-1: width of the low-rank time-step projection
    mamba_inner_rms_eps: Optional[float] = None  # FalconMamba: RMS normalisation (no weights) of dt / B / C inside the mixer
    mamba_inner_norm_weights: bool = False  # Jamba: RMSNorm layers with weights on dt / B / C inside the mixer
    mixer_only_layers: bool = False  # blocks are norm -> mixer -> residual, without a feed-forward (Mamba2ForCausalLM)
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 48
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    scoring_func: str = "softmax"  # softmax | sigmoid
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    first_k_dense_replace: int = 0
    dense_layers: tuple = ()  # layers of a mixture-of-experts model that keep a dense MLP (decoder_sparse_step / mlp_only_layers)
    shared_expert_gate: bool = False  # Qwen: shared output scaled by sigmoid(gate(x))
    # MLA
    use_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # MTP draft head
    num_nextn_predict_layers: int = 0
    # runtime
    dtype: torch.dtype = torch.bfloat16
    max_model_len: int = 4096
    mm_token_ids: Optional[dict] = None  # multimodal checkpoints: modality -> placeholder token id (image_token_id, video_token_id, ...)
    vision_config: Optional[dict] = None  # the checkpoint's vision tower (Qwen2-VL layout), when it has one
    vision_merge_size: int = 2
    mrope_section: Optional[tuple] = None  # rotary frequencies split over the (temporal, height, width) position components (Qwen2-VL family)
    index_topk: int = 0  # DeepSeek-V3.2 sparse attention: keys kept per query by the lightning indexer (0: dense attention)
    quant: QuantConfig = field(default_factory=QuantConfig)
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    seed: int = 0
    load_format: str = "auto"  # auto | safetensors | gguf | dummy
    tokenizer: Optional[str] = None
    enable_lora: bool = False  # build the model so that adapters can be applied (gate|up without the fused SiLU·mul epilogue)
    enable_sleep_mode: bool = False  # weights and KV cache live in releasable device memory (utils/cumem.py)
    max_loras: int = 4
    max_lora_rank: int = 64
    hf_overrides: dict = field(default_factory=dict)
    logits_processors: tuple = ()  # "package.module:ClassName" of user logits processors applied to every sampling step

    def __post_init__(self) -> None:
        if self.num_attention_heads % max(self.num_key_value_heads, 1):
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.layer_types is not None and len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must have one entry per layer")
        if self.max_model_len <= 0:
            raise ValueError("max_model_len must be positive")

    # ---- derived
    @property
    def is_hybrid(self) -> bool:
        return bool(self.layer_types) and any(t in ("linear_attention", "mamba2", "mamba1", "short_conv") for t in self.layer_types)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "full_attention"

    def layer_window(self, i: int) -> int:
        """Sliding window of layer ``i`` in tokens, 0 for full attention."""
        return self.sliding_window if i in self.sliding_layers else 0

    def is_moe_layer(self, i: int) -> bool:
        return self.is_moe and i >= self.first_k_dense_replace and i not in self.dense_layers

    @property
    def rotary_dim(self) -> int:
        d = self.qk_rope_head_dim if self.use_mla else self.head_dim
        return int(d * self.partial_rotary_factor) if not self.use_mla else d

    @property
    def num_attention_layers(self) -> int:
        return sum(1 for i in range(self.num_hidden_layers) if self.layer_type(i) == "full_attention")

    @property
    def kv_cache_head_dim(self) -> int:
        return self.kv_lora_rank + self.qk_rope_head_dim if self.use_mla else self.head_dim

    def compute_hash(self) -> str:
        d = dataclasses.asdict(self)
        d["dtype"] = str(self.dtype)
        return _hash(d)

    @classmethod
    def from_hf_dict(cls, hf: dict, **over) -> "ModelConfig":
        """Normalise an HF config dict. Nested ``text_config`` (Qwen3.5) is flattened."""
        over = dict(over)
        mm_ids = {m: int(hf[k]) for m, k in (("image", "image_token_id"), ("video", "video_token_id"), ("audio", "audio_token_id")) if hf.get(k) is not None}
        if mm_ids:
            over.setdefault("mm_token_ids", mm_ids)
        if isinstance(hf.get("vision_config"), dict):
            over.setdefault("vision_config", dict(hf["vision_config"]))
            over.setdefault("vision_merge_size", int(hf["vision_config"].get("spatial_merge_size", 2)))
        if "text_config" in hf and isinstance(hf["text_config"], dict):
            inner = dict(hf["text_config"])
            inner.setdefault("architectures", hf.get("architectures"))
            inner.setdefault("quantization_config", hf.get("quantization_config"))
            hf = inner
        arch = (hf.get("architectures") or ["LlamaForCausalLM"])[0]
        over = dict(over)
        if arch == "DeepseekV32ForCausalLM":
            over.setdefault("index_topk", int(hf.get("index_topk", 2048)))
        nh = hf.get("num_attention_heads", 8)
        hidden = hf.get("hidden_size", 256)
        kw: dict[str, Any] = dict(
            architecture=arch, vocab_size=hf.get("vocab_size", 32000), hidden_size=hidden,
            intermediate_size=hf.get("intermediate_size", 4 * hidden), num_hidden_layers=hf.get("num_hidden_layers", 4),
            num_attention_heads=nh, num_key_value_heads=hf.get("num_key_value_heads", nh),
            head_dim=hf.get("head_dim") or hidden // nh, rms_norm_eps=hf.get("rms_norm_eps", 1e-6),
            rope_theta=(hf.get("rope_parameters") or {}).get("rope_theta", hf.get("rope_theta", 10000.0)),
            partial_rotary_factor=(hf.get("rope_parameters") or {}).get("partial_rotary_factor", hf.get("partial_rotary_factor", 1.0)),
            max_position_embeddings=hf.get("max_position_embeddings", 32768),
            tie_word_embeddings=hf.get("tie_word_embeddings", False), attention_bias=hf.get("attention_bias", False),
            eos_token_id=hf.get("eos_token_id") if not isinstance(hf.get("eos_token_id"), list) else hf["eos_token_id"][0],
            bos_token_id=hf.get("bos_token_id"), quant=QuantConfig.from_hf(hf.get("quantization_config")),
            num_nextn_predict_layers=hf.get("num_nextn_predict_layers", hf.get("mtp_num_hidden_layers", 0)) or 0,
        )
        a = arch.lower()
        if "qwen2" in a:
            kw["attention_bias"] = hf.get("qkv_bias", True)
        if "qwen3" in a:
            kw["qk_norm"] = True
        if "qwen3next" in a or "qwen3_5" in a or "qwen3_next" in a:
            kw.update(gemma_norm=True, attn_output_gate=hf.get("attn_output_gate", True), layer_types=hf.get("layer_types"),
                      linear_num_key_heads=hf.get("linear_num_key_heads", 16), linear_num_value_heads=hf.get("linear_num_value_heads", 48),
                      linear_key_head_dim=hf.get("linear_key_head_dim", 128), linear_value_head_dim=hf.get("linear_value_head_dim", 128),
                      linear_conv_kernel_dim=hf.get("linear_conv_kernel_dim", 4))
            if kw["layer_types"] is None:
                iv = hf.get("full_attention_interval", 4)
                kw["layer_types"] = ["full_attention" if (i + 1) % iv == 0 else "linear_attention" for i in range(kw["num_hidden_layers"])]
        n_exp = hf.get("num_experts") or hf.get("n_routed_experts") or hf.get("num_local_experts")
        if n_exp:
            # Mixtral has no separate expert width and always renormalises its top-k weights
            kw.update(num_experts=n_exp, num_experts_per_tok=hf.get("num_experts_per_tok", 8),
                      moe_intermediate_size=hf.get("moe_intermediate_size") or hf.get("intermediate_size", 512),
                      norm_topk_prob=hf.get("norm_topk_prob", True) or "mixtral" in a)
            step, only = hf.get("decoder_sparse_step", 1) or 1, set(hf.get("mlp_only_layers") or [])
            if step > 1 or only:
                kw["dense_layers"] = tuple(i for i in range(kw["num_hidden_layers"]) if i in only or (i + 1) % step != 0)
            if "deepseek" in a:
                kw.update(shared_expert_intermediate_size=hf.get("n_shared_experts", 1) * hf.get("moe_intermediate_size", 2048),
                          scoring_func=hf.get("scoring_func", "sigmoid"), n_group=hf.get("n_group", 8), topk_group=hf.get("topk_group", 4),
                          routed_scaling_factor=hf.get("routed_scaling_factor", 2.5), first_k_dense_replace=hf.get("first_k_dense_replace", 3))
            else:
                kw.update(shared_expert_intermediate_size=hf.get("shared_expert_intermediate_size", 0),
                          shared_expert_gate=bool(hf.get("shared_expert_intermediate_size", 0)))
        if ("deepseek" in a or a.startswith("glm4moelite")) and hf.get("kv_lora_rank"):
            kw.update(use_mla=True, q_lora_rank=hf.get("q_lora_rank") or 0, kv_lora_rank=hf["kv_lora_rank"],
                      qk_nope_head_dim=hf.get("qk_nope_head_dim", 128), qk_rope_head_dim=hf.get("qk_rope_head_dim", 64),
                      v_head_dim=hf.get("v_head_dim", 128), head_dim=hf.get("qk_nope_head_dim", 128) + hf.get("qk_rope_head_dim", 64))
        if arch in ("Lfm2ForCausalLM", "Lfm2MoeForCausalLM"):
            inter = int(hf.get("intermediate_size", 4 * hidden))
            if arch == "Lfm2MoeForCausalLM":
                # the dense width is taken as it stands; experts behind a sigmoid router with a selection bias, after the first dense layers
                kw.update(scoring_func="sigmoid", n_group=1, topk_group=1, norm_topk_prob=bool(hf.get("norm_topk_prob", True)),
                          routed_scaling_factor=float(hf.get("routed_scaling_factor", 1.0)), shared_expert_intermediate_size=0, shared_expert_gate=False,
                          dense_layers=tuple(range(int(hf.get("num_dense_layers", 2)))))
            elif hf.get("block_auto_adjust_ff_dim", True):   # the checkpoint's feed-forward width: 2/3 of the nominal one, rounded up to a multiple
                inter = int(2 * inter / 3)
                if hf.get("block_ffn_dim_multiplier") is not None:
                    mult = int(hf.get("block_multiple_of", 256))
                    inter = int(float(hf["block_ffn_dim_multiplier"]) * inter)
                    inter = mult * ((inter + mult - 1) // mult)
            kinds = hf.get("layer_types") or ["full_attention"] * kw["num_hidden_layers"]
            kw.update(layer_types=["full_attention" if t == "full_attention" else "short_conv" for t in kinds], intermediate_size=inter,
                      mamba_d_conv=int(hf.get("conv_L_cache", 3)), mamba_conv_bias=bool(hf.get("conv_bias", False)), qk_norm=True,
                      rms_norm_eps=float(hf.get("norm_eps", 1e-5)), tie_word_embeddings=hf.get("tie_word_embeddings", True))
        if arch == "JambaForCausalLM":
            L = kw["num_hidden_layers"]
            ap, ao = int(hf.get("attn_layer_period", 8)), int(hf.get("attn_layer_offset", 4))
            ep, eo = int(hf.get("expert_layer_period", 2)), int(hf.get("expert_layer_offset", 1))
            rank = hf.get("mamba_dt_rank", "auto")
            kw.update(layer_types=["full_attention" if (i - ao) % ap == 0 else "mamba1" for i in range(L)], nope_layers=tuple(range(L)),
                      mamba_n_heads=1, mamba_d_head=int(hf.get("mamba_expand", 2) * hidden), mamba_d_state=int(hf.get("mamba_d_state", 16)),
                      mamba_d_conv=int(hf.get("mamba_d_conv", 4)), mamba_conv_bias=bool(hf.get("mamba_conv_bias", True)),
                      mamba_proj_bias=bool(hf.get("mamba_proj_bias", False)), mamba_dt_rank=-(-hidden // 16) if rank in (None, "auto") else int(rank),
                      mamba_inner_norm_weights=True)
            if kw.get("num_experts"):
                kw.update(norm_topk_prob=False, dense_layers=tuple(i for i in range(L) if (i - eo) % ep != 0))
        if arch in ("MambaForCausalLM", "FalconMambaForCausalLM"):
            d_inner = int(hf.get("intermediate_size") or hf.get("expand", 2) * hidden)
            rank = hf.get("time_step_rank", "auto")
            kw.update(layer_types=["mamba1"] * kw["num_hidden_layers"], mamba_n_heads=1, mamba_d_head=d_inner, mamba_d_state=int(hf.get("state_size", 16)),
                      mamba_d_conv=int(hf.get("conv_kernel", 4)), mamba_conv_bias=bool(hf.get("use_conv_bias", True)),
                      mamba_proj_bias=bool(hf.get("use_bias", False)), mamba_dt_rank=-(-hidden // 16) if rank in (None, "auto") else int(rank),
                      mamba_inner_rms_eps=float(hf.get("mixer_rms_eps", 1e-6)) if arch.startswith("FalconMamba") else None,
                      mixer_only_layers=True, rms_norm_eps=hf.get("layer_norm_epsilon", 1e-5), intermediate_size=0,
                      tie_word_embeddings=hf.get("tie_word_embeddings", True))
        if arch == "GraniteMoeSharedForCausalLM" and kw.get("num_experts"):
            kw.update(shared_expert_intermediate_size=int(hf.get("shared_intermediate_size") or 0), shared_expert_gate=False, norm_topk_prob=True)
        if arch == "GraniteMoeHybridForCausalLM":
            # Granite 4.0: Bamba's mixers + Granite multipliers + experts with an ungated shared feed-forward (or, without experts,
            # that feed-forward alone)
            kinds = hf.get("layer_types") or ["mamba"] * kw["num_hidden_layers"]
            hf = dict(hf, attn_layer_indices=[i for i, t in enumerate(kinds) if t == "attention"])
            shared = int(hf.get("shared_intermediate_size") or 0)
            if kw.get("num_experts"):
                kw.update(shared_expert_intermediate_size=shared, shared_expert_gate=False, norm_topk_prob=True)
            else:
                kw["intermediate_size"] = shared
            if hf.get("position_embedding_type") == "nope":
                kw["nope_layers"] = tuple(range(kw["num_hidden_layers"]))
        if arch == "NemotronHForCausalLM":
            # every block is norm -> one mixer -> residual; the mixers are Mamba-2, attention without positions, or an ungated feed-forward
            kinds = list(hf.get("layers_block_type") or hf.get("layer_types") or [])
            if not kinds and hf.get("hybrid_override_pattern"):
                kinds = [{"M": "mamba", "*": "attention", "-": "mlp", "E": "moe"}[c] for c in hf["hybrid_override_pattern"]]
            if not kinds or any(k not in ("mamba", "attention", "mlp") for k in kinds):
                raise ValueError("NemotronH is served with mamba / attention / mlp blocks (its expert blocks are not)")
            kw["num_hidden_layers"] = len(kinds)
            hf = dict(hf, attn_layer_indices=[i for i, t in enumerate(kinds) if t == "attention"], mamba_n_heads=hf.get("mamba_num_heads", 128),
                      mamba_d_head=hf.get("mamba_head_dim", 64), mamba_d_state=hf.get("ssm_state_size", 128), mamba_proj_bias=hf.get("use_bias", False))
            kw.update(nope_layers=tuple(range(len(kinds))), mlp_gated=False, hidden_act={"relu2": "relu2", "silu": "silu"}.get(hf.get("mlp_hidden_act", "relu2"), "gelu"),
                      mlp_bias=bool(hf.get("mlp_bias", False)))
        if arch in ("BambaForCausalLM", "Mamba2ForCausalLM", "GraniteMoeHybridForCausalLM", "NemotronHForCausalLM"):
            L = kw["num_hidden_layers"]
            pure = arch in ("Mamba2ForCausalLM", "NemotronHForCausalLM")
            expand = hf.get("mamba_expand", hf.get("expand", 2))
            heads = hf.get("mamba_n_heads", hf.get("num_heads", 128))
            d_head = hf.get("mamba_d_head", hf.get("head_dim", "auto"))
            if d_head in (None, "auto") or pure:
                d_head = int(expand * hidden) // heads if d_head in (None, "auto") else int(d_head)
            attn_idx = set(hf.get("attn_layer_indices") or ())
            def _num(v, default):   # json has no infinity: checkpoints write it as a string or a tagged object
                try:
                    return float(v)
                except (TypeError, ValueError):
                    return default
            lim = hf.get("time_step_limit") or (0.0, float("inf"))
            lim = (_num(lim[0], 0.0), _num(lim[1], float("inf")))
            groups = hf.get("mamba_n_groups", hf.get("n_groups", 1))
            kw.update(layer_types=["full_attention" if i in attn_idx else "mamba2" for i in range(L)], mamba_n_heads=int(heads),
                      mamba_d_head=int(d_head), mamba_n_groups=int(groups), mamba_d_state=int(hf.get("mamba_d_state", hf.get("state_size", 128))),
                      mamba_d_conv=int(hf.get("mamba_d_conv", hf.get("conv_kernel", 4))),
                      mamba_conv_bias=bool(hf.get("mamba_conv_bias", hf.get("use_conv_bias", True))),
                      mamba_proj_bias=bool(hf.get("mamba_proj_bias", hf.get("use_bias", False))),
                      mamba_time_step_limit=(float(lim[0]), float(lim[1])), mamba_norm_groups=int(hf.get("mamba_norm_groups", groups)),
                      mixer_only_layers=pure, rms_norm_eps=hf.get("rms_norm_eps", hf.get("layer_norm_epsilon", 1e-5)))
            if arch == "NemotronHForCausalLM":
                kw["layer_types"] = [{"mamba": "mamba2", "attention": "full_attention", "mlp": "ffn"}[k] for k in kinds]
            elif pure:
                kw.update(tie_word_embeddings=hf.get("tie_word_embeddings", True), intermediate_size=0)
        rp = hf.get("rope_parameters") or hf.get("rope_scaling") or {}
        if rp.get("mrope_section"):
            kw["mrope_section"] = tuple(int(x) for x in rp["mrope_section"])
            rp = {k: v for k, v in rp.items() if k != "mrope_section"}
            if (rp.get("rope_type") or rp.get("type")) == "mrope":  # the sections are the whole difference from the default rule
                rp.pop("rope_type", None)
                rp.pop("type", None)
        if isinstance(rp.get("full_attention"), dict):  # per-layer-type rotary parameters (Gemma3)
            kw["rope_theta"] = rp["full_attention"].get("rope_theta", kw["rope_theta"])
            kw["rope_local_theta"] = (rp.get("sliding_attention") or {}).get("rope_theta")
            rp = rp["full_attention"]
        if (rp.get("rope_type") or rp.get("type") or "default") != "default":
            kw["rope_scaling"] = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
            kw["rope_scaling"].setdefault("rope_type", rp.get("type"))
            if kw["rope_scaling"]["rope_type"] == "dynamic":
                kw["rope_scaling"].setdefault("original_max_position_embeddings", hf.get("max_position_embeddings"))
            if kw["rope_scaling"]["rope_type"] in ("longrope", "su"):
                kw["rope_scaling"].setdefault("max_position_embeddings", hf.get("max_position_embeddings"))
                kw["rope_scaling"].setdefault("original_max_position_embeddings", hf.get("original_max_position_embeddings"))
        lt = hf.get("layer_types")
        if not lt and hf.get("sliding_window") and ("gemma2" in a or "gemma3" in a):
            # configs written before ``layer_types`` existed: Gemma2 alternates, Gemma3 makes every ``sliding_window_pattern``-th layer global
            pat = 2 if "gemma2" in a else int(hf.get("sliding_window_pattern", 6))
            lt = ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(kw["num_hidden_layers"])]
        if "gemma3" in a and kw.get("rope_local_theta") is None and hf.get("rope_local_base_freq"):
            kw["rope_local_theta"] = float(hf["rope_local_base_freq"])
        if lt and any(t == "sliding_attention" for t in lt) and hf.get("sliding_window"):
            kw.update(sliding_window=int(hf["sliding_window"]), sliding_layers=tuple(i for i, t in enumerate(lt) if t == "sliding_attention"))
            if not kw.get("layer_types"):
                kw["layer_types"] = None
        elif hf.get("sliding_window") and hf.get("use_sliding_window", "mistral" in a or "phi3" in a):
            kw.update(sliding_window=int(hf["sliding_window"]), sliding_layers=tuple(range(kw["num_hidden_layers"])))
        act = hf.get("hidden_activation") or hf.get("hidden_act") or "silu"
        if act in ("gelu_pytorch_tanh", "gelu_tanh", "gelu"):
            kw["hidden_act"] = "gelu_tanh"
        if "gemma" in a:
            if "hidden_activation" not in hf and "hidden_act" not in hf:
                kw["hidden_act"] = "gelu_tanh"   # the family's default when the config does not say
            kw.update(gemma_norm=True, embed_scale=float(hidden) ** 0.5, tie_word_embeddings=hf.get("tie_word_embeddings", True))
            if "gemma2" in a or "gemma3" in a:
                kw.update(sandwich_norm=True, attn_scale=float(hf.get("query_pre_attn_scalar", kw["head_dim"])) ** -0.5,
                          attn_softcap=float(hf.get("attn_logit_softcapping") or 0.0), final_softcap=float(hf.get("final_logit_softcapping") or 0.0))
            if "gemma3" in a:
                kw["qk_norm"] = True
            if a.startswith("vaultgemma"):   # Gemma-2's attention (scaling, soft caps, windows by layer type) without the sandwich norms
                kw.update(attn_scale=float(hf.get("query_pre_attn_scalar", kw["head_dim"])) ** -0.5,
                          attn_softcap=float(hf.get("attn_logit_softcapping") or 0.0), final_softcap=float(hf.get("final_logit_softcapping") or 0.0))
        if a.startswith("glm"):
            kw.update(rope_interleaved="moe" not in a, sandwich_norm=a.startswith("glm4for"), qk_norm=bool(hf.get("use_qk_norm", False)))
            if "moe" in a:
                kw.update(shared_expert_intermediate_size=hf.get("n_shared_experts", 1) * hf.get("moe_intermediate_size", 1408),
                          shared_expert_gate=False, scoring_func="sigmoid", n_group=hf.get("n_group", 1), topk_group=hf.get("topk_group", 1),
                          routed_scaling_factor=hf.get("routed_scaling_factor", 1.0), first_k_dense_replace=hf.get("first_k_dense_replace", 1))
        if a.startswith("minimaxm2"):
            # sigmoid router with a selection bias, weights renormalised over the chosen experts; q / k normalised over the whole projection
            kw.update(qk_norm=False, qk_norm_full=bool(hf.get("use_qk_norm", True)), scoring_func="sigmoid",
                      n_group=1, topk_group=1, norm_topk_prob=True, routed_scaling_factor=1.0, shared_expert_intermediate_size=0,
                      shared_expert_gate=False)
            if hf.get("rotary_dim"):
                kw["partial_rotary_factor"] = float(hf["rotary_dim"]) / kw["head_dim"]
        if "smollm3" in a and hf.get("no_rope_layers"):
            kw["nope_layers"] = tuple(i for i, v in enumerate(hf["no_rope_layers"]) if not v)
        if a.startswith("exaone4"):
            # post-norm order with per-head q/k norm; in the hybrid form the full-attention layers apply no rotary embedding
            kw.update(pre_norm=False, sandwich_norm=True, qk_norm=True)
            if kw.get("sliding_layers"):
                kw["nope_layers"] = tuple(i for i in range(kw["num_hidden_layers"]) if i not in kw["sliding_layers"])
        if a.startswith(("solaropen", "glm4moelite")):
            # GLM-4.5-style experts (sigmoid router with a selection bias, shared experts, scaled weights); Solar keeps plain attention,
            # GLM-4-MoE-Lite uses latent attention
            kinds = hf.get("mlp_layer_types") or []
            kw.update(shared_expert_intermediate_size=(hf.get("n_shared_experts") or 0) * hf.get("moe_intermediate_size", 1408), shared_expert_gate=False,
                      scoring_func="sigmoid", n_group=hf.get("n_group", 1), topk_group=hf.get("topk_group", 1), norm_topk_prob=bool(hf.get("norm_topk_prob", True)),
                      routed_scaling_factor=hf.get("routed_scaling_factor", 1.0), first_k_dense_replace=0,
                      dense_layers=tuple(i for i, t in enumerate(kinds) if t != "sparse") if kinds else tuple(range(int(hf.get("first_k_dense_replace", 0)))))
        if a.startswith("arcee"):
            kw.update(mlp_gated=False, hidden_act="relu2")
        # families on mean-and-variance layer norms
        if a.startswith("olmofor"):           # OLMo-1: layer norms without learned parameters, optional clamp of q / k / v
            kw.update(norm_type="layernorm", norm_affine=False, rms_norm_eps=1e-5, qkv_clip=hf.get("clip_qkv"))
        if a.startswith("stablelm"):
            if hf.get("qk_layernorm") or hf.get("use_parallel_residual"):
                raise ValueError("StableLM with per-head layer norms or the parallel residual form is not served")
            kw.update(norm_type="layernorm", norm_bias=True, rms_norm_eps=hf.get("layer_norm_eps", 1e-5),
                      attention_bias=bool(hf.get("use_qkv_bias", False)), attn_o_bias=False)
        if a.startswith("starcoder2"):
            b = bool(hf.get("use_bias", True))
            kw.update(norm_type="layernorm", norm_bias=True, rms_norm_eps=hf.get("norm_epsilon", 1e-5), attention_bias=b, attn_o_bias=b,
                      mlp_bias=b, mlp_gated=False, hidden_act="gelu_tanh", tie_word_embeddings=hf.get("tie_word_embeddings", True))
            if hf.get("sliding_window"):
                kw.update(sliding_window=int(hf["sliding_window"]), sliding_layers=tuple(range(kw["num_hidden_layers"])))
        if a.startswith("nemotronfor"):       # layer norms whose weight is stored minus one; squared-ReLU feed-forward without a gate
            kw.update(norm_type="layernorm", norm_bias=True, gemma_norm=True, rms_norm_eps=hf.get("norm_eps", 1e-5), mlp_gated=False,
                      hidden_act="relu2", attn_o_bias=bool(hf.get("attention_bias", False)))
        if a.startswith("cohere"):            # Command-R: parallel blocks on weight-only layer norms, adjacent-pair rotary, scaled logits
            if hf.get("use_qk_norm"):
                raise ValueError("Cohere checkpoints with per-head q / k layer norms are not served")
            kw.update(norm_type="layernorm", norm_bias=False, rms_norm_eps=hf.get("layer_norm_eps", 1e-5), parallel_block=True,
                      rope_interleaved=True, logit_scale=float(hf.get("logit_scale", 0.0625)),
                      tie_word_embeddings=hf.get("tie_word_embeddings", True), attn_o_bias=bool(hf.get("attention_bias", False)))
            if kw.get("sliding_layers"):          # Command-R7B / Command-A: only the sliding-window layers rotate
                kw["nope_layers"] = tuple(i for i in range(kw["num_hidden_layers"]) if i not in kw["sliding_layers"])
        if a.startswith("jais2"):
            kw.update(norm_type="layernorm", norm_bias=True, rms_norm_eps=hf.get("layer_norm_eps", 1e-5), mlp_gated=False,
                      hidden_act="relu2", attn_o_bias=bool(hf.get("attention_bias", False)))
        if a.startswith("exaonemoe"):
            # pre-norm blocks with per-head q/k norm; global layers of the hybrid form apply no rotary embedding; DeepSeek-V3-style router
            kinds = hf.get("mlp_layer_types") or []
            kw.update(qk_norm=True, shared_expert_intermediate_size=(hf.get("num_shared_experts") or 0) * hf.get("moe_intermediate_size", 1024),
                      shared_expert_gate=False, scoring_func="sigmoid", n_group=hf.get("n_group", 1), topk_group=hf.get("topk_group", 1),
                      routed_scaling_factor=hf.get("routed_scaling_factor", 1.0), norm_topk_prob=bool(hf.get("norm_topk_prob", True)),
                      dense_layers=tuple(i for i, t in enumerate(kinds) if t != "sparse") if kinds else
                      tuple(range(int(hf.get("first_k_dense_replace", 0)))))
            if kw.get("sliding_layers"):
                kw["nope_layers"] = tuple(i for i in range(kw["num_hidden_layers"]) if i not in kw["sliding_layers"])
        if a.startswith("dots1"):
            kw.update(qk_norm=True, shared_expert_intermediate_size=(hf.get("n_shared_experts") or 0) * hf.get("moe_intermediate_size", 1408),
                      shared_expert_gate=False, scoring_func="sigmoid", n_group=hf.get("n_group", 1), topk_group=hf.get("topk_group", 1),
                      routed_scaling_factor=hf.get("routed_scaling_factor", 1.0), first_k_dense_replace=hf.get("first_k_dense_replace", 0))
        if a.startswith("olmoe"):
            kw.update(qk_norm_full=True)
        if a.startswith("gptoss"):
            if kw["quant"].method == "mxfp4":
                # the released checkpoints quantise the experts only (their skip list uses wildcards: name the modules here)
                kw["quant"] = dataclasses.replace(kw["quant"], modules_to_not_convert=["self_attn", "mlp.gate", "lm_head", "embed_tokens"])
            kw.update(attention_bias=True, attn_o_bias=True, attn_sinks=True, router_linear_bias=True, expert_bias=True, moe_act="swiglu_oai",
                      norm_topk_prob=True, num_experts_per_tok=hf.get("num_experts_per_tok", hf.get("experts_per_token", 4)))
        if a.startswith("ernie4_5_moe"):
            start, end = hf.get("moe_layer_start_index", 0), hf.get("moe_layer_end_index", -1)
            end = kw["num_hidden_layers"] - 1 if end is None or end < 0 else end
            iv = hf.get("moe_layer_interval", 1) or 1
            kw.update(num_experts=hf.get("moe_num_experts", 64), num_experts_per_tok=hf.get("moe_k", 6),
                      moe_intermediate_size=hf.get("moe_intermediate_size", 1536), norm_topk_prob=True, router_bias=True, rope_interleaved=True,
                      shared_expert_intermediate_size=(hf.get("moe_num_shared_experts") or 0) * hf.get("moe_intermediate_size", 1536),
                      shared_expert_gate=False, attention_bias=bool(hf.get("use_bias", False)),
                      dense_layers=tuple(i for i in range(kw["num_hidden_layers"]) if not (start <= i <= end and (i + 1) % iv == 0)))
        if a.startswith("hunyuanmoev1"):
            # softmax router renormalised over the chosen experts; an ungated shared feed-forward of the dense width beside them
            topk = hf.get("moe_topk", 2)
            kw.update(qk_norm=bool(hf.get("use_qk_norm", True)), qk_norm_after_rope=True, num_experts_per_tok=int(topk if isinstance(topk, int) else topk[0]),
                      norm_topk_prob=True, moe_intermediate_size=int(hf.get("moe_intermediate_size") or hf.get("intermediate_size", 512))
                      if isinstance(hf.get("moe_intermediate_size"), (int, type(None))) else int(hf["moe_intermediate_size"][0]),
                      shared_expert_intermediate_size=int(hf.get("intermediate_size", 512)), shared_expert_gate=False)
        if a.startswith("hunyuandensev1"):
            kw.update(qk_norm=True, qk_norm_after_rope=True)
        if a.startswith("helium"):
            kw["rope_interleaved"] = True
        if a.startswith("ernie4_5for"):
            kw.update(rope_interleaved=True, attention_bias=bool(hf.get("use_bias", False)))
        if a.startswith(("olmo2", "olmo3", "flexolmo")):
            kw.update(pre_norm=False, sandwich_norm=True, qk_norm_full=True)
        if "granite" in a:
            kw.update(embed_scale=float(hf.get("embedding_multiplier", 1.0)), residual_multiplier=float(hf.get("residual_multiplier", 1.0)),
                      attn_scale=float(hf.get("attention_multiplier", kw["head_dim"] ** -0.5)), logit_scale=1.0 / float(hf.get("logits_scaling", 1.0)))
        # families whose ``attention_bias`` also puts a bias on the output projection (the others keep o_proj bias-free)
        if kw.get("attention_bias") and a.startswith(("llama", "qwen3", "granite", "olmo", "smollm3", "gemma", "hunyuan", "dots1", "ernie4_5")):
            kw["attn_o_bias"] = True
        if a.startswith("seedoss"):
            kw["attn_o_bias"] = bool(hf.get("attention_out_bias", False))
        if hf.get("mlp_bias"):
            kw["mlp_bias"] = True
        if arch.endswith("ForSequenceClassification"):
            kw["num_labels"] = int(hf.get("num_labels") or len(hf.get("id2label") or {}) or 2)
        kw.update(over)
        return cls(**kw)

    @classmethod
    def from_pretrained(cls, path: str, **over) -> "ModelConfig":
        from onecat_vllm.loader import gguf
        gpath = gguf.resolve(path)
        cdir = path if os.path.isdir(path) else os.path.dirname(path)
        if gpath is not None and not os.path.exists(os.path.join(cdir, "config.json")):
            f = gguf.GGUFFile(gpath)  # a bare .gguf file: the architecture comes from its metadata
            hf = gguf.config_from_metadata(f.metadata, f.tensors)
            if over.get("tokenizer") is None and "tokenizer.ggml.tokens" in f.metadata:
                over["tokenizer"] = gpath  # ... and so does the tokenizer, when the file embeds one
        else:
            with open(os.path.join(cdir, "config.json")) as f:
                hf = json.load(f)
        if gpath is not None:
            hf.pop("quantization_config", None)  # ggml blocks are dequantised while loading
            if over.get("load_format", "auto") == "auto":
                over["load_format"] = "gguf"
        return cls.from_hf_dict(hf, model=gpath or path, **over)


# ----------------------------------------------------------------------------- cache / parallel / scheduler
@dataclass
class CacheConfig:
    """Paged KV cache (reference: vllm/config/cache.py). Block size 16 by default."""

    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks_override: Optional[int] = None
    kv_cache_memory_bytes: Optional[int] = None
    enable_prefix_caching: bool = True
    prefix_caching_hash_algo: str = "sha256"
    cache_dtype: str = "auto"  # auto | fp8 | fp8_e4m3 | fp8_e5m2
    mamba_cache_mode: str = "none"  # none | align
    cpu_offload_gb: float = 0.0
    kv_offloading_size: float = 0.0  # GiB of host memory for KV blocks evicted from the GPU prefix cache (0 = off)
    num_cpu_blocks_override: Optional[int] = None
    kv_offloading_policy: str = "lru"  # lru | arc: which host block is dropped when the tier is full
    kv_events_config: Optional[dict] = None  # {"enable_kv_cache_events": true, "endpoint": "tcp://127.0.0.1:5557", "topic": "kv-events"}
    kv_transfer_config: Optional[dict] = None  # {"kv_connector": "SharedStorageConnector", "kv_role": ..., "kv_connector_extra_config": {...}}
    num_gpu_blocks: int = 0  # filled in after profiling
    num_cpu_blocks: int = 0  # filled in with the KV cache

    def __post_init__(self) -> None:
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValueError("block_size must be a power of two")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")

    def compute_hash(self) -> str:
        return _hash([self.block_size, self.cache_dtype])


@dataclass
class ParallelConfig:
    """Parallel layout (reference: vllm/config/parallel.py:116-341)."""

    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    distributed_executor_backend: Optional[str] = None  # None | "uni" | "mp" | "external_launcher"
    tp_comm: str = "fused"  # "fused": peer-memory kernels; "nccl": library collectives (baseline)
    data_parallel_rank: int = 0
    enable_eplb: bool = False
    master_addr: str = "127.0.0.1"
    master_port: int = 0

    def __post_init__(self) -> None:
        for n in ("tensor_parallel_size", "pipeline_parallel_size", "data_parallel_size", "decode_context_parallel_size"):
            if getattr(self, n) < 1:
                raise ValueError(f"{n} must be >= 1")
        if self.tensor_parallel_size % self.decode_context_parallel_size:
            raise ValueError("decode_context_parallel_size must divide tensor_parallel_size")

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size * self.pipeline_parallel_size

    def compute_hash(self) -> str:
        return _hash([self.tensor_parallel_size, self.pipeline_parallel_size, self.enable_expert_parallel])


@dataclass
class SchedulerConfig:
    """Token-budget scheduler (reference: vllm/config/scheduler.py; semantics v1/core/sched/scheduler.py:459-468)."""

    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 256
    max_model_len: int = 4096
    enable_chunked_prefill: bool = True
    long_prefill_token_threshold: int = 0
    policy: str = "fcfs"  # fcfs | priority
    async_scheduling: bool = True  # one step in flight while the next is scheduled (falls back per step when a request needs host tokens)
    cuda_graph_sizes: Optional[list[int]] = None
    max_num_encoder_input_tokens: int = 8192  # multimodal: encoder output positions computed per step
    encoder_cache_size: int = 16384           # multimodal: encoder output positions kept on the workers

    def __post_init__(self) -> None:
        if self.policy not in ("fcfs", "priority"):
            raise ValueError("policy must be 'fcfs' or 'priority'")
        if not self.enable_chunked_prefill and self.max_num_batched_tokens < self.max_model_len:
            raise ValueError("without chunked prefill max_num_batched_tokens must cover max_model_len")

    def graph_capture_sizes(self) -> list[int]:
        """Default capture sizes (reference: vllm/config/vllm.py:2084-2200)."""
        if self.cuda_graph_sizes is not None:
            return sorted(set(self.cuda_graph_sizes))
        mx = min(2 * self.max_num_seqs, 512)
        sizes = [1, 2, 4] + list(range(8, 256, 8)) + list(range(256, mx + 1, 16))
        return [s for s in sizes if s <= mx]


@dataclass
class SpeculativeConfig:
    """Speculative decoding (reference: vllm/config/speculative.py:216-281,1090-1104).

    ``synthetic_acceptance_rates`` are per-position *unconditional* acceptance probabilities; the
    rejection sampler uses the conditional form ``rate[i] / rate[i-1]``.
    """

    method: Optional[str] = None  # None | "mtp" | "ngram" | "suffix" | "eagle" | "eagle3" | "medusa" | "draft_model"
    draft_vocab_size: Optional[int] = None  # eagle3: size of the head's reduced vocabulary (read from its config.json when present)
    eagle_aux_hidden_state_layers: Optional[list] = None  # eagle3: target layers whose input stream feeds the head (default 2, L/2, L-3)
    num_speculative_tokens: int = 0
    model: Optional[str] = None  # eagle / medusa: directory of the draft heads' checkpoint (random weights when absent); draft_model: the draft's checkpoint
    medusa_num_layers: int = 1  # residual blocks per Medusa head
    synthetic_acceptance_rates: Optional[list[float]] = None
    synthetic_acceptance_rate: Optional[float] = None  # conditional per-position Bernoulli rate
    synthetic_seed: int = 0
    prompt_lookup_max: int = 4
    prompt_lookup_min: int = 2

    def __post_init__(self) -> None:
        if self.method is not None and self.num_speculative_tokens < 1:
            raise ValueError("num_speculative_tokens must be >= 1 when a method is set")
        if self.synthetic_acceptance_rates is not None:
            r = self.synthetic_acceptance_rates
            if len(r) != self.num_speculative_tokens or any(not 0 <= x <= 1 for x in r) or any(r[i] > r[i - 1] for i in range(1, len(r))):
                raise ValueError("synthetic_acceptance_rates must be non-increasing probabilities, one per draft position")

    @property
    def enabled(self) -> bool:
        return self.method is not None

    def conditional_rates(self) -> Optional[list[float]]:
        if self.synthetic_acceptance_rate is not None:
            return [self.synthetic_acceptance_rate] * self.num_speculative_tokens
        if self.synthetic_acceptance_rates is None:
            return None
        out, prev = [], 1.0
        for x in self.synthetic_acceptance_rates:
            out.append(0.0 if prev <= 0 else min(1.0, x / prev))
            prev = x
        return out


@dataclass
class ObservabilityConfig:
    otlp_traces_endpoint: Optional[str] = None
    collect_detailed_traces: bool = False
    enable_metrics: bool = True
    log_stats_interval_s: float = 10.0


@dataclass
class VllmConfig:
    model_config: ModelConfig
    cache_config: CacheConfig = field(default_factory=CacheConfig)
    parallel_config: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler_config: SchedulerConfig = field(default_factory=SchedulerConfig)
    speculative_config: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    observability_config: ObservabilityConfig = field(default_factory=ObservabilityConfig)
    device: str = "auto"  # auto | cuda | cpu
    enforce_eager: bool = False
    structured_outputs_backend: str = "auto"  # auto | xgrammar | builtin

    def __post_init__(self) -> None:
        self.scheduler_config.max_model_len = self.model_config.max_model_len
        if self.device == "auto":
            self.device = "cuda" if torch.cuda.is_available() else "cpu"
        m, p = self.model_config, self.parallel_config
        if m.num_attention_heads % p.tensor_parallel_size:
            raise ValueError("tensor_parallel_size must divide num_attention_heads")
        if p.pipeline_parallel_size > 1:
            if p.pipeline_parallel_size > m.num_hidden_layers:
                raise ValueError("pipeline_parallel_size exceeds the number of decoder layers")
            if self.speculative_config.enabled:
                raise ValueError("speculative decoding is not supported together with pipeline parallelism")
            # stage boundaries exchange replicated tensors: tensor-parallel sums inside a stage use the library all-reduce, and the
            # steps run eagerly (send/recv between stages is not captured)
            p.tp_comm = "nccl"
            self.enforce_eager = True

    def compute_hash(self) -> str:
        return _hash([self.model_config.compute_hash(), self.cache_config.compute_hash(), self.parallel_config.compute_hash()])


# ----------------------------------------------------------------------------- EngineArgs
@dataclass
class EngineArgs:
    """User-facing arguments (reference: vllm/engine/arg_utils.py). ``model`` is a checkpoint directory,
    or ``hf_config`` gives the architecture directly (random-init weights, ``load_format='dummy'``)."""

    model: str = "dummy"
    hf_config: Optional[dict] = None
    tokenizer: Optional[str] = None
    dtype: str = "auto"
    seed: int = 0
    max_model_len: Optional[int] = None
    quantization: Optional[str] = None
    load_format: str = "auto"
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    distributed_executor_backend: Optional[str] = None
    tp_comm: str = "fused"
    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks_override: Optional[int] = None
    kv_cache_memory_bytes: Optional[int] = None
    enable_prefix_caching: bool = True
    kv_cache_dtype: str = "auto"
    kv_offloading_size: float = 0.0
    num_cpu_blocks_override: Optional[int] = None
    kv_offloading_policy: str = "lru"  # lru | arc: which host block is dropped when the tier is full
    kv_transfer_config: Optional[Union[dict, str]] = None
    kv_events_config: Optional[Union[dict, str]] = None
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    long_prefill_token_threshold: int = 0
    scheduling_policy: str = "fcfs"
    async_scheduling: bool = True
    enforce_eager: bool = False
    cuda_graph_sizes: Optional[list[int]] = None
    speculative_config: Optional[Union[dict, str]] = None
    device: str = "auto"
    otlp_traces_endpoint: Optional[str] = None
    disable_log_stats: bool = True
    hf_overrides: Optional[dict] = None
    structured_outputs_backend: str = "auto"
    enable_lora: bool = False
    max_loras: int = 4
    max_lora_rank: int = 64
    enable_sleep_mode: bool = False
    logits_processors: Optional[list] = None  # ["package.module:ClassName", ...]

    def create_engine_config(self) -> VllmConfig:
        dt = _DTYPES[self.dtype] if isinstance(self.dtype, str) else self.dtype
        over: dict[str, Any] = dict(seed=self.seed, load_format=self.load_format, tokenizer=self.tokenizer, enable_lora=self.enable_lora,
                                    enable_sleep_mode=self.enable_sleep_mode, max_loras=self.max_loras, max_lora_rank=self.max_lora_rank,
                                    logits_processors=tuple(self.logits_processors or ()))
        if self.hf_config is not None:
            hf = dict(self.hf_config)
            hf.update(self.hf_overrides or {})
            mc = ModelConfig.from_hf_dict(hf, model=self.model, **over)
            if self.load_format == "auto":
                mc.load_format = "dummy"
        else:
            mc = ModelConfig.from_pretrained(self.model, **over)
        device = self.device if self.device != "auto" else ("cuda" if torch.cuda.is_available() else "cpu")
        mc.dtype = dt if dt is not None else (torch.bfloat16 if device == "cuda" else torch.float32)
        if self.quantization:
            if mc.quant.method == "none":
                mc.quant = QuantConfig.from_hf({"quant_method": self.quantization})
            elif mc.quant.method != self.quantization.replace("_marlin", ""):
                raise ValueError(f"quantization={self.quantization} does not match the checkpoint's {mc.quant.method}")
        mc.max_model_len = self.max_model_len or min(mc.max_position_embeddings, 32768)
        if mc.index_topk and mc.max_model_len > mc.index_topk:
            # DeepSeek-V3.2 attends to the index_topk keys its lightning indexer selects; up to that many tokens this equals dense
            # attention, which is what runs here. Longer contexts would silently change the model's outputs, so they are refused.
            if self.max_model_len:
                raise ValueError(f"{mc.architecture}: the sparse-attention indexer is not built; contexts up to index_topk={mc.index_topk} tokens are "
                                 f"exact with dense attention, max_model_len={mc.max_model_len} is not (reference: "
                                 "model_executor/layers/sparse_attn_indexer.py)")
            mc.max_model_len = mc.index_topk
        spec = self.speculative_config
        if isinstance(spec, str):
            spec = json.loads(spec)
        sc = SpeculativeConfig(**spec) if spec else SpeculativeConfig()
        return VllmConfig(
            model_config=mc,
            cache_config=CacheConfig(self.block_size, self.gpu_memory_utilization, self.num_gpu_blocks_override,
                                     self.kv_cache_memory_bytes, self.enable_prefix_caching, cache_dtype=self.kv_cache_dtype,
                                     kv_offloading_size=self.kv_offloading_size, num_cpu_blocks_override=self.num_cpu_blocks_override, kv_offloading_policy=self.kv_offloading_policy,
                                     kv_transfer_config=json.loads(self.kv_transfer_config) if isinstance(self.kv_transfer_config, str)
                                     else self.kv_transfer_config,
                                     kv_events_config=json.loads(self.kv_events_config) if isinstance(self.kv_events_config, str)
                                     else self.kv_events_config),
            parallel_config=ParallelConfig(self.tensor_parallel_size, self.pipeline_parallel_size, self.data_parallel_size,
                                           self.enable_expert_parallel, self.decode_context_parallel_size,
                                           self.distributed_executor_backend, self.tp_comm),
            scheduler_config=SchedulerConfig(self.max_num_batched_tokens, self.max_num_seqs, mc.max_model_len,
                                             self.enable_chunked_prefill, self.long_prefill_token_threshold,
                                             self.scheduling_policy, self.async_scheduling, self.cuda_graph_sizes),
            speculative_config=sc,
            observability_config=ObservabilityConfig(self.otlp_traces_endpoint, enable_metrics=not self.disable_log_stats),
            device=device, enforce_eager=self.enforce_eager, structured_outputs_backend=self.structured_outputs_backend,
        )

    # ---- argparse bridge (reference: arg_utils.py add_cli_args / from_cli_args)
    @classmethod
    def add_cli_args(cls, parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        for f in dataclasses.fields(cls):
            name = "--" + f.name.replace("_", "-")
            if f.name == "hf_config" or f.name == "hf_overrides" or f.name == "speculative_config":
                parser.add_argument(name, type=json.loads, default=None)
            elif f.type in ("bool", bool):
                parser.add_argument(name, action=argparse.BooleanOptionalAction, default=f.default)
            elif "list[int]" in str(f.type):
                parser.add_argument(name, type=int, nargs="*", default=None)
            elif "int" in str(f.type):
                parser.add_argument(name, type=int, default=f.default)
            elif "float" in str(f.type):
                parser.add_argument(name, type=float, default=f.default)
            else:
                parser.add_argument(name, type=str, default=f.default)
        return parser

    @classmethod
    def from_cli_args(cls, ns: argparse.Namespace) -> "EngineArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(ns).items() if k in names})


AsyncEngineArgs = EngineArgs
