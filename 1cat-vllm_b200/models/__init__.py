"""Model registry (reference: model_executor/models/registry.py): HF ``architectures`` name → builder."""
from __future__ import annotations

from onecat_vllm.config import ModelConfig

_REGISTRY = {
    "LlamaForCausalLM": "dense", "MistralForCausalLM": "dense", "Qwen2ForCausalLM": "dense", "Qwen3ForCausalLM": "dense",
    "Phi3ForCausalLM": "dense", "SeedOssForCausalLM": "dense", "InternLM3ForCausalLM": "dense",
    "GemmaForCausalLM": "dense", "Gemma2ForCausalLM": "dense", "Gemma3ForCausalLM": "dense", "GlmForCausalLM": "dense",
    "Glm4ForCausalLM": "dense", "GraniteForCausalLM": "dense", "Glm4MoeForCausalLM": "moe",
    "SmolLM3ForCausalLM": "dense", "Olmo2ForCausalLM": "dense", "Olmo3ForCausalLM": "dense", "OlmoeForCausalLM": "moe",
    "GptOssForCausalLM": "moe", "GraniteMoeForCausalLM": "moe", "GraniteMoeSharedForCausalLM": "moe", "Ernie4_5_MoeForCausalLM": "moe", "HunYuanDenseV1ForCausalLM": "dense", "HeliumForCausalLM": "dense", "CwmForCausalLM": "dense",
    "Ernie4_5ForCausalLM": "dense", "Exaone4ForCausalLM": "dense", "MinistralForCausalLM": "dense", "Dots1ForCausalLM": "moe",
    "Qwen3MoeForCausalLM": "moe", "MiniMaxM2ForCausalLM": "moe", "SolarOpenForCausalLM": "moe", "Glm4MoeLiteForCausalLM": "mla_moe", "ExaoneMoeForCausalLM": "moe", "FlexOlmoForCausalLM": "moe", "Ministral3ForCausalLM": "dense", "ArceeForCausalLM": "dense", "NemotronHForCausalLM": "hybrid", "CohereForCausalLM": "dense", "Cohere2ForCausalLM": "dense", "OlmoForCausalLM": "dense", "StableLmForCausalLM": "dense", "Starcoder2ForCausalLM": "dense", "NemotronForCausalLM": "dense", "Jais2ForCausalLM": "dense", "VaultGemmaForCausalLM": "dense", "HunYuanMoEV1ForCausalLM": "moe", "Qwen2MoeForCausalLM": "moe", "MixtralForCausalLM": "moe",
    "Qwen3NextForCausalLM": "hybrid", "Qwen3_5ForCausalLM": "hybrid", "Qwen3_5ForConditionalGeneration": "hybrid",
    "Qwen3_5MoeForCausalLM": "hybrid", "Qwen3_5MoeForConditionalGeneration": "hybrid",
    "BambaForCausalLM": "hybrid", "Lfm2ForCausalLM": "hybrid", "Lfm2MoeForCausalLM": "hybrid", "JambaForCausalLM": "hybrid", "GraniteMoeHybridForCausalLM": "hybrid", "Mamba2ForCausalLM": "hybrid", "MambaForCausalLM": "hybrid", "FalconMambaForCausalLM": "hybrid",
    "Qwen2VLForConditionalGeneration": "dense", "Qwen2_5_VLForConditionalGeneration": "dense",
    "DeepseekV2ForCausalLM": "mla_moe", "DeepseekV3ForCausalLM": "mla_moe", "DeepseekV32ForCausalLM": "mla_moe",
}


# sequence-classification checkpoints of the dense families: the decoder with a ``score`` head (reference: models/adapters.py
# ``as_seq_cls_model``)
for _a in ("Llama", "Mistral", "Qwen2", "Qwen3", "Gemma", "Gemma2", "Phi3"):
    _REGISTRY[_a + "ForSequenceClassification"] = "dense"


def supported_architectures() -> list[str]:
    return sorted(_REGISTRY)


def register_model(arch: str, family: str = "dense") -> None:
    """Out-of-tree registration hook (reference: ModelRegistry.register_model)."""
    _REGISTRY[arch] = family


def build_model(cfg: ModelConfig, device="cpu"):
    if cfg.architecture not in _REGISTRY:
        raise ValueError(f"architecture {cfg.architecture!r} is not supported; known: {supported_architectures()}")
    from onecat_vllm.models.decoder import CausalLM
    return CausalLM(cfg, device)
