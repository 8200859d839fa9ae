"""Generic pre-norm decoder covering the served architectures.

One ``DecoderLayer`` picks its token mixer (full attention, gated attention, Gated-DeltaNet, MLA) and its
feed-forward (SwiGLU MLP or sparse MoE) from ``ModelConfig`` (reference: models/llama.py, qwen3.py,
qwen3_next.py:635-863, qwen3_5.py, deepseek_v2.py:1076-1596). The residual stream is carried unnormalised;
each sub-block's partial output goes through ``reduce_add_norm`` which fuses the TP reduction, the residual add
and the next RMSNorm.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from onecat_vllm.config import ModelConfig
from onecat_vllm.layers.attention import Attention
from onecat_vllm.layers.common import ParallelLMHead, RMSNorm, VocabParallelEmbedding, make_norm
from onecat_vllm.layers.gdn import GatedDeltaNet
from onecat_vllm.layers.mla import MLAAttention
from onecat_vllm.layers.mlp import MLP
from onecat_vllm.layers.moe import SparseMoeBlock
from onecat_vllm.parallel import state as ps
from onecat_vllm.parallel.tp_ops import reduce_add_norm, reduce_only


class PPMissingLayer(nn.Module):
    """Placeholder for a module that lives on another pipeline stage; keeps checkpoint names aligned
    (reference: model_executor/models/utils.py ``PPMissingLayer``)."""

    kind = "missing"


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, prefix: str, device):
        super().__init__()
        from onecat_vllm.utils.plugins import layer_class
        self.kind = cfg.layer_type(idx)
        if cfg.use_mla:
            self.kind = "mla"
            self.self_attn = layer_class("MLAAttention", MLAAttention)(cfg, idx, prefix + ".self_attn", device)
        elif self.kind == "linear_attention":
            self.linear_attn = layer_class("GatedDeltaNet", GatedDeltaNet)(cfg, idx, prefix + ".linear_attn")
        elif self.kind in ("mamba2", "mamba1", "short_conv", "ffn"):
            if self.kind == "ffn":
                from onecat_vllm.layers.mlp import FeedForwardBlock as Mixer
            elif self.kind == "mamba2":
                from onecat_vllm.layers.mamba2 import Mamba2Mixer as Mixer
            elif self.kind == "mamba1":
                from onecat_vllm.layers.mamba1 import Mamba1Mixer as Mixer
            else:
                from onecat_vllm.layers.short_conv import ShortConv as Mixer
            self.linear_attn = Mixer(cfg, idx, prefix + ".linear_attn")
            self.kind = "linear_attention"   # a state-slot layer like Gated-DeltaNet for the runner and the scheduler
            self.graph_safe = False          # its convolution and scan read batch geometry on the host
        else:
            self.self_attn = layer_class("Attention", Attention)(cfg, idx, prefix + ".self_attn", device)
        if cfg.mixer_only_layers:
            self.mlp = None
            self.input_layernorm = make_norm(cfg)
            return
        if cfg.is_moe_layer(idx):
            self.mlp = layer_class("SparseMoeBlock", SparseMoeBlock)(cfg, prefix + ".mlp")
        elif not cfg.mlp_gated:
            from onecat_vllm.layers.mlp import PlainMLP
            self.mlp = layer_class("PlainMLP", PlainMLP)(cfg.hidden_size, cfg.intermediate_size, cfg.quant, prefix + ".mlp", cfg.dtype, act=cfg.hidden_act,
                                                         bias=cfg.mlp_bias)
        else:
            self.mlp = layer_class("MLP", MLP)(cfg.hidden_size, cfg.intermediate_size, cfg.quant, prefix + ".mlp", cfg.dtype, fuse_act=not cfg.enable_lora,
                           act=cfg.hidden_act, bias=cfg.mlp_bias)
        self.input_layernorm = make_norm(cfg)
        if not cfg.parallel_block:
            self.post_attention_layernorm = make_norm(cfg)
        if cfg.sandwich_norm:
            # Gemma2/3 and GLM-4: post_attention_layernorm normalises the mixer's output, pre_feedforward_layernorm is the pre-norm of
            # the feed-forward, post_feedforward_layernorm normalises its output (GLM-4's names are mapped to these at load)
            self.pre_feedforward_layernorm = make_norm(cfg)
            self.post_feedforward_layernorm = make_norm(cfg)

    def mixer(self, x, md, cache):
        if self.kind == "linear_attention":
            return self.linear_attn(x, md, cache)
        return self.self_attn(x, md, cache)


class DecoderModel(nn.Module):
    """``forward`` returns the final *normalised* hidden states ``[T, hidden]``."""

    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__()
        self.cfg = cfg
        st = ps.get_state()
        self.first_stage, self.last_stage = st.is_first_pp, st.is_last_pp
        self.start, self.end = ps.pp_layer_range(cfg.num_hidden_layers)
        need_embed = self.first_stage or (self.last_stage and cfg.tie_word_embeddings)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype) if need_embed else PPMissingLayer()
        self.layers = nn.ModuleList([DecoderLayer(cfg, i, f"model.layers.{i}", device) if self.start <= i < self.end else PPMissingLayer()
                                     for i in range(cfg.num_hidden_layers)])
        self.norm = make_norm(cfg) if self.last_stage else PPMissingLayer()
        # EAGLE-3 drafting reads the residual stream at a few depths: layer indices to record, and what the last forward recorded
        self.aux_hidden_layers: tuple = ()
        self.last_aux: list = []

    def local_layers(self):
        """(global index, layer) of the decoder layers this pipeline stage owns; KV caches are indexed in this order."""
        return [(i, self.layers[i]) for i in range(self.start, self.end)]

    def forward(self, input_ids: torch.Tensor, md, caches: list, inputs_embeds: Optional[torch.Tensor] = None,
                return_prenorm: bool = False, intermediate: Optional[tuple] = None):
        """First stage: embeds ``input_ids``. Later stages: ``intermediate`` = (reduced block output, residual) of the previous
        stage. A stage that is not the last returns that pair for its successor instead of the final hidden states
        (reference: models/llama.py ``IntermediateTensors`` handling)."""
        layers = self.layers
        cfg = self.cfg
        if intermediate is None:
            if inputs_embeds is None:
                h = self.embed_tokens(input_ids)
                if cfg.embed_scale != 1.0:
                    h = h * torch.tensor(cfg.embed_scale, dtype=h.dtype)  # the factor is rounded to the model dtype first, as in the checkpoint's code
            else:
                h = inputs_embeds
            x, residual = layers[self.start].input_layernorm(h, None)
            residual = h
        else:
            x, residual = layers[self.start].input_layernorm(intermediate[0], intermediate[1])
        if not cfg.pre_norm:
            return self._forward_post_norm(x if intermediate is None else None, residual, md, caches)
        if cfg.parallel_block:
            return self._forward_parallel(residual, md, caches)
        plain = not cfg.sandwich_norm and cfg.residual_multiplier == 1.0
        aux_at = self.aux_hidden_layers
        if aux_at:
            self.last_aux = []
        for li, i in enumerate(range(self.start, self.end)):
            layer = layers[i]
            if aux_at and i in aux_at:
                self.last_aux.append(residual)   # the stream entering layer i (reference: models/llama.py ``aux_hidden_state_layers``)
            part = layer.mixer(x, md, caches[li])
            if layer.mlp is None:   # norm -> mixer -> residual blocks: the next block's norm (or the final one) follows directly
                if i + 1 == self.end and not self.last_stage:
                    return reduce_only(part), residual
                x, residual = reduce_add_norm(part, residual, layers[i + 1].input_layernorm if i + 1 < self.end else self.norm)
                continue
            if plain:
                x, residual = reduce_add_norm(part, residual, layer.post_attention_layernorm)
            else:
                x, residual = self._join(part, residual, layer.post_attention_layernorm if cfg.sandwich_norm else None,
                                         layer.pre_feedforward_layernorm if cfg.sandwich_norm else layer.post_attention_layernorm)
            part = layer.mlp(x)
            last_local = i + 1 == self.end and not self.last_stage
            nxt = None if last_local else (layers[i + 1].input_layernorm if i + 1 < self.end else self.norm)
            if plain:
                if last_local:
                    return reduce_only(part), residual
                x, residual = reduce_add_norm(part, residual, nxt)
            else:
                out = self._join(part, residual, layer.post_feedforward_layernorm if cfg.sandwich_norm else None, nxt)
                if last_local:
                    return out
                x, residual = out
        if return_prenorm:
            return x, residual
        return x

    def _forward_post_norm(self, _x, residual, md, caches):
        """OLMo-2 / OLMo-3 block order: ``h = h + norm(attn(h)); h = h + norm(mlp(h))`` with no norm in front of either sub-block
        (reference: models/olmo2.py). Pipeline stages are not split for this order."""
        if self.start != 0 or not self.last_stage:
            raise ValueError("the post-norm block order is served without pipeline parallelism")
        h = residual
        for li, i in enumerate(range(self.start, self.end)):
            layer = self.layers[i]
            h = h + layer.post_attention_layernorm(reduce_only(layer.mixer(h, md, caches[li])), None)[0]
            h = h + layer.post_feedforward_layernorm(reduce_only(layer.mlp(h)), None)[0]
        return self.norm(h, None)[0]

    def _forward_parallel(self, h, md, caches):
        """Cohere block order: attention and feed-forward both read ``norm(h)`` and their outputs are added to ``h`` together
        (reference: models/commandr.py). The two partial outputs are summed before the tensor-parallel reduction, so a layer costs
        one reduction. Pipeline stages are not split for this order."""
        if self.start != 0 or not self.last_stage:
            raise ValueError("the parallel block order is served without pipeline parallelism")
        for li, i in enumerate(range(self.start, self.end)):
            layer = self.layers[i]
            x = layer.input_layernorm(h, None)[0]
            h = h + reduce_only(layer.mixer(x, md, caches[li]) + layer.mlp(x))
        return self.norm(h, None)[0]

    def _join(self, part, residual, post_norm, next_norm):
        """Sub-block output → residual for the architectures that do more than add: reduce over TP, normalise the output (sandwich
        norms) or scale it (Granite), then add + next pre-norm. With ``next_norm`` None returns (output, residual) for the next stage."""
        p = reduce_only(part)
        if post_norm is not None:
            p = post_norm(p, None)[0]
        if self.cfg.residual_multiplier != 1.0:
            p = p * self.cfg.residual_multiplier
        if next_norm is None:
            return p, residual
        return next_norm(p, residual)


class CausalLM(nn.Module):
    """Decoder + LM head. Parameter names mirror HF checkpoints (``model.layers.N…``, ``lm_head``)."""

    # checkpoint name fragment → (our stacked parameter, shard id)
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", 0), (".qkv_proj", ".k_proj", 1), (".qkv_proj", ".v_proj", 2),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
        (".in_proj_qkvz", ".in_proj_q", 0), (".in_proj_qkvz", ".in_proj_k", 1), (".in_proj_qkvz", ".in_proj_v", 2),
        (".in_proj_qkvz", ".in_proj_z", 3), (".in_proj_ba", ".in_proj_b", 0), (".in_proj_ba", ".in_proj_a", 1),
    ]

    def __init__(self, cfg: ModelConfig, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.model = DecoderModel(cfg, device)
        self.score = None
        if cfg.num_labels > 0:
            from onecat_vllm.layers.linear import ReplicatedLinear
            self.lm_head = None
            self.score = ReplicatedLinear(cfg.hidden_size, cfg.num_labels, quant=None, prefix="score", dtype=cfg.dtype)
        elif cfg.tie_word_embeddings or not ps.get_state().is_last_pp:
            self.lm_head = None
        else:
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.visual = None
        # the tower built here is the Qwen2-VL one; other multimodal checkpoints load their text tower and take image embeddings
        if cfg.architecture == "Qwen2VLForConditionalGeneration" and cfg.vision_config and cfg.vision_config.get("depth") and ps.get_state().is_first_pp:
            from onecat_vllm.models.vision import VisionTower
            self.visual = VisionTower(cfg.vision_config, cfg.dtype)

    def embed_multimodal(self, feature, device) -> torch.Tensor:
        """Embeddings ``[length, hidden]`` of one multimodal item: given ones are passed through, pixel inputs go through the
        vision tower (reference: models/interfaces.py ``SupportsMultiModal.embed_multimodal``)."""
        if feature.kind == "embeds":
            return torch.as_tensor(feature.data).to(device, self.cfg.dtype)
        if self.visual is None:
            raise ValueError("this checkpoint has no vision tower: pass image embeddings instead of pixel values")
        return self.visual(torch.as_tensor(feature.data["pixel_values"]), feature.data["grid_thw"])

    def forward(self, input_ids, md, caches, inputs_embeds=None, intermediate=None):
        return self.model(input_ids, md, caches, inputs_embeds, intermediate=intermediate)

    def greedy_tokens(self, hidden: torch.Tensor):
        """Greedy token per row straight from the sharded LM head (no logits gather), or None when the model post-processes its
        logits in a way arg-max does not commute with across shards."""
        c = self.cfg
        if c.final_softcap > 0:
            return None   # tanh is monotonic, but keep one code path for capped models
        head = self.lm_head if self.lm_head is not None else self.model.embed_tokens
        return ParallelLMHead.greedy_tokens(head, hidden, c.logit_scale)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self.lm_head
        if head is None:
            e = self.model.embed_tokens
            logits = ParallelLMHead.compute_logits(e, hidden)
        else:
            logits = head.compute_logits(hidden)
        c = self.cfg
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        if c.final_softcap > 0:  # Gemma2: cap * tanh(logits / cap)
            logits = torch.tanh(logits.float() / c.final_softcap).mul_(c.final_softcap).to(logits.dtype)
        return logits


class MTPHead(nn.Module):
    """Multi-token-prediction draft head: ``h' = fc([norm_e(embed(tok)) ; norm_h(h_target)])`` followed by one
    full-attention decoder layer and a final norm; embeddings and LM head are shared with the target
    (reference: models/qwen3_5_mtp.py:109-227; models/deepseek_mtp.py)."""

    def __init__(self, cfg: ModelConfig, target: CausalLM, device="cpu"):
        super().__init__()
        import dataclasses
        from onecat_vllm.layers.linear import ReplicatedLinear
        # the module's feed-forward follows the target: sparse for mixture-of-experts targets, dense otherwise
        lcfg = dataclasses.replace(cfg, layer_types=None, num_hidden_layers=1, first_k_dense_replace=0, dense_layers=(), sliding_layers=())
        self.cfg = lcfg
        self.stacked_params_mapping = CausalLM.stacked_params_mapping
        self.pre_fc_norm_embedding = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)
        self.pre_fc_norm_hidden = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)
        self.fc = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, quant=None, prefix="mtp.fc", dtype=cfg.dtype)
        self.layer = DecoderLayer(lcfg, 0, "mtp.layers.0", device)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)
        self._target = [target]  # not registered: weights are shared, not owned

    def forward(self, input_ids, target_hidden, md, cache):
        tgt = self._target[0]
        e, _ = self.pre_fc_norm_embedding(tgt.model.embed_tokens(input_ids))
        h, _ = self.pre_fc_norm_hidden(target_hidden)
        h = self.fc(torch.cat([e, h], dim=-1))
        layer = self.layer
        x, _ = layer.input_layernorm(h, None)
        part = layer.mixer(x, md, cache)
        x, residual = reduce_add_norm(part, h, layer.post_attention_layernorm)
        part = layer.mlp(x)
        x, _ = reduce_add_norm(part, residual, self.norm)
        return x

    def compute_logits(self, hidden):
        return self._target[0].compute_logits(hidden)


class Eagle3Head(nn.Module):
    """EAGLE-3 draft head. The target's residual stream at three depths is concatenated and reduced by ``fc`` to one hidden vector;
    the single decoder layer's attention reads ``[norm(embed(tok)) ; norm(hidden)]`` (twice the hidden size), the residual path
    carries ``hidden``; the layer's output before the final norm is the hidden input of the next drafting pass. The head has its own
    final norm and LM head, possibly over a reduced draft vocabulary that ``d2t`` maps back to target ids
    (reference: models/llama_eagle3.py; spec_decode/eagle.py; v1/spec_decode/static_draft_vocab.py for the reduced vocabulary)."""

    stacked_params_mapping = CausalLM.stacked_params_mapping

    def __init__(self, cfg: ModelConfig, target: CausalLM, device="cpu", draft_vocab_size: Optional[int] = None):
        super().__init__()
        import dataclasses
        from onecat_vllm.layers.attention import Attention
        from onecat_vllm.layers.linear import ReplicatedLinear
        lcfg = dataclasses.replace(cfg, layer_types=None, num_hidden_layers=1, num_experts=0, sliding_layers=(), quant=type(cfg.quant)())
        self.cfg = lcfg
        H = cfg.hidden_size
        self.fc = ReplicatedLinear(3 * H, H, bias=False, quant=None, prefix="fc", dtype=cfg.dtype)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, H, cfg.dtype)
        self.own_embedding = False
        self.layer = DecoderLayer(lcfg, 0, "layers.0", device)
        self.layer.self_attn = Attention(lcfg, 0, "layers.0.self_attn", device, qkv_in=2 * H)
        self.hidden_norm = RMSNorm(H, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)
        self.norm = RMSNorm(H, cfg.rms_norm_eps, cfg.gemma_norm, cfg.dtype)
        self.draft_vocab = int(draft_vocab_size or cfg.vocab_size)
        self.lm_head = ReplicatedLinear(H, self.draft_vocab, bias=False, quant=None, prefix="lm_head", dtype=cfg.dtype)
        self.own_lm_head = False   # set by the loader; without a checkpoint the target's LM head is used
        # draft id -> target id is ``draft id + d2t[draft id]`` (the checkpoints store offsets); identity when the vocabularies agree
        self.register_buffer("d2t", torch.zeros(self.draft_vocab, dtype=torch.long), persistent=False)
        self._target = [target]

    def forward(self, input_ids, target_hidden, md, cache):
        H = self.cfg.hidden_size
        hidden = self.fc(target_hidden) if target_hidden.shape[-1] != H else target_hidden
        emb = self.embed_tokens if self.own_embedding else self._target[0].model.embed_tokens
        layer = self.layer
        x = torch.cat([layer.input_layernorm(emb(input_ids), None)[0], self.hidden_norm(hidden, None)[0]], dim=-1)
        part = layer.mixer(x, md, cache)
        x, residual = reduce_add_norm(part, hidden, layer.post_attention_layernorm)
        return residual + reduce_only(layer.mlp(x))

    def compute_logits(self, hidden):
        x = self.norm(hidden, None)[0]
        if not self.own_lm_head:
            return self._target[0].compute_logits(x)
        lg = self.lm_head(x)
        if self.draft_vocab == self.cfg.vocab_size and not bool(self.d2t.any()):
            return lg
        full = torch.full((lg.shape[0], self.cfg.vocab_size), float("-inf"), dtype=lg.dtype, device=lg.device)
        full[:, torch.arange(self.draft_vocab, device=lg.device) + self.d2t.to(lg.device)] = lg
        return full


class EagleHead(nn.Module):
    """EAGLE-1 draft head: ``h' = fc([embed(tok) ; h_target])`` (with bias), one decoder layer without its input norm, no final
    norm; the LM head is the target's and the embedding table is the head's own when its checkpoint has one
    (reference: models/llama_eagle.py; spec_decode/eagle.py — same drafting loop as the MTP head)."""

    stacked_params_mapping = CausalLM.stacked_params_mapping

    def __init__(self, cfg: ModelConfig, target: CausalLM, device="cpu"):
        super().__init__()
        import dataclasses
        from onecat_vllm.layers.linear import ReplicatedLinear
        lcfg = dataclasses.replace(cfg, layer_types=None, num_hidden_layers=1, num_experts=0, sliding_layers=(), quant=type(cfg.quant)())
        self.cfg = lcfg
        self.fc = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, bias=True, quant=None, prefix="fc", dtype=cfg.dtype)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype)
        self.own_embedding = False  # set by the loader when the checkpoint carries embed_tokens
        self.layer = DecoderLayer(lcfg, 0, "layers.0", device)
        self._target = [target]

    def forward(self, input_ids, target_hidden, md, cache):
        emb = self.embed_tokens if self.own_embedding else self._target[0].model.embed_tokens
        h = self.fc(torch.cat([emb(input_ids), target_hidden], dim=-1))
        layer = self.layer
        part = layer.mixer(h, md, cache)
        x, residual = reduce_add_norm(part, h, layer.post_attention_layernorm)
        return residual + reduce_only(layer.mlp(x))

    def compute_logits(self, hidden):
        return self._target[0].compute_logits(hidden)
