"""Weight loading: safetensors checkpoints (HF layout, sharded over TP on the fly) and dummy random init
(reference: model_executor/model_loader/default_loader.py, dummy_loader.py, weight_utils.py:1451-1475).

Dummy init fills quantised storage with uniform random codes and scales drawn as the benchmark configs
prescribe, so synthetic AWQ/FP8/MXFP4 models exercise the same kernels as real checkpoints."""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Iterable, Iterator

import torch
import torch.nn as nn

from onecat_vllm.logger import init_logger

log = init_logger(__name__)


def iter_safetensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {path}")
    for f in files:
        with safe_open(f, framework="pt", device="cpu") as sf:
            for k in sf.keys():
                yield k, sf.get_tensor(k)


# checkpoint names whose tensors live under another name here (a parameter of the block instead of a sub-module's weight)
_RENAMES = ((".conv.conv.weight", ".linear_attn.conv_weight"), (".conv.conv.bias", ".linear_attn.conv_bias"), (".conv.in_proj.", ".linear_attn.in_proj."),
            (".conv.out_proj.", ".linear_attn.out_proj."), (".feed_forward.w1.", ".mlp.gate_proj."), (".feed_forward.w3.", ".mlp.up_proj."),
            (".feed_forward.w2.", ".mlp.down_proj."), (".operator_norm.", ".input_layernorm."), (".ffn_norm.", ".post_attention_layernorm."),
            ("model.embedding_norm.", "model.norm."), (".self_attn.out_proj.", ".self_attn.o_proj."), (".q_layernorm.weight", ".q_norm"),
            (".k_layernorm.weight", ".k_norm"), (".mlp.c_fc.", ".mlp.up_proj."), (".mlp.c_proj.", ".mlp.down_proj."),
            (".mamba.", ".linear_attn."), (".mixer.", ".linear_attn."), (".feed_forward.", ".mlp."), (".pre_ff_layernorm.", ".post_attention_layernorm."),
            ("model.final_layernorm.", "model.norm."), ("backbone.embeddings.", "model.embed_tokens."), ("backbone.embedding.", "model.embed_tokens."), ("backbone.norm_f.", "model.norm."),
            ("backbone.layers.", "model.layers."), (".linear_attn.conv1d.bias", ".linear_attn.conv_bias"),
            (".q_norm.weight", ".q_norm"), (".k_norm.weight", ".k_norm"), (".query_layernorm.weight", ".q_norm"), (".key_layernorm.weight", ".k_norm"), (".linear_attn.conv1d.weight", ".linear_attn.conv_weight"),
            (".linear_attn.norm.weight", ".linear_attn.norm_weight"), (".mlp.gate.moe_statics.e_score_correction_bias", ".mlp.e_score_correction_bias"),
            (".mlp.moe_statics.e_score_correction_bias", ".mlp.e_score_correction_bias"), (".mlp.router.", ".mlp.gate."), (".mlp.gate.e_score_correction_bias", ".mlp.e_score_correction_bias"),
            (".mlp.shared_experts.", ".mlp.shared_expert."), (".mlp.shared_mlp.", ".mlp.shared_expert."), (".mlp.gate.wg.", ".mlp.gate."), (".mlp.expert_bias", ".mlp.e_score_correction_bias"))
# GLM-4 names of the sandwich norms → the names used here (single pass: its post_attention_layernorm is the feed-forward pre-norm)
_GLM4_NORMS = {"post_attention_layernorm": "pre_feedforward_layernorm", "post_self_attn_layernorm": "post_attention_layernorm",
               "post_mlp_layernorm": "post_feedforward_layernorm"}
_BLOCK_NORM_RE = re.compile(r"(model\.layers\.\d+)\.norm\.")
_GLM4_NORM_RE = re.compile(r"\.(post_attention_layernorm|post_self_attn_layernorm|post_mlp_layernorm)\.")


def _half_split_rows(w: torch.Tensor, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Reorder each head's rotary rows from the adjacent-pair layout (0,1),(2,3),… to the half-split layout used by the rope kernel;
    applied to q and k alike, so q·k is unchanged."""
    perm = torch.cat([torch.arange(0, rotary_dim, 2), torch.arange(1, rotary_dim, 2), torch.arange(rotary_dim, head_dim)])
    heads = w.shape[0] // head_dim
    return w.reshape(heads, head_dim, -1)[:, perm].reshape(w.shape)


_EXPERT_RE = re.compile(r"(.*\.mlp)\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv|weight_scale|bias)$")


def load_weights(model: nn.Module, weights: Iterable[tuple[str, torch.Tensor]]) -> set:
    """Route checkpoint tensors to module ``load_weight`` hooks. Returns the set of consumed names."""
    mods = dict(model.named_modules())
    params = dict(model.named_parameters())
    stacked = getattr(model, "stacked_params_mapping", [])
    cfg = getattr(model, "cfg", None)
    glm4_norms = cfg is not None and cfg.sandwich_norm and cfg.architecture.startswith("Glm4")
    interleaved = cfg is not None and cfg.rope_interleaved
    mixer_only = cfg is not None and getattr(cfg, "mixer_only_layers", False)
    vault = cfg is not None and cfg.architecture.startswith("VaultGemma")
    nemotron_h = cfg is not None and cfg.architecture.startswith("NemotronH")
    loaded = set()
    for name, w in weights:
        if name.startswith("language_model."):
            name = name[len("language_model."):]
        elif name.startswith("model.language_model."):  # text tower of a multimodal checkpoint (Qwen3.5)
            name = "model." + name[len("model.language_model."):]
        if name.startswith(("visual.", "model.visual.")):
            tower = getattr(model, "visual", None)  # multimodal checkpoints: the vision tower, when this model builds one
            if tower is not None and tower.load_weight(name, w):
                loaded.add(name)
            continue
        if "rotary_emb.inv_freq" in name:
            continue
        if nemotron_h and ".mixer." in name:   # one name for every kind of block: attention blocks keep their projections under self_attn
            base = name.split(".mixer.")[0].replace("backbone.layers.", "model.layers.")
            if base + ".self_attn" in mods:
                name = name.replace(".mixer.", ".self_attn.")
        for theirs, ours in _RENAMES:
            if theirs in name:
                name = name.replace(theirs, ours)
        if vault and ".pre_feedforward_layernorm." in name:   # VaultGemma: Gemma-2's blocks without the two post-norms
            name = name.replace(".pre_feedforward_layernorm.", ".post_attention_layernorm.")
        if mixer_only:   # Mamba2ForCausalLM: a block's only norm is the pre-norm of its mixer
            name = _BLOCK_NORM_RE.sub(r"\1.input_layernorm.", name)
        if glm4_norms:
            name = _GLM4_NORM_RE.sub(lambda m: "." + _GLM4_NORMS[m.group(1)] + ".", name)
        if interleaved and (".q_proj." in name or ".k_proj." in name) and "self_attn" in name:
            w = _half_split_rows(w, cfg.head_dim, cfg.rotary_dim)
        if cfg is not None and cfg.moe_act == "swiglu_oai" and ".mlp.experts." in name:
            # GPT-OSS: [E, H, 2I] with gate / up in alternating columns, [E, I, H], and a bias for each
            mod = mods.get(name.split(".mlp.experts.")[0] + ".mlp.experts")
            leaf = name.rsplit(".", 1)[1]
            if mod is not None and leaf in ("gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias"):
                for e in range(w.shape[0]):
                    if leaf == "gate_up_proj":
                        t = w[e].t()
                        mod.load_expert_weight(e, "gate_proj", "weight", t[0::2])
                        mod.load_expert_weight(e, "up_proj", "weight", t[1::2])
                    elif leaf == "gate_up_proj_bias":
                        mod.load_expert_weight(e, "gate_proj", "bias", w[e, 0::2])
                        mod.load_expert_weight(e, "up_proj", "bias", w[e, 1::2])
                    elif leaf == "down_proj":
                        mod.load_expert_weight(e, "down_proj", "weight", w[e].t())
                    else:
                        mod.load_expert_weight(e, "down_proj", "bias", w[e])
                loaded.add(name)
                continue
            if mod is not None and leaf in ("gate_up_proj_blocks", "gate_up_proj_scales", "down_proj_blocks", "down_proj_scales"):
                # MXFP4 release format: [E, rows, K/32, 16] bytes (two e2m1 per byte, low nibble first) and [E, rows, K/32] e8m0
                # scales, in [out, in] orientation; gate / up rows alternate
                if mod.qmethod != "mxfp4":
                    raise ValueError("MXFP4 expert tensors need quantization_config.quant_method = mxfp4")
                pn = "weight" if leaf.endswith("_blocks") else "weight_scale"
                for e in range(w.shape[0]):
                    t = w[e].reshape(w.shape[1], -1)
                    if leaf.startswith("gate_up"):
                        mod.load_expert_weight(e, "gate_proj", pn, t[0::2])
                        mod.load_expert_weight(e, "up_proj", pn, t[1::2])
                    else:
                        mod.load_expert_weight(e, "down_proj", pn, t)
                loaded.add(name)
                continue
        if name.endswith((".mlp.experts.gate_up_proj", ".mlp.experts.down_proj")):
            # all experts of a layer in one tensor (the in-memory layout of recent transformers): [E, 2I, H] and [E, H, I]
            mod = mods.get(name.rsplit(".", 1)[0])
            if mod is not None:
                for e in range(w.shape[0]):
                    if name.endswith("gate_up_proj"):
                        half = w.shape[1] // 2
                        mod.load_expert_weight(e, "gate_proj", "weight", w[e, :half])
                        mod.load_expert_weight(e, "up_proj", "weight", w[e, half:])
                    else:
                        mod.load_expert_weight(e, "down_proj", "weight", w[e])
                loaded.add(name)
            continue
        if ".shared_mlp.input_linear." in name or ".shared_mlp.output_linear." in name:
            # Granite's shared feed-forward keeps gate|up stacked in one tensor: it is the shared expert beside routed experts, or the
            # layer's whole feed-forward when the model has none
            base = name.split(".shared_mlp.")[0] + ".mlp"
            tgt = base + ".shared_expert" if (base + ".shared_expert") in mods else base
            suffix = name.rsplit(".", 1)[1]
            if ".input_linear." in name:
                mods[tgt + ".gate_up_proj"].load_weight(suffix, w[: w.shape[0] // 2], 0)
                mods[tgt + ".gate_up_proj"].load_weight(suffix, w[w.shape[0] // 2:], 1)
            else:
                mods[tgt + ".down_proj"].load_weight(suffix, w, None)
            loaded.add(name)
            continue
        if ".block_sparse_moe.input_linear." in name or ".block_sparse_moe.output_linear." in name:
            # GraniteMoe keeps all experts of a layer in one tensor: gate|up stacked [E, 2I, H] and down [E, H, I]
            mod = mods.get(name.split(".block_sparse_moe.")[0] + ".mlp.experts")
            if mod is not None:
                for e in range(w.shape[0]):
                    if ".input_linear." in name:
                        half = w.shape[1] // 2
                        mod.load_expert_weight(e, "gate_proj", "weight", w[e, :half])
                        mod.load_expert_weight(e, "up_proj", "weight", w[e, half:])
                    else:
                        mod.load_expert_weight(e, "down_proj", "weight", w[e])
                loaded.add(name)
            continue
        if ".block_sparse_moe.router.layer." in name:
            name = name.replace(".block_sparse_moe.router.layer.", ".mlp.gate.")
        if ".block_sparse_moe." in name:  # Mixtral naming: block_sparse_moe.{gate, experts.N.w1|w3|w2}
            name = name.replace(".block_sparse_moe.", ".mlp.")
            for theirs, ours in ((".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj.")):
                name = name.replace(theirs, ours)
        if ".mlp.experts." in name and (".w1." in name or ".w2." in name or ".w3." in name):   # w1 / w3 / w2 naming outside Mixtral (LFM2-MoE)
            for theirs, ours in ((".w1.", ".gate_proj."), (".w3.", ".up_proj."), (".w2.", ".down_proj.")):
                name = name.replace(theirs, ours)
        m = _EXPERT_RE.match(name)
        if m:
            mod = mods.get(m.group(1) + ".experts")
            if mod is not None:
                mod.load_expert_weight(int(m.group(2)), m.group(3), m.group(4), w)
                loaded.add(name)
            continue
        if ".linear_attn.in_proj_qkv." in name:
            # Qwen3.5 keeps q|k|v fused (contiguous segments) and z separate: route the three segments to their slots
            tgt = name.replace(".in_proj_qkv.", ".in_proj_qkvz.")
            mod_name, _, pname = tgt.rpartition(".")
            mod = mods.get(mod_name)
            if mod is not None:
                sizes = mod.output_sizes[:3]
                o = 0
                for i, n in enumerate(sizes):
                    mod.load_weight(pname, w.narrow(0, o, n), i)
                    o += n
                loaded.add(name)
            continue
        target, shard = name, None
        for ours, theirs, sid in stacked:
            if theirs + "." in name:
                cand = name.replace(theirs + ".", ours + ".")
                if cand.rsplit(".", 1)[0] in mods:
                    target, shard = cand, sid
                    break
        mod_name, _, pname = target.rpartition(".")
        mod = mods.get(mod_name)
        if shard is None and (mod_name.endswith(".in_proj_qkvz") or mod_name.endswith(".in_proj_ba")) and pname == "weight":
            w = mods[mod_name.rsplit(".", 1)[0]].deinterleave(mod_name.rsplit(".", 1)[1], w)
        if mod is not None and hasattr(mod, "load_weight"):
            mod.load_weight(pname, w, shard)
            loaded.add(name)
        elif target in params:
            p = params[target]
            if p.shape == w.shape:
                p.data.copy_(w)
            else:  # e.g. conv weight [C,1,k] → [C,k]; TP-sharded vectors
                p.data.copy_(w.reshape(-1, *p.shape[1:])[: p.shape[0]] if w.numel() != p.numel() else w.reshape(p.shape))
            loaded.add(name)
        else:
            log.warning_once(f"checkpoint tensor {name} has no destination")
    return loaded


@torch.no_grad()
def dummy_init(model: nn.Module, seed: int = 0, std: float = 0.02) -> None:
    """Random-init every parameter in place. Floating tensors ~ N(0, std); norm weights = 1 (0 for Gemma-style);
    int4 codes uniform; fp16 group scales |N(0, 0.01)|; fp8 codes from N(0,1) with scales so that the dequantised
    weights have std ≈ ``std``; ue8m0 scales chosen likewise."""
    gens: dict = {}

    def gen(dev):
        if dev not in gens:
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            gens[dev] = g
        return gens[dev]

    for name, p in model.named_parameters():
        g = gen(p.device)
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("weight",) and name.endswith(("layernorm.weight", "norm.weight")) or leaf in ("q_norm", "k_norm", "norm_weight"):
            continue  # keep constructor init (1, or 0 for Gemma-style)
        if p.dtype in (torch.float32, torch.float16, torch.bfloat16):
            if leaf in ("scales",):
                p.copy_(torch.empty(p.shape, device=p.device, dtype=torch.float32).normal_(0, 0.01, generator=g).abs_().clamp_min_(1e-4))
            elif leaf in ("weight_scale_inv", "w13_scale", "w2_scale", "weight_scale"):
                p.fill_(std / 1.0 if leaf != "weight_scale" else std)
            elif leaf == "weight_scale_2":
                p.fill_(std / 2.0)
            elif leaf == "A_log":
                p.copy_(torch.empty(p.shape, device=p.device).uniform_(0.0, 2.0, generator=g).log1p_())
            elif leaf == "dt_bias":
                p.copy_(torch.empty(p.shape, device=p.device).uniform_(0.0, 1.0, generator=g))
            elif leaf == "e_score_correction_bias":
                p.zero_()
            else:
                p.copy_(torch.empty(p.shape, device=p.device, dtype=torch.float32).normal_(0, std, generator=g))
        elif p.dtype == torch.int32:
            if leaf == "g_idx":
                continue
            lo = torch.randint(0, 1 << 16, p.shape, device=p.device, generator=g, dtype=torch.int32)
            hi = torch.randint(0, 1 << 16, p.shape, device=p.device, generator=g, dtype=torch.int32)
            p.copy_((hi << 16) | lo)
        elif p.dtype == torch.float8_e4m3fn:
            if leaf == "weight_scale":  # nvfp4 block scales
                p.copy_(torch.ones(p.shape, device=p.device).to(torch.float8_e4m3fn))
            else:
                # chunked to bound temporary memory on large expert stacks
                flat = p.view(-1)
                step = 1 << 26
                for a in range(0, flat.numel(), step):
                    b = min(a + step, flat.numel())
                    flat[a:b] = torch.empty(b - a, device=p.device, dtype=torch.float32).normal_(0, 1.0, generator=g).to(torch.float8_e4m3fn)
        elif p.dtype == torch.uint8:
            if leaf in ("weight_scale", "w13_scale", "w2_scale"):  # ue8m0: 2^(e-127); e2m1 codes have std ~ 2.6
                p.fill_(127 - 7)
            else:
                flat = p.view(-1)
                step = 1 << 26
                for a in range(0, flat.numel(), step):
                    b = min(a + step, flat.numel())
                    flat[a:b] = torch.randint(0, 256, (b - a,), device=p.device, generator=g, dtype=torch.uint8)


def process_weights_after_loading(model: nn.Module) -> None:
    for m in model.modules():
        if m is not model and hasattr(m, "process_weights_after_loading"):
            m.process_weights_after_loading()


def load_model(cfg, device) -> nn.Module:
    """Build → load (or random-init) → repack for kernels."""
    from onecat_vllm.models import build_model
    dev = torch.device(device)
    torch.manual_seed(cfg.seed)
    with torch.device(dev):
        model = build_model(cfg, dev)
    fmt = cfg.load_format
    if fmt == "auto":
        fmt = "safetensors" if os.path.isdir(cfg.model) else ("gguf" if str(cfg.model).endswith(".gguf") and os.path.isfile(cfg.model) else "dummy")
    if fmt == "dummy":
        dummy_init(model, cfg.seed)
    elif fmt == "gguf":
        from onecat_vllm.loader.gguf import iter_gguf, resolve
        load_weights(model, iter_gguf(resolve(cfg.model) or cfg.model, cfg.dtype))
    else:
        load_weights(model, iter_safetensors(cfg.model))
    process_weights_after_loading(model)
    return model.eval()


_DS_MTP = {"enorm.": "pre_fc_norm_embedding.", "hnorm.": "pre_fc_norm_hidden.", "eh_proj.": "fc.", "shared_head.norm.": "norm."}


def mtp_checkpoint_weights(cfg, weights: Iterable[tuple[str, torch.Tensor]]) -> Iterator[tuple[str, torch.Tensor]]:
    """Checkpoint tensors of the multi-token-prediction module under the names of ``MTPHead``: Qwen3-Next / Qwen3.5 keep them as
    ``mtp.{fc, pre_fc_norm_*, norm, layers.0.*}``; DeepSeek-V3 as decoder layer ``num_hidden_layers`` with ``enorm / hnorm / eh_proj /
    shared_head.norm`` (reference: models/qwen3_5_mtp.py:437 ``load_weights``; models/deepseek_mtp.py). Embeddings and the LM head are
    the target's."""
    ds = f"model.layers.{cfg.num_hidden_layers}."
    for name, w in weights:
        if name.startswith("model.language_model."):
            name = "model." + name[len("model.language_model."):]
        if name.startswith("mtp."):
            n = name[4:]
            if n.startswith("layers.0."):
                n = "layer." + n[len("layers.0."):]
            elif n.startswith("layers."):
                continue  # deeper MTP modules are not used: one module drafts every position
            yield n, w
        elif name.startswith(ds):
            n = name[len(ds):]
            if n.startswith(("embed_tokens.", "shared_head.head.")):
                continue
            for theirs, ours in _DS_MTP.items():
                if n.startswith(theirs):
                    n = ours + n[len(theirs):]
                    break
            else:
                n = "layer." + n
            yield n, w


def load_mtp_weights(mtp: nn.Module, cfg) -> int:
    """Load the draft head from the target's checkpoint directory; returns how many tensors were found."""
    return len(load_weights(mtp, mtp_checkpoint_weights(cfg, iter_safetensors(cfg.model))))


def load_eagle_weights(head: nn.Module, path: str) -> int:
    """EAGLE checkpoints name their tensors ``fc.*``, ``embed_tokens.weight``, ``layers.0.*`` (optionally under ``model.``), in
    safetensors or ``pytorch_model.bin`` (reference: models/llama_eagle.py ``load_weights``)."""
    def tensors():
        if any(f.endswith(".safetensors") for f in os.listdir(path)):
            yield from iter_safetensors(path)
        else:
            yield from torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True).items()

    def renamed():
        for name, w in tensors():
            if name.startswith("model."):
                name = name[len("model."):]
            if name.startswith("lm_head."):
                continue
            if name.startswith("embed_tokens."):
                head.own_embedding = True
            if name.startswith("layers.0."):
                name = "layer." + name[len("layers.0."):]
            if name.startswith("layer.input_layernorm."):
                continue  # EAGLE skips the first layer's input norm
            yield name, w
    return len(load_weights(head, renamed()))


def load_eagle3_weights(head: nn.Module, path: str) -> int:
    """An EAGLE-3 checkpoint: ``fc``, ``midlayer.*`` (the decoder layer incl. ``hidden_norm``), ``norm``, ``lm_head``, optionally
    ``embed_tokens`` and the vocabulary maps ``d2t`` / ``t2d`` (reference: models/llama_eagle3.py ``load_weights``)."""
    def tensors():
        if any(f.endswith(".safetensors") for f in os.listdir(path)):
            yield from iter_safetensors(path)
        else:
            yield from torch.load(os.path.join(path, "pytorch_model.bin"), map_location="cpu", weights_only=True).items()

    def renamed():
        for name, w in tensors():
            if name.startswith("model."):
                name = name[len("model."):]
            if name == "d2t":
                head.d2t = w.to(torch.long).to(head.d2t.device)
                continue
            if name == "t2d":
                continue
            if name.startswith("embed_tokens."):
                head.own_embedding = True
            if name.startswith("lm_head."):
                head.own_lm_head = True
            for a, b in (("midlayer.hidden_norm.", "hidden_norm."), ("midlayer.", "layer."), ("layers.0.hidden_norm.", "hidden_norm."), ("layers.0.", "layer.")):
                if name.startswith(a):
                    name = b + name[len(a):]
                    break
            yield name, w
    return len(load_weights(head, renamed()))


def to_hf_state_dict(model: nn.Module) -> dict:
    """Un-stack fused parameters back to HF checkpoint names (q/k/v, gate/up, per-expert tensors), for saving a
    model built here as a checkpoint that any HF-layout loader (including this one) reads. TP size 1 only."""
    out = {}
    stacked = getattr(model, "stacked_params_mapping", [])
    mods = dict(model.named_modules())
    for name, p in model.state_dict().items():
        mod_name, _, pname = name.rpartition(".")
        mod = mods.get(mod_name)
        hits = [(theirs, sid) for ours, theirs, sid in stacked if mod_name.endswith(ours)]
        if hits and hasattr(mod, "local_output_sizes") and pname in ("weight", "bias", "qweight", "qzeros", "scales"):
            oa, od, _, _ = mod.method.layout(mod, pname) if pname != "bias" else (0, 1, None, 1)
            off = 0
            ours = [o for o, t, s in stacked if mod_name.endswith(o)][0]
            for theirs, sid in hits:
                n = mod.local_output_sizes[sid] // od
                out[mod_name[: -len(ours)] + theirs + "." + pname] = p.narrow(oa, off, n).contiguous()
                off += n
        elif mod_name.endswith(".experts") and pname in ("w13", "w2", "w13_scale", "w2_scale", "w13_bias", "w2_bias"):
            leaf = "weight" if pname in ("w13", "w2") else ("bias" if pname.endswith("bias") else "weight_scale_inv")
            for e in range(p.shape[0]):
                if pname.startswith("w13"):
                    h = p.shape[1] // 2
                    out[f"{mod_name}.{e}.gate_proj.{leaf}"] = p[e, :h].contiguous()
                    out[f"{mod_name}.{e}.up_proj.{leaf}"] = p[e, h:].contiguous()
                else:
                    out[f"{mod_name}.{e}.down_proj.{leaf}"] = p[e].contiguous()
        elif isinstance(mod, (nn.Module,)) and hasattr(mod, "vocab") and pname == "weight":
            out[name] = p[: mod.vocab].contiguous()
        else:
            out[name] = p.contiguous()
    return out


def save_pretrained(model: nn.Module, hf_config: dict, path: str) -> None:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    sd = {k: v.detach().cpu() for k, v in to_hf_state_dict(model).items()}
    save_file(sd, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf_config, f)
