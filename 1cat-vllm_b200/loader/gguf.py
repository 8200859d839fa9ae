"""GGUF checkpoints: a reader for the container (header, metadata, tensor table), dequantisation of the common ggml block
formats, the mapping from GGUF tensor names to the names of an HF checkpoint, and an HF-style config built from the metadata.

The tensors are dequantised to the model's dtype while loading (the quantised layers of this framework take AWQ / GPTQ / FP8 /
FP4 packings; the ggml block formats are not one of them), so a GGUF model runs on the bf16 kernels.
(reference: model_executor/model_loader/gguf_loader.py:60-140 for the file discovery and the name map, which the reference takes
from the ``gguf`` package; model_executor/layers/quantization/gguf.py for the formats it keeps packed.)"""
from __future__ import annotations

import os
import re
import struct
from typing import Any, Iterator

import numpy as np
import torch

GGUF_MAGIC = 0x46554747  # "GGUF", little endian
# value types of the metadata section
_T_U8, _T_I8, _T_U16, _T_I16, _T_U32, _T_I32, _T_F32, _T_BOOL, _T_STR, _T_ARR, _T_U64, _T_I64, _T_F64 = range(13)
_SCALAR = {_T_U8: "<B", _T_I8: "<b", _T_U16: "<H", _T_I16: "<h", _T_U32: "<I", _T_I32: "<i", _T_F32: "<f", _T_BOOL: "<?",
           _T_U64: "<Q", _T_I64: "<q", _T_F64: "<d"}
# ggml tensor types: id -> (name, elements per block, bytes per block)
GGML_TYPES = {0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22), 7: ("Q5_1", 32, 24),
              8: ("Q8_0", 32, 34), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110), 12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176),
              14: ("Q6_K", 256, 210), 24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8),
              30: ("BF16", 1, 2)}


class GGUFFile:
    """Memory-mapped view of one ``.gguf`` file: ``metadata`` (dict) and ``tensors`` (name -> (type id, shape, byte offset))."""

    def __init__(self, path: str):
        self.path = path
        self.buf = np.memmap(path, dtype=np.uint8, mode="r")
        self._o = 0
        magic, version = self._unpack("<II")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        if version not in (2, 3):
            raise ValueError(f"{path}: GGUF version {version} is not supported")
        n_tensors, n_kv = self._unpack("<QQ")
        self.metadata: dict[str, Any] = {}
        for _ in range(n_kv):
            key = self._string()
            (vt,) = self._unpack("<I")
            self.metadata[key] = self._value(vt)
        self.tensors: dict[str, tuple[int, tuple[int, ...], int]] = {}
        infos = []
        for _ in range(n_tensors):
            name = self._string()
            (nd,) = self._unpack("<I")
            dims = self._unpack(f"<{nd}Q")
            ttype, off = self._unpack("<IQ")
            infos.append((name, ttype, tuple(reversed(dims)), off))  # ggml lists the innermost dimension first
        align = int(self.metadata.get("general.alignment", 32))
        base = (self._o + align - 1) // align * align
        for name, ttype, shape, off in infos:
            self.tensors[name] = (ttype, shape, base + off)

    def _unpack(self, fmt: str):
        n = struct.calcsize(fmt)
        out = struct.unpack_from(fmt, self.buf, self._o)
        self._o += n
        return out

    def _string(self) -> str:
        (n,) = self._unpack("<Q")
        s = bytes(self.buf[self._o:self._o + n]).decode("utf-8", errors="replace")
        self._o += n
        return s

    def _value(self, vt: int):
        if vt in _SCALAR:
            return self._unpack(_SCALAR[vt])[0]
        if vt == _T_STR:
            return self._string()
        if vt == _T_ARR:
            et, n = self._unpack("<IQ")
            if et in _SCALAR:
                fmt = _SCALAR[et]
                sz = struct.calcsize(fmt)
                arr = np.frombuffer(self.buf, dtype=np.dtype(fmt), count=n, offset=self._o)
                self._o += sz * n
                return arr
            return [self._value(et) for _ in range(n)]
        raise ValueError(f"{self.path}: unknown metadata value type {vt}")

    def raw(self, name: str) -> tuple[int, tuple[int, ...], np.ndarray]:
        """(type id, logical shape, the tensor's bytes)."""
        ttype, shape, off = self.tensors[name]
        if ttype not in GGML_TYPES:
            raise ValueError(f"{self.path}: tensor {name} has ggml type {ttype}, which this loader does not know")
        _, bl, bb = GGML_TYPES[ttype]
        n = int(np.prod(shape)) if shape else 1
        if n % bl:
            raise ValueError(f"{self.path}: tensor {name} does not fill whole blocks")
        return ttype, shape, self.buf[off:off + n // bl * bb]

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor dequantised to fp32 (integer and fp64 types keep their own dtype; bf16/fp16 keep theirs)."""
        ttype, shape, data = self.raw(name)
        return dequantize(data, ttype).reshape(shape)


# ----------------------------------------------------------------------------- block formats
def _f16(b: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def _k_scale_min(sc: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """The eight 6-bit (scale, min) pairs of a Q4_K / Q5_K block from its 12 packed bytes: pairs 0-3 sit in the low six bits of
    bytes 0-3 / 4-7; pairs 4-7 take their low nibble from bytes 8-11 and their top two bits from the top of bytes 0-3 / 4-7."""
    sc = sc.astype(np.uint8)
    lo_s = sc[:, 0:4] & 63
    lo_m = sc[:, 4:8] & 63
    hi_s = (sc[:, 8:12] & 0x0F) | ((sc[:, 0:4] >> 6) << 4)
    hi_m = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return (np.concatenate([lo_s, hi_s], 1).astype(np.float32), np.concatenate([lo_m, hi_m], 1).astype(np.float32))


def _dq_q8_0(b):
    d = _f16(b[:, 0:2])
    return d * b[:, 2:34].view(np.int8).astype(np.float32)


def _dq_q4_0(b):
    d = _f16(b[:, 0:2])
    qs = b[:, 2:18]
    q = np.concatenate([qs & 0x0F, qs >> 4], 1).astype(np.float32) - 8.0
    return d * q


def _dq_q4_1(b):
    d, m = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    qs = b[:, 4:20]
    return d * np.concatenate([qs & 0x0F, qs >> 4], 1).astype(np.float32) + m


def _fifth_bits(qh: np.ndarray) -> np.ndarray:
    """[blocks, 32] fifth bit of each element from the block's 32-bit mask."""
    word = np.ascontiguousarray(qh).view(np.uint32).astype(np.uint32)  # [blocks, 1]
    return ((word >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.uint8)


def _dq_q5_0(b):
    d = _f16(b[:, 0:2])
    hb = _fifth_bits(b[:, 2:6])
    qs = b[:, 6:22]
    q = np.concatenate([qs & 0x0F, qs >> 4], 1) | (hb << 4)
    return d * (q.astype(np.float32) - 16.0)


def _dq_q5_1(b):
    d, m = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    hb = _fifth_bits(b[:, 4:8])
    qs = b[:, 8:24]
    q = np.concatenate([qs & 0x0F, qs >> 4], 1) | (hb << 4)
    return d * q.astype(np.float32) + m


def _dq_q4_k(b):
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k_scale_min(b[:, 4:16])
    qs = b[:, 16:144].reshape(-1, 4, 32)  # four 64-element chunks: low nibbles are its first 32 elements, high nibbles the next 32
    q = np.stack([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)
    return ((d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]).reshape(-1, 256)


def _dq_q5_k(b):
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k_scale_min(b[:, 4:16])
    qh = b[:, 16:48]                       # bit s of byte l is the fifth bit of element l of sub-block s
    qs = b[:, 48:176].reshape(-1, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32)
    hb = (qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1
    q = (q | (hb << 4)).astype(np.float32)
    return ((d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]).reshape(-1, 256)


def _dq_q6_k(b):
    ql = b[:, 0:128].reshape(-1, 2, 64)    # two halves of 128 elements
    qh = b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = _f16(b[:, 208:210])
    l0, l1 = ql[:, :, 0:32], ql[:, :, 32:64]
    q = np.stack([(l0 & 0x0F) | ((qh & 3) << 4), (l1 & 0x0F) | (((qh >> 2) & 3) << 4),
                  (l0 >> 4) | (((qh >> 4) & 3) << 4), (l1 >> 4) | (((qh >> 6) & 3) << 4)], 2)  # [blocks, 2, 4, 32]
    q = q.astype(np.float32) - 32.0
    s = sc.reshape(-1, 2, 4, 2)            # within a half, elements 32j .. 32j+31 use scales 2j (first 16) and 2j + 1
    s = np.repeat(s, 16, axis=3)           # [blocks, 2, 4, 32]
    return (d[:, :, None, None] * s * q).reshape(-1, 256)


_DEQUANT = {2: _dq_q4_0, 3: _dq_q4_1, 6: _dq_q5_0, 7: _dq_q5_1, 8: _dq_q8_0, 12: _dq_q4_k, 13: _dq_q5_k, 14: _dq_q6_k}
_PLAIN = {0: np.float32, 1: np.float16, 24: np.int8, 25: np.int16, 26: np.int32, 27: np.int64, 28: np.float64}


def dequantize(data: np.ndarray, ttype: int) -> torch.Tensor:
    """Flat tensor of the values stored in ``data`` (bytes of whole blocks of ggml type ``ttype``)."""
    data = np.ascontiguousarray(data)
    if ttype in _PLAIN:
        return torch.from_numpy(data.view(_PLAIN[ttype]).copy())
    if ttype == 30:
        return torch.from_numpy(data.view(np.int16).copy()).view(torch.bfloat16)
    name, bl, bb = GGML_TYPES[ttype]
    blocks = data.reshape(-1, bb)
    fn = _DEQUANT.get(ttype)
    if fn is None:
        try:  # the less common formats (Q2_K, Q3_K) through the gguf package when it is installed
            from gguf import quants
            return torch.from_numpy(np.ascontiguousarray(quants.dequantize(blocks, quants.GGMLQuantizationType(ttype))).reshape(-1).astype(np.float32))
        except ImportError as e:
            raise ValueError(f"ggml type {name} needs the gguf package") from e
    return torch.from_numpy(fn(blocks).reshape(-1).astype(np.float32))


# ----------------------------------------------------------------------------- names and config
_TOP = {"token_embd": "model.embed_tokens", "output_norm": "model.norm", "output": "lm_head"}
_BLK = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
        "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj", "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
        "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj", "ffn_gate_inp": "mlp.gate",
        "post_attention_norm": "post_attention_layernorm", "post_ffw_norm": "post_feedforward_layernorm",
        "ffn_gate_shexp": "mlp.shared_expert.gate_proj", "ffn_up_shexp": "mlp.shared_expert.up_proj",
        "ffn_down_shexp": "mlp.shared_expert.down_proj", "ffn_gate_inp_shexp": "mlp.shared_expert_gate"}
_EXPERTS = {"ffn_gate_exps": "gate_proj", "ffn_up_exps": "up_proj", "ffn_down_exps": "down_proj"}
_BLK_RE = re.compile(r"^blk\.(\d+)\.([a-z_]+)\.(weight|bias)$")
_ARCHS = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen2moe": "Qwen2MoeForCausalLM",
          "qwen3moe": "Qwen3MoeForCausalLM"}


def hf_name(gguf_name: str) -> str | None:
    """HF checkpoint name of a GGUF tensor (None for tensors that have no counterpart, such as ``rope_freqs``). Merged expert
    tensors map to ``...mlp.experts.{gate,up,down}_proj`` + ``.weight`` and are split per expert by ``iter_gguf``."""
    base, _, suffix = gguf_name.rpartition(".")
    if base in _TOP:
        return f"{_TOP[base]}.{suffix}"
    m = _BLK_RE.match(gguf_name)
    if not m:
        return None
    layer, part, suffix = m.groups()
    if part in _BLK:
        return f"model.layers.{layer}.{_BLK[part]}.{suffix}"
    if part in _EXPERTS:
        return f"model.layers.{layer}.mlp.experts.{_EXPERTS[part]}.{suffix}"
    return None


def config_from_metadata(md: dict, tensors: dict) -> dict:
    """An HF ``config.json`` for the architectures whose GGUF tensors map one to one onto the HF checkpoint (llama, which Mistral
    files also use, qwen2, qwen3 and their MoE forms), from the ``{arch}.*`` metadata keys."""
    arch = md.get("general.architecture")
    if arch not in _ARCHS:
        raise ValueError(f"GGUF architecture {arch!r}: pass a directory with config.json beside the file instead")

    def g(key, default=None):
        return md.get(f"{arch}.{key}", default)
    heads = int(g("attention.head_count"))
    hidden = int(g("embedding_length"))
    vocab = len(md["tokenizer.ggml.tokens"]) if "tokenizer.ggml.tokens" in md else int(tensors["token_embd.weight"][1][0])
    cfg = dict(architectures=[_ARCHS[arch]], model_type=arch.replace("qwen2moe", "qwen2_moe").replace("qwen3moe", "qwen3_moe"),
               hidden_size=hidden, num_hidden_layers=int(g("block_count")), num_attention_heads=heads,
               num_key_value_heads=int(g("attention.head_count_kv", heads)), intermediate_size=int(g("feed_forward_length", 4 * hidden)),
               rms_norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-6)), rope_theta=float(g("rope.freq_base", 10000.0)),
               max_position_embeddings=int(g("context_length", 4096)), vocab_size=vocab,
               head_dim=int(g("attention.key_length", hidden // heads)), tie_word_embeddings="output.weight" not in tensors)
    if g("expert_count"):
        cfg.update(num_experts=int(g("expert_count")), num_experts_per_tok=int(g("expert_used_count")),
                   moe_intermediate_size=int(g("expert_feed_forward_length", cfg["intermediate_size"])), norm_topk_prob=True)
    if "tokenizer.ggml.bos_token_id" in md:
        cfg["bos_token_id"] = int(md["tokenizer.ggml.bos_token_id"])
    if "tokenizer.ggml.eos_token_id" in md:
        cfg["eos_token_id"] = int(md["tokenizer.ggml.eos_token_id"])
    if arch == "qwen2":
        cfg["attention_bias"] = True
    return cfg


def gguf_files(path: str) -> list[str]:
    """All shards of a split GGUF model, given any one of them (``name-00001-of-00003.gguf``)."""
    m = re.search(r"-(\d+)-of-(\d+)\.gguf$", path)
    if not m:
        return [path]
    width, total = len(m.group(1)), int(m.group(2))
    out = [f"{path[:m.start(1)]}{i:0{width}d}-of-{m.group(2)}.gguf" for i in range(1, total + 1)]
    return [f for f in out if os.path.isfile(f)] or [path]


def resolve(path: str) -> str | None:
    """The ``.gguf`` file behind a model path: the file itself, or the only such file (or first shard) in a directory."""
    if os.path.isfile(path) and path.endswith(".gguf"):
        return path
    if os.path.isdir(path):
        found = sorted(f for f in os.listdir(path) if f.endswith(".gguf"))
        if found and not any(f.endswith(".safetensors") for f in os.listdir(path)):
            return os.path.join(path, found[0])
    return None


def _unpermute_llama(w: torch.Tensor, heads: int) -> torch.Tensor:
    """llama-architecture GGUF files store q and k with each head's rows regrouped for adjacent-pair rotary embedding; this
    restores the HF (half-split) row order."""
    rows = w.shape[0]
    return w.reshape(heads, rows // heads // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def iter_gguf(path: str, dtype: torch.dtype = torch.float32) -> Iterator[tuple[str, torch.Tensor]]:
    """(HF name, tensor) pairs of a GGUF model, dequantised; 2-D and larger float tensors in ``dtype``."""
    for fpath in gguf_files(path):
        f = GGUFFile(fpath)
        arch = f.metadata.get("general.architecture")
        heads = int(f.metadata.get(f"{arch}.attention.head_count", 0) or 0)
        kv_heads = int(f.metadata.get(f"{arch}.attention.head_count_kv", heads) or heads)
        for name in f.tensors:
            hn = hf_name(name)
            if hn is None:
                continue
            t = f.tensor(name)
            if t.is_floating_point():
                t = t.to(dtype if t.dim() >= 2 else torch.float32)
            if arch == "llama" and heads and (name.endswith("attn_q.weight") or name.endswith("attn_q.bias")):
                t = _unpermute_llama(t, heads)
            if arch == "llama" and kv_heads and (name.endswith("attn_k.weight") or name.endswith("attn_k.bias")):
                t = _unpermute_llama(t, kv_heads)
            if ".mlp.experts." in hn and t.dim() == 3:  # merged [experts, out, in] -> one tensor per expert
                pre, proj, suffix = hn.rsplit(".", 2)
                for e in range(t.shape[0]):
                    yield f"{pre}.{e}.{proj}.{suffix}", t[e]
                continue
            yield hn, t
