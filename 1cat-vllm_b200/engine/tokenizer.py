"""Tokenizer access + incremental detokenisation (reference: vllm/tokenizers/registry.py:55;
v1/engine/detokenizer.py:167,250). HF tokenizers load through ``transformers``; a model without tokenizer serves
token-id prompts only. ``ByteTokenizer`` is a dependency-free stand-in used by tests and the mock engine."""
from __future__ import annotations

from typing import Optional


class ByteTokenizer:
    """ids 0..255 are raw bytes; 256 = BOS, 257 = EOS."""

    vocab_size = 258
    bos_token_id, eos_token_id = 256, 257
    chat_template = None

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        b = bytes(i for i in ids if i < 256)
        return b.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
        text = "".join(f"<|{m['role']}|>{m['content'] if isinstance(m['content'], str) else ''}\n" for m in messages)
        if add_generation_prompt:
            text += "<|assistant|>"
        return self.encode(text) if tokenize else text


def get_tokenizer(path: Optional[str]):
    if path is None:
        return None
    if path == "byte":
        return ByteTokenizer()
    from onecat_vllm.engine.renderers import load_tokenizer
    return load_tokenizer(path)   # HF files, or Mistral's tekken.json when that is all the directory has


class IncrementalDetokenizer:
    """Decodes a growing id list into text deltas, holding back bytes of incomplete UTF-8 sequences, and watches
    for stop strings (reference: detokenizer.py ``check_stop_strings``)."""

    def __init__(self, tokenizer, prompt_ids: list[int], skip_special_tokens: bool = True, stop: Optional[list[str]] = None,
                 include_stop_str: bool = False):
        self.tok = tokenizer
        self.skip = skip_special_tokens
        self.ids: list[int] = []
        self.text = ""
        self._prefix_offset = 0  # ids[:prefix] are fully flushed
        self._read_offset = 0
        self.stop = stop or []
        self.include_stop = include_stop_str
        self._stop_scan_from = 0

    def update(self, new_ids: list[int], finished: bool = False) -> Optional[str]:
        """Append ids; returns the matched stop string, if any (text is truncated accordingly)."""
        if self.tok is None:
            self.ids.extend(new_ids)
            return None
        for t in new_ids:
            self.ids.append(t)
            prefix = self.tok.decode(self.ids[self._prefix_offset:self._read_offset], skip_special_tokens=self.skip)
            full = self.tok.decode(self.ids[self._prefix_offset:], skip_special_tokens=self.skip)
            if len(full) > len(prefix) and not full.endswith("�"):
                self.text += full[len(prefix):]
                self._prefix_offset, self._read_offset = self._read_offset, len(self.ids)
        if finished and self._read_offset < len(self.ids):
            prefix = self.tok.decode(self.ids[self._prefix_offset:self._read_offset], skip_special_tokens=self.skip)
            full = self.tok.decode(self.ids[self._prefix_offset:], skip_special_tokens=self.skip)
            self.text += full[len(prefix):]
            self._read_offset = len(self.ids)
        if self.stop:
            start = max(0, self._stop_scan_from - max(len(s) for s in self.stop))
            for s in self.stop:
                i = self.text.find(s, start)
                if i != -1:
                    self.text = self.text[: i + len(s)] if self.include_stop else self.text[:i]
                    return s
            self._stop_scan_from = len(self.text)
        return None
