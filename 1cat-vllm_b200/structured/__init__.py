"""Structured (grammar-constrained) decoding: per-request grammars compiled once, a packed token bitmask per step, and
matcher advancement on accepted tokens (reference: vllm/v1/structured_output/__init__.py:36 ``StructuredOutputManager``
with ``grammar_init`` / ``grammar_bitmask`` / ``should_advance``; backends ``backend_xgrammar.py:35``, ``backend_types.py``).

The manager lives next to the scheduler. Each step it produces ``[num_structured_requests, ceil(vocab/32)]`` int32 words
(bit set = token allowed) that travel inside the scheduler output; the model runner expands them onto the logits rows
before sampling. Two backends:

* ``xgrammar`` — JSON schema, regex, EBNF grammar, JSON object, choice (used when the library is importable);
* ``builtin`` — a byte-level trie for ``choice``, dependency-free, also the fallback when xgrammar cannot be loaded.

Requests under a grammar do not carry draft tokens: the scheduler drops drafts for them, so one bitmask row per request
per step is enough."""
from __future__ import annotations

from typing import Optional

import numpy as np

from onecat_vllm.logger import init_logger
from onecat_vllm.sampling_params import StructuredOutputsParams

log = init_logger(__name__)


def _vocab_bytes(tokenizer, vocab_size: int) -> list[bytes]:
    """Byte string of every token id (empty for ids the tokenizer cannot render, e.g. padding rows of the embedding)."""
    out: list[bytes] = []
    n_tok = getattr(tokenizer, "vocab_size", vocab_size)
    if hasattr(tokenizer, "get_vocab") and hasattr(tokenizer, "convert_ids_to_tokens"):
        try:
            n_tok = max(n_tok, len(tokenizer.get_vocab()))
        except Exception:
            pass
    special = set(getattr(tokenizer, "all_special_ids", []) or [])
    for i in range(vocab_size):
        if i >= n_tok or i in special:
            out.append(b"")
            continue
        if tokenizer.__class__.__name__ == "ByteTokenizer":
            out.append(bytes([i]) if i < 256 else b"")
            continue
        try:
            out.append(tokenizer.decode([i], skip_special_tokens=False).encode("utf-8"))
        except Exception:
            out.append(b"")
    return out


class Grammar:
    """One request's matcher. ``fill(row)`` writes the allowed-token words, ``accept(token)`` advances."""

    terminated = False

    def fill(self, row: np.ndarray) -> None:
        raise NotImplementedError

    def accept(self, token: int) -> bool:
        raise NotImplementedError

    def rollback(self, n: int) -> None:
        raise NotImplementedError


# ---------------------------------------------------------------------------------------------------------------- builtin
class _TrieGrammar(Grammar):
    """Accepts exactly one of a fixed set of byte strings, then only EOS."""

    def __init__(self, choices: list[bytes], vocab: list[bytes], eos: Optional[int]):
        self.choices = choices
        self.vocab = vocab
        self.eos = eos
        self.pos = b""
        self.history: list[bytes] = []
        self._by_first: dict[int, list[int]] = {}
        for t, b in enumerate(vocab):
            if b:
                self._by_first.setdefault(b[0], []).append(t)

    def _allowed(self) -> list[int]:
        live = [c[len(self.pos):] for c in self.choices if c.startswith(self.pos)]
        ok: list[int] = []
        firsts = {r[0] for r in live if r}
        for f in firsts:
            for t in self._by_first.get(f, ()):
                b = self.vocab[t]
                if any(r.startswith(b) for r in live):
                    ok.append(t)
        if any(len(r) == 0 for r in live) and self.eos is not None:
            ok.append(self.eos)
        return ok

    def fill(self, row: np.ndarray) -> None:
        row[:] = 0
        u = row.view(np.uint32)
        for t in self._allowed():
            u[t >> 5] |= np.uint32(1 << (t & 31))

    def accept(self, token: int) -> bool:
        if self.eos is not None and token == self.eos:
            done = self.pos in self.choices
            self.terminated = done
            self.history.append(b"")
            return done
        b = self.vocab[token] if 0 <= token < len(self.vocab) else b""
        nxt = self.pos + b
        if not b or not any(c.startswith(nxt) for c in self.choices):
            return False
        self.history.append(b)
        self.pos = nxt
        return True

    def rollback(self, n: int) -> None:
        for _ in range(n):
            b = self.history.pop()
            if b:
                self.pos = self.pos[: len(self.pos) - len(b)]
            self.terminated = False


class BuiltinBackend:
    name = "builtin"

    def __init__(self, tokenizer, vocab_size: int, eos: Optional[int]):
        self.vocab = _vocab_bytes(tokenizer, vocab_size)
        self.eos = eos

    def compile(self, so: StructuredOutputsParams) -> Grammar:
        kind = so.kind()
        if kind == "choice":
            return _TrieGrammar([c.encode("utf-8") for c in so.choice], self.vocab, self.eos)
        raise ValueError(f"structured output kind '{kind}' needs the xgrammar backend (only 'choice' is built in)")


# ---------------------------------------------------------------------------------------------------------------- xgrammar
class _XgrGrammar(Grammar):
    def __init__(self, matcher, words: int):
        self.m = matcher
        self.words = words

    @property
    def terminated(self) -> bool:  # type: ignore[override]
        return self.m.is_terminated()

    def fill(self, row: np.ndarray) -> None:
        import torch
        if self.m.is_terminated():
            row[:] = -1
            return
        self.m.fill_next_token_bitmask(torch.from_numpy(row.reshape(1, -1)), 0)

    def accept(self, token: int) -> bool:
        if self.m.is_terminated():
            return True
        return bool(self.m.accept_token(token))

    def rollback(self, n: int) -> None:
        self.m.rollback(n)


class XgrammarBackend:
    name = "xgrammar"

    def __init__(self, tokenizer, vocab_size: int, eos: Optional[int]):
        import xgrammar as xgr
        self.xgr = xgr
        self.vocab_size = vocab_size
        if tokenizer.__class__.__name__ == "ByteTokenizer" or not hasattr(tokenizer, "get_vocab"):
            enc = _vocab_bytes(tokenizer, vocab_size)
            info = xgr.TokenizerInfo(enc, vocab_type=xgr.VocabType.RAW, vocab_size=vocab_size,
                                     stop_token_ids=[eos] if eos is not None else None)
        else:
            info = xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=vocab_size,
                                                      stop_token_ids=[eos] if eos is not None else None)
        self.compiler = xgr.GrammarCompiler(info, max_threads=4, cache_enabled=True)
        self.words = (vocab_size + 31) // 32

    def compile(self, so: StructuredOutputsParams) -> Grammar:
        import json
        kind = so.kind()
        c, xgr = self.compiler, self.xgr
        if kind == "json":
            schema = so.json if isinstance(so.json, str) else json.dumps(so.json)
            cg = c.compile_json_schema(schema, any_whitespace=True)
        elif kind == "json_object":
            cg = c.compile_builtin_json_grammar()
        elif kind == "regex":
            cg = c.compile_regex(so.regex)
        elif kind == "grammar":
            cg = c.compile_grammar(so.grammar)
        elif kind == "choice":
            esc = lambda s: json.dumps(s)
            cg = c.compile_grammar("root ::= " + " | ".join(esc(x) for x in so.choice))
        else:
            raise ValueError(f"unknown structured output kind '{kind}'")
        return _XgrGrammar(xgr.GrammarMatcher(cg, max_rollback_tokens=8), self.words)


# ---------------------------------------------------------------------------------------------------------------- manager
class StructuredOutputManager:
    def __init__(self, tokenizer, vocab_size: int, eos_token_id: Optional[int] = None, backend: str = "auto"):
        self.vocab_size = vocab_size
        self.words = (vocab_size + 31) // 32
        self.tokenizer = tokenizer
        self.eos = eos_token_id if eos_token_id is not None else getattr(tokenizer, "eos_token_id", None)
        self._backend_name = backend
        self._backends: dict[str, object] = {}
        self.grammars: dict[str, Grammar] = {}

    def _backend(self, kind: str):
        name = self._backend_name
        if name == "auto":
            try:
                import xgrammar  # noqa: F401
                name = "xgrammar"
            except Exception:
                name = "builtin"
        if name not in self._backends:
            if self.tokenizer is None:
                raise ValueError("structured outputs need a tokenizer")
            cls = XgrammarBackend if name == "xgrammar" else BuiltinBackend
            try:
                self._backends[name] = cls(self.tokenizer, self.vocab_size, self.eos)
            except Exception as e:
                if name == "xgrammar" and kind == "choice":
                    log.warning(f"xgrammar backend unavailable ({e!r}); using the built-in trie for 'choice'")
                    self._backends[name] = BuiltinBackend(self.tokenizer, self.vocab_size, self.eos)
                else:
                    raise
        return self._backends[name]

    # ---- request lifecycle
    def grammar_init(self, request_id: str, so: Optional[StructuredOutputsParams]) -> bool:
        if so is None or so.kind() == "none":
            return False
        self.grammars[request_id] = self._backend(so.kind()).compile(so)
        return True

    def has(self, request_id: str) -> bool:
        return request_id in self.grammars

    def free(self, request_id: str) -> None:
        self.grammars.pop(request_id, None)

    # ---- per step
    def grammar_bitmask(self, req_ids: list[str]) -> tuple[Optional[np.ndarray], dict[str, int]]:
        """Bitmask rows for those of ``req_ids`` that run under a grammar, and request id → row."""
        rows = {rid: i for i, rid in enumerate(r for r in req_ids if r in self.grammars)}
        if not rows:
            return None, {}
        mask = np.full((len(rows), self.words), -1, dtype=np.int32)
        for rid, i in rows.items():
            self.grammars[rid].fill(mask[i])
        return mask, rows

    def accept_tokens(self, request_id: str, tokens: list[int]) -> bool:
        g = self.grammars.get(request_id)
        if g is None:
            return True
        ok = True
        for t in tokens:
            if not g.accept(int(t)):
                ok = False
                break
        return ok


def unpack_bitmask(mask: np.ndarray, vocab_size: int):
    """``[n, words]`` int32 → ``[n, vocab_size]`` bool (bit set = allowed). Host-side helper and test oracle."""
    bits = np.unpackbits(mask.view(np.uint8), axis=1, bitorder="little")
    return bits[:, :vocab_size].astype(bool)
