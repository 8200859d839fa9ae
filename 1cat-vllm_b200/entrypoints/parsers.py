"""Reasoning and tool-call parsers for chat responses, streaming and non-streaming
(reference: vllm/reasoning/abs_reasoning_parsers.py:26,189; vllm/tool_parsers/abstract_tool_parser.py:43,192; model parsers
hermes_tool_parser.py, qwen3coder_tool_parser.py, deepseekv3_tool_parser.py, deepseek_r1_reasoning_parser.py).

Both kinds work on text. Streaming variants are fed the accumulated text and return the delta that may be shown, holding
back anything that could still turn out to be the start of a tag."""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Optional


# ----------------------------------------------------------------------------- reasoning
class ReasoningParser:
    """``<think> … </think>`` splitter. Models whose template opens the block itself (DeepSeek-R1, Qwen3 thinking) may
    emit only the closing tag; then everything before it is reasoning."""

    start, end = "<think>", "</think>"

    def __init__(self, assume_open: bool = False):
        self.assume_open = assume_open

    def extract(self, text: str) -> tuple[Optional[str], Optional[str]]:
        s, e = text.find(self.start), text.find(self.end)
        if e != -1:
            r0 = s + len(self.start) if s != -1 and s < e else 0
            return text[r0:e] or None, text[e + len(self.end):] or None
        if s != -1:
            return text[s + len(self.start):] or None, None
        return (text or None, None) if self.assume_open else (None, text or None)

    def stream(self, prev: str, cur: str) -> tuple[str, str]:
        """(reasoning delta, content delta) between two accumulated texts."""
        pr, pc = self._split_partial(prev)
        cr, cc = self._split_partial(cur)
        return cr[len(pr):], cc[len(pc):]

    def _split_partial(self, text: str) -> tuple[str, str]:
        # hold back a trailing fragment that is a prefix of a tag
        for tag in (self.end, self.start):
            for k in range(len(tag) - 1, 0, -1):
                if text.endswith(tag[:k]):
                    text = text[:-k]
                    break
        r, c = self.extract(text)
        return r or "", c or ""


REASONING_PARSERS = {"qwen3": lambda: ReasoningParser(False), "deepseek_r1": lambda: ReasoningParser(True),
                     "deepseek_v3": lambda: ReasoningParser(False), "think": lambda: ReasoningParser(False)}


# ----------------------------------------------------------------------------- tools
@dataclass
class ToolCall:
    name: str
    arguments: str  # JSON text
    id: str = field(default_factory=lambda: "chatcmpl-tool-" + uuid.uuid4().hex[:24])

    def to_openai(self, index: Optional[int] = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


class ToolParser:
    """Returns (content without the tool-call markup, tool calls)."""

    def extract(self, text: str) -> tuple[Optional[str], list[ToolCall]]:
        raise NotImplementedError

    def content_so_far(self, text: str) -> str:
        """Streaming: the part of ``text`` that is certainly plain content."""
        i = self._first_marker(text)
        return text if i < 0 else text[:i]

    markers: tuple = ()

    def _first_marker(self, text: str) -> int:
        best = -1
        for m in self.markers:
            i = text.find(m)
            if i != -1 and (best == -1 or i < best):
                best = i
            for k in range(len(m) - 1, 0, -1):  # a partial marker at the very end is held back too
                if text.endswith(m[:k]):
                    j = len(text) - k
                    if best == -1 or j < best:
                        best = j
                    break
        return best


class HermesToolParser(ToolParser):
    markers = ("<tool_call>",)
    _re = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.S)

    def extract(self, text):
        calls = []
        for m in self._re.finditer(text):
            try:
                d = json.loads(m.group(1))
                calls.append(ToolCall(d["name"], json.dumps(d.get("arguments", d.get("parameters", {})), ensure_ascii=False)))
            except (json.JSONDecodeError, KeyError, TypeError):
                continue
        if not calls:
            return text, []
        return text[: text.find("<tool_call>")].strip() or None, calls


class Qwen3CoderToolParser(ToolParser):
    markers = ("<tool_call>", "<function=")
    _fn = re.compile(r"<function=([^>\s]+)>(.*?)(?:</function>|$)", re.S)
    _par = re.compile(r"<parameter=([^>\s]+)>(.*?)(?:</parameter>|(?=<parameter=)|$)", re.S)

    def extract(self, text):
        calls = []
        for m in self._fn.finditer(text):
            args = {}
            for p in self._par.finditer(m.group(2)):
                v = p.group(2).strip("\n")
                try:
                    args[p.group(1)] = json.loads(v)
                except json.JSONDecodeError:
                    args[p.group(1)] = v
            calls.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        i = self._first_marker(text)
        return text[:i].strip() or None, calls


class DeepSeekV3ToolParser(ToolParser):
    B, E = "<｜tool▁calls▁begin｜>", "<｜tool▁calls▁end｜>"
    markers = (B,)
    _re = re.compile(r"<｜tool▁call▁begin｜>(?:function<｜tool▁sep｜>)?([^\n<]+)\n```json\n(.*?)\n```\s*<｜tool▁call▁end｜>", re.S)

    def extract(self, text):
        calls = [ToolCall(m.group(1).strip(), m.group(2).strip()) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return text[: text.find(self.B)].strip() or None, calls


TOOL_PARSERS = {"hermes": HermesToolParser, "qwen3_coder": Qwen3CoderToolParser, "qwen3_xml": Qwen3CoderToolParser,
                "deepseek_v3": DeepSeekV3ToolParser, "deepseek_v31": DeepSeekV3ToolParser}


def get_tool_parser(name: Optional[str]) -> Optional[ToolParser]:
    if not name:
        return None
    if name not in TOOL_PARSERS:
        raise ValueError(f"unknown tool parser {name!r}; available: {sorted(TOOL_PARSERS)}")
    return TOOL_PARSERS[name]()


def get_reasoning_parser(name: Optional[str]) -> Optional[ReasoningParser]:
    if not name:
        return None
    if name not in REASONING_PARSERS:
        raise ValueError(f"unknown reasoning parser {name!r}; available: {sorted(REASONING_PARSERS)}")
    return REASONING_PARSERS[name]()
