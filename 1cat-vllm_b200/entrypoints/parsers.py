"""Reasoning and tool-call parsers for chat responses, streaming and non-streaming
(reference: vllm/reasoning/abs_reasoning_parsers.py:26,189; vllm/tool_parsers/abstract_tool_parser.py:43,192; model parsers
hermes_tool_parser.py, qwen3coder_tool_parser.py, deepseekv3_tool_parser.py, deepseek_r1_reasoning_parser.py; the other
registered names follow the published output formats of the respective model families).

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


class TaggedReasoningParser(ReasoningParser):
    """Same splitter with other tag strings (Mistral ``[THINK]``, Seed-OSS ``<seed:think>``)."""

    def __init__(self, start: str, end: str, assume_open: bool = False):
        super().__init__(assume_open)
        self.start, self.end = start, end


class Gemma4ReasoningParser(TaggedReasoningParser):
    """Gemma-4: reasoning sits in a channel, ``<|channel>thought\n ... <channel|>``; the ``thought`` role label at the start of the
    channel is structure, not reasoning text (reference: reasoning/gemma4_reasoning_parser.py:17-40)."""

    def __init__(self):
        super().__init__("<|channel>", "<channel|>", False)

    @staticmethod
    def _strip_label(r):
        if r is None:
            return None
        for label in ("thought\n", "thought"):
            if r.startswith(label):
                return r[len(label):] or None
        return r

    def extract(self, text):
        r, c = super().extract(text)
        return self._strip_label(r), c

    def _split_partial(self, text):
        r, c = super()._split_partial(text)
        if r and "thought\n".startswith(r):   # the label itself is still arriving
            return "", c
        return self._strip_label(r) or "", c


class PhraseReasoningParser(ReasoningParser):
    """Granite-style: reasoning and answer are introduced by fixed phrases instead of tags."""

    def __init__(self, think: tuple = ("Here is my thought process:", "Here's my thought process:"),
                 answer: tuple = ("Here is my response:", "Here's my response:")):
        super().__init__(False)
        self.think, self.answer = think, answer

    def extract(self, text):
        ti = min((i for i in (text.find(t) for t in self.think) if i != -1), default=-1)
        if ti == -1:
            return None, text or None
        tlen = next(len(t) for t in self.think if text.startswith(t, ti))
        rest = text[ti + tlen:]
        ai = min((i for i in (rest.find(t) for t in self.answer) if i != -1), default=-1)
        if ai == -1:
            return rest.strip() or None, None
        alen = next(len(t) for t in self.answer if rest.startswith(t, ai))
        return rest[:ai].strip() or None, rest[ai + alen:].strip() or None

    def _split_partial(self, text):
        r, c = self.extract(text)
        return r or "", c or ""


class IdentityReasoningParser(ReasoningParser):
    """No reasoning section: everything is content (reference: reasoning/identity_reasoning_parser.py)."""

    def extract(self, text):
        return None, text or None

    def _split_partial(self, text):
        return "", text


class ChannelReasoningParser(ReasoningParser):
    """GPT-OSS / harmony style: ``<|channel|>analysis<|message|>…<|end|>`` carries the reasoning and
    ``<|channel|>final<|message|>…`` the answer (reference: reasoning/gptoss_reasoning_parser.py)."""

    def __init__(self):
        super().__init__(False)

    def extract(self, text):
        import re
        parts = re.split(r"<\|channel\|>(\w+)<\|message\|>", text)
        if len(parts) < 3:
            return None, text or None
        reasoning, content = [], []
        for ch, body in zip(parts[1::2], parts[2::2]):
            body = re.split(r"<\|end\|>|<\|return\|>|<\|start\|>", body)[0]
            (content if ch == "final" else reasoning).append(body)
        return "".join(reasoning) or None, "".join(content) or None

    def _split_partial(self, text):
        cut = text.rfind("<|")
        if cut != -1 and "|>" not in text[cut:]:
            text = text[:cut]   # hold back an unfinished control token
        r, c = self.extract(text)
        return r or "", c or ""


REASONING_PARSERS = {"identity": IdentityReasoningParser, "gptoss": ChannelReasoningParser, "openai_gptoss": ChannelReasoningParser,
                     "nemotron_v3": lambda: ReasoningParser(True), "step3p5": lambda: ReasoningParser(True),
                     "hy_v3": lambda: ReasoningParser(False), "poolside_v1": lambda: ReasoningParser(False),
                     "cohere_command": lambda: TaggedReasoningParser("<|START_THINKING|>", "<|END_THINKING|>"),
                     "qwen3": lambda: ReasoningParser(False), "deepseek_r1": lambda: ReasoningParser(True),
                     "deepseek_v3": lambda: ReasoningParser(False), "think": lambda: ReasoningParser(False),
                     "glm45": lambda: ReasoningParser(False), "ernie45": lambda: ReasoningParser(True), "step3": lambda: ReasoningParser(True),
                     "minimax_m2": lambda: ReasoningParser(True), "olmo3": lambda: ReasoningParser(False), "kimi_k2": lambda: ReasoningParser(False),
                     "mistral": lambda: TaggedReasoningParser("[THINK]", "[/THINK]"),
                     "seed_oss": lambda: TaggedReasoningParser("<seed:think>", "</seed:think>"),
                     "seedoss": lambda: TaggedReasoningParser("<seed:think>", "</seed:think>"), "gemma4": Gemma4ReasoningParser,
                     "hunyuan_a13b": lambda: TaggedReasoningParser("<think>", "</think>"),
                     "granite": lambda: PhraseReasoningParser()}


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


class DeepSeekV31ToolParser(ToolParser):
    """V3.1 drops the ``function`` prefix and the code fence: ``<｜tool▁call▁begin｜>name<｜tool▁sep｜>{json}<｜tool▁call▁end｜>``."""

    B = "<｜tool▁calls▁begin｜>"
    markers = (B,)
    _re = re.compile(r"<｜tool▁call▁begin｜>(.*?)<｜tool▁sep｜>(.*?)<｜tool▁call▁end｜>", re.S)

    def extract(self, text):
        calls = []
        for m in self._re.finditer(text):
            name, args = m.group(1).strip(), m.group(2).strip()
            if name == "function":  # V3 layout: function<sep>name\n```json ... ```
                return DeepSeekV3ToolParser().extract(text)
            calls.append(ToolCall(name, args))
        if not calls:
            return text, []
        return text[: text.find(self.B)].strip() or None, calls


def _calls_from_json(obj, name_keys=("name",), arg_keys=("arguments", "parameters")) -> list:
    items = obj if isinstance(obj, list) else [obj]
    calls = []
    for d in items:
        if not isinstance(d, dict):
            continue
        if "function" in d and isinstance(d["function"], dict):
            d = d["function"]
        name = next((d[k] for k in name_keys if k in d), None)
        if not isinstance(name, str):
            continue
        args = next((d[k] for k in arg_keys if k in d), {})
        calls.append(ToolCall(name, args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)))
    return calls


def _json_values(text: str):
    """Decode consecutive JSON values in ``text`` (separated by whitespace, ``;`` or ``,``)."""
    dec, i, out = json.JSONDecoder(), 0, []
    while i < len(text):
        while i < len(text) and text[i] in " \t\r\n;,":
            i += 1
        if i >= len(text):
            break
        try:
            v, j = dec.raw_decode(text, i)
        except json.JSONDecodeError:
            break
        out.append(v)
        i = j
    return out


class MarkerJsonToolParser(ToolParser):
    """Tool calls as JSON (an object, a list, or several values) after a start marker, optionally closed by an end marker.
    Covers Mistral ``[TOOL_CALLS]``, Granite ``<|tool_call|>`` / ``<tool_call>``, Jamba and Hunyuan ``<tool_calls>…</tool_calls>``,
    Phi-4-mini ``functools``, InternLM ``<|action_start|><|plugin|>…<|action_end|>``, MiniMax line-separated objects."""

    def __init__(self, starts: tuple, end: Optional[str] = None):
        self.markers, self.end = tuple(starts), end

    def extract(self, text):
        i, m = min(((text.find(m), m) for m in self.markers if text.find(m) != -1), default=(-1, None))
        if i == -1:
            return text, []
        body = text[i + len(m):]
        if self.end and self.end in body:
            body = body[: body.find(self.end)]
        calls = []
        for v in _json_values(body):
            calls += _calls_from_json(v)
        if not calls:
            return text, []
        return text[:i].strip() or None, calls


class Llama3JsonToolParser(ToolParser):
    """Llama 3.x / 4 JSON tool calls: the whole answer is one or more ``{"name": …, "parameters": …}`` objects separated by
    ``;``, optionally after ``<|python_tag|>``."""

    markers = ("<|python_tag|>", "{")

    def extract(self, text):
        body = text.strip()
        if body.startswith("<|python_tag|>"):
            body = body[len("<|python_tag|>"):]
        if not body.lstrip().startswith(("{", "[")):
            return text, []
        calls = []
        for v in _json_values(body):
            calls += _calls_from_json(v)
        return (None, calls) if calls else (text, [])

    def content_so_far(self, text):
        t = text.lstrip()
        return "" if (not t or t.startswith(("{", "[", "<|python_tag|>")) or "<|python_tag|>".startswith(t)) else text


class PythonicToolParser(ToolParser):
    """``[get_weather(city="Paris"), f(x=1)]`` (Llama 4 pythonic, OLMo 3): parsed with ``ast``, literals only."""

    markers = ("[",)

    def extract(self, text):
        import ast
        body = text.strip()
        if not (body.startswith("[") and body.endswith("]")):
            return text, []
        try:
            tree = ast.parse(body, mode="eval")
        except SyntaxError:
            return text, []
        if not isinstance(tree.body, ast.List) or not tree.body.elts:
            return text, []
        calls = []
        for e in tree.body.elts:
            if not isinstance(e, ast.Call) or e.args:
                return text, []
            name = ast.unparse(e.func)
            try:
                args = {k.arg: ast.literal_eval(k.value) for k in e.keywords}
            except (ValueError, SyntaxError):
                return text, []
            calls.append(ToolCall(name, json.dumps(args, ensure_ascii=False)))
        return None, calls

    def content_so_far(self, text):
        return "" if text.lstrip().startswith("[") or not text.strip() else text


class KimiK2ToolParser(ToolParser):
    B = "<|tool_calls_section_begin|>"
    markers = (B,)
    _re = re.compile(r"<\|tool_call_begin\|>\s*(?:functions\.)?([\w\.\-]+?)(?::\d+)?\s*<\|tool_call_argument_begin\|>\s*(.*?)\s*<\|tool_call_end\|>", re.S)

    def extract(self, text):
        calls = [ToolCall(m.group(1), m.group(2)) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return text[: text.find(self.B)].strip() or None, calls


class Glm45ToolParser(ToolParser):
    """``<tool_call>name\n<arg_key>k</arg_key>\n<arg_value>v</arg_value>…</tool_call>``."""

    markers = ("<tool_call>",)
    _call = re.compile(r"<tool_call>\s*([^\n<]+)\s*(.*?)(?:</tool_call>|$)", re.S)
    _kv = re.compile(r"<arg_key>(.*?)</arg_key>\s*<arg_value>(.*?)</arg_value>", re.S)

    def extract(self, text):
        calls = []
        for m in self._call.finditer(text):
            args = {}
            for k, v in self._kv.findall(m.group(2)):
                v = v.strip()
                try:
                    args[k.strip()] = json.loads(v)
                except json.JSONDecodeError:
                    args[k.strip()] = v
            calls.append(ToolCall(m.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return text[: text.find("<tool_call>")].strip() or None, calls


class SeedOssToolParser(Qwen3CoderToolParser):
    markers = ("<seed:tool_call>", "<function=")


class TaggedJsonToolParser(HermesToolParser):
    """Hermes layout with other tag strings (LongCat ``<longcat_tool_call>``)."""

    def __init__(self, start: str, end: str):
        self.markers = (start,)
        self._start = start
        self._re = re.compile(re.escape(start) + r"\s*(.*?)\s*(?:" + re.escape(end) + r"|$)", re.S)

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
        return text[: text.find(self._start)].strip() or None, calls


class InvokeXmlToolParser(ToolParser):
    """MiniMax-M2 layout: ``<minimax:tool_call><invoke name="f"><parameter name="k">v</parameter></invoke></minimax:tool_call>``;
    parameter values are JSON when they parse as JSON, else strings."""

    markers = ("<minimax:tool_call>",)
    _inv = re.compile(r"<invoke name=\"?([^\">]+)\"?>(.*?)(?:</invoke>|$)", re.S)
    _par = re.compile(r"<parameter name=\"?([^\">]+)\"?>(.*?)</parameter>", re.S)

    def extract(self, text):
        calls = []
        for m in self._inv.finditer(text):
            args = {}
            for k, v in self._par.findall(m.group(2)):
                v = v.strip("\n")
                try:
                    args[k] = json.loads(v)
                except json.JSONDecodeError:
                    args[k] = v
            calls.append(ToolCall(m.group(1).strip(), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return text[: text.find(self.markers[0])].strip() or None, calls


class WrappedPythonicToolParser(PythonicToolParser):
    """LFM2 layout: a pythonic call list between ``<|tool_call_start|>`` and ``<|tool_call_end|>``; text around it is content."""

    markers = ("<|tool_call_start|>",)
    _re = re.compile(r"<\|tool_call_start\|>(.*?)(?:<\|tool_call_end\|>|$)", re.S)

    def extract(self, text):
        m = self._re.search(text)
        if m is None:
            return text, []
        _, calls = super().extract(m.group(1).strip())
        if not calls:
            return text, []
        rest = (text[: m.start()] + text[m.end():]).strip()
        return rest or None, calls

    def content_so_far(self, text):
        i = text.find(self.markers[0])
        return text if i == -1 else text[:i]


class KeyedJsonListToolParser(ToolParser):
    """Apertus layout: ``<|tools_prefix|>[{"name": {args}}, ...]<|tools_suffix|>`` — a JSON list of single-key objects."""

    markers = ("<|tools_prefix|>",)

    def extract(self, text):
        i = text.find(self.markers[0])
        if i == -1:
            return text, []
        body = text[i + len(self.markers[0]):]
        j = body.find("<|tools_suffix|>")
        body = body if j == -1 else body[:j]
        calls = []
        for v in _json_values(body):
            for d in (v if isinstance(v, list) else [v]):
                if isinstance(d, dict) and len(d) == 1:
                    (name, args), = d.items()
                    calls.append(ToolCall(str(name), args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return text[:i].strip() or None, calls


class DsmlToolParser(ToolParser):
    """DeepSeek-V3.2 / V4 layout: ``<｜DSML｜function_calls>`` (V4: ``tool_calls``) holding ``<｜DSML｜invoke name="f">`` blocks of
    ``<｜DSML｜parameter name="k" string="true|false">v</｜DSML｜parameter>``; non-string parameters are JSON."""

    def __init__(self, section: str = "function_calls"):
        self.markers = (f"<｜DSML｜{section}>",)
        self._inv = re.compile(r"<｜DSML｜invoke name=\"([^\"]+)\">(.*?)(?:</｜DSML｜invoke>|$)", re.S)
        self._par = re.compile(r"<｜DSML｜parameter name=\"([^\"]+)\"(?: string=\"(true|false)\")?>(.*?)</｜DSML｜parameter>", re.S)

    def extract(self, text):
        i = text.find(self.markers[0])
        if i == -1:
            return text, []
        calls = []
        for m in self._inv.finditer(text[i:]):
            args = {}
            for k, is_str, v in self._par.findall(m.group(2)):
                if is_str == "false":
                    try:
                        args[k] = json.loads(v)
                        continue
                    except json.JSONDecodeError:
                        pass
                args[k] = v
            calls.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return text[:i].strip() or None, calls


class CallBraceToolParser(ToolParser):
    """FunctionGemma / Gemma-4 layout: ``<start>call:name{k:v,k2:<escape>text<escape>}<end>``; values are JSON-ish literals, strings may
    be wrapped in ``<escape>`` or ``<|"|>`` tokens."""

    def __init__(self, start: str, end: str, quote: str):
        self.markers = (start,)
        self._re = re.compile(re.escape(start) + r"call:([\w\-\.]+)\{(.*?)\}" + re.escape(end), re.S)
        self._quote = quote

    def _args(self, body: str) -> dict:
        out, q = {}, self._quote
        i, n = 0, len(body)
        while i < n:
            j = body.find(":", i)
            if j == -1:
                break
            key = body[i:j].strip().strip('"')
            i = j + 1
            if body.startswith(q, i):
                k = body.find(q, i + len(q))
                k = n if k == -1 else k
                out[key] = body[i + len(q):k]
                i = body.find(",", k)
                i = n if i == -1 else i + 1
                continue
            depth, k = 0, i
            while k < n and not (body[k] == "," and depth == 0):
                depth += body[k] in "[{"
                depth -= body[k] in "]}"
                k += 1
            raw = body[i:k].strip()
            try:
                out[key] = json.loads(raw)
            except json.JSONDecodeError:
                out[key] = raw
            i = k + 1
        return out

    def extract(self, text):
        calls = [ToolCall(m.group(1), json.dumps(self._args(m.group(2)), ensure_ascii=False)) for m in self._re.finditer(text)]
        if not calls:
            return text, []
        return text[: text.find(self.markers[0])].strip() or None, calls


class GigaChatToolParser(ToolParser):
    """GigaChat-3 layout: ``function call<|role_sep|>\n{"name": ..., "arguments": {...}}`` or ``<|function_call|>{...}``."""

    markers = ("function call<|role_sep|>", "<|function_call|>")
    _re = re.compile(r"(?:function call<\|role_sep\|>\n|<\|function_call\|>)(.*)", re.S)

    def extract(self, text):
        body = text[: text.rfind("</s>")] if text.rstrip().endswith("</s>") else text
        m = self._re.search(body)
        if m is None:
            return text, []
        calls = []
        for v in _json_values(m.group(1)):
            calls += _calls_from_json(v)
        if not calls:
            return text, []
        head = re.split(r"<\|message_sep\|>|<\|function_call\|>|function call<\|role_sep\|>", body, maxsplit=1)[0]
        return head.strip() or None, calls


class SepArgKeyToolParser(Glm45ToolParser):
    """Hunyuan-V3 layout: ``<tool_calls><tool_call>name<tool_sep><arg_key>k</arg_key><arg_value>v</arg_value>…</tool_call></tool_calls>``."""

    markers = ("<tool_calls>", "<tool_call>")
    _call = re.compile(r"<tool_call>(.*?)<tool_sep>(.*?)(?:</tool_call>|$)", re.S)

    def extract(self, text):
        content, calls = super().extract(text)
        if calls and content is not None:
            i = self._first_marker(text)
            content = text[:i].strip() or None
        return content, calls


class FunctionParamXmlToolParser(ToolParser):
    """MiniCPM-5 layout: ``<function name="f"><param name="k">v</param></function>`` (values may be CDATA; JSON when they parse)."""

    markers = ("<function name=", "<function name =", "<functionname=")
    _fn = re.compile(r"<function\s*name\s*=\s*['\"]([^'\"]+)['\"][^>]*>(.*?)(?:</function>|$)", re.S)
    _par = re.compile(r"<param\s*name\s*=\s*['\"]([^'\"]+)['\"]>([\s\S]*?)</param>", re.S)

    def extract(self, text):
        vis = text.rsplit("</think>", 1)[-1] if "</think>" in text else text
        calls = []
        for m in self._fn.finditer(vis):
            args = {}
            for k, v in self._par.findall(m.group(2)):
                v = v.strip()
                if v.startswith("<![CDATA[") and v.endswith("]]>"):
                    v = v[len("<![CDATA["):-3]
                try:
                    args[k] = json.loads(v)
                except json.JSONDecodeError:
                    args[k] = v
            calls.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        i = self._first_marker(vis)
        return vis[:i].strip() or None, calls


class StepTmlToolParser(ToolParser):
    """Step-3 layout: ``<｜tool_calls_begin｜><｜tool_call_begin｜>function<｜tool_sep｜><steptml:invoke name="f"><steptml:parameter
    name="k">v</steptml:parameter></steptml:invoke><｜tool_call_end｜><｜tool_calls_end｜>``."""

    markers = ("<｜tool_calls_begin｜>",)
    _inv = re.compile(r"<steptml:invoke name=\"([^\"]+)\">(.*?)(?:</steptml:invoke>|$)", re.S)
    _par = re.compile(r"<steptml:parameter name=\"([^\"]+)\">([^<]*)</steptml:parameter>", re.S)

    def extract(self, text):
        i = text.find(self.markers[0])
        if i == -1:
            return text, []
        calls = []
        for m in self._inv.finditer(text[i:]):
            args = {}
            for k, v in self._par.findall(m.group(2)):
                try:
                    args[k] = json.loads(v)
                except json.JSONDecodeError:
                    args[k] = v
            calls.append(ToolCall(m.group(1), json.dumps(args, ensure_ascii=False)))
        if not calls:
            return text, []
        return text[:i].strip() or None, calls


class HarmonyToolParser(ToolParser):
    """GPT-OSS harmony text: a message addressed ``to=functions.NAME`` on the commentary channel is a tool call, its body the JSON
    arguments; the ``final`` channel is the content (reference: tool_parsers/openai_tool_parser.py over the harmony encoding)."""

    markers = ("<|channel|>commentary to=functions.", "to=functions.")
    _call = re.compile(r"to=functions\.([\w\-\.]+)[^<]*?(?:<\|constrain\|>\s*json\s*)?<\|message\|>(.*?)(?:<\|call\|>|<\|end\|>|<\|start\|>|$)", re.S)
    _final = re.compile(r"<\|channel\|>final<\|message\|>(.*?)(?:<\|end\|>|<\|return\|>|$)", re.S)

    def extract(self, text):
        calls = [ToolCall(m.group(1), m.group(2).strip()) for m in self._call.finditer(text)]
        if not calls:
            return text, []
        f = self._final.search(text)
        return (f.group(1).strip() or None) if f else None, calls


class CohereActionToolParser(ToolParser):
    """Command-R layout: ``<|START_ACTION|>[{"tool_call_id": "0", "tool_name": "f", "parameters": {...}}]<|END_ACTION|>`` (the reference
    drives an external filter library for this format; the wire format itself is plain JSON between the two tokens)."""

    markers = ("<|START_ACTION|>",)

    def extract(self, text):
        i = text.find(self.markers[0])
        if i == -1:
            return text, []
        body = text[i + len(self.markers[0]):]
        j = body.find("<|END_ACTION|>")
        body = body if j == -1 else body[:j]
        calls = []
        for v in _json_values(body):
            calls += _calls_from_json(v, name_keys=("tool_name", "name"))
        if not calls:
            return text, []
        head = text[:i]
        m = re.search(r"<\|START_RESPONSE\|>(.*?)(?:<\|END_RESPONSE\|>|$)", head, re.S)
        return ((m.group(1) if m else head).strip() or None), calls


TOOL_PARSERS = {
    "longcat": lambda: TaggedJsonToolParser("<longcat_tool_call>", "</longcat_tool_call>"), "ernie45": HermesToolParser,
    "minimax_m2": InvokeXmlToolParser, "lfm2": WrappedPythonicToolParser, "glm4_moe": Glm45ToolParser,
    "hermes": HermesToolParser, "qwen3_coder": Qwen3CoderToolParser, "qwen3_xml": Qwen3CoderToolParser,
    "deepseek_v3": DeepSeekV3ToolParser, "deepseek_v31": DeepSeekV31ToolParser,
    "llama3_json": Llama3JsonToolParser, "llama4_json": Llama3JsonToolParser, "pythonic": PythonicToolParser, "llama4_pythonic": PythonicToolParser,
    "olmo3": PythonicToolParser, "kimi_k2": KimiK2ToolParser, "glm45": Glm45ToolParser, "glm47": Glm45ToolParser, "seed_oss": SeedOssToolParser,
    "mistral": lambda: MarkerJsonToolParser(("[TOOL_CALLS]",)),
    "granite": lambda: MarkerJsonToolParser(("<|tool_call|>", "<tool_call>")),
    "granite-20b-fc": lambda: MarkerJsonToolParser(("<function_call>",)),
    "jamba": lambda: MarkerJsonToolParser(("<tool_calls>",), "</tool_calls>"),
    "hunyuan_a13b": lambda: MarkerJsonToolParser(("<tool_calls>",), "</tool_calls>"),
    "minimax": lambda: MarkerJsonToolParser(("<tool_calls>",), "</tool_calls>"),
    "phi4_mini_json": lambda: MarkerJsonToolParser(("functools",)),
    "internlm": lambda: MarkerJsonToolParser(("<|action_start|><|plugin|>",), "<|action_end|>"),
    "xlam": lambda: MarkerJsonToolParser(("```json", "[TOOL_CALLS]", "<tool_call>", "[")),
    "apertus": KeyedJsonListToolParser, "deepseek_v32": DsmlToolParser, "deepseek_v4": lambda: DsmlToolParser("tool_calls"),
    "functiongemma": lambda: CallBraceToolParser("<start_function_call>", "<end_function_call>", "<escape>"),
    "gemma4": lambda: CallBraceToolParser("<|tool_call>", "<tool_call|>", '<|"|>'),
    "gigachat3": GigaChatToolParser, "granite4": HermesToolParser, "hy_v3": SepArgKeyToolParser, "minicpm5xml": FunctionParamXmlToolParser,
    "openai": HarmonyToolParser, "poolside_v1": Glm45ToolParser, "step3": StepTmlToolParser, "step3p5": Qwen3CoderToolParser,
    "cohere_command": CohereActionToolParser, "internlm2": lambda: MarkerJsonToolParser(("<|action_start|><|plugin|>",), "<|action_end|>"),
    "phi4mini": lambda: MarkerJsonToolParser(("functools",)), "glm47_moe": Glm45ToolParser, "llama": Llama3JsonToolParser,
    "qwen3coder": Qwen3CoderToolParser, "qwen3xml": Qwen3CoderToolParser,
}


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


class ParserManager:
    """One object for a served model's output: splits the reasoning section off first, then looks for tool calls in the remaining
    content (reference: parser/abstract_parser.py, parser/parser_manager.py — the combined reasoning + tool parser)."""

    def __init__(self, reasoning_parser: Optional[str] = None, tool_parser: Optional[str] = None):
        self.reasoning = get_reasoning_parser(reasoning_parser)
        self.tools = get_tool_parser(tool_parser)

    def parse(self, text: str) -> tuple[Optional[str], Optional[str], list]:
        """(reasoning, content, tool calls) of a complete response."""
        reasoning, content = self.reasoning.extract(text) if self.reasoning is not None else (None, text or None)
        calls: list = []
        if self.tools is not None and content:
            content, calls = self.tools.extract(content)
        return reasoning, content, calls
