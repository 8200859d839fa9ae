"""Chat renderers for model families whose prompt format is not a Jinja template in the checkpoint, and the tokenizer for
Mistral's ``tekken.json`` files.

``render_chat(tokenizer, messages, ...)`` is what the servers call: a renderer registered for the model family wins, otherwise the
tokenizer's own ``apply_chat_template``.

* ``MistralRenderer``    ``<s>[INST] user [/INST] assistant</s>`` turns; the system prompt goes into ``[SYSTEM_PROMPT]…`` (format
                         v7 and later) or is prepended to the first user turn; tools in ``[AVAILABLE_TOOLS]``, calls in
                         ``[TOOL_CALLS]``, results in ``[TOOL_RESULTS]``.
* ``DeepseekV32Renderer`` ``<｜User｜>…<｜Assistant｜>`` turns; the last user turn is followed by ``<think>`` in thinking mode and by
                         ``</think>`` otherwise; tool schemas in the system turn, calls as ``｜DSML｜`` blocks, results in
                         ``<function_results>``; reasoning of turns before the last user turn is dropped.
* ``TekkenTokenizer``    byte-pair encoding by rank over regex-split pieces (the tiktoken scheme) with the special tokens in front
                         of the vocabulary.
(reference: vllm/renderers/registry.py, renderers/mistral.py, renderers/deepseek_v32.py; tokenizers/mistral.py,
tokenizers/deepseek_v32_encoding.py:154 ``render_message`` / :315 ``encode_messages``)"""
from __future__ import annotations

import base64
import json
import os
from typing import Any, Callable, Optional

# ------------------------------------------------------------------------------------------------------------------------- tekken


class TekkenTokenizer:
    """``tekken.json``: ``config`` (split pattern, vocabulary size, number of special tokens), ``vocab`` (token bytes by rank) and
    ``special_tokens``. Token id = rank + number of special tokens; special tokens take the ids below that."""

    chat_template = None

    def __init__(self, path: str):
        import regex
        with open(path) as f:
            d = json.load(f)
        cfg = d["config"]
        self.n_special = int(cfg.get("default_num_special_tokens", len(d.get("special_tokens", []))))
        self.vocab_size = int(cfg.get("default_vocab_size", len(d["vocab"]) + self.n_special))
        n_regular = self.vocab_size - self.n_special
        self._pat = regex.compile(cfg["pattern"])
        self._bytes = [base64.b64decode(v["token_bytes"]) for v in d["vocab"][:n_regular]]
        self._rank = {b: i for i, b in enumerate(self._bytes)}
        self.special = {s["token_str"]: int(s["rank"]) for s in d.get("special_tokens", [])}
        self._special_by_id = {i: s for s, i in self.special.items()}
        self.bos_token_id = self.special.get("<s>", 1)
        self.eos_token_id = self.special.get("</s>", 2)
        self.version = str(cfg.get("version", "v3"))
        self._special_pat = regex.compile("|".join(regex.escape(s) for s in sorted(self.special, key=len, reverse=True))) if self.special else None

    def _bpe(self, piece: bytes) -> list[int]:
        if piece in self._rank:
            return [self._rank[piece]]
        parts = [piece[i:i + 1] for i in range(len(piece))]
        while len(parts) > 1:
            best, at = None, -1
            for i in range(len(parts) - 1):
                r = self._rank.get(parts[i] + parts[i + 1])
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            parts[at:at + 2] = [parts[at] + parts[at + 1]]
        return [self._rank[p] for p in parts]

    def _encode_plain(self, text: str) -> list[int]:
        out: list[int] = []
        for m in self._pat.finditer(text):
            out += [r + self.n_special for r in self._bpe(m.group(0).encode("utf-8"))]
        return out

    def encode(self, text: str, add_special_tokens: bool = True, parse_special: bool = True) -> list[int]:
        ids = [self.bos_token_id] if add_special_tokens else []
        if not parse_special or self._special_pat is None:
            return ids + self._encode_plain(text)
        pos = 0
        for m in self._special_pat.finditer(text):
            ids += self._encode_plain(text[pos:m.start()])
            ids.append(self.special[m.group(0)])
            pos = m.end()
        return ids + self._encode_plain(text[pos:])

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        buf = bytearray()
        for i in ids:
            if i < self.n_special:
                if not skip_special_tokens and i in self._special_by_id:
                    buf += self._special_by_id[i].encode("utf-8")
            elif i - self.n_special < len(self._bytes):
                buf += self._bytes[i - self.n_special]
        return buf.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize: bool = False, add_generation_prompt: bool = True, tools=None, **kw):
        text = MistralRenderer(self.version).render(messages, tools=tools, add_generation_prompt=add_generation_prompt)
        return self.encode(text, add_special_tokens=False) if tokenize else text


# ---------------------------------------------------------------------------------------------------------------------- renderers


def _text(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    return "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type", "text") == "text")


class MistralRenderer:
    name = "mistral"

    def __init__(self, version: str = "v3"):
        v = version.lstrip("v")
        self.major = int(v.split(".")[0]) if v and v[0].isdigit() else 3

    def render(self, messages, tools=None, add_generation_prompt: bool = True, **kw) -> str:
        system = "\n\n".join(_text(m["content"]) for m in messages if m["role"] == "system")
        turns = [m for m in messages if m["role"] != "system"]
        last_user = max((i for i, m in enumerate(turns) if m["role"] == "user"), default=-1)
        out = "<s>"
        if system and self.major >= 7:
            out += f"[SYSTEM_PROMPT]{system}[/SYSTEM_PROMPT]"
        first_user = True
        for i, m in enumerate(turns):
            role = m["role"]
            if role == "user":
                if tools and i == last_user:
                    out += "[AVAILABLE_TOOLS]" + json.dumps(tools, ensure_ascii=False) + "[/AVAILABLE_TOOLS]"
                body = _text(m["content"])
                if system and self.major < 7 and first_user:
                    body = system + "\n\n" + body
                first_user = False
                out += f"[INST]{body}[/INST]"
            elif role == "assistant":
                calls = m.get("tool_calls")
                if calls:
                    payload = [{"name": c["function"]["name"],
                                "arguments": json.loads(c["function"]["arguments"]) if isinstance(c["function"]["arguments"], str) else c["function"]["arguments"],
                                **({"id": c["id"]} if c.get("id") else {})} for c in calls]
                    out += "[TOOL_CALLS]" + json.dumps(payload, ensure_ascii=False) + "</s>"
                else:
                    out += _text(m["content"]) + "</s>"
            elif role == "tool":
                out += "[TOOL_RESULTS]" + json.dumps({"content": _text(m["content"]), **({"call_id": m["tool_call_id"]} if m.get("tool_call_id") else {})},
                                                     ensure_ascii=False) + "[/TOOL_RESULTS]"
            else:
                raise ValueError(f"unknown role {role!r}")
        if not add_generation_prompt and turns and turns[-1]["role"] == "assistant" and out.endswith("</s>"):
            out = out[: -len("</s>")]   # continue the final assistant message
        return out


class DeepseekV32Renderer:
    name = "deepseek_v32"
    BOS, EOS = "<｜begin▁of▁sentence｜>", "<｜end▁of▁sentence｜>"
    USER, ASSISTANT = "<｜User｜>", "<｜Assistant｜>"
    THINK, END_THINK = "<think>", "</think>"
    DSML = "｜DSML｜"

    def _tools_block(self, tools) -> str:
        schemas = "\n".join(json.dumps(t.get("function", t), ensure_ascii=False) for t in tools)
        d = self.DSML
        return ("## Tools\nYou have access to a set of tools you can use to answer the user's question.\n"
                f"You can invoke functions by writing a \"<{d}function_calls>\" block like the following as part of your reply to the user:\n"
                f"<{d}function_calls>\n<{d}invoke name=\"$FUNCTION_NAME\">\n"
                f"<{d}parameter name=\"$PARAMETER_NAME\" string=\"true|false\">$PARAMETER_VALUE</{d}parameter>\n...\n</{d}invoke>\n</{d}function_calls>\n"
                "String and scalar parameters should be specified as is without any escaping or quotes, while lists and objects should use JSON format. "
                "The \"string\" attribute should be set to \"true\" for string type parameters and \"false\" for other types.\n"
                "Here are the functions available in JSONSchema format:\n<functions>\n" + schemas + "\n</functions>\n")

    def _call_block(self, calls) -> str:
        d, inv = self.DSML, []
        for c in calls:
            fn = c.get("function", c)
            args = fn["arguments"]
            args = json.loads(args) if isinstance(args, str) else args
            params = "\n".join(
                f"<{d}parameter name=\"{k}\" string=\"{'true' if isinstance(v, str) else 'false'}\">{v if isinstance(v, str) else json.dumps(v, ensure_ascii=False)}</{d}parameter>"
                for k, v in args.items())
            inv.append(f"<{d}invoke name=\"{fn['name']}\">\n{params}\n</{d}invoke>")
        return f"\n\n<{d}function_calls>\n" + "\n".join(inv) + f"\n</{d}function_calls>"

    def render(self, messages, tools=None, add_generation_prompt: bool = True, thinking: bool = False, **kw) -> str:
        msgs = [dict(m) for m in messages]
        if tools:
            if msgs and msgs[0]["role"] == "system":
                msgs[0]["tools"] = tools
            else:
                msgs.insert(0, {"role": "system", "content": "", "tools": tools})
        last_user = max((i for i, m in enumerate(msgs) if m["role"] in ("user", "developer")), default=-1)
        out = self.BOS
        for i, m in enumerate(msgs):
            role = m["role"]
            if role == "system":
                out += _text(m.get("content"))
                if m.get("tools"):
                    out += "\n\n" + self._tools_block(m["tools"])
            elif role in ("user", "developer"):
                out += self.USER + _text(m.get("content")) + self.ASSISTANT
                out += self.THINK if (thinking and i == last_user) else self.END_THINK
            elif role == "assistant":
                calls = m.get("tool_calls")
                reasoning = m.get("reasoning") or m.get("reasoning_content") or ""
                head = (reasoning + self.END_THINK) if (thinking and i > last_user) else ""   # earlier turns lose their reasoning
                if m.get("prefix") and not calls:
                    out += _text(m.get("content"))
                else:
                    out += head + _text(m.get("content")) + (self._call_block(calls) if calls else "") + self.EOS
            elif role == "tool":
                j = i - 1
                while j >= 0 and msgs[j]["role"] == "tool":
                    j -= 1
                if j < 0 or msgs[j]["role"] != "assistant" or not msgs[j].get("tool_calls"):
                    raise ValueError("a tool message needs an assistant message with tool_calls before it")
                order, total = i - j, len(msgs[j]["tool_calls"])
                if order == 1:
                    out += "\n\n<function_results>"
                out += f"\n<result>{_text(m.get('content'))}</result>"
                if order == total:
                    out += "\n</function_results>\n\n" + (self.THINK if (thinking and i >= last_user) else self.END_THINK)
            else:
                raise ValueError(f"unknown role {role!r}")
        return out


RENDERERS: dict[str, Callable[[], Any]] = {"mistral": MistralRenderer, "deepseek_v32": DeepseekV32Renderer}
_BY_ARCH = {"DeepseekV32ForCausalLM": "deepseek_v32", "MistralForCausalLM": None, "MinistralForCausalLM": None}


def register_renderer(name: str, factory: Callable[[], Any], architectures: tuple = ()) -> None:
    RENDERERS[name] = factory
    for a in architectures:
        _BY_ARCH[a] = name


def renderer_for(architecture: Optional[str], tokenizer=None, override: Optional[str] = None):
    """The renderer a chat request goes through, or None for the tokenizer's own chat template."""
    name = override or _BY_ARCH.get(architecture or "")
    if name is None and isinstance(tokenizer, TekkenTokenizer):
        return MistralRenderer(tokenizer.version)
    return RENDERERS[name]() if name else None


def render_chat(tokenizer, messages, architecture: Optional[str] = None, renderer: Optional[str] = None, tools=None,
                add_generation_prompt: bool = True, **kw) -> str:
    r = renderer_for(architecture, tokenizer, renderer)
    if r is not None:
        return r.render(messages, tools=tools, add_generation_prompt=add_generation_prompt, **kw)
    extra = {"tools": tools} if tools else {}
    return tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=add_generation_prompt, **extra, **kw)


def load_tokenizer(path: str, mode: str = "auto"):
    """``mode``: auto | hf | mistral | byte. ``auto`` takes ``tekken.json`` when the directory has one and no HF tokenizer files."""
    if mode == "byte" or path == "byte":
        from onecat_vllm.engine.tokenizer import ByteTokenizer
        return ByteTokenizer()
    if os.path.isfile(path) and path.endswith(".gguf"):  # the tokenizer embedded in a GGUF file, rebuilt by transformers
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(os.path.dirname(path) or ".", gguf_file=os.path.basename(path))
    tek = os.path.join(path, "tekken.json") if os.path.isdir(path) else (path if path.endswith("tekken.json") else None)
    has_hf = os.path.isdir(path) and any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json", "tokenizer.model"))
    if tek and os.path.exists(tek) and (mode == "mistral" or (mode == "auto" and not has_hf)):
        return TekkenTokenizer(tek)
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(path)
