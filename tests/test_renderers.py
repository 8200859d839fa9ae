"""Chat renderers and the tekken tokenizer (CPU)."""
import base64
import json

import pytest

from onecat_vllm.engine import renderers as R


def _tekken(tmp_path, version="v7"):
    # 256 single bytes, then a few merges by rank: "he", "ll", "hell", "hello", " w", "or", " wor"
    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor"]
    special = ["<unk>", "<s>", "</s>", "[INST]", "[/INST]", "[SYSTEM_PROMPT]", "[/SYSTEM_PROMPT]", "[TOOL_CALLS]"]
    d = {"config": {"pattern": r"[^\r\n\p{L}\p{N}]?[\p{L}]+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+",
                    "default_vocab_size": len(toks) + len(special), "default_num_special_tokens": len(special), "version": version},
         "vocab": [{"rank": i, "token_bytes": base64.b64encode(b).decode(), "token_str": None} for i, b in enumerate(toks)],
         "special_tokens": [{"rank": i, "token_str": s, "is_control": True} for i, s in enumerate(special)]}
    p = tmp_path / "tekken.json"
    p.write_text(json.dumps(d))
    return str(tmp_path)


def test_tekken_merges_by_rank_and_round_trips(tmp_path):
    tok = R.load_tokenizer(_tekken(tmp_path))
    assert isinstance(tok, R.TekkenTokenizer) and tok.n_special == 8
    ids = tok.encode("hello world", add_special_tokens=True)
    # "hello" is one token (rank 259), " world" = " wor" (262) + "l" + "d"
    assert ids == [1, 259 + 8, 262 + 8, ord("l") + 8, ord("d") + 8]
    assert tok.decode(ids) == "hello world"
    assert tok.decode(tok.encode("héllo ✓ 12\n", add_special_tokens=False)) == "héllo ✓ 12\n"
    sp = tok.encode("[INST]hello[/INST]", add_special_tokens=False)
    assert sp == [3, 259 + 8, 4] and tok.decode(sp, skip_special_tokens=False) == "[INST]hello[/INST]"
    assert tok.encode("[INST]", add_special_tokens=False, parse_special=False)[0] >= 8     # user text cannot forge control tokens


def test_mistral_rendering_v3_and_v7(tmp_path):
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"},
            {"role": "user", "content": "again"}]
    assert R.MistralRenderer("v3").render(msgs) == "<s>[INST]be brief\n\nhi[/INST]yo</s>[INST]again[/INST]"
    assert R.MistralRenderer("v7").render(msgs) == "<s>[SYSTEM_PROMPT]be brief[/SYSTEM_PROMPT][INST]hi[/INST]yo</s>[INST]again[/INST]"
    tools = [{"type": "function", "function": {"name": "f", "parameters": {}}}]
    calls = [{"id": "abc123xyz", "type": "function", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]
    t = R.MistralRenderer("v3").render([{"role": "user", "content": "q"}, {"role": "assistant", "tool_calls": calls},
                                        {"role": "tool", "content": "42", "tool_call_id": "abc123xyz"}, {"role": "user", "content": "so?"}], tools=tools)
    assert "[TOOL_CALLS][{\"name\": \"f\", \"arguments\": {\"a\": 1}, \"id\": \"abc123xyz\"}]</s>" in t
    assert "[TOOL_RESULTS]{\"content\": \"42\", \"call_id\": \"abc123xyz\"}[/TOOL_RESULTS]" in t
    assert t.index("[AVAILABLE_TOOLS]") > t.index("[/TOOL_RESULTS]")       # tools are announced before the last user turn
    tok = R.load_tokenizer(_tekken(tmp_path))
    assert tok.apply_chat_template([{"role": "user", "content": "hello"}], tokenize=True) == [1, 3, 259 + 8, 4]


def test_deepseek_v32_rendering():
    r = R.DeepseekV32Renderer()
    msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": "a"}, {"role": "assistant", "content": "b", "reasoning": "old thoughts"},
            {"role": "user", "content": "c"}]
    chat = r.render(msgs, thinking=False)
    assert chat == "<｜begin▁of▁sentence｜>sys<｜User｜>a<｜Assistant｜></think>b<｜end▁of▁sentence｜><｜User｜>c<｜Assistant｜></think>"
    think = r.render(msgs, thinking=True)
    assert think.endswith("<｜User｜>c<｜Assistant｜><think>") and "old thoughts" not in think
    calls = [{"type": "function", "function": {"name": "get", "arguments": {"city": "Oslo", "days": 3}}}]
    tools = [{"type": "function", "function": {"name": "get", "parameters": {"type": "object"}}}]
    t = r.render([{"role": "user", "content": "w?"}, {"role": "assistant", "content": "", "tool_calls": calls, "reasoning": "need the tool"},
                  {"role": "tool", "content": "sunny"}], tools=tools, thinking=True)
    assert "## Tools" in t and '{"name": "get"' in t
    assert 'need the tool</think>\n\n<｜DSML｜function_calls>\n<｜DSML｜invoke name="get">' in t
    assert '<｜DSML｜parameter name="city" string="true">Oslo</｜DSML｜parameter>' in t and 'name="days" string="false">3<' in t
    assert t.endswith("\n\n<function_results>\n<result>sunny</result>\n</function_results>\n\n<think>")
    with pytest.raises(ValueError):
        r.render([{"role": "tool", "content": "x"}])


def test_registry_picks_by_architecture_and_falls_back_to_the_template():
    class Tok:
        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
            return "TEMPLATE:" + messages[-1]["content"] + ("|tools" if kw.get("tools") else "")
    m = [{"role": "user", "content": "x"}]
    assert R.render_chat(Tok(), m, architecture="Qwen3ForCausalLM", tools=[{"a": 1}]) == "TEMPLATE:x|tools"
    assert R.render_chat(Tok(), m, architecture="DeepseekV32ForCausalLM").startswith("<｜begin▁of▁sentence｜><｜User｜>x")
    R.register_renderer("shout", lambda: type("S", (), {"render": lambda self, msgs, **kw: msgs[-1]["content"].upper()})(), ("ShoutLM",))
    assert R.render_chat(Tok(), m, architecture="ShoutLM") == "X"
