"""Tokenizer, chat templates and the OpenAI wire protocol (reference tests: tests/unit/tokenizer_test.cpp,
chat_template_test.cpp, harmony_template_test.cpp, openai_proto_test.cpp)."""
import json

import pytest

from machx_inference_engine_b200.formats.synth import gpt2_byte_map
from machx_inference_engine_b200.server import proto
from machx_inference_engine_b200.tokenizer import templates as T
from machx_inference_engine_b200.tokenizer.templates import ChatTurn
from machx_inference_engine_b200.tokenizer.tokenizer import IncrementalDetokenizer, Tokenizer, utf8_safe_prefix


def _bpe(pre="qwen2", extra_merges=(), specials=("<|im_start|>", "<|im_end|>", "<tool_call>")):
    bm = gpt2_byte_map()
    enc = lambda s: "".join(bm[b] for b in s.encode())
    tokens, merges = list(bm), []
    for a, b in [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), (" ", "w"), ("1", "2"), ("12", "3")] + list(extra_merges):
        a, b = enc(a), enc(b)
        merges.append(f"{a} {b}")
        tokens.append(a + b)
    types = [1] * len(tokens) + [3] * len(specials)
    tokens += list(specials)
    return Tokenizer(tokens, merges, types, model="gpt2", pre=pre, eos_id=len(tokens) - 2), tokens


def test_bpe_merges_specials_and_roundtrip():
    tok, tokens = _bpe()
    ids = tok.encode("hello world")
    assert tokens[ids[0]] == "hello" and tok.decode(ids) == "hello world"
    s = "<|im_start|>user\nhello<|im_end|>"
    ids = tok.encode(s, allow_special=True)
    assert ids[0] == tok.find_token("<|im_start|>") and ids[-1] == tok.find_token("<|im_end|>")
    assert tok.decode(ids) == s and tok.decode(ids, skip_special=True) == "user\nhello"
    assert tok.decode(ids, skip_special=True, keep_special=[tok.find_token("<|im_end|>")]) == "user\nhello<|im_end|>"
    plain = tok.encode(s, allow_special=False)              # specials spelled out as ordinary text
    assert tok.find_token("<|im_start|>") not in plain and tok.decode(plain) == s
    for text in ["", "a", "naïve café ☕ 日本語 🙂", "tabs\tand\nnewlines  double  spaces", "x" * 300]:
        assert tok.decode(tok.encode(text)) == text
    assert tok.is_special(tok.find_token("<tool_call>")) and not tok.is_special(ids[1]) and tok.find_token("nope") == -1


def test_pretokenizer_families_split_digits_differently():
    q, qt = _bpe("qwen2")
    l, lt = _bpe("llama-bpe")
    # qwen2 splits digits one by one (no merge can join them); llama-3 keeps runs of up to three digits together
    assert [qt[i] for i in q.encode("123")] == ["1", "2", "3"]
    assert [lt[i] for i in l.encode("123")] == ["123"]
    assert l.decode(l.encode("12345 + 6")) == "12345 + 6"


def test_spm_score_merges_and_byte_fallback():
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁", "h", "e", "l", "o", "he", "ll", "hell", "hello", "▁hello", "▁w"]
    scores = [0.0] * 259 + [-1.0, -5, -5, -5, -5, -2.0, -2.5, -1.5, -1.0, -0.5, -3.0]
    types = [2, 3, 3] + [6] * 256 + [1] * 11
    tok = Tokenizer(pieces, (), types, scores, model="llama", bos_id=1, eos_id=2)
    ids = tok.encode("hello")
    assert ids[0] == 1 and [pieces[i] for i in ids[1:]] == ["▁hello"]
    assert tok.decode(ids[1:]) == " hello" or tok.decode(ids[1:]) == "hello"
    z = tok.encode("hello z", add_bos=False)                 # 'z' is not a piece: byte fallback
    assert pieces[z[-1]] == "<0x7A>" and tok.decode(z).endswith("z")


def test_incremental_detokenizer_never_splits_utf8():
    tok, _ = _bpe()
    text = "héllo 🙂 日本"
    ids = tok.encode(text)
    d = IncrementalDetokenizer(tok)
    out = ""
    for i in ids:
        piece = d.push(i)
        piece.encode("utf-8")                                # every emitted piece is valid on its own
        assert "�" not in piece
        out += piece
    assert out + d.flush() == text
    assert utf8_safe_prefix("🙂".encode()[:2]) == 0 and utf8_safe_prefix(b"ab\xc3") == 2 and utf8_safe_prefix("é".encode()) == 2


# ---------------------------------------------------------------- templates
U, A, S = (lambda c: ChatTurn("user", c)), (lambda c: ChatTurn("assistant", c)), (lambda c: ChatTurn("system", c))


def test_chatml_thinking_tools_and_tool_responses():
    assert T.chatml([S("be brief"), U("hi")]) == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n<think>\n"
    assert T.chatml([U("hi")], enable_thinking=False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert T.chatml([U("hi")], model_has_think=False).endswith("<|im_start|>assistant\n")
    assert T.chatml([U("hi")], add_generation_prompt=False) == "<|im_start|>user\nhi<|im_end|>\n"
    tools = json.dumps([{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {}}}}])
    s = T.chatml([S("sys"), U("weather?"), A('<tool_call>\n{"name": "get_weather", "arguments": {}}\n</tool_call>'),
                  ChatTurn("tool", "sunny"), ChatTurn("tool", "22C")], tools_json=tools)
    assert s.startswith("<|im_start|>system\nsys\n\n# Tools\n\nYou may call one or more functions")
    assert '<tools>\n{"type": "function", "function": {"name": "get_weather"' in s
    # consecutive tool results share ONE user turn
    assert "<|im_start|>user\n<tool_response>\nsunny\n</tool_response>\n<tool_response>\n22C\n</tool_response><|im_end|>\n" in s


def test_other_families_golden_strings():
    turns = [S("sys"), U("q1"), A("a1"), U("q2")]
    assert T.llama3(turns) == ("<|start_header_id|>system<|end_header_id|>\n\nsys<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nq1<|eot_id|>"
                               "<|start_header_id|>assistant<|end_header_id|>\n\na1<|eot_id|><|start_header_id|>user<|end_header_id|>\n\nq2<|eot_id|>"
                               "<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert T.mistral(turns) == "[INST] sys\n\nq1 [/INST] a1</s>[INST] q2 [/INST]"
    assert T.mistral(turns, system_prompt_block=True).startswith("[INST] [SYSTEM_PROMPT]sys[/SYSTEM_PROMPT]\n\nq1 [/INST]")
    assert T.deepseek(turns) == "sys<｜User｜>q1<｜Assistant｜>a1<｜end▁of▁sentence｜><｜User｜>q2<｜Assistant｜><think>\n"
    assert T.granite([U("q")]) == "<|start_of_role|>user<|end_of_role|>q<|end_of_text|>\n<|start_of_role|>assistant<|end_of_role|>"
    assert T.gemma([U("q"), A("a")], add_generation_prompt=False) == "<|turn>user\nq<turn|>\n<|turn>model\na<turn|>\n"
    with pytest.raises(ValueError):
        T.render("llama3", [U("q")], tools_json="[{}]")
    assert T.render("auto", [U("q")]) == T.chatml([U("q")])


def test_harmony_render_and_postprocess():
    tools = json.dumps([{"type": "function", "function": {"name": "get_weather", "description": "Weather for a city", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}, "unit": {"enum": ["c", "f"]}, "days": {"type": "integer"},
                                         "tags": {"type": "array", "items": {"type": "string"}}}, "required": ["city"]}}},
                        {"type": "function", "function": {"name": "ping"}}])
    s = T.harmony([S("be terse"), U("weather in Oslo?"), A('<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'),
                   ChatTurn("tool", '{"t": 3}')], reasoning_effort="high", tools_json=tools, today="2025-01-02")
    assert s.startswith("<|start|>system<|message|>You are ChatGPT, a large language model trained by OpenAI.\nKnowledge cutoff: 2024-06\nCurrent date: 2025-01-02\n\nReasoning: high\n\n")
    assert "Calls to these tools must go to the commentary channel.<|end|>" in s
    assert "<|start|>developer<|message|># Instructions\n\nbe terse\n\n# Tools\n\n## functions\n\nnamespace functions {\n\n// Weather for a city\n" in s
    assert 'type get_weather = (_: { city: string, unit?: "c" | "f", days?: number, tags?: string[] }) => any;' in s
    assert "type ping = () => any;" in s and "} // namespace functions" in s
    assert '<|start|>assistant<|channel|>commentary to=functions.get_weather <|constrain|>json<|message|>{"city":"Oslo"}<|call|>' in s
    assert '<|start|>functions.get_weather to=assistant<|channel|>commentary<|message|>{"t": 3}<|end|>' in s
    assert s.endswith("<|start|>assistant")
    assert T.harmony([U("q"), A("final answer")], add_generation_prompt=False, today="2025-01-02").endswith("<|start|>assistant<|channel|>final<|message|>final answer<|end|>")
    out = T.harmony_postprocess('<|channel|>analysis<|message|>thinking...<|end|><|start|>assistant<|channel|>final<|message|>It is 3C.<|return|>')
    assert out == "It is 3C."
    call = T.harmony_postprocess('<|channel|>commentary to=functions.get_weather <|constrain|>json<|message|>{"city":"Oslo"}<|call|>')
    assert call == '<tool_call>\n{"name": "get_weather", "arguments": {"city":"Oslo"}}\n</tool_call>'
    assert T.schema_to_ts({"type": "object", "properties": {"a": {"type": "boolean"}}}) == "{ a?: boolean }" and T.schema_to_ts(None) == "any"


# ---------------------------------------------------------------- OpenAI protocol
def test_parse_chat_request_fields_and_validation():
    body = {"model": "m", "messages": [{"role": "developer", "content": "d"},
                                        {"role": "user", "content": [{"type": "text", "text": "part1 "}, {"type": "image_url"}, {"type": "text", "text": "part2"}]},
                                        {"role": "assistant", "content": None, "tool_calls": [{"id": "x", "type": "function", "function": {"name": "f", "arguments": "{\"a\": 1}"}}]},
                                        {"role": "tool", "content": "42"}],
            "temperature": 0, "top_p": 0.5, "top_k": 7, "min_p": 0.1, "repeat_penalty": 1.2, "max_completion_tokens": 33, "seed": 9, "stream": True,
            "stream_options": {"include_usage": False}, "chat_template_kwargs": {"enable_thinking": False},
            "tools": [{"type": "function", "function": {"name": "f"}}]}
    r = proto.parse_chat_request(json.dumps(body))
    assert [t.role for t in r.turns] == ["system", "user", "assistant", "tool"] and r.turns[1].content == "part1 part2"
    assert r.turns[2].content == '<tool_call>\n{"name": "f", "arguments": {"a": 1}}\n</tool_call>'
    assert (r.temperature, r.top_p, r.top_k, r.min_p, r.repetition_penalty, r.max_tokens, r.seed) == (0.0, 0.5, 7, 0.1, 1.2, 33, 9)
    assert r.stream and not r.include_usage and not r.enable_thinking and json.loads(r.tools_json)[0]["function"]["name"] == "f"
    assert proto.parse_chat_request({"messages": [{"role": "user", "content": "x"}]}).max_tokens == 0      # omitted = until the context is full
    for bad in ["not json", "[]", {}, {"messages": []}, {"messages": [{"role": "alien", "content": "x"}]}, {"messages": [{"content": "x"}]},
                {"messages": [{"role": "user", "content": "x"}], "temperature": "hot"}, {"messages": [{"role": "user", "content": "x"}], "top_p": 3},
                {"messages": [{"role": "user", "content": "x"}], "tools": [{"function": {}}]}, {"messages": [{"role": "user", "content": {"a": 1}}]}]:
        with pytest.raises(proto.BadRequest):
            proto.parse_chat_request(bad if isinstance(bad, str) else json.dumps(bad))


def test_tool_call_extraction_strict_and_lenient():
    text = 'Let me check.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>'
    rest, calls = proto.extract_tool_calls(text)
    assert rest == "Let me check." and calls[0]["function"] == {"name": "get_weather", "arguments": '{"city": "Oslo"}'} and calls[0]["id"].startswith("call_")
    _, calls = proto.extract_tool_calls('<tool_call>{"name": "a", "arguments": {}}</tool_call> and <tool_call>{"name": "b", "arguments": "{\\"x\\":1}"}</tool_call>')
    assert [c["function"]["name"] for c in calls] == ["a", "b"] and calls[1]["function"]["arguments"] == '{"x":1}'
    # lenient: unquoted name, missing closing brace and closing tag
    _, calls = proto.extract_tool_calls('<tool_call>\n{name: get_weather, "arguments": {"city": "Oslo"}\n')
    assert calls and calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Oslo"}
    rest, calls = proto.extract_tool_calls("<tool_call>garbage</tool_call> tail")
    assert calls == [] and "garbage" in rest
    resp = proto.chat_completion_json("id1", "m", text, "stop", 10, 5, cached_tokens=4)
    ch = resp["choices"][0]
    assert ch["finish_reason"] == "tool_calls" and ch["message"]["tool_calls"][0]["function"]["name"] == "get_weather"
    assert resp["usage"] == {"prompt_tokens": 10, "completion_tokens": 5, "total_tokens": 15, "prompt_tokens_details": {"cached_tokens": 4}}
    plain = proto.chat_completion_json("id2", "m", "hello", "length", 1, 1)
    assert plain["choices"][0]["message"] == {"role": "assistant", "content": "hello"} and plain["choices"][0]["finish_reason"] == "length"


def test_sse_frames_and_stream_holdback():
    fr = proto.chunk_text("c", "m", "héllo")
    assert fr.startswith(b"data: ") and fr.endswith(b"\n\n") and json.loads(fr[6:])["choices"][0]["delta"] == {"content": "héllo"}
    assert json.loads(proto.chunk_role("c", "m")[6:])["choices"][0]["delta"]["role"] == "assistant"
    assert json.loads(proto.chunk_finish("c", "m", "stop")[6:])["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "stop"}
    assert json.loads(proto.chunk_usage("c", "m", 3, 4)[6:])["usage"]["total_tokens"] == 7 and proto.SSE_DONE == b"data: [DONE]\n\n"
    hb = proto.StreamHoldback()
    seen = ""
    for piece in ["Sure", ". <", "tool", "_call>", '\n{"name": "f", "argu', 'ments": {}}\n</tool', "_call>", " done <", "b>"]:
        out = hb.push(piece)
        assert "<tool" not in out
        seen += out
    rest, calls = hb.finish()
    assert seen + rest == "Sure.  done <b>" and [c["function"]["name"] for c in calls] == ["f"]
    hb = proto.StreamHoldback()
    assert hb.push("a <tool_ca") == "a " and hb.finish() == ("<tool_ca", [])          # a prefix that never completes is released at the end
