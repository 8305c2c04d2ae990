"""Chat templates: ChatML (+Qwen tool preamble, tool-response merging, think gating), Llama-3, Mistral,
DeepSeek-R1, Granite, Gemma and Harmony (gpt-oss: system block with date and reasoning effort, developer
block with JSON-schema -> TypeScript function signatures, prior tool calls on the commentary channel).

The strings are the wire formats the model families were trained on; behaviour parity with
src/tokenizer/tokenizer.cpp:734-1097.  One table-driven renderer replaces the reference's seven builders.
"""
from __future__ import annotations

import datetime
import json
from dataclasses import dataclass
from typing import Any, Optional, Sequence


@dataclass
class ChatTurn:
    role: str
    content: str = ""


TOOL_OPEN, TOOL_CLOSE = "<tool_call>", "</tool_call>"


def _tools_preamble(tools_json: str) -> str:
    try:
        tools = json.loads(tools_json)
        lines = "".join("\n" + json.dumps(t, ensure_ascii=False, separators=(", ", ": ")) for t in tools) if isinstance(tools, list) else "\n" + tools_json
    except Exception:
        lines = "\n" + tools_json
    return ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
            "You are provided with function signatures within <tools></tools> XML tags:\n<tools>" + lines + "\n</tools>\n\n"
            "For each function call, return a json object with function name and arguments within <tool_call></tool_call> XML tags:\n"
            "<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>")


def chatml(turns: Sequence[ChatTurn], add_generation_prompt=True, enable_thinking=True, tools_json: str = "", model_has_think=True) -> str:
    out, i, n = [], 0, len(turns)
    if tools_json:
        out.append("<|im_start|>system\n")
        if n and turns[0].role == "system":
            if turns[0].content:
                out.append(turns[0].content + "\n\n")
            i = 1
        out.append(_tools_preamble(tools_json) + "<|im_end|>\n")
    while i < n:
        t = turns[i]
        if t.role == "tool":
            out.append("<|im_start|>user")
            while i < n and turns[i].role == "tool":       # consecutive tool results share one user turn
                out.append("\n<tool_response>\n" + turns[i].content + "\n</tool_response>")
                i += 1
            out.append("<|im_end|>\n")
            continue
        out.append(f"<|im_start|>{t.role}\n{t.content}<|im_end|>\n")
        i += 1
    if add_generation_prompt:
        out.append("<|im_start|>assistant\n")
        if model_has_think:
            out.append("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")
    return "".join(out)


def llama3(turns, add_generation_prompt=True) -> str:
    s = "".join(f"<|start_header_id|>{t.role}<|end_header_id|>\n\n{t.content}<|eot_id|>" for t in turns)
    return s + ("<|start_header_id|>assistant<|end_header_id|>\n\n" if add_generation_prompt else "")


def mistral(turns, add_generation_prompt=True, system_prompt_block=False) -> str:
    sys_txt, rest = ("", list(turns))
    if rest and rest[0].role == "system":
        sys_txt, rest = rest[0].content, rest[1:]
    out, first = [], True
    for t in rest:
        if t.role == "user":
            head = ""
            if first and sys_txt:
                head = f"[SYSTEM_PROMPT]{sys_txt}[/SYSTEM_PROMPT]\n\n" if system_prompt_block else sys_txt + "\n\n"
            out.append(f"[INST] {head}{t.content} [/INST]")
            first = False
        elif t.role == "assistant":
            out.append(f" {t.content}</s>")
    return "".join(out)


_DS_USER, _DS_ASSIST, _DS_EOS = "<｜User｜>", "<｜Assistant｜>", "<｜end▁of▁sentence｜>"


def deepseek(turns, add_generation_prompt=True, enable_thinking=True) -> str:
    rest = list(turns)
    s = ""
    if rest and rest[0].role == "system":
        s, rest = rest[0].content, rest[1:]
    for t in rest:
        if t.role == "user":
            s += _DS_USER + t.content
        elif t.role == "assistant":
            s += _DS_ASSIST + t.content + _DS_EOS
    if add_generation_prompt:
        s += _DS_ASSIST + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")
    return s


def granite(turns, add_generation_prompt=True) -> str:
    s = "".join(f"<|start_of_role|>{t.role}<|end_of_role|>{t.content}<|end_of_text|>\n" for t in turns)
    return s + ("<|start_of_role|>assistant<|end_of_role|>" if add_generation_prompt else "")


def gemma(turns, add_generation_prompt=True) -> str:
    s = "".join(f"<|turn>{'model' if t.role == 'assistant' else t.role}\n{t.content}<turn|>\n" for t in turns)
    return s + ("<|turn>model\n" if add_generation_prompt else "")


# ---- Harmony ---------------------------------------------------------------------------------------
def schema_to_ts(sch: Any) -> str:
    if not isinstance(sch, dict):
        return "any"
    if isinstance(sch.get("enum"), list) and sch["enum"]:
        return " | ".join(f'"{e}"' if isinstance(e, str) else json.dumps(e) for e in sch["enum"])
    ty = sch.get("type", "")
    if ty == "string":
        return "string"
    if ty in ("number", "integer"):
        return "number"
    if ty == "boolean":
        return "boolean"
    if ty == "array":
        return (schema_to_ts(sch["items"]) if "items" in sch else "any") + "[]"
    if ty == "object" or "properties" in sch:
        props = sch.get("properties") if isinstance(sch.get("properties"), dict) else {}
        req = [r for r in sch.get("required", []) if isinstance(r, str)] if isinstance(sch.get("required"), list) else []
        fields = ", ".join(f"{k}{'' if k in req else '?'}: {schema_to_ts(v)}" for k, v in props.items())
        return "{ " + fields + " }"
    return "any"


def _harmony_tools(tools_json: str) -> str:
    try:
        tools = json.loads(tools_json)
    except Exception:
        return ""
    if not isinstance(tools, list) or not tools:
        return ""
    dev = "# Tools\n\n## functions\n\nnamespace functions {\n\n"
    for t in tools:
        fn = t.get("function") if isinstance(t, dict) and "function" in t else (t if isinstance(t, dict) and "name" in t else None)
        if not isinstance(fn, dict) or not isinstance(fn.get("name"), str):
            continue
        if isinstance(fn.get("description"), str) and fn["description"]:
            dev += f"// {fn['description']}\n"
        sig = "() => any;"
        p = fn.get("parameters")
        if isinstance(p, dict) and isinstance(p.get("properties"), dict) and p["properties"]:
            sig = f"(_: {schema_to_ts(p)}) => any;"
        dev += f"type {fn['name']} = {sig}\n\n"
    return dev + "} // namespace functions\n"


def harmony(turns, add_generation_prompt=True, reasoning_effort="medium", tools_json: str = "", today: Optional[str] = None) -> str:
    date = today or datetime.date.today().isoformat()
    s = ("<|start|>system<|message|>You are ChatGPT, a large language model trained by OpenAI.\nKnowledge cutoff: 2024-06\n"
         f"Current date: {date}\n\nReasoning: {reasoning_effort}\n\n"
         "# Valid channels: analysis, commentary, final. Channel must be included for every message.")
    if tools_json:
        s += "\nCalls to these tools must go to the commentary channel."
    s += "<|end|>"
    rest, dev = list(turns), ""
    if rest and rest[0].role == "system":
        if rest[0].content:
            dev += f"# Instructions\n\n{rest[0].content}\n\n"
        rest = rest[1:]
    if tools_json:
        dev += _harmony_tools(tools_json)
    if dev:
        s += f"<|start|>developer<|message|>{dev}<|end|>"
    last_fn = ""
    for t in rest:
        if t.role == "user":
            s += f"<|start|>user<|message|>{t.content}<|end|>"
        elif t.role == "assistant":
            any_call, p = False, 0
            while True:
                a = t.content.find(TOOL_OPEN, p)
                b = t.content.find(TOOL_CLOSE, a) if a >= 0 else -1
                if a < 0 or b < 0:
                    break
                try:
                    call = json.loads(t.content[a + len(TOOL_OPEN):b])
                except Exception:
                    call = None
                if isinstance(call, dict) and isinstance(call.get("name"), str):
                    last_fn = call["name"]
                    args = call.get("arguments")
                    args = "{}" if args is None else (args if isinstance(args, str) else json.dumps(args, ensure_ascii=False, separators=(",", ":")))
                    s += f"<|start|>assistant<|channel|>commentary to=functions.{last_fn} <|constrain|>json<|message|>{args}<|call|>"
                    any_call = True
                p = b + len(TOOL_CLOSE)
            if not any_call:
                s += f"<|start|>assistant<|channel|>final<|message|>{t.content}<|end|>"
        elif t.role == "tool":
            s += f"<|start|>functions.{last_fn or 'tool'} to=assistant<|channel|>commentary<|message|>{t.content}<|end|>"
    if add_generation_prompt:
        s += "<|start|>assistant"
    return s


def harmony_postprocess(text: str) -> str:
    """Generated Harmony text -> client text: a call ``to=functions.NAME ... <|message|>{json}<|call|>`` becomes the
    canonical ``<tool_call>`` block, otherwise the text after the last ``<|message|>`` (the final channel) is kept
    (src/engine/engine.cpp:877-916)."""
    k = text.find("to=functions.")
    if k >= 0:
        name_end = k + len("to=functions.")
        j = name_end
        while j < len(text) and (text[j].isalnum() or text[j] in "_-."):
            j += 1
        name = text[name_end:j]
        m = text.find("<|message|>", j)
        if m >= 0 and name:
            body = text[m + len("<|message|>"):]
            for stop in ("<|call|>", "<|end|>", "<|return|>"):
                c = body.find(stop)
                if c >= 0:
                    body = body[:c]
            body = body.strip() or "{}"
            return f'{TOOL_OPEN}\n{{"name": "{name}", "arguments": {body}}}\n{TOOL_CLOSE}'
    m = text.rfind("<|message|>")
    out = text[m + len("<|message|>"):] if m >= 0 else text
    for stop in ("<|return|>", "<|end|>", "<|call|>"):
        c = out.find(stop)
        if c >= 0:
            out = out[:c]
    return out


def render(family: str, turns: Sequence[ChatTurn], add_generation_prompt=True, enable_thinking=True, tools_json: str = "",
           model_has_think=True, mistral_sysprompt=False) -> str:
    """Template-family dispatch (``Engine::chat``, src/engine/engine.cpp:922-1021).  Tools are supported on the ChatML and
    Harmony families only; other families raise ``ValueError`` when tools are given."""
    if tools_json and family not in ("chatml", "auto", "harmony"):
        raise ValueError(f"tool calling is not supported for the {family} template family")
    if family in ("chatml", "auto"):
        return chatml(turns, add_generation_prompt, enable_thinking, tools_json, model_has_think)
    if family == "llama3":
        return llama3(turns, add_generation_prompt)
    if family == "mistral":
        return mistral(turns, add_generation_prompt, mistral_sysprompt)
    if family == "deepseek":
        return deepseek(turns, add_generation_prompt, enable_thinking)
    if family == "granite":
        return granite(turns, add_generation_prompt)
    if family == "gemma":
        return gemma(turns, add_generation_prompt)
    if family == "harmony":
        return harmony(turns, add_generation_prompt, "high" if enable_thinking else "low", tools_json)
    raise ValueError(f"unknown template family {family}")
