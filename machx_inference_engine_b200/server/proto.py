"""OpenAI chat-completions wire protocol: request validation, response / SSE frame builders and the
tool-call extraction (strict and lenient) from generated text.

Reference parity: src/server/openai_proto.cpp:17-359 (fields accepted: messages incl. multi-part text,
assistant ``tool_calls`` re-rendered as ``<tool_call>`` text, role ``tool``; temperature / top_p / top_k /
min_p / repeat_penalty | repetition_penalty / max_tokens (omitted = unlimited) / seed / stream /
enable_thinking / tools; usage with cached tokens; SSE chunk, tool_calls and usage frames, ``[DONE]``).
"""
from __future__ import annotations

import json
import re
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Optional

from ..tokenizer.templates import TOOL_CLOSE, TOOL_OPEN, ChatTurn


class BadRequest(ValueError):
    def __init__(self, message: str, code: str = "invalid_request_error", status: int = 400):
        super().__init__(message)
        self.code, self.status = code, status


@dataclass
class ChatRequest:
    turns: list = field(default_factory=list)
    model: str = ""
    temperature: float = 0.7
    top_p: float = 0.95
    top_k: int = 40
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    max_tokens: int = 0              # 0 = until the context is full
    seed: int = 0
    stream: bool = False
    enable_thinking: bool = True
    tools_json: str = ""
    include_usage: bool = True


def _text_of(content: Any) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if isinstance(content, list):            # multi-part content: concatenate the text parts
        parts = []
        for p in content:
            if isinstance(p, dict) and p.get("type") in ("text", "input_text") and isinstance(p.get("text"), str):
                parts.append(p["text"])
            elif isinstance(p, str):
                parts.append(p)
        return "".join(parts)
    raise BadRequest("message content must be a string or a list of text parts")


def _num(d, key, default, lo=None, hi=None, cast=float):
    v = d.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise BadRequest(f"'{key}' must be a number")
    v = cast(v)
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise BadRequest(f"'{key}' is out of range")
    return v


def parse_chat_request(body: bytes | str | dict) -> ChatRequest:
    if not isinstance(body, dict):
        try:
            body = json.loads(body)
        except Exception as e:
            raise BadRequest(f"request body is not valid JSON: {e}")
    if not isinstance(body, dict):
        raise BadRequest("request body must be a JSON object")
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs:
        raise BadRequest("'messages' must be a non-empty array")
    req = ChatRequest(model=str(body.get("model", "")))
    for m in msgs:
        if not isinstance(m, dict) or not isinstance(m.get("role"), str):
            raise BadRequest("every message needs a string 'role'")
        role = m["role"]
        if role not in ("system", "developer", "user", "assistant", "tool"):
            raise BadRequest(f"unknown role '{role}'")
        text = _text_of(m.get("content"))
        if role == "assistant" and isinstance(m.get("tool_calls"), list):
            for tc in m["tool_calls"]:                       # prior calls go back into the prompt as <tool_call> text
                fn = tc.get("function", {}) if isinstance(tc, dict) else {}
                name = fn.get("name")
                if not isinstance(name, str):
                    raise BadRequest("tool_calls[].function.name must be a string")
                args = fn.get("arguments", "{}")
                if not isinstance(args, str):
                    args = json.dumps(args)
                try:
                    json.loads(args)
                except Exception:
                    args = json.dumps(args)
                text += f'{TOOL_OPEN}\n{{"name": "{name}", "arguments": {args}}}\n{TOOL_CLOSE}'
        req.turns.append(ChatTurn("system" if role == "developer" else role, text))
    req.temperature = _num(body, "temperature", 0.7, 0.0, 10.0)
    req.top_p = _num(body, "top_p", 0.95, 0.0, 1.0)
    req.top_k = _num(body, "top_k", 40, 0, 1 << 20, int)
    req.min_p = _num(body, "min_p", 0.0, 0.0, 1.0)
    rp = body.get("repetition_penalty", body.get("repeat_penalty", 1.0))
    req.repetition_penalty = _num({"repetition_penalty": rp}, "repetition_penalty", 1.0, 0.01, 100.0)
    mt = body.get("max_tokens", body.get("max_completion_tokens"))
    req.max_tokens = 0 if mt is None else _num({"max_tokens": mt}, "max_tokens", 0, 0, 1 << 30, int)
    req.seed = _num(body, "seed", 0, None, None, int)
    req.stream = bool(body.get("stream", False))
    so = body.get("stream_options")
    req.include_usage = True if not isinstance(so, dict) else bool(so.get("include_usage", True))
    req.enable_thinking = bool(body.get("enable_thinking", True))
    ctk = body.get("chat_template_kwargs")
    if isinstance(ctk, dict) and "enable_thinking" in ctk:
        req.enable_thinking = bool(ctk["enable_thinking"])
    tools = body.get("tools")
    if tools is not None:
        if not isinstance(tools, list):
            raise BadRequest("'tools' must be an array")
        for t in tools:
            fn = t.get("function") if isinstance(t, dict) else None
            if not isinstance(fn, dict) or not isinstance(fn.get("name"), str) or not fn["name"]:
                raise BadRequest("every tool needs function.name")
        if tools:
            req.tools_json = json.dumps(tools, ensure_ascii=False)
    return req


# ---- tool-call extraction -------------------------------------------------------------------------
_LENIENT_NAME = re.compile(r'"?name"?\s*:\s*"?([A-Za-z_][\w.\-]*)"?')


def _parse_call(inner: str) -> Optional[dict]:
    inner = inner.strip()
    try:
        obj = json.loads(inner)
        if isinstance(obj, dict) and isinstance(obj.get("name"), str):
            args = obj.get("arguments", {})
            return {"name": obj["name"], "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}
    except Exception:
        pass
    # lenient: unquoted name, missing closing brace, trailing text
    m = _LENIENT_NAME.search(inner)
    if not m:
        return None
    name = m.group(1)
    a = inner.find("arguments")
    args = "{}"
    if a >= 0:
        b = inner.find("{", a)
        if b >= 0:
            depth, end = 0, -1
            for i in range(b, len(inner)):
                if inner[i] == "{":
                    depth += 1
                elif inner[i] == "}":
                    depth -= 1
                    if depth == 0:
                        end = i
                        break
            cand = inner[b:end + 1] if end >= 0 else inner[b:] + "}" * max(depth, 1)
            try:
                json.loads(cand)
                args = cand
            except Exception:
                args = "{}"
    return {"name": name, "arguments": args}


def extract_tool_calls(text: str) -> tuple[str, list]:
    """Returns (text without the call blocks, [ {id, type, function:{name, arguments}} ... ])."""
    calls, out, p = [], [], 0
    while True:
        a = text.find(TOOL_OPEN, p)
        if a < 0:
            out.append(text[p:])
            break
        b = text.find(TOOL_CLOSE, a)
        inner = text[a + len(TOOL_OPEN): b if b >= 0 else len(text)]
        call = _parse_call(inner)
        out.append(text[p:a])
        if call is not None:
            calls.append({"id": "call_" + uuid.uuid4().hex[:24], "type": "function", "function": call})
        else:
            out.append(text[a: (b + len(TOOL_CLOSE)) if b >= 0 else len(text)])
        if b < 0:
            break
        p = b + len(TOOL_CLOSE)
    return "".join(out).strip() if calls else "".join(out), calls


# ---- responses ----------------------------------------------------------------------------------
def _usage(prompt_tokens: int, completion_tokens: int, cached_tokens: int = 0) -> dict:
    return {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens, "total_tokens": prompt_tokens + completion_tokens,
            "prompt_tokens_details": {"cached_tokens": cached_tokens}}


def new_id() -> str:
    return "chatcmpl-" + uuid.uuid4().hex[:24]


def chat_completion_json(cid: str, model: str, text: str, finish_reason: str, prompt_tokens: int, completion_tokens: int, cached_tokens: int = 0) -> dict:
    content, calls = extract_tool_calls(text)
    msg: dict = {"role": "assistant", "content": content if (content or not calls) else None}
    if calls:
        msg["tool_calls"] = calls
        finish_reason = "tool_calls"
    return {"id": cid, "object": "chat.completion", "created": int(time.time()), "model": model,
            "choices": [{"index": 0, "message": msg, "finish_reason": finish_reason}], "usage": _usage(prompt_tokens, completion_tokens, cached_tokens)}


def _sse(obj: dict) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode() + b"\n\n"


def chunk_role(cid: str, model: str) -> bytes:
    return _sse({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
                 "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]})


def chunk_text(cid: str, model: str, text: str) -> bytes:
    return _sse({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
                 "choices": [{"index": 0, "delta": {"content": text}, "finish_reason": None}]})


def chunk_tool_calls(cid: str, model: str, calls: list) -> bytes:
    delta = [{"index": i, "id": c["id"], "type": "function", "function": c["function"]} for i, c in enumerate(calls)]
    return _sse({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
                 "choices": [{"index": 0, "delta": {"tool_calls": delta}, "finish_reason": None}]})


def chunk_finish(cid: str, model: str, finish_reason: str) -> bytes:
    return _sse({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model,
                 "choices": [{"index": 0, "delta": {}, "finish_reason": finish_reason}]})


def chunk_usage(cid: str, model: str, prompt_tokens: int, completion_tokens: int, cached_tokens: int = 0) -> bytes:
    return _sse({"id": cid, "object": "chat.completion.chunk", "created": int(time.time()), "model": model, "choices": [],
                 "usage": _usage(prompt_tokens, completion_tokens, cached_tokens)})


SSE_DONE = b"data: [DONE]\n\n"


def error_json(message: str, code: str = "invalid_request_error", etype: str = "invalid_request_error") -> dict:
    return {"error": {"message": message, "type": etype, "code": code}}


class StreamHoldback:
    """Streams text while never letting a forming ``<tool_call>`` (or any prefix of the tag) leak to the client
    (src/server/openai_server.cpp:131-141: tail hold-back)."""

    def __init__(self):
        self.buf = ""
        self.in_call = False
        self.calls_text = ""

    def push(self, piece: str) -> str:
        self.buf += piece
        out = ""
        while True:
            if self.in_call:
                b = self.buf.find(TOOL_CLOSE)
                if b < 0:
                    return out
                self.calls_text += self.buf[: b + len(TOOL_CLOSE)]
                self.buf = self.buf[b + len(TOOL_CLOSE):]
                self.in_call = False
                continue
            a = self.buf.find(TOOL_OPEN)
            if a >= 0:
                out += self.buf[:a]
                self.buf = self.buf[a:]
                self.in_call = True
                continue
            # keep back the longest suffix that could still grow into the opening tag
            keep = 0
            for k in range(min(len(TOOL_OPEN) - 1, len(self.buf)), 0, -1):
                if TOOL_OPEN.startswith(self.buf[-k:]):
                    keep = k
                    break
            out += self.buf[: len(self.buf) - keep]
            self.buf = self.buf[len(self.buf) - keep:]
            return out

    def finish(self) -> tuple[str, list]:
        """Remaining visible text and the parsed tool calls."""
        rest = self.buf
        self.buf = ""
        if self.in_call:
            self.calls_text += rest
            rest = ""
        _, calls = extract_tool_calls(self.calls_text) if self.calls_text else ("", [])
        return rest, calls
