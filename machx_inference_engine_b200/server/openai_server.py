"""OpenAI-compatible HTTP server (default port 11435).

Routes: ``GET /health``, ``GET /v1/models``, ``GET /metrics``, ``POST /v1/embeddings`` (501),
``POST /v1/chat/completions`` (JSON and SSE).  Reference parity: src/server/openai_server.cpp:22-199
(same routes, 400 for ``context_length_exceeded``, tail hold-back so a forming ``<tool_call>`` never leaks,
Harmony output buffered then emitted, usage chunk, ``[DONE]``, bind-before-announce).  Unlike the reference,
which serialises generation behind one mutex, every connection thread hands its request to the shared
:class:`~runtime.api.EngineLoop`, so concurrent requests are batched into the same forward passes.
"""
from __future__ import annotations

import json
import queue
import sys
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..runtime.api import Engine, EngineLoop
from ..runtime.engine import SamplingParams
from . import proto


def make_handler(eng: Engine, loop: EngineLoop, model_id: str):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):      # quiet: one [gen] line per request comes from the engine
            pass

        def _json(self, status: int, obj: dict):
            body = json.dumps(obj, ensure_ascii=False).encode()
            self.send_response(status)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path == "/health":
                return self._json(200, {"status": "ok"})
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": model_id, "object": "model", "owned_by": "local"}]})
            if self.path == "/metrics":
                m = loop.metrics
                llm = eng.llm
                lines = [
                    f"mx_requests_total {m['requests']}", f"mx_request_errors_total {m['errors']}", f"mx_tokens_generated_total {m['tokens_out']}",
                    f"mx_ttft_seconds_sum {m['ttft_sum']:.6f}", f"mx_ttft_seconds_count {m['ttft_n']}", f"mx_queue_depth {m['queue_depth']}",
                    f"mx_running_requests {len(llm.sched.running)}", f"mx_kv_blocks_free {llm.bm.n_free()}", f"mx_kv_blocks_total {llm.bm.num_blocks}",
                    f"mx_prefix_cache_hits_total {llm.bm.hits}", f"mx_engine_steps_total {llm.stats['steps']}",
                ]
                body = ("\n".join(lines) + "\n").encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            self._json(404, proto.error_json("not found", "not_found"))

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0") or 0)
            body = self.rfile.read(n) if n else b""
            if self.path == "/v1/embeddings":
                return self._json(501, proto.error_json("embeddings are not implemented", "not_implemented"))
            if self.path != "/v1/chat/completions":
                return self._json(404, proto.error_json("not found", "not_found"))
            try:
                req = proto.parse_chat_request(body)
                ids = eng.encode_chat(req.turns, req.enable_thinking, req.tools_json)
            except proto.BadRequest as e:
                return self._json(e.status, proto.error_json(str(e), e.code))
            except ValueError as e:
                return self._json(400, proto.error_json(str(e)))
            sp = SamplingParams(temperature=req.temperature, top_k=req.top_k, top_p=req.top_p, min_p=req.min_p,
                                repetition_penalty=req.repetition_penalty, max_tokens=req.max_tokens, seed=req.seed)
            cid = proto.new_id()
            events: queue.Queue = queue.Queue()
            ticket = loop.submit(ids, sp, (lambda piece: events.put(("text", piece))) if req.stream else None, lambda res: events.put(("done", res)))
            if not req.stream:
                kind, res = events.get()
                while kind != "done":
                    kind, res = events.get()
                if res.finish_reason == "context_length_exceeded":
                    return self._json(400, proto.error_json(res.error, "context_length_exceeded"))
                if res.finish_reason == "error":
                    return self._json(500, proto.error_json(res.error or "generation failed", "internal_error", "server_error"))
                return self._json(200, proto.chat_completion_json(cid, model_id, res.text, res.finish_reason, res.prompt_tokens, res.completion_tokens,
                                                                 res.cached_tokens))
            # ---- SSE
            first = True
            hold = proto.StreamHoldback()
            try:
                while True:
                    kind, val = events.get()
                    if first:
                        if kind == "done" and val.finish_reason == "context_length_exceeded":
                            return self._json(400, proto.error_json(val.error, "context_length_exceeded"))
                        self.send_response(200)
                        self.send_header("Content-Type", "text/event-stream")
                        self.send_header("Cache-Control", "no-cache")
                        self.send_header("Connection", "close")
                        self.end_headers()
                        self.wfile.write(proto.chunk_role(cid, model_id))
                        first = False
                    if kind == "text":
                        vis = hold.push(val)
                        if vis:
                            self.wfile.write(proto.chunk_text(cid, model_id, vis))
                            self.wfile.flush()
                        continue
                    res = val
                    rest, calls = hold.finish()
                    if rest:
                        self.wfile.write(proto.chunk_text(cid, model_id, rest))
                    finish = res.finish_reason
                    if calls:
                        self.wfile.write(proto.chunk_tool_calls(cid, model_id, calls))
                        finish = "tool_calls"
                    self.wfile.write(proto.chunk_finish(cid, model_id, finish))
                    if req.include_usage:
                        self.wfile.write(proto.chunk_usage(cid, model_id, res.prompt_tokens, res.completion_tokens, res.cached_tokens))
                    self.wfile.write(proto.SSE_DONE)
                    self.wfile.flush()
                    self.close_connection = True
                    return
            except (BrokenPipeError, ConnectionResetError):
                loop.abort(ticket)         # client went away mid-stream: free its KV blocks, keep serving the others
                self.close_connection = True

    return Handler


def run_openai_server(eng: Engine, model_id: str, host: str = "127.0.0.1", port: int = 11435, ready: threading.Event | None = None, par=None):
    """Binds first, then announces (a bind failure exits before any 'listening' line is printed).  With ``par`` (a
    multi-GPU job) this is rank 0's side of the SPMD serving loop; the other ranks run ``EngineLoop(eng, par).run()``."""
    loop = EngineLoop(eng, par)
    try:
        httpd = ThreadingHTTPServer((host, port), make_handler(eng, loop, model_id))
    except OSError as e:
        print(f"error: cannot bind {host}:{port}: {e}", file=sys.stderr)
        return 1
    loop.start()
    print(f"ie serve: listening on http://{host}:{httpd.server_address[1]} (model {model_id})", file=sys.stderr)
    if ready is not None:
        ready.httpd = httpd
        ready.set()
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        loop.stop()
        httpd.server_close()
    return 0
