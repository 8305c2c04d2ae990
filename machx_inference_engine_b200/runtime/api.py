"""Public engine API: load a checkpoint, ``generate`` / ``chat`` text, and the background batching loop that
the server drives.

Reference parity: ``Engine::load / generate / chat`` (src/engine/engine.cpp:30-433, 444-920, 922-1021) with
``GenerateResult`` / ``TokenCallback`` (include/ie/engine.hpp:43-139): per-family stop ids, ``<tool_call>``
handling, context budget error, incremental UTF-8-safe detokenisation, Harmony post-processing, and the
``cache_prefix_len`` idea (here: block-hash prefix sharing makes it automatic).  Where the reference
serialises requests behind a mutex, :class:`EngineLoop` batches them continuously.
"""
from __future__ import annotations

import queue
import sys
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch

from ..formats.model_config import ModelConfig
from ..tokenizer import templates
from ..tokenizer.templates import ChatTurn
from ..tokenizer.tokenizer import IncrementalDetokenizer, Tokenizer
from .engine import ContextLengthExceeded, EngineOptions, LLMEngine, OutOfBlocks, SamplingParams, Sequence as Seq

STOP_TOKENS = {
    "chatml": ["<|im_end|>", "<|endoftext|>"],
    "llama3": ["<|eot_id|>", "<|end_of_text|>", "<|eom_id|>"],
    "mistral": ["</s>"],
    "deepseek": ["<｜end▁of▁sentence｜>"],
    "granite": ["<|end_of_text|>"],
    "gemma": ["<turn|>", "<end_of_turn>", "<eos>"],
    "harmony": ["<|return|>", "<|call|>", "<|endoftext|>"],
    "auto": ["<|im_end|>", "<|endoftext|>", "</s>", "<|eot_id|>"],
}


@dataclass
class GenerateResult:
    text: str = ""
    token_ids: list = field(default_factory=list)
    finish_reason: str = "stop"
    prompt_tokens: int = 0
    completion_tokens: int = 0
    cached_tokens: int = 0
    ttft_s: float = 0.0
    prefill_tok_s: float = 0.0
    decode_tok_s: float = 0.0
    error: str = ""


class Engine:
    def __init__(self, model, tokenizer: Optional[Tokenizer], opts: Optional[EngineOptions] = None, model_id: str = "model"):
        self.model, self.tok, self.cfg = model, tokenizer, model.cfg
        self.model_id = model_id
        self.family = self.cfg.template_family if self.cfg.template_family != "auto" else ("harmony" if self.cfg.arch == "gpt-oss" else "chatml")
        opts = opts or EngineOptions()
        self.stop_ids = self._stop_ids()
        opts.eos_ids = tuple(sorted(set(opts.eos_ids) | set(self.stop_ids)))
        self.llm = LLMEngine(model, opts)
        self.keep_special = tuple(i for i in (self._find("<tool_call>"), self._find("</tool_call>")) if i >= 0)
        self.model_has_think = self._find("<think>") >= 0
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ loading
    @classmethod
    def load(cls, path: str, device="cuda", opts: Optional[EngineOptions] = None, par=None, spec_head: Optional[str] = None) -> "Engine":
        """``spec_head``: a separate draft-head checkpoint (Gemma-4's ``gemma4-assistant`` GGUF); heads stored inside the model file
        (Qwen3-Next's MTP layer) need none."""
        from ..models import load_model
        opts = opts or EngineOptions()
        model, reader = load_model(path, device, par, max_ctx=opts.max_ctx)
        if spec_head:
            from ..models.gemma4_assistant import load_assistant_head
            load_assistant_head(model, spec_head)
        opts.max_ctx = min(opts.max_ctx, model.max_ctx)
        tok = Tokenizer.from_gguf_kv(reader.kv)
        return cls(model, tok, opts, model_id=str(reader.kv.get("general.name", "")) or path.rsplit("/", 1)[-1])

    def _find(self, s: str) -> int:
        return self.tok.find_token(s) if self.tok is not None else -1

    def _stop_ids(self) -> list:
        ids = []
        if self.tok is None:
            return ids
        for s in STOP_TOKENS.get(self.family, STOP_TOKENS["auto"]):
            i = self.tok.find_token(s)
            if i >= 0:
                ids.append(i)
        if self.tok.eos_id >= 0:
            ids.append(self.tok.eos_id)
        return sorted(set(ids))

    # ------------------------------------------------------------------ text API (blocking, single request)
    def encode_chat(self, turns: Sequence[ChatTurn], enable_thinking=True, tools_json: str = "") -> list:
        text = templates.render(self.family, turns, True, enable_thinking, tools_json, self.model_has_think, self.cfg.mistral_sysprompt)
        return self.tok.encode(text, allow_special=True)

    def generate(self, prompt: str | list, sp: Optional[SamplingParams] = None, on_text: Optional[Callable[[str], None]] = None) -> GenerateResult:
        ids = self.tok.encode(prompt, allow_special=True) if isinstance(prompt, str) else list(prompt)
        with self._lock:
            return self._run_blocking(ids, sp or SamplingParams(), on_text)

    def chat(self, turns: Sequence[ChatTurn], sp: Optional[SamplingParams] = None, on_text=None, enable_thinking=True, tools_json: str = "") -> GenerateResult:
        try:
            ids = self.encode_chat(turns, enable_thinking, tools_json)
        except ValueError as e:
            return GenerateResult(finish_reason="error", error=str(e))
        with self._lock:
            return self._run_blocking(ids, sp or SamplingParams(), on_text)

    def _run_blocking(self, ids: list, sp: SamplingParams, on_text) -> GenerateResult:
        st = StreamState(self, on_text)
        t0 = time.perf_counter()
        try:
            seq = self.llm.add_request(ids, sp, on_token=lambda s, t: st.on_token(t))
        except ContextLengthExceeded as e:
            return GenerateResult(finish_reason="context_length_exceeded", error=str(e), prompt_tokens=len(ids))
        while not seq.finished:
            self.llm.step()
        return st.result(seq, t0)


class StreamState:
    """Per-request detokenisation state: incremental UTF-8-safe text, Harmony buffering."""

    def __init__(self, eng: Engine, on_text: Optional[Callable[[str], None]]):
        self.eng, self.on_text = eng, on_text
        self.detok = IncrementalDetokenizer(eng.tok, skip_special=eng.family != "harmony", keep_special=eng.keep_special) if eng.tok else None
        self.text = ""
        self.harmony = eng.family == "harmony"

    def on_token(self, tok: int) -> None:
        if self.detok is None or tok in self.eng.stop_ids:
            return
        piece = self.detok.push(tok)
        if piece:
            self.text += piece
            if self.on_text is not None and not self.harmony:      # Harmony output is post-processed as a whole
                self.on_text(piece)

    def result(self, seq: Seq, t0: float) -> GenerateResult:
        if self.detok is not None:
            tail = self.detok.flush()
            self.text += tail
            if tail and self.on_text is not None and not self.harmony:
                self.on_text(tail)
        text = self.text
        if self.harmony:
            text = templates.harmony_postprocess(text)
            if self.on_text is not None and text:
                self.on_text(text)
        now = time.perf_counter()
        ttft = (seq.t_first_token - seq.t_arrival) if seq.t_first_token else 0.0
        n_gen = seq.n_generated
        gen_ids = seq.tokens[len(seq.prompt):]
        dec_t = now - seq.t_first_token if seq.t_first_token else 0.0
        res = GenerateResult(text=text, token_ids=gen_ids, finish_reason=seq.finish_reason or "stop", prompt_tokens=len(seq.prompt),
                             completion_tokens=n_gen, cached_tokens=seq.n_cached_prefix, ttft_s=ttft,
                             prefill_tok_s=(len(seq.prompt) - seq.n_cached_prefix) / ttft if ttft > 0 else 0.0,
                             decode_tok_s=(n_gen - 1) / dec_t if dec_t > 0 and n_gen > 1 else 0.0)
        print(f"[gen] prefill {res.prompt_tokens} tok ({res.cached_tokens} cached) {res.prefill_tok_s:.1f} tok/s | decode {n_gen} tok {res.decode_tok_s:.1f} tok/s",
              file=sys.stderr)
        return res


class EngineLoop(threading.Thread):
    """Owns the LLMEngine on one thread; any number of client threads submit requests and receive token callbacks.
    One bad request (too long, aborted client) never disturbs the others in the batch.

    Multi-GPU serving is SPMD: every rank runs this loop over its shard of the model.  Rank 0 owns the HTTP front end;
    before each iteration it broadcasts the step plan -- requests admitted and aborted since the last one, and whether to
    step, idle or stop -- over the host-side control group, and every rank applies it in the same order.  Schedulers and
    samplers are deterministic functions of that history (logits are bit-identical on all ranks after the rank-ordered
    reductions), so the ranks stay in lockstep without exchanging tokens.  (The reference drives all GPUs from one host
    thread, include/ie/engine.hpp:146-265; ranks > 0 call :meth:`run` directly as their whole job.)"""

    def __init__(self, eng: Engine, par=None):
        super().__init__(daemon=True, name="engine-loop")
        self.eng = eng
        self.par = par if (par is not None and par.world > 1) else None
        self.inbox: queue.Queue = queue.Queue()
        self.wake = threading.Event()
        self.stopping = False
        self.metrics = {"requests": 0, "errors": 0, "tokens_out": 0, "ttft_sum": 0.0, "ttft_n": 0, "queue_depth": 0}

    def submit(self, ids: list, sp: SamplingParams, on_text: Optional[Callable[[str], None]], on_done: Callable[[GenerateResult], None]):
        ticket = {"ids": ids, "sp": sp, "on_text": on_text, "on_done": on_done, "abort": False, "seq": None}
        self.inbox.put(ticket)
        self.wake.set()
        return ticket

    def abort(self, ticket) -> None:
        ticket["abort"] = True
        self.wake.set()

    def stop(self) -> None:
        self.stopping = True
        self.wake.set()

    def _plan(self, live: dict) -> dict:
        """Rank 0: drain the inbox into a step plan.  Requests that cannot fit the context are answered here and never
        reach the other ranks."""
        new, tickets = [], []
        while True:
            try:
                tk = self.inbox.get_nowait()
            except queue.Empty:
                break
            self.metrics["requests"] += 1
            if len(tk["ids"]) == 0 or len(tk["ids"]) >= self.eng.llm.opts.max_ctx - 8:
                self.metrics["errors"] += 1
                tk["on_done"](GenerateResult(finish_reason="context_length_exceeded", prompt_tokens=len(tk["ids"]),
                                             error=f"prompt of {len(tk['ids'])} tokens does not fit the context of {self.eng.llm.opts.max_ctx}"))
                continue
            new.append((tk["ids"], tk["sp"]))
            tickets.append(tk)
        aborts = [sid for sid, (tk, st, t0) in live.items() if tk is not None and tk["abort"] and not tk["seq"].finished]
        return {"new": new, "abort": aborts, "stop": self.stopping, "_tickets": tickets}

    def run(self) -> None:
        llm = self.eng.llm
        live: dict = {}
        lead = self.par is None or self.par.rank == 0
        while True:
            plan = self._plan(live) if lead else None
            if self.par is not None:
                wire = None if plan is None else {k: v for k, v in plan.items() if k != "_tickets"}
                wire = self.par.broadcast_object(wire, src=0)
                plan = plan if lead else {**wire, "_tickets": [None] * len(wire["new"])}
            if plan["stop"]:
                break
            for (ids, sp), tk in zip(plan["new"], plan["_tickets"]):
                st = StreamState(self.eng, tk["on_text"] if tk else None)
                seq = llm.add_request(ids, sp, on_token=(lambda s, t, st=st: st.on_token(t)) if tk else None)
                if tk is not None:
                    tk["seq"] = seq
                    live[seq.seq_id] = (tk, st, time.perf_counter())
                else:
                    live[seq.seq_id] = (None, seq, 0.0)          # follower rank: keeps the sequence itself
            for sid in plan["abort"]:
                ent = live.get(sid)
                seq = ent[0]["seq"] if (ent and ent[0] is not None) else (ent[1] if ent else None)
                if seq is not None and not seq.finished:
                    llm.abort(seq)
            self.metrics["queue_depth"] = len(llm.sched.waiting)
            if llm.has_work():
                try:
                    llm.step()
                except OutOfBlocks as e:
                    # shed the request that holds the most blocks; the rest of the batch continues
                    seqs_live = [(v[0]["seq"] if v[0] is not None else v[1]) for v in live.values()]
                    victim = max((s_ for s_ in seqs_live if not s_.finished), key=lambda s_: (len(s_.tokens), -s_.seq_id), default=None)
                    if victim is not None:
                        victim.finish_reason = "error"
                        llm.abort(victim)
                        victim.finish_reason = "error"
                except Exception as e:      # a failed step fails the requests that were running, not the server
                    for tk, st, t0 in live.values():
                        seq = tk["seq"] if tk is not None else st
                        if not seq.finished:
                            llm.abort(seq)
                            seq.finish_reason = "error"
                    print(f"[engine-loop] step failed: {e!r}", file=sys.stderr)
            elif lead:
                self.wake.wait(timeout=0.05 if self.par is None else 0.005)
                self.wake.clear()
            for sid, (tk, st, t0) in list(live.items()):
                if tk is None:                      # follower rank: nothing to report, just forget finished sequences
                    if st.finished:
                        del live[sid]
                    continue
                seq = tk["seq"]
                if seq.finished:
                    res = st.result(seq, t0)
                    if seq.finish_reason in ("error", "abort"):
                        self.metrics["errors"] += seq.finish_reason == "error"
                    self.metrics["tokens_out"] += res.completion_tokens
                    if res.ttft_s > 0:
                        self.metrics["ttft_sum"] += res.ttft_s
                        self.metrics["ttft_n"] += 1
                    del live[sid]
                    tk["on_done"](res)
