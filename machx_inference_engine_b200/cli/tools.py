"""Small validation and measurement tools (one entry point, sub-commands):

    python -m machx_inference_engine_b200.cli.tools perplexity   --gguf M.gguf --text FILE | --tokens FILE [--ctx 2048]
    python -m machx_inference_engine_b200.cli.tools det-probe    --gguf M.gguf | --model NAME  [--runs 3]
    python -m machx_inference_engine_b200.cli.tools prompt-bench --gguf M.gguf [--runs 3]
    python -m machx_inference_engine_b200.cli.tools chunk-check  --gguf M.gguf | --model NAME [--chunks 64,256]
    python -m machx_inference_engine_b200.cli.tools soak         --gguf M.gguf | --model NAME --seconds 60
    python -m machx_inference_engine_b200.cli.tools layer-dump   --gguf M.gguf --device cuda --out a.pt [--tokens FILE]
    python -m machx_inference_engine_b200.cli.tools layer-diff   a.pt b.pt [--threshold 0.999]
    python -m machx_inference_engine_b200.cli.tools layer-parity --gguf M.gguf          (CUDA kernels against the fp32 PyTorch path)
    python -m machx_inference_engine_b200.cli.tools spec-accept  --gguf M.gguf | --model NAME [--spec-k 3] [--accept 0.0,0.5,0.8,1.0]
    python -m machx_inference_engine_b200.cli.tools kv-scale     --gguf M.gguf | --model NAME [--tokens-n 512]
    python -m machx_inference_engine_b200.cli.tools partial-stack --gguf M.gguf | --model NAME [--layers 1,2,4]
    python -m machx_inference_engine_b200.cli.tools bug-monitor  --gguf M.gguf | --model NAME [--chains 8] [--iters 32] [--batched] [--live]
    python -m machx_inference_engine_b200.cli.tools kernel-monitor --gguf M.gguf | --model NAME [--decode 32] [--interval 8] [--int8-kv]
    python -m machx_inference_engine_b200.cli.tools debug        --gguf M.gguf | --model NAME        (P <text> | T <ids> | R | Q on standard input)
    python -m machx_inference_engine_b200.cli.tools attn-profile [--ctx 1024,4096,16384] [--mode bf16|int8|both] [--q-heads 16 --kv-heads 2 --head-dim 256]

Reference parity (behaviour, not code): tools/ie_perplexity.cpp (streaming negative log-likelihood), tools/ie_det_probe.cpp and
ie_bug_monitor.cpp (run-to-run bit identity), tools/ie_prompt_bench.cpp (fixed prompts, first run discarded, median),
tools/ie_validate_chunking.cpp (chunked prefill against whole-prompt prefill), scripts/soak_1h.sh (completions per hour, failures),
tools/ie_dense_dump.cpp / ie_qwen35_dump.cpp / llama_dump.cpp + tools/diff_layers.sh (per-layer activation dumps of one prompt and their
layer-by-layer cosine comparison; here the second implementation is this package's own fp32 PyTorch path instead of llama.cpp),
tools/ie_qwen35_mtp_accept.cpp (draft acceptance and the decode speed-up it buys), tools/ie_kv_scale.cpp (what the int8 KV cache costs
in logit accuracy), tools/ie_partial_stack_eval.cpp (the model cut after its first n layers, to find the layer where two builds part).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

PROMPTS = [
    "Explain how a hash table handles collisions.",
    "Write a short poem about the sea at night.",
    "Summarise the causes of the French Revolution in three sentences.",
    "What is the difference between a process and a thread?",
    "Give me a recipe for a simple vegetable soup.",
]


def _load(a, max_ctx=4096, **opts):
    from ..formats.model_config import preset
    from ..models import build_model
    from ..runtime.api import Engine
    from ..runtime.engine import EngineOptions
    dev = torch.device(a.device if (a.device != "cuda" or torch.cuda.is_available()) else "cpu")
    eo = EngineOptions(max_ctx=max_ctx, **opts)
    par = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        # one rank per GPU (torchrun): every rank runs the same tool in lockstep over the sharded graph, rank 0 reports
        # (the reference's multi-GPU perplexity / equality tools: tools/multi_gpu_ppl.cpp, tools/multi_gpu_equality_test.cpp)
        from ..parallel.comm import init_from_env
        par = init_from_env("cuda" if dev.type == "cuda" else "cpu")
        if dev.type == "cuda":
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            from ..parallel.fused import FusedComm
            par.fused = FusedComm.create(par, dev)
    if a.gguf:
        return Engine.load(a.gguf, dev, eo, par=par)
    cfg = preset(a.model)
    quant = a.quant or ("mxfp4" if cfg.arch == "gpt-oss" else "q8_0")
    return Engine(build_model(cfg, dev, par, quant=quant, max_ctx=max_ctx), None, eo)


def _all_logits(eng, ids, chunk):
    """Teacher-forced logits [len(ids), vocab] obtained through the engine's scheduler with prefill chunks of `chunk` tokens."""
    from ..runtime.engine import EngineOptions, LLMEngine, SamplingParams
    m = eng.model
    llm = LLMEngine(m, EngineOptions(max_ctx=eng.llm.opts.max_ctx, max_batch_tokens=chunk, max_seqs=1, enable_prefix_cache=False, cuda_graphs=False,
                                     kv_dtype=eng.llm.opts.kv_dtype))
    orig_build = llm._build_batch

    def build(plan, sampled_rows, pad_to=0):          # ask for the logits of every row of every chunk
        host, mq = orig_build(plan, sampled_rows, pad_to)
        host["logit_rows"] = torch.arange(sum(k for _, k in plan), dtype=torch.int64)
        return host, mq
    llm._build_batch = build
    llm._sample = lambda logits, seqs: torch.zeros(len(seqs), dtype=torch.int32)
    grabbed = []
    m_forward = m.forward

    def grab(fb, *args, **kw):
        if fb.logit_rows is None or fb.logit_rows.numel() != fb.T:
            fb.logit_rows = torch.arange(fb.T, device=fb.ids.device)
        out = m_forward(fb, *args, **kw)
        grabbed.append((out[0] if isinstance(out, tuple) else out).float().cpu())
        return out
    m.forward = grab
    seq = llm.add_request(list(ids), SamplingParams(max_tokens=1, ignore_eos=True))
    try:
        while not seq.finished:
            llm.step()
    finally:
        m.forward = m_forward
    return torch.cat(grabbed)[:len(ids)]


def cmd_perplexity(a) -> int:
    eng = _load(a, max_ctx=a.ctx + 128)
    if a.tokens:
        ids = [int(t) for t in open(a.tokens).read().split()]
    elif a.text:
        ids = eng.tok.encode(open(a.text, encoding="utf-8").read())
    else:
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(0, eng.cfg.vocab, (a.ctx,), generator=g).tolist()
    nll, n = 0.0, 0
    for lo in range(0, len(ids) - 1, a.ctx):
        window = ids[lo:lo + a.ctx + 1]
        if len(window) < 2:
            break
        logits = _all_logits(eng, window[:-1], a.chunk)
        lp = torch.log_softmax(logits, dim=-1)
        tgt = torch.tensor(window[1:])
        nll -= float(lp[torch.arange(len(tgt)), tgt].sum())
        n += len(tgt)
    print(json.dumps({"tokens": n, "nll_per_token": round(nll / max(n, 1), 5), "perplexity": round(math.exp(nll / max(n, 1)), 4)}))
    return 0


def cmd_det_probe(a) -> int:
    """The same prompt run several times must give bit-identical logits (reductions are in fixed order everywhere)."""
    eng = _load(a, max_ctx=1024)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=g).tolist()
    ref, diffs = None, []
    for r in range(a.runs):
        lg = _all_logits(eng, ids, a.chunk)
        if ref is None:
            ref = lg
        else:
            diffs.append(int((lg != ref).sum()))
    ok = all(d == 0 for d in diffs)
    print(json.dumps({"runs": a.runs, "positions": len(ids), "mismatching_logits_per_run": diffs, "bit_identical": ok}))
    return 0 if ok else 1


def cmd_chunk_check(a) -> int:
    eng = _load(a, max_ctx=2048)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=g).tolist()
    whole = _all_logits(eng, ids, len(ids))
    out = {}
    for c in [int(x) for x in a.chunks.split(",")]:
        lg = _all_logits(eng, ids, c)
        cos = torch.nn.functional.cosine_similarity(whole, lg, dim=1)
        out[str(c)] = {"cos_min": round(float(cos.min()), 6), "argmax_agree": round(float((whole.argmax(-1) == lg.argmax(-1)).float().mean()), 4)}
    print(json.dumps({"positions": len(ids), "vs_whole_prompt": out}))
    return 0 if all(v["cos_min"] > 0.99 for v in out.values()) else 1


def cmd_prompt_bench(a) -> int:
    from ..runtime.engine import SamplingParams
    from ..tokenizer.templates import ChatTurn
    eng = _load(a, max_ctx=4096)
    rows = []
    for p in PROMPTS:
        pf, dc = [], []
        for r in range(a.runs + 1):
            if eng.tok is not None:
                res = eng.chat([ChatTurn("user", p)], SamplingParams(max_tokens=a.max_tokens, temperature=0.0, ignore_eos=True))
            else:
                res = eng.generate([ord(ch) % eng.cfg.vocab for ch in p], SamplingParams(max_tokens=a.max_tokens, temperature=0.0, ignore_eos=True))
            if r:                                   # the first run warms caches and graphs
                pf.append(res.prefill_tok_s)
                dc.append(res.decode_tok_s)
        rows.append({"prompt": p[:32], "prefill_tok_s": round(statistics.median(pf), 1), "decode_tok_s": round(statistics.median(dc), 1)})
    print(json.dumps({"runs": a.runs, "prompts": rows, "decode_tok_s_median": round(statistics.median(r["decode_tok_s"] for r in rows), 1)}))
    return 0


def cmd_soak(a) -> int:
    from ..runtime.api import EngineLoop
    from ..runtime.engine import SamplingParams
    eng = _load(a, max_ctx=2048, max_seqs=8)
    loop = EngineLoop(eng)
    loop.start()
    g = torch.Generator().manual_seed(3)
    stats = {"ok": 0, "failed": 0, "tokens": 0}
    lock = threading.Lock()
    inflight = threading.Semaphore(a.concurrency)
    t_end = time.time() + a.seconds

    def done(res):
        with lock:
            good = res.finish_reason in ("length", "stop") and res.completion_tokens > 0
            stats["ok" if good else "failed"] += 1
            stats["tokens"] += res.completion_tokens
        inflight.release()
    while time.time() < t_end:
        inflight.acquire()
        n = int(torch.randint(8, 600, (1,), generator=g))
        ids = torch.randint(0, eng.cfg.vocab, (n,), generator=g).tolist()
        loop.submit(ids, SamplingParams(max_tokens=int(torch.randint(4, 64, (1,), generator=g)), temperature=0.0, ignore_eos=True), None, done)
    for _ in range(a.concurrency):
        inflight.acquire()
    loop.stop()
    print(json.dumps({"seconds": a.seconds, "completions": stats["ok"], "failures": stats["failed"], "tokens_out": stats["tokens"],
                      "completions_per_hour": round(stats["ok"] * 3600 / a.seconds)}))
    return 0 if stats["failed"] == 0 else 1


def _dump(a, device):
    """Per-layer activations of one prompt: the mixer output, the FFN output and the residual stream after every layer."""
    import copy
    b = copy.copy(a)
    b.device = device
    eng = _load(b, max_ctx=2048)
    if a.tokens:
        ids = [int(t) for t in open(a.tokens).read().split()]
    else:
        g = torch.Generator().manual_seed(4)
        ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=g).tolist()
    m = eng.model
    taps: dict = {}

    def tap(li, mixer, ffn, resid):
        if not (torch.is_tensor(mixer) and torch.is_tensor(ffn)):
            raise RuntimeError("layer dumps need a single-rank model (pending fused reductions are not tensors)")
        d = taps.setdefault(li, {"mixer": [], "ffn": [], "resid": []})
        d["mixer"].append(mixer.float().cpu())
        d["ffn"].append(ffn.float().cpu())
        d["resid"].append((resid.float() + ffn.float() * eng.cfg.residual_scale).cpu())
    m.tap = tap
    try:
        logits = _all_logits(eng, ids, a.chunk)
    finally:
        m.tap = None
    layers = [{k: torch.cat(v)[:len(ids)] for k, v in taps[li].items()} for li in sorted(taps)]
    return {"ids": ids, "device": str(device), "arch": eng.cfg.arch, "layers": layers, "logits": logits}


def _diff(da, db, threshold):
    if da["ids"] != db["ids"]:
        raise SystemExit("the two dumps were made from different prompts")
    rows, first_bad = [], None
    cosf = torch.nn.functional.cosine_similarity
    for li, (la, lb) in enumerate(zip(da["layers"], db["layers"])):
        r = {"layer": li}
        for k in ("mixer", "ffn", "resid"):
            c = cosf(la[k], lb[k], dim=1)
            r[k + "_cos_min"] = round(float(c.min()), 6)
            r[k + "_max_abs"] = round(float((la[k] - lb[k]).abs().max()), 5)
        if first_bad is None and r["resid_cos_min"] < threshold:
            first_bad = li
        rows.append(r)
    c = cosf(da["logits"], db["logits"], dim=1)
    return {"layers": rows, "first_layer_below_threshold": first_bad, "threshold": threshold, "logits_cos_min": round(float(c.min()), 6),
            "argmax_agree": round(float((da["logits"].argmax(-1) == db["logits"].argmax(-1)).float().mean()), 4)}


def cmd_layer_dump(a) -> int:
    d = _dump(a, a.device)
    torch.save(d, a.out)
    print(json.dumps({"out": a.out, "layers": len(d["layers"]), "positions": len(d["ids"]), "device": d["device"]}))
    return 0


def cmd_layer_diff(a) -> int:
    r = _diff(torch.load(a.a, weights_only=False), torch.load(a.b, weights_only=False), a.threshold)
    print(json.dumps(r if a.verbose else {k: v for k, v in r.items() if k != "layers"} | {"worst_layer": min(r["layers"], key=lambda x: x["resid_cos_min"])}))
    return 0 if r["first_layer_below_threshold"] is None else 1


def cmd_layer_parity(a) -> int:
    """The same checkpoint on the CUDA kernels and on the fp32 PyTorch path, compared layer by layer."""
    if not a.gguf:
        raise SystemExit("layer-parity needs --gguf (both runs must load identical weights)")
    other = "cuda" if torch.cuda.is_available() else "cpu"
    r = _diff(_dump(a, "cpu"), _dump(a, other), a.threshold)
    print(json.dumps({"against": other} | {k: v for k, v in r.items() if k != "layers"} | {"worst_layer": min(r["layers"], key=lambda x: x["resid_cos_min"])}))
    return 0 if r["first_layer_below_threshold"] is None else 1


def cmd_spec_accept(a) -> int:
    """Self-speculative decoding: acceptance of the model's own draft head, and decode tokens/s as a function of acceptance.  The
    speed-up curve is measured, not modelled: the head still runs every round (its cost is paid), then a fraction `p` of its draft
    positions is replaced by the true greedy continuation (known from a plain run) and the rest by a wrong token, so the verify
    forward accepts as a head of that quality would."""
    import random
    from ..runtime.engine import EngineOptions, LLMEngine, SamplingParams
    eng = _load(a, max_ctx=2048)
    m = eng.model
    if getattr(m, "mtp", None) is None:
        raise SystemExit("this model has no draft head (Qwen3-Next / Qwen3.5 files carry one; Gemma-4 takes --spec-head on ie run / serve)")
    V = m.cfg.vocab
    g = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, V, (a.prompt_n,), generator=g).tolist()
    sp = SamplingParams(max_tokens=a.max_tokens, ignore_eos=True)
    mk = lambda k: LLMEngine(m, EngineOptions(max_ctx=2048, max_batch_tokens=a.chunk, max_seqs=1, enable_prefix_cache=False, spec_k=k))

    def timed(llm, hook=None):
        seq = llm.add_request(prompt, sp)
        llm.step()                                   # prefill
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        while not seq.finished:
            if hook:
                hook(seq)
            llm.step()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        return seq.tokens[len(prompt):], (len(seq.tokens) - len(prompt) - 1) / dt
    truth, plain_tps = timed(mk(0))
    llm = mk(a.spec_k)
    own, own_tps = timed(llm)
    st = llm.stats
    rows = [{"draft": "model's own head", "acceptance": round(st["spec_accepted"] / max(st["spec_drafted"], 1), 3), "tok_s": round(own_tps, 1),
             "speedup": round(own_tps / plain_tps, 3), "lossless": own == truth}]
    real = m.mtp.draft
    for p_acc in [float(x) for x in a.accept.split(",")]:
        rnd = random.Random(5)
        llm = mk(a.spec_k)
        cur = {}

        def draft(h, tok, k, ctx=None):
            real(h, tok, k, ctx)                     # the head's cost stays in the measurement
            gpos = len(cur["seq"].tokens) - len(prompt)
            want = (list(truth[gpos:gpos + k]) + [0] * k)[:k]
            return [t if rnd.random() < p_acc else (t + 1) % V for t in want]
        m.mtp.draft = draft
        try:
            out, tps = timed(llm, hook=lambda s: cur.__setitem__("seq", s))
        finally:
            m.mtp.draft = real
        st = llm.stats
        rows.append({"draft": f"oracle, per-position hit rate {p_acc}", "acceptance": round(st["spec_accepted"] / max(st["spec_drafted"], 1), 3),
                     "tok_s": round(tps, 1), "speedup": round(tps / plain_tps, 3), "lossless": out == truth})
    print(json.dumps({"plain_tok_s": round(plain_tps, 1), "spec_k": a.spec_k, "rows": rows}))
    return 0 if all(r["lossless"] for r in rows) else 1


def cmd_kv_scale(a) -> int:
    """What the int8 KV cache (one scale per cached row) costs: teacher-forced logits of one prompt with the bf16 cache and with the
    int8 cache, cosine and arg-max agreement per position, and the negative log-likelihood of the prompt under both."""
    from ..runtime.engine import EngineOptions
    res = {}
    eng = _load(a, max_ctx=2048)
    ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=torch.Generator().manual_seed(3)).tolist()
    for dt in ("bf16", "int8"):
        res[dt] = _all_logits(type(eng)(eng.model, eng.tok, EngineOptions(max_ctx=2048, kv_dtype=dt)), ids, a.chunk)
    cos = torch.nn.functional.cosine_similarity(res["bf16"], res["int8"], dim=1)
    tgt = torch.tensor(ids[1:])
    nll = {k: float(-torch.log_softmax(v[:-1].float(), -1).gather(1, tgt[:, None]).mean()) for k, v in res.items()}
    print(json.dumps({"positions": len(ids), "cos_min": float(cos.min()), "cos_mean": float(cos.mean()),
                      "argmax_agree": float((res["bf16"].argmax(-1) == res["int8"].argmax(-1)).float().mean()), "nll_bf16": nll["bf16"], "nll_int8": nll["int8"]}))
    return 0


def cmd_partial_stack(a) -> int:
    """Logits of the model cut after its first n layers (final norm and head applied to that residual), for each n asked: two builds
    or two devices that part at layer n show it here without a per-layer dump."""
    eng = _load(a, max_ctx=2048)
    m = eng.model
    ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=torch.Generator().manual_seed(3)).tolist()
    full = list(m.layers)
    out = []
    try:
        for n in [int(x) for x in a.layers.split(",")] + [len(full)]:
            m.layers = full[:max(1, min(n, len(full)))]
            lg = _all_logits(eng, ids, a.chunk)
            out.append({"layers": len(m.layers), "logit_rms": float(lg.float().pow(2).mean().sqrt()), "argmax_checksum": int(lg.argmax(-1).sum()),
                        "last_argmax": int(lg[-1].argmax())})
    finally:
        m.layers = full
    print(json.dumps({"positions": len(ids), "cuts": out}))
    return 0


def cmd_kernel_monitor(a) -> int:
    """Per-op device time of every decode step, in dispatch order, as a feed: one table per ``--interval`` steps on stderr (first
    dispatch order, time per step, share bar) and a JSON summary at the end.  Runs the model on a fixed prompt without CUDA graphs so
    that every op is timed on its own (src: tools/ie_kernel_monitor.cpp).  On the CPU path the times are wall-clock times of the
    PyTorch restatement."""
    from ..runtime.engine import EngineOptions, LLMEngine, SamplingParams
    from ..utils.profiler import profiler
    eng = _load(a, max_ctx=2048)
    llm = LLMEngine(eng.model, EngineOptions(max_ctx=2048, max_batch_tokens=a.chunk, max_seqs=1, enable_prefix_cache=False, cuda_graphs=False,
                                             kv_dtype="int8" if a.int8_kv else "bf16"))
    ids = torch.randint(0, eng.cfg.vocab, (a.tokens_n,), generator=torch.Generator().manual_seed(7)).tolist()
    seq = llm.add_request(ids, SamplingParams(max_tokens=a.warmup + a.decode + 2, ignore_eos=True))
    while seq.n_generated < 1:
        llm.step()                                   # prefill (chunked when the prompt is longer than a chunk)
    for _ in range(a.warmup):
        llm.step()
    order, tot, win, steps = [], {}, {}, 0

    def table(acc, n):
        total = sum(v[1] for v in acc.values()) or 1.0
        lines = [f"{'op (dispatch order)':<26}{'calls/step':>11}{'us/step':>11}{'share':>8}"]
        for k in order:
            if k in acc:
                c, ms = acc[k]
                lines.append(f"{k:<26}{c / n:>11.1f}{ms / n * 1e3:>11.1f}{ms / total * 100:>7.1f}% {'#' * int(round(ms / total * 40))}")
        lines.append(f"{'TOTAL':<26}{'':>11}{total / n * 1e3:>11.1f}")
        return "\n".join(lines)

    for i in range(a.decode):
        profiler.start()
        llm.step()
        profiler.stop()
        for name, ms in profiler.harvest_ordered():
            if name not in tot:
                order.append(name)
            for acc in (tot, win):
                c = acc.setdefault(name, [0, 0.0])
                c[0] += 1
                c[1] += ms
        steps += 1
        if a.interval and steps % a.interval == 0:
            print(f"-- steps {steps - a.interval + 1}..{steps}\n" + table(win, a.interval), file=sys.stderr)
            win = {}
    total = sum(v[1] for v in tot.values()) or 1.0
    print(json.dumps({"steps": steps, "ms_per_step": total / max(steps, 1),
                      "ops": [{"op": k, "calls_per_step": tot[k][0] / max(steps, 1), "us_per_step": tot[k][1] / max(steps, 1) * 1e3,
                               "share": tot[k][1] / total} for k in order]}))
    return 0


def cmd_attn_profile(a) -> int:
    """Decode attention alone at a list of context lengths, on synthetic paged caches (no model): time per call with the bf16 cache and
    with the int8 cache, KV bytes per call and the rate they are read at (src: tools/ie_attn_profile.cpp)."""
    from .. import ops
    from ..models.transformer import KV_BLOCK
    dev = torch.device(a.device if (a.device != "cuda" or torch.cuda.is_available()) else "cpu")
    hq, hkv, hd = a.q_heads, a.kv_heads, a.head_dim
    rows = []
    for ctx in [int(x) for x in a.ctx.split(",")]:
        nb = (ctx + KV_BLOCK - 1) // KV_BLOCK
        q = torch.randn(1, hq, hd, device=dev).to(torch.bfloat16)
        bt = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).unsqueeze(0)
        lens = torch.tensor([ctx], dtype=torch.int32, device=dev)
        cu = torch.tensor([0, 1], dtype=torch.int32, device=dev)
        row = {"ctx": ctx}
        for mode in ([m for m in ("bf16", "int8") if a.mode in (m, "both")]):
            # a.layers caches in turn, so that one call's keys are not the previous call's cache lines
            caches = []
            for _ in range(a.layers):
                k = torch.randn(nb + 1, hkv, KV_BLOCK, hd, device=dev)
                v = torch.randn(nb + 1, hkv, KV_BLOCK, hd, device=dev)
                if mode == "int8":
                    ks, vs = k.abs().amax(-1) / 127.0, v.abs().amax(-1) / 127.0
                    caches.append(((k / ks.unsqueeze(-1)).round().to(torch.int8), (v / vs.unsqueeze(-1)).round().to(torch.int8), (ks.float().contiguous(), vs.float().contiguous())))
                else:
                    caches.append((k.to(torch.bfloat16), v.to(torch.bfloat16), None))
            call = lambda i: ops.attention(q, caches[i % a.layers][0], caches[i % a.layers][1], bt, lens, cu, 1, scale=hd ** -0.5,
                                           kv_scales=caches[i % a.layers][2], max_kv_len=ctx)
            for i in range(a.warmup):
                call(i)
            if dev.type == "cuda":
                torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(a.steps):
                call(i)
            if dev.type == "cuda":
                torch.cuda.synchronize()
            us = (time.perf_counter() - t0) / a.steps * 1e6
            kv_bytes = 2 * ctx * hkv * hd * (1 if mode == "int8" else 2) + (2 * ctx * hkv * 4 if mode == "int8" else 0)
            row[mode] = {"us_per_call": us, "kv_bytes": kv_bytes, "gb_s": kv_bytes / us / 1e3}
        rows.append(row)
    print(json.dumps({"q_heads": hq, "kv_heads": hkv, "head_dim": hd, "rows": rows}))
    return 0


def cmd_debug(a) -> int:
    """Long-running prompt loop: the model is loaded once, then commands are read from standard input, one per line:
    ``P <text>`` appends the text to the context (``T <id id ...>`` appends token ids), runs it and prints the arg-max and the top five
    tokens of the last position as one JSON line; ``R`` clears the context; ``Q`` or end of input quits (src: tools/ie_debug.cpp).
    With ``--dump FILE`` every ``P`` / ``T`` also writes the per-layer activations of the run (the format of ``layer-dump``)."""
    eng = _load(a, max_ctx=4096)
    ctx: list = []
    n = 0
    for line in (a.script.split(";") if a.script else sys.stdin):
        line = line.strip()
        if not line:
            continue
        cmd, _, rest = line.partition(" ")
        cmd = cmd.upper()
        if cmd == "Q":
            break
        if cmd == "R":
            ctx = []
            print(json.dumps({"reset": True}), flush=True)
            continue
        if cmd == "P":
            if eng.tok is None:
                print(json.dumps({"error": "this model has no tokenizer: use T <ids>"}), flush=True)
                continue
            ids = eng.tok.encode(rest, add_bos=not ctx)
        elif cmd == "T":
            try:
                ids = [int(x) for x in rest.replace(",", " ").split()]
            except ValueError:
                ids = []
            if not ids or min(ids) < 0 or max(ids) >= eng.cfg.vocab:
                print(json.dumps({"error": "T takes token ids inside the vocabulary"}), flush=True)
                continue
        else:
            print(json.dumps({"error": f"unknown command {cmd!r} (P <text> | T <ids> | R | Q)"}), flush=True)
            continue
        ctx += ids
        t0 = time.perf_counter()
        lg = _all_logits(eng, ctx, a.chunk)[-1].float()
        top = torch.topk(lg, 5)
        row = {"context_tokens": len(ctx), "argmax": int(top.indices[0]), "ms": round((time.perf_counter() - t0) * 1e3, 2),
               "top5": [{"id": int(i), "logit": round(float(v), 4), **({"text": eng.tok.decode([int(i)])} if eng.tok is not None else {})}
                        for v, i in zip(top.values, top.indices)]}
        print(json.dumps(row), flush=True)
        n += 1
    return 0


def _fingerprint(t: torch.Tensor) -> tuple:
    """Exact content fingerprint of a tensor computed on its device: the sum of its bit patterns and a position-weighted sum (int64
    arithmetic wraps, which is fine for equality)."""
    v = t.detach().contiguous().view(-1)
    v = v.view(torch.int32 if v.element_size() == 4 else (torch.int16 if v.element_size() == 2 else torch.int8)).to(torch.int64)
    w = torch.arange(v.numel(), device=v.device, dtype=torch.int64) % 8191 + 1
    return (int(v.sum()), int((v * w).sum()))


def cmd_bug_monitor(a) -> int:
    """N identical decode chains, each with its own KV blocks and recurrent-state slot, stepped side by side; after every step the
    persistent buffers of every chain (per layer: DeltaNet state and conv window, or the K and V rows; then the logits) are
    fingerprinted and compared with chain 0 in producer order.  Reports the first buffer that differs per chain and pins the first
    divergence ever seen (step, chain, buffer).  ``--batched`` runs the chains as one batch instead of one forward each, which also
    checks that a sequence does not depend on its batch neighbours.  ``--inject step,chain,layer`` flips one bit in that chain's state
    (or K rows) before that step: the self-test of the monitor."""
    from ..models.transformer import KV_BLOCK, ForwardBatch
    eng = _load(a, max_ctx=2048)
    m, cfg = eng.model, eng.cfg
    dev = m.device
    N, iters = a.chains, a.iters
    prompt = torch.randint(0, cfg.vocab, (a.tokens_n,), generator=torch.Generator().manual_seed(5)).tolist()
    T0 = len(prompt)
    nb = (T0 + iters + KV_BLOCK - 1) // KV_BLOCK
    kv = m.new_kv_cache(1 + N * nb)
    st = m.new_state(N) if hasattr(m, "new_state") else None
    tables = [torch.arange(1 + c * nb, 1 + (c + 1) * nb, dtype=torch.int32, device=dev) for c in range(N)]
    inject = tuple(int(x) for x in a.inject.split(",")) if a.inject else None

    def batch(chains, toks, pos0):
        ids, pos, slot, cu, lens = [], [], [], [0], []
        for c, t in zip(chains, toks):
            p = torch.arange(pos0, pos0 + len(t), dtype=torch.int32, device=dev)
            ids += t
            pos.append(p)
            slot.append(tables[c][(p // KV_BLOCK).long()].long() * KV_BLOCK + (p % KV_BLOCK).long())
            cu.append(cu[-1] + len(t))
            lens.append(pos0 + len(t))
        return ForwardBatch(torch.tensor(ids, dtype=torch.int32, device=dev), torch.cat(pos), torch.cat(slot), torch.stack([tables[c] for c in chains]),
                            torch.tensor(lens, dtype=torch.int32, device=dev), torch.tensor(cu, dtype=torch.int32, device=dev), max(len(t) for t in toks),
                            state_slots=torch.tensor(chains, dtype=torch.int32, device=dev), state_slots_host=list(chains),
                            q_lens_host=[len(t) for t in toks], start_host=[pos0] * len(chains), max_kv_len=max(lens))

    def step(toks, pos0):
        groups = [list(range(N))] if a.batched else [[c] for c in range(N)]
        out = [None] * N
        for g in groups:
            lg = m.forward(batch(g, [toks[c] for c in g], pos0), kv, st) if st is not None else m.forward(batch(g, [toks[c] for c in g], pos0), kv)
            for i, c in enumerate(g):
                out[c] = lg[i]
        return out

    def buffers(c, n_pos):
        """(tag, tensor) of chain c in producer order."""
        rows = tables[c][: (n_pos + KV_BLOCK - 1) // KV_BLOCK].long()
        for li in m.layer_ids if hasattr(m, "layer_ids") else range(cfg.n_layers):
            if st is not None and li in st.S:
                yield f"DN_state[{li}]", st.S[li][c]
                yield f"DN_conv[{li}]", st.conv[li][c]
            elif li in kv.k:
                yield f"KV_K[{li}]", kv.k[li][rows]
                yield f"KV_V[{li}]", kv.v[li][rows]

    first, diverged_now, t_dec = None, [], 0.0
    logits = step([prompt] * N, 0)
    toks = [[int(l.argmax())] for l in logits]
    for it in range(iters):
        pos = T0 + it
        if inject and inject[0] == it:
            _, c, li = inject
            tgt = st.S[li][c] if (st is not None and li in st.S) else kv.k[li][tables[c][0].long()]
            flat = tgt.view(-1).view(torch.int32 if tgt.element_size() == 4 else torch.int16)
            flat[0] ^= 1
        t0 = time.perf_counter()
        logits = step(toks, pos)
        if dev.type == "cuda":
            torch.cuda.synchronize()
        t_dec += time.perf_counter() - t0
        ref = [(tag, _fingerprint(t)) for tag, t in buffers(0, pos + 1)] + [("logits", _fingerprint(logits[0]))]
        diverged_now = []
        for c in range(1, N):
            mine = [(tag, _fingerprint(t)) for tag, t in buffers(c, pos + 1)] + [("logits", _fingerprint(logits[c]))]
            bad = next((tag for (tag, x), (_, y) in zip(mine, ref) if x != y), None)
            if bad is not None:
                diverged_now.append({"chain": c, "buffer": bad})
                if first is None:
                    first = {"step": it, "chain": c, "buffer": bad}
        if a.live:
            print(f"step {it:4d}  {'DIVERGED ' + json.dumps(diverged_now) if diverged_now else 'ok'}", file=sys.stderr)
        toks = [[int(l.argmax())] for l in logits]
    print(json.dumps({"chains": N, "steps": iters, "batched": bool(a.batched), "diverged": first is not None, "first_divergence": first,
                      "diverged_at_end": diverged_now, "decode_tok_s_per_chain": iters / t_dec if t_dec > 0 else None}))
    return 1 if (first is not None and not inject) else 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ie-tools")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("--gguf", default=None)
        p.add_argument("--model", default="tiny-llama")
        p.add_argument("--quant", default=None)
        p.add_argument("--device", default="cuda")
        p.add_argument("--chunk", type=int, default=512)
    p = sub.add_parser("perplexity"); common(p); p.add_argument("--text"); p.add_argument("--tokens"); p.add_argument("--ctx", type=int, default=2048)
    p = sub.add_parser("det-probe"); common(p); p.add_argument("--runs", type=int, default=3); p.add_argument("--tokens-n", type=int, default=300)
    p = sub.add_parser("chunk-check"); common(p); p.add_argument("--chunks", default="64,256"); p.add_argument("--tokens-n", type=int, default=700)
    p = sub.add_parser("prompt-bench"); common(p); p.add_argument("--runs", type=int, default=3); p.add_argument("--max-tokens", type=int, default=64)
    p = sub.add_parser("soak"); common(p); p.add_argument("--seconds", type=float, default=60); p.add_argument("--concurrency", type=int, default=4)
    p = sub.add_parser("layer-dump"); common(p); p.add_argument("--out", required=True); p.add_argument("--tokens"); p.add_argument("--tokens-n", type=int, default=96)
    p = sub.add_parser("layer-diff"); p.add_argument("a"); p.add_argument("b"); p.add_argument("--threshold", type=float, default=0.999); p.add_argument("--verbose", action="store_true")
    p = sub.add_parser("layer-parity"); common(p); p.add_argument("--tokens"); p.add_argument("--tokens-n", type=int, default=96); p.add_argument("--threshold", type=float, default=0.999)
    p = sub.add_parser("spec-accept"); common(p); p.add_argument("--spec-k", type=int, default=3); p.add_argument("--accept", default="0.0,0.5,0.8,1.0")
    p.add_argument("--prompt-n", type=int, default=256); p.add_argument("--max-tokens", type=int, default=96)
    p = sub.add_parser("kv-scale"); common(p); p.add_argument("--tokens-n", type=int, default=512)
    p = sub.add_parser("debug"); common(p); p.add_argument("--script", default="", help="commands separated by ';' instead of standard input")
    p = sub.add_parser("kernel-monitor"); common(p); p.add_argument("--decode", type=int, default=32); p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--tokens-n", type=int, default=64); p.add_argument("--interval", type=int, default=8); p.add_argument("--int8-kv", action="store_true")
    p = sub.add_parser("attn-profile"); p.add_argument("--device", default="cuda"); p.add_argument("--ctx", default="1024,4096,16384")
    p.add_argument("--steps", type=int, default=20); p.add_argument("--warmup", type=int, default=4); p.add_argument("--layers", type=int, default=10)
    p.add_argument("--mode", default="both", choices=["bf16", "int8", "both"]); p.add_argument("--q-heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=2); p.add_argument("--head-dim", type=int, default=256)
    p = sub.add_parser("bug-monitor"); common(p); p.add_argument("--chains", type=int, default=8); p.add_argument("--iters", type=int, default=32)
    p.add_argument("--tokens-n", type=int, default=24); p.add_argument("--batched", action="store_true"); p.add_argument("--inject", default="")
    p.add_argument("--live", action="store_true")
    p = sub.add_parser("partial-stack"); common(p); p.add_argument("--layers", default="1,2"); p.add_argument("--tokens-n", type=int, default=128)
    a = ap.parse_args(argv)
    if int(os.environ.get("RANK", "0")) != 0:          # multi-rank runs: one report, from rank 0
        sys.stdout = open(os.devnull, "w")
    return {"debug": cmd_debug, "kernel-monitor": cmd_kernel_monitor, "attn-profile": cmd_attn_profile, "bug-monitor": cmd_bug_monitor, "spec-accept": cmd_spec_accept, "kv-scale": cmd_kv_scale, "partial-stack": cmd_partial_stack, "layer-dump": cmd_layer_dump, "layer-diff": cmd_layer_diff, "layer-parity": cmd_layer_parity, "perplexity": cmd_perplexity, "det-probe": cmd_det_probe, "chunk-check": cmd_chunk_check, "prompt-bench": cmd_prompt_bench,
            "soak": cmd_soak}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main())
