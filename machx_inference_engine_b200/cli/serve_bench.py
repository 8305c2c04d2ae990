"""Concurrent-serving benchmark: N requests with random-token prompts arrive at once at the engine loop (the layer the
HTTP handlers call), every request decodes a fixed number of tokens; reports TTFT percentiles and aggregate throughput.

    python -m machx_inference_engine_b200.cli.serve_bench --model gpt-oss-120b --requests 64 --min-prompt 256 --max-prompt 4096 --decode 256
    torchrun --nproc-per-node 8 -m machx_inference_engine_b200.cli.serve_bench --model gpt-oss-120b ...      (SPMD: rank 0 drives)

The reference serves one request at a time (src/server/openai_server.cpp:25) and publishes no concurrent-serving number;
this tool measures the continuous-batching path.  Prompts are token ids (the model is random-init, so there is no text to
tokenize); TTFT is arrival -> first token as seen by the engine loop; wall time is first arrival -> last completion.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="serve-bench")
    ap.add_argument("--gguf", default=None)
    ap.add_argument("--model", default="gpt-oss-120b")
    ap.add_argument("--quant", default=None)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--min-prompt", type=int, default=256)
    ap.add_argument("--max-prompt", type=int, default=4096)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--chunk", type=int, default=4096, help="prefill token budget per step")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--baseline-comm", action="store_true")
    a = ap.parse_args(argv)

    from ..formats.model_config import preset
    from ..models import build_model, load_model
    from ..parallel.comm import init_from_env
    from ..runtime.api import Engine, EngineLoop
    from ..runtime.engine import EngineOptions, SamplingParams

    cuda = a.device.startswith("cuda")
    par = init_from_env("cuda" if cuda else "cpu")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
        if par.world > 1 and not a.baseline_comm:
            from ..parallel.fused import FusedComm
            par.fused = FusedComm.create(par, dev, max_tokens=a.chunk)
    max_ctx = ((a.max_prompt + a.decode + 16 + 127) // 128) * 128
    if a.gguf:
        model, _ = load_model(a.gguf, dev, par, max_ctx=max_ctx)
    else:
        cfg = preset(a.model)
        model = build_model(cfg, dev, par, quant=a.quant or ("mxfp4" if cfg.arch == "gpt-oss" else "q4_k_m" if cfg.arch == "llama" else "q8_0"),
                            max_ctx=max_ctx)
    cfg = model.cfg
    eng = Engine(model, None, EngineOptions(max_ctx=max_ctx, max_batch_tokens=a.chunk, max_seqs=a.requests, enable_prefix_cache=False))
    loop = EngineLoop(eng, par)
    if par.rank != 0:
        loop.run()
        os._exit(0)

    g = torch.Generator().manual_seed(a.seed)
    lens = torch.randint(a.min_prompt, a.max_prompt + 1, (a.requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in lens]
    sp = SamplingParams(max_tokens=a.decode, temperature=0.0, ignore_eos=True)
    # warm-up: one short request end to end (kernel attributes, graphs for batch 1)
    loop.start()
    ev = threading.Event()
    loop.submit(prompts[0][:64], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True), None, lambda r: ev.set())
    ev.wait(600)
    results, done = [], threading.Event()
    lock = threading.Lock()

    def on_done(res):
        with lock:
            results.append(res)
            if len(results) == a.requests:
                done.set()
    if cuda:
        torch.cuda.synchronize()
    t0 = time.perf_counter()
    for p in prompts:
        loop.submit(p, sp, None, on_done)
    done.wait(3600)
    wall = time.perf_counter() - t0
    loop.stop()
    loop.join(60)
    ttft = sorted(r.ttft_s for r in results)
    gen = sum(r.completion_tokens for r in results)
    pin = sum(r.prompt_tokens for r in results)
    pct = lambda q: ttft[min(len(ttft) - 1, int(q * len(ttft)))]
    steps = eng.llm.stats
    out = {"bench": "concurrent serving", "model": a.model if not a.gguf else a.gguf, "n_gpus": par.world, "requests": a.requests,
           "prompt_tokens": pin, "generated_tokens": gen, "wall_s": round(wall, 3), "ttft_p50_s": round(pct(0.5), 3), "ttft_p90_s": round(pct(0.9), 3),
           "ttft_max_s": round(ttft[-1], 3), "aggregate_decode_tok_s": round(gen / wall, 1), "aggregate_total_tok_s": round((gen + pin) / wall, 1),
           "engine_steps": steps["steps"], "graph_replays": steps["graph_replays"], "errors": sum(1 for r in results if r.finish_reason not in ("length", "stop")),
           "comm": ("nccl-baseline" if a.baseline_comm else "fused") if par.world > 1 else "none"}
    print(json.dumps(out))
    sys.stdout.flush()
    if par.world > 1:
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
