"""``ie`` command line: ``run`` (REPL), ``serve`` (OpenAI server on :11435), ``bench`` (ie-bench), ``import``
(AWQ / GPTQ safetensors -> GGUF), ``pull`` (model fetch helper), ``inspect`` (GGUF listing), ``synth`` (write a
random-init GGUF of a named architecture).

Reference parity: src/cli/main.cpp:13-157 (sub-commands and the flags ``--ctx --port --host --gpus --int8-kv
--spec --spec-k --spec-head``; REPL commands ``/reset`` ``/quit``; ``IE_PERF`` per-turn statistics).
Multi-GPU: ``ie serve --gpus N`` re-launches itself under ``torch.distributed.run`` with one process per GPU.
"""
from __future__ import annotations

import argparse
import os
import sys


def _engine_options(a):
    from ..runtime.engine import EngineOptions
    return EngineOptions(max_ctx=a.ctx, max_batch_tokens=min(a.ctx, a.chunk), max_seqs=a.max_seqs, spec_k=a.spec_k if a.spec else 0,
                         kv_dtype="int8" if a.int8_kv else "bf16")


def _relaunch_multi_gpu(a, argv) -> int:
    """`--gpus N` with N > 1 outside torchrun: start one rank per GPU on this node."""
    import subprocess
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + os.getpid() % 1000), "-m", "machx_inference_engine_b200.cli.main", *argv]
    return subprocess.call(cmd)


def _load(a):
    import torch
    from ..parallel.comm import init_from_env
    from ..runtime.api import Engine
    cuda = torch.cuda.is_available() and not a.cpu
    par = init_from_env("cuda" if cuda else "cpu")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
        if par.world > 1:
            from ..parallel.fused import FusedComm
            par.fused = FusedComm.create(par, dev, max_tokens=min(a.ctx, a.chunk))
    from ..formats.memory_plan import plan_placement
    if par.rank == 0:
        print(plan_placement(a.model, n_gpus=max(par.world, 1), ctx=a.ctx).describe(), file=sys.stderr)
    return Engine.load(a.model, dev, _engine_options(a), par, spec_head=a.spec_head), par


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser(prog="ie")
    sub = ap.add_subparsers(dest="cmd", required=True)

    def common(p):
        p.add_argument("model")
        p.add_argument("--ctx", type=int, default=8192)
        p.add_argument("--gpus", type=int, default=0, help="0 = decide from the memory plan")
        p.add_argument("--chunk", type=int, default=4096, help="prefill chunk (tokens per step)")
        p.add_argument("--max-seqs", type=int, default=64)
        p.add_argument("--int8-kv", action="store_true", help="store K/V rows as int8 with a per-row scale (half the cache memory)")
        p.add_argument("--spec", action="store_true")
        p.add_argument("--spec-k", type=int, default=3)
        p.add_argument("--spec-head", default=None, help="draft-head GGUF for --spec (Gemma-4: the gemma4-assistant file)")
        p.add_argument("--cpu", action="store_true")

    p = sub.add_parser("run"); common(p)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--max-tokens", type=int, default=512)
    p = sub.add_parser("serve"); common(p)
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=11435)
    p = sub.add_parser("bench"); p.add_argument("rest", nargs=argparse.REMAINDER)
    p = sub.add_parser("perf", help="optimisation-loop tools: ledger / roofline / viz (cli/perf.py)"); p.add_argument("rest", nargs=argparse.REMAINDER)
    p = sub.add_parser("import"); p.add_argument("hf_dir"); p.add_argument("out"); p.add_argument("--tokenizer-gguf", default=None); p.add_argument("--stream", action="store_true")
    p = sub.add_parser("pull"); p.add_argument("name"); p.add_argument("--dir", default=os.path.expanduser("~/.cache/ie/models"))
    p = sub.add_parser("inspect"); p.add_argument("gguf"); p.add_argument("--tensors", action="store_true")
    p = sub.add_parser("synth"); p.add_argument("preset"); p.add_argument("out"); p.add_argument("--quant", default="q8_0"); p.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)

    if a.cmd == "bench":
        from .ie_bench import main as bench_main
        return bench_main(a.rest)
    if a.cmd == "perf":
        from .perf import main as perf_main
        return perf_main(a.rest)
    if a.cmd == "import":
        from ..formats.hf_import import import_to_gguf
        import_to_gguf(a.hf_dir, a.out, tokenizer_gguf=a.tokenizer_gguf, stream=a.stream)
        return 0
    if a.cmd == "pull":
        from .pull import pull
        return pull(a.name, a.dir)
    if a.cmd == "inspect":
        from .inspect_gguf import inspect
        return inspect(a.gguf, a.tensors)
    if a.cmd == "synth":
        from ..formats.synth import write_synthetic_gguf
        from ..formats.model_config import preset
        write_synthetic_gguf(preset(a.preset), a.out, quant=a.quant, seed=a.seed)
        print(f"wrote {a.out}")
        return 0

    if a.gpus == 0:
        from ..formats.memory_plan import plan_placement
        a.gpus = plan_placement(a.model, n_gpus=0, ctx=a.ctx).n_gpus
    if a.gpus > 1 and "RANK" not in os.environ:
        return _relaunch_multi_gpu(a, argv)

    eng, par = _load(a)
    if a.cmd == "serve":
        from ..server.openai_server import run_openai_server
        if par.rank != 0:
            return _follower_loop(eng, par)
        return run_openai_server(eng, eng.model_id, a.host, a.port, par=par)
    # ---- REPL
    from ..runtime.engine import SamplingParams
    from ..tokenizer.templates import ChatTurn
    turns: list = []
    perf = bool(os.environ.get("IE_PERF"))
    print("ie run: /reset clears the conversation, /quit exits", file=sys.stderr)
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        if line.strip() == "/quit":
            break
        if line.strip() == "/reset":
            turns = []
            continue
        turns.append(ChatTurn("user", line))
        res = eng.chat(turns, SamplingParams(temperature=a.temperature, max_tokens=a.max_tokens), on_text=lambda s: (sys.stdout.write(s), sys.stdout.flush()))
        print()
        turns.append(ChatTurn("assistant", res.text))
        if perf:
            print(f"[perf] ttft {res.ttft_s * 1e3:.1f} ms | prefill {res.prefill_tok_s:.1f} tok/s | decode {res.decode_tok_s:.1f} tok/s", file=sys.stderr)
    return 0


def _follower_loop(eng, par) -> int:
    """Ranks > 0 of a multi-GPU server: they execute the same steps as rank 0.  Rank 0 broadcasts every admitted request
    (token ids + sampling) before the step that first schedules it; followers mirror the scheduler deterministically."""
    from ..runtime.api import EngineLoop
    EngineLoop(eng, par).run()
    return 0


if __name__ == "__main__":
    sys.exit(main())
