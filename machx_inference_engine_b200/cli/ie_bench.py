"""``ie-bench``: prefill / decode throughput of one model, device-timed.

    python -m machx_inference_engine_b200.cli.ie_bench --gguf M.gguf --prefill 512,2048 --decode 128
    python -m machx_inference_engine_b200.cli.ie_bench --model gpt-oss-20b --quant mxfp4 --prefill 2048 --kprofile
    torchrun --nproc-per-node 8 -m machx_inference_engine_b200.cli.ie_bench --model gpt-oss-120b ...   (TP/EP over 8 GPUs)

Same protocol and TSV trailer as the reference tool (tools/ie_bench.cpp:70-453): synthetic ids
``(i*1103515245+12345) % vocab``; per prefill length: fresh state, ONE prefill forward, warm-up decodes,
N timed decodes fed with the argmax.  Differences: timing is CUDA events on the launching stream
(max over ranks) instead of host wall-clock, multi-GPU runs are supported (the reference tool is
single-GPU only), and ``--kprofile`` / ``--kprofile-decode`` print a per-op device-time table.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch


def synthetic_ids(n: int, vocab: int) -> list:
    return [(i * 1103515245 + 12345) % vocab for i in range(n)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ie-bench")
    ap.add_argument("--gguf", default=None)
    ap.add_argument("--model", default=None, help="named random-init architecture when no --gguf is given")
    ap.add_argument("--quant", default=None)
    ap.add_argument("--prefill", default="512")
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--warmup-decode", type=int, default=4)
    ap.add_argument("--repeat", type=int, default=3, help="prefill repetitions (the best is reported next to the first)")
    ap.add_argument("--kprofile", action="store_true", help="per-op device time of one prefill")
    ap.add_argument("--kprofile-decode", action="store_true", help="per-op device time of the decode steps")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--spec-k", type=int, default=0, help="MTP self-speculative decode with this draft length (models with an MTP head)")
    ap.add_argument("--int8-kv", action="store_true", help="int8 KV cache with per-row scales")
    ap.add_argument("--baseline-comm", action="store_true")
    ap.add_argument("--replicated", action="store_true", help="multi-GPU: replicated activations + fused all-reduce instead of the row-sharded prefill")
    ap.add_argument("--expert-budget-gb", type=float, default=None, help="expert banks past this many GB stay in host memory and are staged per forward")
    ap.add_argument("--device", default="cuda")
    args = ap.parse_args(argv)
    if args.expert_budget_gb is not None:
        from ..models import spill
        spill.configure(args.expert_budget_gb)

    from ..formats.model_config import preset
    from ..models import build_model, load_model
    from ..parallel.comm import init_from_env
    from ..runtime.engine import EngineOptions, LLMEngine, SamplingParams
    from ..utils.profiler import KernelProfiler, profiler

    cuda = args.device.startswith("cuda")
    par = init_from_env("cuda" if cuda else "cpu")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
        if par.world > 1 and not args.baseline_comm:
            from ..parallel.fused import FusedComm
            par.fused = FusedComm.create(par, dev)
    lens = [int(x) for x in args.prefill.split(",") if x]
    max_ctx = ((max(lens) + args.decode + args.warmup_decode + 16 + 127) // 128) * 128
    if args.gguf:
        model, _ = load_model(args.gguf, dev, par, max_ctx=max_ctx)
    else:
        cfg = preset(args.model or "tiny-llama")
        quant = args.quant or ("mxfp4" if cfg.arch == "gpt-oss" else "q4_k_m")
        model = build_model(cfg, dev, par, quant=quant, max_ctx=max_ctx)
    cfg = model.cfg
    if cuda and par.fused is not None and not args.replicated:
        from ..parallel.sharded import attach
        attach(par, dev, cfg, max(lens))                     # row-sharded prefill for chunks that divide over the ranks
    eng = LLMEngine(model, EngineOptions(max_ctx=max_ctx, max_batch_tokens=max(lens), max_seqs=1, enable_prefix_cache=False, spec_k=args.spec_k,
                                         kv_dtype="int8" if args.int8_kv else "bf16", cuda_graphs=cuda and not args.no_graphs and not args.kprofile_decode))

    def sync():
        par.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(fn):
        if not cuda:
            import time
            t0 = time.perf_counter(); fn(); return (time.perf_counter() - t0) * 1e3
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync(); e0.record(); fn(); e1.record(); sync()
        ms = e0.elapsed_time(e1)
        if par.world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    rows = []
    for P in lens:
        ids = synthetic_ids(P, cfg.vocab)
        pp = []
        for rep in range(max(1, args.repeat)):
            seq = eng.add_request(ids, SamplingParams(max_tokens=(args.decode + args.warmup_decode + 1) * (1 + args.spec_k), ignore_eos=True))
            if args.kprofile and rep == max(1, args.repeat) - 1:
                profiler.start()
            pp.append(timed(eng.step))
            if profiler.enabled:
                profiler.stop()
                if par.rank == 0:
                    print(f"# kprofile prefill T={P}\n" + KernelProfiler.format(profiler.harvest()), file=sys.stderr)
            if rep != max(1, args.repeat) - 1:
                eng.abort(seq)
        for _ in range(args.warmup_decode):
            eng.step()
        if args.kprofile_decode:
            profiler.start()

        gen0 = seq.n_generated

        def dec():
            for _ in range(args.decode):
                eng.step()
        tg = timed(dec) if args.decode > 0 else 0.0
        n_dec = max(seq.n_generated - gen0, 1)           # speculative rounds emit more than one token per step
        if args.kprofile_decode:
            profiler.stop()
            if par.rank == 0:
                print(f"# kprofile decode ctx={P} steps={args.decode}\n" + KernelProfiler.format(profiler.harvest()), file=sys.stderr)
        eng.abort(seq)
        rows.append((P, pp[0], min(pp), tg / n_dec))
        if args.spec_k and par.rank == 0:
            st = eng.stats
            print(f"# spec: {st['spec_rounds']} rounds, {st['spec_accepted']}/{st['spec_drafted']} drafts accepted, {n_dec} tokens in {args.decode} steps", file=sys.stderr)
    if par.rank == 0:
        print("# T_pp\tpp_ms\tpp_tok_s\ttg_ms_tok\ttg_tok_s\tpp_first_ms")
        for P, first, best, tgms in rows:
            print(f"{P}\t{best:.3f}\t{P / best * 1e3:.1f}\t{tgms:.3f}\t{(1e3 / tgms) if tgms > 0 else 0:.1f}\t{first:.3f}")
    sys.stdout.flush()
    if par.world > 1:
        par.barrier()
        if cuda:
            torch.cuda.synchronize()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
