#!/usr/bin/env python
"""Headline benchmark: gpt-oss-120b-architecture (MXFP4 experts, bf16 attention, random-init weights,
random-token prompts) prefill and decode throughput on N GPUs of one node, device-timed.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--model gpt-oss-120b] [--prefill 2048] [--decode 128]
    torchrun ... bench.py --gpus N ...           (N > 1: one rank per GPU, NCCL)

One timed "step" is one full prefill forward of a fresh P-token prompt (the reference's
``ie-bench --prefill P`` measurement, tools/ie_bench.cpp:281-300).  ``value`` is prefill tokens/s
aggregated over the whole job; decode tokens/s at that context (``ie-bench --decode``) is reported
next to it.  The ``e2e`` block runs the same work through the public ``LLMEngine`` API including the
host->device copy of each prompt from pinned memory and the device->host read of the sampled token.
Weights (>= 12 GB even for the 20b model) are far larger than the 126 MB L2, so every step streams
them from HBM; no explicit L2 flush is needed and none is done.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# published by the reference for this metric (gpt-oss-120b prefill, ctx <= 16k, 2x Arc B70 TP): 538-679 tok/s
BASELINE_PREFILL_TOK_S = {"gpt-oss-120b": 679.0, "gpt-oss-20b": 4147.0, "llama-3-8b": 1190.4}
BASELINE_DECODE_TOK_S = {"gpt-oss-120b": 32.05, "gpt-oss-20b": 58.3, "llama-3-8b": 43.66}


def reference_arm():
    # The reference is a C++20/SYCL (icpx, Level-Zero) project for Intel Arc with no Python packaging;
    # a pip install of its source tree fails ("neither setup.py nor pyproject.toml"), and no SYCL compiler,
    # oneAPI runtime or Intel GPU exists on this box, so its public path (ie-bench) cannot run here.
    print(json.dumps({"impl": "reference", "unavailable": "reference is C++/SYCL for Intel Arc (no setup.py/pyproject.toml; needs icpx + Level-Zero + an Intel GPU); it has no CUDA path to run on a B200"}))
    return 0


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        # nvidia-smi numbers physical GPUs and ignores CUDA_VISIBLE_DEVICES: address the device that cuda:<index> really is by
        # its UUID, so that on a shared machine the clocks reported are this process's GPU's
        self.index, self.rows, self.proc = str(index), [], None
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            self.index = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            pass

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", self.index, "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            pass
        sm, mx, reasons, pw = [], None, set(), []
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx = float(f[1]); pw.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(pw) if pw else None}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gpt-oss-120b")
    ap.add_argument("--quant", default=None)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--baseline-comm", action="store_true", help="plain NCCL all-reduce instead of the fused GEMM+all-reduce kernels")
    ap.add_argument("--pdl", type=int, default=-1, help="1/0: programmatic dependent launch for the decode chain (default: the library's setting)")
    ap.add_argument("--reduce-scatter", type=int, default=-1, help="ranks from which prefill collectives take the reduce-scatter form (default: the library's)")
    ap.add_argument("--baseline", action="store_true",
                    help="library baseline arm: the same model graph with plain PyTorch ops (cuBLAS bf16 GEMMs on decoded weights, ATen kernels) "
                         "and NCCL all-reduce; no kernel of this engine runs")
    ap.add_argument("--replicated", action="store_true", help="keep the activations replicated on every rank (fused all-reduce) instead of the row-sharded prefill")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    args.warmup = max(args.warmup, 3)

    import torch
    from machx_inference_engine_b200.formats.model_config import preset
    from machx_inference_engine_b200.models import build_model
    from machx_inference_engine_b200.ops import cuda as K
    from machx_inference_engine_b200.parallel.comm import init_from_env
    from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams

    t_start = time.time()

    def note(msg):
        if os.environ.get("MX_BENCH_VERBOSE"):
            print(f"[bench +{time.time() - t_start:6.1f}s rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)

    if args.baseline:
        from machx_inference_engine_b200 import ops as _ops
        from machx_inference_engine_b200.models.transformer import MoEFFN
        _ops.set_backend("torch")
        MoEFFN.MXF4_TENSOR_CORE = False        # bf16 activations into the experts: what a library GEMM multiplies
        args.baseline_comm = True
        args.decode = min(args.decode, 16)     # the eager per-token loop of the baseline is slow; 16 tokens time it well enough
    par = init_from_env("cuda")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if par.world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={par.world}: launch with torchrun --nproc-per-node {args.gpus}")
    if par.world > 1 and not args.baseline_comm:
        from machx_inference_engine_b200.parallel.fused import FusedComm
        par.fused = FusedComm.create(par, dev)

    if args.pdl >= 0:
        K.set_pdl(bool(args.pdl))
    if args.reduce_scatter >= 0 and par.fused is not None:
        par.fused.RS_MIN_WORLD = args.reduce_scatter
    note("process group + comm ready")
    cfg = preset(args.model)
    if par.fused is not None and not args.replicated:
        from machx_inference_engine_b200.parallel.sharded import attach
        attach(par, dev, cfg, max(args.prefill, 128 * par.world))
    quant = args.quant or ("mxfp4" if cfg.arch == "gpt-oss" else "q4_k_m" if cfg.arch == "llama" else "q8_0")
    P, D = args.prefill, args.decode
    max_ctx = ((P + D + 16 + 127) // 128) * 128
    t0 = time.time()
    model = build_model(cfg, dev, par, quant=quant, max_ctx=max_ctx, seed=0)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    note(f"model built in {build_s:.1f}s")
    if args.baseline:
        # decoded bf16 weights stay resident as far as memory allows (all of them from two GPUs up for the 120b shape); the rest
        # is decoded per call
        from machx_inference_engine_b200.ops import ref as _ref
        free, _ = torch.cuda.mem_get_info(dev)
        _ref.set_matmul_dtype(torch.bfloat16, dense_budget_bytes=max(0, free - (24 << 30)))
    eng = LLMEngine(model, EngineOptions(max_ctx=max_ctx, max_batch_tokens=max(P, 1), max_seqs=1, enable_prefix_cache=False,
                                         cuda_graphs=not args.baseline, prefill_graphs=not args.baseline))

    g = torch.Generator().manual_seed(1234)
    n_prompts = args.warmup + args.steps + 4
    prompts = [torch.randint(0, cfg.vocab, (P,), generator=g, dtype=torch.int64).tolist() for _ in range(n_prompts)]

    def barrier():
        par.barrier()
        torch.cuda.synchronize()

    def reduce_max_ms(ms: float) -> float:
        if par.world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    # ---------------- device-timed prefill: K forwards of fresh P-token prompts
    def prefill_once(i):
        seq = eng.add_request(prompts[i], SamplingParams(max_tokens=1))
        eng.step()
        return seq

    for i in range(args.warmup):
        prefill_once(i)
        note(f"warmup prefill {i} done")
    barrier()
    K.check_status()
    sampler = ClockSampler(local)       # samples through the timed prefill, the end-to-end pass and the timed decode
    sampler.start()
    time.sleep(0.35)                    # let nvidia-smi come up: a five-step region can be shorter than its first sample
    l0 = K.launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(args.steps):
        prefill_once(args.warmup + i)
    ev1.record()
    barrier()
    prefill_ms = reduce_max_ms(ev0.elapsed_time(ev1)) / args.steps
    note(f"timed prefill done: {prefill_ms:.2f} ms/step")
    launches = K.launches() - l0

    # ---------------- end-to-end prefill through the public API with host wall clock (includes H2D of ids, D2H of the token)
    h0, d0 = eng.stats["h2d_bytes"], eng.stats["d2h_bytes"]
    barrier()
    w0 = time.perf_counter()
    for i in range(args.steps):
        out = eng.generate([prompts[(args.warmup + i) % n_prompts]], SamplingParams(max_tokens=1))
    torch.cuda.synchronize()
    e2e_ms = reduce_max_ms((time.perf_counter() - w0) * 1e3) / args.steps
    note("e2e prefill done")
    h2d = (eng.stats["h2d_bytes"] - h0) // args.steps
    d2h = (eng.stats["d2h_bytes"] - d0) // args.steps

    # ---------------- decode at context P: D greedy tokens (CUDA-graphed), device-timed and end-to-end
    seq = eng.add_request(prompts[-1], SamplingParams(max_tokens=D + 8, ignore_eos=True))
    eng.step()
    for _ in range(4):
        eng.step()
    note("decode warm-up done")
    barrier()
    ev0.record()
    w0 = time.perf_counter()
    nd = 0
    while not seq.finished and nd < D:
        eng.step()
        nd += 1
    ev1.record()
    torch.cuda.synchronize()
    dec_wall_ms = reduce_max_ms((time.perf_counter() - w0) * 1e3)
    dec_ms = reduce_max_ms(ev0.elapsed_time(ev1))
    note("decode done")
    clocks = sampler.stop()
    eng.abort(seq)
    K.check_status()

    if par.rank == 0:
        value = P / (prefill_ms / 1e3)
        base = BASELINE_PREFILL_TOK_S.get(args.model)
        line = {
            "metric": f"{args.model} MXFP4 prefill tok/s (pp{P}), device-timed" if cfg.arch == "gpt-oss" else f"{args.model} {quant} prefill tok/s (pp{P}), device-timed",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(prefill_ms, 3), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / base, 2) if base else None, "dtype": "bf16", "data": "synthetic (random-init weights, random token ids)",
            "config": {"model": args.model, "global_batch": 1, "seq_len": P, "decode_tokens": D, "weights": quant,
                       "parallelism": f"tp{args.gpus}+ep{args.gpus}" if args.gpus > 1 else "tp1",
                       "comm": ("nccl-baseline" if args.baseline_comm else ("fused-gemm-allreduce" if par.sharded is None else "row-sharded: all-gather->GEMM, GEMM->reduce-scatter, expert all-to-all")) if args.gpus > 1 else "none",
                       "compute": "pytorch ops (cuBLAS bf16, ATen), no engine kernel" if args.baseline else "engine kernels (sm_100a)",
                       "l2": "inputs (weights) larger than L2; no flush", "model_build_s": round(build_s, 1),
                       "weight_gb_per_gpu": round(model.weight_bytes() / 1e9, 2)},
            "decode_tok_s": round(nd / (dec_ms / 1e3), 1), "decode_ms_per_token": round(dec_ms / max(nd, 1), 3),
            "decode_vs_baseline": round(nd / (dec_ms / 1e3) / BASELINE_DECODE_TOK_S[args.model], 2) if args.model in BASELINE_DECODE_TOK_S else None,
            "e2e": {"value": round(P / (e2e_ms / 1e3), 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "decode_tok_s": round(nd / (dec_wall_ms / 1e3), 1)},
            "gpu_launches": 0 if args.baseline else int(launches), "clocks": clocks, "impl": "library-baseline" if args.baseline else "ours",
        }
        print(json.dumps(line))
    sys.stdout.flush()
    if par.world > 1:
        # all ranks are idle here; leave without running communicator / CUDA-graph destructors, whose teardown
        # order across ranks is not defined (a captured NCCL all-gather made destroy_process_group wait for ever)
        par.barrier()
        torch.cuda.synchronize()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
