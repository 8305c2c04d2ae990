"""Micro-benchmarks of single kernels on model-shaped problems (CUDA events, L2-sized inputs), and the
small cases that the committed ``ncu`` summaries under ``profiles/`` were captured on.

    python -m machx_inference_engine_b200.cli.kernel_bench moe_gemm --experts 128 --tokens 2048 --topk 4 --hidden 2880 --ffn 2880
    python -m machx_inference_engine_b200.cli.kernel_bench gemm --m 2048 --n 5120 --k 2880 --fmt bf16
    python -m machx_inference_engine_b200.cli.kernel_bench gemv --n 201088 --k 2880 --fmt q8
    python -m machx_inference_engine_b200.cli.kernel_bench attention --tokens 2048 --heads 64 --kv-heads 8 --head-dim 64
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 -m machx_inference_engine_b200.cli.kernel_bench \
        allreduce --tokens 2048 --hidden 2880 --ffn 4096

Each prints achieved TFLOP/s or GB/s and the fraction of the measured peak (MEASURED_PEAKS.json when
present, otherwise the stated fallback).  Reference parity: bench/bench_{gemm_fp16,gemv_q4k,dequant,attention}.cpp.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


GRAPH_REPS = 0      # > 0: capture that many back-to-back calls in a CUDA graph and report time per call (launch gaps of an
                    # eager loop would otherwise dominate kernels of a few microseconds)


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if GRAPH_REPS > 0:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(GRAPH_REPS):
                fn()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / GRAPH_REPS)
        ts.sort()
        return ts[len(ts) // 2], ts[0]
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def report(name, ms_med, ms_min, flops=None, bytes_=None, extra=None):
    pk = peaks()
    out = {"kernel": name, "ms_median": round(ms_med, 4), "ms_min": round(ms_min, 4)}
    if flops:
        out["tflops"] = round(flops / ms_med / 1e9, 1)
        out[f"frac_of_{pk['src']}_bf16_burst"] = round(flops / ms_med / 1e9 / pk["bf16_tflops"], 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms_med / 1e6, 1)
        out[f"frac_of_{pk['src']}_hbm"] = round(bytes_ / ms_med / 1e6 / pk["hbm_gbs"], 3)
    if extra:
        out.update(extra)
    print(json.dumps(out))


def bench_allreduce(a):
    """Row-parallel projection + all-reduce + residual/RMSNorm on W ranks (run under torchrun): the fused peer-memory
    path (all-to-all stores and the reduce-scatter form) against GEMM + NCCL all-reduce + norm.  Device-timed, max over
    ranks.  The wire roofline is bytes that must leave a rank / 770 GB/s (measured peer copy, one direction)."""
    import torch.distributed as dist
    from ..ops import cuda as K
    from ..ops.weights import WFormat, from_dense
    from ..parallel.comm import init_from_env
    from ..parallel.fused import FusedComm
    par = init_from_env("cuda")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    W = par.world
    T, H, Kfull = a.tokens, a.hidden, a.ffn     # long option names only: torchrun's parser claims abbreviations like --m / --n
    Kl = Kfull // W // 64 * 64
    fc = FusedComm.create(par, dev, max_tokens=T, max_width=H)
    torch.manual_seed(par.rank)
    w = from_dense(torch.randn(1, H, Kl, device=dev) * 0.02, WFormat.BF16)
    x = (torch.randn(T, Kl, device=dev) * 0.5).to(torch.bfloat16)
    res = torch.zeros(T, H, device=dev)
    nw = torch.ones(H, device=dev)

    def timed(fn, iters=a.iters):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(iters):
            par.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]

    def fused(rs_world):
        fc.RS_MIN_WORLD = rs_world
        return timed(lambda: fc.rmsnorm(res, nw, 1e-5, fc.linear_all_reduce(x, w, None)))

    def baseline():
        def fn():
            y = K.linear(x, w, out_f32=True)
            dist.all_reduce(y)
            K.rmsnorm(res, nw, 1e-5, delta=y)
        return timed(fn)
    gemm_only = timed(lambda: K.linear(x, w))
    t_all, t_rs, t_nccl = fused(99), fused(2), baseline()
    K.check_status()
    if par.rank == 0:
        bytes_all = (W - 1) * T * H * 2                     # bf16 partial to every peer
        bytes_rs = 2 * (W - 1) * T * H * 2 // W             # rows to their owner + reduced rows back
        flops = 2.0 * T * H * Kl
        for name, ms, by in (("fused all-to-all stores", t_all, bytes_all), ("fused reduce-scatter + gather", t_rs, bytes_rs), ("gemm + NCCL all-reduce + norm", t_nccl, bytes_rs)):
            wire_ms = by / 770e9 * 1e3
            comp_ms = flops / (peaks()["bf16_tflops"] * 1e12) * 1e3
            print(json.dumps({"path": name, "ranks": W, "T": T, "H": H, "K_per_rank": Kl, "ms": round(ms, 4), "gemm_alone_ms": round(gemm_only, 4),
                              "wire_bytes_per_rank": by, "roofline_ms": round(max(wire_ms, comp_ms), 4),
                              "fraction_of_roofline": round(max(wire_ms, comp_ms) / ms, 3)}))
    sys.stdout.flush()
    par.barrier()
    torch.cuda.synchronize()
    os._exit(0)


def main(argv=None):
    from ..ops import cuda as K
    from ..ops import ref
    from ..ops.weights import WFormat, from_dense

    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "moe_gemm", "gemv", "expert_gemv", "attention", "rmsnorm", "deltanet", "allreduce"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=2880)
    ap.add_argument("--fmt", default="bf16")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--topk", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=2880)
    ap.add_argument("--ffn", type=int, default=2880)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=0)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--graph-reps", type=int, default=0, help="time N back-to-back calls inside one CUDA graph (per-call time without launch gaps)")
    ap.add_argument("--bf16-wide", type=int, default=None, help="gemv over bf16 weights: 1 = eight consumer warps per CTA, 0 = four")
    ap.add_argument("--no-tma", action="store_true", help="gemv: chunked rows through one bulk copy per row instead of tiled TMA loads")
    ap.add_argument("--gated", action="store_true", help="gemv: the rows are 16-row interleaved gate / up pairs and the epilogue is SwiGLU")
    ap.add_argument("--gemv-path", default="auto", choices=["auto", "register", "stream"], help="which decode GEMV kernel to time")
    ap.add_argument("--decode-once", action="store_true", help="gemm: time ops.linear (weight decoded once to bf16 + TMA-fed kernel)")
    ap.add_argument("--layers", type=int, default=1, help="distinct weight copies cycled through so that weights are never L2-resident")
    a = ap.parse_args(argv)
    if a.kernel == "allreduce":
        return bench_allreduce(a)
    dev = torch.device("cuda:0")
    K.set_gemv_path(a.gemv_path)
    K.set_gemv_tma(not a.no_tma)
    if a.bf16_wide is not None:
        K.set_gemv_bf16_wide(bool(a.bf16_wide))
    global GRAPH_REPS
    GRAPH_REPS = a.graph_reps
    exl3_bits = int(a.fmt[5:]) if a.fmt.startswith("exl3-") else (4 if a.fmt == "exl3" else 0)
    fmt = WFormat.EXL3 if exl3_bits else {"bf16": WFormat.BF16, "q8": WFormat.Q8, "q4k": WFormat.Q4K, "q6k": WFormat.Q6K, "mxfp4": WFormat.MXFP4,
                                          "mxf4t": WFormat.MXFP4}[a.fmt]
    torch.manual_seed(0)

    def weight(N, Kd, E=1):
        if exl3_bits:       # (gemv / gemm --decode-once: the layer's three steps, Hadamard transforms included)
            from ..formats import exl3
            from ..ops.weights import from_exl3
            return from_exl3(*exl3.random_layer(N, Kd, exl3_bits, torch.Generator(device=dev).manual_seed(N + Kd))).to(dev)
        parts = [from_dense(torch.randn(1, N, Kd, device=dev) * 0.02, fmt) for _ in range(E)]
        if E == 1:
            return parts[0]
        from ..ops.weights import QuantWeight
        planes = [None if parts[0].planes()[i] is None else torch.cat([p.planes()[i] for p in parts], 0).contiguous() for i in range(4)]
        return QuantWeight(fmt, N, Kd, E, *planes)

    if a.kernel == "gemm":
        ws = [weight(a.n, a.k) for _ in range(a.layers)]
        x = (torch.randn(a.m, a.k, device=dev) * 0.5).to(torch.bfloat16)
        i = [0]

        def fn():
            if a.decode_once:         # the model's `linear`: quantised weight decoded once to bf16, then the TMA-fed kernel
                K.linear(x, ws[i[0] % a.layers])
            else:                     # the tcgen05 kernel with in-kernel weight decode
                K.gemm(x, ws[i[0] % a.layers], bn=a.bn or None)
            i[0] += 1
        med, mn = timeit(fn, a.iters)
        report(f"gemm[{a.fmt}{', decode-once' if a.decode_once else ''}] {a.m}x{a.n}x{a.k}", med, mn, flops=2.0 * a.m * a.n * a.k, bytes_=ws[0].nbytes + x.numel() * 2 + a.m * a.n * 2)
    elif a.kernel == "moe_gemm" and a.fmt == "mxf4t":
        # the block-scaled tensor-core kernel: MXFP4 tiles x MXFP8 activations (a.layers distinct banks keep the weights out of L2)
        from ..ops.weights import to_mxf4_tiles
        T, E, H, F, k = a.tokens, a.experts, a.hidden, a.ffn, a.topk
        banks = [(to_mxf4_tiles(weight(F, H, E), weight(F, H, E)), to_mxf4_tiles(weight(H, F, E))) for _ in range(a.layers)]
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        idx, w = K.moe_route(torch.randn(T, E, device=dev), None, k)
        pair = T <= 8
        i = [0]
        if pair:
            n = T * k
            quant = lambda: K.moe_quant(x, n, n, 1, x_div=k)
            kw = dict(default_valid=1)
            args = (idx.reshape(-1), n, 1)
        else:
            pk = K.moe_pack(idx, E)
            mt = pk.tile_expert.numel()
            quant = lambda: K.moe_quant(x, pk.max_rows, mt, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
            kw = dict(tile_valid=pk.tile_valid, num_tiles=pk.num_tiles)
            args = (pk.tile_expert, mt, 128)
        xq, sfx = quant()
        aq, sfa = K.mxf4_gemm(banks[0][0], xq, sfx, *args, act=ref.ACT_SWIGLU_OAI, **kw)

        def f_gu():
            K.mxf4_gemm(banks[i[0] % a.layers][0], xq, sfx, *args, act=ref.ACT_SWIGLU_OAI, **kw)
            i[0] += 1

        def f_dn():
            K.mxf4_gemm(banks[i[0] % a.layers][1], aq, sfa, *args, **kw)
            i[0] += 1
        touched = min(E, T * k) / E if pair else 1.0
        med, mn = timeit(f_gu, a.iters)
        report(f"moe gate+up[mxf4 block-scaled] T={T} E={E} top{k} 2x{F}x{H}", med, mn, flops=2.0 * T * k * 2 * F * H,
               bytes_=banks[0][0].nbytes * touched)
        med, mn = timeit(f_dn, a.iters)
        report(f"moe down[mxf4 block-scaled] T={T} E={E} top{k} {H}x{F}", med, mn, flops=2.0 * T * k * F * H, bytes_=banks[0][1].nbytes * touched)
        med, mn = timeit(quant, a.iters)
        report(f"moe activation quantiser T={T} top{k} H={H}", med, mn, bytes_=T * k * H * 3.0)
        K.check_status()
    elif a.kernel == "moe_gemm":
        T, E, H, F, k = a.tokens, a.experts, a.hidden, a.ffn, a.topk
        gu = weight(2 * F, H, E)
        dn = weight(H, F, E)
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        idx, w = K.moe_route(torch.randn(T, E, device=dev), None, k)
        pk = K.moe_pack(idx, E)
        f16 = False
        mid = torch.float16 if f16 else torch.bfloat16
        xp = K.moe_gather(x, pk, f16=f16)
        hmid = K.grouped_linear(xp, gu, pk.tile_expert, pk.num_tiles, act=ref.ACT_SWIGLU_OAI, out_dtype=mid)
        med, mn = timeit(lambda: K.grouped_linear(xp, gu, pk.tile_expert, pk.num_tiles, act=ref.ACT_SWIGLU_OAI, out_dtype=mid), a.iters)
        tiles = int(pk.num_tiles[0])
        report(f"moe gate_up[{a.fmt}] T={T} E={E} top{k} {2 * F}x{H}", med, mn, flops=2.0 * T * k * 2 * F * H, bytes_=gu.nbytes,
               extra={"m_tiles": tiles, "padded_rows": int(pk.num_tiles[1])})
        med, mn = timeit(lambda: K.grouped_linear(hmid, dn, pk.tile_expert, pk.num_tiles), a.iters)
        report(f"moe down[{a.fmt}] T={T} E={E} top{k} {H}x{F}", med, mn, flops=2.0 * T * k * F * H, bytes_=dn.nbytes)
    elif a.kernel == "gemv":
        ws = [weight(a.n, a.k) for _ in range(max(a.layers, 2))]
        x = torch.randn(1, a.k, device=dev).to(torch.bfloat16)
        i = [0]

        def fn():
            K.linear(x, ws[i[0] % len(ws)], act=ref.ACT_SWIGLU if a.gated else ref.ACT_NONE)
            i[0] += 1
        med, mn = timeit(fn, a.iters)
        report(f"gemv[{a.fmt}{' gated' if a.gated else ''}] {a.n}x{a.k}", med, mn, bytes_=ws[0].nbytes)
    elif a.kernel == "expert_gemv":
        E, H, F, k = a.experts, a.hidden, a.ffn, a.topk
        gu = weight(2 * F, H, E)
        x = torch.randn(1, H, device=dev).to(torch.bfloat16)
        se = torch.randperm(E, device=dev)[:k].to(torch.int32)
        med, mn = timeit(lambda: K.expert_gemv(x, gu, se, x_div=k, act=ref.ACT_SWIGLU_OAI), a.iters)
        report(f"expert_gemv gate_up[{a.fmt}] top{k} {2 * F}x{H}", med, mn, bytes_=gu.nbytes // E * k)
        dn = weight(H, F, E)
        h = torch.randn(k, F, device=dev).to(torch.bfloat16)
        med, mn = timeit(lambda: K.expert_gemv(h, dn, se, x_div=1), a.iters)
        report(f"expert_gemv down[{a.fmt}] top{k} {H}x{F}", med, mn, bytes_=dn.nbytes // E * k)
    elif a.kernel == "attention":
        T, nq, nkv, hd = a.tokens, a.heads, a.kv_heads, a.head_dim
        ctx = a.ctx or T
        nblk = (ctx + 127) // 128
        kc = torch.randn(nblk + 1, nkv, 128, hd, device=dev).to(torch.bfloat16)
        vc = torch.randn(nblk + 1, nkv, 128, hd, device=dev).to(torch.bfloat16)
        bt = torch.arange(1, nblk + 1, dtype=torch.int32, device=dev).unsqueeze(0)
        q = torch.randn(T, nq, hd, device=dev).to(torch.bfloat16)
        sl = torch.tensor([ctx], dtype=torch.int32, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        sinks = torch.zeros(nq, device=dev)
        med, mn = timeit(lambda: K.attention(q, kc, vc, bt, sl, cu, T, sinks=sinks, window=a.window), a.iters)
        # causal: each query attends to (ctx - T + its index + 1) keys; window clips that
        keys = sum(min(ctx - T + i + 1, a.window or 10 ** 9) for i in range(T))
        report(f"attention T={T} ctx={ctx} nq={nq} nkv={nkv} hd={hd} window={a.window}", med, mn, flops=4.0 * keys * nq * hd,
               bytes_=2 * ctx * nkv * hd * 2 + 2 * T * nq * hd * 2)
    elif a.kernel == "rmsnorm":
        x = torch.randn(a.m, a.k, device=dev)
        d = torch.randn(a.m, a.k, device=dev).to(torch.bfloat16)
        w = torch.ones(a.k, device=dev)
        med, mn = timeit(lambda: K.rmsnorm(x, w, 1e-5, delta=d), a.iters)
        report(f"rmsnorm {a.m}x{a.k}", med, mn, bytes_=a.m * a.k * (4 + 4 + 2 + 2))
    elif a.kernel == "deltanet":
        # Qwen3-Next layer geometry by default: 16 k-heads, 32 v-heads of width 128, conv kernel 4
        T, n_k, n_v, Dh = a.tokens, a.kv_heads * 2 if a.kv_heads != 8 else 16, a.heads if a.heads != 64 else 32, 128
        Cc = (2 * n_k + n_v) * Dh
        xin = torch.randn(T, Cc, device=dev).to(torch.bfloat16)
        cw = torch.randn(Cc, 4, device=dev)
        cst = torch.zeros(1, 3, Cc, dtype=torch.bfloat16, device=dev)
        slots = torch.zeros(1, dtype=torch.int32, device=dev)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        med, mn = timeit(lambda: K.conv1d_silu(xin, cw, cst, slots, cu, T), a.iters)
        report(f"conv1d_silu T={T} C={Cc}", med, mn, bytes_=2 * T * Cc * 2)
        ab = torch.randn(T, 2 * n_v, device=dev).to(torch.bfloat16)
        ai = torch.arange(n_v, dtype=torch.int32, device=dev)
        kv = (ai // (n_v // n_k)).to(torch.int32)
        sa, db = -torch.rand(n_v, device=dev) - 0.05, torch.zeros(n_v, device=dev)
        S = torch.zeros(1, n_v, Dh, Dh, device=dev)
        for chunked in ((False, True) if T >= 128 else (False,)):
            med, mn = timeit(lambda: K.deltanet_scan(xin, n_k, ab, ai, ai + n_v, kv, sa, db, S, slots, cu, n_v, chunked=chunked), a.iters)
            report(f"deltanet_scan[{'chunked, tensor cores' if chunked else 'sequential'}] T={T} n_k={n_k} n_v={n_v}", med, mn,
                   flops=6.0 * T * n_v * Dh * Dh, bytes_=T * Cc * 2 + T * n_v * Dh * 4, extra={"us_per_token": round(med * 1e3 / T, 3)})
        K.check_status()
    K.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
