"""Worker for the multi-process tests (launched with torch.distributed.run; gloo on CPU, NCCL on GPUs).

Prints one JSON line on rank 0: greedy tokens of a tiny model under tensor/expert parallelism, so the
parent test can compare them with the single-process run (the reference's multi_gpu_tp_test asks for
identical greedy tokens: tools/multi_gpu_tp_test.cpp).
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.parallel.comm import init_from_env
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams


def main():
    name, quant, device, comm = sys.argv[1], sys.argv[2], sys.argv[3], sys.argv[4]
    par = init_from_env("cuda" if device == "cuda" else "cpu", timeout_s=120)
    if comm == "pp":
        par.mode = "pp"
    if device == "cuda":
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        if comm in ("fused", "fused-rs", "sharded") and par.world > 1:
            from machx_inference_engine_b200.parallel.fused import FusedComm
            par.fused = FusedComm.create(par, dev, max_tokens=1024, max_width=4096)
            if comm == "fused-rs":          # force the reduce-scatter form (normally from 4 ranks up) so that two GPUs exercise it
                par.fused.RS_MIN_WORLD, par.fused.RS_MIN_ROWS_PER_RANK = 2, 16
    else:
        dev = torch.device("cpu")
    cfg = preset(name)
    if os.environ.get("MX_TEST_EXPERT_TP"):              # split every expert's FFN width over the ranks instead of sharding experts whole
        from machx_inference_engine_b200.models.transformer import MoEFFN
        MoEFFN.EXPERT_TP = True
    n_pre = int(os.environ.get("MX_TEST_PREFILL", "200"))     # 1024 lets the sharded path take the chunk on 2, 4 and 8 ranks
    ctx = max(1024, (n_pre + 8 + 255) // 128 * 128)
    if comm == "sharded" and par.fused is not None:      # row-sharded prefill for chunks that divide over the ranks
        from machx_inference_engine_b200.models.transformer import TransformerModel
        from machx_inference_engine_b200.parallel.sharded import attach
        attach(par, dev, cfg, ctx)
        TransformerModel.SHARD_MIN_TOKENS = 128
    model = build_model(cfg, dev, par, quant=quant, max_ctx=ctx, gen_device="cpu")
    eng = LLMEngine(model, EngineOptions(max_ctx=ctx, max_batch_tokens=512, max_seqs=4))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 260, 9)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=10))
    # teacher-forced logits of every position of one prompt: prefill chunk, then single-token steps (the decode kernels)
    from machx_inference_engine_b200.models.transformer import KV_BLOCK, ForwardBatch
    ids = prompts[1]
    ids = (ids * ((n_pre + 8) // len(ids) + 1))[: n_pre + 8]
    n_blk = (n_pre + 8 + 127) // 128
    kv = model.new_kv_cache(n_blk + 2)
    bt = torch.arange(1, n_blk + 1, dtype=torch.int32, device=dev).unsqueeze(0)

    hybrid = getattr(model, "needs_state", False)
    st = model.new_state(2) if hybrid else None

    def fwd(lo, hi):
        pos = torch.arange(lo, hi, dtype=torch.int32, device=dev)
        slot = bt[0][(pos // KV_BLOCK).long()].long() * KV_BLOCK + (pos % KV_BLOCK).long()
        fb = ForwardBatch(torch.tensor(ids[lo:hi], dtype=torch.int32, device=dev), pos, slot, bt, torch.tensor([hi], dtype=torch.int32, device=dev),
                          torch.tensor([0, hi - lo], dtype=torch.int32, device=dev), hi - lo, logit_rows=torch.arange(hi - lo, device=dev))
        if hybrid:
            fb.state_slots, fb.state_slots_host, fb.start_host = torch.tensor([1], dtype=torch.int32, device=dev), [1], [lo]
            return model.forward(fb, kv, st).float().cpu()
        return model.forward(fb, kv).float().cpu()
    logits = torch.cat([fwd(0, n_pre)] + [fwd(i, i + 1) for i in range(n_pre, n_pre + 8)])
    if comm == "pp":
        # a long single-sequence chunk goes through the stages as token micro-batches: same logits as one piece
        ids = (ids * 3)[:600]
        kv = model.new_kv_cache(8)
        bt = torch.arange(1, 7, dtype=torch.int32, device=dev).unsqueeze(0)
        whole = fwd(0, 600)
        model._micro_batches = lambda fb, min_tokens=256: [(fb, True)]
        kv = model.new_kv_cache(8)
        logits = torch.cat([logits, whole, fwd(0, 600)])
    if par.rank == 0 and len(sys.argv) > 5:
        torch.save(logits, sys.argv[5])
    if device == "cuda":
        from machx_inference_engine_b200.ops import cuda as K
        K.check_status()
    if par.rank == 0:
        print("RESULT " + json.dumps({"world": par.world, "tokens": outs}))
    sys.stdout.flush()
    if par.world > 1:
        torch.distributed.barrier()
        if device == "cuda":
            torch.cuda.synchronize()
    # leave without running the communicator / CUDA-graph destructors: nothing is in flight any more
    os._exit(0)


if __name__ == "__main__":
    main()
