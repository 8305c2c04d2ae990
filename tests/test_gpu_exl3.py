"""EXL3 layers on the GPU: the Hadamard kernel, the trellis decoders (register GEMV and decode-to-bf16 for the tensor-core GEMM) against
the host decoder and the dense effective weight, and a model whose projections and head are EXL3 against the CPU path."""
from dataclasses import replace

import pytest
import torch

from machx_inference_engine_b200.formats import exl3
from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.ops.weights import from_exl3

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


def K():
    from machx_inference_engine_b200.ops import cuda
    return cuda


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-12))


def test_hadamard128_kernel():
    k = K()
    x = torch.randn(37, 512, device=dev())
    pre, post, bias = torch.randn(512, device=dev()), torch.randn(512, device=dev()), torch.randn(512, device=dev())
    xb = x.to(torch.bfloat16)
    got = k.hadamard128(xb, pre=pre, out_f32=True)
    assert rel_err(got, ref.hadamard128(xb.cpu(), pre=pre.cpu(), out_f32=True)) < 1e-5
    got = k.hadamard128(x, post=post, bias=bias)
    assert rel_err(got, ref.hadamard128(x.cpu(), post=post.cpu(), bias=bias.cpu())) < 4e-3          # bf16 output rounding
    # twice is the identity; a strided destination
    wide = torch.zeros(37, 1024, device=dev())
    k.hadamard128(k.hadamard128(x, out_f32=True), out_f32=True, out=wide[:, 512:])
    assert rel_err(wide[:, 512:], x) < 1e-5 and float(wide[:, :512].abs().max()) == 0.0


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 8])
def test_trellis_decode_kernels(bits):
    k = K()
    g = torch.Generator().manual_seed(bits)
    N, Kd = 384, 512
    tr, suh, svh = exl3.random_layer(N, Kd, bits, g)
    w = from_exl3(tr, suh, svh).to(dev())
    host = exl3.decode_trellis(tr, transpose=True)                       # [N, K], fp16-valued
    assert torch.equal(k.exl3_dequant(w).cpu(), host.to(torch.bfloat16))
    for M in (1, 3, 8, 100):
        x = torch.randn(M, Kd, device=dev()).to(torch.bfloat16)
        bias = torch.randn(N, device=dev())
        got = k.linear(x, w, bias=bias, out_f32=True)
        want = ref.linear(x.cpu(), w.to("cpu"), bias=bias.cpu(), out_f32=True)
        assert rel_err(got, want) < 1e-2, (bits, M)
    # into a column slice of a wider output (the way fused projections of mixed formats share one buffer)
    x = torch.randn(2, Kd, device=dev()).to(torch.bfloat16)
    wide = torch.zeros(2, N + 128, dtype=torch.bfloat16, device=dev())
    k.linear(x, w, out=wide[:, 128:])
    assert rel_err(wide[:, 128:], ref.linear(x.cpu(), w.to("cpu"))) < 1e-2 and float(wide[:, :128].abs().max()) == 0.0


def test_exl3_model_gpu_matches_cpu():
    """Every projection and the head as EXL3 layers (3 bits per weight): greedy tokens of the kernel path against the CPU oracle, with
    CUDA-graphed decode steps."""
    from machx_inference_engine_b200.models import build_model
    from machx_inference_engine_b200.ops.weights import WFormat
    from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams
    cfg = replace(preset("tiny-llama"), ffn=768)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 130, 9)]
    outs = {}
    for d in ("cpu", "cuda:0"):
        model = build_model(cfg, torch.device(d), quant="exl3-3", max_ctx=512, gen_device="cpu")
        assert model.lm_head.w.fmt == WFormat.EXL3 and model.layers[0]["ffn"].split[0].w.fmt == WFormat.EXL3
        eng = LLMEngine(model, EngineOptions(max_ctx=512, max_batch_tokens=256, max_seqs=4, cuda_graphs=True))
        outs[d] = eng.generate(prompts, SamplingParams(max_tokens=10))
    same = sum(int(a == b) for x, y in zip(outs["cpu"], outs["cuda:0"]) for a, b in zip(x, y))
    total = sum(len(x) for x in outs["cpu"])
    assert all(x[0] == y[0] for x, y in zip(outs["cpu"], outs["cuda:0"])), outs
    assert same >= 0.7 * total, outs
