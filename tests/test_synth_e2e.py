"""Whole file path on CPU: synthesise a checkpoint -> GGUF loader -> model graph -> tokenizer -> Engine.generate/chat,
plus the placement planner, `ie inspect`, `ie pull` name resolution and split-shard loading."""
import io
import os

import pytest
import torch

from machx_inference_engine_b200.cli.inspect_gguf import inspect
from machx_inference_engine_b200.cli.pull import pull, resolve
from machx_inference_engine_b200.formats.gguf import GGUFReader
from machx_inference_engine_b200.formats.memory_plan import plan_placement
from machx_inference_engine_b200.formats.model_config import preset, read_config
from machx_inference_engine_b200.formats.synth import tensor_plan, write_synthetic_gguf
from machx_inference_engine_b200.runtime.api import Engine
from machx_inference_engine_b200.runtime.engine import EngineOptions, SamplingParams
from machx_inference_engine_b200.tokenizer.templates import ChatTurn


@pytest.fixture(scope="module")
def ckpts(tmp_path_factory):
    d = tmp_path_factory.mktemp("ckpt")
    out = {}
    for name, quant in (("tiny-llama", "q4_k_m"), ("tiny-gpt-oss", "mxfp4"), ("tiny-qwen3moe", "q8_0"), ("tiny-qwen3next", "q8_0")):
        p = str(d / f"{name}.gguf")
        write_synthetic_gguf(preset(name), p, quant=quant, seed=1)
        out[name] = p
    return out


@pytest.mark.parametrize("name", ["tiny-llama", "tiny-gpt-oss", "tiny-qwen3moe", "tiny-qwen3next"])
def test_synth_roundtrip_config_and_generate(ckpts, name):
    cfg = preset(name)
    r = GGUFReader(ckpts[name])
    got = read_config(r.kv, r.tensors.keys())
    for f in ("arch", "n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "vocab", "n_experts", "n_experts_used", "expert_ffn",
              "sliding_window", "full_attn_interval", "ssm_n_v_heads", "nextn_predict_layers"):
        assert getattr(got, f) == getattr(cfg, f), f
    assert set(r.tensors) == {t[0] for t in tensor_plan(cfg)}
    eng = Engine.load(ckpts[name], "cpu", EngineOptions(max_ctx=1024, max_seqs=2))
    res = eng.generate("Hello world, the answer is", SamplingParams(max_tokens=6, temperature=0.0))
    assert res.completion_tokens >= 1 and res.prompt_tokens > 3 and res.finish_reason in ("stop", "length")
    again = eng.generate("Hello world, the answer is", SamplingParams(max_tokens=6, temperature=0.0))
    assert again.token_ids == res.token_ids                      # greedy is deterministic
    chat = eng.chat([ChatTurn("system", "be brief"), ChatTurn("user", "hi")], SamplingParams(max_tokens=4, temperature=0.0))
    assert chat.finish_reason in ("stop", "length") and chat.error == ""


@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-phi3", "tiny-granite", "tiny-qwen35", "tiny-qwen35moe"])
def test_more_families_load_from_file_and_generate(tmp_path, name):
    """Qwen2 (q/k/v biases), Phi-3 (fused attn_qkv and gate|up tensors), Granite (embedding / residual / attention / logit
    scales) and the dense hybrid: file -> loader -> graph -> tokens; the file path equals the in-memory random-init path."""
    cfg = preset(name)
    path = str(tmp_path / "m.gguf")
    write_synthetic_gguf(cfg, path, quant="q8_0", seed=2)
    r = GGUFReader(path)
    got = read_config(r.kv, r.tensors.keys())
    for f in ("arch", "n_layers", "hidden", "n_heads", "n_kv_heads", "ffn", "embedding_scale", "residual_scale", "attention_scale"):
        assert getattr(got, f) == pytest.approx(getattr(cfg, f)), f
    if name == "tiny-granite":
        assert got.logit_scale == pytest.approx(cfg.logit_scale)
    if name == "tiny-phi3":
        assert "blk.0.attn_qkv.weight" in r.tensors and "blk.0.attn_q.weight" not in r.tensors and "blk.0.ffn_gate.weight" not in r.tensors
    eng = Engine.load(path, "cpu", EngineOptions(max_ctx=512, max_seqs=2))
    res = eng.generate("the sea and the sky", SamplingParams(max_tokens=5, temperature=0.0))
    assert res.completion_tokens >= 1 and eng.generate("the sea and the sky", SamplingParams(max_tokens=5, temperature=0.0)).token_ids == res.token_ids


def test_file_weights_equal_direct_dequant(ckpts):
    """A tensor read back through the loader decodes to the values the writer quantised."""
    from machx_inference_engine_b200.models.sources import GGUFSource
    r = GGUFReader(ckpts["tiny-gpt-oss"])
    src = GGUFSource(r, "cpu")
    cfg = preset("tiny-gpt-oss")
    w = src.matrix("blk.0.ffn_down_exps.weight", cfg.hidden, cfg.expert_ffn, cfg.n_experts)
    want = torch.from_numpy(r.tensor("blk.0.ffn_down_exps.weight").to_float32().copy())
    assert torch.equal(w.dequantize(torch.float32).reshape(want.shape), want)
    sub = src.matrix("blk.0.ffn_down_exps.weight", cfg.hidden, cfg.expert_ffn, cfg.n_experts, experts=(2, 5))
    assert torch.equal(sub.dequantize(torch.float32).reshape(3, cfg.hidden, cfg.expert_ffn), want[2:5])


def test_memory_plan_decisions(ckpts):
    p = plan_placement(ckpts["tiny-llama"], n_gpus=0, ctx=2048, avail=8, per_gpu_bytes=10 ** 12)
    assert p.n_gpus == 1 and p.fits and "fits" in p.note
    small = p.weights_bytes + p.kv_bytes + p.ws_bytes
    p2 = plan_placement(ckpts["tiny-llama"], n_gpus=0, ctx=2048, avail=8, per_gpu_bytes=p.ws_bytes + (small - p.ws_bytes) // 3)
    assert p2.n_gpus == 4 and p2.fits
    p3 = plan_placement(ckpts["tiny-llama"], n_gpus=0, ctx=2048, avail=1, per_gpu_bytes=p.ws_bytes + 10)
    assert p3.n_gpus == 1 and not p3.fits
    p4 = plan_placement(ckpts["tiny-llama"], n_gpus=16, ctx=2048, avail=8, per_gpu_bytes=10 ** 12)
    assert p4.forced and p4.n_gpus == 8
    hy = plan_placement(ckpts["tiny-qwen3next"], ctx=1024, avail=1, per_gpu_bytes=10 ** 12)
    cfg = preset("tiny-qwen3next")
    assert hy.state_bytes > 0
    assert hy.kv_bytes == 2 * (cfg.n_layers // cfg.full_attn_interval) * cfg.n_kv_heads * cfg.head_dim * 1024 * 2
    assert "GPU" in hy.describe()


def test_inspect_and_pull(ckpts, tmp_path):
    buf = io.StringIO()
    assert inspect(ckpts["tiny-qwen3moe"], tensors=True, out=buf) == 0
    text = buf.getvalue()
    assert "general.architecture = qwen3moe" in text and "blk.0.ffn_gate_exps.weight" in text and "config: arch=qwen3moe" in text
    d = os.path.dirname(ckpts["tiny-llama"])
    assert resolve("tiny-llama", d) == ckpts["tiny-llama"]
    assert resolve(ckpts["tiny-llama"], str(tmp_path)) == ckpts["tiny-llama"]
    assert pull("no-such-model", str(tmp_path)) == 1


def test_cli_synth_and_inspect(tmp_path, capsys):
    from machx_inference_engine_b200.cli.main import main
    out = str(tmp_path / "m.gguf")
    assert main(["synth", "tiny-qwen3", out, "--quant", "bf16"]) == 0
    assert main(["inspect", out]) == 0
    assert "arch=qwen3" in capsys.readouterr().out
