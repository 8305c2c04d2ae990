"""EXL3 (trellis-coded) weights on the CPU: the C++ decoder against an independent bit-level numpy decoder and fixed vectors, the
128-point Hadamard transform against the explicit matrix, the three-step layer against its dense effective weight, and the file
path (synthetic GGUF with type-37 trellis tensors + suh / svh siblings -> loader -> graph -> tokens).  The reference tests its host
decode the same way against a numpy oracle (tools/ie_exl3_test.cpp, tools/exl3/make_oracle.py)."""
from dataclasses import replace

import numpy as np
import pytest
import torch

from machx_inference_engine_b200 import ops
from machx_inference_engine_b200.formats import exl3
from machx_inference_engine_b200.formats.gguf import GGMLType, GGUFReader, type_name
from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
from machx_inference_engine_b200.models.sources import SynthSource, default_policy
from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.ops.weights import WFormat, from_exl3
from machx_inference_engine_b200.runtime.api import Engine
from machx_inference_engine_b200.runtime.engine import EngineOptions, SamplingParams


def test_codebook_fixed_vectors():
    # x = code * 89226354 + 64248484; x = (x & 0x8fff8fff) ^ 0x3b603b60; value = fp16(lo) + fp16(hi) rounded to fp16
    def by_hand(code):
        x = (code * 89226354 + 64248484) & 0xFFFFFFFF
        x = (x & 0x8FFF8FFF) ^ 0x3B603B60
        h = np.array([x & 0xFFFF, x >> 16], dtype=np.uint16).view(np.float16).astype(np.float32)
        return float(np.float16(h[0] + h[1]))
    codes = np.array([0, 1, 2, 255, 4660, 32768, 65535], dtype=np.uint32)
    got = exl3.code_value_numpy(codes)
    assert [float(v) for v in got] == [by_hand(int(c)) for c in codes]
    assert by_hand(0) == pytest.approx(0.76806640625)         # 0x03d45aa4 -> 0x38b431c4: fp16 0x31c4 + fp16 0x38b4
    allv = exl3.code_value_numpy(np.arange(65536, dtype=np.uint32))
    assert abs(float(allv.mean())) < 1e-3 and float(allv.std()) == pytest.approx(exl3.CODEBOOK_STD, rel=1e-4)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_host_decoder_matches_bit_level_oracle(bits):
    g = torch.Generator().manual_seed(bits)
    tr, _, _ = exl3.random_layer(256, 384, bits, g)
    a = exl3.decode_trellis(tr).numpy()
    assert a.shape == (384, 256)
    assert np.array_equal(a, exl3.decode_trellis_numpy(tr.numpy()))
    assert np.array_equal(exl3.decode_trellis(tr, transpose=True).numpy(), a.T)


def test_single_tile_window_positions():
    # a tile whose stream is all zeros except one 16-bit window: exactly the weights whose windows overlap it change
    bits = 4
    tr = torch.zeros(1, 1, 16 * bits, dtype=torch.int16)
    base = exl3.decode_trellis(tr)
    assert float(base.min()) == float(base.max()) == pytest.approx(0.76806640625)
    tr[0, 0, 1] = -1                      # bits 0..15 of the tile (high half of the first 32-bit word)
    w = exl3.decode_trellis(tr)
    changed = int((w != base).sum())
    # windows end at (t + 1) * 4: t = 0..3 end inside bits 0..15, t = 4..6 still overlap them -> 7 weights
    assert changed == 7


def test_hadamard128_is_the_sylvester_matrix_and_its_own_inverse():
    H = torch.tensor([[1.0]])
    while H.shape[0] < 128:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    H = H / 128 ** 0.5
    x = torch.randn(5, 384)
    h = exl3.hadamard128(x)
    for b in range(3):
        assert torch.allclose(h[:, 128 * b:128 * b + 128], x[:, 128 * b:128 * b + 128] @ H, atol=1e-5)
    assert torch.allclose(exl3.hadamard128(h), x, atol=1e-5)
    assert torch.allclose(exl3.hadamard128(x.t().contiguous(), dim=0), h.t(), atol=1e-5)
    got = ref.hadamard128(x.to(torch.bfloat16), pre=torch.full((384,), 2.0), post=torch.full((384,), 0.5), bias=torch.ones(384), out_f32=True)
    assert torch.allclose(got, exl3.hadamard128(x.to(torch.bfloat16).float()) + 1.0, atol=1e-4)


def test_layer_three_steps_equal_the_effective_weight():
    g = torch.Generator().manual_seed(3)
    tr, suh, svh = exl3.random_layer(256, 384, 3, g)
    w = from_exl3(tr, suh, svh)
    assert (w.fmt, w.N, w.K, w.bits) == (WFormat.EXL3, 256, 384, 3)
    x = torch.randn(4, 384).to(torch.bfloat16)
    steps = exl3.hadamard128(exl3.hadamard128(x.float() * suh.float()) @ exl3.decode_trellis(tr)) * svh.float()
    assert torch.allclose(ref.linear(x, w, out_f32=True), steps, atol=2e-3, rtol=1e-2)
    eff = w.dequantize()[0]
    assert eff.shape == (256, 384) and 0.5 * 0.02 < float(eff.std()) < 2 * 0.02
    for bad in (lambda: w.slice_rows(0, 128), lambda: w.slice_k(0, 128), lambda: type(w).cat_rows([w, w])):
        with pytest.raises(ValueError):
            bad()


def test_synth_source_and_file_path(tmp_path):
    cfg = replace(preset("tiny-llama"), ffn=768)
    path = str(tmp_path / "exl3.gguf")
    info = write_synthetic_gguf(cfg, path, quant="exl3-3", seed=4)
    r = GGUFReader(path)
    t = r.tensor("blk.0.attn_q.weight")
    assert int(t.type) == GGMLType.EXL3 and type_name(t.type) == "EXL3" and tuple(t.dims) == (48, 16, 16)
    assert r.has_tensor("blk.0.attn_q.suh") and r.has_tensor("blk.0.ffn_down.svh") and int(r.tensor("token_embd.weight").type) == GGMLType.BF16
    assert int(r.tensor("output.weight").type) == GGMLType.EXL3
    # the loader hands the graph the same layer the file holds
    from machx_inference_engine_b200.models.sources import GGUFSource
    w = GGUFSource(r, "cpu").matrix("blk.1.ffn_down.weight", cfg.hidden, cfg.ffn)
    raw = np.frombuffer(np.array(r.tensor("blk.1.ffn_down.weight").raw(), copy=True), dtype=np.int16).reshape(cfg.ffn // 16, cfg.hidden // 16, 48)
    assert w.fmt == WFormat.EXL3 and w.bits == 3 and np.array_equal(w.p0[0].numpy(), raw)
    eng = Engine.load(path, "cpu", EngineOptions(max_ctx=256, max_seqs=1))
    res = eng.generate("Hello world", SamplingParams(max_tokens=5, temperature=0.0))
    assert res.completion_tokens >= 1 and res.token_ids == eng.generate("Hello world", SamplingParams(max_tokens=5, temperature=0.0)).token_ids
    assert info["tensors"] > 20
    # random-init source: EXL3 where the shapes allow the rotations, dense elsewhere
    src = SynthSource("cpu", default_policy("llama", "exl3"))
    assert src.matrix("blk.0.attn_q.weight", 256, 256).fmt == WFormat.EXL3
    assert src.matrix("blk.0.ffn_gate.weight", 688, 256).fmt == WFormat.BF16
    assert src.matrix("token_embd.weight", 4096, 256).fmt == WFormat.BF16


def test_import_exl3_directory(tmp_path):
    """An exllamav3-style directory (``<module>.trellis`` / ``.suh`` / ``.svh`` in safetensors, quant_method exl3) becomes a GGUF whose
    layers are the same bits, and runs."""
    import json
    import os
    from machx_inference_engine_b200.formats.hf_import import ImportError_, import_to_gguf
    from machx_inference_engine_b200.formats.safetensors import write_safetensors
    from machx_inference_engine_b200.formats.synth import gpt2_byte_map
    d = str(tmp_path)
    H, F, V, L, nh, nkv, hd = 256, 384, 384, 2, 4, 2, 64
    cfg = {"model_type": "llama", "num_hidden_layers": L, "hidden_size": H, "num_attention_heads": nh, "num_key_value_heads": nkv,
           "intermediate_size": F, "vocab_size": V, "head_dim": hd, "rope_theta": 1e4, "rms_norm_eps": 1e-5, "max_position_embeddings": 2048,
           "tie_word_embeddings": False, "quantization_config": {"quant_method": "exl3", "bits": 3.0}}
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    g = torch.Generator().manual_seed(9)
    tensors, layers = {}, {}

    def lin(name, out_f, in_f, bits):
        tr, suh, svh = exl3.random_layer(out_f, in_f, bits, g)
        tensors[name + ".trellis"], tensors[name + ".suh"], tensors[name + ".svh"] = tr.numpy(), suh.numpy(), svh.numpy()
        layers[name] = (tr, suh, svh)
    for l in range(L):
        p = f"model.layers.{l}."
        lin(p + "self_attn.q_proj", nh * hd, H, 3); lin(p + "self_attn.k_proj", nkv * hd, H, 3); lin(p + "self_attn.v_proj", nkv * hd, H, 4)
        lin(p + "self_attn.o_proj", H, nh * hd, 3); lin(p + "mlp.gate_proj", F, H, 2); lin(p + "mlp.up_proj", F, H, 2); lin(p + "mlp.down_proj", H, F, 4)
        for n in ("input_layernorm", "post_attention_layernorm"):
            tensors[p + n + ".weight"] = np.ones(H, dtype=np.float16)
    tensors["model.embed_tokens.weight"] = (np.random.default_rng(1).standard_normal((V, H)) * 0.02).astype(np.float16)
    lin("lm_head", V, H, 6)
    tensors["model.norm.weight"] = np.ones(H, dtype=np.float16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    bm = gpt2_byte_map()
    vocab = {ch: i for i, ch in enumerate(bm)}
    json.dump({"model": {"type": "BPE", "vocab": vocab, "merges": []},
               "added_tokens": [{"id": 300, "content": "<|eot|>", "special": True}]}, open(os.path.join(d, "tokenizer.json"), "w"))
    json.dump({"eos_token": "<|eot|>"}, open(os.path.join(d, "tokenizer_config.json"), "w"))
    out = str(tmp_path / "out.gguf")
    info = import_to_gguf(d, out, log=lambda s: None)
    r = GGUFReader(out)
    assert info["arch"] == "llama" and r.kv["llama.block_count"] == 2
    t = r.tensor("blk.1.ffn_down.weight")
    assert int(t.type) == GGMLType.EXL3 and tuple(t.dims) == (64, H // 16, F // 16)
    tr, suh, svh = layers["model.layers.1.mlp.down_proj"]
    assert np.array_equal(np.frombuffer(np.array(t.raw(), copy=True), dtype=np.int16).reshape(tr.shape), tr.numpy())
    assert np.array_equal(r.tensor("blk.1.ffn_down.svh").to_float32().reshape(-1), svh.float().numpy())
    assert tuple(r.tensor("output.weight").dims) == (96, V // 16, H // 16) and int(r.tensor("token_embd.weight").type) == GGMLType.F16
    eng = Engine.load(out, "cpu", EngineOptions(max_ctx=256, max_seqs=1))
    # the q projection of the loaded graph is the imported layer, rows in the file's (Hugging Face) order
    part = eng.model.layers[0]["attn"].qkv.parts[0].w            # separate projections: EXL3 layers are never concatenated
    assert part.fmt == WFormat.EXL3 and np.array_equal(part.p0[0].numpy(), layers["model.layers.0.self_attn.q_proj"][0].numpy())
    res = eng.generate("hello hello", SamplingParams(max_tokens=4, temperature=0.0))
    assert res.completion_tokens >= 1
    # a layer with another codebook is refused
    tensors["model.layers.0.mlp.up_proj.mcg"] = np.zeros(1, dtype=np.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(ImportError_):
        import_to_gguf(d, out, log=lambda s: None)
