"""`ie import`: safetensors reader, AWQ / GPTQ decoders against independent numpy packers, and a whole
Hugging-Face-directory -> GGUF -> Engine round trip (reference tests: tests/unit/safetensors_test.cpp, awq_test.cpp,
gptq_test.cpp, hf_import_test.cpp)."""
import json
import os

import numpy as np
import pytest

from machx_inference_engine_b200.formats.gguf import GGMLType, GGUFReader
from machx_inference_engine_b200.formats.hf_import import ImportError_, hf_to_gguf_name, import_to_gguf, parse_hf_config
from machx_inference_engine_b200.formats.safetensors import (SafetensorsFile, SafetensorsModel, awq_dequant, gptq_dequant,
                                                             write_safetensors)

AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]           # logical column j of a packed word sits in nibble AWQ_ORDER[j]


def pack_awq(q):                                # q: [rows, out] ints 0..15 -> int32 [rows, out/8]
    rows, out = q.shape
    w = np.zeros((rows, out // 8), dtype=np.uint32)
    for j in range(8):
        w |= q[:, j::8].astype(np.uint32) << (4 * AWQ_ORDER[j])
    return w.view(np.int32)


def make_awq(rng, in_f, out_f, group):
    q = rng.integers(0, 16, size=(in_f, out_f))
    z = rng.integers(0, 16, size=(in_f // group, out_f))
    s = (rng.random((in_f // group, out_f)) * 0.02 + 0.001).astype(np.float16)
    dense = ((q - np.repeat(z, group, axis=0)) * np.repeat(s.astype(np.float32), group, axis=0)).T.astype(np.float32)   # [out, in]
    return pack_awq(q), pack_awq(z), s, dense


def test_safetensors_reader_and_shards(tmp_path):
    a = np.arange(24, dtype=np.float32).reshape(4, 6)
    b = (np.arange(10) * 3).astype(np.int32)
    bf = np.array([0x3F80, 0x4000, 0xBF80], dtype=np.uint16)        # 1.0, 2.0, -1.0 in bf16
    write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), {"a": a, "odd": np.array([7], dtype=np.uint8), "b": b}, {"format": "pt"})
    write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), {"c": ("BF16", bf)})
    json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00001-of-00002.safetensors",
                              "odd": "model-00001-of-00002.safetensors", "c": "model-00002-of-00002.safetensors"}},
              open(tmp_path / "model.safetensors.index.json", "w"))
    f = SafetensorsFile(str(tmp_path / "model-00001-of-00002.safetensors"))
    assert f.metadata == {"format": "pt"} and np.array_equal(f.numpy("a"), a)
    assert np.array_equal(f.numpy("b"), b)                           # payload starts at an odd offset: unaligned-safe
    m = SafetensorsModel(str(tmp_path))
    assert sorted(m.names()) == ["a", "b", "c", "odd"] and m.shape("a") == (4, 6) and m.dtype("c") == "BF16"
    assert np.array_equal(m.float32("c"), np.array([1.0, 2.0, -1.0], dtype=np.float32))
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(IOError):
        SafetensorsFile(str(bad))
    trunc = tmp_path / "trunc.safetensors"
    trunc.write_bytes(open(tmp_path / "model-00001-of-00002.safetensors", "rb").read()[:-20])
    with pytest.raises(IOError):
        SafetensorsFile(str(trunc))


def test_awq_dequant_matches_numpy():
    rng = np.random.default_rng(0)
    qw, qz, s, dense = make_awq(rng, 256, 64, 128)
    got = awq_dequant(qw, qz, s, 128)
    assert got.shape == (64, 256) and np.allclose(got, dense, atol=1e-6)
    with pytest.raises(ValueError):
        awq_dequant(qw, qz[:1], s, 128)


def test_gptq_dequant_matches_numpy():
    rng = np.random.default_rng(1)
    in_f, out_f, group = 128, 32, 32
    q = rng.integers(0, 16, size=(in_f, out_f))
    z = rng.integers(0, 15, size=(in_f // group, out_f))
    s = (rng.random((in_f // group, out_f)) * 0.02 + 0.001).astype(np.float16)
    g_idx = rng.permutation(np.repeat(np.arange(in_f // group), group)).astype(np.int32)
    qw = np.zeros((in_f // 8, out_f), dtype=np.uint32)
    for i in range(in_f):
        qw[i // 8] |= q[i].astype(np.uint32) << (4 * (i % 8))
    qz = np.zeros((in_f // group, out_f // 8), dtype=np.uint32)
    for o in range(out_f):
        qz[:, o // 8] |= z[:, o].astype(np.uint32) << (4 * (o % 8))
    for gi in (None, g_idx):
        grp = (np.arange(in_f) // group) if gi is None else gi
        want = ((q - (z[grp] + 1)) * s.astype(np.float32)[grp]).T
        got = gptq_dequant(qw.view(np.int32), qz.view(np.int32), s, group, gi)
        assert np.allclose(got, want, atol=1e-6)


def test_name_mapping_and_config_errors():
    assert hf_to_gguf_name("model.layers.12.self_attn.q_proj.qweight") == "blk.12.attn_q.qweight"
    assert hf_to_gguf_name("model.layers.3.mlp.down_proj.weight") == "blk.3.ffn_down.weight"
    assert hf_to_gguf_name("model.layers.3.post_attention_layernorm.weight") == "blk.3.ffn_norm.weight"
    assert hf_to_gguf_name("model.embed_tokens.weight") == "token_embd.weight"
    assert hf_to_gguf_name("model.layers.0.self_attn.rotary_emb.inv_freq") == ""
    base = {"model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
            "intermediate_size": 512, "vocab_size": 300}
    m = parse_hf_config(json.dumps({**base, "quantization_config": {"quant_method": "awq", "w_bit": 4, "q_group_size": 64, "version": "GEMM"}}))
    assert (m.quant_method, m.group_size, m.head_dim) == ("awq", 64, 64)
    for bad in ({"quant_method": "awq", "bits": 8}, {"quant_method": "awq", "bits": 4, "version": "gemv"}, {"quant_method": "bnb"}):
        with pytest.raises(ImportError_):
            parse_hf_config(json.dumps({**base, "quantization_config": bad}))
    with pytest.raises(ImportError_):
        parse_hf_config(json.dumps({k: v for k, v in base.items() if k != "hidden_size"}))


def _fake_hf_dir(d, awq=True):
    rng = np.random.default_rng(2)
    H, F, V, L, nh, nkv, hd, G = 256, 512, 320, 2, 4, 2, 64, 128
    cfg = {"model_type": "qwen3", "num_hidden_layers": L, "hidden_size": H, "num_attention_heads": nh, "num_key_value_heads": nkv,
           "intermediate_size": F, "vocab_size": V, "head_dim": hd, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "max_position_embeddings": 2048,
           "tie_word_embeddings": False}
    if awq:
        cfg["quantization_config"] = {"quant_method": "awq", "bits": 4, "group_size": G, "version": "gemm", "zero_point": True}
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    tensors, dense = {}, {}

    def lin(name, out_f, in_f):
        if awq:
            qw, qz, s, dn = make_awq(rng, in_f, out_f, G)
            tensors[name + ".qweight"], tensors[name + ".qzeros"], tensors[name + ".scales"] = qw, qz, s
        else:
            dn = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
            tensors[name + ".weight"] = dn.astype(np.float16)
        dense[name] = dn
    for l in range(L):
        p = f"model.layers.{l}."
        lin(p + "self_attn.q_proj", nh * hd, H); lin(p + "self_attn.k_proj", nkv * hd, H); lin(p + "self_attn.v_proj", nkv * hd, H)
        lin(p + "self_attn.o_proj", H, nh * hd); lin(p + "mlp.gate_proj", F, H); lin(p + "mlp.up_proj", F, H); lin(p + "mlp.down_proj", H, F)
        for n in ("input_layernorm", "post_attention_layernorm"):
            tensors[p + n + ".weight"] = np.ones(H, dtype=np.float16)
        for n in ("self_attn.q_norm", "self_attn.k_norm"):
            tensors[p + n + ".weight"] = np.ones(hd, dtype=np.float16)
    tensors["model.embed_tokens.weight"] = (rng.standard_normal((V, H)) * 0.02).astype(np.float16)
    tensors["lm_head.weight"] = (rng.standard_normal((V, H)) * 0.02).astype(np.float16)
    tensors["model.norm.weight"] = np.ones(H, dtype=np.float16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    from machx_inference_engine_b200.formats.synth import gpt2_byte_map
    bm = gpt2_byte_map()
    vocab = {ch: i for i, ch in enumerate(bm)}
    vocab["he"] = 256; vocab["ll"] = 257
    json.dump({"model": {"type": "BPE", "vocab": vocab, "merges": ["h e", ["l", "l"]]},
               "added_tokens": [{"id": 300, "content": "<|im_start|>", "special": True}, {"id": 301, "content": "<|im_end|>", "special": True},
                                {"id": 302, "content": "<|endoftext|>", "special": True}]}, open(os.path.join(d, "tokenizer.json"), "w"))
    json.dump({"eos_token": "<|im_end|>", "pad_token": {"content": "<|endoftext|>"}, "chat_template": "{{ '<|im_start|>' }}"},
              open(os.path.join(d, "tokenizer_config.json"), "w"))
    return cfg, dense


@pytest.mark.parametrize("awq", [True, False])
def test_import_directory_to_gguf_and_run(tmp_path, awq):
    d = str(tmp_path)
    cfg, dense = _fake_hf_dir(d, awq)
    out = str(tmp_path / "out.gguf")
    info = import_to_gguf(d, out, stream=True, log=lambda s: None)
    r = GGUFReader(out)
    assert info["arch"] == "qwen3" and r.kv["qwen3.block_count"] == 2 and len(r.kv["tokenizer.ggml.tokens"]) == 320
    assert r.kv["tokenizer.ggml.eos_token_id"] == 301 and r.kv["tokenizer.ggml.merges"] == ["h e", "l l"]
    t = r.tensor("blk.1.ffn_down.weight")
    assert t.type == GGMLType.Q4_K and tuple(t.dims) == (512, 256)
    assert r.tensor("token_embd.weight").type == GGMLType.Q6_K and r.tensor("blk.0.attn_norm.weight").type == GGMLType.F32
    want = dense["model.layers.1.mlp.down_proj"]
    got = t.to_float32()
    assert got.shape == want.shape
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 0.12, err                                          # Q4_K re-encoding error of a 4-bit source
    from machx_inference_engine_b200.runtime.api import Engine
    from machx_inference_engine_b200.runtime.engine import EngineOptions, SamplingParams
    eng = Engine.load(out, "cpu", EngineOptions(max_ctx=256, max_seqs=1))
    assert eng.tok.encode("hello", add_bos=False) == [256, 257, ord("o")]    # 'he' 'll' 'o' merges from tokenizer.json
    res = eng.generate("hello hello", SamplingParams(max_tokens=4, temperature=0.0))
    assert res.completion_tokens >= 1


def test_import_tokenizer_from_reference_gguf_is_padded(tmp_path):
    from machx_inference_engine_b200.formats.model_config import preset
    from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
    d = str(tmp_path / "hf"); os.makedirs(d)
    _fake_hf_dir(d, awq=False)
    os.remove(os.path.join(d, "tokenizer.json"))
    with pytest.raises(ImportError_):
        import_to_gguf(d, str(tmp_path / "x.gguf"), log=lambda s: None)
    ref = str(tmp_path / "ref.gguf")
    c = preset("tiny-qwen3"); c.vocab = 300                              # smaller than the 320 embedding rows
    write_synthetic_gguf(c, ref, quant="q8_0")
    out = str(tmp_path / "out.gguf")
    import_to_gguf(d, out, tokenizer_gguf=ref, log=lambda s: None)
    toks = GGUFReader(out).kv["tokenizer.ggml.tokens"]
    assert len(toks) == 320 and toks[-1] == "[PAD319]"
