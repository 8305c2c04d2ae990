"""Host-side format tests: codecs, GGUF container, runtime repack (CPU only).

Follows the reference's host unit tests: gguf_writer_test (round trip through the reader),
quantize_q6k_test, mxfp4_dequant_test (bit-exact decode formula), quant_soa_test (repack parity).
"""
import numpy as np
import pytest
import torch

from machx_inference_engine_b200.formats import gguf, quant
from machx_inference_engine_b200.formats.gguf import GGMLType as T
from machx_inference_engine_b200.ops import weights as W


def _rand(rows, cols, seed=0, scale=0.02):
    return np.random.default_rng(seed).normal(0, scale, (rows, cols)).astype(np.float32)


@pytest.mark.parametrize("t,tol", [(T.Q8_0, 0.01), (T.Q4_0, 0.12), (T.MXFP4, 0.15), (T.Q4_K, 0.1), (T.Q5_K, 0.05), (T.Q6_K, 0.03),
                                   (T.F16, 1e-3), (T.BF16, 4e-3)])
def test_codec_roundtrip_error(t, tol):
    x = _rand(16, 512)
    q = quant.quantize(x, t)
    assert q.size == gguf.bytes_for(t, x.size)
    y = quant.dequantize(q, t, x.size).reshape(x.shape)
    assert np.sqrt(((x - y) ** 2).mean()) / x.std() < tol


def test_mxfp4_decode_formula_bit_exact():
    # every (exponent, code) pair: value = 2^(e-127) * E2M1(code); low nibble = element j, high = j+16
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for e in (0, 1, 100, 127, 128, 200, 254):
        blk = np.zeros(17, dtype=np.uint8)
        blk[0] = e
        for j in range(16):
            blk[1 + j] = j | (((15 - j) & 15) << 4)
        y = quant.dequantize(blk, T.MXFP4, 32)
        for j in range(16):
            lo = mags[j & 7] * (-1 if j & 8 else 1)
            hi = mags[(15 - j) & 7] * (-1 if (15 - j) & 8 else 1)
            s = np.float32(2.0) ** np.float32(e - 127)
            assert y[j] == np.float32(lo) * s and y[j + 16] == np.float32(hi) * s


def test_block_sizes():
    assert (gguf.block_bytes(T.Q8_0), gguf.block_bytes(T.Q4_0), gguf.block_bytes(T.MXFP4)) == (34, 18, 17)
    assert (gguf.block_bytes(T.Q4_K), gguf.block_bytes(T.Q5_K), gguf.block_bytes(T.Q6_K)) == (144, 176, 210)


def test_quantize_rejects_ragged_rows():
    with pytest.raises(ValueError):
        quant.quantize(np.zeros((2, 688), dtype=np.float32), T.Q4_K)


def test_gguf_roundtrip_and_metadata(tmp_path):
    x = _rand(64, 512)
    q4 = quant.quantize(x, T.Q4_K)
    w = gguf.GGUFWriter()
    w.add_kv("general.architecture", "llama")
    w.add_kv("llama.block_count", 2)
    w.add_kv("llama.rope.freq_base", 500000.0)
    w.add_kv("flag", True)
    w.add_kv("big", 2 ** 40)
    w.add_kv("neg", -5)
    w.add_kv("tokenizer.ggml.tokens", ["a", 'b"c', "\n", "é", "\\"])
    w.add_kv("tokenizer.ggml.scores", [0.5, -1.25])
    w.add_kv("tokenizer.ggml.token_type", [1, 2, 3])
    w.add_tensor("blk.0.attn_q.weight", [512, 64], T.Q4_K, q4)
    w.add_tensor("output_norm.weight", [512], T.F32, lambda: x[0].copy())
    p = tmp_path / "m.gguf"
    w.write(str(p))
    with gguf.GGUFReader(str(p)) as r:
        assert r.version == 3
        assert r.kv["general.architecture"] == "llama" and r.kv["llama.block_count"] == 2 and r.kv["flag"] is True
        assert r.kv["big"] == 2 ** 40 and r.kv["neg"] == -5 and abs(r.kv["llama.rope.freq_base"] - 500000.0) < 1
        assert r.kv["tokenizer.ggml.tokens"] == ["a", 'b"c', "\n", "é", "\\"]
        assert r.kv["tokenizer.ggml.scores"] == [0.5, -1.25] and r.kv["tokenizer.ggml.token_type"] == [1, 2, 3]
        t = r.tensor("blk.0.attn_q.weight")
        assert t.dims == (512, 64) and t.shape == (64, 512) and t.type == T.Q4_K
        assert np.array_equal(t.raw(), q4)
        assert np.allclose(r.tensor("output_norm.weight").to_float32(), x[0])
        # payloads are 32-byte aligned inside the mapping
        assert r.tensor("blk.0.attn_q.weight").raw().ctypes.data % 32 == 0


def test_gguf_split_shards(tmp_path):
    a, b = _rand(4, 64, 1), _rand(4, 64, 2)
    for i, (name, arr) in enumerate([("t.a", a), ("t.b", b)], start=1):
        w = gguf.GGUFWriter()
        if i == 1:
            w.add_kv("general.architecture", "llama")
        w.add_kv("split.no", i - 1)
        w.add_kv("split.count", 2)
        w.add_kv("split.tensors.count", 2)
        w.add_tensor(name, [64, 4], T.F32, arr)
        w.write(str(tmp_path / f"m-{i:05d}-of-00002.gguf"))
    with gguf.GGUFReader(str(tmp_path / "m-00001-of-00002.gguf")) as r:
        assert len(r.shards) == 2 and set(r.tensors) == {"t.a", "t.b"}
        assert r.kv["general.architecture"] == "llama"
        assert np.allclose(r.tensor("t.b").to_float32(), b)


def test_gguf_corrupt_header_and_truncation(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUX" + b"\0" * 64)
    with pytest.raises(ValueError, match="magic"):
        gguf.GGUFReader(str(p))
    p.write_bytes(b"GGUF" + (2).to_bytes(4, "little") + b"\0" * 64)
    with pytest.raises(ValueError, match="version 3"):
        gguf.GGUFReader(str(p))
    w = gguf.GGUFWriter()
    w.add_tensor("x", [64, 4], T.F32, _rand(4, 64))
    good = tmp_path / "good.gguf"
    w.write(str(good))
    data = good.read_bytes()
    p.write_bytes(data[:-100])
    with pytest.raises(ValueError, match="past the end|truncated"):
        gguf.GGUFReader(str(p))


@pytest.mark.parametrize("t", [T.Q8_0, T.Q4_K, T.Q6_K, T.MXFP4, T.F16, T.BF16, T.F32, T.Q5_K, T.Q4_0])
def test_runtime_repack_matches_host_decoder(t):
    E, N, K = 2, 8, 512
    x = _rand(E * N, K, seed=3)
    q = quant.quantize(x, t)
    want = quant.dequantize(q, t, x.size).reshape(E, N, K)
    qw = W.from_ggml(torch.from_numpy(q.copy()), t, N, K, E)
    got = qw.dequantize().numpy()
    if t in (T.F32, T.F16, T.Q5_K, T.Q4_0):          # widened to bf16 at load
        assert np.allclose(got, want, rtol=1e-2, atol=1e-4)
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("fmt,tol", [(W.WFormat.Q8, 0.01), (W.WFormat.Q4K, 0.1), (W.WFormat.Q6K, 0.03), (W.WFormat.MXFP4, 0.15)])
def test_torch_quantisers(fmt, tol):
    w = torch.randn(2, 16, 512) * 0.02
    qw = W.from_dense(w, fmt)
    err = float((qw.dequantize() - w).norm() / w.norm())
    assert err < tol
    if fmt == W.WFormat.Q4K:       # emits native ggml blocks: the host decoder must agree
        host = quant.dequantize(qw.p0.numpy(), T.Q4_K, w.numel()).reshape(w.shape)
        assert np.allclose(host, qw.dequantize().numpy(), atol=1e-7)


def test_weight_surgery():
    w = torch.randn(1, 64, 512) * 0.05
    for fmt in W.WFormat:
        if fmt in (W.WFormat.MXF4T, W.WFormat.EXL3):       # a tiled layout made from whole MXFP4 banks: sliced before tiling (checked
            continue                                       # below); EXL3 layers are never cut (tests/test_exl3.py)
        qw = W.from_dense(w, fmt)
        full = qw.dequantize()[0]
        assert torch.equal(qw.slice_rows(16, 48).dequantize()[0], full[16:48])
        assert torch.equal(qw.slice_k(256, 512).dequantize()[0], full[:, 256:])
        g, u = qw.slice_rows(0, 32), qw.slice_rows(32, 64)
        il = W.QuantWeight.interleave_gate_up(g, u).dequantize()[0]
        assert torch.equal(il[0:16], full[0:16]) and torch.equal(il[16:32], full[32:48]) and torch.equal(il[32:48], full[16:32])
        assert torch.equal(W.QuantWeight.cat_rows([g, u]).dequantize()[0], full)
    with pytest.raises(ValueError):
        W.from_dense(w, W.WFormat.Q4K).slice_k(32, 512)


def test_mxf4_tiles_roundtrip_and_padding():
    # ragged N and K (not multiples of the 192 x 128 tile): the tiled layout decodes to the same values, experts slice, and
    # the padding holds code 0 / exponent 127; the scale atom order is row r, k-block q -> (r % 32) * 16 + (r // 32) * 4 + q
    w = W.from_dense(torch.randn(3, 200, 288) * 0.05, W.WFormat.MXFP4)
    t = W.to_mxf4_tiles(w)
    assert t.p0.shape == (3, 2, 3, 192, 64) and t.p1.shape == (3, 2, 3, 2, 512) and not t.dual
    assert torch.equal(t.dequantize(), w.dequantize())
    assert torch.equal(t.slice_experts(1, 3).dequantize(), w.dequantize()[1:3])
    back = W.from_mxf4_tiles(t)
    assert torch.equal(back.p0, w.p0) and torch.equal(back.p1[..., :9], w.p1[..., :9])
    assert int(t.p0[0, 1, :, 8:, :].max()) == 0 and int(t.p0[0, :, 2, :, 16:].max()) == 0      # rows >= 200, k >= 288
    # tile 1 row 5 = matrix row 197; k-block 9 does not exist (K = 288 = 9 blocks): its scale is the unit exponent
    assert int(t.p1[0, 1, 2, 0, 5 * 16 + 0]) == int(w.p1[0, 197, 8]) and int(t.p1[0, 1, 2, 0, 5 * 16 + 1]) == 127
    # a gated pair: tile fb holds gate rows 96 fb.. then the same up rows; rows 128..191 of a tile live in the second atom
    u = W.from_dense(torch.randn(3, 200, 288) * 0.05, W.WFormat.MXFP4)
    gu = W.to_mxf4_tiles(w, u)
    assert gu.dual and gu.p0.shape == (3, 3, 3, 192, 64)
    g2, u2 = W.from_mxf4_tiles(gu)
    assert torch.equal(g2.p0, w.p0) and torch.equal(u2.p0, u.p0)
    assert torch.equal(gu.p0[1, 1, 0, 96 + 7], u.p0[1, 96 + 7, :64]) and torch.equal(gu.p0[1, 1, 0, 7], w.p0[1, 96 + 7, :64])
    r = 96 + 40          # tile row 136 = up row 96 + 40 of tile 1 -> atom 1, row 8
    assert int(gu.p1[2, 1, 1, 1, 8 * 16 + 0 * 4 + 3]) == int(u.p1[2, 96 + 40, 7])


def test_kquant_fits_compared():
    """RMS error of the two Q4_K / Q5_K sub-block fits (alternating least squares; ggml's importance-weighted grid search) and of
    the default, which takes the better of the two per sub-block, on Gaussian and on heavy-tailed rows."""
    from machx_inference_engine_b200.formats import quant
    from machx_inference_engine_b200.formats.gguf import GGMLType
    rng = np.random.default_rng(3)
    data = {"gauss": rng.standard_normal((64, 1024)).astype(np.float32) * 0.02,
            "heavy": (rng.standard_t(3, size=(64, 1024)) * 0.02).astype(np.float32)}
    try:
        for t in (GGMLType.Q4_K, GGMLType.Q5_K):
            for name, x in data.items():
                rms = {}
                for mode in (0, 1, 2):
                    quant.set_kquant_fit(mode)
                    back = quant.dequantize(quant.quantize(x, int(t)), int(t), x.size).reshape(x.shape)
                    rms[mode] = float(np.sqrt(np.mean((back - x) ** 2)) / np.sqrt(np.mean(x ** 2)))
                # the default is at least as good as either fit alone (up to the effect of the shared 6-bit super-block scales)
                assert rms[0] <= min(rms[1], rms[2]) * 1.01, (t, name, rms)
                # both fits are sound K-quant encoders: 4-bit ~ 7-9 % relative RMS, 5-bit about half of that
                assert rms[1] < (0.10 if t == GGMLType.Q4_K else 0.05) and rms[2] < (0.10 if t == GGMLType.Q4_K else 0.05), (t, name, rms)
                print(f"{GGMLType(t).name} {name}: best-of-both {rms[0]:.4f}  alternating-LS {rms[1]:.4f}  weighted-grid {rms[2]:.4f}")
    finally:
        quant.set_kquant_fit(0)
