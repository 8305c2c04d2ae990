"""Runtime weight layouts and the load-time repack from ggml blocks.

A :class:`QuantWeight` is a (stack of) [N, K] matrix stored in one of five runtime formats that
the sm_100a GEMV and GEMM kernels decode in registers:

========  =====================================================================================
BF16      ``p0`` bf16 [E,N,K]
Q8        ``p0`` int8 [E,N,K], ``p1`` fp16 scale [E,N,K/32]
Q4K       ``p0`` uint8 [E,N,K/256*144] -- ggml Q4_K blocks unchanged (they are 16-byte friendly)
Q6K       ``p0`` lo nibbles [E,N,K/2] (natural order), ``p1`` hi 2-bit plane [E,N,K/4] (one 32-bit
          word per 16 elements, byte b = e[2b] | e[2b+1]<<2 | e[8+2b]<<4 | e[9+2b]<<6),
          ``p2`` int8 sub-block scales [E,N,K/16], ``p3`` fp16 super scale [E,N,K/256]
MXFP4     ``p0`` E2M1 codes [E,N,K/2] (natural order: byte i = e[2i] | e[2i+1]<<4),
          ``p1`` e8m0 exponent [E,N,K/32]
MXF4T     the same codes cut into tiles of 192 rows x 128 elements, ``p0`` [E,FB,KB,192,64] (rows and K
          zero-padded to whole tiles), so that one TMA box is one contiguous 12 KiB run; ``p1`` the
          exponents as 512-byte atoms [E,FB,KB,2,512] in the order the tensor core's scale-factor
          registers want: row r, k-block q of an atom at byte (r % 32) * 16 + (r // 32) * 4 + q.
          A gated pair shares one bank: 96 gate rows + the same 96 up rows per tile (``dual``)
EXL3      ``p0`` the trellis int16 [1,K/16,N/16,16*bits] as stored in the checkpoint, ``p1`` suh fp32 [1,K],
          ``p2`` svh fp32 [1,N]: y = had128(had128(x * suh) W_rot) * svh (see formats/exl3.py).  One matrix per
          weight (no expert stacks), never concatenated or sliced: every projection has its own rotation
========  =====================================================================================

The rows of the small scale planes (Q8 ``p1``, Q6K ``p3``, MXFP4 ``p1``) are zero-padded to 16 bytes
so every row starts 16-byte aligned (the GEMM producers fetch them with 4-byte async copies).

All repacks are plain torch ops, so they run on the GPU for large checkpoints and on the CPU in
tests.  Reference parity: the load-time SoA repacks of src/model/gptoss.cpp:176-214,
include/ie/quant_soa.hpp:33-157 and src/ops/gemv_q6_soa.cpp (bit-plane SoA); the layouts here
are this engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import IntEnum
from typing import Optional

import torch

from ..formats.gguf import GGMLType


class WFormat(IntEnum):
    BF16 = 0
    Q8 = 1
    Q4K = 2
    Q6K = 3
    MXFP4 = 4
    MXF4T = 5      # MXFP4 in 128 x 128 tiles for the block-scaled tensor-core kernel (see to_mxf4_tiles)
    EXL3 = 6       # trellis-coded weights with Hadamard rotations on both sides (formats/exl3.py)


def _pad_last(t: torch.Tensor, mult: int) -> torch.Tensor:
    """Zero-pad the last dimension to a multiple of ``mult`` (scale planes keep 16-byte aligned rows)."""
    n = t.shape[-1]
    m = (n + mult - 1) // mult * mult
    if m == n:
        return t.contiguous()
    out = torch.zeros(*t.shape[:-1], m, dtype=t.dtype, device=t.device)
    out[..., :n] = t
    return out


# (plane index -> (elements of K per plane element, row padding multiple)) for the padded scale planes
_AUX_PAD = {1: {1: (32, 8)}, 3: {3: (256, 8)}, 4: {1: (32, 16)}}     # WFormat value -> {plane: (k per elem, pad)}


_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


@dataclass
class QuantWeight:
    fmt: WFormat
    N: int
    K: int
    E: int = 1                       # number of stacked experts (1 = plain matrix)
    p0: Optional[torch.Tensor] = None
    p1: Optional[torch.Tensor] = None
    p2: Optional[torch.Tensor] = None
    p3: Optional[torch.Tensor] = None
    _dense_cache: Optional[torch.Tensor] = field(default=None, repr=False)
    dual: bool = False               # MXF4T only: the bank interleaves a gate and an up matrix (N = rows of each)

    # -------------------------------------------------------------- basics
    def planes(self) -> list[Optional[torch.Tensor]]:
        return [self.p0, self.p1, self.p2, self.p3]

    @property
    def device(self) -> torch.device:
        return self.p0.device

    def to(self, device) -> "QuantWeight":
        mv = lambda t: None if t is None else t.to(device).contiguous()
        return QuantWeight(self.fmt, self.N, self.K, self.E, mv(self.p0), mv(self.p1), mv(self.p2), mv(self.p3), dual=self.dual)

    @property
    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.planes() if t is not None)

    # -------------------------------------------------------------- row / column surgery
    def _map_planes(self, fn) -> "QuantWeight":
        out = [None if t is None else fn(t) for t in self.planes()]
        return QuantWeight(self.fmt, self.N, self.K, self.E, *out, dual=self.dual)

    def _no_exl3(self, what: str) -> None:
        if self.fmt == WFormat.EXL3:
            raise ValueError(f"an EXL3 weight cannot be {what}: its rows and columns are mixed by the layer's Hadamard rotations")

    @property
    def bits(self) -> int:
        """EXL3: bits per weight of the trellis."""
        return int(self.p0.shape[-1]) // 16

    def select_rows(self, idx: torch.Tensor) -> "QuantWeight":
        """Rows (output features) ``idx`` of every expert."""
        self._no_exl3("row-permuted")
        idx = idx.to(self.device)
        w = self._map_planes(lambda t: t.index_select(1, idx).contiguous())
        w.N = int(idx.numel())
        return w

    def slice_rows(self, lo: int, hi: int) -> "QuantWeight":
        self._no_exl3("sliced by rows")
        w = self._map_planes(lambda t: t[:, lo:hi].contiguous())
        w.N = hi - lo
        return w

    def slice_experts(self, lo: int, hi: int) -> "QuantWeight":
        w = self._map_planes(lambda t: t[lo:hi].contiguous())
        w.E = hi - lo
        return w

    def k_granule(self) -> int:
        return {WFormat.BF16: 8, WFormat.Q8: 32, WFormat.Q4K: 256, WFormat.Q6K: 256, WFormat.MXFP4: 32}[self.fmt]

    def slice_k(self, lo: int, hi: int, requant: bool = False) -> "QuantWeight":
        """Input-dimension slice [lo, hi) (row-parallel shards).  Bounds must sit on block boundaries; with
        ``requant`` a slice that cuts a block is re-encoded instead (Q8 when the slice is a multiple of 32 wide,
        else bf16) -- the case of a 256-element super-block format sharded finer than its blocks."""
        self._no_exl3("sliced along K")
        g = self.k_granule()
        if lo % g or hi % g:
            if not requant:
                raise ValueError(f"K slice [{lo},{hi}) is not aligned to the {g}-element blocks of {self.fmt.name}")
            dense = self.dequantize(torch.float32)[:, :, lo:hi].contiguous()
            return from_dense(dense, WFormat.Q8 if (hi - lo) % 32 == 0 else WFormat.BF16)
        per_elem = {
            WFormat.BF16: (1, None, None, None), WFormat.Q8: (1, 32, None, None), WFormat.Q4K: (256 / 144, None, None, None),
            WFormat.Q6K: (2, 4, 16, 256), WFormat.MXFP4: (2, 32, None, None),
        }[self.fmt]
        outs = []
        pads = _AUX_PAD.get(int(self.fmt), {})
        for i, (t, div) in enumerate(zip(self.planes(), per_elem)):
            if t is None:
                outs.append(None)
            else:
                a, b = int(round(lo / div)), int(round(hi / div))
                sl = t[:, :, a:b]
                outs.append(_pad_last(sl, pads[i][1]) if i in pads else sl.contiguous())
        w = QuantWeight(self.fmt, self.N, hi - lo, self.E, *outs)
        return w

    @staticmethod
    def cat_rows(ws: list["QuantWeight"]) -> "QuantWeight":
        f = ws[0]
        f._no_exl3("concatenated")
        assert all(w.fmt == f.fmt and w.K == f.K and w.E == f.E for w in ws), "cannot concatenate mixed formats"
        outs = []
        for i in range(4):
            ps = [w.planes()[i] for w in ws]
            outs.append(None if ps[0] is None else torch.cat(ps, dim=1).contiguous())
        return QuantWeight(f.fmt, sum(w.N for w in ws), f.K, f.E, *outs)

    @staticmethod
    def interleave_gate_up(gate: "QuantWeight", up: "QuantWeight") -> "QuantWeight":
        """Rows in groups of 16: [g0..g15, u0..u15, g16..g31, u16..u31, ...] (kernel epilogues rely on it)."""
        assert gate.fmt == up.fmt and gate.N == up.N and gate.K == up.K and gate.E == up.E
        gate._no_exl3("interleaved")
        if gate.N % 16:
            raise ValueError("gate/up interleave needs a multiple of 16 output features")
        def il(a, b):
            if a is None:
                return None
            E, N = a.shape[0], a.shape[1]
            a2 = a.reshape(E, N // 16, 16, -1)
            b2 = b.reshape(E, N // 16, 16, -1)
            return torch.cat([a2, b2], dim=2).reshape(E, 2 * N, -1).contiguous()
        outs = [il(a, b) for a, b in zip(gate.planes(), up.planes())]
        return QuantWeight(gate.fmt, 2 * gate.N, gate.K, gate.E, *outs)

    # -------------------------------------------------------------- decode (oracle / CPU path)
    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        """[E,N,K] (or [N,K] when E == 1 and squeeze) in ``dtype``; exact decode of the stored values."""
        E, N, K = self.E, self.N, self.K
        if self.fmt == WFormat.BF16:
            w = self.p0.to(torch.float32)
        elif self.fmt == WFormat.Q8:
            w = self.p0.to(torch.float32).reshape(E, N, K // 32, 32) * self.p1[..., :K // 32].to(torch.float32).unsqueeze(-1)
        elif self.fmt == WFormat.Q4K:
            w = _dequant_q4k_blocks(self.p0.reshape(E, N, K // 256, 144))
        elif self.fmt == WFormat.Q6K:
            lo = self.p0.to(torch.int32)
            q = torch.stack([lo & 15, lo >> 4], dim=-1).reshape(E, N, K // 16, 16)
            hb = self.p1.to(torch.int32).reshape(E, N, K // 16, 4)          # byte b of each 16-group
            h = torch.empty(E, N, K // 16, 16, dtype=torch.int32, device=lo.device)
            for b in range(4):
                h[..., 2 * b] = hb[..., b] & 3
                h[..., 2 * b + 1] = (hb[..., b] >> 2) & 3
                h[..., 8 + 2 * b] = (hb[..., b] >> 4) & 3
                h[..., 9 + 2 * b] = (hb[..., b] >> 6) & 3
            q = (q | (h << 4)) - 32
            sc = self.p2.to(torch.float32).unsqueeze(-1)
            d = self.p3[..., :K // 256].to(torch.float32).repeat_interleave(16, dim=-1).unsqueeze(-1)
            w = q.to(torch.float32) * sc * d
        elif self.fmt == WFormat.MXF4T:
            planes = from_mxf4_tiles(self)
            if self.dual:                 # gate rows, then up rows
                return torch.cat([planes[0].dequantize(dtype), planes[1].dequantize(dtype)], dim=1)
            return planes.dequantize(dtype)
        elif self.fmt == WFormat.EXL3:
            # the dense matrix of the whole layer (rotations and sign / scale vectors included), so that x W^T is the layer
            from ..formats import exl3
            return exl3.effective_weight(self.p0[0], self.p1[0], self.p2[0]).to(self.p0.device).reshape(1, N, K).to(dtype)
        elif self.fmt == WFormat.MXFP4:
            codes = self.p0.to(torch.int64)
            c = torch.stack([codes & 15, codes >> 4], dim=-1).reshape(E, N, K // 32, 32)
            vals = _E2M1.to(codes.device)[c]
            w = vals * _e8m0_to_f32(self.p1[..., :K // 32]).unsqueeze(-1)
        else:  # pragma: no cover
            raise ValueError(self.fmt)
        return w.reshape(E, N, K).to(dtype)


def _e8m0_to_f32(e: torch.Tensor) -> torch.Tensor:
    return torch.exp2(e.to(torch.float32) - 127.0)


def _dequant_q4k_blocks(blk: torch.Tensor) -> torch.Tensor:
    """blk: uint8 [..., 144] -> float32 [..., 256]."""
    d = blk[..., 0:2].contiguous().view(torch.float16).to(torch.float32)        # [...,1]
    dmin = blk[..., 2:4].contiguous().view(torch.float16).to(torch.float32)
    s = blk[..., 4:16].to(torch.int32)
    sc = torch.empty(*blk.shape[:-1], 8, dtype=torch.int32, device=blk.device)
    mn = torch.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[..., j] = s[..., j] & 63
            mn[..., j] = s[..., j + 4] & 63
        else:
            sc[..., j] = (s[..., j + 4] & 15) | ((s[..., j - 4] >> 6) << 4)
            mn[..., j] = (s[..., j + 4] >> 4) | ((s[..., j] >> 6) << 4)
    qs = blk[..., 16:144].to(torch.int32).reshape(*blk.shape[:-1], 4, 32)
    q = torch.stack([qs & 15, qs >> 4], dim=-2).reshape(*blk.shape[:-1], 8, 32)   # sub-block major
    w = d.unsqueeze(-1) * sc.unsqueeze(-1) * q - dmin.unsqueeze(-1) * mn.unsqueeze(-1)
    return w.reshape(*blk.shape[:-1], 256)


# ------------------------------------------------------------------ repack from ggml payloads
def from_ggml(raw: torch.Tensor, ttype: int, N: int, K: int, E: int = 1, keep_q8_for: bool = True) -> QuantWeight:
    """``raw``: uint8 tensor holding E*N rows of K elements of ggml type ``ttype``."""
    t = int(ttype)
    raw = raw.reshape(-1)
    dev = raw.device
    if t == GGMLType.F32:
        return QuantWeight(WFormat.BF16, N, K, E, raw.view(torch.float32).reshape(E, N, K).to(torch.bfloat16).contiguous())
    if t == GGMLType.F16:
        return QuantWeight(WFormat.BF16, N, K, E, raw.view(torch.float16).reshape(E, N, K).to(torch.bfloat16).contiguous())
    if t == GGMLType.BF16:
        return QuantWeight(WFormat.BF16, N, K, E, raw.view(torch.bfloat16).reshape(E, N, K).contiguous())
    if t == GGMLType.Q8_0:
        b = raw.reshape(E, N, K // 32, 34)
        d = b[..., 0:2].contiguous().view(torch.float16).reshape(E, N, K // 32)
        q = b[..., 2:34].contiguous().view(torch.int8).reshape(E, N, K)
        return QuantWeight(WFormat.Q8, N, K, E, q, _pad_last(d, 8))
    if t == GGMLType.Q4_K:
        return QuantWeight(WFormat.Q4K, N, K, E, raw.reshape(E, N, K // 256 * 144).contiguous())
    if t == GGMLType.Q6_K:
        b = raw.reshape(E, N, K // 256, 210)
        ql = b[..., 0:128].to(torch.int32).reshape(E, N, K // 256, 2, 2, 32)      # (half, which32, l)
        qh = b[..., 128:192].to(torch.int32).reshape(E, N, K // 256, 2, 1, 32)
        low = torch.cat([ql & 15, ql >> 4], dim=-2)                               # (half, quarter, l)
        shifts = torch.tensor([0, 2, 4, 6], device=dev, dtype=torch.int32).reshape(1, 1, 1, 1, 4, 1)
        high = (qh >> shifts) & 3
        q = (low | (high << 4)).reshape(E, N, K)                                  # natural element order, 0..63
        lo4 = q & 15
        p0 = (lo4[..., 0::2] | (lo4[..., 1::2] << 4)).to(torch.uint8)
        h = (q >> 4).reshape(E, N, K // 16, 16)
        hb = [h[..., 2 * bb] | (h[..., 2 * bb + 1] << 2) | (h[..., 8 + 2 * bb] << 4) | (h[..., 9 + 2 * bb] << 6) for bb in range(4)]
        p1 = torch.stack(hb, dim=-1).reshape(E, N, K // 4).to(torch.uint8)
        p2 = b[..., 192:208].contiguous().view(torch.int8).reshape(E, N, K // 16)
        p3 = b[..., 208:210].contiguous().view(torch.float16).reshape(E, N, K // 256)
        return QuantWeight(WFormat.Q6K, N, K, E, p0.contiguous(), p1.contiguous(), p2.contiguous(), _pad_last(p3, 8))
    if t == GGMLType.MXFP4:
        b = raw.reshape(E, N, K // 32, 17)
        e = b[..., 0].contiguous()
        qs = b[..., 1:17].to(torch.int32)
        c = torch.cat([qs & 15, qs >> 4], dim=-1)                                 # natural order codes [.., 32]
        p0 = (c[..., 0::2] | (c[..., 1::2] << 4)).to(torch.uint8).reshape(E, N, K // 2)
        return QuantWeight(WFormat.MXFP4, N, K, E, p0.contiguous(), _pad_last(e, 16))
    if t == GGMLType.EXL3:
        raise ValueError("an EXL3 trellis needs its suh / svh vectors: use from_exl3")
    if t in (GGMLType.Q5_K, GGMLType.Q4_0):
        # rare formats: decode once on the host and keep bf16 (the reference also widens these at load)
        import numpy as np
        from ..formats import quant
        f = quant.dequantize(raw.cpu().numpy(), t, E * N * K)
        return QuantWeight(WFormat.BF16, N, K, E, torch.from_numpy(f).reshape(E, N, K).to(torch.bfloat16).to(dev).contiguous())
    raise ValueError(f"unsupported ggml tensor type {t}")


MXF4_TILE_ROWS = 192


def _mxf4_atoms(ex: torch.Tensor) -> torch.Tensor:
    """Exponent bytes [E, FB, 192, KB*4] -> scale atoms [E, FB, KB, 2, 512]: the 192 rows of a tile fill one and a half atoms of
    128 rows (the rest holds 127); row r = r1 * 32 + r0 of an atom, k-block q at byte r0 * 16 + r1 * 4 + q."""
    E, FB, _, K4 = ex.shape
    KB = K4 // 4
    full = torch.full((E, FB, 256, K4), 127, dtype=torch.uint8, device=ex.device)
    full[:, :, :MXF4_TILE_ROWS] = ex
    return full.reshape(E, FB, 2, 4, 32, KB, 4).permute(0, 1, 5, 2, 4, 3, 6).contiguous().reshape(E, FB, KB, 2, 512)


def _mxf4_pad(w: QuantWeight, rows: int, KB: int):
    """Codes and exponents of an MXFP4 plane weight padded to ``rows`` x KB*128 (code 0 = +0.0, exponent 127 = scale 1)."""
    E, N, K = w.E, w.N, w.K
    dev = w.p0.device
    codes = torch.zeros(E, rows, KB * 64, dtype=torch.uint8, device=dev)
    codes[:, :N, :K // 2] = w.p0
    ex = torch.full((E, rows, KB * 4), 127, dtype=torch.uint8, device=dev)
    ex[:, :N, :K // 32] = w.p1[..., :K // 32]
    return codes, ex


def to_mxf4_tiles(w: QuantWeight, up: Optional[QuantWeight] = None) -> QuantWeight:
    """MXFP4 planes -> the tiled layout of the block-scaled tensor-core kernel (csrc/cuda/gemm_mxf4.cu): tiles of 192 rows x 128
    elements, ``p0`` [E, FB, KB, 192, 64] codes and ``p1`` [E, FB, KB, 2, 512] scale atoms.  With ``up`` (``w`` = gate) tile fb
    holds gate rows 96 fb .. 96 fb + 95 followed by the same rows of ``up``; a single matrix puts rows 192 fb .. 192 fb + 191
    into tile fb."""
    assert w.fmt == WFormat.MXFP4 and (up is None or (up.fmt == WFormat.MXFP4 and (up.N, up.K, up.E) == (w.N, w.K, w.E)))
    E, N, K = w.E, w.N, w.K
    KB = (K + 127) // 128
    if up is None:
        FB = (N + MXF4_TILE_ROWS - 1) // MXF4_TILE_ROWS
        codes, ex = _mxf4_pad(w, FB * MXF4_TILE_ROWS, KB)
        codes = codes.reshape(E, FB, MXF4_TILE_ROWS, KB, 64)
        ex = ex.reshape(E, FB, MXF4_TILE_ROWS, KB * 4)
    else:
        half = MXF4_TILE_ROWS // 2
        FB = (N + half - 1) // half
        cg, eg = _mxf4_pad(w, FB * half, KB)
        cu, eu = _mxf4_pad(up, FB * half, KB)
        codes = torch.cat([cg.reshape(E, FB, half, KB, 64), cu.reshape(E, FB, half, KB, 64)], dim=2)
        ex = torch.cat([eg.reshape(E, FB, half, KB * 4), eu.reshape(E, FB, half, KB * 4)], dim=2)
        del cg, cu, eg, eu
    tiles = codes.permute(0, 1, 3, 2, 4).contiguous()
    return QuantWeight(WFormat.MXF4T, N, K, E, tiles, _mxf4_atoms(ex), dual=up is not None)


def from_mxf4_tiles(w: QuantWeight):
    """Inverse of :func:`to_mxf4_tiles` (oracle / CPU path): the MXFP4 plane weight, or (gate, up) for a gated pair."""
    assert w.fmt == WFormat.MXF4T
    E, N, K = w.E, w.N, w.K
    FB, KB = w.p0.shape[1], w.p0.shape[2]
    codes = w.p0.permute(0, 1, 3, 2, 4)                                               # [E, FB, 192, KB, 64]
    ex = w.p1.reshape(E, FB, KB, 2, 32, 4, 4).permute(0, 1, 3, 5, 4, 2, 6).reshape(E, FB, 256, KB * 4)[:, :, :MXF4_TILE_ROWS]

    def plane(c, e):
        rows = c.shape[1] * c.shape[2]
        return QuantWeight(WFormat.MXFP4, N, K, E, c.reshape(E, rows, KB * 64)[:, :N, :K // 2].contiguous(),
                           _pad_last(e.reshape(E, rows, KB * 4)[:, :N, :K // 32], 16))
    if not w.dual:
        return plane(codes, ex)
    half = MXF4_TILE_ROWS // 2
    return plane(codes[:, :, :half], ex[:, :, :half]), plane(codes[:, :, half:], ex[:, :, half:])


# ------------------------------------------------------------------ torch-side quantisers (device synthesis)
def quantize_mxfp4(w: torch.Tensor) -> QuantWeight:
    """Round ``w`` [E,N,K] (or [N,K]) to MXFP4 directly in the runtime layout (any device)."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    E, N, K = w.shape
    x = w.to(torch.float32).reshape(E, N, K // 32, 32)
    amax = x.abs().amax(dim=-1, keepdim=True)
    e = torch.where(amax > 0, torch.floor(torch.log2(amax.clamp_min(1e-38))) - 2 + 127, torch.zeros_like(amax)).clamp_(0, 254)
    y = x * torch.exp2(127.0 - e)
    # nearest E2M1 magnitude through the midpoints between consecutive codes
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=w.device)
    idx = torch.bucketize(y.abs(), bounds).to(torch.int32)
    code = idx | ((y < 0) & (idx > 0)).to(torch.int32) * 8
    code = code.reshape(E, N, K)
    p0 = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8).contiguous()
    return QuantWeight(WFormat.MXFP4, N, K, E, p0, _pad_last(e.reshape(E, N, K // 32).to(torch.uint8), 16))


def quantize_q8(w: torch.Tensor) -> QuantWeight:
    if w.dim() == 2:
        w = w.unsqueeze(0)
    E, N, K = w.shape
    x = w.to(torch.float32).reshape(E, N, K // 32, 32)
    d = x.abs().amax(dim=-1, keepdim=True) / 127.0
    q = torch.where(d > 0, torch.round(x / d.clamp_min(1e-30)), torch.zeros_like(x)).clamp_(-127, 127)
    return QuantWeight(WFormat.Q8, N, K, E, q.reshape(E, N, K).to(torch.int8).contiguous(), _pad_last(d.reshape(E, N, K // 32).to(torch.float16), 8))


def quantize_q4k(w: torch.Tensor) -> QuantWeight:
    """Q4_K encode with torch ops (min/max affine per 32, 6-bit scales per 256) -> native ggml blocks."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    E, N, K = w.shape
    x = w.to(torch.float32).reshape(E, N, K // 256, 8, 32)
    lo = x.amin(dim=-1).clamp_max(0.0)
    hi = x.amax(dim=-1)
    s = ((hi - lo) / 15.0).clamp_min(0.0)
    m = -lo
    d = s.amax(dim=-1, keepdim=True) / 63.0
    dm = m.amax(dim=-1, keepdim=True) / 63.0
    d16, dm16 = d.to(torch.float16), dm.to(torch.float16)
    df, dmf = d16.to(torch.float32), dm16.to(torch.float32)
    sc = torch.where(df > 0, torch.round(s / df.clamp_min(1e-30)), torch.zeros_like(s)).clamp_(0, 63).to(torch.int32)
    mn = torch.where(dmf > 0, torch.round(m / dmf.clamp_min(1e-30)), torch.zeros_like(m)).clamp_(0, 63).to(torch.int32)
    es = (df * sc).unsqueeze(-1)
    em = (dmf * mn).unsqueeze(-1)
    q = torch.where(es > 0, torch.round((x + em) / es.clamp_min(1e-30)), torch.zeros_like(x)).clamp_(0, 15).to(torch.int32)
    blk = torch.zeros(E, N, K // 256, 144, dtype=torch.uint8, device=w.device)
    blk[..., 0:2] = d16.contiguous().view(torch.uint8).reshape(E, N, K // 256, 2)
    blk[..., 2:4] = dm16.contiguous().view(torch.uint8).reshape(E, N, K // 256, 2)
    sb = torch.zeros(E, N, K // 256, 12, dtype=torch.int32, device=w.device)
    for j in range(8):
        if j < 4:
            sb[..., j] |= sc[..., j] & 63
            sb[..., j + 4] |= mn[..., j] & 63
        else:
            sb[..., j + 4] |= (sc[..., j] & 15) | ((mn[..., j] & 15) << 4)
            sb[..., j - 4] |= (sc[..., j] >> 4) << 6
            sb[..., j] |= (mn[..., j] >> 4) << 6
    blk[..., 4:16] = sb.to(torch.uint8)
    q = q.reshape(E, N, K // 256, 4, 2, 32)
    blk[..., 16:144] = (q[..., 0, :] | (q[..., 1, :] << 4)).to(torch.uint8).reshape(E, N, K // 256, 128)
    return QuantWeight(WFormat.Q4K, N, K, E, blk.reshape(E, N, K // 256 * 144).contiguous())


def quantize_q6k(w: torch.Tensor) -> QuantWeight:
    """Q6_K-grade encode straight into the plane layout (symmetric, int8 scale per 16, fp16 scale per 256)."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    E, N, K = w.shape
    x = w.to(torch.float32).reshape(E, N, K // 256, 16, 16)
    s = x.abs().amax(dim=-1) / 31.0
    d = (s.amax(dim=-1, keepdim=True) / 127.0)
    d16 = d.to(torch.float16)
    df = d16.to(torch.float32)
    sc = torch.where(df > 0, torch.round(s / df.clamp_min(1e-30)), torch.zeros_like(s)).clamp_(-128, 127)
    es = (df * sc).unsqueeze(-1)
    q = (torch.where(es != 0, torch.round(x / torch.where(es != 0, es, torch.ones_like(es))), torch.zeros_like(x)).clamp_(-32, 31) + 32).to(torch.int32)
    q = q.reshape(E, N, K)
    lo4 = q & 15
    p0 = (lo4[..., 0::2] | (lo4[..., 1::2] << 4)).to(torch.uint8)
    h = (q >> 4).reshape(E, N, K // 16, 16)
    hb = [h[..., 2 * b] | (h[..., 2 * b + 1] << 2) | (h[..., 8 + 2 * b] << 4) | (h[..., 9 + 2 * b] << 6) for b in range(4)]
    p1 = torch.stack(hb, dim=-1).reshape(E, N, K // 4).to(torch.uint8)
    return QuantWeight(WFormat.Q6K, N, K, E, p0.contiguous(), p1.contiguous(), sc.reshape(E, N, K // 16).to(torch.int8).contiguous(),
                       _pad_last(d16.reshape(E, N, K // 256), 8))


def from_exl3(trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor) -> QuantWeight:
    """trellis int16 [K/16, N/16, 16*bits], suh [K], svh [N] (any float type) -> the runtime weight."""
    assert trellis.dtype == torch.int16 and trellis.dim() == 3
    K, N = int(trellis.shape[0]) * 16, int(trellis.shape[1]) * 16
    if K % 128 or N % 128 or suh.numel() != K or svh.numel() != N or not 1 <= int(trellis.shape[2]) // 16 <= 8 or int(trellis.shape[2]) % 16:
        raise ValueError(f"inconsistent EXL3 layer: trellis {tuple(trellis.shape)}, suh {suh.numel()}, svh {svh.numel()}")
    dev = trellis.device
    return QuantWeight(WFormat.EXL3, N, K, 1, trellis.unsqueeze(0).contiguous(), suh.to(dev, torch.float32).reshape(1, K).contiguous(),
                       svh.to(dev, torch.float32).reshape(1, N).contiguous())


def from_dense(w: torch.Tensor, fmt: WFormat) -> QuantWeight:
    if fmt == WFormat.BF16:
        if w.dim() == 2:
            w = w.unsqueeze(0)
        return QuantWeight(WFormat.BF16, w.shape[1], w.shape[2], w.shape[0], w.to(torch.bfloat16).contiguous())
    return {WFormat.Q8: quantize_q8, WFormat.Q4K: quantize_q4k, WFormat.Q6K: quantize_q6k, WFormat.MXFP4: quantize_mxfp4}[fmt](w)
