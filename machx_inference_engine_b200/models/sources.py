"""Where model weights come from: a GGUF file or an on-device random initialiser.

Both hand the model graphs :class:`~ops.weights.QuantWeight` matrices in the runtime layouts, so
the graphs have one loading path.  ``GGUFSource`` repacks ggml payloads (on the target device);
``SynthSource`` draws N(0, std) weights and quantises them to the format a policy names -- the
same bytes a GGUF of that type would hold after repack -- without going through the file system,
which is what makes the 120b-class benchmarks possible on a box without a checkpoint.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch

from ..formats.gguf import GGMLType, GGUFReader
from ..ops.weights import QuantWeight, WFormat, from_dense, from_exl3, from_ggml


class GGUFSource:
    def __init__(self, reader: GGUFReader, device):
        self.r = reader
        self.device = torch.device(device)

    def has(self, name: str) -> bool:
        return self.r.has_tensor(name)

    def matrix(self, name: str, N: int, K: int, E: int = 1, experts: Optional[tuple[int, int]] = None) -> QuantWeight:
        t = self.r.tensor(name)
        if int(t.type) == GGMLType.EXL3:
            # a verbatim trellis {16*bits, N/16, K/16} with its sign / scale vectors beside it (<root>.suh, <root>.svh)
            if E != 1 or len(t.dims) != 3 or (int(t.dims[2]) * 16, int(t.dims[1]) * 16) != (K, N):
                raise ValueError(f"{name}: EXL3 trellis dims {tuple(t.dims)} do not describe a [{N}, {K}] matrix")
            root = name[:-len(".weight")] if name.endswith(".weight") else name
            tr = torch.from_numpy(np.frombuffer(np.array(t.raw(), copy=True), dtype=np.int16).reshape(K // 16, N // 16, int(t.dims[0])))
            return from_exl3(tr.to(self.device), self.vector(root + ".suh", K), self.vector(root + ".svh", N))
        want = (K, N) if E == 1 else (K, N, E)
        if tuple(t.dims) != want:
            raise ValueError(f"{name}: expected ggml dims {want}, file has {tuple(t.dims)}")
        raw = torch.from_numpy(np.array(t.raw(), copy=True))
        if experts is not None:
            per = t.nbytes // E
            raw = raw[experts[0] * per: experts[1] * per]
            E = experts[1] - experts[0]
        return from_ggml(raw.to(self.device), t.type, N, K, E)

    def vector(self, name: str, n: int) -> torch.Tensor:
        t = self.r.tensor(name)
        v = torch.from_numpy(t.to_float32().reshape(-1).copy())
        if v.numel() != n:
            raise ValueError(f"{name}: expected {n} elements, file has {v.numel()}")
        return v.to(self.device)

    def table(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        t = self.r.tensor(name)
        v = torch.from_numpy(t.to_float32().copy())
        if tuple(v.shape) != tuple(shape):
            raise ValueError(f"{name}: expected shape {shape}, file has {tuple(v.shape)}")
        return v.to(self.device)


def default_policy(arch: str, quant: str) -> Callable[[str], WFormat]:
    """Weight format per tensor name for a named quantisation recipe.

    ``q4_k_m``: Q4_K projections, Q6_K output / half of attn_v and ffn_down (llama.cpp's recipe);
    ``q8_0``: everything Q8; ``mxfp4``: MXFP4 experts, bf16 attention, Q8 embeddings/head (gpt-oss);
    ``bf16``: everything bf16; ``exl3`` / ``exl3-<bits>``: every projection and the head as EXL3 trellis layers (4 bits per
    weight unless said), embeddings bf16 -- the layout of an imported EXL3 checkpoint (src/loaders/hf_import.cpp:536-592).
    """
    quant = quant.lower()
    exl3_bits = 0
    if quant == "exl3" or quant.startswith("exl3-"):
        exl3_bits = int(quant[5:]) if quant.startswith("exl3-") else 4
        if not 1 <= exl3_bits <= 8:
            raise ValueError("EXL3 takes 1 to 8 bits per weight")
        quant = "exl3"

    def pol(name: str) -> WFormat:
        if quant == "bf16":
            return WFormat.BF16
        if quant == "q8_0":
            return WFormat.Q8
        if quant == "exl3":
            return WFormat.BF16 if name == "token_embd.weight" else WFormat.EXL3
        if quant == "mxfp4":
            if "_exps" in name:
                return WFormat.MXFP4
            if name in ("token_embd.weight", "output.weight"):
                return WFormat.Q8
            return WFormat.BF16
        if quant == "q4_k_m":
            if name == "output.weight":
                return WFormat.Q6K
            if name.endswith("attn_v.weight") or name.endswith("ffn_down.weight") or "ffn_down_exps" in name:
                return WFormat.Q6K if _more_bits(name) else WFormat.Q4K
            return WFormat.Q4K
        raise ValueError(f"unknown quantisation recipe {quant}")

    pol.exl3_bits = exl3_bits
    return pol


_N_LAYERS_HINT = {"n": 32}


def _more_bits(name: str) -> bool:
    try:
        i = int(name.split(".")[1])
    except Exception:
        return False
    n = _N_LAYERS_HINT["n"]
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


class SynthSource:
    """Deterministic random weights.  Every tensor has its own seed derived from its name, so ranks
    that ask for different slices of the same tensor see consistent values."""

    def __init__(self, device, policy: Callable[[str], WFormat], seed: int = 0, std: float = 0.02, n_layers: int = 32, gen_device=None):
        self.device = torch.device(device)
        # random streams differ between CPU and CUDA generators: draw on ``gen_device`` (default: the
        # target device) and move, so a CPU oracle and a GPU model can share identical weights
        self.gen_device = torch.device(gen_device) if gen_device is not None else self.device
        self.policy = policy
        self.seed = seed
        self.std = std
        _N_LAYERS_HINT["n"] = n_layers

    def has(self, name: str) -> bool:      # the graph decides by config which optional tensors exist
        return True

    def _gen(self, name: str, extra: int = 0) -> torch.Generator:
        h = 1469598103934665603
        for ch in (name + f"#{extra}").encode():
            h = ((h ^ ch) * 1099511628211) & ((1 << 63) - 1)
        g = torch.Generator(device=self.gen_device)
        g.manual_seed((h + self.seed) & ((1 << 63) - 1))
        return g

    def matrix(self, name: str, N: int, K: int, E: int = 1, experts: Optional[tuple[int, int]] = None) -> QuantWeight:
        fmt = self.policy(name)
        if fmt == WFormat.EXL3:
            if E == 1 and N % 128 == 0 and K % 128 == 0:
                from ..formats import exl3
                tr, suh, svh = exl3.random_layer(N, K, getattr(self.policy, "exl3_bits", 4) or 4, self._gen(name), self.std)
                return from_exl3(tr, suh, svh).to(self.device)
            fmt = WFormat.BF16            # expert stacks and shapes off the 128-point rotation stay dense
        gran = {WFormat.BF16: 8, WFormat.Q8: 32, WFormat.Q4K: 256, WFormat.Q6K: 256, WFormat.MXFP4: 32}[fmt]
        if K % gran:                      # llama.cpp's fallback for ragged rows
            fmt = WFormat.Q8 if K % 32 == 0 else WFormat.BF16
        lo, hi = experts if experts is not None else (0, E)
        parts = []
        # one expert at a time keeps the fp32 staging small (a 120b expert layer is 2.1 G elements)
        for e in range(lo, hi):
            w = torch.randn(1, N, K, generator=self._gen(name, e), device=self.gen_device, dtype=torch.float32) * self.std
            parts.append(from_dense(w, fmt).to(self.device) if self.gen_device != self.device else from_dense(w, fmt))
            del w
        if len(parts) == 1:
            return parts[0]
        planes = []
        for i in range(4):
            ps = [p.planes()[i] for p in parts]
            planes.append(None if ps[0] is None else torch.cat(ps, dim=0).contiguous())
        return QuantWeight(fmt, N, K, hi - lo, *planes)

    def vector(self, name: str, n: int) -> torch.Tensor:
        g = self._gen(name)
        if name.endswith("norm.weight") or "_norm" in name or name.endswith(".scale") or name.endswith("layer_output_scale.weight"):
            return (1.0 + 0.05 * torch.randn(n, generator=g, device=self.gen_device)).to(self.device)
        if name.endswith("ssm_a"):
            return (-torch.exp(torch.randn(n, generator=g, device=self.gen_device) * 0.5)).to(self.device)
        return (0.02 * torch.randn(n, generator=g, device=self.gen_device)).to(self.device)

    def table(self, name: str, shape: tuple[int, ...]) -> torch.Tensor:
        g = self._gen(name)
        return (0.1 * torch.randn(*shape, generator=g, device=self.gen_device)).to(self.device)
