"""Row-sharded prefill: every rank keeps T / W rows of the residual stream and the collectives live inside the kernels around them.

``ShardedComm`` owns one workspace per rank (a raw CUDA allocation that every peer maps over NVLink with CUDA IPC) and drives
the kernels of ``csrc/cuda/shard.cu``:

* ``norm``: residual add (+ the sum of the reduce-scattered partials of the row-parallel projection before it) + RMSNorm on the
  rank's own rows; the normalised rows can be stored straight into every rank's gather buffer,
* ``linear_gathered``: the column-parallel projection on the gathered rows: the tcgen05 GEMM waits per row chunk for its owner's
  flag (all-gather -> GEMM),
* ``dispatch`` / ``combine``: expert parallelism with an all-to-all of MXFP8 rows and bf16 results instead of an all-reduce of
  replicated activations; every rank routes, packs and quantises only its own rows.

The row-parallel projections use the reduce-scatter epilogue of the fused all-reduce path (``parallel/fused.py``, ``rs_rows``).
Reference parity: replaces the replicated-x tensor parallelism of src/model/dense_tp.cpp:330-439 and the replicated packing of
src/model/qwen3moe_tp.cpp:600-684; the per-kernel protocol is documented in ``csrc/cuda/shard.cu``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import cuda as K
from ..ops.weights import QuantWeight, WFormat

_vp = C.c_void_p


class _WsStruct(C.Structure):
    _fields_ = [("base", C.c_void_p * 8), ("world", C.c_int), ("my_rank", C.c_int),
                ("off_gather", C.c_longlong), ("gather_stride", C.c_longlong), ("off_cnt", C.c_longlong), ("off_xq", C.c_longlong),
                ("off_sf", C.c_longlong), ("off_meta", C.c_longlong), ("off_ret", C.c_longlong), ("off_flags", C.c_longlong),
                ("seq", C.c_void_p), ("ticket", C.c_void_p), ("wait_cycles_log2", C.c_int)]


class _Raw:
    """A window of the workspace as something torch can wrap without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _align(n: int, a: int = 4096) -> int:
    return (n + a - 1) // a * a


@dataclass
class DispatchPlan:
    pair_pos: torch.Tensor
    tile_expert: torch.Tensor
    tile_valid: torch.Tensor
    num_tiles: torch.Tensor
    max_tiles: int


class ShardedComm:
    FL_GATHER = 0

    def __init__(self, par, device, hidden: int, max_tokens: int, n_experts: int = 0, top_k: int = 0, wait_cycles_log2: int = 31):
        self.par, self.device, self.world, self.rank = par, torch.device(device), par.world, par.rank
        W = self.world
        self.H = hidden
        self.t_max = _align(max_tokens, 128 * W)
        self.r_max = self.t_max // W
        self.E, self.topk = n_experts, top_k
        self.e_per_rank = (n_experts + W - 1) // W if n_experts else 0
        self.Kp = (hidden + 127) // 128 * 128
        self.sf_ld = (self.Kp // 32 + 15) // 16 * 16
        # every pair of the whole chunk could land on one rank
        self.p_max = _align(self.t_max * max(top_k, 1), 128) + self.e_per_rank * 128 if n_experts else 0
        self.max_tiles = max(self.p_max // 128, 1)
        off = 0
        lay = {}
        for name, size in (("gather", 2 * self.t_max * hidden * 2), ("cnt", W * max(n_experts, 1) * 4), ("xq", self.p_max * self.Kp),
                           ("sf", self.p_max * self.sf_ld), ("meta", self.p_max * 4), ("ret", self.r_max * max(top_k, 1) * hidden * 2),
                           ("flags", 4 * 8 * 4)):
            lay[name] = off
            off += _align(max(size, 16))
        self.total = off
        lib = _lib.cuda()
        lib.mx_raw_alloc.restype = C.c_void_p
        lib.mx_raw_alloc.argtypes = [C.c_longlong]
        lib.mx_ipc_import.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        self._base = lib.mx_raw_alloc(self.total)
        if not self._base:
            raise MemoryError(f"cannot allocate the {self.total >> 20} MiB sharded-prefill workspace")
        self.peer_ptrs, self._opened = [self._base], []
        if W > 1:
            h = C.create_string_buffer(64)
            rc = lib.mx_ipc_export(_vp(self._base), h)
            if rc != 0:
                raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
            handles = [None] * W
            dist.all_gather_object(handles, bytes(h.raw), group=par.group)
            self.peer_ptrs = []
            for r, hb in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self._base)
                    continue
                out = C.c_void_p()
                rc = lib.mx_ipc_import(hb, C.byref(out))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle from rank {r} failed ({rc})")
                self._opened.append(out.value)
                self.peer_ptrs.append(out.value)
        self.seq = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.ticket = torch.zeros(4, dtype=torch.int32, device=self.device)
        ws = _WsStruct()
        for r in range(W):
            ws.base[r] = self.peer_ptrs[r]
        ws.world, ws.my_rank = W, self.rank
        ws.off_gather, ws.gather_stride = lay["gather"], self.t_max * hidden * 2
        ws.off_cnt, ws.off_xq, ws.off_sf, ws.off_meta, ws.off_ret, ws.off_flags = (lay[k] for k in ("cnt", "xq", "sf", "meta", "ret", "flags"))
        ws.seq, ws.ticket = self.seq.data_ptr(), self.ticket.data_ptr()
        ws.wait_cycles_log2 = wait_cycles_log2
        assert C.sizeof(ws) == lib.mx_shard_ws_struct_bytes()
        self.ws, self.lay = ws, lay
        self._ws_ref = C.byref(ws)
        self.xq_view = torch.as_tensor(_Raw(self._base + lay["xq"], self.p_max * self.Kp), device=self.device).view(self.p_max, self.Kp) if n_experts else None
        self._gbuf = 0
        torch.cuda.synchronize(self.device)
        par.barrier()

    # ------------------------------------------------------------------ geometry
    def can_shard(self, T: int) -> bool:
        return T > 0 and T % (128 * self.world) == 0 and T <= self.t_max

    def rows(self, T: int) -> tuple[int, int]:
        """(row0, R): this rank's rows of a T-token chunk."""
        R = T // self.world
        return self.rank * R, R

    # ------------------------------------------------------------------ norm (+ reduce-scatter consumer, + all-gather producer)
    @K._profiled("shard_norm")
    def norm(self, x: torch.Tensor, w: torch.Tensor, eps: float, T: int, delta=None, one_plus_w: bool = False, delta_scale: float = 1.0,
             want_local: bool = False, gather: bool = False):
        """``x`` [R, H] fp32 += delta; returns (local bf16 rows or None, gather-buffer index or None).  ``delta``: None, a local
        fp32 / bf16 tensor [R, H], or the ReducedDelta of a row-parallel projection launched with ``rs_rows = R``."""
        R, H = x.shape
        row0, _ = self.rows(T)
        out = torch.empty(R, H, dtype=torch.bfloat16, device=x.device) if want_local else None
        mode, dptr, dbias, inbox, slot_bytes, iseq, ibf16 = 0, _vp(0), _vp(0), _vp(0), 0, _vp(0), 0
        if delta is not None:
            if isinstance(delta, torch.Tensor):
                assert delta.is_contiguous() and delta.shape == x.shape
                mode = 1 if delta.dtype == torch.float32 else 2
                dptr = K._p(delta)
            else:
                assert delta.rs_rows == R and not delta.gathered
                fc = delta.comm
                mode, inbox, slot_bytes, iseq, ibf16 = 3, _vp(fc.peer_ptrs[fc.rank]), fc.slot_bytes, K._p(fc.seq), int(delta.bf16)
                dbias = K._p(delta.bias)
        gbuf = 0
        if gather:
            self._gbuf ^= 1
            gbuf = self._gbuf
        K._check(_lib.cuda().mx_shard_norm(self._ws_ref, K._p(x), R, H, K._p(w), C.c_float(eps), int(one_plus_w), C.c_float(delta_scale), mode, dptr,
                                           dbias, inbox, C.c_longlong(slot_bytes), iseq, ibf16, row0, K._p(out), int(gather), gbuf, K._stream()),
                 "shard_norm")
        K._count()
        return out, (gbuf if gather else None)

    # ------------------------------------------------------------------ all-gather -> GEMM
    @K._profiled("gemm_gathered")
    def linear_gathered(self, lin, T: int, gbuf: int, out_f32: bool = False) -> torch.Tensor:
        """Column-parallel projection of the gathered rows [T, H] (gather buffer ``gbuf``); ``lin`` is a Linear or a MultiLinear."""
        parts = getattr(lin, "parts", None) or [lin]
        outs = [self._gemm_gathered(p.w, p.bias, p.act, p.act_alpha, p.act_limit, T, gbuf, out_f32) for p in parts]
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=1)

    def _gemm_gathered(self, w: QuantWeight, bias, act, act_alpha, act_limit, T, gbuf, out_f32):
        assert w.K == self.H and w.E == 1
        n_out = w.N // 2 if act else w.N
        out = torch.empty(T, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16, device=self.device)
        lib = _lib.cuda()
        fmt, p0, p1, p2, p3 = K._planes(w)
        if fmt != int(WFormat.BF16):          # quantised dense weight: decoded once, like ops.cuda.linear does for long chunks
            wb = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=self.device)
            K._check(lib.mx_dequant_bf16(fmt, p0, p1, p2, p3, C.c_longlong(w.N), w.K, K._p(wb), K._stream()), "dequant_bf16")
            K._count()
            fmt, p0, p1, p2, p3 = int(WFormat.BF16), K._p(wb), _vp(0), _vp(0), _vp(0)
        R = T // self.world
        a_ptr = self._base + self.lay["gather"] + gbuf * self.ws.gather_stride
        flags = self._base + self.lay["flags"] + self.FL_GATHER * 8 * 4
        K._check(lib.mx_gemm_gathered(_vp(a_ptr), fmt, p0, p1, p2, p3, K._p(out), n_out, int(out_f32), K._p(bias), int(act), C.c_float(act_alpha),
                                      C.c_float(act_limit), T, w.N, w.K, K._pick_bn(T, w.N), _vp(flags), _vp(self.seq.data_ptr() + 4 * self.FL_GATHER),
                                      R, self.world, (self.rank * R) // 128, K._stream()), "gemm_gathered")
        K._count()
        return out

    # ------------------------------------------------------------------ expert all-to-all
    @K._profiled("moe_dispatch")
    def dispatch(self, h: torch.Tensor, idx: torch.Tensor):
        """Routes this rank's rows ``h`` [R, H] (bf16) to the ranks that own their top-k experts ``idx`` [R, K].  Returns
        (xq view, sfx scale atoms, DispatchPlan): the inputs of the grouped expert GEMM over this rank's own experts."""
        R, Kt = idx.shape
        lib = _lib.cuda()
        dev = self.device
        n = R * Kt
        pair_pos = torch.empty(n, dtype=torch.int32, device=dev)
        # (entries past the live tile count are never read: the grouped GEMM and the return kernel stop at num_tiles)
        tile_expert = torch.empty(self.max_tiles, dtype=torch.int32, device=dev)
        tile_valid = torch.empty(self.max_tiles, dtype=torch.int32, device=dev)
        num_tiles = torch.empty(2, dtype=torch.int32, device=dev)
        K._check(lib.mx_moe_dispatch_plan(self._ws_ref, K._p(idx), n, self.E, self.e_per_rank, K._p(pair_pos), K._p(tile_expert), K._p(tile_valid),
                                          K._p(num_tiles), self.max_tiles, K._stream()), "moe_dispatch_plan")
        K._check(lib.mx_moe_dispatch_send(self._ws_ref, K._p(h), R, self.H, self.Kp, self.sf_ld, K._p(idx), K._p(pair_pos), Kt, self.e_per_rank,
                                          K._stream()), "moe_dispatch_send")
        sfx = torch.empty(self.Kp // 128, self.max_tiles, 512, dtype=torch.uint8, device=dev)
        K._check(lib.mx_moe_recv_finalize(self._ws_ref, K._p(num_tiles), self.sf_ld, self.Kp // 32, self.max_tiles, K._p(sfx), K._stream()),
                 "moe_recv_finalize")
        K._count(3)
        return self.xq_view, sfx, DispatchPlan(pair_pos, tile_expert, tile_valid, num_tiles, self.max_tiles)

    @K._profiled("moe_return+combine")
    def combine(self, y: torch.Tensor, plan: DispatchPlan, w: torch.Tensor) -> torch.Tensor:
        """Sends every expert output row ``y`` [packed rows, H] (bf16) back to its token's owner and returns this rank's
        weighted sums [R, H] fp32."""
        R, Kt = w.shape
        lib = _lib.cuda()
        K._check(lib.mx_moe_return(self._ws_ref, K._p(y), self.H, K._p(plan.num_tiles), K._p(plan.tile_valid), plan.max_tiles, K._stream()), "moe_return")
        out = torch.empty(R, self.H, dtype=torch.float32, device=self.device)
        K._check(lib.mx_moe_combine_wait(self._ws_ref, K._p(w), K._p(out), R, self.H, Kt, K._stream()), "moe_combine_wait")
        K._count(2)
        return out

    def close(self) -> None:
        lib = _lib.cuda()
        for p in self._opened:
            lib.mx_ipc_release(_vp(p))
        self._opened = []
        if self._base:
            lib.mx_raw_free(_vp(self._base))
            self._base = None


def attach(par, device, cfg, max_tokens: int, force: bool = False) -> Optional[ShardedComm]:
    """Gives ``par`` a :class:`ShardedComm` sized for model ``cfg`` and prefill chunks of up to ``max_tokens`` tokens.  Needs the
    fused reduce-scatter path (``par.fused``); single-rank contexts only get one with ``force`` (tests)."""
    if par.fused is None or par.mode != "tp" or (par.world == 1 and not force):
        return None
    if max_tokens < 128 * par.world:
        return None
    n_exp = int(getattr(cfg, "n_experts", 0) or 0)
    par.sharded = ShardedComm(par, device, cfg.hidden, max_tokens, n_experts=n_exp, top_k=int(getattr(cfg, "n_experts_used", 0) or 0))
    return par.sharded
