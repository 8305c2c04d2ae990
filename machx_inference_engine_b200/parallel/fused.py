"""Peer-memory collectives fused into their producer and consumer kernels (product path for TP/EP).

``FusedComm`` owns this rank's inbox (CUDA IPC allocation mapped by every peer over NVLink) and the
peers' mappings.  A row-parallel projection is launched through :meth:`linear_all_reduce`: its GEMV
(decode) or tcgen05 GEMM (prefill) epilogue stores the partial tile directly into every rank's inbox
and the kernel's last CTA publishes a sequence number; nothing is written locally and no collective
kernel runs.  The returned :class:`ReducedDelta` is consumed by ``ops.rmsnorm`` (the residual add +
RMSNorm that follows every such projection), which waits for the peers' sequence numbers and sums
the partials in rank order, or by :meth:`ReducedDelta.materialize`.

The plain NCCL path (``ParallelCtx.all_reduce``) stays available as the measured baseline.
Layout, ordering and the safety argument for the two-parity slot reuse are in ``csrc/cuda/comm.cuh``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .. import _lib
from ..ops import cuda as K
from ..ops.weights import QuantWeight

_vp = C.c_void_p


@dataclass
class ReducedDelta:
    """A tensor [T, H] that exists as W partials in this rank's inbox until a consumer sums them."""
    comm: "FusedComm"
    T: int
    H: int
    bf16: bool
    bias: Optional[torch.Tensor] = None
    rs_rows: int = 0            # > 0: reduce-scatter form (rows per owner); the owner step has to run before a consumer
    gathered: bool = False      # the owner step has been issued: consumers read the gather region

    @property
    def shape(self):
        return (self.T, self.H)

    def materialize(self) -> torch.Tensor:
        return self.comm.reduce(self)

    def index_select(self, dim: int, rows: torch.Tensor) -> torch.Tensor:
        assert dim == 0
        return self.materialize().index_select(0, rows)


class FusedComm:
    def __init__(self, par, device, slot_bytes: int):
        self.par, self.device, self.world, self.rank = par, device, par.world, par.rank
        self.slot_bytes = int(slot_bytes)
        lib = _lib.cuda()
        lib.mx_ipc_import.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        lib.mx_comm_inbox_bytes.restype = C.c_longlong
        total = int(lib.mx_comm_inbox_bytes(self.world, C.c_longlong(self.slot_bytes)))
        lib.mx_raw_alloc.restype = C.c_void_p
        lib.mx_raw_alloc.argtypes = [C.c_longlong]
        self._base = lib.mx_raw_alloc(total)          # dedicated cudaMalloc allocation, zero-filled
        if not self._base:
            raise MemoryError(f"cannot allocate the {total >> 20} MiB collective inbox")
        h = C.create_string_buffer(64)
        rc = lib.mx_ipc_export(_vp(self._base), h)
        if rc != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
        handles = [(bytes(h.raw), 0)]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, (bytes(h.raw), 0), group=par.group)
        self.peer_ptrs = []
        self._opened = []
        for r, (hb, off) in enumerate(handles):
            if r == self.rank:
                self.peer_ptrs.append(self._base)
                continue
            out = C.c_void_p()
            rc = lib.mx_ipc_import(hb, C.byref(out))
            if rc != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle from rank {r} failed ({rc})")
            self._opened.append(out.value)
            self.peer_ptrs.append(out.value + off)
        self._ptr_array = (C.c_void_p * self.world)(*self.peer_ptrs)
        self.seq = torch.zeros(1, dtype=torch.int32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        par.barrier()

    @classmethod
    def create(cls, par, device, max_tokens: int = 4096, max_width: int = 8192) -> "FusedComm":
        """Slots hold one [max_tokens, max_width] fp32 tensor (bf16 GEMM partials use half of it)."""
        return cls(par, device, slot_bytes=max_tokens * max_width * 4)

    # Collectives of at least this many rows per rank take the reduce-scatter form (each row goes to its owner only, the
    # owner sums and re-broadcasts bf16 rows): 2 (W-1)/W [T,H] on the wire instead of (W-1) [T,H].  Pays from 4 ranks up.
    RS_MIN_ROWS_PER_RANK = 64
    RS_MIN_WORLD = 99           # off until enabled (set to 4 to take the reduce-scatter form from four ranks up)

    def _rs_rows(self, T: int) -> int:
        if self.world < self.RS_MIN_WORLD or T < self.RS_MIN_ROWS_PER_RANK * self.world:
            return 0
        return (T + self.world - 1) // self.world

    def _owner_step(self, d: ReducedDelta) -> None:
        if d.rs_rows and not d.gathered:
            row0 = min(self.rank * d.rs_rows, d.T) if self.rank < self.world - 1 else min((self.world - 1) * d.rs_rows, d.T)
            row1 = min(row0 + d.rs_rows, d.T) if self.rank < self.world - 1 else d.T
            K._check(_lib.cuda().mx_comm_rs_gather(self._ptr_array, self.world, self.rank, C.c_longlong(self.slot_bytes), K._p(self.seq),
                                                   K._p(self.ticket), int(d.bf16), K._p(d.bias), row0, row1, d.H, K._stream()), "comm_rs_gather")
            K._count()
            d.gathered = True

    # ---- producers -----------------------------------------------------------------------
    @K._profiled("gemm_allreduce")
    def linear_all_reduce(self, x: torch.Tensor, w: QuantWeight, bias: Optional[torch.Tensor], rs_rows: Optional[int] = None) -> ReducedDelta:
        """``rs_rows``: force the reduce-scatter epilogue with that many rows per owner and leave the partials in the owners'
        inboxes (the row-sharded prefill path consumes them with ``ShardedComm.norm``)."""
        M = x.shape[0]
        fmt, p0, p1, p2, p3 = K._planes(w)
        lib = _lib.cuda()
        st = K._stream()
        # the bias of a row-parallel layer is added once, by the consumer (rank 0 carries it)
        if M <= K.GEMV_MAX_M:
            K._check(lib.mx_gemv_allreduce(fmt, p0, p1, p2, p3, K._p(x), _vp(0), M, w.N, w.K, self._ptr_array, self.world, self.rank,
                                           C.c_longlong(self.slot_bytes), K._p(self.seq), K._p(self.ticket), st), "gemv_allreduce")
            bf16 = False
        else:
            bf16 = True
            if M * w.N * 2 > self.slot_bytes:
                raise ValueError(f"fused all-reduce slot too small for [{M},{w.N}]")
            rs = self._rs_rows(M) if rs_rows is None else int(rs_rows)
            if fmt != int(K.WFormat.BF16) and M >= K.DEQUANT_ONCE_MIN_M:
                # quantised row-parallel weight: decode it once to bf16 (see ops.cuda.linear); the TMA-fed kernel is also the one
                # whose epilogue stages its peer stores into 128-byte row segments
                wb = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=x.device)
                K._check(lib.mx_dequant_bf16(fmt, p0, p1, p2, p3, C.c_longlong(w.N), w.K, K._p(wb), st), "dequant_bf16")
                K._count()
                fmt, p0, p1, p2, p3 = int(K.WFormat.BF16), K._p(wb), _vp(0), _vp(0), _vp(0)
            K._check(lib.mx_gemm_allreduce(K._p(x), fmt, p0, p1, p2, p3, _vp(0), 0, M, w.N, w.K, K._pick_bn(M, w.N), self._ptr_array, self.world,
                                           self.rank, C.c_longlong(self.slot_bytes), K._p(self.seq), K._p(self.ticket), rs, st), "gemm_allreduce")
            K._count()
            return ReducedDelta(self, M, w.N, bf16, bias, rs_rows=rs)
        K._count()
        return ReducedDelta(self, M, w.N, bf16, bias)

    def push(self, t: torch.Tensor) -> ReducedDelta:
        """All-reduce of an existing tensor (fp32 or bf16, contiguous): push now, sum in the consumer."""
        assert t.is_contiguous() and t.dtype in (torch.float32, torch.bfloat16)
        nbytes = t.numel() * t.element_size()
        K._check(_lib.cuda().mx_comm_push(K._p(t), C.c_longlong(nbytes), self._ptr_array, self.world, self.rank, C.c_longlong(self.slot_bytes),
                                          K._p(self.seq), K._p(self.ticket), K._stream()), "comm_push")
        K._count()
        return ReducedDelta(self, t.shape[0], t.shape[1], t.dtype == torch.bfloat16)

    @K._profiled("moe_combine_push")
    def moe_combine_push(self, yp: torch.Tensor, pair_to_packed: torch.Tensor, w: torch.Tensor) -> ReducedDelta:
        """MoE combine fused with the expert-parallel all-reduce: sum_k w[t,k] * yp[pos(t,k)] goes straight into every rank's
        inbox (fp32 for decode-sized batches, bf16 for prefill, like the row-parallel GEMM partials)."""
        T, Kt = w.shape
        H = yp.shape[1]
        f32 = T <= K.GEMV_MAX_M
        rs = 0 if f32 else self._rs_rows(T)
        K._check(_lib.cuda().mx_moe_combine_push(K._p(yp), K._p(pair_to_packed), K._p(w), int(f32), T, H, Kt, self._ptr_array, self.world, self.rank,
                                                 C.c_longlong(self.slot_bytes), K._p(self.seq), K._p(self.ticket), rs, K._stream()), "moe_combine_push")
        K._count()
        return ReducedDelta(self, T, H, not f32, rs_rows=rs)

    # ---- consumers -----------------------------------------------------------------------
    def reduce(self, d: ReducedDelta) -> torch.Tensor:
        out = torch.empty(d.T, d.H, dtype=torch.float32, device=self.device)
        self._owner_step(d)
        g = int(d.gathered)
        K._check(_lib.cuda().mx_comm_reduce(_vp(self.peer_ptrs[self.rank]), self.world, C.c_longlong(self.slot_bytes), K._p(self.seq), 1 if g else int(d.bf16),
                                            None if g else K._p(d.bias), K._p(out), C.c_longlong(d.T * d.H), d.H, g, K._stream()), "comm_reduce")
        K._count()
        return out

    @K._profiled("rmsnorm_reduce")
    def rmsnorm(self, x: torch.Tensor, w: torch.Tensor, eps: float, d: ReducedDelta, one_plus_w: bool = False, delta_scale: float = 1.0,
                want_out: bool = True) -> Optional[torch.Tensor]:
        T, H = x.shape
        out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if want_out else None
        self._owner_step(d)
        g = int(d.gathered)
        K._check(_lib.cuda().mx_comm_rmsnorm_reduce(K._p(x), _vp(self.peer_ptrs[self.rank]), self.world, C.c_longlong(self.slot_bytes), K._p(self.seq),
                                                    1 if g else int(d.bf16), None if g else K._p(d.bias), K._p(w), K._p(out), C.c_float(eps), T, H,
                                                    int(one_plus_w), C.c_float(delta_scale), g, K._stream()), "comm_rmsnorm_reduce")
        K._count()
        return out

    def close(self) -> None:
        lib = _lib.cuda()
        for p in self._opened:
            lib.mx_ipc_release(_vp(p))
        self._opened = []
        if self._base:
            lib.mx_raw_free(_vp(self._base))
            self._base = None
