"""bf16 GEMM on the tcgen05 tensor cores and its fusions with collectives.

* ``gemm(a, w)``                : ``a @ w.T`` (``w`` is ``[N, K]`` like ``nn.Linear.weight``).
* ``AllGatherGemm`` (``ag_gemm``): ``allgather(a_shard) @ w.T`` for a column-parallel layer whose input is
  sharded over the token dimension (sequence parallelism).  One kernel: a few CTAs push this rank's rows
  to the peers while the others multiply, starting with the rows that are already there.
* ``GemmReduceScatter`` (``gemm_rs``): ``reduce_scatter(a @ w.T)`` over token rows for a row-parallel
  layer.  One kernel: partial tiles go straight from the epilogue into the owner's memory over NVLink, the
  owner sums them in fp32.

Shapes: tokens ``M`` a multiple of ``128 * world``, ``N`` of 256, ``K`` of 64.  The reference has no such
ops; its README (README.md:5) names fusion with other kernels as the purpose of the library.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from .. import _native as N

TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]
BM, BN, BK = 128, 256, 64


def _check(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous() or t.dim() != 2:
        raise ValueError(f"{name} must be a contiguous 2-D bfloat16 CUDA tensor")


def gemm(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, nctas: int = 0) -> torch.Tensor:
    """``a [M, K] @ w[N, K].T -> [M, N]`` in bf16 with fp32 accumulation (hand-written tcgen05 kernel)."""
    _check(a, "a")
    _check(w, "w")
    M, K = a.shape
    Nn, K2 = w.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if out is None:
        out = torch.empty(M, Nn, device=a.device, dtype=torch.bfloat16)
    _check(out, "out")
    stream = torch.cuda.current_stream(a.device).cuda_stream
    if N.lib().mt_gemm(stream, a.data_ptr(), w.data_ptr(), out.data_ptr(), M, Nn, K, out.stride(0), nctas) < 0:
        raise RuntimeError(f"mt_gemm: {N.last_error()}")
    return out


class _Fused:
    def __init__(self, comm):
        self.comm = comm
        self.epoch = 0

    def _lists(self, t: TensorOrList) -> List[torch.Tensor]:
        ts = [t] if isinstance(t, torch.Tensor) else list(t)
        if len(ts) != self.comm.nlocal:
            raise ValueError(f"expected {self.comm.nlocal} tensors")
        return ts

    def _off(self, t: TensorOrList) -> int:
        t0 = t[0] if isinstance(t, (list, tuple)) else t
        return t0.data_ptr() - self.comm.heap_base[0]


class AllGatherGemm(_Fused):
    """Plan for ``allgather(a_shard)[M, K] @ w[N, K].T``: owns the gathered-input buffer and the arrival
    counters in the symmetric heap.  Create it collectively (same order on every rank), call it every step."""

    # "fan": every 32 KiB piece of this rank's rows is read once and stored to all peers from shared memory
    MODES = {"push": 0, "pull": 1, "push_st": 2, "fan": 3}

    def __init__(self, comm, M: int, N_: int, K: int, ncomm: Optional[int] = None, mode: str = "push", split: int = 1,
                 fp8: bool = False):
        super().__init__(comm)
        self.mode = self.MODES[mode]
        self.fp8 = fp8
        if ncomm is None:
            nw = comm.world_size
            ncomm = self.pick_ncomm((M // BM) * (N_ // BN), flops=2.0 * M * N_ * K,
                                    bytes_in=(nw - 1) / max(nw, 1) * M * K * (1 if fp8 else 2), fp8=fp8)
        self.split = max(1, min(split, ncomm))
        n = comm.world_size
        if mode == "fan" and split == 1 and n > 1:
            # the work units of the fan-out push are this rank's 128-row chunks: more comm CTAs than chunks share them
            chunks = max(1, M // n // BM)
            ncomm = (ncomm + 1) & ~1
            sp = max(1, ncomm // min(ncomm, chunks))
            while ncomm % sp:
                sp -= 1
            self.split = sp
        if M % (BM * n) or N_ % BN or K % BK:
            raise ValueError("M must be a multiple of 128 x world, N of 256, K of 64")
        self.M, self.N, self.K, self.ncomm = M, N_, K, ncomm
        if fp8 and K % 128:
            raise ValueError("MXFP8: K must be a multiple of 128")
        self.gathered = comm.symm_empty((M, K), torch.uint8 if fp8 else torch.bfloat16)
        # MXFP8: the tiled scales of all ranks' rows, gathered by a small all-gather before the fused kernel
        self.sfa_all = comm.symm_empty((n, (M // n // 128) * (K // 128) * 512), torch.uint8) if fp8 else None
        self.flags = comm.symm_zeros((n * (M // n // BM),), torch.int64)
        torch.cuda.synchronize()
        comm.control.barrier()

    def call_mxfp8(self, a_data: TensorOrList, a_scale: TensorOrList, w_data: TensorOrList, w_scale: TensorOrList,
                   out: Optional[TensorOrList] = None, nctas: int = 0, w_scale_tiled: bool = False):
        """MXFP8 operands: ``a_data`` uint8 ``[M / n, K]`` (e4m3) with row-major scales ``[M / n, K / 32]``, ``w_data``
        ``[N, K]`` with scales ``[N, K / 32]`` (or already in the layout of ``ops.mxfp8.tile_scales`` with
        ``w_scale_tiled``: weights are tiled once); bf16 result.  The payload rows are gathered inside the fused
        kernel, the (32 x smaller) scales by an all-gather of this library just before it."""
        from . import mxfp8 as mx
        if not self.fp8:
            raise ValueError("create the plan with fp8=True")
        c = self.comm
        a_s, ws = self._lists(a_data), self._lists(w_data)
        a_sc, w_sc = self._lists(a_scale), self._lists(w_scale)
        outs = self._lists(out) if out is not None else [torch.empty(self.M, self.N, device=a_s[0].device, dtype=torch.bfloat16) for _ in a_s]
        ranks = range(c.world_size) if c.emulated else [c.rank]
        sfa_all = self.sfa_all if c.emulated else [self.sfa_all]
        for lr, r in enumerate(ranks):
            sfa_all[lr][r].copy_(mx.tile_scales(a_sc[lr]))
        c.allgather(self.sfa_all)
        sfb = list(w_sc) if w_scale_tiled else [mx.tile_scales(t) for t in w_sc]
        self.epoch += 1
        rc = c.lib.mt_ag_gemm_mxfp8(c._handle, c._stream(), N.ptr_array([t.data_ptr() for t in a_s]),
                                    N.ptr_array([t.data_ptr() for t in sfa_all]), N.ptr_array([t.data_ptr() for t in ws]),
                                    N.ptr_array([t.data_ptr() for t in sfb]), N.ptr_array([t.data_ptr() for t in outs]),
                                    self._off(self.gathered), self._off(self.flags), self.epoch, self.M, self.N, self.K,
                                    outs[0].stride(0), self.ncomm, nctas)
        if rc < 0:
            raise RuntimeError(f"mt_ag_gemm_mxfp8: {N.last_error()}")
        self._keep = sfb  # the kernel reads them asynchronously
        return outs if c.emulated else outs[0]

    @staticmethod
    def pick_ncomm(tiles: int, sms: int = 148, lo: int = 16, hi: int = 24, flops: Optional[float] = None,
                   bytes_in: Optional[float] = None, fp8: bool = False) -> int:
        """Comm CTAs for a problem of ``tiles`` output tiles.  The transfer has to keep pace with the GEMM and no
        more: one comm CTA moves about 28 GB/s (24 of them 680 GB/s on 8 GPUs), the GEMM CTAs sustain about
        1.3 PFLOP/s in bf16 and 2.2 in MXFP8, so ``bytes_in / (flops / rate) / 28e9`` CTAs (plus a quarter) are
        wanted, at most ``hi``; a GEMM-bound problem (few ranks, wide N) gets few and keeps its SMs.  Among the
        allowed counts the GEMM takes ceil(tiles / (sms - ncomm)) waves: take the most comm CTAs that do not add
        a wave over the fewest allowed."""
        if flops and bytes_in is not None:
            t = flops / (2.2e15 if fp8 else 1.3e15)
            want = int(bytes_in / t / 28e9 * 1.25) + 1
            hi = max(2, min(hi, want))
            lo = max(2, min(lo, hi - 2))
        waves = lambda nc: -(-tiles // (sms - nc))  # noqa: E731
        best = min(waves(nc) for nc in range(lo, hi + 1))
        return max(nc for nc in range(lo, hi + 1) if waves(nc) == best)

    def __call__(self, a_shard: TensorOrList, w: TensorOrList, out: Optional[TensorOrList] = None, nctas: int = 0):
        c = self.comm
        a_s, ws = self._lists(a_shard), self._lists(w)
        if out is None:
            outs = [torch.empty(self.M, self.N, device=a_s[0].device, dtype=torch.bfloat16) for _ in a_s]
        else:
            outs = self._lists(out)
        for t in a_s + ws + outs:
            _check(t, "operand")
        if tuple(a_s[0].shape) != (self.M // c.world_size, self.K) or tuple(ws[0].shape) != (self.N, self.K):
            raise ValueError("operand shapes do not match the plan")
        shard_off = 0
        if self.mode == 1:  # the peers read this rank's rows: they must sit at the same heap offset everywhere
            offs = [c.symm_offset(t, lr) for lr, t in enumerate(a_s)]
            if offs[0] is None or any(o != offs[0] for o in offs):
                raise ValueError("mode='pull' needs a_shard from the symmetric heap")
            shard_off = offs[0]
        self.epoch += 1
        rc = c.lib.mt_ag_gemm(c._handle, c._stream(), N.ptr_array([t.data_ptr() for t in a_s]),
                              N.ptr_array([t.data_ptr() for t in ws]), N.ptr_array([t.data_ptr() for t in outs]),
                              self._off(self.gathered), self._off(self.flags), self.epoch, self.M, self.N, self.K,
                              outs[0].stride(0), self.ncomm, nctas, self.mode, shard_off, self.split)
        if rc < 0:
            raise RuntimeError(f"mt_ag_gemm: {N.last_error()}")
        return outs if c.emulated else outs[0]


class GemmReduceScatter(_Fused):
    """Plan for ``reduce_scatter(a[M, K_local] @ w[N, K_local].T)`` over token rows: owns the staging area
    for partial tiles (double-buffered across calls) and their arrival counters in the symmetric heap."""

    def __init__(self, comm, M: int, N_: int, K: int, nred: Optional[int] = None):
        super().__init__(comm)
        n = comm.world_size
        if M % (BM * n) or N_ % BN or K % BK:
            raise ValueError("M must be a multiple of 128 x world, N of 256, K of 64")
        self.M, self.N, self.K = M, N_, K
        if nred is None:
            nred = self.pick_nred(M, N_, K, n)
        self.nred = nred if n > 1 else 0
        # two halves used alternately: a fast peer may already write the next call's partial tiles while this
        # rank still reduces the current ones
        self.stage = comm.symm_empty((2, n, M // n, N_), torch.bfloat16)
        self.flags = comm.symm_zeros((n * (M // n // BM) * (N_ // BN) + 2,), torch.int64)
        torch.cuda.synchronize()
        comm.control.barrier()

    @staticmethod
    def pick_nred(M: int, N_: int, K: int, n: int) -> int:
        """Dedicated reducer CTAs: they read n partial tiles and write one for every output tile of this rank while
        the GEMM runs, about 70 GB/s per CTA (12 CTAs keep up with the 8-rank Llama-3-8B down projection:
        75 MB in 92 us).  A longer GEMM over the same bytes needs fewer, which leaves the SMs to the GEMM."""
        t = 2.0 * M * N_ * K / 1.3e15
        bytes_red = (M // n) * N_ * 2.0 * (n + 1)
        return max(2, min(16, int(bytes_red / t / 70e9 + 0.999)))

    def __call__(self, a: TensorOrList, w: TensorOrList, out: Optional[TensorOrList] = None, nctas: int = 0):
        c = self.comm
        a_s, ws = self._lists(a), self._lists(w)
        rows = self.M // c.world_size
        if out is None:
            outs = [torch.empty(rows, self.N, device=a_s[0].device, dtype=torch.bfloat16) for _ in a_s]
        else:
            outs = self._lists(out)
        for t in a_s + ws + outs:
            _check(t, "operand")
        if tuple(a_s[0].shape) != (self.M, self.K) or tuple(ws[0].shape) != (self.N, self.K):
            raise ValueError("operand shapes do not match the plan")
        self.epoch += 1
        rc = c.lib.mt_gemm_rs(c._handle, c._stream(), N.ptr_array([t.data_ptr() for t in a_s]),
                              N.ptr_array([t.data_ptr() for t in ws]), N.ptr_array([t.data_ptr() for t in outs]),
                              self._off(self.stage), self._off(self.flags), self.epoch, self.M, self.N, self.K,
                              min(self.nred, 148 // c.nlocal - 1) if c.emulated else self.nred, nctas)
        if rc < 0:
            raise RuntimeError(f"mt_gemm_rs: {N.last_error()}")
        return outs if c.emulated else outs[0]

    def call_mxfp8(self, a_data: TensorOrList, a_scale: TensorOrList, w_data: TensorOrList, w_scale: TensorOrList,
                   out: Optional[TensorOrList] = None, nctas: int = 0, w_scale_tiled: bool = False):
        """MXFP8 operands (e4m3 payloads, row-major ue8m0 scales per 32 elements along K; ``w_scale_tiled``: the
        weight scales are already in the layout of ``ops.mxfp8.tile_scales``); bf16 partial tiles and result,
        fp32 accumulation in the tensor core and in the cross-rank sum."""
        from . import mxfp8 as mx
        c = self.comm
        a_s, ws = self._lists(a_data), self._lists(w_data)
        rows = self.M // c.world_size
        outs = self._lists(out) if out is not None else [torch.empty(rows, self.N, device=a_s[0].device, dtype=torch.bfloat16) for _ in a_s]
        sfa = [mx.tile_scales(t) for t in self._lists(a_scale)]
        sfb = list(self._lists(w_scale)) if w_scale_tiled else [mx.tile_scales(t) for t in self._lists(w_scale)]
        self.epoch += 1
        rc = c.lib.mt_gemm_rs_mxfp8(c._handle, c._stream(), N.ptr_array([t.data_ptr() for t in a_s]),
                                    N.ptr_array([t.data_ptr() for t in sfa]), N.ptr_array([t.data_ptr() for t in ws]),
                                    N.ptr_array([t.data_ptr() for t in sfb]), N.ptr_array([t.data_ptr() for t in outs]),
                                    self._off(self.stage), self._off(self.flags), self.epoch, self.M, self.N, self.K,
                                    min(self.nred, 148 // c.nlocal - 1) if c.emulated else self.nred, nctas)
        if rc < 0:
            raise RuntimeError(f"mt_gemm_rs_mxfp8: {N.last_error()}")
        self._keep = (sfa, sfb)
        return outs if c.emulated else outs[0]
