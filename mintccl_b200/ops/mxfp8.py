"""MXFP8 (block-scaled fp8) tensors and their sum over ranks.

Format: ``float8_e4m3fn`` payload, one ``ue8m0`` scale byte (a power of two, value ``2 ** (e - 127)``) per
block of 32 consecutive elements.  The scale of a block is the smallest power of two that brings the
block's largest magnitude to at most 448, the largest e4m3 value, so quantisation never saturates.

``allreduce_mxfp8`` / ``reducescatter_mxfp8`` sum such tensors over the ranks with fp32 accumulation and a
single requantisation (kernel: ``csrc/kernels/mxfp8.cu``).  The torch functions here are the oracle for the
kernel and a convenience for callers.  fp8 reductions are on the reference's roadmap only (README.md:58-60).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from .. import _native as N

BLOCK = 32
TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]


def scale_for_amax(amax: torch.Tensor) -> torch.Tensor:
    """ue8m0 byte of the smallest power of two ``s`` with ``amax / s <= 448`` (fp32 in, uint8 out)."""
    m, e = torch.frexp(amax.float())            # amax = m * 2**e, m in [0.5, 1)
    s = e - 9 + (m * 2 > 1.75).to(e.dtype) + 127
    s = torch.where(amax > 0, s, torch.full_like(s, 127 - 8))
    return s.clamp(1, 254).to(torch.uint8)


def scale_to_float(scale: torch.Tensor) -> torch.Tensor:
    return torch.pow(2.0, scale.float() - 127.0)


def quantize_mxfp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32/bf16/fp16 tensor (numel a multiple of 32) -> (payload uint8 [numel], scales uint8 [numel / 32])."""
    flat = x.detach().float().reshape(-1, BLOCK)
    scale = scale_for_amax(flat.abs().amax(dim=1))
    q = (flat / scale_to_float(scale)[:, None]).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(-1), scale


def dequantize_mxfp8(data: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (data.view(torch.float8_e4m3fn).float().reshape(-1, BLOCK) * scale_to_float(scale)[:, None]).reshape(-1)


def _lists(comm, t):
    ts = [t] if isinstance(t, torch.Tensor) else list(t)
    if len(ts) != comm.nlocal:
        raise ValueError(f"expected {comm.nlocal} tensors")
    return ts


def _off(comm, ts, what):
    offs = [comm.symm_offset(t, lr) for lr, t in enumerate(ts)]
    if offs[0] is None or any(o != offs[0] for o in offs):
        raise ValueError(f"{what} must come from the symmetric heap (same offset on every rank)")
    return offs[0]


def _cpu_reduce(comm, data: torch.Tensor, scale: torch.Tensor, out_data: torch.Tensor, out_scale: torch.Tensor,
                scatter: bool) -> None:
    """The same sum on the CPU reference backend (gloo): dequantise, add in fp32 across the ranks, quantise once."""
    if scale.numel() * BLOCK != data.numel():
        raise ValueError("one scale byte per 32 payload bytes")
    total = comm._sum_fp32(dequantize_mxfp8(data.reshape(-1), scale.reshape(-1)))
    if scatter:
        per = total.numel() // comm.world_size
        if per % BLOCK or per * comm.world_size != total.numel():
            raise ValueError("the blocks must divide evenly over the ranks")
        total = total[comm.rank * per:(comm.rank + 1) * per]
    q, sc = quantize_mxfp8(total)
    out_data.reshape(-1).copy_(q)
    out_scale.reshape(-1).copy_(sc)


def allreduce_mxfp8(comm, data: TensorOrList, scale: TensorOrList, out_data: Optional[TensorOrList] = None,
                    out_scale: Optional[TensorOrList] = None, nctas: int = 64) -> None:
    """Sum the MXFP8 tensors of all ranks; the result (requantised once) replaces ``data`` / ``scale`` on every
    rank, or goes to ``out_data`` / ``out_scale``.  All tensors must be symmetric uint8 tensors."""
    if not hasattr(comm, "lib"):
        return _cpu_reduce(comm, data, scale, out_data if out_data is not None else data,
                           out_scale if out_scale is not None else scale, scatter=False)
    d, s = _lists(comm, data), _lists(comm, scale)
    od = _lists(comm, out_data) if out_data is not None else d
    os_ = _lists(comm, out_scale) if out_scale is not None else s
    n_el = d[0].numel()
    if s[0].numel() * BLOCK != n_el:
        raise ValueError("one scale byte per 32 payload bytes")
    rc = comm.lib.mt_mxfp8_reduce(comm._handle, comm._stream(), 0, _off(comm, d, "data"), _off(comm, s, "scale"),
                                  _off(comm, od, "out_data"), _off(comm, os_, "out_scale"), None, None, n_el, nctas)
    if rc < 0:
        raise RuntimeError(f"mt_mxfp8_reduce: {N.last_error()}")


def reducescatter_mxfp8(comm, data: TensorOrList, scale: TensorOrList, out_data: TensorOrList, out_scale: TensorOrList,
                        nctas: int = 64) -> None:
    """Shard ``rank`` (a contiguous 1/world of the blocks) of the sum lands in the local ``out_data`` / ``out_scale``."""
    if not hasattr(comm, "lib"):
        return _cpu_reduce(comm, data, scale, out_data, out_scale, scatter=True)
    d, s = _lists(comm, data), _lists(comm, scale)
    od, os_ = _lists(comm, out_data), _lists(comm, out_scale)
    n_el = d[0].numel()
    rc = comm.lib.mt_mxfp8_reduce(comm._handle, comm._stream(), 1, _off(comm, d, "data"), _off(comm, s, "scale"), 0, 0,
                                  N.ptr_array([t.data_ptr() for t in od]), N.ptr_array([t.data_ptr() for t in os_]),
                                  n_el, nctas)
    if rc < 0:
        raise RuntimeError(f"mt_mxfp8_reduce: {N.last_error()}")


# ---- MXFP8 GEMM operands -------------------------------------------------------------------------------------
def quantize_rows_mxfp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[rows, K]`` -> (payload uint8 ``[rows, K]``, scales uint8 ``[rows, K / 32]``): blocks of 32 along K."""
    rows, K = x.shape
    data, scale = quantize_mxfp8(x.contiguous())
    return data.view(rows, K), scale.view(rows, K // BLOCK)


def tile_scales(scale: torch.Tensor) -> torch.Tensor:
    """Row-major scales ``[rows, K / 32]`` -> the layout the tensor core reads: ``[rows / 128][K / 128][512]`` bytes
    with byte ``(r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4`` for row ``r`` and 32-element block ``kb``."""
    rows, kb = scale.shape
    if rows % 128 or kb % 4:
        raise ValueError("rows must be a multiple of 128 and K of 128")
    t = scale.view(rows // 128, 4, 32, kb // 4, 4)       # [R, r/32, r%32, KB, kb%4]
    return t.permute(0, 3, 2, 1, 4).contiguous().view(-1)  # [R, KB, r%32, r/32, kb%4]


def gemm_mxfp8(a_data: torch.Tensor, a_scale: torch.Tensor, w_data: torch.Tensor, w_scale: torch.Tensor,
               out: Optional[torch.Tensor] = None, nctas: int = 0, scales_tiled: bool = False) -> torch.Tensor:
    """``dequant(a) [M, K] @ dequant(w)[N, K].T -> bf16 [M, N]`` on the block-scaled tensor cores
    (``tcgen05.mma.kind::mxf8f6f4.block_scale``).  ``a_scale`` / ``w_scale`` are row-major ``[rows, K / 32]``,
    or already in the tensor-core layout of ``tile_scales`` (``scales_tiled``: weights are tiled once, not per call)."""
    M, K = a_data.shape
    Nn = w_data.shape[0]
    if out is None:
        out = torch.empty(M, Nn, device=a_data.device, dtype=torch.bfloat16)
    sfa, sfb = (a_scale, w_scale) if scales_tiled else (tile_scales(a_scale), tile_scales(w_scale))
    stream = torch.cuda.current_stream(a_data.device).cuda_stream
    rc = N.lib().mt_gemm_mxfp8(stream, a_data.data_ptr(), sfa.data_ptr(), w_data.data_ptr(), sfb.data_ptr(),
                               out.data_ptr(), M, Nn, K, out.stride(0), nctas)
    if rc < 0:
        raise RuntimeError(f"mt_gemm_mxfp8: {N.last_error()}")
    return out
