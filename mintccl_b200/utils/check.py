"""Element-wise error bounds for sums over ranks, shared by the benchmark's self-check and the examples.

The reference compares its reductions with NCCL bit for bit (5_reduce.py:145, 7_reducescatter.py:117), which
cannot hold once the order of the additions differs.  The bounds here follow from the arithmetic instead of being
blanket tolerances: the one-hop kernels (direct, NVLS, one-shot) add all ranks in fp32 and round once into the
output type, so the error is at most half an ulp of the result plus the fp32 accumulation error; a ring rounds the
partial sum into the storage type at each combine, and a partial sum is at most ``sum |x_r|``.
"""
from __future__ import annotations

from typing import Sequence

import torch


def sum_oracle(srcs: Sequence[torch.Tensor]):
    """fp32 sum of the ranks' inputs (added in rank order) and the sum of their magnitudes."""
    ref = torch.zeros_like(srcs[0], dtype=torch.float32)
    absum = torch.zeros_like(ref)
    for s in srcs:
        ref += s.float()
        absum += s.float().abs()
    return ref, absum


def sum_error_bound(ref: torch.Tensor, absum: torch.Tensor, dtype: torch.dtype, nranks: int, hops: int = 1) -> torch.Tensor:
    half = torch.finfo(dtype).eps / 2
    acc_err = nranks * 2.0 ** -22 * absum
    if hops <= 1 or dtype == torch.float32:
        bound = 1.01 * half * ref.abs() + acc_err
    else:
        bound = 1.01 * half * hops * absum + acc_err
    return bound + torch.finfo(dtype).smallest_normal * torch.finfo(dtype).eps


def sum_within_bound(got: torch.Tensor, srcs: Sequence[torch.Tensor], hops: int = 1) -> bool:
    """True if ``got`` is the sum of ``srcs`` up to the rounding its type and the number of combines allow."""
    ref, absum = sum_oracle(srcs)
    err = (got.float() - ref).abs()
    return not bool((err > sum_error_bound(ref, absum, got.dtype, len(srcs), hops)).any())
