"""Tensor-parallel MLP block (Megatron-style column-parallel up projection, row-parallel down
projection, activations sharded over tokens between blocks) built on the fused kernels:

    x_shard [T / n, H]  --all-gather -> GEMM-->  h [T, F / n]  --act-->  --GEMM -> reduce-scatter-->  y_shard [T / n, H]

The forward pass is two kernel launches (``AllGatherGemm``, ``GemmReduceScatter``) plus the activation.
The backward pass runs the transposed products through the same tcgen05 GEMM and the library's own
collectives.  This is the "fuse the collectives with your own kernels" use case the reference names as its
purpose (README.md:5) but does not implement; the shapes of the benchmark are the Llama-3-8B MLP ones
(tokens 8192, hidden 4096, ffn 14336, TP = 8).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.gemm import AllGatherGemm, GemmReduceScatter, gemm


class _MLPFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w_up, w_down, mlp):
        h = mlp.ag_gemm(x_shard, w_up)                       # [T, F/n]
        a = torch.nn.functional.silu(h)
        y = mlp.gemm_rs(a, w_down)                           # [T/n, H]
        ctx.mlp = mlp
        ctx.save_for_backward(x_shard, w_up, w_down, h, a)
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        mlp = ctx.mlp
        comm = mlp.comm
        x_shard, w_up, w_down, h, a = ctx.saved_tensors
        n, T = comm.world_size, mlp.tokens
        dy_shard = dy_shard.contiguous()
        # all-gather dy and x over tokens (plain collectives of this library)
        dy = mlp._gather(dy_shard)                           # [T, H]
        x = mlp.ag_gemm.gathered if n > 1 else x_shard       # gathered x is still in the plan's buffer
        if n > 1:
            x = x.clone()
            x[comm.rank * (T // n):(comm.rank + 1) * (T // n)].copy_(x_shard)
        # da = dy @ w_down            (w_down: [H, F/n])  -> B operand is w_down^T stored [F/n, H]
        da = gemm(dy, w_down.t().contiguous())               # [T, F/n]
        dw_down = gemm(dy.t().contiguous(), a.t().contiguous())   # [H, F/n] = dy^T @ a
        sig = torch.sigmoid(h.float())
        dh = (da.float() * (sig * (1 + h.float() * (1 - sig)))).to(torch.bfloat16)
        dw_up = gemm(dh.t().contiguous(), x.t().contiguous())     # [F/n, H] = dh^T @ x
        # dx = reduce_scatter(dh @ w_up)   (w_up: [F/n, H]) -> B operand [H, F/n]
        dx_shard = mlp.gemm_rs_bwd(dh, w_up.t().contiguous())
        return dx_shard, dw_up, dw_down, None


class TensorParallelMLP(torch.nn.Module):
    """``tokens`` is the global token count of a step (fixed: the fused plans own buffers of that size)."""

    def __init__(self, comm, tokens: int, hidden: int, ffn: int, ncomm: Optional[int] = None, seed: int = 0):
        super().__init__()
        n = comm.world_size
        if ffn % n or tokens % n:
            raise ValueError("ffn and tokens must be divisible by the world size")
        self.comm, self.tokens, self.hidden, self.ffn_local = comm, tokens, hidden, ffn // n
        dev = torch.device("cuda", comm.device)
        g = torch.Generator(device=dev).manual_seed(seed + 1000 * comm.rank)
        self.w_up = torch.nn.Parameter((torch.randn(self.ffn_local, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16))
        self.w_down = torch.nn.Parameter((torch.randn(hidden, self.ffn_local, generator=g, device=dev) * 0.02).to(torch.bfloat16))
        self.ag_gemm = AllGatherGemm(comm, tokens, self.ffn_local, hidden, ncomm=ncomm)
        self.gemm_rs = GemmReduceScatter(comm, tokens, hidden, self.ffn_local)
        self.gemm_rs_bwd = GemmReduceScatter(comm, tokens, hidden, self.ffn_local)
        self._gbuf: Optional[torch.Tensor] = None

    def _gather(self, shard: torch.Tensor) -> torch.Tensor:
        n = self.comm.world_size
        if n == 1:
            return shard
        if self._gbuf is None:
            self._gbuf = self.comm.symm_empty((n, shard.shape[0], shard.shape[1]), torch.bfloat16)
        self.comm.allgather(self._gbuf, inp=shard)
        return self._gbuf.view(-1, shard.shape[1])

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        return _MLPFunction.apply(x_shard, self.w_up, self.w_down, self)


def smoke_mlp() -> None:
    """One tiny forward + backward of the block on ``cuda:0`` (world size 1), checked against PyTorch."""
    import mintccl_b200
    from mintccl_b200 import Config
    cfg = Config.from_env(max_channels=2, num_blocks=2, buff_size=1 << 20, heap_bytes=256 << 20, scratch_bytes=1 << 20,
                          wait_timeout_ms=4000)
    from mintccl_b200.parallel.rendezvous import SingleControl
    comm = mintccl_b200.Communicator(control=SingleControl(), device=0, config=cfg)
    T, H, F = 256, 256, 512
    mlp = TensorParallelMLP(comm, T, H, F)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_(True)
    y = mlp(x)
    y.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    comm.check()
    ref = torch.nn.functional.silu(x.detach().float() @ mlp.w_up.detach().float().t()) @ mlp.w_down.detach().float().t()
    torch.testing.assert_close(y.detach().float(), ref, rtol=5e-2, atol=5e-2)
    assert x.grad is not None and mlp.w_up.grad is not None and mlp.w_down.grad is not None
    assert torch.isfinite(x.grad.float()).all()
    comm.close()
