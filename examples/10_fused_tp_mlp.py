"""Tensor-parallel MLP on the fused kernels: all-gather -> GEMM and GEMM -> reduce-scatter in one launch each.

Run:  python -m mintccl_b200.launch -np 2 examples/10_fused_tp_mlp.py     (or torchrun; one process per GPU)
Needs GPUs (tcgen05 kernels); on a machine without CUDA it says so and exits 0.  The forward pass is checked
against the same block computed without tensor parallelism in fp32, the MXFP8 projection against the product
of the dequantised operands.  MINTCCL_TEST_COUNT sets the number of tokens (rounded to 256 x world).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mintccl_b200 as m  # noqa: E402

rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
if not torch.cuda.is_available():
    print(f"# rank {rank}: the fused GEMM kernels need a GPU (sm_100a); nothing to do on the CPU backend", flush=True)
    sys.exit(0)
m.set_gpu(int(os.environ.get("LOCAL_RANK", rank)))
comm = m.init()
from mintccl_b200.models.tp_mlp import TensorParallelMLP  # noqa: E402
from mintccl_b200.ops import mxfp8 as mx  # noqa: E402
from mintccl_b200.ops.gemm import AllGatherGemm  # noqa: E402

unit = 256 * world
T = max(unit, int(os.environ.get("MINTCCL_TEST_COUNT", 2048)) // unit * unit)
H, F = 1024, 512 * world
ok = True


def check(what, cond):
    global ok
    ok = ok and bool(cond)
    print(f"# rank {rank}, {what}: {bool(cond)}", flush=True)


def gather(t):
    """Every rank's tensor, concatenated along dim 0 (plain all-gather of this library)."""
    buf = comm.symm_empty((world,) + tuple(t.shape), t.dtype)
    comm.allgather(buf, inp=t.contiguous())
    return buf.flatten(0, 1)


# ---- bf16 block, forward and backward
mlp = TensorParallelMLP(comm, T, H, F)
x_full = torch.randn(T, H, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).cuda()
x_shard = x_full[rank * (T // world):(rank + 1) * (T // world)].clone().requires_grad_(True)
y_shard = mlp(x_shard)                                        # [T / world, H]
y_shard.float().pow(2).mean().backward()
torch.cuda.synchronize()
comm.check()
w_up = gather(mlp.w_up.detach())                              # [F, H]: the column-parallel weight, whole
w_down = gather(mlp.w_down.detach().t().contiguous()).t()     # [H, F]: the row-parallel weight, whole
ref = torch.nn.functional.silu(x_full.float() @ w_up.float().t()) @ w_down.float().t()
mine = ref[rank * (T // world):(rank + 1) * (T // world)]
check("fused MLP forward", torch.allclose(y_shard.detach().float(), mine, rtol=5e-2, atol=5e-2))
check("gradients", all(g is not None and bool(torch.isfinite(g.float()).all()) for g in (x_shard.grad, mlp.w_up.grad, mlp.w_down.grad)))

# ---- the up projection on block-scaled fp8 operands (e4m3 payload, one power-of-two scale per 32 elements)
plan = AllGatherGemm(comm, T, F // world, H, fp8=True)
qx = mx.quantize_rows_mxfp8(x_shard.detach().float())
qw = mx.quantize_rows_mxfp8(mlp.w_up.detach().float())
h8 = plan.call_mxfp8(qx[0], qx[1], qw[0], qw[1])              # [T, F / world] bf16
torch.cuda.synchronize()
comm.check()
x_dq = gather(mx.dequantize_mxfp8(qx[0].reshape(-1), qx[1].reshape(-1)).view(T // world, H))
w_dq = mx.dequantize_mxfp8(qw[0].reshape(-1), qw[1].reshape(-1)).view(F // world, H)
check("MXFP8 all-gather -> GEMM", torch.allclose(h8.float(), x_dq @ w_dq.t(), rtol=2e-2, atol=5e-2))

m.shutdown()
sys.exit(0 if ok else 1)
