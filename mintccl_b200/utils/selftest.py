"""Self-test mode of the example scripts: ``MINTCCL_TEST_MODE=1`` also runs the equivalent operation through
``torch.distributed`` (NCCL on GPUs, gloo on the CPU backend) and prints ``# rank r, <what> vs torch.distributed:
equal|close: True|False``; ``MINTCCL_TEST_VERBOSE=1`` adds the first and last 16 elements of both results.

This is the oracle branch of the reference's scripts (``if TEST_MODE:`` in 1_sendrecv_direct.py:93-107,
4_broadcast.py:110-126, 5_reduce.py:138-155, 6_allgather.py:172-179, 7_reducescatter.py:105-117).  Copies are
compared bit for bit.  Sums are compared within a few units in the last place of the element type: the reference
uses ``torch.equal`` there too (5_reduce.py:145), which cannot hold once two libraries add in different orders.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..config import env_bool


def enabled() -> bool:
    return env_bool("MINTCCL_TEST_MODE", False)


def verbose() -> bool:
    return env_bool("MINTCCL_TEST_VERBOSE", False)


class TorchOracle:
    """The same collectives through torch.distributed, on copies of the inputs."""

    def __init__(self, comm):
        import torch.distributed as dist
        self.dist = dist
        self.rank, self.world = comm.rank, comm.world_size
        self.cuda = torch.cuda.is_available() and not getattr(comm, "is_cpu", False)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "12355")   # the reference's port (1_sendrecv_direct.py:97)
            dist.init_process_group("nccl" if self.cuda else "gloo", rank=self.rank, world_size=self.world)
            self.group = dist.group.WORLD
        elif self.cuda and "nccl" not in str(dist.get_backend()):
            self.group = dist.new_group(backend="nccl")
        else:
            self.group = dist.group.WORLD

    def broadcast(self, t: torch.Tensor, root: int) -> torch.Tensor:
        o = t.clone()
        self.dist.broadcast(o, src=root, group=self.group)
        return o

    def reduce(self, t: torch.Tensor, root: int) -> torch.Tensor:
        o = t.clone()
        self.dist.reduce(o, dst=root, group=self.group)
        return o

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        o = t.clone()
        self.dist.all_reduce(o, group=self.group)
        return o

    def all_gather(self, shard: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world,) + tuple(shard.shape), dtype=shard.dtype, device=shard.device)
        self.dist.all_gather_into_tensor(out.view(-1), shard.contiguous().view(-1), group=self.group)
        return out

    def reduce_scatter(self, full: torch.Tensor) -> torch.Tensor:
        out = torch.empty(full.shape[1:], dtype=full.dtype, device=full.device)
        if self.cuda:
            self.dist.reduce_scatter_tensor(out.view(-1), full.contiguous().view(-1), group=self.group)
        else:  # gloo has no reduce-scatter: all-reduce and keep the own row
            tmp = full.clone()
            self.dist.all_reduce(tmp, group=self.group)
            out.copy_(tmp[self.rank])
        return out

    def all_to_all(self, full: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(full)
        if self.cuda:
            self.dist.all_to_all_single(out.view(-1), full.contiguous().view(-1), group=self.group)
        else:
            gathered = [torch.empty_like(full) for _ in range(self.world)]
            self.dist.all_gather(gathered, full.contiguous(), group=self.group)
            for p in range(self.world):
                out[p].copy_(gathered[p][self.rank])
        return out

    def sendrecv(self, t: torch.Tensor, src: int, dst: int) -> Optional[torch.Tensor]:
        if self.rank == src:
            self.dist.send(t.contiguous(), dst=dst, group=self.group)
            return None
        if self.rank == dst:
            o = torch.empty_like(t)
            self.dist.recv(o, src=src, group=self.group)
            return o
        return None


_oracle = None


def oracle(comm) -> TorchOracle:
    global _oracle
    if _oracle is None:
        _oracle = TorchOracle(comm)
    return _oracle


def compare(rank: int, what: str, got: torch.Tensor, want: torch.Tensor, exact: bool, roundings: int = 2) -> bool:
    """Print the reference's self-test line and return the outcome.  ``roundings``: how many roundings into the
    element type the two results may be apart (a library that adds in the element type rounds at every add)."""
    g, w = got.detach().float().cpu().reshape(-1), want.detach().float().cpu().reshape(-1)
    if exact:
        ok = bool(torch.equal(got.detach().cpu(), want.detach().cpu()))
        word = "equal"
    else:
        eps = torch.finfo(got.dtype).eps * max(1, roundings)
        ok = bool(((g - w).abs() <= eps * torch.maximum(g.abs(), w.abs()) + eps * float(w.abs().max()) * 1e-2).all())
        word = "close"
    print(f"# rank {rank}, {what} vs torch.distributed: {word}: {ok}", flush=True)
    if verbose() or not ok:
        print(f"# rank {rank}, mintccl_b200 head: {g[:16].tolist()}", flush=True)
        print(f"# rank {rank}, torch.dist   head: {w[:16].tolist()}", flush=True)
        print(f"# rank {rank}, mintccl_b200 tail: {g[-16:].tolist()}", flush=True)
        print(f"# rank {rank}, torch.dist   tail: {w[-16:].tolist()}", flush=True)
        if not ok:
            bad = ((g - w).abs() > 0).nonzero()
            if bad.numel():
                i = int(bad[0])
                print(f"# rank {rank}, first difference at {i}: {float(g[i])} against {float(w[i])}", flush=True)
    return ok
