"""Algorithm / protocol / CTA-count policy of the communicator, checked without a GPU (the methods only look at
sizes, alignment and configuration)."""
import pytest
import torch

from mintccl_b200 import Config
from mintccl_b200 import _native as N
from mintccl_b200.parallel.comm import Communicator


def policy(world=8, nvls=True, emulated=False, nlocal=1, **cfg):
    c = object.__new__(Communicator)          # no device, no heap: policy only
    c.cfg = Config.from_env(**cfg)
    c.world_size, c.nvls, c.emulated, c.nlocal = world, nvls, emulated, nlocal
    return c


def test_protocol_by_size():
    c = policy()
    assert c._pick_proto(8, None) == N.PROTO_LL128
    assert c._pick_proto(c.cfg.ll128_max_bytes, None) == N.PROTO_LL128
    assert c._pick_proto(c.cfg.ll128_max_bytes + 1, None) == N.PROTO_SIMPLE
    assert c._pick_proto(8, "simple") == N.PROTO_SIMPLE and c._pick_proto(1 << 30, "ll128") == N.PROTO_LL128
    assert policy(world=1)._pick_proto(8, "ll128") == N.PROTO_SIMPLE     # one rank only copies


def test_nvls_needs_four_ranks_size_and_alignment():
    t = [torch.empty(1 << 16)]
    assert policy(world=8)._want_nvls(1 << 20, t)
    assert policy(world=4)._want_nvls(1 << 20, t)
    assert not policy(world=2)._want_nvls(1 << 20, t)                    # the switch only adds a hop
    assert not policy(world=8, nvls=False)._want_nvls(1 << 20, t)
    assert not policy(world=8)._want_nvls(1 << 10, t)                    # below MINTCCL_NVLS_MIN_BYTES
    assert not policy(world=8)._want_nvls((1 << 20) + 8, t)              # multimem moves 16 bytes
    assert not policy(world=8)._want_nvls(1 << 20, [torch.empty(1 << 16)[1:]])   # 4-byte offset


def test_cta_counts_grow_with_the_message_and_respect_caps():
    c = policy()
    small, mid, big = (c._direct_ctas(x, None) for x in (4 << 10, 2 << 20, 1 << 30))
    assert 1 <= small <= mid <= big <= 128 and small == 1 and mid == 32
    assert c._direct_ctas(1 << 30, 200) == 148 and c._direct_ctas(1 << 30, 3) == 3
    e = policy(emulated=True, nlocal=4)
    assert e._direct_ctas(1 << 30, None) <= 148 // 4 and e._ring_channels(1 << 30, N.PROTO_SIMPLE, None) <= 148 // 4
    assert c._ring_channels(8, N.PROTO_LL128, None) == 1
    assert c._ring_channels(1 << 30, N.PROTO_SIMPLE, None) == c.cfg.max_channels
    assert policy(num_blocks=16)._ring_channels(1 << 30, N.PROTO_SIMPLE, None) == 16      # MINTCCL_NUM_BLOCKS caps it
    assert policy(world=1)._ring_channels(1 << 30, N.PROTO_SIMPLE, None) == 296           # local copies: no FIFO limit


def test_algorithm_names_per_collective():
    c = policy()
    assert c._algo(None, "allreduce") == "auto"
    assert c._algo("oneshot", "allreduce") == "oneshot"
    with pytest.raises(ValueError):
        c._algo("pull", "reducescatter")
    with pytest.raises(ValueError):
        c._algo("oneshot", "allgather")
    c.cfg.algo = "ll"                      # MINTCCL_ALGO=ll: all-reduce has it, the others fall back to automatic
    assert c._algo(None, "allreduce") == "ll" and c._algo(None, "broadcast") == "auto"
