"""Communicator: symmetric heap, peer mappings, algorithm choice and kernel launches.

One ``Communicator`` per process and GPU.  Creating it is the only expensive step: it allocates the
symmetric heap, exchanges the heap handles through the control plane (POSIX fds of a cuMem allocation
over unix sockets, or cudaIpc handles), maps every peer, optionally binds the NVLS multicast object and
uploads the device descriptor.  After that every collective is exactly one kernel launch on the current
CUDA stream, with no host communication and no allocation.

The reference has no such object (every call of e.g. ``allgather`` re-allocates its staging buffer and
re-exchanges IPC handles over MPI, 6_allgather.py:141-158); its module-level functions are provided by
``mintccl_b200.ops.collectives`` on top of a default communicator.

``Communicator.emulated(n)`` creates a world of ``n`` ranks on ONE GPU in one process: the same kernels
run with ``gridDim.y = n`` (cooperative launch), which is how the single-GPU tests exercise every
multi-rank protocol path.  In that mode every tensor argument is a list with one tensor per rank.
"""
from __future__ import annotations

import bisect
import ctypes as C
import os
import uuid
from typing import List, Optional, Sequence, Union

import torch

from .. import _native as N
from ..config import Config, env_bool
from ..topology import find_ring, find_route, get_topology, uniform_topology
from ..tuning import TuningTable
from .rendezvous import ControlPlane, SingleControl, connect, local_rank_default

TensorOrList = Union[torch.Tensor, Sequence[torch.Tensor]]

_DT = {torch.float32: N.DT_F32, torch.float16: N.DT_F16, torch.bfloat16: N.DT_BF16}
_HEAP_TAG = 1 << 63   # MT_PUB_HEAP_TAG: "offset inside the announcing rank's symmetric heap"


class _Segment:
    """One device allocation of this process that every peer has mapped (CUDA IPC), with its base address in each
    peer's address space.  ``keep`` holds a storage inside the allocation, so the caching allocator cannot hand
    the allocation back to the driver while peers still map it."""
    __slots__ = ("base", "size", "handle", "peer_base", "keep")

    def __init__(self, base, size, handle, peer_base, keep):
        self.base, self.size, self.handle, self.peer_base, self.keep = base, size, handle, peer_base, keep


class CollectiveError(RuntimeError):
    """A device-side wait gave up (timeout or abort).  The communicator must be re-created."""

    def __init__(self, status):
        self.code, self.rank, self.channel, self.where = status.code, status.rank, status.channel, status.where
        self.expected, self.seen, self.step = status.expected, status.seen, status.step
        super().__init__(f"{N.ERR_NAMES.get(status.code, status.code)} on rank {status.rank} channel "
                         f"{status.channel} (where={status.where}, expected={status.expected}, seen={status.seen}, "
                         f"step={status.step})")


CollectiveTimeout = CollectiveError


class _RawCuda:
    """Wraps a raw device pointer so that torch can build a tensor over it (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _dtype_code(t: torch.Tensor, reduce: bool) -> int:
    if t.dtype in _DT:
        return _DT[t.dtype]
    if reduce:
        raise TypeError(f"reductions support float32/float16/bfloat16, got {t.dtype}")
    return N.DT_U8


class Communicator:
    def __init__(self, control: Optional[ControlPlane] = None, device: Optional[int] = None,
                 config: Optional[Config] = None, group=None, _emulate: int = 0):
        self.cfg = config or Config.from_env()
        self.lib = N.lib()
        self._handle = None
        self._pending: list = []
        self._allocs: dict[int, int] = {}
        self._free: list[tuple[int, int]] = []
        self._registered: dict = {}
        self._segs: dict[int, _Segment] = {}     # allocation base -> shared allocation
        self._seg_bases: list[int] = []          # sorted keys of _segs
        self._unsharable: set[int] = set()       # allocation bases CUDA IPC refused
        self._reg_secret = ""
        self._reg_token = None
        self._plans: dict = {}
        self._rec_key = None
        self._tuning = TuningTable.from_env()   # MINTCCL_TUNING_FILE: measured choices, or None
        self.emulated = _emulate > 0
        if self.emulated:
            self.control = SingleControl()
            self.rank, self.world_size, self.nlocal = 0, _emulate, _emulate
            self.device = 0 if device is None else device
        else:
            self.control = control or connect(group)
            self.rank, self.world_size, self.nlocal = self.control.rank, self.control.world_size, 1
            self.device = local_rank_default(self.rank) if device is None else device
        if not torch.cuda.is_available():
            raise RuntimeError("mintccl_b200.Communicator needs a CUDA device; use the CPU backend "
                               "(mintccl_b200.parallel.cpu_backend) on machines without one")
        if self.world_size > N.MT_MAX_RANKS:
            raise ValueError(f"at most {N.MT_MAX_RANKS} ranks per node")
        torch.cuda.set_device(self.device)
        torch.cuda.init()
        torch.zeros(1, device=f"cuda:{self.device}")  # make sure the primary context exists
        self._create()

    # ------------------------------------------------------------------------------------------ set-up
    @classmethod
    def emulated(cls, nranks: int, device: int = 0, config: Optional[Config] = None) -> "Communicator":
        return cls(device=device, config=config, _emulate=nranks)

    def _mtconfig(self, heap_kind: int) -> N.MtConfig:
        c = self.cfg
        return N.MtConfig(nchannels=c.max_channels, simple_slot_bytes=c.simple_slot_bytes, simple_slots=c.simple_slots,
                          ll128_slot_bytes=c.ll128_slot_bytes, ll128_slots=c.ll128_slots, ll_bytes=c.ll_bytes,
                          scratch_bytes=c.scratch_bytes, heap_bytes=c.heap_bytes, timeout_ms=c.wait_timeout_ms,
                          heap_kind=heap_kind)

    def _create(self) -> None:
        L, n = self.lib, self.world_size
        self.nvls = False
        if self.emulated:
            mc = self._mtconfig(1)
            self._handle = L.mt_comm_create_emulated(n, self.device, C.byref(mc))
            if not self._handle:
                raise RuntimeError(f"mt_comm_create_emulated: {N.last_error()}")
            self.heap_kind = "emulated"
        else:
            kinds = {"vmm": [0], "ipc": [1], "auto": [0, 1]}[self.cfg.heap_kind]
            last = ""
            for kind in kinds:
                ok, err = self._try_create(kind)
                oks = self.control.allgather(ok)
                if all(oks):
                    break
                last = err or "a peer failed"
                if self._handle:
                    L.mt_comm_destroy(self._handle)
                    self._handle = None
            else:
                raise RuntimeError(f"could not create and exchange the symmetric heap: {last}")
            if self.heap_kind == "vmm" and n > 1 and self.cfg.nvls != "off":
                self._try_nvls()
                if self.cfg.nvls == "on" and not self.nvls:
                    raise RuntimeError("MINTCCL_NVLS=on but the multicast object could not be set up")
            if n > 1:
                self._start_registration_service()
        ring = self._choose_ring()
        arr = (C.c_int * N.MT_MAX_RANKS)(*ring)
        N.check(L.mt_comm_finalize(self._handle, arr), "mt_comm_finalize")
        self.ring = ring
        lay = N.MtHeapLayout()
        L.mt_comm_layout(self._handle, C.byref(lay))
        self.layout = lay
        self.heap_bytes = lay.heap_bytes
        self.user_off = lay.user_off
        self._free = [(lay.user_off, lay.heap_bytes - lay.user_off)]
        self.heap_base = [L.mt_comm_heap_ptr(self._handle, lr, lr if self.emulated else self.rank)
                          for lr in range(self.nlocal)]
        self.ll_capacity = L.mt_ll_capacity(self._handle)
        self.control.barrier()

    def _try_create(self, kind: int):
        L, n = self.lib, self.world_size
        mc = self._mtconfig(kind)
        self._handle = L.mt_comm_create(self.rank, n, self.device, C.byref(mc))
        if not self._handle:
            return False, N.last_error()
        self.heap_kind = "vmm" if kind == 0 else "ipc"
        if n == 1:
            return True, ""
        try:
            if kind == 1:
                buf = C.create_string_buffer(64)
                N.check(L.mt_comm_export_ipc(self._handle, buf), "export_ipc")
                handles = self.control.allgather(buf.raw)
                for p, h in enumerate(handles):
                    if p != self.rank:
                        N.check(L.mt_comm_import_ipc(self._handle, p, h), f"import_ipc({p})")
            else:
                # the socket name is public (/proc/net/unix); the key travels over the control plane only and comes
                # back in the tag of every descriptor, next to the sender's rank
                token, key = self.control.bcast((uuid.uuid4().hex[:12], uuid.uuid4().int & 0x3fffff), 0)
                self._sock_token, self._sock_key = token, key
                sock = L.mt_fd_listen(f"mintccl-{token}-{self.rank}".encode())
                if sock < 0:
                    raise RuntimeError("cannot listen on the fd-passing socket")
                self._sock = sock
                self.control.barrier()
                fd = N.check(L.mt_comm_export_fd(self._handle), "export_fd")
                try:
                    for p in range(n):
                        if p != self.rank:
                            N.check(L.mt_fd_send(f"mintccl-{token}-{p}".encode(), (key << 8) | self.rank, fd, 20000),
                                    f"fd_send({p})")
                    seen = set()
                    while len(seen) < n - 1:
                        tag = C.c_int(-1)
                        rfd = L.mt_fd_accept(sock, C.byref(tag), 20000)
                        if rfd < 0:
                            raise RuntimeError("did not receive a peer's heap descriptor")
                        try:
                            src = tag.value & 0xff
                            if tag.value >> 8 != key or src >= n or src == self.rank or src in seen:
                                continue   # not one of this communicator's peers, or a repeat: ignore it
                            N.check(L.mt_comm_import_fd(self._handle, src, rfd), f"import_fd({src})")
                            seen.add(src)
                        finally:
                            L.mt_fd_close(rfd)
                finally:
                    L.mt_fd_close(fd)
            return True, ""
        except RuntimeError as e:  # reported to all ranks by the caller's allgather
            return False, str(e)

    def _start_registration_service(self) -> None:
        """One thread per communicator that maps a peer's ordinary allocation into this process when the peer asks
        (``csrc/host/regsrv.cpp``).  Socket name and secret come from rank 0 over the control plane."""
        token, secret = self.control.bcast((uuid.uuid4().hex[:12], uuid.uuid4().hex[:30]), 0)
        self._reg_token, self._reg_secret = token, secret
        ok = self.lib.mt_reg_start(self._handle, self._reg_sock(self.rank), secret.encode()) == 0
        if not all(self.control.allgather(ok)):
            raise RuntimeError(f"could not start the registration service: {N.last_error()}")

    def _reg_sock(self, rank: int) -> bytes:
        return f"mintccl-{self._reg_token}-reg-{rank}".encode()

    def _try_nvls(self) -> None:
        L, n = self.lib, self.world_size
        sup = self.control.allgather(bool(L.mt_comm_mc_supported(self._handle)))
        if not all(sup):
            return
        ok = True
        try:
            if self.rank == 0:
                fd = N.check(L.mt_comm_mc_create(self._handle), "mc_create")
                for p in range(1, n):
                    N.check(L.mt_fd_send(f"mintccl-{self._sock_token}-{p}".encode(), (self._sock_key << 8) | 0xff, fd, 20000),
                            "mc fd_send")
                L.mt_fd_close(fd)
            else:
                tag = C.c_int(-1)
                rfd = L.mt_fd_accept(self._sock, C.byref(tag), 20000)
                if rfd < 0 or tag.value != ((self._sock_key << 8) | 0xff):
                    raise RuntimeError("did not receive the multicast descriptor")
                N.check(L.mt_comm_mc_import(self._handle, rfd), "mc_import")
                L.mt_fd_close(rfd)
        except RuntimeError:
            ok = False
        if not all(self.control.allgather(ok)):
            return
        ok = L.mt_comm_mc_add_device(self._handle) == 0
        if not all(self.control.allgather(ok)):
            return
        ok = L.mt_comm_mc_bind(self._handle) == 0
        if not all(self.control.allgather(ok)):
            raise RuntimeError(f"multicast bind failed on some rank ({N.last_error()}); cannot continue safely")
        self.nvls = True

    def _topology(self):
        """Link map behind the ring and the routes.  An NVSwitch node (every HGX B200 board) is uniform: every
        pair at full bandwidth; that is the default and needs no probing.  ``MINTCCL_TOPO_FILE`` names a cached
        topology (the ``topo.json`` of :func:`mintccl_b200.topology.get_topology`, as in the reference,
        topology.py:128-149), discovered and written by rank 0 if the file does not exist yet;
        ``MINTCCL_TOPO_DISCOVER=1`` discovers without a file (peer-access matrix from the driver, bandwidths
        measured with ``MINTCCL_TOPO_MEASURE=1``).  Rank 0 decides and shares the result, so every rank derives
        the same ring and routes."""
        topo = getattr(self, "_topo", None)
        if topo is not None:
            return topo
        path = os.environ.get("MINTCCL_TOPO_FILE", "")
        if path or env_bool("MINTCCL_TOPO_DISCOVER", False):
            topo = get_topology(path, ndev=self.world_size) if self.rank == 0 else None
            topo = self.control.bcast(topo, root=0)
        else:
            topo = uniform_topology(self.world_size)
        self._topo = topo
        return topo

    def _choose_ring(self) -> List[int]:
        n = self.world_size
        env = os.environ.get("MINTCCL_RING")
        if env:
            ring = [int(x) for x in env.split(",")]
            if sorted(ring) != list(range(n)):
                raise ValueError("MINTCCL_RING must be a permutation of the ranks")
            return ring
        seed = os.environ.get("MINTCCL_RING_SEED")
        if seed is not None:
            g = torch.Generator().manual_seed(int(seed))
            return torch.randperm(n, generator=g).tolist()
        ring = find_ring(self._topology())
        return ring[:n] if ring else list(range(n))

    def set_ring(self, ring: Sequence[int]) -> None:
        arr = (C.c_int * N.MT_MAX_RANKS)(*ring)
        N.check(self.lib.mt_comm_set_ring(self._handle, arr), "set_ring")
        self.ring = list(ring)

    def set_timeout_ms(self, ms: int) -> None:
        N.check(self.lib.mt_comm_set_timeout_ms(self._handle, ms), "set_timeout")

    def close(self) -> None:
        if self._handle:
            torch.cuda.synchronize(self.device)
            self.control.barrier()             # nobody still runs a kernel that touches a peer's memory
            self.lib.mt_reg_stop(self._handle)  # unmap what this rank opened for its peers
            self.control.barrier()
            self._segs.clear()
            self._seg_bases.clear()
            self._plans.clear()
            self.lib.mt_comm_destroy(self._handle)
            self._handle = None
            if getattr(self, "_sock", None) is not None:
                self.lib.mt_fd_close(self._sock)
                self._sock = None

    def __del__(self):
        try:
            if self._handle:
                self.lib.mt_comm_destroy(self._handle)
                self._handle = None
        except Exception:
            pass

    # ------------------------------------------------------------------------------------- status
    def status(self, local_rank: int = 0) -> N.MtStatus:
        st = N.MtStatus()
        N.check(self.lib.mt_comm_status(self._handle, local_rank, C.byref(st)), "status")
        return st

    def check(self) -> None:
        """Raise :class:`CollectiveError` if any device-side wait gave up.  Reading the status record waits for all
        work queued on the device (``mt_comm_status`` synchronises it), so after ``check()`` returns every
        collective launched so far has completed."""
        for lr in range(self.nlocal):
            st = self.status(lr)
            if st.code != 0 or st.abort != 0:
                raise CollectiveError(st)

    # ------------------------------------------------------------------------------ symmetric memory
    def _alloc_off(self, nbytes: int, align: int = 256) -> int:
        nbytes = max(align, (nbytes + align - 1) // align * align)
        for i, (off, size) in enumerate(self._free):
            if size >= nbytes:
                if size == nbytes:
                    self._free.pop(i)
                else:
                    self._free[i] = (off + nbytes, size - nbytes)
                self._allocs[off] = nbytes
                return off
        raise MemoryError(f"symmetric heap exhausted ({nbytes} bytes requested); raise MINTCCL_HEAP_BYTES")

    def symm_free(self, t: TensorOrList) -> None:
        t0 = t[0] if isinstance(t, (list, tuple)) else t
        off = t0.data_ptr() - self.heap_base[0]
        size = self._allocs.pop(off)
        self._free.append((off, size))
        self._free.sort()
        merged: list[tuple[int, int]] = []
        for o, s in self._free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self._free = merged

    def symm_empty(self, shape, dtype=torch.float32) -> TensorOrList:
        """Allocate a tensor in the symmetric heap.  Collective in spirit: every rank must allocate the
        same sizes in the same order so that the tensor has the same heap offset everywhere."""
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        off = self._alloc_off(nbytes)
        outs = []
        for lr in range(self.nlocal):
            raw = torch.as_tensor(_RawCuda(self.heap_base[lr] + off, max(nbytes, 1)), device=f"cuda:{self.device}")
            outs.append(raw[:nbytes].view(dtype).view(shape))
        return outs if self.emulated else outs[0]

    def symm_zeros(self, shape, dtype=torch.float32) -> TensorOrList:
        t = self.symm_empty(shape, dtype)
        for x in (t if self.emulated else [t]):
            x.zero_()
        return t

    def symm_offset(self, t: torch.Tensor, lr: int = 0) -> Optional[int]:
        """Heap offset of ``t`` if it lies inside the symmetric heap of local rank ``lr``, else None."""
        off = t.data_ptr() - self.heap_base[lr]
        nbytes = t.numel() * t.element_size()
        if off >= self.user_off and off + nbytes <= self.heap_bytes:
            return off
        return None

    # ------------------------------------------------------------------------------ helpers
    def _lists(self, t: Optional[TensorOrList]) -> Optional[List[torch.Tensor]]:
        if t is None:
            return None
        if isinstance(t, torch.Tensor):
            if self.emulated:
                raise TypeError("emulated communicator: pass one tensor per rank")
            ts = [t]
        else:
            ts = list(t)
            if len(ts) != self.nlocal:
                raise ValueError(f"expected {self.nlocal} tensors")
        for x in ts:
            if not x.is_cuda or not x.is_contiguous():
                raise ValueError("tensors must be contiguous CUDA tensors")
        return ts

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _symm_off_all(self, ts: List[torch.Tensor]) -> Optional[int]:
        offs = [self.symm_offset(t, lr) for lr, t in enumerate(ts)]
        if offs[0] is None or any(o != offs[0] for o in offs):
            return None
        return offs[0]

    def _ring_channels(self, nbytes: int, proto: int, nch: Optional[int]) -> int:
        cap = self.cfg.num_blocks or self.cfg.max_channels
        if self.world_size == 1:
            cap = 296  # local copies only: no FIFO limits the channel count, fill the 148 SMs twice
        if self.emulated:
            cap = min(cap, 148 // self.nlocal)
        if nch is not None:
            return max(1, min(nch, cap))
        per = 64 << 10 if proto == N.PROTO_LL128 else 256 << 10
        return max(1, min(cap, (nbytes + per - 1) // per))

    def _direct_ctas(self, nbytes: int, nctas: Optional[int]) -> int:
        cap = self.cfg.direct_ctas or 128
        if self.emulated:
            cap = min(cap, 148 // self.nlocal)
        if nctas is not None:
            return max(1, min(nctas, 148 // self.nlocal if self.emulated else 148))
        # one CTA per 64 KiB up to 32, then one more per 256 KiB: small messages stay on few SMs (the
        # cross-rank barrier is per CTA), large ones need most SMs to keep enough bytes in flight
        n = (nbytes + (64 << 10) - 1) // (64 << 10)
        if n > 32:
            n = 32 + (nbytes - (2 << 20)) // (256 << 10)
        return max(1, min(cap, n))

    def _bulk_ctas(self, nbytes: int) -> int:
        """CTAs of a copy-engine variant: one thread per CTA issues the copies, so the bytes in flight grow with
        the CTA count; one CTA per 64 KiB up to MINTCCL_BULK_CTAS (128: measured best from 16 MiB on)."""
        cap = self.cfg.bulk_ctas
        if self.emulated:
            cap = min(cap, 148 // self.nlocal)
        return max(1, min(cap, (nbytes + (64 << 10) - 1) // (64 << 10)))

    def _pick_proto(self, nbytes: int, proto: Optional[str]) -> int:
        p = proto or self.cfg.proto
        if self.world_size == 1:
            return N.PROTO_SIMPLE  # a single rank only copies locally: no flags to carry
        if p == "simple":
            return N.PROTO_SIMPLE
        if p == "ll128":
            return N.PROTO_LL128
        return N.PROTO_LL128 if nbytes <= self.cfg.ll128_max_bytes else N.PROTO_SIMPLE

    def _launch_ring(self, op, ins, outs, nbytes, dtype, proto, root=0, spatial=False, chain=None, nch=None):
        nch = self._ring_channels(nbytes, proto, nch)
        if spatial:
            n = self.world_size
            nch = max(n, nch // n * n)
            if nch > self.cfg.max_channels or (self.emulated and nch * n > 148):
                spatial = False
                nch = self._ring_channels(nbytes, proto, None)
        inp = N.ptr_array([t.data_ptr() if t is not None else 0 for t in ins]) if ins else None
        outp = N.ptr_array([t.data_ptr() if t is not None else 0 for t in outs]) if outs else None
        ch_arr = (C.c_int * (N.MT_MAX_RANKS + 1))(*(chain or []))
        self._run(self.lib.mt_ring, (proto, dtype, op, inp, outp, nbytes, root, 1 if spatial else 0, ch_arr,
                                     len(chain or []), nch))

    # ---------------------------------------------------------------- ordinary tensors as peer memory
    def share(self, t: torch.Tensor) -> List[int]:
        """Make an ordinary CUDA tensor addressable by every peer and return, for every rank, the address of THIS
        rank's tensor in that rank's address space.  One-sided: only the caller takes part (the peers' registration
        services answer), so ranks may call it at different times.  The allocation that contains the tensor is
        exported once through CUDA IPC (base + offset: the reference sends the handle of the block and drops the
        offset, common.py:24-26) and stays mapped, and alive, until :meth:`unshare_all` or :meth:`close`."""
        ptr = t.data_ptr()
        if self.emulated or self.world_size == 1:
            return [ptr] * max(1, self.world_size)
        seg = self._segment_of(ptr, t.numel() * t.element_size())
        if seg is None:
            seg = self._share_allocation(t)
        return [ptr if p == self.rank else seg.peer_base[p] + (ptr - seg.base) for p in range(self.world_size)]

    def _segment_of(self, ptr: int, nbytes: int) -> Optional[_Segment]:
        i = bisect.bisect_right(self._seg_bases, ptr) - 1
        if i < 0:
            return None
        seg = self._segs[self._seg_bases[i]]
        return seg if ptr + nbytes <= seg.base + seg.size else None

    def _share_allocation(self, t: torch.Tensor) -> _Segment:
        buf = C.create_string_buffer(64)
        off, size = C.c_uint64(0), C.c_uint64(0)
        ptr = t.data_ptr()
        if self.lib.mt_ipc_export(ptr, buf, C.byref(off), C.byref(size)) < 0:
            raise RuntimeError(f"this allocation cannot be exported through CUDA IPC: {N.last_error()}")
        base = ptr - off.value
        peer_base = [0] * self.world_size
        done = []
        try:
            for p in range(self.world_size):
                if p == self.rank:
                    peer_base[p] = base
                    continue
                va = C.c_uint64(0)
                N.check(self.lib.mt_reg_share(self._reg_sock(p), self._reg_secret.encode(), self.rank, buf.raw,
                                              size.value, C.byref(va), 20000), f"share with rank {p}")
                peer_base[p] = va.value
                done.append(p)
        except RuntimeError:
            for p in done:
                self.lib.mt_reg_unshare(self._reg_sock(p), self._reg_secret.encode(), self.rank, buf.raw, 5000)
            raise
        seg = _Segment(base, size.value, buf.raw, peer_base, t.untyped_storage())
        self._segs[base] = seg
        bisect.insort(self._seg_bases, base)
        return seg

    def unshare_all(self) -> None:
        """Ask every peer to unmap the allocations shared so far and let go of them.  Collective in effect: call it
        on every rank, with no collective in flight, e.g. before ``torch.cuda.empty_cache()``."""
        torch.cuda.synchronize(self.device)
        self.control.barrier()
        for seg in self._segs.values():
            for p in range(self.world_size):
                if p != self.rank:
                    self.lib.mt_reg_unshare(self._reg_sock(p), self._reg_secret.encode(), self.rank, seg.handle, 5000)
        self._segs.clear()
        self._seg_bases.clear()
        self._unsharable.clear()
        self._plans.clear()
        self.control.barrier()

    def _peer_ok(self, ts: List[torch.Tensor]) -> bool:
        """Can the peers address these tensors?  Heap tensors and (emulation) everything in the one address space:
        yes.  Ordinary tensors: when automatic registration is on and CUDA IPC takes the allocation."""
        if self.emulated or self.world_size == 1:
            return True
        t = ts[0]
        if self.symm_offset(t) is not None:
            return True
        if self._segment_of(t.data_ptr(), t.numel() * t.element_size()) is not None:
            return True
        if not self.cfg.auto_register:
            return False
        sbase = t.untyped_storage().data_ptr()
        if sbase in self._unsharable:
            return False
        try:
            self._share_allocation(t)
            return True
        except RuntimeError:
            self._unsharable.add(sbase)   # e.g. an allocator CUDA IPC cannot export: this memory takes the ring
            return False

    def _peer_views(self, ts: List[torch.Tensor], extra: int = 0) -> List[int]:
        """What this rank announces to each peer as the place of ``ts[0]`` (+ ``extra`` bytes)."""
        t = ts[0]
        off = self.symm_offset(t)
        if off is not None:
            return [_HEAP_TAG | (off + extra)] * self.world_size
        if self._segment_of(t.data_ptr(), t.numel() * t.element_size()) is None and not self.cfg.auto_register:
            raise ValueError("this algorithm needs memory the peers can address: a tensor from "
                             "Communicator.symm_empty, or an ordinary tensor passed to Communicator.share() first")
        return [v + extra for v in self.share(t)]

    def _launch_direct(self, dop, ins, outs, nbytes, dtype, root=0, variant=0, nvls=False, nctas=None,
                       peers_read_in=False, peers_write_out=False, out_dtype=None, in_extra=0, in_from_out=False):
        """One launch of the one-hop kernel.  ``peers_read_in`` / ``peers_write_out``: whether the peers touch this
        rank's input / output, i.e. whether it must be announced to them (and, for an ordinary tensor, shared).
        ``in_from_out``: the contribution is a slice of the output buffer, ``in_extra`` bytes into it."""
        nctas = self._direct_ctas(nbytes, nctas if nctas is not None or not nvls else min(self.cfg.nvls_ctas, self._direct_ctas(nbytes, None)))
        mc_in = mc_out = 0
        if nvls:
            mc_in, mc_out = self._symm_off_all(ins), self._symm_off_all(outs)
            if (nbytes % 16 or (mc_in or 0) % 16 or (mc_out or 0) % 16
                    or any(t is not None and t.data_ptr() % 16 for t in list(ins) + list(outs))):
                raise ValueError("NVLS algorithms need 16-byte aligned buffers and a byte count that is a multiple of 16")
        n = self.world_size
        if self.emulated or n == 1:
            pin = pout = None
        else:
            pout = self._peer_views(outs) if peers_write_out else [0] * n
            if not peers_read_in:
                pin = [0] * n
            elif in_from_out:
                pin = self._peer_views(outs, in_extra)
            else:
                pin = self._peer_views(ins)
            pin, pout = N.u64_array(pin), N.u64_array(pout)
        inp = N.ptr_array([t.data_ptr() if t is not None else 0 for t in ins])
        outp = N.ptr_array([t.data_ptr() if t is not None else 0 for t in outs])
        self._run(self.lib.mt_direct, (dtype, dtype if out_dtype is None else out_dtype, dop, inp, outp, pin, pout,
                                       mc_in or 0, mc_out or 0, nbytes, root, variant, 1 if nvls else 0, nctas))

    _ALGOS = {
        "allreduce": ("auto", "ring", "direct", "nvls", "ll", "oneshot"),
        "allgather": ("auto", "ring", "direct", "nvls", "pull", "bulk", "bulkpull"),
        "reducescatter": ("auto", "ring", "direct", "nvls"),
        "broadcast": ("auto", "ring", "direct", "nvls", "pull", "push", "nvls1", "bulk"),
        "reduce": ("auto", "ring", "direct", "direct2", "nvls", "direct1", "nvls1"),
    }

    def _algo(self, algo: Optional[str], collective: str) -> str:
        """The algorithm of one call: ``algo=`` must be one this collective has; the process-wide default
        (``MINTCCL_ALGO``) applies where the collective has it and means ``auto`` elsewhere."""
        known = self._ALGOS[collective]
        if algo is not None:
            if algo not in known:
                raise ValueError(f"{collective}: unknown algo {algo!r} (one of {', '.join(known)})")
            return algo
        return self.cfg.algo if self.cfg.algo in known else "auto"

    def _tuned(self, collective: str, nbytes: int, algo: Optional[str], nch: Optional[int], symmetric: bool,
               tensors=(), unit: Optional[int] = None):
        """Where the caller left ``algo`` and ``nch`` open and a tuning table (``MINTCCL_TUNING_FILE``) has a row for
        this collective, rank count, size and kind of memory, that row decides; otherwise nothing changes.  A row
        that asks for NVLS is skipped for buffers NVLS cannot take (``unit``, the bytes one multimem stream moves,
        and every pointer must be multiples of 16)."""
        table = getattr(self, "_tuning", None)
        if table is None or algo is not None or nch is not None:
            return algo, nch
        hit = table.lookup(collective, self.world_size, nbytes, symmetric)
        if hit is None:
            return algo, nch
        if hit[0].startswith("nvls") and (not self.nvls or (unit if unit is not None else nbytes) % 16
                                          or any(t.data_ptr() % 16 for t in tensors)):
            return algo, nch
        if hit[0] not in ("auto", "ring", "ll") and not symmetric and not all(self._peer_ok([t]) for t in tensors):
            return algo, nch     # a one-hop row, but the peers cannot address this memory
        return hit

    def _want_nvls(self, nbytes: int, tensors) -> bool:
        """In-switch reduction / replication pays off from four ranks on (with two ranks the switch only
        adds a hop: measured 394 against 606 GB/s for a 256 MiB all-reduce) and needs 16-byte alignment."""
        return (self.nvls and self.world_size >= 4 and nbytes >= self.cfg.nvls_min_bytes and nbytes % 16 == 0
                and all(t.data_ptr() % 16 == 0 for t in tensors))

    # Launch plans: the first call of a collective on given buffers validates the arguments, picks the
    # algorithm and records the native call; later calls with the same buffers replay it directly, which
    # keeps the host cost of a collective at a few microseconds.  The key holds everything the choice depends
    # on: both buffers (address, size, type), the per-call arguments, and the process-wide settings that may
    # change between calls (``cfg.algo``, ``cfg.proto``, the route mode).
    def _run(self, fn, args) -> None:
        if fn(self._handle, torch.cuda.current_stream(self.device).cuda_stream, *args) < 0:
            raise RuntimeError(f"{fn.__name__}: {N.last_error()}")
        if self._rec_key is not None:
            if len(self._plans) > 8192:
                self._plans.clear()
            self._plans[self._rec_key] = (fn, args)
            self._rec_key = None

    def _replay(self, key) -> bool:
        p = self._plans.get(key)
        if p is None:
            self._rec_key = key
            return False
        if p[0](self._handle, torch.cuda.current_stream(self.device).cuda_stream, *p[1]) < 0:
            raise RuntimeError(f"{p[0].__name__}: {N.last_error()}")
        return True

    def _key(self, tag, a, b, *rest):
        return (tag, a.data_ptr(), a.numel(), a.dtype, *((0, 0, None) if b is None else (b.data_ptr(), b.numel(), b.dtype)),
                self.cfg.algo, self.cfg.proto, *rest)

    @staticmethod
    def _nbytes(t: torch.Tensor) -> int:
        return t.numel() * t.element_size()

    def _check_out(self, what: str, ins, outs, in_numel: int, allow_cast: bool = True) -> None:
        """``out`` must hold exactly the result: the element count is fixed by the input, the element type is the
        input's or (reducing one-hop paths) its fp32 / 16-bit counterpart.  Anything else would read or write
        outside a buffer on the device, here and on the peers."""
        for i, o in zip(ins, outs):
            if o.numel() != in_numel:
                raise ValueError(f"{what}: out has {o.numel()} elements, the result has {in_numel}")
            if o.dtype != i.dtype:
                pair = {i.dtype, o.dtype}
                if not allow_cast or torch.float32 not in pair or not pair <= {torch.float32, torch.float16, torch.bfloat16}:
                    raise ValueError(f"{what}: out is {o.dtype}, the input is {i.dtype} (conversions: fp16/bf16 <-> fp32 "
                                     "on the one-hop reducing paths)")

    # ------------------------------------------------------------------------------ collectives
    def allreduce(self, x: TensorOrList, out: Optional[TensorOrList] = None, algo: Optional[str] = None,
                  proto: Optional[str] = None, nch: Optional[int] = None) -> None:
        """Sum over all ranks; in place unless ``out`` is given.  ``out`` may be fp32 for a 16-bit ``x`` or 16-bit for
        an fp32 ``x``: the one-hop kernels then sum in fp32 and round once, into ``out``'s type."""
        if not self.emulated and type(x) is torch.Tensor:
            if self._replay(self._key("allreduce", x, out, algo, proto, nch)):
                return
        try:
            return self._allreduce_slow(x, out, algo, proto, nch)
        finally:
            self._rec_key = None

    def _allreduce_slow(self, x, out, algo, proto, nch):
        ins = self._lists(x)
        outs = self._lists(out) or ins
        self._check_out("allreduce", ins, outs, ins[0].numel())
        nbytes = self._nbytes(ins[0])
        dt = _dtype_code(ins[0], True)
        odt = _dtype_code(outs[0], True)
        cast = odt != dt
        symm = self._symm_off_all(ins) is not None and self._symm_off_all(outs) is not None
        algo, nch = self._tuned("allreduce", nbytes, algo, nch, symm, ins + outs)
        algo = self._algo(algo, "allreduce")
        if self.world_size == 1:
            algo = "ring" if not cast else "oneshot"  # a single rank: a local copy (converted by the one-hop kernel)
        if algo == "auto":
            if nbytes <= min(self.cfg.ll_max_bytes, self.ll_capacity) and not cast:
                algo = "ll"
            elif symm and not cast and self._want_nvls(nbytes, ins + outs):
                algo = "nvls"
            elif self._peer_ok(ins) and self._peer_ok(outs):
                algo = "direct"
            elif cast and self._peer_ok(ins):
                algo = "oneshot"
            else:
                algo = "ring"
        if cast and algo not in ("direct", "oneshot"):
            raise ValueError(f"allreduce into another element type runs on the one-hop paths (direct, oneshot), not {algo}")
        if algo == "ll":
            if nbytes > self.ll_capacity:
                raise ValueError("message too large for the one-shot path")
            self._run(self.lib.mt_ll_allreduce, (dt, N.ptr_array([t.data_ptr() for t in ins]),
                                                 N.ptr_array([t.data_ptr() for t in outs]), nbytes))
        elif algo in ("direct", "nvls", "oneshot"):
            if algo == "nvls" and not (self.nvls and symm):
                raise ValueError("algo=nvls needs the multicast mapping and tensors from the symmetric heap "
                                 "(Communicator.symm_empty) at the same offset on every rank")
            variant = 1 if algo == "oneshot" else 0
            if variant == 1 and any(i.data_ptr() == o.data_ptr() for i, o in zip(ins, outs)):
                raise ValueError("one-shot all-reduce cannot run in place")
            self._launch_direct(N.DOP_ALLREDUCE, ins, outs, nbytes, dt, variant=variant, nvls=algo == "nvls", nctas=nch,
                                peers_read_in=True, peers_write_out=variant == 0, out_dtype=odt)
        elif algo == "ring":
            self._launch_ring(N.OP_ALLREDUCE, ins, outs, nbytes, dt, self._pick_proto(nbytes, proto), nch=nch)
        else:
            raise ValueError(f"unknown algo {algo}")

    def allgather(self, buff: TensorOrList, inp: Optional[TensorOrList] = None, mode: str = "temporal",
                  algo: Optional[str] = None, proto: Optional[str] = None, nch: Optional[int] = None) -> None:
        """``buff`` is ``[world, ...]``; row ``rank`` (or ``inp``) is the contribution, all rows the result
        (same in-place convention as the reference, 6_allgather.py:14-16)."""
        if not self.emulated and type(buff) is torch.Tensor:
            if self._replay(self._key("allgather", buff, inp, mode, algo, proto, nch)):
                return
        try:
            return self._allgather_slow(buff, inp, mode, algo, proto, nch)
        finally:
            self._rec_key = None

    def _allgather_slow(self, buff, inp, mode, algo, proto, nch):
        outs = self._lists(buff)
        n = self.world_size
        if outs[0].shape[0] != n:
            raise ValueError("first dimension must equal the world size")
        ranks = range(n) if self.emulated else [self.rank]
        ins = self._lists(inp) or [o[r] for o, r in zip(outs, ranks)]
        B = self._nbytes(ins[0])
        if B * n != self._nbytes(outs[0]) or ins[0].dtype != outs[0].dtype:
            raise ValueError("contribution and buffer sizes (or element types) do not match")
        dt = _dtype_code(outs[0], False)
        symm = self._symm_off_all(outs) is not None
        algo, nch = self._tuned("allgather", B * n, algo, nch, symm, ins + outs, B)
        algo = self._algo(algo, "allgather")
        if n == 1:
            algo = "ring"
        if algo == "auto":
            if B * n >= (32 << 20) and self._peer_ok(outs):
                algo = "bulk"      # copy engine: every piece read once, stored to all ranks (676 against 615 GB/s at 1 GiB on 8 GPUs)
            elif symm and self._want_nvls(B, ins + outs):
                algo = "nvls"
            else:
                algo = "direct" if self._peer_ok(outs) else "ring"
        if algo in ("direct", "nvls", "pull", "bulk", "bulkpull"):
            if algo == "nvls" and not (self.nvls and symm):
                raise ValueError("algo=nvls needs the multicast mapping and a symmetric output buffer")
            pull = algo in ("pull", "bulkpull")
            # "bulk": the push through the copy engine (cp.async.bulk), each piece of the shard read once and
            # stored to every rank from shared memory; few CTAs (nch) are enough
            # "bulkpull": the same engine pulling every peer's contribution (loads fill the link a little better
            # than stores)
            if algo in ("bulk", "bulkpull") and nch is None:
                nch = self._bulk_ctas(B)
            variant = {"pull": 1, "bulk": 4, "bulkpull": 5}.get(algo, 0)
            self._launch_direct(N.DOP_ALLGATHER, ins, outs, B, dt, variant=variant, nvls=algo == "nvls",
                                nctas=nch, peers_read_in=pull, peers_write_out=not pull,
                                in_from_out=pull and inp is None, in_extra=self.rank * B)
        else:
            self._launch_ring(N.OP_ALLGATHER, ins, outs, B, dt, self._pick_proto(B * (n - 1), proto),
                              spatial=mode == "spatial", nch=nch)

    def reducescatter(self, buff: TensorOrList, out: Optional[TensorOrList] = None, mode: str = "temporal",
                      algo: Optional[str] = None, proto: Optional[str] = None, nch: Optional[int] = None) -> None:
        """``buff`` is ``[world, ...]``; the sum over ranks of row ``rank`` lands in row ``rank`` of the
        local ``buff`` (or in ``out``, whose element type may be the fp32 / 16-bit counterpart of ``buff``'s),
        as in the reference (7_reducescatter.py:105-117)."""
        if not self.emulated and type(buff) is torch.Tensor:
            if self._replay(self._key("reducescatter", buff, out, mode, algo, proto, nch)):
                return
        try:
            return self._reducescatter_slow(buff, out, mode, algo, proto, nch)
        finally:
            self._rec_key = None

    def _reducescatter_slow(self, buff, out, mode, algo, proto, nch):
        ins = self._lists(buff)
        n = self.world_size
        if ins[0].shape[0] != n:
            raise ValueError("first dimension must equal the world size")
        ranks = range(n) if self.emulated else [self.rank]
        outs = self._lists(out) or [i[r] for i, r in zip(ins, ranks)]
        self._check_out("reducescatter", ins, outs, ins[0].numel() // n)
        B = self._nbytes(ins[0]) // n
        dt = _dtype_code(ins[0], True)
        odt = _dtype_code(outs[0], True)
        cast = odt != dt
        symm = self._symm_off_all(ins) is not None
        algo, nch = self._tuned("reducescatter", B * n, algo, nch, symm, ins + outs, B)
        algo = self._algo(algo, "reducescatter")
        if n == 1:
            algo = "ring" if not cast else "direct"
        if algo == "auto":
            # in-switch sums up to 32 MiB in total; above, pulling the shard from every peer measured faster on 4 GPUs
            # (128 MiB: 535 GB/s against 446) as on 8 (where the tuning table says the same)
            if symm and not cast and B * n <= (32 << 20) and self._want_nvls(B, ins + outs):
                algo = "nvls"
            else:
                algo = "direct" if self._peer_ok(ins) else "ring"
        if cast and algo != "direct":
            raise ValueError(f"reducescatter into another element type runs on the one-hop path (direct), not {algo}")
        if algo in ("direct", "nvls"):
            if algo == "nvls" and not (self.nvls and symm):
                raise ValueError("algo=nvls needs the multicast mapping and a symmetric input buffer")
            self._launch_direct(N.DOP_REDUCESCATTER, ins, outs, B, dt, nvls=algo == "nvls", nctas=nch,
                                peers_read_in=True, out_dtype=odt)
        else:
            self._launch_ring(N.OP_REDUCESCATTER, ins, outs, B, dt, self._pick_proto(B * (n - 1), proto),
                              spatial=mode == "spatial", nch=nch)

    def _auto_rooted(self, coll: str, nbytes: int, symm: bool, peer_ok: bool, separate: bool) -> str:
        """Automatic algorithm of broadcast and reduce.

        The chain over the FIFOs has no entry or exit barrier, so consecutive calls overlap: called back to back it
        measures fastest at most sizes (8 GPUs, 64 MiB broadcast: 511 GB/s against 424 for the multicast variant).
        A single call between other work pays the fill of the chain instead: the message crosses ``n - 1`` links
        one after the other, a FIFO step at a time.  On 8 GPUs a step of five collectives at 64 MiB took 1.42 ms
        with chain broadcast and reduce against 0.70 ms with the one-hop kernels, although each chain measured
        faster alone.  So the chain serves what it is good at: small messages (LL128: a few microseconds per
        link, no barriers), two ranks (one link, nothing to fill) and buffers the peers cannot address.  Larger
        messages take a kernel in which every byte crosses the switch at most twice."""
        n = self.world_size
        if n == 2:
            # two ranks: the chain is a single link; above 64 MiB the plain one-hop copy / sum measured faster
            if nbytes >= (128 << 20) and peer_ok and separate:
                return "pull" if coll == "broadcast" else "direct"
            return "ring"
        # one call at a time on 8 GPUs, 256 KiB: broadcast 22.6 us on the LL128 chain as through the switch; reduce 42 us
        # on the chain (every hop adds its own input) against 21.6 us in the switch
        small = (256 << 10) if coll == "broadcast" else (64 << 10)
        if nbytes <= min(small, self.cfg.ll128_max_bytes) or not separate:
            return "ring"
        if coll == "broadcast" and nbytes >= (8 << 20) and peer_ok:
            # pull + replicate over the n - 1 other ranks with plain loads and stores: every link carries one message
            # size.  One call at a time: 588 GB/s at 64 MiB and 678 at 256 MiB on 4 GPUs (544 / 655 on 8), against
            # 445 / 502 (425 / 487) for the multicast variant and 478 / 646 (440 / 552) for the copy engine.
            return "direct"
        if self.nvls and symm:
            return "nvls"
        return "direct" if peer_ok else "ring"

    def broadcast(self, buff: TensorOrList, root: int = 0, algo: Optional[str] = None, proto: Optional[str] = None,
                  nch: Optional[int] = None) -> None:
        """Copy ``buff`` of ``root`` into ``buff`` of every rank (4_broadcast.py:79-101)."""
        if not self.emulated and type(buff) is torch.Tensor:
            if self._replay(self._key("broadcast", buff, None, root, algo, proto, nch)):
                return
        try:
            return self._broadcast_slow(buff, root, algo, proto, nch)
        finally:
            self._rec_key = None

    def _broadcast_slow(self, buff, root, algo, proto, nch):
        ts = self._lists(buff)
        nbytes = self._nbytes(ts[0])
        dt = _dtype_code(ts[0], False)
        if not 0 <= root < self.world_size:
            raise ValueError("bad root")
        if self.world_size == 1:
            return
        symm = self._symm_off_all(ts) is not None
        algo, nch = self._tuned("broadcast", nbytes, algo, nch, symm, ts)
        algo = self._algo(algo, "broadcast")
        if algo == "auto":
            algo = self._auto_rooted("broadcast", nbytes, symm, self._peer_ok(ts), True)
        if algo in ("direct", "nvls", "pull", "push", "nvls1", "bulk"):
            if algo in ("nvls", "nvls1") and not (self.nvls and symm):
                raise ValueError(f"algo={algo} needs the multicast mapping and a symmetric buffer")
            # "direct"/"nvls": pull + replicate (every rank reads one sub-slice from the root and stores it to
            # all ranks, through the switch's multicast with "nvls"); "push": the root writes everything to
            # everybody; "pull": everybody reads the root; "nvls1": only the root issues multicast stores.
            # With two ranks pull + replicate is the plain push.  The multicast stores of pull + replicate move
            # whole 16-byte vectors; the plain variant takes any size and alignment.
            replicate = self.world_size > 2 and (algo in ("direct", "bulk") or nbytes % 16 == 0)
            variant = {"pull": 1, "push": 0, "nvls1": 0, "bulk": 4}.get(algo, 2 if replicate else 0)
            if algo == "bulk" and nch is None:
                nch = self._bulk_ctas(nbytes)
            self._launch_direct(N.DOP_BROADCAST, ts, ts, nbytes, dt, root=root, variant=variant,
                                nvls=algo in ("nvls", "nvls1"), nctas=nch, peers_read_in=variant != 0,
                                peers_write_out=variant != 1)
        else:
            self._launch_ring(N.OP_BROADCAST, ts, ts, nbytes, dt, self._pick_proto(nbytes, proto), root=root, nch=nch)

    def reduce(self, buff: TensorOrList, root: int = 0, out: Optional[TensorOrList] = None, algo: Optional[str] = None,
               proto: Optional[str] = None, nch: Optional[int] = None) -> None:
        """Sum of ``buff`` over all ranks, stored in ``buff`` (or ``out``) of ``root`` (5_reduce.py:99-121).  ``out``
        may be the fp32 / 16-bit counterpart of ``buff``'s element type (one-hop paths).  ``algo``: ``ring`` (chain
        over the FIFOs, any memory, in place or not), ``direct`` (the other ranks sum a slice each into the root's
        ``out``), ``direct2`` (the same without any read of the root's memory: the root adds its own input; two
        roundings), ``nvls`` (sums in the switch; heap tensors), ``direct1`` / ``nvls1`` (the root sums everything)."""
        if not self.emulated and type(buff) is torch.Tensor:
            if self._replay(self._key("reduce", buff, out, root, algo, proto, nch)):
                return
        try:
            return self._reduce_slow(buff, root, out, algo, proto, nch)
        finally:
            self._rec_key = None

    def _reduce_slow(self, buff, root, out, algo, proto, nch):
        ins = self._lists(buff)
        outs = self._lists(out) or ins
        self._check_out("reduce", ins, outs, ins[0].numel())
        if not 0 <= root < self.world_size:
            raise ValueError("bad root")
        nbytes = self._nbytes(ins[0])
        dt = _dtype_code(ins[0], True)
        odt = _dtype_code(outs[0], True)
        cast = odt != dt
        symm = self._symm_off_all(ins) is not None
        separate = all(o.data_ptr() != i.data_ptr() for i, o in zip(ins, outs))
        algo, nch = self._tuned("reduce", nbytes, algo, nch, symm and separate, ins + outs)
        algo = self._algo(algo, "reduce")
        if self.world_size == 1:
            algo = "ring" if not cast else "direct1"
        if algo == "auto":
            if cast:   # a result in another element type needs the one-hop kernel
                algo = "direct" if separate and self._peer_ok(ins) else "ring"
            else:
                algo = self._auto_rooted("reduce", nbytes, symm, self._peer_ok(ins), separate)
                # large messages the switch cannot sum: keep every read away from the root (4 GPUs, 256 MiB: 482 us
                # against 567; 64 MiB: 159 against 165; smaller messages lose to the extra pass of the root)
                if algo == "direct" and self.world_size > 2 and nbytes >= (64 << 20) and nbytes % 16 == 0 and \
                        not any(t.data_ptr() % 16 for t in ins + outs) and self._peer_ok(outs):
                    algo = "direct2"
        if cast and algo not in ("direct", "direct1"):
            raise ValueError(f"reduce into another element type runs on the one-hop paths (direct, direct1), not {algo}")
        if algo == "direct2":
            # The other ranks sum their own inputs slice by slice into the root's output and the root adds its own
            # input as the chunks arrive: nobody reads the root's memory, whose incoming link is full of the partial
            # sums.  Two roundings into the element type (partial sum, then the root's addition).
            if cast or not separate or self.world_size < 3 or nbytes % 16 or \
                    any(t.data_ptr() % 16 for t in ins + outs) or not (self._peer_ok(ins) and self._peer_ok(outs)):
                raise ValueError("algo=direct2 needs three or more ranks, a separate output of the same element type that "
                                 "the peers can address, 16-byte aligned buffers and a byte count that is a multiple of 16")
            self._launch_direct(N.DOP_REDUCE, ins, outs, nbytes, dt, root=root, variant=5, nctas=nch,
                                peers_read_in=True, peers_write_out=True, out_dtype=odt)
            return
        if algo in ("direct", "nvls", "direct1", "nvls1"):
            if algo.startswith("nvls") and not (self.nvls and symm):
                raise ValueError(f"algo={algo} needs the multicast mapping and a symmetric buffer")
            # the root reads every peer's buffer and writes its own: not safe in place
            if not separate:
                raise ValueError("direct/NVLS reduce needs a separate output on the root (pass out=)")
            # when the peers can address the root's output every rank sums one sub-slice and stores it there
            # ("reduce-scatter + gather"); otherwise ("direct1"/"nvls1" force this) the root sums everything
            spread = (not algo.endswith("1") and self.world_size > 2 and nbytes % 16 == 0 and self._peer_ok(outs))
            # NVLS: every rank sums 1/n in the switch; plain loads: the n - 1 other ranks sum 1/(n-1) each
            variant = 0 if not spread else (2 if algo.startswith("nvls") else 3)
            self._launch_direct(N.DOP_REDUCE, ins, outs, nbytes, dt, root=root, variant=variant,
                                nvls=algo.startswith("nvls"), nctas=nch, peers_read_in=True, peers_write_out=spread,
                                out_dtype=odt)
        else:
            self._launch_ring(N.OP_REDUCE, ins, outs, nbytes, dt, self._pick_proto(nbytes, proto), root=root, nch=nch)

    def alltoall(self, inp: TensorOrList, out: TensorOrList, algo: Optional[str] = None,
                 nch: Optional[int] = None) -> None:
        """Row ``p`` of ``inp`` goes to rank ``p``; row ``p`` of ``out`` comes from rank ``p``.  The default pushes
        into the peers' ``out``; ``algo="pull"`` reads the peers' ``inp``."""
        if not self.emulated and type(inp) is torch.Tensor:
            if self._replay(self._key("alltoall", inp, out, algo, nch)):
                return
        try:
            return self._alltoall_slow(inp, out, algo, nch)
        finally:
            self._rec_key = None

    def _alltoall_slow(self, inp, out, algo, nch):
        ins, outs = self._lists(inp), self._lists(out)
        n = self.world_size
        if ins[0].shape[0] != n or outs[0].shape[0] != n:
            raise ValueError("first dimension must equal the world size")
        if self._nbytes(ins[0]) != self._nbytes(outs[0]) or ins[0].dtype != outs[0].dtype:
            raise ValueError("alltoall: inp and out must have the same size and element type")
        B = self._nbytes(ins[0]) // n
        dt = _dtype_code(ins[0], False)
        if n == 1:
            outs[0].copy_(ins[0])
            return
        if algo not in (None, "auto", "push", "pull", "direct", "bulk"):
            raise ValueError("alltoall: algo is push (default), pull or bulk (push through the copy engine)")
        if algo == "bulk" and nch is None:
            nch = self._bulk_ctas(B)
        pull = (algo == "pull") or (algo in (None, "auto") and not self._peer_ok(outs) and self._peer_ok(ins))
        if not self._peer_ok(ins if pull else outs):
            raise ValueError("alltoall needs an output (push) or an input (pull) the peers can address")
        self._launch_direct(N.DOP_ALLTOALL, ins, outs, B, dt, variant=1 if pull else (4 if algo == "bulk" else 0), nctas=nch,
                            peers_read_in=pull, peers_write_out=not pull)

    # ------------------------------------------------------------------------------ point to point
    def sendrecv_route(self, route: Sequence[int], src: Optional[TensorOrList], dst: Optional[TensorOrList],
                       nbytes: Optional[int] = None, proto: Optional[str] = None, nch: Optional[int] = None) -> None:
        """Move ``src`` on ``route[0]`` to ``dst`` on ``route[-1]`` through the jump hosts in between
        (store-and-forward through their FIFOs, never through their user memory).  Every rank on the route
        calls this with the same ``route``; ranks off the route may call it too (no-op).  Real mode: pass
        ``src`` on the first rank, ``dst`` on the last, ``nbytes`` on jump hosts."""
        route = list(route)
        if len(set(route)) != len(route) or len(route) < 2:
            raise ValueError("route must list at least two distinct ranks")
        if self.emulated:
            ins = [None] * self.nlocal
            outs = [None] * self.nlocal
            s, d = self._lists(src), self._lists(dst)
            ins[route[0]] = s[route[0]]
            outs[route[-1]] = d[route[-1]]
            ref = s[route[0]]
        else:
            if self.rank not in route:
                return
            ins = [src if self.rank == route[0] else None]
            outs = [dst if self.rank == route[-1] else None]
            ref = ins[0] if ins[0] is not None else outs[0]
        if nbytes is None:
            if ref is None:
                raise ValueError("jump hosts must pass nbytes")
            nbytes = ref.numel() * ref.element_size()
        self._launch_ring(N.OP_SENDRECV, ins, outs, nbytes, N.DT_U8, self._pick_proto(nbytes, proto), chain=route,
                          nch=nch)

    _P2P_MODES = {"sys": 0, "weak": 1, "bulk": 2}

    def p2p_copy(self, src_rank: int, dst_rank: int, src_ptr: int, dst_ptr: int, nbytes: int, pull: bool = True,
                 nctas: Optional[int] = None, mode: Optional[str] = None) -> None:
        """One direct copy over a peer-mapped pointer (both ranks call this with the same arguments; the
        pointer of the remote side must be valid in the copier's address space).  ``mode``: "sys" (16-byte
        system-scope loads / stores from every thread), "weak" (volatile loads, weak stores) or "bulk" (the copy
        engine, staged in shared memory); default ``MINTCCL_P2P_MODE`` or "sys"."""
        if self.emulated or self.rank in (src_rank, dst_rank):
            m = self._P2P_MODES[(mode or os.environ.get("MINTCCL_P2P_MODE", "sys")).lower()]
            nctas = self._direct_ctas(nbytes, nctas) if (m != 2 or nctas is not None) else self._bulk_ctas(nbytes)
            N.check(self.lib.mt_p2p_mode(self._handle, self._stream(), src_rank, dst_rank, src_ptr, dst_ptr, nbytes,
                                         1 if pull else 0, nctas, m), "mt_p2p")

    def sendrecv_direct(self, src_rank: int, dst_rank: int, buff: TensorOrList, pull: bool = True,
                        nctas: Optional[int] = None, mode: Optional[str] = None) -> None:
        """Direct send/recv of a symmetric tensor: ``buff`` of ``src_rank`` is copied into ``buff`` of
        ``dst_rank`` by a single kernel on the copying side (the receiver when ``pull``), which waits for the
        other side's ready signal and answers with a done signal (1_sendrecv_direct.py:60-79 has no such
        handshake).  Both ranks call this."""
        ts = self._lists(buff)
        off = self._symm_off_all(ts)
        if off is None:
            raise ValueError("sendrecv_direct needs a symmetric tensor; use register() for ordinary tensors")
        nbytes = ts[0].numel() * ts[0].element_size()
        L = self.lib
        if self.emulated:
            sp = L.mt_comm_heap_ptr(self._handle, dst_rank, src_rank) + off
            dp = L.mt_comm_heap_ptr(self._handle, src_rank, dst_rank) + off
        else:
            sp = L.mt_comm_heap_ptr(self._handle, 0, src_rank) + off
            dp = L.mt_comm_heap_ptr(self._handle, 0, dst_rank) + off
        self.p2p_copy(src_rank, dst_rank, sp, dp, nbytes, pull, nctas, mode)

    def register(self, t: torch.Tensor) -> List[int]:
        """Make an ordinary CUDA tensor readable and writable by every peer: returns, for every rank, the
        address of that rank's tensor in THIS process.  Collective (uses the control plane once); the
        mapping is cached by allocation.  Uses cudaIpc on the allocation that contains the tensor plus the
        tensor's offset inside it (the reference sends the handle only, common.py:24-26)."""
        if self.emulated or self.world_size == 1:
            return [t.data_ptr()] * max(1, self.world_size)
        buf = C.create_string_buffer(64)
        off, size = C.c_uint64(0), C.c_uint64(0)
        N.check(self.lib.mt_ipc_export(t.data_ptr(), buf, C.byref(off), C.byref(size)), "ipc_export")
        infos = self.control.allgather((buf.raw, off.value))
        ptrs = []
        for p, (h, o) in enumerate(infos):
            if p == self.rank:
                ptrs.append(t.data_ptr())
            else:
                base = self.lib.mt_ipc_open(h)
                if not base:
                    raise RuntimeError(f"cannot open the IPC handle of rank {p}: {N.last_error()}")
                ptrs.append(base + o)
        return ptrs

    # deferred send / recv / sync, as in 2_sendrecv_indirect.py:96-167 and 3_sendrecv_buffer.py:78-151
    def send(self, buff: torch.Tensor, peer: int, rank: Optional[int] = None) -> None:
        self._pending.append(("send", self.rank if rank is None else rank, peer, buff))

    def recv(self, buff: torch.Tensor, peer: int, rank: Optional[int] = None) -> None:
        self._pending.append(("recv", self.rank if rank is None else rank, peer, buff))

    def route(self, src: int, dst: int) -> List[int]:
        """Route of a deferred transfer: the direct link on a switch; with MINTCCL_ROUTE=ring the ring
        order from ``src`` to ``dst`` (forces multi-hop forwarding through the neighbours)."""
        if os.environ.get("MINTCCL_ROUTE", "direct").lower() == "ring":
            pos = self.ring.index(src)
            out = [src]
            while out[-1] != dst:
                pos = (pos + 1) % self.world_size
                out.append(self.ring[pos])
            return out
        r = find_route(src, dst, self._topology())
        return r or [src, dst]

    def sync(self, proto: Optional[str] = None) -> None:
        """Execute all posted send/recv pairs.  Every rank calls it (jump hosts included).  Unlike the
        reference there is no master rank: the posted metadata is all-gathered and every rank derives the
        same matching and the same routes."""
        mine = [(k, r, p, b.numel() * b.element_size()) for (k, r, p, b) in self._pending]
        everyone = self.control.allgather(mine)
        sends, recvs = {}, {}
        for lst in everyone:
            for (k, r, p, nb) in lst:
                (sends if k == "send" else recvs).setdefault((r, p) if k == "send" else (p, r), []).append(nb)
        for key in sorted(set(sends) | set(recvs)):
            s, r = sends.get(key, []), recvs.get(key, [])
            if len(s) != len(r) or any(a != b for a, b in zip(s, r)):
                self._pending.clear()
                raise ValueError(f"unmatched or size-mismatched send/recv between ranks {key}: sends {s}, recvs {r}")
        cursor: dict = {}
        for (src, dst) in sorted(sends):
            for nb in sends[(src, dst)]:
                i = cursor.get((src, dst), 0)
                cursor[(src, dst)] = i + 1
                route = self.route(src, dst)
                sb = [b for (k, r, p, b) in self._pending if k == "send" and r == src and p == dst]
                rb = [b for (k, r, p, b) in self._pending if k == "recv" and r == dst and p == src]
                if self.emulated:
                    ins = [None] * self.nlocal
                    outs = [None] * self.nlocal
                    ins[src], outs[dst] = sb[i], rb[i]
                    self._launch_ring(N.OP_SENDRECV, ins, outs, nb, N.DT_U8, self._pick_proto(nb, proto), chain=route)
                elif self.rank in route:
                    self._launch_ring(N.OP_SENDRECV, [sb[i] if self.rank == src else None],
                                      [rb[i] if self.rank == dst else None], nb, N.DT_U8,
                                      self._pick_proto(nb, proto), chain=route)
        self._pending.clear()

    # ------------------------------------------------------------------------------ self tests
    def test_wait_timeout(self) -> N.MtStatus:
        """Launch a wait that nothing satisfies; it must give up after the communicator's time limit and
        leave an error record instead of hanging.  Returns the status of local rank 0."""
        N.check(self.lib.mt_test_wait_timeout(self._handle, self._stream()), "test_wait_timeout")
        return self.status(0)

    def clear_status(self) -> None:
        N.check(self.lib.mt_comm_clear_status(self._handle), "clear_status")
