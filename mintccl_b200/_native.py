"""ctypes binding of ``_C/libmintccl_b200.so`` (interface: ``csrc/mintccl.h``).

The library is built in-tree by ``mintccl_b200.build``.  On a machine with a GPU a missing library is an
error (there is no silent PyTorch fallback for the CUDA path); on a CPU-only machine the host-side parts
(topology search, fd passing, protocol simulator) are still usable and the GPU entry points are simply
never called.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "_C" / "libmintccl_b200.so"
_lib = None

MT_MAX_RANKS = 8
MT_MAX_CHANNELS = 96
PROTO_SIMPLE, PROTO_LL128 = 0, 1
DT_F32, DT_F16, DT_BF16, DT_U8 = 0, 1, 2, 3
OP_SENDRECV, OP_BROADCAST, OP_REDUCE, OP_ALLGATHER, OP_REDUCESCATTER, OP_ALLREDUCE = range(6)
DOP_ALLGATHER, DOP_REDUCESCATTER, DOP_ALLREDUCE, DOP_ALLTOALL, DOP_BROADCAST, DOP_REDUCE = range(6)

ERR_NAMES = {0: "ok", 1: "timeout waiting for data (tail)", 2: "timeout waiting for a credit (head)",
             3: "timeout waiting for an LL128 flag", 4: "timeout in cross-rank barrier",
             5: "timeout waiting for a p2p signal", 6: "aborted by another CTA or rank", 7: "bad argument"}


class MtConfig(C.Structure):
    _fields_ = [("nchannels", C.c_uint32), ("simple_slot_bytes", C.c_uint64), ("simple_slots", C.c_uint32),
                ("ll128_slot_bytes", C.c_uint64), ("ll128_slots", C.c_uint32), ("ll_bytes", C.c_uint64),
                ("scratch_bytes", C.c_uint64), ("heap_bytes", C.c_uint64), ("timeout_ms", C.c_uint64),
                ("heap_kind", C.c_int32)]


class MtStatus(C.Structure):
    _fields_ = [("code", C.c_uint32), ("rank", C.c_uint32), ("channel", C.c_uint32), ("where", C.c_uint32),
                ("expected", C.c_uint64), ("seen", C.c_uint64), ("step", C.c_uint64), ("abort", C.c_uint32),
                ("_pad", C.c_uint32 * 5)]


class MtHeapLayout(C.Structure):
    _fields_ = [("status_off", C.c_uint64), ("conn_off", C.c_uint64 * 2), ("fifo_off", C.c_uint64 * 2),
                ("fifo_slot_bytes", C.c_uint64 * 2), ("fifo_slots", C.c_uint32 * 2), ("nchannels", C.c_uint32),
                ("_pad", C.c_uint32), ("bar_off", C.c_uint64), ("sig_off", C.c_uint64), ("ll_off", C.c_uint64),
                ("ll_bytes", C.c_uint64), ("ll_epoch_off", C.c_uint64), ("scratch_off", C.c_uint64),
                ("scratch_bytes", C.c_uint64), ("user_off", C.c_uint64), ("heap_bytes", C.c_uint64)]


def available() -> bool:
    return _LIB_PATH.exists()


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """Load (once) and return the native library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m mintccl_b200.build`")
    L = C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)
    vp, i32, u64, cp = C.c_void_p, C.c_int, C.c_uint64, C.c_char_p
    pp = C.POINTER(C.c_void_p)
    ip = C.POINTER(C.c_int)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("mt_last_error", cp)
    sig("mt_version", i32)
    sig("mt_launch_count", u64)
    sig("mt_reset_launch_count", None)
    sig("mt_stats_count", i32)
    sig("mt_stats_name", cp, i32)
    sig("mt_stats_get", i32, i32, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64))
    sig("mt_stats_reset", None)
    sig("mt_comm_create", vp, i32, i32, i32, C.POINTER(MtConfig))
    sig("mt_layout_user_off", u64, i32, C.POINTER(MtConfig))
    sig("mt_comm_create_emulated", vp, i32, i32, C.POINTER(MtConfig))
    sig("mt_comm_destroy", None, vp)
    sig("mt_comm_heap_kind", i32, vp)
    sig("mt_comm_export_fd", i32, vp)
    sig("mt_comm_export_ipc", i32, vp, C.c_char_p)
    sig("mt_comm_import_fd", i32, vp, i32, i32)
    sig("mt_comm_import_ipc", i32, vp, i32, C.c_char_p)
    sig("mt_comm_mc_supported", i32, vp)
    sig("mt_comm_mc_create", i32, vp)
    sig("mt_comm_mc_import", i32, vp, i32)
    sig("mt_comm_mc_add_device", i32, vp)
    sig("mt_comm_mc_bind", i32, vp)
    sig("mt_comm_finalize", i32, vp, ip)
    sig("mt_comm_set_ring", i32, vp, ip)
    sig("mt_comm_set_timeout_ms", i32, vp, u64)
    sig("mt_comm_heap_ptr", vp, vp, i32, i32)
    sig("mt_comm_mc_ptr", vp, vp)
    sig("mt_comm_layout", i32, vp, C.POINTER(MtHeapLayout))
    sig("mt_comm_status", i32, vp, i32, C.POINTER(MtStatus))
    sig("mt_comm_clear_status", i32, vp)
    sig("mt_comm_nlocal", i32, vp)
    sig("mt_ipc_export", i32, vp, C.c_char_p, C.POINTER(u64), C.POINTER(u64))
    sig("mt_ipc_open", vp, C.c_char_p)
    sig("mt_ipc_close", i32, C.c_char_p)
    sig("mt_ipc_close_all", i32)
    sig("mt_reg_start", i32, vp, cp, cp)
    sig("mt_reg_stop", i32, vp)
    sig("mt_reg_share", i32, cp, cp, i32, C.c_char_p, u64, C.POINTER(u64), i32)
    sig("mt_reg_unshare", i32, cp, cp, i32, C.c_char_p, i32)
    sig("mt_fd_listen", i32, cp)
    sig("mt_fd_accept", i32, i32, ip, i32)
    sig("mt_fd_send", i32, cp, i32, i32, i32)
    sig("mt_fd_close", None, i32)
    sig("mt_ring", i32, vp, vp, i32, i32, i32, pp, pp, u64, i32, i32, ip, i32, i32)
    sig("mt_direct", i32, vp, vp, i32, i32, i32, pp, pp, C.POINTER(u64), C.POINTER(u64), u64, u64, u64, i32, i32, i32, i32)
    sig("mt_ll_allreduce", i32, vp, vp, i32, pp, pp, u64)
    sig("mt_ll_capacity", u64, vp)
    sig("mt_p2p", i32, vp, vp, i32, i32, vp, vp, u64, i32, i32)
    sig("mt_p2p_mode", i32, vp, vp, i32, i32, vp, vp, u64, i32, i32, i32)
    sig("mt_gemm", i32, vp, vp, vp, vp, i32, i32, i32, i32, i32)
    sig("mt_gemm_mxfp8", i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32)
    sig("mt_sim_direct", i32, i32, i32, i32, C.c_uint32, i32, i32, i32, i32, u64)
    sig("mt_sim_fused", i32, i32, i32, i32, i32, i32, i32, i32, i32, C.c_uint32, i32, i32, i32, u64)
    sig("mt_sched_fused_tile", None, i32, i32, i32, i32, i32, i32, i32, i32, i32, ip)
    sig("mt_gemm_pair_error", i32)
    sig("mt_gemm_set_pair", None, i32)
    sig("mt_ag_gemm", i32, vp, vp, pp, pp, pp, u64, u64, u64, i32, i32, i32, i32, i32, i32, i32, u64, i32)
    sig("mt_gemm_rs", i32, vp, vp, pp, pp, pp, u64, u64, u64, i32, i32, i32, i32, i32)
    sig("mt_ag_gemm_mxfp8", i32, vp, vp, pp, pp, pp, pp, pp, u64, u64, u64, i32, i32, i32, i32, i32, i32)
    sig("mt_gemm_rs_mxfp8", i32, vp, vp, pp, pp, pp, pp, pp, u64, u64, u64, i32, i32, i32, i32, i32)
    sig("mt_mxfp8_reduce", i32, vp, vp, i32, u64, u64, u64, u64, pp, pp, u64, i32)
    sig("mt_test_wait_timeout", i32, vp, vp)
    sig("mt_find_ring", i32, C.POINTER(C.c_double), i32, ip)
    sig("mt_find_route", i32, C.POINTER(C.c_double), i32, i32, i32, ip)
    sig("mt_topo_probe", i32, i32, C.POINTER(C.c_double), i32, u64)
    sig("mt_topo_probe_pair", i32, i32, i32, u64, C.POINTER(C.c_double))
    _lib = L
    return L


def last_error() -> str:
    return lib().mt_last_error().decode(errors="replace")


def check(rc: int, what: str) -> int:
    if rc is None or rc < 0:
        raise RuntimeError(f"{what}: {last_error()}")
    return rc


def ptr_array(ptrs) -> "C.Array":
    arr = (C.c_void_p * MT_MAX_RANKS)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


def u64_array(vals) -> "C.Array":
    arr = (C.c_uint64 * MT_MAX_RANKS)()
    for i, v in enumerate(vals):
        arr[i] = v
    return arr
