// C interface of the native library (loaded from Python with ctypes).
//
// The communicator owns the symmetric heap, the peer mappings, the optional NVLS multicast mapping
// and the device-side descriptor; every collective is one kernel launch on the caller's stream.
// This layer takes the place of the reference's `common.py` (set_gpu / send_ptr / recv_ptr,
// common.py:10-38), which re-allocates staging memory and re-opens CUDA IPC handles on every call.
#pragma once
#include <stddef.h>
#include <stdint.h>
#include "device/layout.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct MtComm MtComm;

typedef struct {
  uint32_t nchannels;          // channels the FIFOs are sized for (<= MT_MAX_CHANNELS)
  uint64_t simple_slot_bytes;  // Simple protocol: bytes per FIFO slot
  uint32_t simple_slots;
  uint64_t ll128_slot_bytes;   // LL128: wire bytes per FIFO slot (multiple of 2048)
  uint32_t ll128_slots;
  uint64_t ll_bytes;           // one-shot area: wire bytes per (parity, sender)
  uint64_t scratch_bytes;
  uint64_t heap_bytes;         // whole heap (control + user part)
  uint64_t timeout_ms;         // time limit of device-side waits
  int32_t heap_kind;           // 0 = cuMem VMM (fd export, NVLS capable), 1 = cudaMalloc + cudaIpc
} MtConfig;

const char* mt_last_error(void);
int mt_version(void);
uint64_t mt_launch_count(void);          // kernels launched by this library in this process
void mt_reset_launch_count(void);
// Per-family counters of successful launches: calls, and work (message bytes for collectives and copies,
// floating-point operations for GEMMs).  Families: mt_stats_name(0 .. mt_stats_count() - 1).
int mt_stats_count(void);
const char* mt_stats_name(int kind);
int mt_stats_get(int kind, uint64_t* calls, uint64_t* work);
void mt_stats_reset(void);

// ---- communicator life cycle ------------------------------------------------------------------------
// Real communicator: one rank per process.  Steps: create -> export -> (exchange) -> import peers ->
// [multicast create/import/bind] -> finalize.
MtComm* mt_comm_create(int rank, int nranks, int device, const MtConfig* cfg);
// Bytes of the control region (FIFOs, flow-control words, barrier slots, ...) this configuration needs at the start
// of the heap; creation fails when heap_bytes is smaller.  Pure arithmetic, no GPU.
uint64_t mt_layout_user_off(int nranks, const MtConfig* cfg);
// Emulated world: `nranks` ranks on one GPU in one process; kernels are launched once for all of them
// (cooperative launch, gridDim.y = nranks).  Used by single-GPU tests and benchmarks.
MtComm* mt_comm_create_emulated(int nranks, int device, const MtConfig* cfg);
void mt_comm_destroy(MtComm* c);
int mt_comm_heap_kind(MtComm* c);                              // 0 VMM, 1 IPC
int mt_comm_export_fd(MtComm* c);                              // VMM: POSIX fd of the local heap (caller closes)
int mt_comm_export_ipc(MtComm* c, unsigned char handle[64]);   // IPC: cudaIpcMemHandle_t of the local heap
int mt_comm_import_fd(MtComm* c, int peer, int fd);
int mt_comm_import_ipc(MtComm* c, int peer, const unsigned char handle[64]);
int mt_comm_mc_supported(MtComm* c);
int mt_comm_mc_create(MtComm* c);                              // rank 0: returns fd of the multicast object
int mt_comm_mc_import(MtComm* c, int fd);                      // other ranks
int mt_comm_mc_add_device(MtComm* c);                          // all ranks, before any bind
int mt_comm_mc_bind(MtComm* c);                                // all ranks, after every rank added its device
int mt_comm_finalize(MtComm* c, const int* ring);              // ring: nranks entries; uploads descriptors
int mt_comm_set_ring(MtComm* c, const int* ring);
int mt_comm_set_timeout_ms(MtComm* c, uint64_t ms);
void* mt_comm_heap_ptr(MtComm* c, int local_rank, int peer);   // heap base of `peer` as mapped by local rank
void* mt_comm_mc_ptr(MtComm* c);
int mt_comm_layout(MtComm* c, MtHeapLayout* out);
int mt_comm_status(MtComm* c, int local_rank, MtStatus* out);  // synchronises the device
int mt_comm_clear_status(MtComm* c);
int mt_comm_nlocal(MtComm* c);

// ---- registration of ordinary device allocations (cudaIpc with base + offset) ---------------------
int mt_ipc_export(const void* ptr, unsigned char handle[64], uint64_t* offset, uint64_t* alloc_bytes);
void* mt_ipc_open(const unsigned char handle[64]);             // returns the mapped allocation base (cached, counted)
int mt_ipc_close(const unsigned char handle[64]);              // drops one reference; the last one unmaps
int mt_ipc_close_all(void);
// Registration service (host/regsrv.cpp): a thread per communicator that opens the peers' IPC handles on request,
// so that an owner can make an allocation addressable everywhere without the peers' main threads taking part.
int mt_reg_start(MtComm* c, const char* sock_name, const char* secret);
int mt_reg_stop(MtComm* c);                                    // also closes what the service opened
// Ask the service listening at `peer_sock` to map the allocation behind `handle`; *va = its base over there.
int mt_reg_share(const char* peer_sock, const char* secret, int my_rank, const unsigned char handle[64], uint64_t size,
                 uint64_t* va, int timeout_ms);
int mt_reg_unshare(const char* peer_sock, const char* secret, int my_rank, const unsigned char handle[64],
                   int timeout_ms);

// ---- file-descriptor passing over abstract unix sockets --------------------------------------------
int mt_fd_listen(const char* name);                            // returns a listening socket
int mt_fd_accept(int sock, int* tag, int timeout_ms);          // returns the received fd, tag = sender's tag
int mt_fd_send(const char* name, int tag, int fd, int timeout_ms);
void mt_fd_close(int fd);

// ---- collectives ------------------------------------------------------------------------------------
// `in` / `out` are arrays with one pointer per local rank (one entry outside emulation).
// dtype: 0 f32, 1 f16, 2 bf16, 3 bytes (copy-only ops).  proto: 0 Simple, 1 LL128.
// op (ring): 0 sendrecv(chain) 1 broadcast 2 reduce 3 allgather 4 reducescatter 5 allreduce.
int mt_ring(MtComm* c, void* stream, int proto, int dtype, int op, const void* const* in, void* const* out,
            uint64_t nbytes, int root, int spatial, const int* chain, int chain_len, int nchannels);
// op (direct): 0 allgather 1 reducescatter 2 allreduce 3 alltoall 4 broadcast 5 reduce.
// pub_in[p] / pub_out[p] (nranks entries; ignored in an emulated world): where this rank's input / output is as
// rank p addresses it, either an address valid in p's process (a CUDA IPC mapping, mt_reg_share) or
// MT_PUB_HEAP_TAG | offset inside this rank's heap; 0 where peers never touch the buffer.  mc_in_off / mc_out_off:
// heap offsets for the NVLS variants (the same on every rank).  out_dtype != dtype (reducing ops, not NVLS):
// fp16/bf16 -> fp32 or fp32 -> fp16/bf16, summed in fp32 and rounded once.  nbytes counts input bytes.
int mt_direct(MtComm* c, void* stream, int dtype, int out_dtype, int op, const void* const* in, void* const* out,
              const uint64_t* pub_in, const uint64_t* pub_out, uint64_t mc_in_off, uint64_t mc_out_off, uint64_t nbytes,
              int root, int variant, int nvls, int nctas);
int mt_ll_allreduce(MtComm* c, void* stream, int dtype, const void* const* in, void* const* out, uint64_t nbytes);
uint64_t mt_ll_capacity(MtComm* c);
// Direct copy between two ranks.  Real mode: `local_rank_role` 1 = this rank copies, 2 = passive.
// pull != 0: the receiver copies (reads the sender's memory); else the sender copies.
int mt_p2p(MtComm* c, void* stream, int src_rank, int dst_rank, const void* src_ptr, void* dst_ptr, uint64_t nbytes,
           int pull, int nctas);
// The same with the way the payload moves chosen by the caller: 0 system-scope relaxed 16-byte loads / stores (what
// mt_p2p does), 1 volatile loads and weak stores, 2 bulk copies (cp.async.bulk) staged in shared memory.
int mt_p2p_mode(MtComm* c, void* stream, int src_rank, int dst_rank, const void* src_ptr, void* dst_ptr, uint64_t nbytes,
                int pull, int nctas, int mode);

// ---- tcgen05 GEMM and its fusions with collectives (bf16, fp32 accumulate; B is [N, K] like nn.Linear) ----
int mt_gemm(void* stream, const void* A, const void* B, void* C, int M, int N, int K, int ldc, int nctas);
int mt_gemm_mxfp8(void* stream, const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                  int K, int ldc, int nctas);
// Plain GEMMs with M % 256 == 0 run on CTA pairs (tcgen05 cta_group::2) when MINTCCL_GEMM_PAIR is not 0; a wait
// of that kernel that expired leaves 1 here (synchronises the device).
int mt_gemm_pair_error(void);
void mt_gemm_set_pair(int mode);                          // 1 pairs, 0 single CTA, -1 environment / default
int mt_ag_gemm(MtComm* c, void* stream, const void* const* a_shard, const void* const* B, void* const* C,
               uint64_t gather_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int ldc, int ncomm,
               int nctas, int comm_mode, uint64_t shard_off, int comm_split);
int mt_gemm_rs(MtComm* c, void* stream, const void* const* A, const void* const* B, void* const* out,
               uint64_t stage_off, uint64_t flags_off, uint64_t epoch, int M, int N, int K, int nred, int nctas);

int mt_ag_gemm_mxfp8(MtComm* c, void* stream, const void* const* a_shard, const void* const* sfa, const void* const* B,
                     const void* const* sfb, void* const* C, uint64_t gather_off, uint64_t flags_off, uint64_t epoch,
                     int M, int N, int K, int ldc, int ncomm, int nctas);
int mt_gemm_rs_mxfp8(MtComm* c, void* stream, const void* const* A, const void* const* sfa, const void* const* B,
                     const void* const* sfb, void* const* out, uint64_t stage_off, uint64_t flags_off, uint64_t epoch,
                     int M, int N, int K, int nred, int nctas);
int mt_mxfp8_reduce(MtComm* c, void* stream, int op, uint64_t data_in_off, uint64_t scale_in_off,
                    uint64_t data_out_off, uint64_t scale_out_off, void* const* data_out, void* const* scale_out,
                    uint64_t nelems, int nctas);

// ---- device-wait self test: a wait nothing satisfies must time out and report, not hang -----------
int mt_test_wait_timeout(MtComm* c, void* stream);

// ---- host model of the fused GEMM + collective protocols (threads and atomics, no GPU; sim/sim_fused.cpp) ----
// op: 0 all-gather -> GEMM, 1 GEMM -> reduce-scatter.  Returns 0 ok, 1 data of another call was read, 2 a wait gave
// up, -1 bad argument.
void mt_sched_fused_tile(int mode, int t, int M, int N, int nranks, int rank, int raster, int tile_rows, int tile_cols,
                         int* out);   // tile order of the GEMM kernels: {row block, column block, owner, block in owner}
int mt_sim_fused(int op, int nranks, int per, int nbs, int ngemm, int nextra, int pair, int iters, uint32_t seed,
                 int dead_rank, int slow_rank, int double_buffer, uint64_t timeout_ms);

// Host model of the one-hop collectives (entry / exit barrier per CTA index, in-place buffers rewritten between
// calls) and of the one-shot all-reduce (sim/sim_direct.cpp).  only_op: -1 random mix, 0 two-shot all-reduce,
// 1 all-gather, 2 reduce-scatter, 3 all-to-all, 4 one-shot all-reduce.  Returns 0 ok, 1 wrong data, 2 a wait gave up.
int mt_sim_direct(int nranks, int nctas, int iters, uint32_t seed, int only_op, int slow_rank, int dead_rank,
                  int exit_barrier, uint64_t timeout_ms);

// ---- topology ---------------------------------------------------------------------------------------
// bw: n*n row-major matrix of link bandwidth (0 = no link).  Results are written to `out`.
int mt_find_ring(const double* bw, int n, int* out);                          // returns length (n+1) or 0
int mt_find_route(const double* bw, int n, int src, int dst, int* out);       // returns length or 0
int mt_topo_probe(int ndev, double* bw, int measure, uint64_t probe_bytes);   // fills n*n matrix (GB/s or 1.0)
int mt_topo_probe_pair(int src, int dst, uint64_t probe_bytes, double* gbs);  // one pair: GB/s, 0 without peer access

#ifdef __cplusplus
}
#endif
