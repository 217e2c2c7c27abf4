// Shared host/device description of a communicator: heap layout, control words, status codes.
//
// Every rank owns one "symmetric heap": a device allocation that all peers map into their own
// address space.  The first part of the heap is a control region whose layout is identical on every
// rank (so a rank can compute the address of a peer's control word from the peer's heap base alone),
// the rest is handed out to users as symmetric tensors.
//
// Replaces the per-call `torch.zeros(BUFF_SIZE)` staging buffers and the per-call IPC exchange of the
// reference (common.py:22-38, 3_sendrecv_buffer.py:131-139): here everything is mapped once.
#pragma once
#include <stdint.h>

#define MT_MAX_RANKS 8
#define MT_MAX_CHANNELS 96
#define MT_MAX_BAR_SLOTS 160   // one barrier slot per CTA of a direct/NVLS kernel (>= 148 SMs)

// Protocol ids (index into per-protocol arrays of the layout).
#define MT_PROTO_SIMPLE 0
#define MT_PROTO_LL128 1
#define MT_NUM_PROTOS 2

// Status codes written by kernels into MtStatus::code.  0 means "no error".
#define MT_OK 0
#define MT_ERR_TIMEOUT_TAIL 1     // consumer gave up waiting for data (Simple tail counter)
#define MT_ERR_TIMEOUT_HEAD 2     // producer gave up waiting for a credit
#define MT_ERR_TIMEOUT_FLAG 3     // LL128 consumer gave up waiting for an in-line flag
#define MT_ERR_TIMEOUT_BARRIER 4  // cross-rank barrier gave up
#define MT_ERR_TIMEOUT_SIGNAL 5   // p2p ready/done signal never arrived
#define MT_ERR_REMOTE_ABORT 6     // another CTA or rank raised the abort flag
#define MT_ERR_BAD_ARG 7

// One error record per rank, at heap offset L.status_off.  First writer wins (atomicCAS on code).
struct MtStatus {
  uint32_t code;
  uint32_t rank;
  uint32_t channel;
  uint32_t where;      // MT_WHERE_* tag of the wait that expired
  uint64_t expected;
  uint64_t seen;
  uint64_t step;
  uint32_t abort;      // set locally on error and remotely by a failing peer; polled by all waits
  uint32_t _pad[5];
};

// Flow-control words of one connection (protocol, channel, peer) as seen from the local rank.
// `tail` and `head` are written remotely by `peer` and polled locally; the two step counters are
// private to the local rank and persist from one kernel to the next so that flags never repeat.
struct MtConnCtrl {
  uint64_t tail;       // steps `peer` has produced into my FIFO for it          (remote-written)
  uint64_t head;       // steps `peer` has consumed out of its FIFO for me       (remote-written)
  uint64_t _pad0[14];
  uint64_t recv_step;  // steps I have consumed from `peer`                      (local)
  uint64_t send_step;  // steps I have produced to `peer`                        (local)
  uint64_t _pad1[14];
};

// Cross-rank barrier slot: arrive[p] is written remotely by rank p, epoch is local.  pin[p] / pout[p] carry
// what rank p announced with its arrival at the entry barrier of a one-hop collective: where ITS input and
// output live in MY address space (a plain address, or MT_PUB_HEAP_TAG | offset inside p's heap).  They are
// written before arrive[p] (release) and read after it (acquire), and not overwritten before the exit barrier
// of the same call has passed on both sides.
struct MtBarSlot {
  uint64_t arrive[MT_MAX_RANKS];
  uint64_t epoch;
  uint64_t _pad[7];
  uint64_t pin[MT_MAX_RANKS];
  uint64_t _pad1[8];
  uint64_t pout[MT_MAX_RANKS];
  uint64_t xflag[MT_MAX_RANKS];   // progress counters inside one call: [p] is written by rank p (reduce with a summing root)
};
// Announced buffer addresses: bit 63 set means "offset into the announcing rank's symmetric heap".
#define MT_PUB_HEAP_TAG 0x8000000000000000ull

// Point-to-point signal words between a pair of ranks (direct send/recv handshakes).
struct MtSigSlot {
  uint64_t ready;      // written by the peer when its buffer may be read / written
  uint64_t done;       // written by the peer when it finished with my buffer
  uint64_t ready_seq;  // local count of ready signals I consumed from the peer
  uint64_t done_seq;   // local count of done signals I consumed from the peer
  uint64_t sent_ready; // local count of ready signals I sent to the peer
  uint64_t sent_done;  // local count of done signals I sent to the peer
  uint64_t _pad[10];
};

struct MtHeapLayout {
  uint64_t status_off;
  uint64_t conn_off[MT_NUM_PROTOS];        // MtConnCtrl[channel][peer]
  uint64_t fifo_off[MT_NUM_PROTOS];        // bytes [channel][peer][slot][slot_bytes]
  uint64_t fifo_slot_bytes[MT_NUM_PROTOS]; // wire bytes of one slot
  uint32_t fifo_slots[MT_NUM_PROTOS];
  uint32_t nchannels;                      // channels the control region was sized for
  uint32_t _pad;
  uint64_t bar_off;                        // MtBarSlot[MT_MAX_BAR_SLOTS]
  uint64_t sig_off;                        // MtSigSlot[MT_MAX_RANKS]
  uint64_t ll_off;                         // one-shot low-latency staging: [2 parities][rank][ll_bytes]
  uint64_t ll_bytes;                       // wire bytes per (parity, rank) of the one-shot area
  uint64_t ll_epoch_off;                   // local u64 epoch of the one-shot area
  uint64_t scratch_off;                    // symmetric scratch used by staged algorithms
  uint64_t scratch_bytes;
  uint64_t user_off;                       // first byte handed to the symmetric allocator
  uint64_t heap_bytes;
};

// Everything a kernel needs to know about the communicator.  One per rank, stored in device memory;
// an emulated world (several ranks on one GPU, used by the single-GPU tests) stores one per emulated
// rank in a contiguous array and launches the kernel with gridDim.y = number of emulated ranks.
struct MtDevComm {
  int32_t rank;
  int32_t nranks;
  int32_t ring_pos;                    // my position in ring[]
  int32_t ring[MT_MAX_RANKS];          // ring order: ring[i+1] is the successor of ring[i]
  int32_t has_mc;                      // multicast (NVLS) mapping available
  uint64_t timeout_ns;                 // time limit of every device-side wait
  uint8_t* heap[MT_MAX_RANKS];         // heap base of every rank in MY address space
  uint8_t* mc;                         // multicast alias of the heap (all ranks at once) or nullptr
  MtHeapLayout L;
};

#ifdef __cplusplus
static_assert(sizeof(MtStatus) == 64, "MtStatus is one 64-byte record");
static_assert(sizeof(MtConnCtrl) == 256, "MtConnCtrl is two 128-byte lines");
static_assert(sizeof(MtBarSlot) == 384, "MtBarSlot is three 128-byte lines");
static_assert(sizeof(MtSigSlot) == 128, "MtSigSlot is one 128-byte line");
#endif

// Tags for MtStatus::where.
#define MT_WHERE_SIMPLE_RECV 1
#define MT_WHERE_SIMPLE_SEND 2
#define MT_WHERE_LL128_RECV 3
#define MT_WHERE_LL128_SEND 4
#define MT_WHERE_BARRIER 5
#define MT_WHERE_P2P_READY 6
#define MT_WHERE_P2P_DONE 7
#define MT_WHERE_LL_ONESHOT 8
#define MT_WHERE_GEMM_FLAG 9
#define MT_WHERE_TEST 10
#define MT_WHERE_BULK 11
#define MT_WHERE_CHUNK_FLAG 12
