// Pure index arithmetic shared by the CUDA kernels, the host runtime and the host-side protocol
// simulator: how a message is split over channels and steps, which shard a ring rank touches at
// which step, where a FIFO slot lives, and the LL128 line geometry.
//
// The reference scatters this arithmetic through every kernel (e.g. 6_allgather.py:33-44,
// 7_reducescatter.py:22-34) and drops message tails (count // 120); here tails are part of the math.
#pragma once
#include <stdint.h>
#include "layout.h"

#if defined(__CUDACC__)
#define MT_HD __host__ __device__ __forceinline__
#else
#define MT_HD static inline
#endif

// ---- LL128 geometry -------------------------------------------------------------------------------
// A line is 128 bytes: eight 16-byte lane words; the last lane word is 8 bytes of payload + an 8-byte
// flag, so a line carries 120 payload bytes (protocol.py:41-52 of the reference uses the same line).
// A warp moves 16 lines per iteration (4 coalesced 512-byte accesses): 2048 wire / 1920 payload bytes.
// Lines are grouped in pairs that carry 240 contiguous payload bytes, which keeps every payload access
// 16-byte aligned: pair p covers payload [240p, 240p+240).
#define MT_LL128_LINE 128
#define MT_LL128_LINE_PAYLOAD 120
#define MT_LL128_PAIR_PAYLOAD 240
#define MT_LL128_WARP_LINES 16
#define MT_LL128_WARP_WIRE 2048
#define MT_LL128_WARP_PAYLOAD 1920

struct MtRange {
  uint64_t lo, hi;
};

MT_HD uint64_t mt_div_up(uint64_t a, uint64_t b) { return (a + b - 1) / b; }
MT_HD uint64_t mt_round_up(uint64_t a, uint64_t b) { return mt_div_up(a, b) * b; }
MT_HD uint64_t mt_min64(uint64_t a, uint64_t b) { return a < b ? a : b; }

// Split [0, total) into `parts` contiguous ranges whose interior boundaries are multiples of `align`
// (align must be a multiple of the element size so that no element straddles two ranges).
MT_HD MtRange mt_split(uint64_t total, uint32_t parts, uint32_t idx, uint64_t align) {
  uint64_t units = mt_div_up(total, align);
  uint64_t per = units / parts, rem = units % parts;
  uint64_t lo_u = (uint64_t)idx * per + (idx < rem ? idx : rem);
  uint64_t hi_u = lo_u + per + (idx < rem ? 1 : 0);
  MtRange r;
  r.lo = mt_min64(lo_u * align, total);
  r.hi = mt_min64(hi_u * align, total);
  return r;
}

// Number of FIFO steps needed to move `bytes` when one step carries at most `step_payload` bytes.
MT_HD uint64_t mt_num_steps(uint64_t bytes, uint64_t step_payload) { return mt_div_up(bytes, step_payload); }

// Payload bytes one FIFO slot carries under each protocol.
MT_HD uint64_t mt_slot_payload(int proto, uint64_t slot_wire_bytes) {
  if (proto == MT_PROTO_LL128) return slot_wire_bytes / MT_LL128_WARP_WIRE * MT_LL128_WARP_PAYLOAD;
  return slot_wire_bytes;
}

// Wire bytes an LL128 message of `payload` bytes occupies (whole lines, pairs may be half used).
MT_HD uint64_t mt_ll128_wire_lines(uint64_t payload) {
  uint64_t pairs = payload / MT_LL128_PAIR_PAYLOAD;
  uint64_t rest = payload % MT_LL128_PAIR_PAYLOAD;
  return pairs * 2 + (rest == 0 ? 0 : (rest <= MT_LL128_LINE_PAYLOAD ? 1 : 2));
}

// Line index, inside a warp chunk, of pair p / half h (h = 0 or 1).  Access k of the warp touches
// lines 4k..4k+3, lane group g = lane / 8 owns line 4k+g: pair = (k/2)*4 + g, half = k & 1.
MT_HD uint32_t mt_ll128_line_of(uint32_t pair, uint32_t half) {
  uint32_t k = (pair / 4) * 2 + half, g = pair % 4;
  return k * 4 + g;
}

// ---- ring schedules --------------------------------------------------------------------------------
// Positions are indices into the ring order; shards are identified by ring position of their owner.
MT_HD int mt_mod(int a, int n) { int r = a % n; return r < 0 ? r + n : r; }

// All-gather: at step j (0..n-1) the rank at position q handles the shard owned by position q - j:
// j == 0 is its own shard (send), 1..n-2 receive+copy+forward, n-1 receive+copy only.
MT_HD int mt_ag_shard_pos(int q, int j, int n) { return mt_mod(q - j, n); }

// Reduce-scatter: at step j the rank at position q handles shard q - j - 1: j == 0 send,
// 1..n-2 receive+reduce+forward, n-1 receive+reduce+store of its own shard q.
MT_HD int mt_rs_shard_pos(int q, int j, int n) { return mt_mod(q - j - 1, n); }

// ---- FIFO addressing -------------------------------------------------------------------------------
// Offset (inside the owner's heap) of the FIFO that `src_peer` produces into for channel `ch`.
MT_HD uint64_t mt_fifo_off(const MtHeapLayout& L, int proto, int nranks, int ch, int src_peer) {
  uint64_t per_conn = L.fifo_slot_bytes[proto] * L.fifo_slots[proto];
  return L.fifo_off[proto] + ((uint64_t)ch * nranks + src_peer) * per_conn;
}
// Offset of the control words of connection (proto, ch, peer) inside the owner's heap.
MT_HD uint64_t mt_conn_off(const MtHeapLayout& L, int proto, int nranks, int ch, int peer) {
  return L.conn_off[proto] + ((uint64_t)ch * nranks + peer) * sizeof(MtConnCtrl);
}

// Build the heap layout for a communicator (host side, also used by the simulator and tests).
MT_HD MtHeapLayout mt_make_layout(int nranks, uint32_t nchannels, uint64_t simple_slot_bytes,
                                  uint32_t simple_slots, uint64_t ll128_slot_bytes, uint32_t ll128_slots,
                                  uint64_t ll_bytes, uint64_t scratch_bytes, uint64_t heap_bytes) {
  MtHeapLayout L;
  uint64_t off = 0;
  L.status_off = off;
  off += 4096;
  L.nchannels = nchannels;
  L._pad = 0;
  L.fifo_slot_bytes[MT_PROTO_SIMPLE] = simple_slot_bytes;
  L.fifo_slots[MT_PROTO_SIMPLE] = simple_slots;
  L.fifo_slot_bytes[MT_PROTO_LL128] = ll128_slot_bytes;
  L.fifo_slots[MT_PROTO_LL128] = ll128_slots;
  for (int p = 0; p < MT_NUM_PROTOS; ++p) {
    L.conn_off[p] = off;
    off += (uint64_t)nchannels * nranks * sizeof(MtConnCtrl);
  }
  L.bar_off = off;
  off += (uint64_t)MT_MAX_BAR_SLOTS * sizeof(MtBarSlot);
  L.sig_off = off;
  off += (uint64_t)MT_MAX_RANKS * sizeof(MtSigSlot);
  L.ll_epoch_off = off;
  off += 4096;
  off = mt_round_up(off, 4096);
  L.ll_off = off;
  L.ll_bytes = ll_bytes;
  off += 2 * (uint64_t)nranks * ll_bytes;
  off = mt_round_up(off, 4096);
  for (int p = 0; p < MT_NUM_PROTOS; ++p) {
    L.fifo_off[p] = off;
    off += (uint64_t)nchannels * nranks * L.fifo_slot_bytes[p] * L.fifo_slots[p];
    off = mt_round_up(off, 4096);
  }
  L.scratch_off = off;
  L.scratch_bytes = scratch_bytes;
  off += scratch_bytes;
  off = mt_round_up(off, 1 << 21);
  L.user_off = off;
  L.heap_bytes = heap_bytes;
  return L;
}
