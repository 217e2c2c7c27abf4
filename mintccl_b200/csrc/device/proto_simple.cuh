// Simple protocol: bulk 16-byte copies through a FIFO of slots in the receiver's heap, synchronised
// by two step counters per connection.  `tail` (in the receiver's memory, written by the sender with
// release semantics after the payload) says how many steps have been produced; `head` (in the
// sender's memory, written by the receiver) says how many have been consumed.  Both sides only ever
// poll their own memory, step counters grow monotonically across kernels (so nothing is ever cleared
// and a stale value can never satisfy a wait), and every wait is bounded.
//
// This is the protocol the reference lists as future work (protocol.py:8-10 "Simple: a protocol using
// system-level barrier like threadfence_system()"); its flow control replaces post_ll128/wait_ll128
// (protocol.py:161-189), whose zero-means-free convention races with the sender's first line.
#pragma once
#include "prims.cuh"
#include "reduce_ops.cuh"
#include "sched.h"

namespace mt {

template <class T, int NTHREADS>
struct SimplePrims {
  static constexpr int kProto = MT_PROTO_SIMPLE;
  static constexpr int kUnroll = 8;
  const MtDevComm& c;
  const int ch;
  int* s_fail;  // shared-memory word, 0 while healthy
  int recv_peer, send_peer;
  uint8_t* recv_fifo;        // local
  uint8_t* send_fifo;        // in send_peer's heap
  MtConnCtrl* recv_conn;     // local words about recv_peer
  MtConnCtrl* send_conn;     // local words about send_peer
  uint64_t* recv_head_rem;   // recv_peer's `head` word about me
  uint64_t* send_tail_rem;   // send_peer's `tail` word about me
  uint64_t recv_step, send_step;
  uint32_t slots;
  uint64_t slot_bytes;

  __device__ SimplePrims(const MtDevComm& comm, int channel, int recvPeer, int sendPeer, int* sfail)
      : c(comm), ch(channel), s_fail(sfail), recv_peer(recvPeer), send_peer(sendPeer) {
    slots = c.L.fifo_slots[kProto];
    slot_bytes = c.L.fifo_slot_bytes[kProto];
    recv_step = send_step = 0;
    recv_fifo = send_fifo = nullptr;
    recv_conn = send_conn = nullptr;
    recv_head_rem = send_tail_rem = nullptr;
    if (recv_peer >= 0) {
      recv_fifo = c.heap[c.rank] + mt_fifo_off(c.L, kProto, c.nranks, ch, recv_peer);
      recv_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, kProto, c.nranks, ch, recv_peer));
      recv_head_rem = &((MtConnCtrl*)(c.heap[recv_peer] + mt_conn_off(c.L, kProto, c.nranks, ch, c.rank)))->head;
      recv_step = load64(&recv_conn->recv_step);
    }
    if (send_peer >= 0) {
      send_fifo = c.heap[send_peer] + mt_fifo_off(c.L, kProto, c.nranks, ch, c.rank);
      send_conn = (MtConnCtrl*)(c.heap[c.rank] + mt_conn_off(c.L, kProto, c.nranks, ch, send_peer));
      send_tail_rem = &((MtConnCtrl*)(c.heap[send_peer] + mt_conn_off(c.L, kProto, c.nranks, ch, c.rank)))->tail;
      send_step = load64(&send_conn->send_step);
    }
    if (threadIdx.x == 0) *s_fail = 0;
    __syncthreads();
  }

  // Persist the step counters for the next kernel on this connection.  Must be called by all threads.
  __device__ void finish() {
    __syncthreads();
    if (threadIdx.x == 0 && *s_fail == 0) {
      if (recv_peer >= 0) store64(&recv_conn->recv_step, recv_step);
      if (send_peer >= 0) store64(&send_conn->send_step, send_step);
    }
  }

  __device__ __forceinline__ uint64_t step_payload() const { return slot_bytes; }

  // One FIFO step moving `nbytes` (<= slot_bytes):
  //   RECV: take the payload from the next slot of recv_peer's FIFO (else from `src`)
  //   SRC : with RECV, combine the received payload with `src` (sum)
  //   DST : store the result to `dst` (local memory)
  //   SEND: store the result into the next slot of my FIFO at send_peer
  // Returns false (uniformly for the CTA) if a wait expired; the caller must stop issuing steps.
  template <bool RECV, bool SEND, bool SRC, bool DST>
  __device__ __noinline__ bool step(const uint8_t* src, uint8_t* dst, uint64_t nbytes) {
    const int tid = threadIdx.x;
    // --- wait for data and for a free slot (two threads poll, the rest go straight to the barrier)
    if (RECV && tid == 0) {
      const uint64_t want = recv_step + 1;
      const uint64_t* w = &recv_conn->tail;
      if (!bounded_wait(
              c, [&] { return load64_acquire_sys(w) >= want; }, MT_ERR_TIMEOUT_TAIL, ch, MT_WHERE_SIMPLE_RECV, want,
              recv_step, (const volatile uint64_t*)w))
        atomicExch(s_fail, 1);
    }
    if (SEND && tid == 32) {
      const uint64_t want = send_step + 1;  // need head + slots >= send_step + 1
      const uint64_t* w = &send_conn->head;
      const uint64_t nslots = slots;
      if (!bounded_wait(
              c, [&] { return load64_acquire_sys(w) + nslots >= want; }, MT_ERR_TIMEOUT_HEAD, ch, MT_WHERE_SIMPLE_SEND,
              want, send_step, (const volatile uint64_t*)w))
        atomicExch(s_fail, 1);
    }
    __syncthreads();
    if (*s_fail) return false;

    const uint8_t* rslot = RECV ? recv_fifo + (recv_step % slots) * slot_bytes : nullptr;
    uint8_t* sslot = SEND ? send_fifo + (send_step % slots) * slot_bytes : nullptr;

    // --- payload.  Slots are 16-byte aligned; user pointers may not be.
    const bool aligned = (!(SRC || !RECV) || ((uintptr_t)src & 15) == 0) && (!DST || ((uintptr_t)dst & 15) == 0);
    if (aligned) {
      const uint64_t nvec = nbytes >> 4;
      constexpr uint64_t kTile = (uint64_t)NTHREADS * kUnroll;
      const uint64_t full = nvec / kTile * kTile;
      // Whole tiles: every thread moves kUnroll vectors that sit NTHREADS vectors apart, addressed from one
      // pointer per stream plus compile-time offsets (keeps the loop inside the 128 registers a 512-thread CTA
      // has; with one index computation and one bounds check per vector the loads of a tile spilled to local
      // memory).  All loads of a tile are issued before the first use.
      const uint64_t t16 = (uint64_t)tid << 4;
      for (uint64_t base = 0; base < full; base += kTile) {
        const uint64_t o = (base << 4) + t16;
        u128 v[kUnroll];
        if (RECV) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) v[u] = load128(rslot + o + (uint64_t)u * NTHREADS * 16);
          if (SRC) {
            u128 w[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) w[u] = load128_stream(src + o + (uint64_t)u * NTHREADS * 16);
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) v[u] = sum128<T>(v[u], w[u]);
          }
        } else {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) v[u] = load128_stream(src + o + (uint64_t)u * NTHREADS * 16);
        }
        if (SEND) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) store128_relaxed_sys(sslot + o + (uint64_t)u * NTHREADS * 16, v[u]);
        }
        if (DST) {
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) *reinterpret_cast<u128*>(dst + o + (uint64_t)u * NTHREADS * 16) = v[u];
        }
      }
      // the vectors behind the last whole tile, one per thread and pass
      for (uint64_t i = full + tid; i < nvec; i += NTHREADS) {
        u128 v;
        if (RECV) {
          v = load128(rslot + (i << 4));
          if (SRC) v = sum128<T>(v, load128_stream(src + (i << 4)));
        } else {
          v = load128_stream(src + (i << 4));
        }
        if (SEND) store128_relaxed_sys(sslot + (i << 4), v);
        if (DST) *reinterpret_cast<u128*>(dst + (i << 4)) = v;
      }
      // tail of fewer than 16 bytes, element by element
      using E = typename T::elem;
      const uint64_t done = nvec << 4;
      const uint64_t nel = (nbytes - done) / sizeof(E);
      if ((uint64_t)tid < nel) {
        const uint64_t o = done + (uint64_t)tid * sizeof(E);
        E e = RECV ? *reinterpret_cast<const volatile E*>(rslot + o) : *reinterpret_cast<const E*>(src + o);
        if (RECV && SRC) e = sum_elem<T>(e, *reinterpret_cast<const E*>(src + o));
        if (SEND) *reinterpret_cast<volatile E*>(sslot + o) = e;
        if (DST) *reinterpret_cast<E*>(dst + o) = e;
      }
    } else {
      using E = typename T::elem;
      const uint64_t nel = nbytes / sizeof(E);
      for (uint64_t i = tid; i < nel; i += NTHREADS) {
        const uint64_t o = i * sizeof(E);
        E e = RECV ? *reinterpret_cast<const volatile E*>(rslot + o) : *reinterpret_cast<const E*>(src + o);
        if (RECV && SRC) e = sum_elem<T>(e, *reinterpret_cast<const E*>(src + o));
        if (SEND) *reinterpret_cast<volatile E*>(sslot + o) = e;
        if (DST) *reinterpret_cast<E*>(dst + o) = e;
      }
    }

    // --- publish: every thread's stores happen-before the barrier, thread 0's release makes them
    // visible to the peer before the counter.
    __syncthreads();
    if (SEND) {
      ++send_step;
      // the release store is itself a system-scope fence followed by the store: the payload stores of all
      // threads (ordered before it by the block barrier) are visible at the peer before the counter
      if (tid == 0) store64_release_sys(send_tail_rem, send_step);
    }
    if (RECV) {
      ++recv_step;
      if (tid == 32) store64_release_sys(recv_head_rem, recv_step);
    }
    return true;
  }
};

}  // namespace mt
