// Registration service: maps ordinary device allocations of the peers into this process on request.
//
// A collective on an ordinary `torch.Tensor` needs the peers to address that tensor.  The owner exports the
// CUDA IPC handle of the allocation that contains it and asks every peer to open it; the peer answers with the
// address the allocation got in ITS address space, which the owner later announces, plus the tensor's offset,
// inside the kernel (rank_barrier_xchg in device/prims.cuh).  The request is served by a thread of its own, so
// the owner never depends on what the peer's main thread is doing: registration is one-sided, happens once per
// allocation, and ranks may discover new allocations at different times without any collective host step.
//
// The reference opens an IPC handle on every call, through MPI messages that both sides must post, and sends the
// handle of the containing block without the tensor's offset (common.py:22-38).
//
// Wire format: one fixed-size request and one fixed-size reply per connection over an abstract unix socket.
// Requests are accepted from processes of the same user only (SO_PEERCRED) and must carry the communicator's
// secret, which travelled over the control plane and never appears in a socket name.
#include <errno.h>
#include <poll.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../mintccl.h"
#include "comm_internal.h"

namespace {

constexpr uint32_t kMagic = 0x4d545247u;  // "MTRG"
enum : uint32_t { REG_OPEN = 1, REG_CLOSE = 2 };

struct RegMsg {
  uint32_t magic, op;
  int32_t rank;
  uint32_t _pad;
  uint64_t size;
  char secret[32];
  unsigned char handle[64];
};
struct RegReply {
  int32_t status;
  uint32_t _pad;
  uint64_t va;
  char err[112];
};

socklen_t abstract_addr(const char* name, sockaddr_un* a) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  const size_t n = strnlen(name, sizeof(a->sun_path) - 2);
  memcpy(a->sun_path + 1, name, n);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool same_user(int fd) {
  ucred cr{};
  socklen_t len = sizeof(cr);
  return getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cr, &len) == 0 && cr.uid == geteuid();
}

bool read_all(int fd, void* buf, size_t n, int timeout_ms) {
  size_t got = 0;
  while (got < n) {
    pollfd p{fd, POLLIN, 0};
    if (poll(&p, 1, timeout_ms) <= 0) return false;
    const ssize_t r = recv(fd, (char*)buf + got, n - got, 0);
    if (r <= 0) return false;
    got += (size_t)r;
  }
  return true;
}

bool write_all(int fd, const void* buf, size_t n) {
  size_t put = 0;
  while (put < n) {
    const ssize_t r = send(fd, (const char*)buf + put, n - put, MSG_NOSIGNAL);
    if (r <= 0) return false;
    put += (size_t)r;
  }
  return true;
}

}  // namespace

struct MtRegService {
  int device = 0;
  int sock = -1;
  char secret[32] = {};
  std::atomic<bool> stop{false};
  std::thread th;
  std::mutex mu;
  std::vector<std::string> opened;  // handles this service opened (closed again when it stops)

  void handle_one(int cs) {
    RegMsg m;
    RegReply r;
    memset(&r, 0, sizeof(r));
    if (!same_user(cs) || !read_all(cs, &m, sizeof(m), 2000) || m.magic != kMagic ||
        memcmp(m.secret, secret, sizeof(secret)) != 0) {
      r.status = -1;
      snprintf(r.err, sizeof(r.err), "request rejected");
      write_all(cs, &r, sizeof(r));
      return;
    }
    const std::string key((const char*)m.handle, 64);
    if (m.op == REG_OPEN) {
      void* p = mt_ipc_open(m.handle);
      if (!p) {
        r.status = -1;
        snprintf(r.err, sizeof(r.err), "%s", mt_last_error());
      } else {
        r.va = (uint64_t)(uintptr_t)p;
        std::lock_guard<std::mutex> lk(mu);
        opened.push_back(key);
      }
    } else if (m.op == REG_CLOSE) {
      {
        std::lock_guard<std::mutex> lk(mu);
        for (size_t i = 0; i < opened.size(); ++i)
          if (opened[i] == key) {
            opened.erase(opened.begin() + i);
            break;
          }
      }
      mt_ipc_close(m.handle);
    } else {
      r.status = -1;
      snprintf(r.err, sizeof(r.err), "unknown request");
    }
    write_all(cs, &r, sizeof(r));
  }

  void run() {
    cudaSetDevice(device);
    while (!stop.load(std::memory_order_acquire)) {
      pollfd p{sock, POLLIN, 0};
      if (poll(&p, 1, 50) <= 0) continue;
      const int cs = accept(sock, nullptr, nullptr);
      if (cs < 0) continue;
      handle_one(cs);
      close(cs);
    }
  }
};

extern "C" {

int mt_reg_start(MtComm* c, const char* sock_name, const char* secret) {
  if (!c) return mthost::fail("no communicator");
  if (c->reg) return 0;
  MtRegService* s = new MtRegService();
  s->device = c->device;
  strncpy(s->secret, secret ? secret : "", sizeof(s->secret) - 1);
  s->sock = socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un a;
  const socklen_t len = abstract_addr(sock_name, &a);
  if (s->sock < 0 || bind(s->sock, (sockaddr*)&a, len) != 0 || listen(s->sock, 64) != 0) {
    if (s->sock >= 0) close(s->sock);
    delete s;
    return mthost::fail(std::string("registration service: cannot listen on ") + sock_name);
  }
  s->th = std::thread([s] { s->run(); });
  c->reg = s;
  return 0;
}

int mt_reg_stop(MtComm* c) {
  if (!c || !c->reg) return 0;
  MtRegService* s = c->reg;
  s->stop.store(true, std::memory_order_release);
  if (s->th.joinable()) s->th.join();
  close(s->sock);
  cudaSetDevice(c->device);
  for (const std::string& k : s->opened) mt_ipc_close((const unsigned char*)k.data());
  delete s;
  c->reg = nullptr;
  return 0;
}

static int reg_request(const char* peer_sock, const char* secret, uint32_t op, int my_rank, const unsigned char handle[64],
                       uint64_t size, uint64_t* va, int timeout_ms) {
  sockaddr_un a;
  const socklen_t len = abstract_addr(peer_sock, &a);
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  int s = -1;
  while (true) {
    s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) return mthost::fail("socket() failed");
    if (connect(s, (sockaddr*)&a, len) == 0) break;
    close(s);
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    if ((t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000 > timeout_ms)
      return mthost::fail(std::string("registration service of the peer does not answer: ") + peer_sock);
    usleep(1000);
  }
  RegMsg m;
  memset(&m, 0, sizeof(m));
  m.magic = kMagic;
  m.op = op;
  m.rank = my_rank;
  m.size = size;
  strncpy(m.secret, secret ? secret : "", sizeof(m.secret) - 1);
  memcpy(m.handle, handle, 64);
  RegReply r;
  const bool ok = write_all(s, &m, sizeof(m)) && read_all(s, &r, sizeof(r), timeout_ms);
  close(s);
  if (!ok) return mthost::fail("registration request: no reply");
  if (r.status != 0) {
    r.err[sizeof(r.err) - 1] = 0;
    return mthost::fail(std::string("peer could not map the allocation: ") + r.err);
  }
  if (va) *va = r.va;
  return 0;
}

int mt_reg_share(const char* peer_sock, const char* secret, int my_rank, const unsigned char handle[64], uint64_t size,
                 uint64_t* va, int timeout_ms) {
  return reg_request(peer_sock, secret, REG_OPEN, my_rank, handle, size, va, timeout_ms);
}

int mt_reg_unshare(const char* peer_sock, const char* secret, int my_rank, const unsigned char handle[64],
                   int timeout_ms) {
  return reg_request(peer_sock, secret, REG_CLOSE, my_rank, handle, 0, nullptr, timeout_ms);
}

}  // extern "C"
