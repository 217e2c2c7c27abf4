// Passing file descriptors between the rank processes of one node over abstract unix sockets
// (SCM_RIGHTS).  A cuMem allocation is exported as a POSIX fd; the peer needs that very descriptor in
// its own process to import and map the allocation.  The reference exchanges 64-byte cudaIpc handles
// through MPI instead (common.py:22-38); fds cannot travel through MPI or a key-value store.
#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <string>

#include "../mintccl.h"

static socklen_t make_addr(const char* name, sockaddr_un* a) {
  memset(a, 0, sizeof(*a));
  a->sun_family = AF_UNIX;
  const size_t n = strnlen(name, sizeof(a->sun_path) - 2);
  a->sun_path[0] = '\0';  // abstract namespace: no file to clean up
  memcpy(a->sun_path + 1, name, n);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

extern "C" int mt_fd_listen(const char* name) {
  int s = socket(AF_UNIX, SOCK_STREAM, 0);
  if (s < 0) return -1;
  sockaddr_un a;
  socklen_t len = make_addr(name, &a);
  if (bind(s, (sockaddr*)&a, len) != 0 || listen(s, 64) != 0) {
    close(s);
    return -1;
  }
  return s;
}

// Only processes of the same user may hand us a descriptor: the socket name is visible to everybody in the
// network namespace, and whatever arrives is mapped as a peer's heap.
static bool same_user(int fd) {
  ucred cr{};
  socklen_t len = sizeof(cr);
  return getsockopt(fd, SOL_SOCKET, SO_PEERCRED, &cr, &len) == 0 && cr.uid == geteuid();
}

extern "C" int mt_fd_accept(int sock, int* tag, int timeout_ms) {
  int cs = -1;
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  while (true) {  // connections of other users are dropped without using up the caller's accept
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const long left = timeout_ms - ((t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000);
    pollfd p{sock, POLLIN, 0};
    if (left <= 0 || poll(&p, 1, (int)left) <= 0) return -1;
    cs = accept(sock, nullptr, nullptr);
    if (cs < 0) return -1;
    if (same_user(cs)) break;
    close(cs);
  }
  int payload = -1;
  iovec iov{&payload, sizeof(payload)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  pollfd q{cs, POLLIN, 0};
  int fd = -1;
  if (poll(&q, 1, timeout_ms) > 0 && recvmsg(cs, &msg, 0) == (ssize_t)sizeof(payload)) {
    for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(&fd, CMSG_DATA(c), sizeof(int));
    }
  }
  close(cs);
  if (tag) *tag = payload;
  return fd;
}

extern "C" int mt_fd_send(const char* name, int tag, int fd, int timeout_ms) {
  sockaddr_un a;
  socklen_t len = make_addr(name, &a);
  timespec t0;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  int s = -1;
  while (true) {  // the listener may not be up yet: retry until the time limit runs out
    s = socket(AF_UNIX, SOCK_STREAM, 0);
    if (s < 0) return -1;
    if (connect(s, (sockaddr*)&a, len) == 0) break;
    close(s);
    timespec t1;
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const long ms = (t1.tv_sec - t0.tv_sec) * 1000 + (t1.tv_nsec - t0.tv_nsec) / 1000000;
    if (ms > timeout_ms) return -1;
    usleep(2000);
  }
  iovec iov{&tag, sizeof(tag)};
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  // A descriptor in flight is kept alive by the kernel, so the sender may close at once; with the
  // listen backlog this lets every rank send to all peers first and accept afterwards.
  const int rc = sendmsg(s, &msg, 0) == (ssize_t)sizeof(tag) ? 0 : -1;
  close(s);
  return rc;
}

extern "C" void mt_fd_close(int fd) {
  if (fd >= 0) close(fd);
}
