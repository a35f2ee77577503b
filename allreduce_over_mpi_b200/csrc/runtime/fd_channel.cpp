// File-descriptor passing between the processes of one node (SCM_RIGHTS over abstract
// unix-domain sockets).  CUDA VMM allocations and multicast objects are shared between
// ranks as POSIX file descriptors; a descriptor only has meaning inside one process, so
// it has to travel through the kernel like this rather than through a key-value store.
//
// Protocol: the receiver listens on "\0<name>"; every sender connects, sends one message
// {tag} with the descriptor attached, and closes (no reply is awaited).  Names are chosen by the caller (the
// Python package uses "ft-<session>-<rank>").
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include "../api/flextree_comm.h"

namespace {
socklen_t make_addr(const char* name, sockaddr_un* a) {
  std::memset(a, 0, sizeof *a);
  a->sun_family = AF_UNIX;
  size_t n = std::strlen(name);
  if (n > sizeof(a->sun_path) - 2) n = sizeof(a->sun_path) - 2;
  a->sun_path[0] = '\0';  // abstract namespace: no file system entry, vanishes with the socket
  std::memcpy(a->sun_path + 1, name, n);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}
double now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}
}  // namespace

extern "C" {

int ft_fd_listen(const char* name) {
  int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) return -1;
  sockaddr_un a;
  socklen_t len = make_addr(name, &a);
  if (bind(s, (sockaddr*)&a, len) != 0 || listen(s, 128) != 0) {
    close(s);
    return -1;
  }
  return s;
}

int ft_fd_send(const char* name, int fd_to_send, int tag, int timeout_ms) {
  sockaddr_un a;
  socklen_t len = make_addr(name, &a);
  const double t0 = now_ms();
  int s = -1;
  for (;;) {  // the listener may not be up yet: retry until the limit
    s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (s < 0) return -1;
    if (connect(s, (sockaddr*)&a, len) == 0) break;
    close(s);
    s = -1;
    if (now_ms() - t0 > timeout_ms) return -2;
    usleep(2000);
  }
  msghdr msg{};
  iovec io{&tag, sizeof tag};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_control = ctl;
  msg.msg_controllen = sizeof ctl;
  cmsghdr* cm = CMSG_FIRSTHDR(&msg);
  cm->cmsg_level = SOL_SOCKET;
  cm->cmsg_type = SCM_RIGHTS;
  cm->cmsg_len = CMSG_LEN(sizeof(int));
  std::memcpy(CMSG_DATA(cm), &fd_to_send, sizeof(int));
  // No acknowledgement: a descriptor in flight holds its own reference in the kernel, so the
  // sender may close both the socket and its copy at once, and two ranks that send to each
  // other before either receives cannot deadlock.
  int rc = sendmsg(s, &msg, 0) == (ssize_t)sizeof tag ? 0 : -3;
  close(s);
  return rc;
}

int ft_fd_recv(int listen_sock, int* tag_out, int timeout_ms) {
  pollfd p{listen_sock, POLLIN, 0};
  if (poll(&p, 1, timeout_ms) <= 0) return -1;
  int s = accept4(listen_sock, nullptr, nullptr, SOCK_CLOEXEC);
  if (s < 0) return -1;
  int tag = -1, fd = -1;
  msghdr msg{};
  iovec io{&tag, sizeof tag};
  msg.msg_iov = &io;
  msg.msg_iovlen = 1;
  alignas(cmsghdr) char ctl[CMSG_SPACE(sizeof(int))] = {};
  msg.msg_control = ctl;
  msg.msg_controllen = sizeof ctl;
  pollfd q{s, POLLIN, 0};
  if (poll(&q, 1, timeout_ms) > 0 && recvmsg(s, &msg, 0) == (ssize_t)sizeof tag) {
    for (cmsghdr* cm = CMSG_FIRSTHDR(&msg); cm; cm = CMSG_NXTHDR(&msg, cm))
      if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) std::memcpy(&fd, CMSG_DATA(cm), sizeof(int));
  }
  close(s);
  if (tag_out) *tag_out = tag;
  return fd;
}

void ft_fd_close(int fd) {
  if (fd >= 0) close(fd);
}

}  // extern "C"
