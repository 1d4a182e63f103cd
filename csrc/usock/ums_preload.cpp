// LD_PRELOAD shim: unmodified TCP applications get the UMS data path. It interposes the socket calls of libc, lets
// the real calls run, and hands stream sockets over to the UMS library (listen -> announce the port, accept / connect
// -> handshake, send / recv / read / write / close -> ring buffers). Everything else, and every socket UMS does not
// own, goes straight to libc. Enable with `LD_PRELOAD=libums_preload.so` (the `ums_run` wrapper does that), the same
// usage as the reference's ums_run (src/usock/ums/tools/ums-preload.c:77-100, which maps AF_INET stream sockets to
// its kernel protocol family).
#include <dlfcn.h>
#include <errno.h>
#include <stdarg.h>
#include <stdlib.h>
#include <sys/socket.h>
#include <unistd.h>

#include "ums.h"

namespace {
template <typename T>
T real(const char* name) {
  return reinterpret_cast<T>(dlsym(RTLD_NEXT, name));
}
bool enabled() {
  static const bool on = [] {
    const char* e = getenv("UMS_DISABLE");
    return !(e && *e == '1');
  }();
  return on;
}
}  // namespace

extern "C" {

__attribute__((visibility("default"))) int listen(int fd, int backlog) {
  static auto fn = real<int (*)(int, int)>("listen");
  const int rc = fn(fd, backlog);
  if (rc == 0 && enabled()) ums_adopt_listener(fd);
  return rc;
}
__attribute__((visibility("default"))) int accept(int fd, struct sockaddr* addr, socklen_t* len) {
  static auto fn = real<int (*)(int, struct sockaddr*, socklen_t*)>("accept");
  const int nfd = fn(fd, addr, len);
  if (nfd >= 0 && enabled() && ums_owns(fd)) ums_adopt_accepted(fd, nfd);
  return nfd;
}
__attribute__((visibility("default"))) int accept4(int fd, struct sockaddr* addr, socklen_t* len, int flags) {
  static auto fn = real<int (*)(int, struct sockaddr*, socklen_t*, int)>("accept4");
  const int nfd = fn(fd, addr, len, flags);
  if (nfd >= 0 && enabled() && ums_owns(fd)) ums_adopt_accepted(fd, nfd);
  return nfd;
}
__attribute__((visibility("default"))) int connect(int fd, const struct sockaddr* addr, socklen_t len) {
  static auto fn = real<int (*)(int, const struct sockaddr*, socklen_t)>("connect");
  const int rc = fn(fd, addr, len);
  if (rc == 0 && enabled() && addr && addr->sa_family == AF_INET) {
    int type = 0;
    socklen_t tl = sizeof(type);
    if (getsockopt(fd, SOL_SOCKET, SO_TYPE, &type, &tl) == 0 && type == SOCK_STREAM) ums_adopt_connected(fd, addr);
  }
  return rc;
}
__attribute__((visibility("default"))) ssize_t send(int fd, const void* buf, size_t n, int flags) {
  if (enabled() && ums_is_accelerated(fd) == 1) return ums_send(fd, buf, n, flags);
  static auto fn = real<ssize_t (*)(int, const void*, size_t, int)>("send");
  return fn(fd, buf, n, flags);
}
__attribute__((visibility("default"))) ssize_t recv(int fd, void* buf, size_t n, int flags) {
  if (enabled() && ums_is_accelerated(fd) == 1) return ums_recv(fd, buf, n, flags);
  static auto fn = real<ssize_t (*)(int, void*, size_t, int)>("recv");
  return fn(fd, buf, n, flags);
}
__attribute__((visibility("default"))) ssize_t write(int fd, const void* buf, size_t n) {
  if (enabled() && ums_is_accelerated(fd) == 1) return ums_send(fd, buf, n, 0);
  static auto fn = real<ssize_t (*)(int, const void*, size_t)>("write");
  return fn(fd, buf, n);
}
__attribute__((visibility("default"))) ssize_t read(int fd, void* buf, size_t n) {
  if (enabled() && ums_is_accelerated(fd) == 1) return ums_recv(fd, buf, n, 0);
  static auto fn = real<ssize_t (*)(int, void*, size_t)>("read");
  return fn(fd, buf, n);
}
__attribute__((visibility("default"))) int shutdown(int fd, int how) {
  if (enabled() && ums_is_accelerated(fd) == 1) return ums_shutdown(fd, how);
  static auto fn = real<int (*)(int, int)>("shutdown");
  return fn(fd, how);
}
__attribute__((visibility("default"))) int close(int fd) {
  if (enabled() && ums_owns(fd)) return ums_close(fd);
  static auto fn = real<int (*)(int)>("close");
  return fn(fd);
}

}  // extern "C"
