// Client side of the UMS token agent: one request / one reply over the agent's Unix socket.
#include <errno.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "ums_agent_proto.h"

namespace {

bool io_full(int fd, void* buf, size_t n, bool wr) {
  char* p = static_cast<char*>(buf);
  while (n) {
    pollfd pf{fd, static_cast<short>(wr ? POLLOUT : POLLIN), 0};
    if (poll(&pf, 1, 5000) <= 0) return false;
    const ssize_t r = wr ? ::send(fd, p, n, MSG_NOSIGNAL) : ::recv(fd, p, n, 0);
    if (r <= 0) {
      if (r < 0 && (errno == EINTR || errno == EAGAIN)) continue;
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

// Sends *m and overwrites it with the reply. -1 = the agent is not there (or hung up).
int roundtrip(const char* sock, ums_agent_msg_t* m) {
  const char* path = sock && *sock ? sock : getenv("UMS_AGENT_SOCK");
  if (!path || !*path) path = UMS_AGENT_DEFAULT_SOCK;
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  if (strlen(path) >= sizeof(a.sun_path)) return -1;
  snprintf(a.sun_path, sizeof(a.sun_path), "%s", path);
  const int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  int rc = -1;
  if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0 && io_full(fd, m, sizeof(*m), true) &&
      io_full(fd, m, sizeof(*m), false) && m->magic == UMS_AGENT_MAGIC)
    rc = static_cast<int>(m->status);
  close(fd);
  return rc;
}

}  // namespace

extern "C" {

int ums_agent_put(const char* sock, uint64_t token_id, const void* value, uint32_t len) {
  if (!value || len == 0 || len > UMS_AGENT_MAX_VALUE) return UMS_AGENT_EINVAL;
  ums_agent_msg_t m{};
  m.magic = UMS_AGENT_MAGIC;
  m.op = UMS_AGENT_PUT;
  m.token_id = token_id;
  m.len = len;
  memcpy(m.value, value, len);
  return roundtrip(sock, &m);
}

int ums_agent_del(const char* sock, uint64_t token_id) {
  ums_agent_msg_t m{};
  m.magic = UMS_AGENT_MAGIC;
  m.op = UMS_AGENT_DEL;
  m.token_id = token_id;
  return roundtrip(sock, &m);
}

int ums_agent_get(const char* sock, const char* peer, uint64_t token_id, void* value, uint32_t* len) {
  if (!value || !len) return UMS_AGENT_EINVAL;
  ums_agent_msg_t m{};
  m.magic = UMS_AGENT_MAGIC;
  m.op = UMS_AGENT_GET;
  m.token_id = token_id;
  if (peer && strlen(peer) >= sizeof(m.peer)) return UMS_AGENT_EINVAL;
  if (peer) snprintf(m.peer, sizeof(m.peer), "%s", peer);
  const int rc = roundtrip(sock, &m);
  if (rc != 0) return rc;
  if (m.len > UMS_AGENT_MAX_VALUE || m.len > *len) return UMS_AGENT_EINVAL;
  memcpy(value, m.value, m.len);
  *len = m.len;
  return 0;
}

int ums_agent_stats(const char* sock, char* text, uint32_t cap) {
  if (!text || cap == 0) return UMS_AGENT_EINVAL;
  ums_agent_msg_t m{};
  m.magic = UMS_AGENT_MAGIC;
  m.op = UMS_AGENT_STATS;
  const int rc = roundtrip(sock, &m);
  if (rc != 0) return rc;
  const uint32_t n = m.len < cap - 1 ? m.len : cap - 1;
  memcpy(text, m.value, n);
  text[n] = 0;
  return 0;
}

}  // extern "C"
