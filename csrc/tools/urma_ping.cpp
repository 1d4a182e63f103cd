// urma_ping: endpoint-level reachability and round-trip probe over URMA two-sided messages.
//
//   urma_ping --dev shm0 --server 18600                 echo service (one client at a time, Ctrl-C / EOF ends it)
//   urma_ping --dev shm0 --client 127.0.0.1 18600 [--count 5] [--size 64] [--interval-ms 100] [--timeout-ms 1000]
//   urma_ping --dev shm0 [--count 5]                    both ends in this process (self test of the device)
//
// Every probe is a SEND carrying a sequence number and a timestamp; the far side answers with a SEND of the same
// payload. Output follows ping(8): one line per reply with the round-trip time, then sent / received / loss and
// min / avg / max. Jetty information is exchanged over TCP, like the reference's perftest and sample programs do;
// the reference's own tool resolves the peer by EID through netlink (src/urma/tools/urma_ping/ping_run.c), which has
// no counterpart without the kernel modules.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/select.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <vector>

#include "ub_util.h"
#include "urma_simple.h"

namespace {

constexpr uint32_t kMaxProbe = 65536;

struct Probe {
  uint64_t seq;
  uint64_t t_ns;
};

int fail(const char* w) {
  fprintf(stderr, "urma_ping: FAILED: %s\n", w);
  return 1;
}
bool xfer(int fd, void* b, size_t n, bool tx) {
  char* p = static_cast<char*>(b);
  while (n) {
    const ssize_t r = tx ? write(fd, p, n) : read(fd, p, n);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}

// Echo side: every received message goes back to `peer`. Runs until `stop()` says so.
template <typename Stop>
void echo_loop(urma_simple_ep_t* ep, urma_target_jetty_t* peer, uint32_t size, Stop stop) {
  constexpr int kSlots = 16;
  std::vector<std::vector<uint8_t>> rb(kSlots, std::vector<uint8_t>(size));
  for (int i = 0; i < kSlots; ++i) urma_simple_post_recv(ep, rb[i].data(), size, i);
  while (!stop()) {
    int st[16];
    uint64_t uc[16];
    uint32_t ln[16], fl[16];
    const int n = urma_simple_poll(ep, 16, st, uc, ln, nullptr, fl);
    for (int i = 0; i < n; ++i) {
      if (!(fl[i] & URMA_CR_FLAG_RECV) || st[i] != 0) continue;
      urma_simple_post(ep, peer, URMA_OPC_SEND, nullptr, 0, nullptr, (uint64_t)rb[uc[i]].data(), ln[i], 0, 1000, 0);
      urma_simple_post_recv(ep, rb[uc[i]].data(), size, uc[i]);
    }
    if (n <= 0) sched_yield();
  }
}

}  // namespace

int main(int argc, char** argv) {
  std::string dev = "shm0", host = "127.0.0.1";
  int server = -1, client = -1, count = 5, interval_ms = 100, timeout_ms = 1000;
  uint32_t size = 64;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--dev") && i + 1 < argc) dev = argv[++i];
    else if (!strcmp(argv[i], "--count") && i + 1 < argc) count = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--interval-ms") && i + 1 < argc) interval_ms = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--timeout-ms") && i + 1 < argc) timeout_ms = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--server") && i + 1 < argc) server = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--client") && i + 2 < argc) {
      host = argv[++i];
      client = atoi(argv[++i]);
    } else {
      fprintf(stderr, "usage: urma_ping --dev <dev> [--server <port> | --client <host> <port>] [--count n] "
                      "[--size bytes] [--interval-ms n] [--timeout-ms n]\n");
      return 2;
    }
  }
  size = std::min<uint32_t>(std::max<uint32_t>(size, sizeof(Probe)), kMaxProbe);
  urma_context_t* ctx = urma_simple_open(dev.c_str());
  if (!ctx) return fail("open device");
  urma_simple_ep_t* ep = urma_simple_ep_create(ctx, 64, 7, 0);
  if (!ep) return fail("endpoint");
  uint8_t mine[URMA_SIMPLE_JETTY_BLOB], theirs[URMA_SIMPLE_JETTY_BLOB];
  urma_simple_ep_blob(ep, mine);

  if (server >= 0) {
    const int ls = socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(server);
    a.sin_addr.s_addr = htonl(INADDR_ANY);
    if (bind(ls, (sockaddr*)&a, sizeof(a)) || listen(ls, 1)) return fail("listen");
    printf("urma_ping server ready on port %d (device %s)\n", server, dev.c_str());
    fflush(stdout);
    const int tcp = accept(ls, nullptr, nullptr);
    close(ls);
    if (tcp < 0 || !xfer(tcp, mine, sizeof(mine), true) || !xfer(tcp, theirs, sizeof(theirs), false))
      return fail("exchange");
    urma_target_jetty_t* peer = urma_simple_ep_import(ctx, theirs, 7);
    if (!peer) return fail("import");
    echo_loop(ep, peer, kMaxProbe, [&] {   // the client chooses the probe size
      fd_set s;
      FD_ZERO(&s);
      FD_SET(tcp, &s);
      timeval tv{0, 0};
      char c;
      return select(tcp + 1, &s, nullptr, nullptr, &tv) > 0 && read(tcp, &c, 1) <= 0;
    });
    printf("urma_ping server: client left\n");
    return 0;
  }

  // ---- probing side ----
  urma_simple_ep_t* echo_ep = nullptr;
  urma_context_t* echo_ctx = nullptr;
  int tcp = -1;
  if (client >= 0) {
    tcp = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(client);
    a.sin_addr.s_addr = inet_addr(host.c_str());
    if (connect(tcp, (sockaddr*)&a, sizeof(a))) return fail("connect");
    if (!xfer(tcp, theirs, sizeof(theirs), false) || !xfer(tcp, mine, sizeof(mine), true)) return fail("exchange");
  } else {
    echo_ctx = urma_simple_open(dev.c_str());
    echo_ep = echo_ctx ? urma_simple_ep_create(echo_ctx, 64, 7, 0) : nullptr;
    if (!echo_ep) return fail("second endpoint");
    urma_simple_ep_blob(echo_ep, theirs);
  }
  urma_target_jetty_t* peer = urma_simple_ep_import(ctx, theirs, 7);
  if (!peer) return fail("import");
  urma_target_jetty_t* back = echo_ep ? urma_simple_ep_import(echo_ctx, mine, 7) : nullptr;

  std::vector<uint8_t> tx(size, 0), rx(size, 0);
  std::vector<uint8_t> echo_buf(size);
  if (echo_ep) urma_simple_post_recv(echo_ep, echo_buf.data(), size, 0);
  printf("URMA PING %s (%s): %u data bytes\n", client >= 0 ? host.c_str() : "self", dev.c_str(), size);
  int received = 0;
  double mn = 1e30, mx = 0, sum = 0;
  for (int seq = 0; seq < count; ++seq) {
    urma_simple_post_recv(ep, rx.data(), size, 1);
    Probe p{(uint64_t)seq, ub::now_ns()};
    memcpy(tx.data(), &p, sizeof(p));
    if (urma_simple_post(ep, peer, URMA_OPC_SEND, nullptr, 0, nullptr, (uint64_t)tx.data(), size, 0, 2, 0) != 0)
      return fail("post send");
    const uint64_t deadline = p.t_ns + (uint64_t)timeout_ms * 1000000ull;
    bool got = false;
    while (!got && ub::now_ns() < deadline) {
      if (echo_ep) {  // self test: play the far side too
        int st;
        uint64_t uc;
        uint32_t ln, fl;
        if (urma_simple_poll(echo_ep, 1, &st, &uc, &ln, nullptr, &fl) == 1 && (fl & URMA_CR_FLAG_RECV) && st == 0) {
          urma_simple_post(echo_ep, back, URMA_OPC_SEND, nullptr, 0, nullptr, (uint64_t)echo_buf.data(), ln, 0, 3, 0);
          urma_simple_post_recv(echo_ep, echo_buf.data(), size, 0);
        }
      }
      int st;
      uint64_t uc;
      uint32_t ln, fl;
      if (urma_simple_poll(ep, 1, &st, &uc, &ln, nullptr, &fl) == 1 && (fl & URMA_CR_FLAG_RECV)) {
        Probe r;
        memcpy(&r, rx.data(), sizeof(r));
        if (st == 0 && r.seq == (uint64_t)seq) {
          const double us = (ub::now_ns() - r.t_ns) / 1e3;
          printf("%u bytes from %s: seq=%d time=%.2f us\n", ln, client >= 0 ? host.c_str() : "self", seq, us);
          mn = std::min(mn, us);
          mx = std::max(mx, us);
          sum += us;
          ++received;
          got = true;
        }
      }
    }
    if (!got) printf("seq=%d timed out after %d ms\n", seq, timeout_ms);
    if (seq + 1 < count && interval_ms > 0) usleep(interval_ms * 1000);
  }
  printf("--- %s ping statistics ---\n%d sent, %d received, %.0f%% loss\n", dev.c_str(), count, received,
         count ? 100.0 * (count - received) / count : 0.0);
  if (received) printf("rtt min/avg/max = %.2f/%.2f/%.2f us\n", mn, sum / received, mx);
  if (tcp >= 0) close(tcp);
  return received == count ? 0 : 1;
}
