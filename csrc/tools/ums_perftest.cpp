// ums_perftest: ping-pong latency and streaming throughput of a UMS connection compared with plain TCP on loopback,
// plus a self-check of the fallback path. `ums_perftest [--size N] [--iters N] [--selftest]`
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <chrono>
#include <thread>
#include <vector>

#include "ub_util.h"
#include "ums.h"

static int fail(const char* w) {
  fprintf(stderr, "ums_perftest: FAILED: %s\n", w);
  return 1;
}
struct Api {
  int (*sock)(int, int, int);
  int (*listen_)(int, int);
  int (*accept_)(int, sockaddr*, socklen_t*);
  int (*connect_)(int, const sockaddr*, socklen_t);
  ssize_t (*send_)(int, const void*, size_t, int);
  ssize_t (*recv_)(int, void*, size_t, int);
  int (*close_)(int);
};
static bool xfer_all(const Api& a, int fd, char* buf, size_t n, bool tx) {
  size_t done = 0;
  while (done < n) {
    const ssize_t r = tx ? a.send_(fd, buf + done, n - done, 0) : a.recv_(fd, buf + done, n - done, 0);
    if (r <= 0) return false;
    done += r;
  }
  return true;
}
static int run(const Api& a, const char* name, size_t size, int iters, double* lat_us, double* gbps, bool* accel) {
  const int ls = a.sock(AF_INET, SOCK_STREAM, 0);
  sockaddr_in ad{};
  ad.sin_family = AF_INET;
  ad.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (bind(ls, (sockaddr*)&ad, sizeof(ad)) || a.listen_(ls, 8)) return fail("listen");
  socklen_t l = sizeof(ad);
  getsockname(ls, (sockaddr*)&ad, &l);
  bool ok = true;
  std::thread srv([&] {
    const int c = a.accept_(ls, nullptr, nullptr);
    std::vector<char> b(size);
    for (int i = 0; i < iters && ok; ++i) ok &= xfer_all(a, c, b.data(), size, false) && xfer_all(a, c, b.data(), size, true);
    std::vector<char> big(1 << 20);
    size_t total = 0;
    for (;;) {
      const ssize_t r = a.recv_(c, big.data(), big.size(), 0);
      if (r <= 0) break;
      total += r;
    }
    a.send_(c, &total, sizeof(total), 0);
    a.close_(c);
  });
  const int c = a.sock(AF_INET, SOCK_STREAM, 0);
  if (a.connect_(c, (sockaddr*)&ad, sizeof(ad))) return fail("connect");
  int one = 1;
  setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  *accel = ums_is_accelerated(c) == 1;
  std::vector<char> b(size), e(size);
  for (size_t i = 0; i < size; ++i) b[i] = (char)(i * 13 + 7);
  uint64_t t0 = ub::now_ns();
  for (int i = 0; i < iters && ok; ++i) {
    ok &= xfer_all(a, c, b.data(), size, true) && xfer_all(a, c, e.data(), size, false);
    if (ok && memcmp(b.data(), e.data(), size)) ok = false;
  }
  *lat_us = (ub::now_ns() - t0) / 1e3 / iters / 2;
  std::vector<char> big(1 << 20, 'x');
  const size_t stream = 512u << 20;
  t0 = ub::now_ns();
  for (size_t s = 0; s < stream && ok; s += big.size()) ok &= xfer_all(a, c, big.data(), big.size(), true);
  shutdown(c, SHUT_WR);
  if (*accel) ums_shutdown(c, SHUT_WR);
  size_t got = 0;
  ok &= xfer_all(a, c, (char*)&got, sizeof(got), false);
  *gbps = stream / ((ub::now_ns() - t0) * 1e-9) / 1e9;
  a.close_(c);
  srv.join();
  a.close_(ls);
  if (!ok || got != stream) return fail(name);
  return 0;
}

int main(int argc, char** argv) {
  size_t size = 8192;
  int iters = 20000;
  bool selftest = false;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--selftest")) selftest = true;
  }
  const Api ums{ums_socket, ums_listen, ums_accept, ums_connect, ums_send, ums_recv, ums_close};
  const Api tcp{socket, listen, accept, connect, send, recv, close};
  double lu, gu, lt, gt;
  bool au, at;
  if (run(ums, "ums", size, iters, &lu, &gu, &au)) return 1;
  if (run(tcp, "tcp", size, iters, &lt, &gt, &at)) return 1;
  printf("size=%zu: UMS one-way latency %.2f us, stream %.2f GB/s (accelerated=%d) | TCP loopback %.2f us, %.2f GB/s | "
         "latency %.0f%% lower\n", size, lu, gu, (int)au, lt, gt, (1.0 - lu / lt) * 100.0);
  if (!au) return fail("connection to a UMS listener was not accelerated");
  if (selftest) {
    // a UMS client talking to a plain TCP server must fall back without disturbing the byte stream
    const int ls = socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in ad{};
    ad.sin_family = AF_INET;
    ad.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    bind(ls, (sockaddr*)&ad, sizeof(ad));
    listen(ls, 4);
    socklen_t l = sizeof(ad);
    getsockname(ls, (sockaddr*)&ad, &l);
    std::thread srv([&] {
      const int c = accept(ls, nullptr, nullptr);
      char b[5];
      size_t n = 0;
      while (n < 5) n += recv(c, b + n, 5 - n, 0);
      send(c, b, 5, 0);
      close(c);
    });
    const int c = ums_socket(AF_INET, SOCK_STREAM, 0);
    if (ums_connect(c, (sockaddr*)&ad, sizeof(ad))) return fail("fallback connect");
    if (ums_is_accelerated(c) != 0) return fail("plain TCP peer must not be accelerated");
    char b[5] = {'h', 'e', 'l', 'l', 'o'}, e[5] = {0};
    ums_send(c, b, 5, 0);
    size_t n = 0;
    while (n < 5) n += ums_recv(c, e + n, 5 - n, 0);
    srv.join();
    ums_close(c);
    close(ls);
    if (memcmp(b, e, 5)) return fail("fallback data");
    // the other direction: an ordinary TCP client that sends five bytes at once to a UMS listener, and one that
    // first waits for a banner from the server; neither may lose bytes nor be held up by the handshake probe
    for (int banner = 0; banner < 2; ++banner) {
      const int ul = ums_socket(AF_INET, SOCK_STREAM, 0);
      sockaddr_in ua{};
      ua.sin_family = AF_INET;
      ua.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
      if (ums_bind(ul, (sockaddr*)&ua, sizeof(ua)) || ums_listen(ul, 4)) return fail("ums listen");
      socklen_t ll = sizeof(ua);
      getsockname(ul, (sockaddr*)&ua, &ll);
      bool srv_ok = false;
      std::thread usrv([&] {
        const int sc = ums_accept(ul, nullptr, nullptr);
        if (sc < 0 || ums_is_accelerated(sc) != 0) return;
        if (banner && ums_send(sc, "READY", 5, 0) != 5) return;
        char bb[5];
        size_t got = 0;
        while (got < 5) {
          const ssize_t r = ums_recv(sc, bb + got, 5 - got, 0);
          if (r <= 0) return;
          got += (size_t)r;
        }
        srv_ok = ums_send(sc, bb, 5, 0) == 5;
        ums_close(sc);
      });
      const int pc = socket(AF_INET, SOCK_STREAM, 0);
      if (connect(pc, (sockaddr*)&ua, sizeof(ua))) return fail("plain connect");
      char rb[5] = {0};
      const auto tb0 = std::chrono::steady_clock::now();
      if (banner) {
        size_t got = 0;
        while (got < 5) {
          const ssize_t r = recv(pc, rb + got, 5 - got, 0);
          if (r <= 0) return fail("banner");
          got += (size_t)r;
        }
        if (memcmp(rb, "READY", 5)) return fail("banner bytes");
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - tb0).count();
        if (ms > 1000.0) return fail("a client that waits for a banner was held up by the handshake probe");
      }
      send(pc, "plain", 5, 0);
      size_t got = 0;
      while (got < 5) {
        const ssize_t r = recv(pc, rb + got, 5 - got, 0);
        if (r <= 0) return fail("plain client: server closed early (bytes were swallowed?)");
        got += (size_t)r;
      }
      usrv.join();
      close(pc);
      ums_close(ul);
      if (!srv_ok || memcmp(rb, "plain", 5)) return fail("plain client to a UMS listener lost bytes");
    }
    ums_stats_t st;
    ums_get_stats(&st);
    if (st.conns_ums < 2 || st.conns_fallback < 1 || st.bytes_tx_ring == 0) return fail("statistics");
  }
  printf("ums_perftest: OK\n");
  return 0;
}
