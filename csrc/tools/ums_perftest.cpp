// ums_perftest: ping-pong latency and streaming throughput of a UMS connection compared with plain TCP on loopback,
// plus a self-check of the fallback path. `ums_perftest [--size N] [--iters N] [--conns N] [--selftest] [--linkgroups]`
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
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
  std::atomic<bool> ok{true};   // written by both threads
  std::thread srv([&] {
    const int c = a.accept_(ls, nullptr, nullptr);
    std::vector<char> b(size);
    for (int i = 0; i < iters && ok; ++i)
      if (!(xfer_all(a, c, b.data(), size, false) && xfer_all(a, c, b.data(), size, true))) ok = false;
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
    if (!(xfer_all(a, c, b.data(), size, true) && xfer_all(a, c, e.data(), size, false))) ok = false;
    if (ok && memcmp(b.data(), e.data(), size)) ok = false;
  }
  *lat_us = (ub::now_ns() - t0) / 1e3 / iters / 2;
  std::vector<char> big(1 << 20, 'x');
  const size_t stream = 512u << 20;
  t0 = ub::now_ns();
  for (size_t s = 0; s < stream && ok; s += big.size())
    if (!xfer_all(a, c, big.data(), big.size(), true)) ok = false;
  shutdown(c, SHUT_WR);
  if (*accel) ums_shutdown(c, SHUT_WR);
  size_t got = 0;
  if (!xfer_all(a, c, (char*)&got, sizeof(got), false)) ok = false;
  *gbps = stream / ((ub::now_ns() - t0) * 1e-9) / 1e9;
  a.close_(c);
  srv.join();
  a.close_(ls);
  if (!ok || got != stream) return fail(name);
  return 0;
}

// `conns` connections at once, each a ping-pong between a client thread and a server thread of its own: the average
// one-way latency over all of them (the reference's "10 connections" row).
static int run_many(const Api& a, const char* name, size_t size, int iters, int conns, double* lat_us) {
  const int ls = a.sock(AF_INET, SOCK_STREAM, 0);
  sockaddr_in ad{};
  ad.sin_family = AF_INET;
  ad.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (bind(ls, (sockaddr*)&ad, sizeof(ad)) || a.listen_(ls, conns + 4)) return fail("listen");
  socklen_t l = sizeof(ad);
  getsockname(ls, (sockaddr*)&ad, &l);
  std::atomic<bool> ok{true};
  std::atomic<int> ready{0};
  std::vector<std::thread> servers, clients;
  std::thread acceptor([&] {
    for (int k = 0; k < conns; ++k) {
      const int c = a.accept_(ls, nullptr, nullptr);
      if (c < 0) {
        ok = false;
        return;
      }
      servers.emplace_back([&, c] {
        std::vector<char> b(size);
        for (int i = 0; i < iters && ok; ++i)
          if (!(xfer_all(a, c, b.data(), size, false) && xfer_all(a, c, b.data(), size, true))) ok = false;
        a.close_(c);
      });
    }
  });
  std::vector<double> each(conns, 0.0);
  for (int k = 0; k < conns; ++k)
    clients.emplace_back([&, k] {
      const int c = a.sock(AF_INET, SOCK_STREAM, 0);
      if (a.connect_(c, (sockaddr*)&ad, sizeof(ad))) {
        ok = false;
        ++ready;
        return;
      }
      int one = 1;
      setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::vector<char> b(size, (char)(k + 1)), e(size);
      ++ready;
      while (ready.load() < conns && ok) std::this_thread::yield();   // all connections start together
      const uint64_t t0 = ub::now_ns();
      for (int i = 0; i < iters && ok; ++i) {
        if (!(xfer_all(a, c, b.data(), size, true) && xfer_all(a, c, e.data(), size, false))) ok = false;
        if (ok && (e[0] != b[0] || e[size - 1] != b[size - 1])) ok = false;
      }
      each[k] = (ub::now_ns() - t0) / 1e3 / iters / 2;
      a.close_(c);
    });
  for (auto& t : clients) t.join();
  acceptor.join();
  for (auto& t : servers) t.join();
  a.close_(ls);
  if (!ok) return fail(name);
  double sum = 0;
  for (double v : each) sum += v;
  *lat_us = sum / conns;
  return 0;
}

// Link groups, control messages and receive moderation: 40 connections to one listener must share two link files
// (32 slots + 8), closed slots are reused, TEST LINK is answered by a peer that sleeps in recv, empty links go away
// after the linger time, and the busy-poll budget of a connection whose peer is slow comes down.
static int linkgroup_check() {
  ums_stats_t s0;
  ums_get_stats(&s0);
  const int ls = ums_socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in ad{};
  ad.sin_family = AF_INET;
  ad.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (bind(ls, (sockaddr*)&ad, sizeof(ad)) || ums_listen(ls, 64)) return fail("listen");
  socklen_t l = sizeof(ad);
  getsockname(ls, (sockaddr*)&ad, &l);
  constexpr int kConns = 40, kExtra = 10;
  std::atomic<int> slow_ms{0};
  std::vector<std::thread> workers;
  std::thread acceptor([&] {
    for (int i = 0; i < kConns + kExtra; ++i) {
      const int c = ums_accept(ls, nullptr, nullptr);
      if (c < 0) return;
      workers.emplace_back([c, &slow_ms] {   // echo until the client closes
        char b[256];
        for (;;) {
          const ssize_t r = ums_recv(c, b, sizeof(b), 0);
          if (r <= 0) break;
          if (slow_ms.load()) std::this_thread::sleep_for(std::chrono::milliseconds(slow_ms.load()));
          ums_send(c, b, r, 0);
        }
        ums_close(c);
      });
    }
  });
  auto echo = [](int fd, int tag) {
    char out[64], in[64];
    const int n = snprintf(out, sizeof(out), "conn %d says hello", tag);
    if (ums_send(fd, out, n, 0) != n) return false;
    int got = 0;
    while (got < n) {
      const ssize_t r = ums_recv(fd, in + got, n - got, 0);
      if (r <= 0) return false;
      got += (int)r;
    }
    return memcmp(in, out, n) == 0;
  };
  std::vector<int> fds;
  std::vector<ums_conn_info_t> info(kConns);
  for (int i = 0; i < kConns; ++i) {
    const int fd = ums_socket(AF_INET, SOCK_STREAM, 0);
    if (ums_connect(fd, (sockaddr*)&ad, sizeof(ad)) || ums_is_accelerated(fd) != 1) return fail("connect");
    fds.push_back(fd);
    if (ums_conn_info(fd, &info[i]) || !info[i].link[0]) return fail("connection is not on a link");
  }
  for (int i = 0; i < kConns; ++i)
    if (!echo(fds[i], i)) return fail("echo on a link slot");
  // first 32 connections on one link, slots 0..31; the rest on a second link of the group
  for (int i = 0; i < kConns; ++i) {
    const bool first = i < 32;
    if (strcmp(info[i].link, info[first ? 0 : 32].link) || info[i].slot != (uint32_t)(first ? i : i - 32))
      return fail("slot assignment");
  }
  if (!strcmp(info[0].link, info[32].link)) return fail("a 33rd connection needs a second link");
  ums_stats_t s1;
  ums_get_stats(&s1);
  // both ends live in this process: every link is mapped once per role
  if (s1.links_created - s0.links_created != 4 || s1.conns_on_links - s0.conns_on_links != 2 * kConns)
    return fail("link statistics");
  if (s1.llc_tx == s0.llc_tx || s1.llc_rx == s0.llc_rx) return fail("no control messages were exchanged");
  ums_conn_info(fds[0], &info[0]);
  if (info[0].link_state != 1 || info[0].link_conns != 32) return fail("link not ACTIVE after CONFIRM LINK");
  // TEST LINK: the peers sit in recv (asleep on their descriptors) and must still answer
  std::this_thread::sleep_for(std::chrono::milliseconds(20));
  if (ums_link_test(fds[0], 2000) || ums_link_test(fds[39], 2000)) return fail("TEST LINK was not answered");
  // closed slots are handed out again, no new link is made
  for (int i = 5; i < 5 + kExtra; ++i) ums_close(fds[i]);
  std::this_thread::sleep_for(std::chrono::milliseconds(50));   // the echo threads close their ends
  for (int i = 5; i < 5 + kExtra; ++i) {
    const int fd = ums_socket(AF_INET, SOCK_STREAM, 0);
    if (ums_connect(fd, (sockaddr*)&ad, sizeof(ad)) || ums_is_accelerated(fd) != 1) return fail("reconnect");
    ums_conn_info_t ci;
    ums_conn_info(fd, &ci);
    if (strcmp(ci.link, info[0].link) || ci.slot < 5 || ci.slot >= 5 + (uint32_t)kExtra) return fail("slot not reused");
    if (!echo(fd, 100 + i)) return fail("echo on a reused slot");
    fds[i] = fd;
  }
  ums_stats_t s2;
  ums_get_stats(&s2);
  if (s2.links_created != s1.links_created) return fail("a link was created although slots were free");
  // receive moderation: a partner that answers after 3 ms makes busy-polling pointless; the level comes down
  ums_conn_info(fds[1], &info[1]);
  const uint32_t level0 = info[1].dim_level;
  slow_ms = 3;
  for (int i = 0; i < 70; ++i)
    if (!echo(fds[1], i)) return fail("echo (slow partner)");
  slow_ms = 0;
  ums_conn_info(fds[1], &info[1]);
  ums_stats_t s3;
  ums_get_stats(&s3);
  if (!(info[1].dim_level < level0) || s3.dim_down == s2.dim_down) return fail("moderation level did not come down");
  // a partner that answers at once: polling catches the answer, nothing pushes the level further down
  const uint32_t level1 = info[1].dim_level;
  for (int i = 0; i < 200; ++i)
    if (!echo(fds[2], i)) return fail("echo (fast partner)");
  ums_conn_info(fds[2], &info[2]);
  if (info[2].dim_level < 1) return fail("moderation gave up polling although the partner is fast");
  (void)level1;
  for (int fd : fds) ums_close(fd);
  acceptor.join();
  for (auto& w : workers) w.join();
  ums_close(ls);
  // links linger for UMS_LINK_LINGER_MS after their last connection, then their files are removed
  const char* lg = getenv("UMS_LINK_LINGER_MS");
  std::this_thread::sleep_for(std::chrono::milliseconds((lg ? atoi(lg) : 1000) + 100));
  ums_stats_t s4;
  ums_get_stats(&s4);
  ums_get_stats(&s4);   // the second pass frees the accepting side's mappings of files that are now gone
  if (s4.links_active != 0 || s4.links_freed - s0.links_freed != 4) return fail("links were not freed after the linger time");
  printf("link groups: %d connections on 2 links, %llu control messages, moderation level %u -> %u: OK\n", kConns,
         (unsigned long long)(s4.llc_tx - s0.llc_tx), level0, info[1].dim_level);
  return 0;
}

int main(int argc, char** argv) {
  size_t size = 8192;
  int iters = 20000;
  bool selftest = false;
  int conns = 0;
  for (int i = 1; i < argc; ++i)
    if (!strcmp(argv[i], "--linkgroups")) return linkgroup_check();
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--selftest")) selftest = true;
    else if (!strcmp(argv[i], "--conns") && i + 1 < argc) conns = atoi(argv[++i]);
  }
  const Api ums{ums_socket, ums_listen, ums_accept, ums_connect, ums_send, ums_recv, ums_close};
  const Api tcp{socket, listen, accept, connect, send, recv, close};
  if (conns > 0) {
    double mu, mt;
    if (run_many(ums, "ums (many connections)", size, iters, conns, &mu)) return 1;
    if (run_many(tcp, "tcp (many connections)", size, iters, conns, &mt)) return 1;
    printf("size=%zu, %d connections at once: UMS one-way latency %.2f us | TCP loopback %.2f us | latency %.0f%% lower\n",
           size, conns, mu, mt, (1.0 - mu / mt) * 100.0);
    printf("ums_perftest: OK\n");
    return 0;
  }
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
