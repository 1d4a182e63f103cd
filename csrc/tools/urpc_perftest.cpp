// urpc_perftest: latency / call-rate measurement and self-check of the URPC framework (server thread + client in
// one process by default; `--server PORT` / `--client PORT` run the two sides as separate processes).
//   urpc_perftest [--size N] [--iters N] [--queues N] [--server-threads N] [--selftest]
// --queues N gives the channel N explicit queue pairs (calls spread over them in turn).
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#include "ub_util.h"
#include "urpc_api.h"

static int echo_fn(const void* a, uint32_t len, void* rsp, uint32_t* rlen, void*) {
  if (len > *rlen) return -1;
  memcpy(rsp, a, len);
  *rlen = len;
  return 0;
}
// Checksum of the argument bytes: 64-bit words (plus the tail bytes), so that the handler reads every byte the
// transport delivered without costing more than the transport itself.
static uint64_t word_sum(const void* a, uint32_t len) {
  uint64_t s = 0;
  const uint8_t* p = static_cast<const uint8_t*>(a);
  uint32_t i = 0;
  for (; i + 8 <= len; i += 8) {
    uint64_t w;
    memcpy(&w, p + i, 8);
    s += w;
  }
  for (; i < len; ++i) s += p[i];
  return s;
}
static int sum_fn(const void* a, uint32_t len, void* rsp, uint32_t* rlen, void*) {
  const uint64_t s = word_sum(a, len);
  memcpy(rsp, &s, 8);
  *rlen = 8;
  return 0;
}
static std::atomic<int> g_lost{0};
static void ka_cb(uint32_t, int alive, void*) {
  if (!alive) ++g_lost;
}
static int fail(const char* w) {
  fprintf(stderr, "urpc_perftest: FAILED: %s\n", w);
  return 1;
}

int main(int argc, char** argv) {
  uint32_t size = 4096, iters = 5000;
  bool selftest = false;
  int hold_ms = 0;  // keep the process (and its management socket) alive this long after the run
  int server_port = -1, client_port = -1, queues = 1, server_threads = 1;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--selftest")) selftest = true;
    else if (!strcmp(argv[i], "--queues") && i + 1 < argc) queues = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--hold-ms") && i + 1 < argc) hold_ms = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--server") && i + 1 < argc) server_port = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--client") && i + 1 < argc) client_port = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--server-threads") && i + 1 < argc) server_threads = std::max(1, atoi(argv[++i]));
  }
  urpc_config_t cfg{};
  cfg.role = URPC_ROLE_SERVER_CLIENT;
  cfg.keepalive_interval_ms = selftest ? 50 : 0;
  cfg.keepalive_miss_limit = 3;
  cfg.default_timeout_ms = 3000;
  if (urpc_init(&cfg) != URPC_SUCCESS) return fail("urpc_init");
  urpc_keepalive_callback_register(ka_cb, nullptr);
  std::atomic<bool> stop{false}, serve{true};
  std::vector<std::thread> srv;
  int port = client_port;
  if (client_port < 0) {
    urpc_func_register(1, echo_fn, nullptr);
    urpc_func_register(2, sum_fn, nullptr);
    port = urpc_server_start("127.0.0.1", server_port > 0 ? server_port : 0);
    if (port <= 0) return fail("server_start");
    // each server thread serves its share of the attached clients (session number modulo the thread count)
    for (int k = 0; k < server_threads; ++k) srv.emplace_back([&, k] {
      urpc_poll_msg_t m[8];
      while (!stop.load()) {
        if (!serve.load()) {
          usleep(1000);
          continue;
        }
        const int n = urpc_server_poll_shard((uint32_t)k, (uint32_t)server_threads, m, 8);
        for (int i = 0; i < n; ++i) {
          if (m[i].func_id == 7) {  // handled by the application: reverse the bytes
            std::vector<uint8_t> r(static_cast<uint8_t*>(m[i].data), static_cast<uint8_t*>(m[i].data) + m[i].len);
            for (size_t a = 0, b = r.size(); a + 1 < b; ++a, --b) std::swap(r[a], r[b - 1]);
            urpc_func_return(&m[i], r.data(), (uint32_t)r.size(), 0);
          }  // func 9: never answered (timeout test)
          urpc_msg_release(&m[i]);
        }
        if (n == 0) sched_yield();
      }
    });
    if (server_port > 0) {
      printf("urpc server on port %d\n", port);
      fflush(stdout);
      pause();
    }
  }
  const int ch = urpc_channel_create();
  std::vector<uint64_t> lanes;
  for (int i = 0; ch >= 0 && queues > 1 && i < queues; ++i) {
    const uint64_t q = urpc_queue_create(nullptr);
    if (!q || urpc_channel_queue_add(ch, q) != URPC_SUCCESS) return fail("queue add");
    lanes.push_back(q);
  }
  if (ch < 0 || urpc_channel_server_attach(ch, "127.0.0.1", (uint16_t)port) != URPC_SUCCESS) return fail("attach");
  std::vector<uint8_t> arg(size), rsp(size + 64);
  for (uint32_t i = 0; i < size; ++i) arg[i] = (uint8_t)(i * 7 + 1);
  urpc_sge_t sg{arg.data(), size};
  urpc_call_wr_t wr{1, &sg, 1, 0};
  uint32_t rlen = 0;
  urpc_call_option_t sync{0, 1, rsp.data(), (uint32_t)rsp.size(), &rlen};
  int rc = 0;
  // synchronous echo: latency
  uint64_t t0 = ub::now_ns();
  const uint32_t lat_iters = iters < 2000 ? iters : 2000;
  for (uint32_t i = 0; i < lat_iters; ++i) {
    arg[0] = (uint8_t)i;
    if (urpc_func_call(ch, &wr, &sync) != 0 || rlen != size || memcmp(arg.data(), rsp.data(), size)) {
      rc = fail("sync echo");
      break;
    }
  }
  const double lat_us = (ub::now_ns() - t0) / 1e3 / lat_iters;
  // pipelined asynchronous calls: rate
  t0 = ub::now_ns();
  uint32_t sent = 0, done = 0;
  urpc_poll_msg_t m[32];
  wr.func_id = 2;
  const uint64_t expect = word_sum(arg.data(), size);
  while (done < iters && rc == 0) {
    while (sent < iters && sent - done < 64) {
      wr.user_ctx = sent;
      const int r = urpc_func_call(ch, &wr, nullptr);
      if (r == URPC_ERR_EAGAIN) break;
      if (r < 0) {
        rc = fail("async call");
        break;
      }
      ++sent;
    }
    const int n = urpc_func_poll(ch, m, 32);
    for (int i = 0; i < n; ++i) {
      uint64_t s = 0;
      if (m[i].event != URPC_POLL_RSP || m[i].len != 8 || (memcpy(&s, m[i].data, 8), s != expect)) rc = fail("async rsp");
      urpc_msg_release(&m[i]);
      ++done;
    }
  }
  const double sec = (ub::now_ns() - t0) * 1e-9;
  uint64_t cnt, avg, p99;
  urpc_perf_get(&cnt, &avg, &p99);
  for (uint64_t q : lanes) {   // every lane carried its share
    uint64_t st[4] = {0, 0, 0, 0};
    if (urpc_queue_stats_get(q, st, 4) != 4 || st[0] < (iters + lat_iters) / lanes.size() - 1 || st[2] < st[0] - 1)
      rc = fail("lane share");
  }
  printf("size=%u queues=%d: sync echo %.1f us/call; async %.0f calls/s (%.1f MB/s args); call latency avg %.1f us p99 %.1f us\n",
         size, queues, lat_us, iters / sec, iters * (double)size / sec / 1e6, avg / 1e3, p99 / 1e3);
  if (selftest && rc == 0) {
    // request handled by the application through poll / return
    wr.func_id = 7;
    if (urpc_func_call(ch, &wr, &sync) != 0 || rlen != size || rsp[0] != arg[size - 1] || rsp[size - 1] != arg[0])
      rc = fail("manual return");
    // a queue pair joins the attached channel through the control plane, carries calls, and leaves again while
    // the server thread keeps polling (protocol version 2; the task engine serves both requests)
    {
      urpc_channel_cfg_t cc{};
      urpc_channel_cfg_get(ch, &cc);
      if (cc.proto_version >= 2) {
        urpc_ctl_stats_t t0{}, t1{};
        urpc_ctl_stats_get(&t0);
        const uint64_t lq = urpc_queue_create(nullptr);
        if (!lq || urpc_channel_queue_add(ch, lq) != URPC_SUCCESS) rc = fail("queue add on an attached channel");
        wr.func_id = 1;
        for (int i = 0; i < 50 && rc == 0; ++i)
          if (urpc_func_call_on(ch, lq, &wr, &sync) != 0 || rlen != size) rc = fail("call on the new lane");
        for (int i = 0; i < 8 && rc == 0; ++i) {   // calls in flight while the lane leaves
          urpc_call_option_t async_opt{2000, 0, nullptr, 0, nullptr};
          if (urpc_func_call_on(ch, lq, &wr, &async_opt) < 0) rc = fail("async call on the new lane");
        }
        if (rc == 0 && urpc_channel_queue_rm(ch, lq) != URPC_SUCCESS) rc = fail("queue remove on an attached channel");
        int answered = 0;
        for (int tries = 0; tries < 2000 && answered < 8 && rc == 0; ++tries) {
          const int n = urpc_func_poll(ch, m, 4);
          for (int i = 0; i < n; ++i) {
            answered += m[i].event == URPC_POLL_RSP;
            urpc_msg_release(&m[i]);
          }
          if (n == 0) usleep(200);
        }
        if (rc == 0 && answered != 8) rc = fail("calls in flight on a leaving lane lost their answers");
        if (lq) urpc_queue_destroy(lq);
        urpc_ctl_stats_get(&t1);
        if (rc == 0 && (t1.tasks_done - t0.tasks_done != 2 || t1.tasks_live != 0)) rc = fail("control task accounting");
        if (urpc_func_call(ch, &wr, &sync) != 0) rc = fail("call after the lane left");
      }
    }
    // a call that the server never answers times out, synchronously and asynchronously
    wr.func_id = 9;
    urpc_call_option_t quick{200, 1, rsp.data(), (uint32_t)rsp.size(), &rlen};
    if (urpc_func_call(ch, &wr, &quick) != URPC_ERR_TIMEOUT) rc = fail("sync timeout");
    urpc_call_option_t aq{200, 0, nullptr, 0, nullptr};
    if (urpc_func_call(ch, &wr, &aq) < 0) rc = fail("async call for timeout");
    bool got_timeout = false;
    for (int tries = 0; tries < 2000 && !got_timeout; ++tries) {
      const int n = urpc_func_poll(ch, m, 4);
      for (int i = 0; i < n; ++i) got_timeout |= m[i].event == URPC_POLL_TIMEOUT;
      usleep(1000);
    }
    if (!got_timeout) rc = fail("async timeout event");
    // unknown function id with nobody handling it
    urpc_stats_t st{};
    urpc_stats_get(&st);
    if (st.timeouts < 2 || st.calls < iters) rc = fail("statistics");
    // the server stops polling: keepalive probes go unanswered and the callback fires; later calls fail fast
    serve = false;
    for (int i = 0; i < 400 && g_lost.load() == 0; ++i) usleep(10000);
    if (g_lost.load() == 0) rc = fail("keepalive did not detect the silent server");
    wr.func_id = 1;
    if (urpc_func_call(ch, &wr, &sync) != URPC_ERR_SESSION_CLOSE) rc = fail("call on a lost channel must fail");
    serve = true;
  }
  if (selftest && rc == 0) {
    char rep[1024];
    if (urpc_admin_query("stats", rep, sizeof(rep)) <= 0 || !strstr(rep, "calls ") || !strstr(rep, "timeouts "))
      rc = fail("management report");
    if (urpc_admin_query("channels", rep, sizeof(rep)) <= 0 || !strstr(rep, "channel ")) rc = fail("channel report");
  }
  if (hold_ms > 0) {
    printf("urpc_perftest: holding\n");
    fflush(stdout);
    usleep(hold_ms * 1000);
  }
  urpc_channel_server_detach(ch);
  urpc_channel_destroy(ch);
  for (uint64_t q : lanes) urpc_queue_destroy(q);
  stop = true;
  for (auto& t : srv) t.join();
  urpc_uninit();
  if (rc == 0) printf("urpc_perftest: OK\n");
  return rc;
}
