// umq_perftest: latency / message-rate test and self-check of the UMQ layer between two queues of one process (or
// of two threads), in the spirit of the reference's src/urpc/tools/perftest umq_perftest.
//   umq_perftest [--size N] [--iters N] [--flow-control] [--pro] [--selftest]
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <thread>

#include "ub_util.h"
#include "umq_api.h"

static int fail(const char* what) {
  fprintf(stderr, "umq_perftest: FAILED: %s\n", what);
  return 1;
}

int main(int argc, char** argv) {
  uint32_t size = 4096, iters = 20000;
  bool fc = false, pro = false, selftest = false;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--flow-control")) fc = true;
    else if (!strcmp(argv[i], "--pro")) pro = true;
    else if (!strcmp(argv[i], "--selftest")) selftest = true;
  }
  umq_init_cfg_t cfg{};
  cfg.feature = UMQ_FEATURE_API_BASE | UMQ_FEATURE_API_PRO | UMQ_FEATURE_STATS | UMQ_FEATURE_PERF |
                (fc ? UMQ_FEATURE_FLOW_CONTROL : 0);
  cfg.block_size_kb = 8;
  if (umq_init(&cfg) != UMQ_SUCCESS) return fail("umq_init");
  umq_create_option_t o{};
  snprintf(o.name, sizeof(o.name), "a");
  o.rx_depth = 64;
  o.tx_depth = 64;
  o.token = 5;
  if (size > 8192) o.rx_buf_size = o.tx_buf_size = size;  // receive buffers must hold a whole message
  const uint64_t a = umq_create(&o);
  snprintf(o.name, sizeof(o.name), "b");
  const uint64_t b = umq_create(&o);
  if (!a || !b) return fail("umq_create");
  uint8_t ia[UMQ_BIND_INFO_SIZE], ib[UMQ_BIND_INFO_SIZE];
  const uint32_t la = umq_bind_info_get(a, ia, sizeof(ia)), lb = umq_bind_info_get(b, ib, sizeof(ib));
  if (!la || !lb) return fail("bind_info_get");
  if (umq_bind(a, ib, lb) || umq_bind(b, ia, la)) return fail("umq_bind");
  if (umq_state_get(a) != UMQ_STATE_READY) return fail("state after bind");
  umq_stats_perf_start();

  // receiver thread echoes a checksum back every message when self-testing
  std::atomic<uint64_t> received{0}, bad_payload{0};
  std::atomic<bool> stop{false};
  std::thread rx([&] {
    while (!stop.load()) {
      umq_buf_t* m = pro ? nullptr : umq_dequeue(b);
      if (pro) {
        umq_buf_t* v[16];
        const int n = umq_poll(b, UMQ_IO_RX, v, 16);
        for (int i = 0; i < n; ++i) {
          if (v[i]->data_size != size) ++bad_payload;
          else if (size >= 8 && memcmp(v[i]->buf_data + 4, "umq!", 4) != 0) ++bad_payload;
          umq_buf_free(v[i]);
          ++received;
        }
        if (n == 0) sched_yield();
        continue;
      }
      if (!m) {
        sched_yield();
        continue;
      }
      if (m->data_size != size) ++bad_payload;
      else if (size >= 8 && memcmp(m->buf_data + 4, "umq!", 4) != 0) ++bad_payload;
      umq_buf_free(m);
      ++received;
    }
  });

  const uint64_t t0 = ub::now_ns();
  uint64_t eagain = 0;
  for (uint32_t i = 0; i < iters; ++i) {
    umq_buf_t* m = umq_buf_alloc(size, 1, a);
    if (!m) {  // pool exhausted because the receiver lags: wait for it
      --i;
      sched_yield();
      if (pro) {
        umq_buf_t* d[16];
        const int n = umq_poll(a, UMQ_IO_TX, d, 16);
        for (int k = 0; k < n; ++k) umq_buf_free(d[k]);
      }
      continue;
    }
    if (size >= 8) {
      memcpy(m->buf_data, &i, 4);
      memcpy(m->buf_data + 4, "umq!", 4);
    }
    umq_buf_t* bad = nullptr;
    int rc;
    for (;;) {
      rc = pro ? umq_post(a, m, UMQ_IO_TX, &bad) : umq_enqueue(a, m, &bad);
      if (rc != UMQ_ERR_EAGAIN) break;
      ++eagain;
      sched_yield();
      if (pro) {
        umq_buf_t* d[16];
        const int n = umq_poll(a, UMQ_IO_TX, d, 16);
        for (int k = 0; k < n; ++k) umq_buf_free(d[k]);
      } else {
        umq_buf_t* none = umq_dequeue(a);
        if (none) umq_buf_free(none);
      }
    }
    if (rc != UMQ_SUCCESS) {
      stop = true;
      rx.join();
      return fail("send");
    }
    if (pro) {
      umq_buf_t* d[16];
      const int n = umq_poll(a, UMQ_IO_TX, d, 16);
      for (int k = 0; k < n; ++k) umq_buf_free(d[k]);
    }
  }
  const uint64_t deadline = ub::now_ns() + 20000000000ull;
  while (received.load() < iters && ub::now_ns() < deadline) {
    if (pro) {
      umq_buf_t* d[16];
      const int n = umq_poll(a, UMQ_IO_TX, d, 16);
      for (int k = 0; k < n; ++k) umq_buf_free(d[k]);
    } else {
      umq_buf_t* none = umq_dequeue(a);  // drives completions and credit returns on the sender
      if (none) umq_buf_free(none);
    }
    sched_yield();
  }
  const double sec = (ub::now_ns() - t0) * 1e-9;
  stop = true;
  rx.join();
  umq_io_stats_t ioa{}, iob{};
  umq_fc_stats_t fca{};
  umq_qbuf_stats_t qs{};
  umq_stats_io_get(a, &ioa);
  umq_stats_io_get(b, &iob);
  umq_stats_flow_control_get(a, &fca);
  umq_stats_qbuf_pool_get(&qs);
  umq_perf_entry_t pe[UMQ_PERF_RECORD_MAX];
  umq_stats_perf_get(pe);
  char info[512];
  umq_info_to_str(a, info, sizeof(info));
  printf("%s\n", info);
  printf("size=%u iters=%u api=%s fc=%d: %.0f msg/s, %.2f MB/s, eagain=%llu, credits granted=%llu stalls=%llu\n", size,
         iters, pro ? "pro" : "base", (int)fc, iters / sec, iters * (double)size / sec / 1e6,
         (unsigned long long)eagain, (unsigned long long)fca.credits_granted, (unsigned long long)fca.stalls);
  printf("enqueue/post avg %llu ns p99 %llu ns; pool blocks %llu free %llu\n",
         (unsigned long long)pe[pro ? UMQ_PERF_POST_TX : UMQ_PERF_ENQUEUE].avg_ns,
         (unsigned long long)pe[pro ? UMQ_PERF_POST_TX : UMQ_PERF_ENQUEUE].p99_ns, (unsigned long long)qs.blocks_total,
         (unsigned long long)qs.blocks_free);
  int rc = 0;
  if (received.load() != iters) rc = fail("not every message arrived");
  if (bad_payload.load()) rc = fail("payload corrupted");
  if (ioa.tx_msgs != iters || iob.rx_msgs != iters) rc = fail("io statistics disagree with the message count");
  if (fc && fca.credits_granted == 0 && iters > 64) rc = fail("flow control never returned credits");
  if (selftest) {
    // huge buffer path and headroom handling
    umq_buf_t* h = umq_buf_alloc(1u << 20, 1, a);
    if (!h || h->buf_size < (1u << 20)) rc = fail("huge buffer");
    if (h && (umq_buf_headroom_reset(h, 64) != UMQ_SUCCESS || h->headroom_size != 64)) rc = fail("headroom");
    if (h) umq_buf_free(h);
    if (umq_buf_alloc(UMQ_MAX_MSG_SIZE + 1, 1, a) != nullptr) rc = fail("oversized request must be refused");
    if (umq_unbind(a) != UMQ_SUCCESS || umq_state_get(a) != UMQ_STATE_IDLE) rc = fail("unbind");
    // main / sub queues over the jetty pool, with one message large enough to be pulled by the receiver
    {
      umq_create_option_t mo{};
      snprintf(mo.name, sizeof(mo.name), "main");
      mo.rx_depth = mo.tx_depth = 64;
      mo.create_flag = UMQ_CREATE_FLAG_MAIN | UMQ_CREATE_FLAG_SHARE_TRANSPORT;
      const uint64_t ma = umq_create(&mo), mb = umq_create(&mo);
      uint8_t info[UMQ_BIND_INFO_SIZE];
      uint64_t sa[4], sb[4];
      bool ok = ma && mb;
      for (int i = 0; i < 4 && ok; ++i) {
        umq_create_option_t so{};
        snprintf(so.name, sizeof(so.name), "sub%d", i);
        so.rx_depth = so.tx_depth = 8;
        so.create_flag = UMQ_CREATE_FLAG_SUB;
        so.share_rq_umqh = ma;
        sa[i] = umq_create(&so);
        so.share_rq_umqh = mb;
        sb[i] = umq_create(&so);
        ok = sa[i] && sb[i];
        uint32_t n = ok ? umq_bind_info_get(sb[i], info, sizeof(info)) : 0;
        ok = ok && n && umq_bind(sa[i], info, n) == UMQ_SUCCESS;
        n = ok ? umq_bind_info_get(sa[i], info, sizeof(info)) : 0;
        ok = ok && n && umq_bind(sb[i], info, n) == UMQ_SUCCESS;
      }
      auto xfer = [&](uint64_t from, uint64_t to, uint32_t bytes, char fill) {
        umq_buf_t* b = umq_buf_alloc(bytes, 1, from);
        if (!b) return false;
        memset(b->buf_data, fill, bytes);
        b->data_size = b->total_data_size = bytes;
        umq_buf_t* bad = nullptr;
        for (int tries = 0; umq_enqueue(from, b, &bad) != UMQ_SUCCESS; ++tries) {
          if (tries > 100000) return false;
          sched_yield();
        }
        for (int tries = 0; tries < 2000000; ++tries) {
          umq_buf_t* r = umq_dequeue(to);
          if (r) {
            const bool good = r->data_size == bytes && r->buf_data[0] == fill && r->buf_data[bytes - 1] == fill;
            umq_buf_free(r);
            umq_dequeue(from);   // lets the sender see its completion
            return good;
          }
          umq_dequeue(from);
        }
        return false;
      };
      for (int round = 0; round < 20 && ok; ++round)
        for (int i = 0; i < 4 && ok; ++i) ok = xfer(sa[i], sb[i], 300 + round, 'a' + i) && xfer(sb[i], sa[i], 700, 'A' + i);
      {   // two threads on different sub-queue pairs of the same main queues at the same time
        std::atomic<bool> tok{true};
        auto pump = [&](int i) {
          for (int round = 0; round < 150 && tok; ++round)
            if (!(xfer(sa[i], sb[i], 1000 + round, 'x') && xfer(sb[i], sa[i], 64, 'y'))) tok = false;
        };
        std::thread t1(pump, 0), t2(pump, 1);
        t1.join();
        t2.join();
        ok = ok && tok;
      }
      ok = ok && xfer(sa[2], sb[2], 200000, 'P');   // beyond the receive buffer size: descriptor + read
      umq_io_stats_t ps{};
      if (ok) umq_stats_io_get(sb[2], &ps);
      umq_jetty_pool_stats_t jp{};
      umq_jetty_pool_stats_get(&jp);
      if (!ok || ps.pull_rx != 1 || jp.total_num != 2 || jp.sub_queues != 8 || jp.acc_alloc_num < 700)
        rc = fail("sub queues / jetty pool / pulled message");
      if (umq_destroy(ma) == UMQ_SUCCESS) rc = fail("a main queue must outlive its sub queues");
      for (int i = 0; i < 4; ++i) {
        if (sa[i]) umq_destroy(sa[i]);
        if (sb[i]) umq_destroy(sb[i]);
      }
      if (ma) umq_destroy(ma);
      if (mb) umq_destroy(mb);
    }
  }
  umq_destroy(a);
  umq_destroy(b);
  umq_uninit();
  if (rc == 0) printf("umq_perftest: OK\n");
  return rc;
}
