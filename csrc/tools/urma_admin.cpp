// urma_admin: inspection tool for the URMA layer.
//   urma_admin show                 devices, providers, EIDs and attributes
//   urma_admin perf <seconds>       samples the data-plane calls of a built-in loopback workload and prints the
//                                   per-call latency table (avg / min / max / p90 / p99 / p99.99)
//   urma_admin ping <dev>           round-trip of a NOP work request on <dev> (link check)
// Mirrors the `show` / `perf start|show` commands of the reference's urma_admin
// (doc/en/urma/URMA User Guide.md:1874-2010) and the EID-level reachability check of its urma_ping.
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <vector>

#include "ub_util.h"
#include "urma_simple.h"

static int show() {
  urma_init_attr_t attr{};
  urma_init(&attr);
  int n = 0;
  urma_device_t** devs = urma_get_device_list(&n);
  printf("%-8s %-8s %-42s %-6s %-8s %-10s %s\n", "name", "provider", "eid", "ports", "max_sge", "max_msg", "modes");
  for (int i = 0; i < n; ++i) {
    urma_device_attr_t a;
    char eid[64];
    urma_eid_to_str(&devs[i]->eid, eid, sizeof(eid));
    if (urma_query_device(devs[i], &a) != URMA_SUCCESS) continue;
    printf("%-8s %-8s %-42s %-6u %-8u %-10llu %s%s%s\n", devs[i]->name, devs[i]->provider, eid, a.port_cnt, a.max_sge,
           (unsigned long long)a.max_msg_size, (a.transport_modes & URMA_TM_RM) ? "RM " : "",
           (a.transport_modes & URMA_TM_RC) ? "RC " : "", (a.transport_modes & URMA_TM_UM) ? "UM" : "");
  }
  urma_free_device_list(devs);
  return n > 0 ? 0 : 1;
}

static int ping(const char* dev, int count) {
  urma_context_t* ctx = urma_simple_open(dev);
  if (!ctx) {
    fprintf(stderr, "urma_admin: no such device %s\n", dev);
    return 1;
  }
  urma_simple_ep_t* ep = urma_simple_ep_create(ctx, 16, 0, 0);
  uint8_t blob[URMA_SIMPLE_JETTY_BLOB];
  urma_simple_ep_blob(ep, blob);
  urma_target_jetty_t* self = urma_simple_ep_import(ctx, blob, 0);
  if (!ep || !self) return 1;
  int lost = 0;
  ub::PerfHist h;
  for (int i = 0; i < count; ++i) {
    const uint64_t t0 = ub::now_ns();
    int st = -1;
    uint64_t uc;
    uint32_t fl;
    if (urma_simple_post(ep, self, URMA_OPC_NOP, nullptr, 0, nullptr, 0, 0, 0, i, 1) != 0) {
      ++lost;
      continue;
    }
    const int n = urma_simple_wait(ep, 1, 3000, 1, &st, &uc, nullptr, nullptr, &fl);
    if (n != 1 || st != 0) ++lost;
    else h.add(ub::now_ns() - t0);
  }
  printf("ping %s: %d sent, %d lost, rtt avg %.2f us min %.2f us max %.2f us\n", dev, count, lost, h.mean() / 1e3,
         h.min() / 1e3, h.max() / 1e3);
  return lost ? 1 : 0;
}

static int perf(int seconds) {
  urma_context_t* ctx = urma_simple_open("shm0");
  if (!ctx) return 1;
  urma_simple_ep_t* ep = urma_simple_ep_create(ctx, 64, 0, 0);
  uint8_t blob[URMA_SIMPLE_JETTY_BLOB], sblob[URMA_SIMPLE_SEG_BLOB];
  urma_simple_ep_blob(ep, blob);
  urma_target_jetty_t* self = urma_simple_ep_import(ctx, blob, 0);
  std::vector<uint8_t> mem(8192);
  urma_target_seg_t* seg = urma_simple_seg_register(ctx, mem.data(), mem.size(), 14, 3, sblob);
  urma_target_seg_t* rseg = urma_simple_seg_import(ctx, sblob, 3);
  if (!self || !seg || !rseg) return 1;
  urma_start_perf();
  const uint64_t end = ub::now_ns() + uint64_t(seconds) * 1000000000ull;
  int st;
  uint64_t uc;
  uint32_t fl;
  while (ub::now_ns() < end) {
    urma_simple_post(ep, self, URMA_OPC_WRITE, rseg, rseg->seg.ubva.va, nullptr, (uint64_t)mem.data() + 4096, 1024, 0,
                     1, 1);
    urma_simple_wait(ep, 1, 1000, 1, &st, &uc, nullptr, nullptr, &fl);
  }
  urma_stop_perf();
  char text[4096];
  uint32_t len = sizeof(text);
  urma_get_perf_info(nullptr, text, &len);
  fputs(text, stdout);
  return 0;
}

int main(int argc, char** argv) {
  if (argc >= 2 && !strcmp(argv[1], "show")) return show();
  if (argc >= 3 && !strcmp(argv[1], "perf")) return perf(atoi(argv[2]));
  if (argc >= 3 && !strcmp(argv[1], "ping")) return ping(argv[2], argc >= 4 ? atoi(argv[3]) : 5);
  fprintf(stderr, "usage: urma_admin show | perf <seconds> | ping <dev> [count]\n");
  return 2;
}
