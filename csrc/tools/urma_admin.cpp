// urma_admin: inspection tool for the URMA layer.
//   urma_admin show                 devices, providers, EIDs and attributes
//   urma_admin perf <seconds>       samples the data-plane calls of a built-in loopback workload and prints the
//                                   per-call latency table (avg / min / max / p90 / p99 / p99.99)
//   urma_admin ping <dev>           round-trip of a NOP work request on <dev> (link check)
//   urma_admin agg [name]           members of an aggregation device (default bond0)
//   urma_admin topo                 discovered topology: nodes, ports, and the path set between the first two nodes
//   urma_admin stats <bond-dev> [seconds]   per-path state and counters of a multipath device while a loopback
//                                   workload runs on it (up, sent, errors, failovers, failbacks, admin state)
//   urma_admin eid add <dev> <eid> [index] | eid del <dev> <index> | eid show [dev] | eid mode <dev> static|dynamic
//                                   extra EIDs of a device (indexes 1..8; contexts are created on them with
//                                   urma_create_context(dev, index)) and how indexes are handed out
//   urma_admin ns mode exclusive|shared     device visibility between namespaces (a system-wide setting)
//   urma_admin sharing <dev> on|off         whether several processes may open the device at the same time
//   urma_admin system show                  the system-wide settings and every device record
// The eid / ns / sharing commands are sent to the library as TLV messages (urma_cmd_tlv.h), the form the reference's
// tool uses towards its kernel core (admin_cmd_eid.c, admin_cmd_system.c).
// Mirrors the `show` / `perf start|show` commands of the reference's urma_admin
// (doc/en/urma/URMA User Guide.md:1874-2010) and the EID-level reachability check of its urma_ping.
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "ub_util.h"
#include "urma_cmd_tlv.h"
#include "urma_simple.h"
#include "uvs_topo.h"

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

static int agg(const char* name) {
  urma_init_attr_t attr{};
  urma_init(&attr);
  uvs_agg_dev_t d;
  if (uvs_get_agg_dev(name, &d) != 0) {
    // nothing registered under this name: a multipath device then takes $BOND_DEVICES or every shm* device
    urma_device_t* dev = urma_get_device_by_name(name);
    if (!dev) {
      fprintf(stderr, "urma_admin: no aggregation device %s\n", name);
      return 1;
    }
    const char* env = getenv("BOND_DEVICES");
    printf("%s: not in the aggregation registry; members = %s\n", name, env ? env : "every shm* device");
    return 0;
  }
  char eid[64];
  urma_eid_to_str(&d.agg_eid, eid, sizeof(eid));
  printf("%s eid %s members %u\n", d.name, eid, d.member_num);
  for (uint32_t i = 0; i < d.member_num; ++i) {
    urma_eid_to_str(&d.member_eids[i], eid, sizeof(eid));
    printf("  member %u: %-8s %s\n", i, d.member_names[i], eid);
  }
  return 0;
}

static int topo() {
  urma_init_attr_t attr{};
  urma_init(&attr);
  if (uvs_discover_local_topology() <= 0) {
    fprintf(stderr, "urma_admin: topology discovery failed\n");
    return 1;
  }
  std::vector<uvs_topo_node_t> nodes(UVS_MAX_NODES);
  uint32_t n = 0;
  if (uvs_get_topo_info(nodes.data(), UVS_MAX_NODES, &n) != 0) return 1;
  printf("%u node(s)\n", n);
  for (uint32_t i = 0; i < n; ++i) {
    char eid[64];
    urma_eid_to_str(&nodes[i].primary_eid, eid, sizeof(eid));
    printf("  node %u: %s, %u port(s), eid %s%s\n", nodes[i].node_id,
           nodes[i].type == UVS_TOPO_CLOS_PLANES ? "switch planes" : "full mesh", nodes[i].port_num, eid,
           nodes[i].is_current ? " (this process)" : "");
  }
  if (n >= 2) {
    uvs_path_set_t ps;
    if (uvs_get_path_set(&nodes[0].primary_eid, &nodes[1].primary_eid, UVS_RTP, &ps) == 0) {
      printf("paths node %u -> node %u: %u\n", nodes[0].node_id, nodes[1].node_id, ps.path_count);
      for (uint32_t i = 0; i < ps.path_count && i < 4; ++i)
        printf("  port %u -> port %u\n", ps.paths[i].src_port, ps.paths[i].dst_port);
      if (ps.path_count > 4) printf("  ...\n");
    }
  }
  return 0;
}

static int stats(const char* dev, int seconds) {
  urma_context_t* ctx = urma_simple_open(dev);
  if (!ctx) {
    fprintf(stderr, "urma_admin: no such device %s\n", dev);
    return 1;
  }
  urma_simple_ep_t* ep = urma_simple_ep_create(ctx, 64, 0, 0);
  uint8_t blob[URMA_SIMPLE_JETTY_BLOB], sblob[URMA_SIMPLE_SEG_BLOB];
  std::vector<uint8_t> mem(8192);
  urma_target_seg_t* seg = ep ? urma_simple_seg_register(ctx, mem.data(), mem.size(), 14, 5, sblob) : nullptr;
  if (!ep || !seg) return 1;
  urma_simple_ep_blob(ep, blob);
  urma_target_jetty_t* self = urma_simple_ep_import(ctx, blob, 0);
  urma_target_seg_t* rseg = urma_simple_seg_import(ctx, sblob, 5);
  if (!self || !rseg) return 1;
  const uint64_t end = ub::now_ns() + uint64_t(seconds) * 1000000000ull;
  int st;
  uint64_t uc;
  uint32_t fl;
  uint64_t ops = 0;
  do {
    urma_simple_post(ep, self, URMA_OPC_WRITE, rseg, rseg->seg.ubva.va, nullptr, (uint64_t)mem.data() + 4096, 512, 0, 1,
                     1);
    urma_simple_wait(ep, 1, 1000, 1, &st, &uc, nullptr, nullptr, &fl);
    ++ops;
  } while (ub::now_ns() < end);
  uint64_t table[UVS_MAX_MEMBERS * 4][6];
  urma_user_ctl_in_t in{0, 0, 1};
  urma_user_ctl_out_t out{reinterpret_cast<uint64_t>(table), (uint32_t)sizeof(table), 0};
  if (urma_user_ctl(ctx, &in, &out) != 0) {
    fprintf(stderr, "urma_admin: %s has no path statistics (not a multipath device)\n", dev);
    return 1;
  }
  printf("%s: %llu loopback writes, %u path(s)\n", dev, (unsigned long long)ops, out.rsv);
  printf("%-5s %-5s %-10s %-8s %-10s %-10s %s\n", "path", "up", "sent", "errors", "failovers", "failbacks", "admin");
  for (uint32_t i = 0; i < out.rsv; ++i)
    printf("%-5u %-5llu %-10llu %-8llu %-10llu %-10llu %s\n", i, (unsigned long long)table[i][0],
           (unsigned long long)table[i][1], (unsigned long long)table[i][2], (unsigned long long)table[i][3],
           (unsigned long long)table[i][4], table[i][5] ? "down" : "up");
  return 0;
}

extern "C" int urma_admin_cmd_exec(const uint8_t* cmd, uint32_t len, uint8_t* out, uint32_t* out_len);

static int run_tlv(const urma_tlv::Encoder& enc) {
  urma_init_attr_t attr{};
  urma_init(&attr);
  const std::vector<uint8_t> cmd = enc.finish();
  std::vector<uint8_t> out(1 << 16);
  uint32_t n = static_cast<uint32_t>(out.size());
  if (urma_admin_cmd_exec(cmd.data(), static_cast<uint32_t>(cmd.size()), out.data(), &n) != 0) {
    fprintf(stderr, "urma_admin: command rejected\n");
    return 1;
  }
  urma_tlv::Decoder d;
  int32_t status = -1;
  std::string text;
  if (!d.parse(out.data(), n) || !d.get_i32(urma_tlv::ATTR_STATUS, &status)) return 1;
  d.get_str(urma_tlv::ATTR_TEXT, &text);
  if (!text.empty()) fprintf(status == 0 ? stdout : stderr, "%s%s", text.c_str(), text.back() == '\n' ? "" : "\n");
  return status == 0 ? 0 : 1;
}

static int admin_settings(int argc, char** argv) {
  using namespace urma_tlv;
  const std::string a = argv[1], b = argc >= 3 ? argv[2] : "";
  if (a == "eid" && b == "add" && argc >= 5) {
    urma_eid_t eid;
    if (urma_str_to_eid(argv[4], &eid) != 0) {
      fprintf(stderr, "urma_admin: bad EID %s\n", argv[4]);
      return 2;
    }
    struct stat sb{};
    uint64_t ns = stat("/proc/self/ns/net", &sb) == 0 ? (uint64_t)sb.st_ino : 0;
    Encoder e(CMD_EID_ADD);
    e.put_str(ATTR_DEV_NAME, argv[3]).put_bytes(ATTR_EID, eid.raw, 16).put_u64(ATTR_NS, ns);
    if (argc >= 6) e.put_u32(ATTR_EID_INDEX, (uint32_t)atoi(argv[5]));
    return run_tlv(e);
  }
  if (a == "eid" && b == "del" && argc >= 5)
    return run_tlv(Encoder(CMD_EID_DEL).put_str(ATTR_DEV_NAME, argv[3]).put_u32(ATTR_EID_INDEX, (uint32_t)atoi(argv[4])));
  if (a == "eid" && b == "show") {
    Encoder e(CMD_EID_SHOW);
    if (argc >= 4) e.put_str(ATTR_DEV_NAME, argv[3]);
    return run_tlv(e);
  }
  if (a == "eid" && b == "mode" && argc >= 5)
    return run_tlv(Encoder(CMD_EID_MODE).put_str(ATTR_DEV_NAME, argv[3]).put_u32(ATTR_FLAG, !strcmp(argv[4], "dynamic")));
  if (a == "ns" && b == "mode" && argc >= 4)
    return run_tlv(Encoder(CMD_NS_MODE).put_u32(ATTR_FLAG, !strcmp(argv[3], "shared")));
  if (a == "sharing" && argc >= 4)
    return run_tlv(Encoder(CMD_SHARING).put_str(ATTR_DEV_NAME, argv[2]).put_u32(ATTR_FLAG, !strcmp(argv[3], "on")));
  if (a == "system" && b == "show") return run_tlv(Encoder(CMD_SYSTEM_SHOW));
  return -1;
}

int main(int argc, char** argv) {
  if (argc >= 2 && (!strcmp(argv[1], "eid") || !strcmp(argv[1], "ns") || !strcmp(argv[1], "sharing") ||
                    !strcmp(argv[1], "system"))) {
    const int rc = admin_settings(argc, argv);
    if (rc >= 0) return rc;
  }
  if (argc >= 2 && !strcmp(argv[1], "show")) return show();
  if (argc >= 3 && !strcmp(argv[1], "perf")) return perf(atoi(argv[2]));
  if (argc >= 3 && !strcmp(argv[1], "ping")) return ping(argv[2], argc >= 4 ? atoi(argv[3]) : 5);
  if (argc >= 2 && !strcmp(argv[1], "agg")) return agg(argc >= 3 ? argv[2] : "bond0");
  if (argc >= 2 && !strcmp(argv[1], "topo")) return topo();
  if (argc >= 3 && !strcmp(argv[1], "stats")) return stats(argv[2], argc >= 4 ? atoi(argv[3]) : 0);
  fprintf(stderr, "usage: urma_admin show | perf <seconds> | ping <dev> [count] | agg [name] | topo | "
                  "stats <bond-dev> [seconds] | eid add|del|show|mode ... | ns mode exclusive|shared | "
                  "sharing <dev> on|off | system show\n");
  return 2;
}
