// "bond" URMA provider: one virtual device ("bond0") aggregated over several physical devices of another provider.
// Every virtual object (context, completion queue, jetty, segment, imported target) owns one physical object per
// path; work requests are scheduled onto a path, remembered until their completion arrives, and re-sent on another
// path when the first one fails; receives are de-duplicated with a message sequence number and a sliding window; a
// health thread probes failed paths and brings them back (failback).
//
// Behaviour taken from the reference's multipath provider (src/urma/lib/urma/bond/): aggregation modes
// STANDALONE / ACTIVE_BACKUP / BALANCE (bondp_types.h:103-260), path scheduling (bondp_datapath_schedule.c:44-215),
// store-and-resend of work requests (bondp_wr_buf.h:129-166, bondp_datapath.c:1274-1372), MSN + sliding window
// (utils/bondp_slide_window.h:36-49), periodic health probes (bondp_dp_health.c:249-423, default 1000 ms) and failback
// (bondp_dp_failback.c:249-483), switches BOND_ENABLE_FAILOVER / BOND_ENABLE_FAILBACK / BOND_ENABLE_HEALTH_CHECK /
// BOND_HEALTH_CHECK_ACTIVE_INTERVAL (bondp_env.c:18-24). Like the reference, only Jetty objects are supported on
// the bond device (no stand-alone JFS / JFR, no event channel).
//
// Path scheduling in BALANCE mode follows one of five policies (BOND_SCHED_POLICY or user_ctl 5; the reference's
// priority / chip-affinity / least-load / random selection, bondp_datapath_schedule.c:44-215, 236-259):
//   round_robin  paths in turn (default)
//   priority     the first usable path of an ordered list (BOND_PATH_PRIORITY="2,0,1", user_ctl 6)
//   affinity     the path that belongs to the calling thread's CPU (cpu % npaths, the stand-in for the chip a
//                thread runs on), then the priority list as the failover route
//   least_load   the usable path with the fewest work requests in flight, ties broken at random
//   random       any usable path, uniformly
// A work request whose path failed is not resent at once: the resend is put on a timing wheel (bond_timewheel.h,
// BOND_RESEND_DELAY_MS, default one tick of 5 ms) so that a burst of failures does not pile onto the surviving paths
// while their own completions are still draining, and failback probes are wheel tasks too. The wheel is advanced by
// the context's timer thread (the health thread of the earlier design).
#include <fcntl.h>
#include <sched.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "bond_timewheel.h"
#include "bond_window.h"
#include "ub_util.h"
#include "urma_api.h"
#include "urma_provider.h"
#include "uvs_topo.h"

namespace {

constexpr int kMaxPaths = 4;
constexpr uint32_t kRegEntries = 8192;
constexpr uint32_t kBondMagic = 0x424f4e44;  // "BOND"
enum BondMode { MODE_STANDALONE = 0, MODE_ACTIVE_BACKUP = 1, MODE_BALANCE = 2 };
enum BondPolicy { POL_ROUND_ROBIN = 0, POL_PRIORITY = 1, POL_AFFINITY = 2, POL_LEAST_LOAD = 3, POL_RANDOM = 4, POL_LAST = 4 };
enum RegType : uint32_t { REG_FREE = 0, REG_BUSY = 1, REG_JETTY = 2, REG_SEG = 3 };

struct RegEntry {
  std::atomic<uint32_t> type;
  uint32_t v_uasid, v_id, npaths;
  uint32_t p_uasid[kMaxPaths], p_id[kMaxPaths];
  uint64_t va, len;
  uint32_t attr, pad;
};
struct BondReg {
  std::atomic<uint32_t> magic, next_uasid, next_id, pad;
  RegEntry e[kRegEntries];
};

struct BondHdr {  // prepended to every two-sided message
  uint32_t magic, src_uasid, src_jetty, msn;
};

bool env_on(const char* name, bool dflt) {
  const char* e = getenv(name);
  if (!e || !*e) return dflt;
  return !(e[0] == '0' || e[0] == 'f' || e[0] == 'F' || e[0] == 'n' || e[0] == 'N');
}

struct BondDev {
  urma_eid_t eid;
  BondReg* reg = nullptr;
  std::vector<std::string> phys;
};
BondDev g_dev;

struct BondCtx;
struct BJfc {
  urma_jfc_t pub;
  urma_jfc_t* p[kMaxPaths] = {nullptr};
  int next_poll = 0;
  std::deque<urma_cr_t> ready;  // completions produced while handling another one
  std::mutex mu;
};
struct StoredWr {
  urma_jfs_wr_t wr;
  std::vector<urma_sge_t> sg_a, sg_b;  // deep copies (src / dst or send payload)
  urma_sge_t cas_dst, cas_src;
  BondHdr hdr;
  uint64_t user_ctx;
  uint32_t flag;
  int path;
  int tries;
  struct BJetty* jetty;
  struct BTarget* target;
};
struct BJetty {
  urma_jetty_t pub;
  urma_jetty_t* p[kMaxPaths] = {nullptr};
  BJfc *sjfc, *rjfc;
  uint32_t v_id;
  std::atomic<uint32_t> msn{1};
  std::mutex mu;
  std::unordered_map<uint64_t, bond::SlideWindow> windows;       // (src uasid, src jetty) -> seen MSNs
  // Receives: every path keeps internal bounce buffers posted; an arriving message is copied into the next
  // application receive (or parked until one is posted), so a sender may use any path at any time.
  std::vector<std::vector<uint8_t>> bounce[kMaxPaths];
  struct VRecv {
    std::vector<urma_sge_t> sges;
    uint64_t user_ctx;
  };
  struct VMsg {
    std::vector<uint8_t> data;
    uint64_t imm;
    urma_cr_opcode_t opc;
    uint32_t src_uasid, src_jetty;
  };
  std::deque<VRecv> v_posted;
  std::deque<VMsg> v_unexp;
  uint32_t recv_depth = 0;
};
constexpr uint32_t kBounceBytes = 16384 + sizeof(BondHdr);  // largest two-sided message on the bond device: 16 KiB
struct BTarget {
  urma_target_jetty_t pub;
  urma_target_jetty_t* p[kMaxPaths] = {nullptr};
};
struct BSeg {
  urma_target_seg_t pub;
  urma_target_seg_t* p[kMaxPaths] = {nullptr};
};
struct PathState {
  std::atomic<bool> up{true};
  std::atomic<bool> admin_down{false};
  std::atomic<uint64_t> tx{0}, errors{0}, failovers{0}, failbacks{0};
  std::atomic<int64_t> inflight{0};   // work requests posted on this path whose completion has not been seen
  urma_jfc_t* probe_jfc = nullptr;
  urma_jetty_t* probe_jetty = nullptr;
  urma_target_jetty_t* probe_self = nullptr;
};
struct BondCtx {
  urma_context_t pub;
  int npaths = 0;
  urma_context_t* p[kMaxPaths] = {nullptr};
  PathState path[kMaxPaths];
  int mode = MODE_BALANCE;
  std::atomic<int> policy{POL_ROUND_ROBIN};
  int priority[kMaxPaths] = {0, 1, 2, 3};   // path numbers, most preferred first
  bool failover = true, failback = true, health = true;
  uint32_t health_ms = 1000;
  uint32_t resend_delay_ms = 5;
  bond::TimeWheel wheel{5, 256};
  std::atomic<uint64_t> deferred_resends{0};
  std::atomic<uint32_t> rr{0};
  std::mutex mu;
  std::unordered_map<uint64_t, StoredWr*> store;
  std::atomic<uint64_t> next_wr{1};
  std::thread health_thr;
  std::atomic<bool> stop{false};
  std::mutex hmu;
  std::condition_variable hcv;
};
BondCtx* C(urma_context_t* c) { return reinterpret_cast<BondCtx*>(c->priv); }

// ------------------------------------------------------------------------------------------- registry
RegEntry* reg_find(uint32_t type, uint32_t uasid, uint32_t id) {
  uint32_t h = ub::hash_u64((uint64_t(uasid) << 32) | id) & (kRegEntries - 1);
  for (uint32_t i = 0; i < kRegEntries; ++i) {
    RegEntry& e = g_dev.reg->e[(h + i) & (kRegEntries - 1)];
    const uint32_t t = e.type.load(std::memory_order_acquire);
    if (t == REG_FREE) return nullptr;
    if (t == type && e.v_uasid == uasid && e.v_id == id) return &e;
  }
  return nullptr;
}
RegEntry* reg_claim(uint32_t uasid, uint32_t id) {
  uint32_t h = ub::hash_u64((uint64_t(uasid) << 32) | id) & (kRegEntries - 1);
  for (uint32_t i = 0; i < kRegEntries; ++i) {
    RegEntry& e = g_dev.reg->e[(h + i) & (kRegEntries - 1)];
    uint32_t exp = REG_FREE;
    if (e.type.compare_exchange_strong(exp, REG_BUSY)) return &e;
  }
  return nullptr;
}
void reg_release(uint32_t type, uint32_t uasid, uint32_t id) {
  // tombstone: keep the probe chain intact by leaving the slot busy with an impossible key
  if (RegEntry* e = reg_find(type, uasid, id)) {
    e->v_uasid = 0;
    e->v_id = 0;
    e->type.store(REG_BUSY, std::memory_order_release);
  }
}

// ------------------------------------------------------------------------------------------- scheduling
bool path_usable(BondCtx* c, int i) { return c->path[i].up.load() && !c->path[i].admin_down.load(); }
int pick_path(BondCtx* c, int avoid = -1) {
  if (c->mode == MODE_STANDALONE) return path_usable(c, 0) && avoid != 0 ? 0 : -1;
  if (c->mode == MODE_ACTIVE_BACKUP) {
    for (int i = 0; i < c->npaths; ++i)
      if (i != avoid && path_usable(c, i)) return i;
    return -1;
  }
  auto first_of_priority = [&]() {
    for (int k = 0; k < c->npaths; ++k) {
      const int i = c->priority[k];
      if (i >= 0 && i < c->npaths && i != avoid && path_usable(c, i)) return i;
    }
    return -1;
  };
  static thread_local uint64_t rng = ub::now_ns() ^ (uint64_t)(uintptr_t)&rng;
  auto next_rand = [&]() {
    rng ^= rng << 13;
    rng ^= rng >> 7;
    rng ^= rng << 17;
    return rng;
  };
  switch (c->policy.load()) {
    case POL_PRIORITY: return first_of_priority();
    case POL_AFFINITY: {
      const int cpu = sched_getcpu();
      const int i = cpu >= 0 ? cpu % c->npaths : 0;
      if (i != avoid && path_usable(c, i)) return i;
      return first_of_priority();   // the failover route
    }
    case POL_LEAST_LOAD: {
      int cand[kMaxPaths], n = 0;
      int64_t best = INT64_MAX;
      for (int i = 0; i < c->npaths; ++i) {
        if (i == avoid || !path_usable(c, i)) continue;
        const int64_t v = c->path[i].inflight.load();
        if (v < best) {
          best = v;
          n = 0;
        }
        if (v == best) cand[n++] = i;
      }
      return n == 0 ? -1 : cand[next_rand() % n];
    }
    case POL_RANDOM: {
      int cand[kMaxPaths], n = 0;
      for (int i = 0; i < c->npaths; ++i)
        if (i != avoid && path_usable(c, i)) cand[n++] = i;
      return n == 0 ? -1 : cand[next_rand() % n];
    }
    default: break;
  }
  const uint32_t start = c->rr.fetch_add(1);
  for (int k = 0; k < c->npaths; ++k) {
    const int i = (start + k) % c->npaths;
    if (i != avoid && path_usable(c, i)) return i;
  }
  return -1;
}

void mark_down(BondCtx* c, int path) {
  if (c->path[path].up.exchange(false)) {
    urma_log(URMA_VLOG_LEVEL_WARNING, __func__, __LINE__, "bond: path %d marked down", path);
    c->hcv.notify_all();
  }
}

// posts the stored WR on its current path; returns URMA status
urma_status_t post_stored(BondCtx* c, StoredWr* s, uint64_t id) {
  urma_jfs_wr_t w = s->wr;
  const int p = s->path;
  w.tjetty = s->target->p[p];
  w.user_ctx = id;
  w.flag = s->flag | URMA_WR_FLAG_COMPLETE_ENABLE;  // the bond layer needs every completion to free its copy
  std::vector<urma_sge_t> a = s->sg_a, b = s->sg_b;
  auto xlate = [&](std::vector<urma_sge_t>& v, bool remote) {
    for (auto& g : v)
      if (g.tseg && remote) g.tseg = reinterpret_cast<BSeg*>(g.tseg->priv)->p[p];
      else if (g.tseg) g.tseg = nullptr;
  };
  urma_sge_t cd = s->cas_dst, cs = s->cas_src;
  switch (w.opcode) {
    case URMA_OPC_WRITE:
    case URMA_OPC_WRITE_IMM:
    case URMA_OPC_WRITE_NOTIFY:
      xlate(a, false);
      xlate(b, true);
      w.rw.src = urma_sg_t{a.data(), (uint32_t)a.size()};
      w.rw.dst = urma_sg_t{b.data(), (uint32_t)b.size()};
      break;
    case URMA_OPC_READ:
      xlate(a, true);
      xlate(b, false);
      w.rw.src = urma_sg_t{a.data(), (uint32_t)a.size()};
      w.rw.dst = urma_sg_t{b.data(), (uint32_t)b.size()};
      break;
    case URMA_OPC_SEND:
    case URMA_OPC_SEND_IMM:
      xlate(a, false);
      w.send.src = urma_sg_t{a.data(), (uint32_t)a.size()};
      break;
    case URMA_OPC_CAS:
    case URMA_OPC_SWAP:
      cd.tseg = reinterpret_cast<BSeg*>(cd.tseg->priv)->p[p];
      cs.tseg = nullptr;
      w.cas.dst = &cd;
      w.cas.src = s->wr.cas.src ? &cs : nullptr;
      break;
    case URMA_OPC_FADD:
    case URMA_OPC_FSUB:
    case URMA_OPC_FAND:
    case URMA_OPC_FOR:
    case URMA_OPC_FXOR:
      cd.tseg = reinterpret_cast<BSeg*>(cd.tseg->priv)->p[p];
      cs.tseg = nullptr;
      w.faa.dst = &cd;
      w.faa.src = s->wr.faa.src ? &cs : nullptr;
      break;
    default: return URMA_EINVAL;
  }
  w.next = nullptr;
  urma_jfs_wr_t* bad = nullptr;
  c->path[p].tx.fetch_add(1);
  c->path[p].inflight.fetch_add(1);
  const urma_status_t rc = urma_post_jetty_send_wr(s->jetty->p[p], &w, &bad);
  if (rc != URMA_SUCCESS) c->path[p].inflight.fetch_sub(1);
  return rc;
}

// ------------------------------------------------------------------------------------------- ops
urma_jfc_t* op_create_jfc(urma_context_t* ctx, const urma_jfc_cfg_t* cfg) {
  BondCtx* c = C(ctx);
  BJfc* j = new BJfc();
  urma_jfc_cfg_t pc = *cfg;
  pc.jfce = nullptr;
  for (int i = 0; i < c->npaths; ++i) {
    j->p[i] = urma_create_jfc(c->p[i], &pc);
    if (!j->p[i]) {
      for (int k = 0; k < i; ++k) urma_delete_jfc(j->p[k]);
      delete j;
      return nullptr;
    }
  }
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jfc(urma_jfc_t*, uint32_t, uint32_t) { return URMA_SUCCESS; }
urma_status_t op_delete_jfc(urma_jfc_t* jfc) {
  BJfc* j = reinterpret_cast<BJfc*>(jfc->priv);
  for (auto* p : j->p)
    if (p) urma_delete_jfc(p);
  delete j;
  return URMA_SUCCESS;
}

urma_jetty_t* op_create_jetty(urma_context_t* ctx, const urma_jetty_cfg_t* cfg) {
  BondCtx* c = C(ctx);
  if (cfg->shared_jfr) return nullptr;  // shared receive queues are not supported on the bond device
  BJetty* j = new BJetty();
  j->sjfc = reinterpret_cast<BJfc*>(cfg->jfs_cfg.jfc->priv);
  j->rjfc = reinterpret_cast<BJfc*>(cfg->jfr_cfg.jfc->priv);
  j->v_id = g_dev.reg->next_id.fetch_add(1) + 1;
  RegEntry* e = reg_claim(ctx->uasid, j->v_id);
  if (!e) {
    delete j;
    return nullptr;
  }
  e->v_uasid = ctx->uasid;
  e->v_id = j->v_id;
  e->npaths = c->npaths;
  for (int i = 0; i < c->npaths; ++i) {
    urma_jetty_cfg_t pc = *cfg;
    pc.id = 0;
    pc.jfs_cfg.jfc = j->sjfc->p[i];
    pc.jfr_cfg.jfc = j->rjfc->p[i];
    pc.jfs_cfg.max_sge = 2;
    pc.jfr_cfg.max_sge = 2;
    if (pc.jfs_cfg.err_timeout == 0) pc.jfs_cfg.err_timeout = 2;  // 400 ms: fail over quickly
    j->p[i] = urma_create_jetty(c->p[i], &pc);
    if (!j->p[i]) {
      for (int k = 0; k < i; ++k) urma_delete_jetty(j->p[k]);
      e->type.store(REG_BUSY);
      delete j;
      return nullptr;
    }
    e->p_uasid[i] = j->p[i]->jetty_id.uasid;
    e->p_id[i] = j->p[i]->jetty_id.id;
  }
  e->type.store(REG_JETTY, std::memory_order_release);
  j->recv_depth = cfg->jfr_cfg.depth;
  const uint32_t nb = std::min<uint32_t>(cfg->jfr_cfg.depth, 128);
  for (int i = 0; i < c->npaths; ++i) {
    j->bounce[i].resize(nb);
    for (uint32_t b = 0; b < nb; ++b) {
      j->bounce[i][b].resize(kBounceBytes);
      urma_sge_t g{reinterpret_cast<uint64_t>(j->bounce[i][b].data()), kBounceBytes, nullptr};
      urma_jfr_wr_t w{};
      w.src = urma_sg_t{&g, 1};
      w.user_ctx = b;
      urma_jfr_wr_t* bad = nullptr;
      urma_post_jetty_recv_wr(j->p[i], &w, &bad);
    }
  }
  j->pub.jetty_id.eid = g_dev.eid;
  j->pub.jetty_id.uasid = ctx->uasid;
  j->pub.jetty_id.id = j->v_id;
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jetty(urma_jetty_t* jt, urma_jetty_state_t st) {
  BJetty* j = reinterpret_cast<BJetty*>(jt->priv);
  for (auto* p : j->p)
    if (p) urma_modify_jetty(p, st);
  return URMA_SUCCESS;
}
urma_status_t op_delete_jetty(urma_jetty_t* jt) {
  BJetty* j = reinterpret_cast<BJetty*>(jt->priv);
  BondCtx* c = C(jt->ctx);
  reg_release(REG_JETTY, jt->ctx->uasid, j->v_id);
  {
    std::lock_guard<std::mutex> l(c->mu);
    for (auto it = c->store.begin(); it != c->store.end();) {
      if (it->second->jetty == j) {
        delete it->second;
        it = c->store.erase(it);
      } else {
        ++it;
      }
    }
  }
  for (auto* p : j->p)
    if (p) urma_delete_jetty(p);
  delete j;
  return URMA_SUCCESS;
}
urma_target_jetty_t* op_import_jetty(urma_context_t* ctx, const urma_rjetty_t* rj, const urma_token_t* token) {
  BondCtx* c = C(ctx);
  RegEntry* e = reg_find(REG_JETTY, rj->jetty_id.uasid, rj->jetty_id.id);
  if (!e) return nullptr;
  BTarget* t = new BTarget();
  for (int i = 0; i < c->npaths && i < (int)e->npaths; ++i) {
    urma_rjetty_t pr = *rj;
    pr.jetty_id.eid = c->p[i]->eid;
    pr.jetty_id.uasid = e->p_uasid[i];
    pr.jetty_id.id = e->p_id[i];
    t->p[i] = urma_import_jetty(c->p[i], &pr, token);
    if (!t->p[i]) {
      for (int k = 0; k < i; ++k) urma_unimport_jetty(t->p[k]);
      delete t;
      return nullptr;
    }
  }
  t->pub.id = rj->jetty_id;
  t->pub.trans_mode = rj->trans_mode;
  t->pub.type = rj->type;
  t->pub.priv = t;
  return &t->pub;
}
urma_status_t op_unimport_jetty(urma_target_jetty_t* tj) {
  BTarget* t = reinterpret_cast<BTarget*>(tj->priv);
  for (auto* p : t->p)
    if (p) urma_unimport_jetty(p);
  delete t;
  return URMA_SUCCESS;
}
urma_status_t op_bind(urma_jetty_t*, urma_target_jetty_t*) { return URMA_SUCCESS; }
urma_status_t op_unbind(urma_jetty_t*) { return URMA_SUCCESS; }

urma_token_id_t* op_alloc_token(urma_context_t*) {
  urma_token_id_t* t = new urma_token_id_t();
  t->token_id = g_dev.reg->next_id.fetch_add(1) + 1;
  return t;
}
urma_status_t op_free_token(urma_token_id_t* t) {
  delete t;
  return URMA_SUCCESS;
}
urma_target_seg_t* op_register_seg(urma_context_t* ctx, const urma_seg_cfg_t* cfg) {
  BondCtx* c = C(ctx);
  BSeg* s = new BSeg();
  RegEntry* e = reg_claim(ctx->uasid, cfg->token_id->token_id);
  if (!e) {
    delete s;
    return nullptr;
  }
  e->v_uasid = ctx->uasid;
  e->v_id = cfg->token_id->token_id;
  e->npaths = c->npaths;
  e->va = cfg->va;
  e->len = cfg->len;
  e->attr = cfg->access;
  for (int i = 0; i < c->npaths; ++i) {
    urma_seg_cfg_t pc = *cfg;
    pc.token_id = nullptr;
    s->p[i] = urma_register_seg(c->p[i], &pc);
    if (!s->p[i]) {
      for (int k = 0; k < i; ++k) urma_unregister_seg(s->p[k]);
      e->type.store(REG_BUSY);
      delete s;
      return nullptr;
    }
    e->p_uasid[i] = s->p[i]->seg.ubva.uasid;
    e->p_id[i] = s->p[i]->seg.token_id;
  }
  e->type.store(REG_SEG, std::memory_order_release);
  s->pub.seg.ubva.eid = g_dev.eid;
  s->pub.seg.ubva.uasid = ctx->uasid;
  s->pub.seg.ubva.va = cfg->va;
  s->pub.seg.len = cfg->len;
  s->pub.seg.attr = cfg->access;
  s->pub.seg.token_id = cfg->token_id->token_id;
  s->pub.priv = s;
  return &s->pub;
}
urma_status_t op_unregister_seg(urma_target_seg_t* ts) {
  BSeg* s = reinterpret_cast<BSeg*>(ts->priv);
  reg_release(REG_SEG, ts->seg.ubva.uasid, ts->seg.token_id);
  for (auto* p : s->p)
    if (p) urma_unregister_seg(p);
  delete s;
  return URMA_SUCCESS;
}
urma_target_seg_t* op_import_seg(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token, uint64_t addr,
                                 uint32_t flag) {
  BondCtx* c = C(ctx);
  RegEntry* e = reg_find(REG_SEG, seg->ubva.uasid, seg->token_id);
  if (!e) return nullptr;
  BSeg* s = new BSeg();
  for (int i = 0; i < c->npaths && i < (int)e->npaths; ++i) {
    urma_seg_t ps = *seg;
    ps.ubva.eid = c->p[i]->eid;
    ps.ubva.uasid = e->p_uasid[i];
    ps.token_id = e->p_id[i];
    s->p[i] = urma_import_seg(c->p[i], &ps, token, addr, flag);
    if (!s->p[i]) {
      for (int k = 0; k < i; ++k) urma_unimport_seg(s->p[k]);
      delete s;
      return nullptr;
    }
  }
  s->pub.seg = *seg;
  s->pub.priv = s;
  return &s->pub;
}
urma_status_t op_unimport_seg(urma_target_seg_t* ts) {
  BSeg* s = reinterpret_cast<BSeg*>(ts->priv);
  for (auto* p : s->p)
    if (p) urma_unimport_seg(p);
  delete s;
  return URMA_SUCCESS;
}

urma_status_t op_post_send(urma_jetty_t* jt, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  BondCtx* c = C(jt->ctx);
  BJetty* j = reinterpret_cast<BJetty*>(jt->priv);
  for (urma_jfs_wr_t* w = wr; w; w = w->next) {
    urma_target_jetty_t* tj = w->tjetty ? w->tjetty : jt->remote_jetty;
    const int path = pick_path(c);
    if (!tj || path < 0) {
      *bad = w;
      return path < 0 ? URMA_FAIL : URMA_EINVAL;
    }
    StoredWr* s = new StoredWr();
    s->wr = *w;
    s->user_ctx = w->user_ctx;
    s->flag = w->flag;
    s->path = path;
    s->tries = 1;
    s->jetty = j;
    s->target = reinterpret_cast<BTarget*>(tj->priv);
    switch (w->opcode) {
      case URMA_OPC_WRITE:
      case URMA_OPC_WRITE_IMM:
      case URMA_OPC_WRITE_NOTIFY:
      case URMA_OPC_READ:
        s->sg_a.assign(w->rw.src.sge, w->rw.src.sge + w->rw.src.num_sge);
        s->sg_b.assign(w->rw.dst.sge, w->rw.dst.sge + w->rw.dst.num_sge);
        break;
      case URMA_OPC_SEND:
      case URMA_OPC_SEND_IMM: {
        uint32_t total = 0;
        for (uint32_t q = 0; q < w->send.src.num_sge; ++q) total += w->send.src.sge[q].len;
        if (total + sizeof(BondHdr) > kBounceBytes || w->send.src.num_sge + 1 > URMA_MAX_SGE) {
          delete s;
          *bad = w;
          return URMA_EINVAL;
        }
        s->hdr = BondHdr{kBondMagic, jt->ctx->uasid, j->v_id, j->msn.fetch_add(1)};
        s->sg_a.push_back(urma_sge_t{reinterpret_cast<uint64_t>(&s->hdr), sizeof(BondHdr), nullptr});
        s->sg_a.insert(s->sg_a.end(), w->send.src.sge, w->send.src.sge + w->send.src.num_sge);
        break;
      }
      case URMA_OPC_CAS:
      case URMA_OPC_SWAP:
        s->cas_dst = *w->cas.dst;
        if (w->cas.src) s->cas_src = *w->cas.src;
        break;
      case URMA_OPC_FADD:
      case URMA_OPC_FSUB:
      case URMA_OPC_FAND:
      case URMA_OPC_FOR:
      case URMA_OPC_FXOR:
        s->cas_dst = *w->faa.dst;
        if (w->faa.src) s->cas_src = *w->faa.src;
        break;
      default:
        delete s;
        *bad = w;
        return URMA_EINVAL;
    }
    const uint64_t id = c->next_wr.fetch_add(1);
    {
      std::lock_guard<std::mutex> l(c->mu);
      c->store[id] = s;
    }
    const urma_status_t st = post_stored(c, s, id);
    if (st != URMA_SUCCESS) {
      std::lock_guard<std::mutex> l(c->mu);
      c->store.erase(id);
      delete s;
      *bad = w;
      return st;
    }
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}

// Copies a parked or freshly arrived message into an application receive and queues the completion record.
void deliver_v(BJetty* j, const BJetty::VMsg& m, const BJetty::VRecv& r) {
  urma_cr_t cr{};
  cr.user_ctx = r.user_ctx;
  cr.flag = URMA_CR_FLAG_RECV;
  cr.opcode = m.opc;
  cr.imm_data = m.imm;
  cr.local_id = j->v_id;
  cr.remote_id.eid = g_dev.eid;
  cr.remote_id.uasid = m.src_uasid;
  cr.remote_id.id = m.src_jetty;
  uint32_t cap = 0;
  for (auto& g : r.sges) cap += g.len;
  if (m.data.size() > cap) {
    cr.status = URMA_CR_LOC_LEN_ERR;
  } else {
    size_t off = 0;
    for (auto& g : r.sges) {
      if (off >= m.data.size()) break;
      const size_t n = std::min<size_t>(g.len, m.data.size() - off);
      memcpy(reinterpret_cast<void*>(g.addr), m.data.data() + off, n);
      off += n;
    }
    cr.status = URMA_CR_SUCCESS;
    cr.completion_len = static_cast<uint32_t>(m.data.size());
  }
  std::lock_guard<std::mutex> l(j->rjfc->mu);
  j->rjfc->ready.push_back(cr);
}

urma_status_t op_post_recv(urma_jetty_t* jt, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  BJetty* j = reinterpret_cast<BJetty*>(jt->priv);
  for (urma_jfr_wr_t* w = wr; w; w = w->next) {
    BJetty::VRecv r;
    r.user_ctx = w->user_ctx;
    r.sges.assign(w->src.sge, w->src.sge + w->src.num_sge);
    std::unique_lock<std::mutex> l(j->mu);
    if (!j->v_unexp.empty()) {
      BJetty::VMsg m = std::move(j->v_unexp.front());
      j->v_unexp.pop_front();
      l.unlock();
      deliver_v(j, m, r);
      continue;
    }
    if (j->v_posted.size() >= j->recv_depth) {
      *bad = w;
      return URMA_EAGAIN;
    }
    j->v_posted.push_back(std::move(r));
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}

// Translates one physical send-side completion; returns true when a virtual completion was produced in *out.
bool translate(BondCtx* c, BJfc* vj, int path, const urma_cr_t& pc, urma_cr_t* out) {
  StoredWr* s = nullptr;
  {
    std::lock_guard<std::mutex> l(c->mu);
    auto it = c->store.find(pc.user_ctx);
    if (it == c->store.end()) return false;
    s = it->second;
  }
  c->path[path].inflight.fetch_sub(1);
  if (pc.status != URMA_CR_SUCCESS && pc.status != URMA_CR_REM_ACCESS_ABORT_ERR &&
      pc.status != URMA_CR_REM_OPERATION_ERR) {
    // transport-level failure: the path is suspect
    c->path[path].errors.fetch_add(1);
    mark_down(c, path);
    urma_modify_jetty(s->jetty->p[path], URMA_JETTY_STATE_READY);  // clear the error state for later failback
    if (c->failover && s->tries < c->npaths + 1) {
      const int np = pick_path(c, path);
      if (np >= 0) {
        s->path = np;
        ++s->tries;
        c->path[np].failovers.fetch_add(1);
        if (c->resend_delay_ms > 0 && c->health_thr.joinable()) {
          // resend from the timing wheel; if that post fails too the request completes with an error there
          const uint64_t id = pc.user_ctx;
          const urma_cr_t orig = pc;
          c->deferred_resends.fetch_add(1);
          c->wheel.schedule(c->resend_delay_ms, [c, s, id, orig, vj](bond::TimeWheel::Reason why) {
            if (why == bond::TimeWheel::kExecuted && post_stored(c, s, id) == URMA_SUCCESS) return;
            {
              std::lock_guard<std::mutex> l(c->mu);
              c->store.erase(id);
            }
            urma_cr_t out = orig;
            out.user_ctx = s->user_ctx;
            out.local_id = s->jetty->v_id;
            out.remote_id = s->target->pub.id;
            {
              std::lock_guard<std::mutex> l(vj->mu);
              vj->ready.push_back(out);
            }
            delete s;
          });
          return false;
        }
        if (post_stored(c, s, pc.user_ctx) == URMA_SUCCESS) return false;  // completion will come from the new path
      }
    }
  }
  {
    std::lock_guard<std::mutex> l(c->mu);
    c->store.erase(pc.user_ctx);
  }
  const bool report = (s->flag & URMA_WR_FLAG_COMPLETE_ENABLE) || pc.status != URMA_CR_SUCCESS;
  if (report) {
    *out = pc;
    out->user_ctx = s->user_ctx;
    out->local_id = s->jetty->v_id;
    out->remote_id = s->target->pub.id;
    if (s->wr.opcode == URMA_OPC_SEND || s->wr.opcode == URMA_OPC_SEND_IMM)
      out->completion_len = pc.completion_len >= sizeof(BondHdr) ? pc.completion_len - sizeof(BondHdr) : 0;
  }
  delete s;
  (void)vj;
  return report;
}

}  // namespace

// receive-side translation needs the owning jetty: keep a per-context index physical jetty id -> virtual jetty
namespace {
std::mutex g_idx_mu;
std::unordered_map<uint64_t, BJetty*> g_pj_index;  // (path, physical uasid, physical jetty id) -> virtual jetty
uint64_t pj_key(int path, uint32_t uasid, uint32_t id) { return (uint64_t(path) << 60) ^ (uint64_t(uasid) << 32) ^ id; }

int op_poll_jfc(urma_jfc_t* jfc, int n, urma_cr_t* cr) {
  BondCtx* c = C(jfc->ctx);
  BJfc* vj = reinterpret_cast<BJfc*>(jfc->priv);
  int k = 0;
  auto drain_ready = [&]() {
    std::lock_guard<std::mutex> l(vj->mu);
    while (k < n && !vj->ready.empty()) {
      cr[k++] = vj->ready.front();
      vj->ready.pop_front();
    }
  };
  drain_ready();
  for (int step = 0; step < c->npaths && k < n; ++step) {
    const int p = (vj->next_poll + step) % c->npaths;
    urma_cr_t pc[16];
    const int got = urma_poll_jfc(vj->p[p], std::min(16, n - k), pc);
    for (int i = 0; i < got; ++i) {
      if (pc[i].flag & URMA_CR_FLAG_RECV) {
        BJetty* j = nullptr;
        {
          std::lock_guard<std::mutex> l(g_idx_mu);
          auto it = g_pj_index.find(pj_key(p, c->p[p]->uasid, pc[i].local_id));
          if (it != g_pj_index.end()) j = it->second;
        }
        if (!j || pc[i].user_ctx >= j->bounce[p].size()) continue;
        std::vector<uint8_t>& bb = j->bounce[p][pc[i].user_ctx];
        BondHdr h;
        memcpy(&h, bb.data(), sizeof(h));
        bool keep = pc[i].status == URMA_CR_SUCCESS && h.magic == kBondMagic &&
                    pc[i].completion_len >= sizeof(BondHdr);
        BJetty::VMsg m;
        BJetty::VRecv r;
        bool have_recv = false;
        if (keep) {
          std::lock_guard<std::mutex> l(j->mu);
          bond::SlideWindow& w = j->windows[(uint64_t(h.src_uasid) << 32) | h.src_jetty];
          keep = w.accept(h.msn);  // false: second copy of a message that was re-sent after a path failure
          if (keep) {
            m.data.assign(bb.begin() + sizeof(BondHdr), bb.begin() + pc[i].completion_len);
            m.imm = pc[i].imm_data;
            m.opc = pc[i].opcode;
            m.src_uasid = h.src_uasid;
            m.src_jetty = h.src_jetty;
            if (!j->v_posted.empty()) {
              r = std::move(j->v_posted.front());
              j->v_posted.pop_front();
              have_recv = true;
            } else {
              j->v_unexp.push_back(m);
            }
          }
        }
        {  // hand the bounce buffer back to the path
          urma_sge_t g{reinterpret_cast<uint64_t>(bb.data()), kBounceBytes, nullptr};
          urma_jfr_wr_t w{};
          w.src = urma_sg_t{&g, 1};
          w.user_ctx = pc[i].user_ctx;
          urma_jfr_wr_t* bad = nullptr;
          urma_post_jetty_recv_wr(j->p[p], &w, &bad);
        }
        if (keep && have_recv) deliver_v(j, m, r);
      } else {
        urma_cr_t v;
        if (translate(c, vj, p, pc[i], &v)) cr[k++] = v;
      }
      if (k >= n) break;
    }
  }
  vj->next_poll = (vj->next_poll + 1) % c->npaths;
  drain_ready();
  return k;
}

void index_jetty(BondCtx* c, BJetty* j, bool add) {
  std::lock_guard<std::mutex> l(g_idx_mu);
  for (int i = 0; i < c->npaths; ++i) {
    if (!j->p[i]) continue;
    const uint64_t key = pj_key(i, c->p[i]->uasid, j->p[i]->jetty_id.id);
    if (add) g_pj_index[key] = j;
    else g_pj_index.erase(key);
  }
}
urma_jetty_t* op_create_jetty_indexed(urma_context_t* ctx, const urma_jetty_cfg_t* cfg) {
  urma_jetty_t* j = op_create_jetty(ctx, cfg);
  if (j) index_jetty(C(ctx), reinterpret_cast<BJetty*>(j->priv), true);
  return j;
}
urma_status_t op_delete_jetty_indexed(urma_jetty_t* jt) {
  index_jetty(C(jt->ctx), reinterpret_cast<BJetty*>(jt->priv), false);
  return op_delete_jetty(jt);
}

urma_status_t op_query_jetty(urma_jetty_t* jt, urma_jetty_cfg_t* cfg, urma_jetty_state_t* st) {
  *cfg = jt->cfg;
  // the virtual jetty is as ready as its best member: READY while any member path is, else the first member's state
  BJetty* j = reinterpret_cast<BJetty*>(jt->priv);
  urma_jetty_state_t first = URMA_JETTY_STATE_READY;
  bool have = false, ready = false;
  for (auto* p : j->p) {
    if (!p) continue;
    urma_jetty_cfg_t pc;
    urma_jetty_state_t ps;
    if (urma_query_jetty(p, &pc, &ps) != URMA_SUCCESS) continue;
    if (!have) first = ps;
    have = true;
    ready |= ps == URMA_JETTY_STATE_READY;
  }
  *st = (!have || ready) ? URMA_JETTY_STATE_READY : first;
  return URMA_SUCCESS;
}

// user_ctl: 1 = path statistics -> out->addr points to uint64[npaths][6] {up, tx, errors, failovers, failbacks, admin}
//           2 = administratively set path state: in->addr = path, in->len = 1 (down) / 0 (up)
//           3 = set aggregation mode: in->addr = 0 standalone, 1 active-backup, 2 balance
//           4 = inject a link fault on a physical path: in->addr = path, in->len = 1 (drop) / 0 (restore)
//           5 = set the scheduling policy of BALANCE mode: in->addr = 0 round-robin, 1 priority, 2 affinity,
//               3 least-load, 4 random
//           6 = set the priority list: in->addr = path numbers packed 4 bits each, most preferred in the low nibble
//           7 = scheduler statistics -> out->addr points to uint64[2 + npaths] {policy, deferred resends, in flight...}
int op_user_ctl(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out) {
  BondCtx* c = C(ctx);
  switch (in->opcode) {
    case 1: {
      uint64_t* o = reinterpret_cast<uint64_t*>(out->addr);
      if (!o || out->len < sizeof(uint64_t) * 6 * c->npaths) return -1;
      for (int i = 0; i < c->npaths; ++i) {
        o[i * 6 + 0] = c->path[i].up.load();
        o[i * 6 + 1] = c->path[i].tx.load();
        o[i * 6 + 2] = c->path[i].errors.load();
        o[i * 6 + 3] = c->path[i].failovers.load();
        o[i * 6 + 4] = c->path[i].failbacks.load();
        o[i * 6 + 5] = c->path[i].admin_down.load();
      }
      out->rsv = c->npaths;
      return 0;
    }
    case 2:
      if (in->addr >= (uint64_t)c->npaths) return -1;
      c->path[in->addr].admin_down = in->len != 0;
      return 0;
    case 3:
      if (in->addr > MODE_BALANCE) return -1;
      c->mode = static_cast<int>(in->addr);
      return 0;
    case 4: {
      if (in->addr >= (uint64_t)c->npaths) return -1;
      urma_user_ctl_in_t pin{in->len, 0, 4};
      urma_user_ctl_out_t pout{};
      return urma_user_ctl(c->p[in->addr], &pin, &pout);
    }
    case 5:
      if (in->addr > POL_LAST) return -1;
      c->policy = static_cast<int>(in->addr);
      return 0;
    case 6: {
      int order[kMaxPaths];
      uint32_t seen = 0;
      for (int k = 0; k < c->npaths; ++k) {
        order[k] = static_cast<int>((in->addr >> (4 * k)) & 0xf);
        if (order[k] >= c->npaths || (seen & (1u << order[k]))) return -1;
        seen |= 1u << order[k];
      }
      for (int k = 0; k < c->npaths; ++k) c->priority[k] = order[k];
      return 0;
    }
    case 7: {
      uint64_t* o = reinterpret_cast<uint64_t*>(out->addr);
      if (!o || out->len < sizeof(uint64_t) * (2 + c->npaths)) return -1;
      o[0] = static_cast<uint64_t>(c->policy.load());
      o[1] = c->deferred_resends.load();
      for (int i = 0; i < c->npaths; ++i) o[2 + i] = static_cast<uint64_t>(std::max<int64_t>(0, c->path[i].inflight.load()));
      out->rsv = c->npaths;
      return 0;
    }
    default: return -1;
  }
}

void probe_paths(BondCtx* c);

// Timer thread: advances the timing wheel by wall-clock ticks. Failback probing is itself a wheel task that puts
// itself back on the wheel every `health_ms` (and at once when a path goes down: hcv).
void health_loop(BondCtx* c) {
  urma_log_set_thread_tag("bond-timer");
  uint64_t last = ub::now_ns();
  std::function<void(bond::TimeWheel::Reason)> probe_task = [&, c](bond::TimeWheel::Reason why) {
    if (why != bond::TimeWheel::kExecuted || c->stop.load()) return;
    if (c->health) probe_paths(c);
    c->wheel.schedule(c->health_ms, probe_task);
  };
  c->wheel.schedule(c->health_ms, probe_task);
  while (!c->stop.load()) {
    {
      std::unique_lock<std::mutex> l(c->hmu);
      c->hcv.wait_for(l, std::chrono::milliseconds(c->wheel.tick_ms()));
    }
    if (c->stop.load()) break;
    const uint64_t now = ub::now_ns();
    const uint64_t ticks = (now - last) / (1000000ull * c->wheel.tick_ms());
    if (ticks > 0) {
      c->wheel.advance(static_cast<uint32_t>(std::min<uint64_t>(ticks, 1024)));
      last += ticks * 1000000ull * c->wheel.tick_ms();
    }
  }
}

void probe_paths(BondCtx* c) {
  {
    for (int i = 0; i < c->npaths; ++i) {
      PathState& ps = c->path[i];
      if (ps.up.load() || !c->failback || !ps.probe_jetty) continue;
      // probe: a NOP through the physical path to our own probe jetty
      urma_modify_jetty(ps.probe_jetty, URMA_JETTY_STATE_READY);
      urma_jfs_wr_t w{};
      w.opcode = URMA_OPC_NOP;
      w.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
      w.tjetty = ps.probe_self;
      w.user_ctx = 0x70726f6265ull;
      urma_jfs_wr_t* bad = nullptr;
      if (urma_post_jetty_send_wr(ps.probe_jetty, &w, &bad) != URMA_SUCCESS) continue;
      const uint64_t deadline = ub::now_ns() + 600000000ull;
      urma_cr_t cr;
      bool ok = false, done = false;
      while (!done && ub::now_ns() < deadline && !c->stop.load()) {
        if (urma_poll_jfc(ps.probe_jfc, 1, &cr) == 1) {
          ok = cr.status == URMA_CR_SUCCESS;
          done = true;
        } else {
          usleep(200);
        }
      }
      if (ok) {
        ps.up = true;
        ps.failbacks.fetch_add(1);
        urma_log(URMA_VLOG_LEVEL_WARNING, __func__, __LINE__, "bond: path %d is back", i);
      }
    }
  }
}

const urma_ops_t g_ops = {
    "bond",
    op_create_jfc, op_modify_jfc, op_delete_jfc, nullptr, nullptr,
    nullptr, nullptr, nullptr, nullptr, nullptr,           // stand-alone JFS: not supported
    nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,  // stand-alone JFR: not supported
    op_create_jetty_indexed, op_modify_jetty, op_query_jetty, nullptr, op_delete_jetty_indexed,
    op_import_jetty, op_unimport_jetty, op_bind, op_unbind, nullptr, nullptr,
    op_alloc_token, op_free_token, op_register_seg, op_unregister_seg, op_import_seg, op_unimport_seg,
    nullptr, nullptr, op_post_send, op_post_recv, op_poll_jfc, nullptr, nullptr, nullptr,
    nullptr, nullptr, op_user_ctl,
};

urma_status_t prov_init(const urma_init_attr_t*) {
  memset(g_dev.eid.raw, 0, 16);
  memcpy(g_dev.eid.raw, "bond", 4);
  const uint32_t uid = getuid();
  memcpy(g_dev.eid.raw + 8, &uid, 4);
  g_dev.eid.raw[15] = 1;
  return URMA_SUCCESS;
}
urma_status_t prov_uninit(void) { return URMA_SUCCESS; }
int prov_get_devices(urma_device_t* devs, int max) {
  if (max < 1) return 0;
  memset(&devs[0], 0, sizeof(urma_device_t));
  snprintf(devs[0].name, sizeof(devs[0].name), "bond0");
  devs[0].eid = g_dev.eid;
  return 1;
}
urma_status_t prov_query(const urma_device_t*, urma_device_attr_t* a) {
  memset(a, 0, sizeof(*a));
  a->max_jfc = a->max_jetty = 65536;
  a->max_seg = 1u << 16;
  a->max_jfc_depth = a->max_jfs_depth = a->max_jfr_depth = 65536;
  a->max_sge = URMA_MAX_SGE - 1;
  a->max_msg_size = 1ull << 30;
  a->transport_modes = URMA_TM_RM;
  a->port_cnt = kMaxPaths;
  a->atomic_supported = true;
  return URMA_SUCCESS;
}

urma_context_t* prov_create_context(urma_device_t*, uint32_t) {
  if (!g_dev.reg) {
    const char* e = getenv("URMA_SHM_DIR");
    const std::string dir = (e && *e) ? e : "/dev/shm/umdk_urma_" + std::to_string(getuid());
    mkdir(dir.c_str(), 0700);
    const std::string path = dir + "/bond0.reg";
    int fd = open(path.c_str(), O_RDWR | O_CREAT, 0600);
    if (fd < 0) return nullptr;
    if (ftruncate(fd, sizeof(BondReg)) != 0) {
      close(fd);
      return nullptr;
    }
    void* p = mmap(nullptr, sizeof(BondReg), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return nullptr;
    g_dev.reg = static_cast<BondReg*>(p);
    uint32_t exp = 0;
    g_dev.reg->magic.compare_exchange_strong(exp, kBondMagic);
  }
  BondCtx* c = new BondCtx();
  // physical paths: $BOND_DEVICES="shm0,shm1" or every shm* device
  std::vector<std::string> names;
  if (const char* e = getenv("BOND_DEVICES")) {
    std::string s(e);
    size_t pos = 0;
    while (pos <= s.size()) {
      const size_t comma = s.find(',', pos);
      names.push_back(s.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos));
      if (comma == std::string::npos) break;
      pos = comma + 1;
    }
  } else {
    // members registered for the aggregation device "bond0" in the topology library, else every shm* device
    uvs_agg_dev_t agg;
    if (uvs_get_agg_dev("bond0", &agg) == 0) {
      for (uint32_t i = 0; i < agg.member_num; ++i) names.push_back(agg.member_names[i]);
    } else {
      for (int i = 0; i < kMaxPaths; ++i) names.push_back("shm" + std::to_string(i));
    }
  }
  for (auto& n : names) {
    if (c->npaths >= kMaxPaths) break;
    urma_device_t* d = urma_get_device_by_name(n.c_str());
    if (!d) continue;
    urma_context_t* pc = urma_create_context(d, 0);
    if (pc) c->p[c->npaths++] = pc;
  }
  if (c->npaths == 0) {
    delete c;
    return nullptr;
  }
  c->failover = env_on("BOND_ENABLE_FAILOVER", true);
  c->failback = env_on("BOND_ENABLE_FAILBACK", true);
  c->health = env_on("BOND_ENABLE_HEALTH_CHECK", true);
  if (const char* e = getenv("BOND_HEALTH_CHECK_ACTIVE_INTERVAL")) c->health_ms = std::max(10, atoi(e));
  if (const char* e = getenv("BOND_MODE")) c->mode = std::max(0, std::min(2, atoi(e)));
  if (const char* e = getenv("BOND_SCHED_POLICY")) {
    static const char* names[] = {"round_robin", "priority", "affinity", "least_load", "random"};
    for (int i = 0; i <= POL_LAST; ++i)
      if (!strcmp(e, names[i]) || (e[0] == '0' + i && !e[1])) c->policy = i;
  }
  if (const char* e = getenv("BOND_PATH_PRIORITY")) {   // "2,0,1": paths not named keep their order behind those named
    std::vector<int> order;
    for (const char* q = e; *q;) {
      const int v = atoi(q);
      if (v >= 0 && v < c->npaths && std::find(order.begin(), order.end(), v) == order.end()) order.push_back(v);
      while (*q && *q != ',') ++q;
      if (*q == ',') ++q;
    }
    for (int i = 0; i < c->npaths; ++i)
      if (std::find(order.begin(), order.end(), i) == order.end()) order.push_back(i);
    for (int i = 0; i < c->npaths; ++i) c->priority[i] = order[i];
  }
  if (const char* e = getenv("BOND_RESEND_DELAY_MS")) c->resend_delay_ms = static_cast<uint32_t>(std::max(0, atoi(e)));
  c->pub.ops = &g_ops;
  c->pub.eid = g_dev.eid;
  c->pub.uasid = g_dev.reg->next_uasid.fetch_add(1) + 1;
  c->pub.priv = c;
  c->pub.async_fd = -1;
  for (int i = 0; i < c->npaths; ++i) {  // self-probe objects per path
    PathState& ps = c->path[i];
    urma_jfc_cfg_t cc{};
    cc.depth = 16;
    ps.probe_jfc = urma_create_jfc(c->p[i], &cc);
    urma_jetty_cfg_t jc{};
    jc.jfs_cfg.depth = 8;
    jc.jfs_cfg.jfc = ps.probe_jfc;
    jc.jfs_cfg.err_timeout = 1;
    jc.jfr_cfg.depth = 8;
    jc.jfr_cfg.jfc = ps.probe_jfc;
    ps.probe_jetty = ps.probe_jfc ? urma_create_jetty(c->p[i], &jc) : nullptr;
    if (ps.probe_jetty) {
      urma_rjetty_t rj{ps.probe_jetty->jetty_id, URMA_TM_RM, 1};
      urma_token_t t{0};
      ps.probe_self = urma_import_jetty(c->p[i], &rj, &t);
    }
  }
  c->health_thr = std::thread(health_loop, c);   // timer thread: timing wheel (deferred resends, failback probes)
  return &c->pub;
}
urma_status_t prov_delete_context(urma_context_t* ctx) {
  BondCtx* c = C(ctx);
  c->stop = true;
  c->hcv.notify_all();
  if (c->health_thr.joinable()) c->health_thr.join();
  for (auto& kv : c->store) delete kv.second;
  for (int i = 0; i < c->npaths; ++i) {
    PathState& ps = c->path[i];
    if (ps.probe_self) urma_unimport_jetty(ps.probe_self);
    if (ps.probe_jetty) urma_delete_jetty(ps.probe_jetty);
    if (ps.probe_jfc) urma_delete_jfc(ps.probe_jfc);
    urma_delete_context(c->p[i]);
  }
  delete c;
  return URMA_SUCCESS;
}

const urma_provider_ops_t g_prov = {"bond",     prov_init,           prov_uninit,        prov_get_devices,
                                    prov_query, prov_create_context, prov_delete_context};
__attribute__((constructor)) void bond_provider_ctor() { urma_register_provider_ops(&g_prov); }

}  // namespace
