// Extended control plane of the URMA API: two-phase object creation, batch deletion, asynchronous import / bind with
// notifiers, peer descriptions, transport-path attributes and addressing helpers. Everything here is built on the
// provider vtable calls of urma_core.cpp, so it works the same over every provider.
//
// Reference: src/urma/lib/urma/core/include/urma_api.h (alloc/set_opt/active :144-186 and the jfs / jfr / jetty
// counterparts, *_batch :198, *_ex :371, :531, :579, asynchronous forms and notifiers :624-735, rjetty / seg ctx
// :606, :851, transport paths and addresses :1065-1171). There the work is done by the kernel driver and the
// transport-path service; on one box an import or a bind completes at once, a transport path is an entry of a
// table kept per context, and an EID doubles as its own network address.
#include <poll.h>
#include <string.h>
#include <sys/eventfd.h>
#include <unistd.h>

#include <deque>
#include <map>
#include <mutex>
#include <set>
#include <string>

#include "urma_api.h"
#include "urma_provider.h"

namespace {

// ------------------------------------------------------------------------------------------------ two-phase objects
// Objects made by urma_alloc_*: address -> active?  (objects made by urma_create_* are not in the table)
std::mutex g_tp_mu;
std::map<const void*, bool> g_two_phase;

void tp_track(const void* obj) {
  std::lock_guard<std::mutex> l(g_tp_mu);
  g_two_phase[obj] = false;
}
// 0 = not a two-phase object, 1 = allocated, 2 = active
int tp_state(const void* obj) {
  std::lock_guard<std::mutex> l(g_tp_mu);
  auto it = g_two_phase.find(obj);
  return it == g_two_phase.end() ? 0 : (it->second ? 2 : 1);
}
void tp_set_active(const void* obj, bool on) {
  std::lock_guard<std::mutex> l(g_tp_mu);
  auto it = g_two_phase.find(obj);
  if (it != g_two_phase.end()) it->second = on;
}
void tp_forget(const void* obj) {
  std::lock_guard<std::mutex> l(g_tp_mu);
  g_two_phase.erase(obj);
}

template <typename T>
urma_status_t opt_out(void* buf, uint32_t len, T v) {
  if (!buf || len < sizeof(T)) return URMA_EINVAL;
  memcpy(buf, &v, sizeof(T));
  return URMA_SUCCESS;
}
template <typename T>
bool opt_in(const void* buf, uint32_t len, T* v) {
  if (!buf || len < sizeof(T)) return false;
  memcpy(v, buf, sizeof(T));
  return true;
}

// per-JFC moderation settings chosen before activation (applied by urma_active_jfc)
struct JfcPending {
  uint32_t count = 0, period = 0;
  bool set = false;
};
std::map<const urma_jfc_t*, JfcPending> g_jfc_pending;
std::map<const urma_jfr_t*, uint32_t> g_jfr_threshold;

// ------------------------------------------------------------------------------------------------ notifiers
struct Notifier {
  urma_notifier_t pub;
  std::mutex mu;
  std::deque<urma_notify_t> q;
};
void notifier_push(urma_notifier_t* n, const urma_notify_t& ev) {
  Notifier* p = static_cast<Notifier*>(n->priv);
  {
    std::lock_guard<std::mutex> l(p->mu);
    p->q.push_back(ev);
  }
  const uint64_t one = 1;
  if (write(n->fd, &one, sizeof(one)) < 0) {
    // the counter is saturated: a reader will still find the queue non-empty
  }
}

// ------------------------------------------------------------------------------------------------ transport paths
struct TpKey {
  urma_eid_t local, peer;
  uint32_t mode;
  bool operator<(const TpKey& o) const {
    const int a = memcmp(&local, &o.local, sizeof(local));
    if (a) return a < 0;
    const int b = memcmp(&peer, &o.peer, sizeof(peer));
    if (b) return b < 0;
    return mode < o.mode;
  }
};
struct TpEntry {
  uint64_t handle;
  uint32_t bitmap = 0;
  urma_tp_attr_value_t value{};
  urma_tp_attr_t attr{0, 1, 0, 0, 4096};
};
struct TpTable {
  std::map<TpKey, uint64_t> by_key;
  std::map<uint64_t, TpEntry> by_handle;
  uint64_t next = 1;
};
std::mutex g_tpt_mu;
std::map<const urma_context_t*, TpTable> g_tp_tables;

struct CtxOpts {
  std::string log_tag;
  uint64_t user_data = 0;
};
std::map<const urma_context_t*, CtxOpts> g_ctx_opts;

void eid_to_mac(const urma_eid_t* eid, uint8_t* mac) {
  memcpy(mac, eid->raw + URMA_EID_SIZE - URMA_MAC_BYTES, URMA_MAC_BYTES);
  mac[0] = (uint8_t)((mac[0] & 0xfe) | 0x02);  // locally administered, unicast
}

}  // namespace

extern "C" {

// ================================================================================================ JFC
urma_status_t urma_alloc_jfc(urma_context_t* ctx, urma_jfc_cfg_t* cfg, urma_jfc_t** jfc) {
  if (!ctx || !cfg || !jfc) return URMA_EINVAL;
  urma_jfc_t* j = urma_create_jfc(ctx, cfg);
  if (!j) return URMA_FAIL;
  tp_track(j);
  *jfc = j;
  return URMA_SUCCESS;
}
urma_status_t urma_set_jfc_opt(urma_jfc_t* jfc, uint64_t opt, void* buf, uint32_t len) {
  if (!jfc) return URMA_EINVAL;
  if (tp_state(jfc) != 1) return URMA_ENOPERM;  // options are set between alloc and active
  std::lock_guard<std::mutex> l(g_tp_mu);
  switch (opt) {
    case URMA_OPT_USER_CTX: return opt_in(buf, len, &jfc->cfg.user_ctx) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_MODERATE_COUNT:
      if (!opt_in(buf, len, &g_jfc_pending[jfc].count)) return URMA_EINVAL;
      g_jfc_pending[jfc].set = true;
      return URMA_SUCCESS;
    case URMA_OPT_MODERATE_PERIOD:
      if (!opt_in(buf, len, &g_jfc_pending[jfc].period)) return URMA_EINVAL;
      g_jfc_pending[jfc].set = true;
      return URMA_SUCCESS;
    case URMA_OPT_DEPTH:
    case URMA_OPT_FLAG:
    case URMA_OPT_ID:
    case URMA_OPT_STATE: return URMA_ENOPERM;  // fixed by the cfg given to urma_alloc_jfc
    default: return URMA_EINVAL;
  }
}
urma_status_t urma_get_jfc_opt(urma_jfc_t* jfc, uint64_t opt, void* buf, uint32_t len) {
  if (!jfc) return URMA_EINVAL;
  switch (opt) {
    case URMA_OPT_DEPTH: return opt_out(buf, len, jfc->cfg.depth);
    case URMA_OPT_FLAG: return opt_out(buf, len, jfc->cfg.flag);
    case URMA_OPT_USER_CTX: return opt_out(buf, len, jfc->cfg.user_ctx);
    case URMA_OPT_ID: return opt_out(buf, len, jfc->id);
    case URMA_OPT_STATE: return opt_out<uint32_t>(buf, len, tp_state(jfc) == 1 ? 0u : 1u);
    case URMA_OPT_MODERATE_COUNT:
    case URMA_OPT_MODERATE_PERIOD: {
      std::lock_guard<std::mutex> l(g_tp_mu);
      auto it = g_jfc_pending.find(jfc);
      const JfcPending p = it == g_jfc_pending.end() ? JfcPending() : it->second;
      return opt_out(buf, len, opt == URMA_OPT_MODERATE_COUNT ? p.count : p.period);
    }
    default: return URMA_EINVAL;
  }
}
urma_status_t urma_active_jfc(urma_jfc_t* jfc) {
  if (!jfc || tp_state(jfc) != 1) return URMA_EINVAL;
  JfcPending p;
  {
    std::lock_guard<std::mutex> l(g_tp_mu);
    auto it = g_jfc_pending.find(jfc);
    if (it != g_jfc_pending.end()) p = it->second;
  }
  if (p.set) {
    const urma_status_t s = urma_modify_jfc(jfc, p.count, p.period);
    if (s != URMA_SUCCESS) return s;
  }
  tp_set_active(jfc, true);
  return URMA_SUCCESS;
}
urma_status_t urma_deactive_jfc(urma_jfc_t* jfc) {
  if (!jfc || tp_state(jfc) != 2) return URMA_EINVAL;
  if (__atomic_load_n(&jfc->refcnt, __ATOMIC_RELAXED) > 1) return URMA_EAGAIN;  // queues still complete into it
  tp_set_active(jfc, false);
  return URMA_SUCCESS;
}
urma_status_t urma_free_jfc(urma_jfc_t* jfc) {
  if (!jfc || tp_state(jfc) == 0) return URMA_EINVAL;
  const urma_status_t s = urma_delete_jfc(jfc);
  if (s == URMA_SUCCESS) {
    tp_forget(jfc);
    std::lock_guard<std::mutex> l(g_tp_mu);
    g_jfc_pending.erase(jfc);
  }
  return s;
}

// ================================================================================================ JFS
urma_status_t urma_alloc_jfs(urma_context_t* ctx, urma_jfs_cfg_t* cfg, urma_jfs_t** jfs) {
  if (!ctx || !cfg || !jfs) return URMA_EINVAL;
  urma_jfs_t* j = urma_create_jfs(ctx, cfg);
  if (!j) return URMA_FAIL;
  if (urma_modify_jfs(j, URMA_JETTY_STATE_RESET) != URMA_SUCCESS) {
    urma_delete_jfs(j);
    return URMA_FAIL;
  }
  tp_track(j);
  *jfs = j;
  return URMA_SUCCESS;
}
static urma_status_t set_sq_opt(urma_jfs_cfg_t* c, uint64_t opt, void* buf, uint32_t len) {
  switch (opt) {
    case URMA_OPT_USER_CTX: return opt_in(buf, len, &c->user_ctx) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_PRIORITY: return opt_in(buf, len, &c->priority) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_RNR_RETRY: return opt_in(buf, len, &c->rnr_retry) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_ERR_TIMEOUT: return opt_in(buf, len, &c->err_timeout) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_DEPTH:
    case URMA_OPT_FLAG:
    case URMA_OPT_TRANS_MODE:
    case URMA_OPT_ID:
    case URMA_OPT_STATE: return URMA_ENOPERM;
    default: return URMA_EINVAL;
  }
}
static urma_status_t get_sq_opt(const urma_jfs_cfg_t* c, uint64_t opt, void* buf, uint32_t len) {
  switch (opt) {
    case URMA_OPT_DEPTH: return opt_out(buf, len, c->depth);
    case URMA_OPT_FLAG: return opt_out(buf, len, c->flag);
    case URMA_OPT_USER_CTX: return opt_out(buf, len, c->user_ctx);
    case URMA_OPT_TRANS_MODE: return opt_out<uint32_t>(buf, len, (uint32_t)c->trans_mode);
    case URMA_OPT_PRIORITY: return opt_out(buf, len, c->priority);
    case URMA_OPT_RNR_RETRY: return opt_out(buf, len, c->rnr_retry);
    case URMA_OPT_ERR_TIMEOUT: return opt_out(buf, len, c->err_timeout);
    default: return URMA_EINVAL;
  }
}
urma_status_t urma_set_jfs_opt(urma_jfs_t* jfs, uint64_t opt, void* buf, uint32_t len) {
  if (!jfs) return URMA_EINVAL;
  if (tp_state(jfs) != 1) return URMA_ENOPERM;
  return set_sq_opt(&jfs->cfg, opt, buf, len);
}
urma_status_t urma_get_jfs_opt(urma_jfs_t* jfs, uint64_t opt, void* buf, uint32_t len) {
  if (!jfs) return URMA_EINVAL;
  if (opt == URMA_OPT_ID) return opt_out(buf, len, jfs->jfs_id.id);
  if (opt == URMA_OPT_STATE) {
    urma_jfs_cfg_t c;
    urma_jetty_state_t st;
    if (urma_query_jfs(jfs, &c, &st) != URMA_SUCCESS) return URMA_FAIL;
    return opt_out<uint32_t>(buf, len, (uint32_t)st);
  }
  return get_sq_opt(&jfs->cfg, opt, buf, len);
}
urma_status_t urma_active_jfs(urma_jfs_t* jfs) {
  if (!jfs || tp_state(jfs) != 1) return URMA_EINVAL;
  const urma_status_t s = urma_modify_jfs(jfs, URMA_JETTY_STATE_READY);
  if (s == URMA_SUCCESS) tp_set_active(jfs, true);
  return s;
}
urma_status_t urma_deactive_jfs(urma_jfs_t* jfs) {
  if (!jfs || tp_state(jfs) != 2) return URMA_EINVAL;
  const urma_status_t s = urma_modify_jfs(jfs, URMA_JETTY_STATE_RESET);
  if (s == URMA_SUCCESS) tp_set_active(jfs, false);
  return s;
}
urma_status_t urma_free_jfs(urma_jfs_t* jfs) {
  if (!jfs || tp_state(jfs) == 0) return URMA_EINVAL;
  const urma_status_t s = urma_delete_jfs(jfs);
  if (s == URMA_SUCCESS) tp_forget(jfs);
  return s;
}

// ================================================================================================ JFR
urma_status_t urma_alloc_jfr(urma_context_t* ctx, urma_jfr_cfg_t* cfg, urma_jfr_t** jfr) {
  if (!ctx || !cfg || !jfr) return URMA_EINVAL;
  urma_jfr_t* j = urma_create_jfr(ctx, cfg);
  if (!j) return URMA_FAIL;
  if (urma_modify_jfr(j, URMA_JETTY_STATE_RESET, 0) != URMA_SUCCESS) {
    urma_delete_jfr(j);
    return URMA_FAIL;
  }
  tp_track(j);
  *jfr = j;
  return URMA_SUCCESS;
}
urma_status_t urma_set_jfr_opt(urma_jfr_t* jfr, uint64_t opt, void* buf, uint32_t len) {
  if (!jfr) return URMA_EINVAL;
  if (tp_state(jfr) != 1) return URMA_ENOPERM;
  switch (opt) {
    case URMA_OPT_USER_CTX: return opt_in(buf, len, &jfr->cfg.user_ctx) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_MIN_RNR_TIMER: return opt_in(buf, len, &jfr->cfg.min_rnr_timer) ? URMA_SUCCESS : URMA_EINVAL;
    case URMA_OPT_RX_THRESHOLD: {
      uint32_t v;
      if (!opt_in(buf, len, &v)) return URMA_EINVAL;
      std::lock_guard<std::mutex> l(g_tp_mu);
      g_jfr_threshold[jfr] = v;
      return URMA_SUCCESS;
    }
    case URMA_OPT_DEPTH:
    case URMA_OPT_FLAG:
    case URMA_OPT_TRANS_MODE:
    case URMA_OPT_ID:
    case URMA_OPT_STATE: return URMA_ENOPERM;
    default: return URMA_EINVAL;
  }
}
urma_status_t urma_get_jfr_opt(urma_jfr_t* jfr, uint64_t opt, void* buf, uint32_t len) {
  if (!jfr) return URMA_EINVAL;
  switch (opt) {
    case URMA_OPT_DEPTH: return opt_out(buf, len, jfr->cfg.depth);
    case URMA_OPT_FLAG: return opt_out(buf, len, jfr->cfg.flag);
    case URMA_OPT_USER_CTX: return opt_out(buf, len, jfr->cfg.user_ctx);
    case URMA_OPT_TRANS_MODE: return opt_out<uint32_t>(buf, len, (uint32_t)jfr->cfg.trans_mode);
    case URMA_OPT_MIN_RNR_TIMER: return opt_out(buf, len, jfr->cfg.min_rnr_timer);
    case URMA_OPT_ID: return opt_out(buf, len, jfr->jfr_id.id);
    case URMA_OPT_RX_THRESHOLD: {
      std::lock_guard<std::mutex> l(g_tp_mu);
      auto it = g_jfr_threshold.find(jfr);
      return opt_out<uint32_t>(buf, len, it == g_jfr_threshold.end() ? 0u : it->second);
    }
    case URMA_OPT_STATE: {
      urma_jfr_cfg_t c;
      urma_jetty_state_t st;
      if (urma_query_jfr(jfr, &c, &st) != URMA_SUCCESS) return URMA_FAIL;
      return opt_out<uint32_t>(buf, len, (uint32_t)st);
    }
    default: return URMA_EINVAL;
  }
}
urma_status_t urma_active_jfr(urma_jfr_t* jfr) {
  if (!jfr || tp_state(jfr) != 1) return URMA_EINVAL;
  uint32_t thr = 0;
  {
    std::lock_guard<std::mutex> l(g_tp_mu);
    auto it = g_jfr_threshold.find(jfr);
    if (it != g_jfr_threshold.end()) thr = it->second;
  }
  const urma_status_t s = urma_modify_jfr(jfr, URMA_JETTY_STATE_READY, thr);
  if (s == URMA_SUCCESS) tp_set_active(jfr, true);
  return s;
}
urma_status_t urma_deactive_jfr(urma_jfr_t* jfr) {
  if (!jfr || tp_state(jfr) != 2) return URMA_EINVAL;
  const urma_status_t s = urma_modify_jfr(jfr, URMA_JETTY_STATE_RESET, 0);
  if (s == URMA_SUCCESS) tp_set_active(jfr, false);
  return s;
}
urma_status_t urma_free_jfr(urma_jfr_t* jfr) {
  if (!jfr || tp_state(jfr) == 0) return URMA_EINVAL;
  const urma_status_t s = urma_delete_jfr(jfr);
  if (s == URMA_SUCCESS) {
    tp_forget(jfr);
    std::lock_guard<std::mutex> l(g_tp_mu);
    g_jfr_threshold.erase(jfr);
  }
  return s;
}

// ================================================================================================ Jetty
urma_status_t urma_alloc_jetty(urma_context_t* ctx, urma_jetty_cfg_t* cfg, urma_jetty_t** jetty) {
  if (!ctx || !cfg || !jetty) return URMA_EINVAL;
  urma_jetty_t* j = urma_create_jetty(ctx, cfg);
  if (!j) return URMA_FAIL;
  if (urma_modify_jetty(j, URMA_JETTY_STATE_RESET) != URMA_SUCCESS) {
    urma_delete_jetty(j);
    return URMA_FAIL;
  }
  tp_track(j);
  *jetty = j;
  return URMA_SUCCESS;
}
urma_status_t urma_set_jetty_opt(urma_jetty_t* jetty, uint64_t opt, void* buf, uint32_t len) {
  if (!jetty) return URMA_EINVAL;
  if (tp_state(jetty) != 1) return URMA_ENOPERM;
  if (opt == URMA_OPT_USER_CTX) return opt_in(buf, len, &jetty->cfg.user_ctx) ? URMA_SUCCESS : URMA_EINVAL;
  if (opt == URMA_OPT_MIN_RNR_TIMER)
    return opt_in(buf, len, &jetty->cfg.jfr_cfg.min_rnr_timer) ? URMA_SUCCESS : URMA_EINVAL;
  return set_sq_opt(&jetty->cfg.jfs_cfg, opt, buf, len);
}
urma_status_t urma_get_jetty_opt(urma_jetty_t* jetty, uint64_t opt, void* buf, uint32_t len) {
  if (!jetty) return URMA_EINVAL;
  if (opt == URMA_OPT_ID) return opt_out(buf, len, jetty->jetty_id.id);
  if (opt == URMA_OPT_USER_CTX) return opt_out(buf, len, jetty->cfg.user_ctx);
  if (opt == URMA_OPT_FLAG) return opt_out(buf, len, jetty->cfg.flag);
  if (opt == URMA_OPT_MIN_RNR_TIMER) return opt_out(buf, len, jetty->cfg.jfr_cfg.min_rnr_timer);
  if (opt == URMA_OPT_STATE) {
    urma_jetty_cfg_t c;
    urma_jetty_state_t st;
    if (urma_query_jetty(jetty, &c, &st) != URMA_SUCCESS) return URMA_FAIL;
    return opt_out<uint32_t>(buf, len, (uint32_t)st);
  }
  return get_sq_opt(&jetty->cfg.jfs_cfg, opt, buf, len);
}
urma_status_t urma_active_jetty(urma_jetty_t* jetty) {
  if (!jetty || tp_state(jetty) != 1) return URMA_EINVAL;
  const urma_status_t s = urma_modify_jetty(jetty, URMA_JETTY_STATE_READY);
  if (s == URMA_SUCCESS) tp_set_active(jetty, true);
  return s;
}
urma_status_t urma_deactive_jetty(urma_jetty_t* jetty) {
  if (!jetty || tp_state(jetty) != 2) return URMA_EINVAL;
  const urma_status_t s = urma_modify_jetty(jetty, URMA_JETTY_STATE_RESET);
  if (s == URMA_SUCCESS) tp_set_active(jetty, false);
  return s;
}
urma_status_t urma_free_jetty(urma_jetty_t* jetty) {
  if (!jetty || tp_state(jetty) == 0) return URMA_EINVAL;
  const urma_status_t s = urma_delete_jetty(jetty);
  if (s == URMA_SUCCESS) tp_forget(jetty);
  return s;
}

// ================================================================================================ batch deletion
#define UMDK_DELETE_BATCH(NAME, TYPE, DEL)                                      \
  urma_status_t NAME(TYPE** arr, int num, TYPE** bad) {                         \
    if (bad) *bad = nullptr;                                                    \
    if (!arr || num < 0) return URMA_EINVAL;                                    \
    for (int i = 0; i < num; ++i) {                                             \
      const urma_status_t s = arr[i] ? DEL(arr[i]) : URMA_EINVAL;               \
      if (s != URMA_SUCCESS) {                                                  \
        if (bad) *bad = arr[i];                                                 \
        return s;                                                               \
      }                                                                         \
      tp_forget(arr[i]);                                                        \
    }                                                                           \
    return URMA_SUCCESS;                                                        \
  }
UMDK_DELETE_BATCH(urma_delete_jfc_batch, urma_jfc_t, urma_delete_jfc)
UMDK_DELETE_BATCH(urma_delete_jfs_batch, urma_jfs_t, urma_delete_jfs)
UMDK_DELETE_BATCH(urma_delete_jfr_batch, urma_jfr_t, urma_delete_jfr)
UMDK_DELETE_BATCH(urma_delete_jetty_batch, urma_jetty_t, urma_delete_jetty)
#undef UMDK_DELETE_BATCH

// ================================================================================================ *_ex, async, notifiers
static bool path_known(urma_context_t* ctx, uint64_t handle) {
  if (handle == 0) return true;
  std::lock_guard<std::mutex> l(g_tpt_mu);
  auto it = g_tp_tables.find(ctx);
  return it != g_tp_tables.end() && it->second.by_handle.count(handle) != 0;
}
urma_target_jetty_t* urma_import_jetty_ex(urma_context_t* ctx, urma_rjetty_t* rjetty, urma_token_t* token_value,
                                          urma_import_jetty_ex_cfg_t* cfg) {
  if (cfg && !path_known(ctx, cfg->tp_handle)) return nullptr;  // a handle must come from urma_get_tp_list
  return urma_import_jetty(ctx, rjetty, token_value);
}
urma_target_jetty_t* urma_import_jfr_ex(urma_context_t* ctx, urma_rjfr_t* rjfr, urma_token_t* token_value,
                                        urma_import_jfr_ex_cfg_t* cfg) {
  if (cfg && !path_known(ctx, cfg->tp_handle)) return nullptr;
  return urma_import_jfr(ctx, rjfr, token_value);
}
urma_status_t urma_bind_jetty_ex(urma_jetty_t* jetty, urma_target_jetty_t* tjetty, urma_bind_jetty_ex_cfg_t* cfg) {
  if (!jetty) return URMA_EINVAL;
  if (cfg && !path_known(jetty->ctx, cfg->tp_handle)) return URMA_EINVAL;
  return urma_bind_jetty(jetty, tjetty);
}

urma_notifier_t* urma_create_notifier(urma_context_t* ctx) {
  if (!ctx) return nullptr;
  Notifier* n = new Notifier();
  n->pub.ctx = ctx;
  n->pub.fd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  n->pub.priv = n;
  if (n->pub.fd < 0) {
    delete n;
    return nullptr;
  }
  return &n->pub;
}
urma_status_t urma_delete_notifier(urma_notifier_t* notifier) {
  if (!notifier) return URMA_EINVAL;
  Notifier* n = static_cast<Notifier*>(notifier->priv);
  close(notifier->fd);
  delete n;
  return URMA_SUCCESS;
}
urma_target_jetty_t* urma_import_jetty_async(urma_notifier_t* notifier, const urma_rjetty_t* rjetty,
                                             const urma_token_t* token_value, uint64_t user_ctx, int) {
  if (!notifier || !rjetty) return nullptr;
  urma_target_jetty_t* t = urma_import_jetty(notifier->ctx, rjetty, token_value);
  urma_notify_t ev{};
  ev.type = URMA_IMPORT_JETTY_NOTIFY;
  ev.status = t ? URMA_SUCCESS : URMA_FAIL;
  ev.user_ctx = user_ctx;
  ev.tjetty = t;
  notifier_push(notifier, ev);
  return t;
}
urma_status_t urma_unimport_jetty_async(urma_target_jetty_t* tjetty) { return urma_unimport_jetty(tjetty); }
urma_status_t urma_bind_jetty_async(urma_notifier_t* notifier, urma_jetty_t* jetty, urma_target_jetty_t* tjetty,
                                    uint64_t user_ctx, int) {
  if (!notifier || !jetty || !tjetty) return URMA_EINVAL;
  urma_notify_t ev{};
  ev.type = URMA_BIND_JETTY_NOTIFY;
  ev.status = urma_bind_jetty(jetty, tjetty);
  ev.user_ctx = user_ctx;
  ev.jetty = jetty;
  notifier_push(notifier, ev);
  return URMA_SUCCESS;  // the outcome is in the notification
}
urma_status_t urma_unbind_jetty_async(urma_jetty_t* jetty) { return urma_unbind_jetty(jetty); }
urma_status_t urma_advise_jfr_async(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_advise_async_cb_func cb_fun,
                                    void* cb_arg) {
  if (!jfs || !tjfr) return URMA_EINVAL;
  const urma_status_t s = urma_advise_jfr(jfs, tjfr);
  if (cb_fun) cb_fun(s, cb_arg);
  return URMA_SUCCESS;
}
int urma_wait_notify(urma_notifier_t* notifier, uint32_t cnt, urma_notify_t* notify, int timeout) {
  if (!notifier || !notify || cnt == 0) return -1;
  Notifier* n = static_cast<Notifier*>(notifier->priv);
  for (int round = 0; round < 2; ++round) {
    {
      std::lock_guard<std::mutex> l(n->mu);
      uint32_t got = 0;
      while (got < cnt && !n->q.empty()) {
        notify[got++] = n->q.front();
        n->q.pop_front();
      }
      if (got) {
        uint64_t drained;
        if (n->q.empty() && read(notifier->fd, &drained, sizeof(drained)) < 0) {
          // nothing to drain: another waiter already did
        }
        return (int)got;
      }
    }
    if (round == 1) break;
    pollfd pf{notifier->fd, POLLIN, 0};
    if (poll(&pf, 1, timeout) <= 0) return 0;
  }
  return 0;
}
urma_status_t urma_ack_notify(urma_context_t* ctx, uint32_t cnt, urma_notify_t* notify) {
  // notifications are copied out by urma_wait_notify and hold no resources
  return (ctx && (notify || cnt == 0)) ? URMA_SUCCESS : URMA_EINVAL;
}

// ================================================================================================ peer descriptions
urma_status_t urma_get_rjetty(urma_jetty_t* jetty, urma_rjetty_t** rjetty, uint32_t* length) {
  if (!jetty || !rjetty) return URMA_EINVAL;
  urma_rjetty_t* r = new urma_rjetty_t();
  r->jetty_id = jetty->jetty_id;
  r->trans_mode = jetty->cfg.jfs_cfg.trans_mode;
  r->type = 1;
  *rjetty = r;
  if (length) *length = sizeof(urma_rjetty_t);
  return URMA_SUCCESS;
}
void urma_put_rjetty(urma_rjetty_t* rjetty) { delete rjetty; }
urma_status_t urma_get_seg_ctx(urma_target_seg_t* tseg, urma_seg_t** seg, uint32_t* size) {
  if (!tseg || !seg) return URMA_EINVAL;
  *seg = new urma_seg_t(tseg->seg);
  if (size) *size = sizeof(urma_seg_t);
  return URMA_SUCCESS;
}
void urma_put_seg_ctx(urma_seg_t* seg) { delete seg; }
urma_token_id_t* urma_alloc_token_id_ex(urma_context_t* ctx, urma_token_id_flag_t) {
  // every token id here may cover several segments, so the flag asks for nothing extra
  return urma_alloc_token_id(ctx);
}
urma_status_t urma_set_context_opt(urma_context_t* ctx, urma_opt_name_t opt_name, const void* opt_value,
                                   size_t opt_len) {
  if (!ctx || !opt_value) return URMA_EINVAL;
  std::lock_guard<std::mutex> l(g_tpt_mu);
  CtxOpts& o = g_ctx_opts[ctx];
  switch (opt_name) {
    case URMA_OPT_CTX_LOG_TAG:
      o.log_tag.assign(static_cast<const char*>(opt_value), strnlen(static_cast<const char*>(opt_value), opt_len));
      urma_log_set_thread_tag(o.log_tag.c_str());
      return URMA_SUCCESS;
    case URMA_OPT_CTX_USER_DATA:
      if (opt_len < sizeof(uint64_t)) return URMA_EINVAL;
      memcpy(&o.user_data, opt_value, sizeof(uint64_t));
      return URMA_SUCCESS;
    default: return URMA_EINVAL;
  }
}

// ================================================================================================ transport paths
int urma_get_tpn(urma_jetty_t* jetty) {
  if (!jetty) return -1;
  // a bound (RC) jetty owns one transport path, numbered after the jetty; unbound jetties share path 0
  return jetty->remote_jetty ? (int)jetty->jetty_id.id : 0;
}
urma_status_t urma_get_tp_list(urma_context_t* ctx, urma_get_tp_cfg_t* cfg, uint32_t* tp_cnt,
                               urma_tp_info_t* tp_list) {
  if (!ctx || !cfg || !tp_cnt || !tp_list || *tp_cnt == 0) return URMA_EINVAL;
  TpKey k{cfg->local_eid, cfg->peer_eid, (uint32_t)cfg->trans_mode};
  std::lock_guard<std::mutex> l(g_tpt_mu);
  TpTable& t = g_tp_tables[ctx];
  auto it = t.by_key.find(k);
  if (it == t.by_key.end()) {
    const uint64_t h = ((uint64_t)ctx->uasid << 32) | t.next++;
    it = t.by_key.emplace(k, h).first;
    TpEntry e;
    e.handle = h;
    memcpy(e.value.sip, cfg->local_eid.raw, URMA_IP_ADDR_BYTES);
    memcpy(e.value.dip, cfg->peer_eid.raw, URMA_IP_ADDR_BYTES);
    eid_to_mac(&cfg->local_eid, e.value.sma);
    eid_to_mac(&cfg->peer_eid, e.value.dma);
    e.value.ttl = 64;
    e.bitmap = URMA_TP_ATTR_SIP | URMA_TP_ATTR_DIP | URMA_TP_ATTR_SMA | URMA_TP_ATTR_DMA | URMA_TP_ATTR_TTL;
    t.by_handle[h] = e;
  }
  tp_list[0].tp_handle = it->second;
  *tp_cnt = 1;
  return URMA_SUCCESS;
}
urma_status_t urma_set_tp_attr(const urma_context_t* ctx, const uint64_t tp_handle, const uint8_t tp_attr_cnt,
                               const uint32_t tp_attr_bitmap, const urma_tp_attr_value_t* tp_attr) {
  if (!ctx || !tp_attr || tp_attr_cnt != __builtin_popcount(tp_attr_bitmap)) return URMA_EINVAL;
  std::lock_guard<std::mutex> l(g_tpt_mu);
  auto t = g_tp_tables.find(ctx);
  if (t == g_tp_tables.end()) return URMA_EINVAL;
  auto it = t->second.by_handle.find(tp_handle);
  if (it == t->second.by_handle.end()) return URMA_EINVAL;
  urma_tp_attr_value_t& v = it->second.value;
  if (tp_attr_bitmap & URMA_TP_ATTR_RETRY) v.retry_times_init = tp_attr->retry_times_init;
  if (tp_attr_bitmap & URMA_TP_ATTR_AT) v.at = tp_attr->at, v.at_times = tp_attr->at_times;
  if (tp_attr_bitmap & URMA_TP_ATTR_SIP) memcpy(v.sip, tp_attr->sip, sizeof(v.sip));
  if (tp_attr_bitmap & URMA_TP_ATTR_DIP) memcpy(v.dip, tp_attr->dip, sizeof(v.dip));
  if (tp_attr_bitmap & URMA_TP_ATTR_SMA) memcpy(v.sma, tp_attr->sma, sizeof(v.sma));
  if (tp_attr_bitmap & URMA_TP_ATTR_DMA) memcpy(v.dma, tp_attr->dma, sizeof(v.dma));
  if (tp_attr_bitmap & URMA_TP_ATTR_VLAN) v.vlan_id = tp_attr->vlan_id, v.vlan_en = tp_attr->vlan_en;
  if (tp_attr_bitmap & URMA_TP_ATTR_DSCP) v.dscp = tp_attr->dscp;
  if (tp_attr_bitmap & URMA_TP_ATTR_SL) v.sl = tp_attr->sl;
  if (tp_attr_bitmap & URMA_TP_ATTR_TTL) v.ttl = tp_attr->ttl;
  if (tp_attr_bitmap & URMA_TP_ATTR_UDP_PORTS)
    v.ack_udp_srcport = tp_attr->ack_udp_srcport, v.data_udp_srcport = tp_attr->data_udp_srcport;
  it->second.bitmap |= tp_attr_bitmap;
  return URMA_SUCCESS;
}
urma_status_t urma_get_tp_attr(const urma_context_t* ctx, const uint64_t tp_handle, uint8_t* tp_attr_cnt,
                               uint32_t* tp_attr_bitmap, urma_tp_attr_value_t* tp_attr) {
  if (!ctx || !tp_attr_cnt || !tp_attr_bitmap || !tp_attr) return URMA_EINVAL;
  std::lock_guard<std::mutex> l(g_tpt_mu);
  auto t = g_tp_tables.find(ctx);
  if (t == g_tp_tables.end()) return URMA_EINVAL;
  auto it = t->second.by_handle.find(tp_handle);
  if (it == t->second.by_handle.end()) return URMA_EINVAL;
  *tp_attr = it->second.value;
  *tp_attr_bitmap = it->second.bitmap;
  *tp_attr_cnt = (uint8_t)__builtin_popcount(it->second.bitmap);
  return URMA_SUCCESS;
}
int urma_modify_tp(urma_context_t* ctx, uint32_t tpn, urma_tp_cfg_t* cfg, urma_tp_attr_t* attr,
                   urma_tp_attr_mask_t mask) {
  if (!ctx || !cfg || !attr) return -1;
  urma_get_tp_cfg_t g{0, cfg->trans_mode, cfg->local_eid, cfg->peer_eid};
  urma_tp_info_t info;
  uint32_t n = 1;
  if (urma_get_tp_list(ctx, &g, &n, &info) != URMA_SUCCESS) return -1;
  std::lock_guard<std::mutex> l(g_tpt_mu);
  TpEntry& e = g_tp_tables[ctx].by_handle[info.tp_handle];
  (void)tpn;
  if (mask & 1u) e.attr.peer_tpn = attr->peer_tpn;
  if (mask & 2u) e.attr.state = attr->state;
  if (mask & 4u) e.attr.tx_psn = attr->tx_psn;
  if (mask & 8u) e.attr.rx_psn = attr->rx_psn;
  if (mask & 16u) e.attr.mtu = attr->mtu;
  *attr = e.attr;
  return 0;
}

// ================================================================================================ addressing
urma_net_addr_info_t* urma_get_net_addr_list(urma_context_t* ctx, uint32_t* cnt) {
  if (!ctx || !cnt) return nullptr;
  urma_net_addr_info_t* a = new urma_net_addr_info_t[1]();
  urma_get_ip_by_eid(ctx, &ctx->eid, &a[0].netaddr);
  a[0].index = ctx->eid_index;
  *cnt = 1;
  return a;
}
void urma_free_net_addr_list(urma_net_addr_info_t* net_addr_list) { delete[] net_addr_list; }
urma_status_t urma_get_eid_by_ip(const urma_context_t* ctx, const urma_net_addr_t* net_addr, urma_eid_t* eid) {
  if (!ctx || !net_addr || !eid) return URMA_EINVAL;
  if (net_addr->sin_family != 10 /* AF_INET6 */) return URMA_EINVAL;
  memcpy(eid->raw, net_addr->addr, URMA_EID_SIZE);
  return URMA_SUCCESS;
}
urma_status_t urma_get_ip_by_eid(const urma_context_t* ctx, const urma_eid_t* eid, urma_net_addr_t* net_addr) {
  if (!ctx || !eid || !net_addr) return URMA_EINVAL;
  memset(net_addr, 0, sizeof(*net_addr));
  net_addr->sin_family = 10;  // AF_INET6: the 128-bit EID is the address
  memcpy(net_addr->addr, eid->raw, URMA_EID_SIZE);
  eid_to_mac(eid, net_addr->mac);
  net_addr->prefix_len = 128;
  return URMA_SUCCESS;
}
urma_status_t urma_get_smac(const urma_context_t* ctx, uint8_t* mac) {
  if (!ctx || !mac) return URMA_EINVAL;
  eid_to_mac(&ctx->eid, mac);
  return URMA_SUCCESS;
}
urma_status_t urma_get_dmac(const urma_context_t* ctx, const urma_net_addr_t* net_addr, uint8_t* mac) {
  if (!ctx || !net_addr || !mac) return URMA_EINVAL;
  urma_eid_t eid;
  if (urma_get_eid_by_ip(ctx, net_addr, &eid) != URMA_SUCCESS) return URMA_EINVAL;
  eid_to_mac(&eid, mac);
  return URMA_SUCCESS;
}

}  // extern "C"
