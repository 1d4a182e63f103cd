// URMA core: provider registry, device list, argument validation and reference counting around the provider
// vtable, thin data-plane dispatch with optional latency sampling, logging.
//
// Reference behaviour reproduced here (files under src/urma/lib/urma/core/):
//   urma_main.c:161-255   urma_init loads every liburma*.so found in the provider directory; providers register
//                         themselves from a constructor; the device list is the merge of all providers' devices
//   urma_cp_api.c         every control call validates its arguments, bumps a reference count on the parent object
//                         and forwards to ctx->ops; 3025-3050: segment access rules (LOCAL_ONLY exclusive,
//                         WRITE requires READ, ATOMIC requires READ and WRITE)
//   urma_dp_api.c:133-396 urma_write/read/send/recv build a single-SGE work request; post/poll forward to ops with
//                         perf sampling hooks around them
#include <dirent.h>
#include <dlfcn.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <syslog.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "ub_util.h"
#include "urma_api.h"
#include "urma_provider.h"

namespace {

struct Core {
  std::mutex mu;
  bool inited = false;
  urma_init_attr_t attr{};
  std::vector<const urma_provider_ops_t*> providers;
  std::vector<void*> dl_handles;
  std::vector<urma_device_t*> devices;  // owned
  std::vector<const urma_provider_ops_t*> device_provider;
};
Core& core() {
  static Core c;
  return c;
}

// ------------------------------------------------------------------------------------------------ logging
std::atomic<int> g_log_level{URMA_VLOG_LEVEL_WARNING};
urma_log_cb_t g_log_cb = nullptr;
urma_loc_log_cb g_loc_log_cb = nullptr;
thread_local char t_tag[32] = "";
std::atomic<uint64_t> g_last_log_ns{0};
std::atomic<uint32_t> g_suppressed{0};

void init_log_level_from_env() {
  const char* e = getenv("URMA_LOG_LEVEL");
  if (e && *e) {
    const int v = atoi(e);
    if (v >= URMA_VLOG_LEVEL_EMERG && v <= URMA_VLOG_LEVEL_DEBUG) g_log_level = v;
  }
}

// ------------------------------------------------------------------------------------------------ perf
struct PerfState {
  std::atomic<bool> on{false};
  std::mutex mu;
  ub::PerfHist hist[URMA_PERF_OP_MAX];
};
PerfState& perf() {
  static PerfState p;
  return p;
}
struct PerfScope {
  urma_perf_op_t op;
  uint64_t t0;
  explicit PerfScope(urma_perf_op_t o) : op(o), t0(perf().on.load(std::memory_order_relaxed) ? ub::now_ns() : 0) {}
  ~PerfScope() {
    if (t0) {
      const uint64_t dt = ub::now_ns() - t0;
      std::lock_guard<std::mutex> l(perf().mu);
      perf().hist[op].add(dt);
    }
  }
};
const char* kPerfNames[URMA_PERF_OP_MAX] = {"write", "read", "send", "recv", "post_jfs_wr", "post_jfr_wr",
                                            "post_jetty_send_wr", "post_jetty_recv_wr", "poll_jfc"};

bool access_ok(uint32_t a) {
  if (a == 0) return false;
  if (a & URMA_ACCESS_LOCAL_ONLY) return a == URMA_ACCESS_LOCAL_ONLY;
  if ((a & URMA_ACCESS_WRITE) && !(a & URMA_ACCESS_READ)) return false;
  if ((a & URMA_ACCESS_ATOMIC) && ((a & (URMA_ACCESS_READ | URMA_ACCESS_WRITE)) != (URMA_ACCESS_READ | URMA_ACCESS_WRITE)))
    return false;
  return true;
}

void ctx_get(urma_context_t* c) { __atomic_add_fetch(&c->refcnt, 1, __ATOMIC_RELAXED); }
void ctx_put(urma_context_t* c) { __atomic_sub_fetch(&c->refcnt, 1, __ATOMIC_RELAXED); }

void load_plugins(const char* dir) {
  if (!dir || !*dir) return;
  DIR* d = opendir(dir);
  if (!d) return;
  while (dirent* e = readdir(d)) {
    const char* n = e->d_name;
    if (strncmp(n, "liburma-", 8) != 0 || !strstr(n, ".so")) continue;
    const std::string path = std::string(dir) + "/" + n;
    void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      urma_log(URMA_VLOG_LEVEL_WARNING, __func__, __LINE__, "dlopen(%s) failed: %s", path.c_str(), dlerror());
      continue;
    }
    core().dl_handles.push_back(h);  // the plug-in's constructor has called urma_register_provider_ops
  }
  closedir(d);
}

}  // namespace

// ================================================================================================ logging API
extern "C" {

void urma_log(int level, const char* func, int line, const char* fmt, ...) {
  if (level > g_log_level.load(std::memory_order_relaxed)) return;
  // rate limit: at most one message per 100 us burst window, count the rest
  const uint64_t now = ub::now_ns();
  const uint64_t last = g_last_log_ns.load(std::memory_order_relaxed);
  if (level >= URMA_VLOG_LEVEL_WARNING && now - last < 100000 && last != 0) {
    g_suppressed.fetch_add(1, std::memory_order_relaxed);
    return;
  }
  g_last_log_ns.store(now, std::memory_order_relaxed);
  char msg[1024];
  const char* sep = getenv("URMA_LOG_SEPARATOR");
  int off = snprintf(msg, sizeof(msg), "URMA%s%s%s%s:%d%s", sep ? sep : "|", t_tag, sep ? sep : "|", func, line,
                     sep ? sep : "|");
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg + off, sizeof(msg) - off, fmt, ap);
  va_end(ap);
  if (g_loc_log_cb) {
    g_loc_log_cb(level, func, line, msg + off);
  } else if (g_log_cb) {
    g_log_cb(level, msg);
  } else {
    syslog(level, "%s", msg);
    if (getenv("URMA_LOG_STDERR")) fprintf(stderr, "%s\n", msg);
  }
}

urma_status_t urma_register_log_func(urma_log_cb_t func) {
  if (!func) return URMA_EINVAL;
  g_log_cb = func;
  return URMA_SUCCESS;
}
urma_status_t urma_unregister_log_func(void) {
  g_log_cb = nullptr;
  return URMA_SUCCESS;
}
urma_vlog_level_t urma_log_get_level(void) { return static_cast<urma_vlog_level_t>(g_log_level.load()); }
void urma_log_set_level(urma_vlog_level_t level) {
  if (level >= URMA_VLOG_LEVEL_EMERG && level <= URMA_VLOG_LEVEL_DEBUG) g_log_level = level;
}
void urma_log_set_thread_tag(const char* tag) { snprintf(t_tag, sizeof(t_tag), "%s", tag ? tag : ""); }
const char* urma_log_get_thread_tag(void) { return t_tag; }
urma_status_t urma_register_loc_log_func(urma_loc_log_cb func) {
  g_loc_log_cb = func;  // NULL goes back to the plain callback / syslog
  return URMA_SUCCESS;
}

// ================================================================================================ perf API
urma_status_t urma_start_perf(void) {
  std::lock_guard<std::mutex> l(perf().mu);
  for (auto& h : perf().hist) h.reset();
  perf().on = true;
  return URMA_SUCCESS;
}
urma_status_t urma_stop_perf(void) {
  perf().on = false;
  return URMA_SUCCESS;
}
urma_status_t urma_get_perf_info(urma_perf_entry_t* entries, char* text, uint32_t* text_len) {
  std::lock_guard<std::mutex> l(perf().mu);
  ub::DString s;
  s.printf("%-20s %10s %10s %10s %10s %10s %10s %10s\n", "op", "count", "avg_ns", "min_ns", "max_ns", "p90", "p99",
           "p99.99");
  for (int i = 0; i < URMA_PERF_OP_MAX; ++i) {
    const ub::PerfHist& h = perf().hist[i];
    urma_perf_entry_t e{h.count(), h.min(), h.max(), static_cast<uint64_t>(h.mean()), h.quantile(0.90),
                        h.quantile(0.99), h.quantile(0.9999)};
    if (entries) entries[i] = e;
    if (h.count())
      s.printf("%-20s %10llu %10llu %10llu %10llu %10llu %10llu %10llu\n", kPerfNames[i],
               (unsigned long long)e.count, (unsigned long long)e.avg_ns, (unsigned long long)e.min_ns,
               (unsigned long long)e.max_ns, (unsigned long long)e.p90_ns, (unsigned long long)e.p99_ns,
               (unsigned long long)e.p9999_ns);
  }
  if (text && text_len && *text_len > 0) {
    const size_t n = std::min<size_t>(*text_len - 1, s.str().size());
    memcpy(text, s.c_str(), n);
    text[n] = '\0';
    *text_len = static_cast<uint32_t>(n);
  }
  return URMA_SUCCESS;
}

// ================================================================================================ providers
int urma_register_provider_ops(const urma_provider_ops_t* ops) {
  if (!ops || !ops->name) return -1;
  std::lock_guard<std::mutex> l(core().mu);
  for (auto* p : core().providers)
    if (p == ops || strcmp(p->name, ops->name) == 0) return 0;
  core().providers.push_back(ops);
  return 0;
}
int urma_unregister_provider_ops(const urma_provider_ops_t* ops) {
  std::lock_guard<std::mutex> l(core().mu);
  auto& v = core().providers;
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i] == ops) {
      v.erase(v.begin() + i);
      return 0;
    }
  return -1;
}

// ================================================================================================ lifecycle
urma_status_t urma_init(const urma_init_attr_t* attr) {
  init_log_level_from_env();
  Core& c = core();
  {
    std::lock_guard<std::mutex> l(c.mu);
    if (c.inited) return URMA_EEXIST;
    if (attr) c.attr = *attr;
  }
  // plug-in providers: <dir of this library>/urma, $URMA_PROVIDER_PATH, attr->provider_dir
  Dl_info info;
  if (dladdr(reinterpret_cast<void*>(&urma_init), &info) && info.dli_fname) {
    std::string p(info.dli_fname);
    const size_t slash = p.rfind('/');
    if (slash != std::string::npos) load_plugins((p.substr(0, slash) + "/urma").c_str());
  }
  load_plugins(getenv("URMA_PROVIDER_PATH"));
  if (attr && attr->provider_dir) load_plugins(attr->provider_dir);

  std::vector<const urma_provider_ops_t*> provs;
  {
    std::lock_guard<std::mutex> l(c.mu);
    provs = c.providers;
  }
  for (auto* p : provs) {
    if (p->init && p->init(attr) != URMA_SUCCESS) {
      urma_log(URMA_VLOG_LEVEL_WARNING, __func__, __LINE__, "provider %s failed to initialise", p->name);
      continue;
    }
    urma_device_t tmp[64];
    const int n = p->get_devices ? p->get_devices(tmp, 64) : 0;
    std::lock_guard<std::mutex> l(c.mu);
    for (int i = 0; i < n && i < 64; ++i) {
      urma_device_t* d = new urma_device_t(tmp[i]);
      d->index = static_cast<uint32_t>(c.devices.size());
      snprintf(d->provider, sizeof(d->provider), "%s", p->name);
      c.devices.push_back(d);
      c.device_provider.push_back(p);
    }
  }
  std::lock_guard<std::mutex> l(c.mu);
  c.inited = true;
  return URMA_SUCCESS;
}

urma_status_t urma_uninit(void) {
  Core& c = core();
  std::vector<const urma_provider_ops_t*> provs;
  {
    std::lock_guard<std::mutex> l(c.mu);
    if (!c.inited) return URMA_FAIL;
    provs = c.providers;
    c.inited = false;
  }
  for (auto* p : provs)
    if (p->uninit) p->uninit();
  std::lock_guard<std::mutex> l(c.mu);
  for (auto* d : c.devices) delete d;
  c.devices.clear();
  c.device_provider.clear();
  return URMA_SUCCESS;
}

// ================================================================================================ devices
urma_device_t** urma_get_device_list(int* num) {
  Core& c = core();
  std::lock_guard<std::mutex> l(c.mu);
  if (!c.inited) {
    if (num) *num = 0;
    return nullptr;
  }
  urma_device_t** list = static_cast<urma_device_t**>(calloc(c.devices.size() + 1, sizeof(urma_device_t*)));
  for (size_t i = 0; i < c.devices.size(); ++i) list[i] = c.devices[i];
  if (num) *num = static_cast<int>(c.devices.size());
  return list;
}
void urma_free_device_list(urma_device_t** list) { free(list); }
urma_device_t* urma_get_device_by_name(const char* name) {
  if (!name) return nullptr;
  Core& c = core();
  std::lock_guard<std::mutex> l(c.mu);
  for (auto* d : c.devices)
    if (strcmp(d->name, name) == 0) return d;
  return nullptr;
}
urma_device_t* urma_get_device_by_eid(urma_eid_t eid) {
  Core& c = core();
  std::lock_guard<std::mutex> l(c.mu);
  for (auto* d : c.devices)
    if (memcmp(d->eid.raw, eid.raw, URMA_EID_SIZE) == 0) return d;
  return nullptr;
}
urma_status_t urma_query_device(urma_device_t* dev, urma_device_attr_t* attr) {
  if (!dev || !attr) return URMA_EINVAL;
  Core& c = core();
  const urma_provider_ops_t* p = nullptr;
  {
    std::lock_guard<std::mutex> l(c.mu);
    if (dev->index >= c.devices.size() || c.devices[dev->index] != dev) return URMA_EINVAL;
    p = c.device_provider[dev->index];
  }
  return p->query_device ? p->query_device(dev, attr) : URMA_FAIL;
}
extern "C" int urma_eid_table_get(const char* dev_name, urma_eid_info_t* out, int max);
extern "C" int urma_eid_table_claim(const char* dev_name);

// Index 0 is the EID the provider reports; indexes 1..8 are EIDs an administrator added (urma_admin eid add).
urma_eid_info_t* urma_get_eid_list(urma_device_t* dev, uint32_t* cnt) {
  if (!dev || !cnt) return nullptr;
  urma_eid_info_t* l = static_cast<urma_eid_info_t*>(calloc(9, sizeof(urma_eid_info_t)));
  l[0].eid = dev->eid;
  l[0].eid_index = 0;
  *cnt = 1 + static_cast<uint32_t>(urma_eid_table_get(dev->name, l + 1, 8));
  return l;
}
void urma_free_eid_list(urma_eid_info_t* list) { free(list); }

int urma_str_to_eid(const char* s, urma_eid_t* eid) {
  if (!s || !eid) return -1;
  // 32 hex digits, optionally separated by ':' every 4 digits
  uint8_t out[URMA_EID_SIZE];
  int n = 0;
  int hi = -1;
  for (const char* p = s; *p; ++p) {
    if (*p == ':') continue;
    int v;
    if (*p >= '0' && *p <= '9') v = *p - '0';
    else if (*p >= 'a' && *p <= 'f') v = *p - 'a' + 10;
    else if (*p >= 'A' && *p <= 'F') v = *p - 'A' + 10;
    else return -1;
    if (hi < 0) hi = v;
    else {
      if (n >= URMA_EID_SIZE) return -1;
      out[n++] = static_cast<uint8_t>(hi << 4 | v);
      hi = -1;
    }
  }
  if (n != URMA_EID_SIZE || hi >= 0) return -1;
  memcpy(eid->raw, out, URMA_EID_SIZE);
  return 0;
}
void urma_eid_to_str(const urma_eid_t* eid, char* buf, size_t len) {
  if (!eid || !buf || len == 0) return;
  size_t off = 0;
  for (int i = 0; i < URMA_EID_SIZE && off + 3 < len; ++i) {
    off += snprintf(buf + off, len - off, "%02x", eid->raw[i]);
    if ((i & 1) && i != URMA_EID_SIZE - 1 && off + 1 < len) buf[off++] = ':';
  }
  buf[off < len ? off : len - 1] = '\0';
}

// ================================================================================================ context
urma_context_t* urma_create_context(urma_device_t* dev, uint32_t eid_index) {
  if (!dev) return nullptr;
  Core& c = core();
  const urma_provider_ops_t* p = nullptr;
  {
    std::lock_guard<std::mutex> l(c.mu);
    if (!c.inited || dev->index >= c.devices.size() || c.devices[dev->index] != dev) return nullptr;
    p = c.device_provider[dev->index];
  }
  if (!p->create_context) return nullptr;
  urma_eid_t extra{};
  if (eid_index > 0) {   // an EID added by the administrator: it must exist
    urma_eid_info_t l[8];
    const int n = urma_eid_table_get(dev->name, l, 8);
    bool found = false;
    for (int i = 0; i < n; ++i)
      if (l[i].eid_index == eid_index) {
        extra = l[i].eid;
        found = true;
      }
    if (!found) {
      urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "%s has no EID with index %u", dev->name, eid_index);
      return nullptr;
    }
  }
  if (!urma_eid_table_claim(dev->name)) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "%s is exclusive and held by another process", dev->name);
    return nullptr;
  }
  // the provider only knows its own EID (index 0); an added EID is attached to the context here
  urma_context_t* ctx = p->create_context(dev, 0);
  if (ctx) {
    ctx->dev = dev;
    ctx->refcnt = 1;
    if (eid_index > 0) {
      ctx->eid = extra;
      ctx->eid_index = eid_index;
    }
  }
  return ctx;
}
urma_status_t urma_delete_context(urma_context_t* ctx) {
  if (!ctx) return URMA_EINVAL;
  if (__atomic_load_n(&ctx->refcnt, __ATOMIC_RELAXED) > 1) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "context still has %d child objects", ctx->refcnt - 1);
    return URMA_EAGAIN;
  }
  Core& c = core();
  const urma_provider_ops_t* p = nullptr;
  {
    std::lock_guard<std::mutex> l(c.mu);
    if (ctx->dev && ctx->dev->index < c.devices.size()) p = c.device_provider[ctx->dev->index];
  }
  if (!p || !p->delete_context) return URMA_FAIL;
  return p->delete_context(ctx);
}
uint32_t urma_get_uasid(urma_context_t* ctx) { return ctx ? ctx->uasid : 0; }

#define CTX_OP(ctx, op) ((ctx) && (ctx)->ops && (ctx)->ops->op)

// ================================================================================================ JFC / JFCE
urma_jfc_t* urma_create_jfc(urma_context_t* ctx, const urma_jfc_cfg_t* cfg) {
  if (!cfg || cfg->depth == 0 || !CTX_OP(ctx, create_jfc)) return nullptr;
  if (cfg->jfce && cfg->jfce->ctx != ctx) return nullptr;
  urma_jfc_t* j = ctx->ops->create_jfc(ctx, cfg);
  if (j) {
    j->ctx = ctx;
    j->cfg = *cfg;
    j->refcnt = 1;
    ctx_get(ctx);
  }
  return j;
}
urma_status_t urma_modify_jfc(urma_jfc_t* jfc, uint32_t count, uint32_t period) {
  if (!jfc || !CTX_OP(jfc->ctx, modify_jfc)) return URMA_EINVAL;
  return jfc->ctx->ops->modify_jfc(jfc, count, period);
}
urma_status_t urma_delete_jfc(urma_jfc_t* jfc) {
  if (!jfc || !CTX_OP(jfc->ctx, delete_jfc)) return URMA_EINVAL;
  if (__atomic_load_n(&jfc->refcnt, __ATOMIC_RELAXED) > 1) return URMA_EAGAIN;  // still bound to a JFS/JFR/Jetty
  urma_context_t* ctx = jfc->ctx;
  const urma_status_t s = ctx->ops->delete_jfc(jfc);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}
urma_jfce_t* urma_create_jfce(urma_context_t* ctx) {
  if (!CTX_OP(ctx, create_jfce)) return nullptr;
  urma_jfce_t* e = ctx->ops->create_jfce(ctx);
  if (e) {
    e->ctx = ctx;
    ctx_get(ctx);
  }
  return e;
}
urma_status_t urma_delete_jfce(urma_jfce_t* jfce) {
  if (!jfce || !CTX_OP(jfce->ctx, delete_jfce)) return URMA_EINVAL;
  urma_context_t* ctx = jfce->ctx;
  const urma_status_t s = ctx->ops->delete_jfce(jfce);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}

static void jfc_get(urma_jfc_t* j) {
  if (j) __atomic_add_fetch(&j->refcnt, 1, __ATOMIC_RELAXED);
}
static void jfc_put(urma_jfc_t* j) {
  if (j) __atomic_sub_fetch(&j->refcnt, 1, __ATOMIC_RELAXED);
}

// ================================================================================================ JFS
urma_jfs_t* urma_create_jfs(urma_context_t* ctx, const urma_jfs_cfg_t* cfg) {
  if (!cfg || cfg->depth == 0 || !cfg->jfc || cfg->jfc->ctx != ctx || !CTX_OP(ctx, create_jfs)) return nullptr;
  urma_jfs_t* j = ctx->ops->create_jfs(ctx, cfg);
  if (j) {
    j->ctx = ctx;
    j->cfg = *cfg;
    ctx_get(ctx);
    jfc_get(cfg->jfc);
  }
  return j;
}
urma_status_t urma_modify_jfs(urma_jfs_t* jfs, urma_jetty_state_t state) {
  if (!jfs || !CTX_OP(jfs->ctx, modify_jfs)) return URMA_EINVAL;
  return jfs->ctx->ops->modify_jfs(jfs, state);
}
urma_status_t urma_query_jfs(urma_jfs_t* jfs, urma_jfs_cfg_t* cfg, urma_jetty_state_t* state) {
  if (!jfs || !cfg || !state || !CTX_OP(jfs->ctx, query_jfs)) return URMA_EINVAL;
  return jfs->ctx->ops->query_jfs(jfs, cfg, state);
}
int urma_flush_jfs(urma_jfs_t* jfs, int cr_cnt, urma_cr_t* cr) {
  if (!jfs || cr_cnt <= 0 || !cr || !CTX_OP(jfs->ctx, flush_jfs)) return -1;
  return jfs->ctx->ops->flush_jfs(jfs, cr_cnt, cr);
}
urma_status_t urma_delete_jfs(urma_jfs_t* jfs) {
  if (!jfs || !CTX_OP(jfs->ctx, delete_jfs)) return URMA_EINVAL;
  urma_context_t* ctx = jfs->ctx;
  urma_jfc_t* jfc = jfs->cfg.jfc;
  const urma_status_t s = ctx->ops->delete_jfs(jfs);
  if (s == URMA_SUCCESS) {
    jfc_put(jfc);
    ctx_put(ctx);
  }
  return s;
}

// ================================================================================================ JFR
urma_jfr_t* urma_create_jfr(urma_context_t* ctx, const urma_jfr_cfg_t* cfg) {
  if (!cfg || cfg->depth == 0 || !cfg->jfc || cfg->jfc->ctx != ctx || !CTX_OP(ctx, create_jfr)) return nullptr;
  urma_jfr_t* j = ctx->ops->create_jfr(ctx, cfg);
  if (j) {
    j->ctx = ctx;
    j->cfg = *cfg;
    ctx_get(ctx);
    jfc_get(cfg->jfc);
  }
  return j;
}
urma_status_t urma_modify_jfr(urma_jfr_t* jfr, urma_jetty_state_t state, uint32_t thr) {
  if (!jfr || !CTX_OP(jfr->ctx, modify_jfr)) return URMA_EINVAL;
  return jfr->ctx->ops->modify_jfr(jfr, state, thr);
}
urma_status_t urma_query_jfr(urma_jfr_t* jfr, urma_jfr_cfg_t* cfg, urma_jetty_state_t* state) {
  if (!jfr || !cfg || !state || !CTX_OP(jfr->ctx, query_jfr)) return URMA_EINVAL;
  return jfr->ctx->ops->query_jfr(jfr, cfg, state);
}
urma_status_t urma_delete_jfr(urma_jfr_t* jfr) {
  if (!jfr || !CTX_OP(jfr->ctx, delete_jfr)) return URMA_EINVAL;
  urma_context_t* ctx = jfr->ctx;
  urma_jfc_t* jfc = jfr->cfg.jfc;
  const urma_status_t s = ctx->ops->delete_jfr(jfr);
  if (s == URMA_SUCCESS) {
    jfc_put(jfc);
    ctx_put(ctx);
  }
  return s;
}
urma_target_jetty_t* urma_import_jfr(urma_context_t* ctx, const urma_rjfr_t* rjfr, const urma_token_t* token) {
  if (!rjfr || !CTX_OP(ctx, import_jfr)) return nullptr;
  urma_target_jetty_t* t = ctx->ops->import_jfr(ctx, rjfr, token);
  if (t) {
    t->ctx = ctx;
    ctx_get(ctx);
  }
  return t;
}
urma_status_t urma_unimport_jfr(urma_target_jetty_t* t) {
  if (!t || !CTX_OP(t->ctx, unimport_jfr)) return URMA_EINVAL;
  urma_context_t* ctx = t->ctx;
  const urma_status_t s = ctx->ops->unimport_jfr(t);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}
urma_status_t urma_advise_jfr(urma_jfs_t* jfs, urma_target_jetty_t* t) { return (jfs && t) ? URMA_SUCCESS : URMA_EINVAL; }
urma_status_t urma_unadvise_jfr(urma_jfs_t* jfs, urma_target_jetty_t* t) {
  return (jfs && t) ? URMA_SUCCESS : URMA_EINVAL;
}

// ================================================================================================ Jetty
urma_jetty_t* urma_create_jetty(urma_context_t* ctx, const urma_jetty_cfg_t* cfg) {
  if (!cfg || !CTX_OP(ctx, create_jetty)) return nullptr;
  if (cfg->jfs_cfg.depth == 0 || !cfg->jfs_cfg.jfc || cfg->jfs_cfg.jfc->ctx != ctx) return nullptr;
  if (!cfg->shared_jfr && (cfg->jfr_cfg.depth == 0 || !cfg->jfr_cfg.jfc || cfg->jfr_cfg.jfc->ctx != ctx)) return nullptr;
  if (cfg->shared_jfr && cfg->shared_jfr->ctx != ctx) return nullptr;
  urma_jetty_t* j = ctx->ops->create_jetty(ctx, cfg);
  if (j) {
    j->ctx = ctx;
    j->cfg = *cfg;
    j->remote_jetty = nullptr;
    ctx_get(ctx);
    jfc_get(cfg->jfs_cfg.jfc);
    if (!cfg->shared_jfr) jfc_get(cfg->jfr_cfg.jfc);
  }
  return j;
}
urma_status_t urma_modify_jetty(urma_jetty_t* j, urma_jetty_state_t state) {
  if (!j || !CTX_OP(j->ctx, modify_jetty)) return URMA_EINVAL;
  return j->ctx->ops->modify_jetty(j, state);
}
urma_status_t urma_query_jetty(urma_jetty_t* j, urma_jetty_cfg_t* cfg, urma_jetty_state_t* state) {
  if (!j || !cfg || !state || !CTX_OP(j->ctx, query_jetty)) return URMA_EINVAL;
  return j->ctx->ops->query_jetty(j, cfg, state);
}
int urma_flush_jetty(urma_jetty_t* j, int cr_cnt, urma_cr_t* cr) {
  if (!j || cr_cnt <= 0 || !cr || !CTX_OP(j->ctx, flush_jetty)) return -1;
  return j->ctx->ops->flush_jetty(j, cr_cnt, cr);
}
urma_status_t urma_delete_jetty(urma_jetty_t* j) {
  if (!j || !CTX_OP(j->ctx, delete_jetty)) return URMA_EINVAL;
  urma_context_t* ctx = j->ctx;
  urma_jfc_t* sjfc = j->cfg.jfs_cfg.jfc;
  urma_jfc_t* rjfc = j->cfg.shared_jfr ? nullptr : j->cfg.jfr_cfg.jfc;
  const urma_status_t s = ctx->ops->delete_jetty(j);
  if (s == URMA_SUCCESS) {
    jfc_put(sjfc);
    jfc_put(rjfc);
    ctx_put(ctx);
  }
  return s;
}
urma_target_jetty_t* urma_import_jetty(urma_context_t* ctx, const urma_rjetty_t* rj, const urma_token_t* token) {
  if (!rj || !CTX_OP(ctx, import_jetty)) return nullptr;
  urma_target_jetty_t* t = ctx->ops->import_jetty(ctx, rj, token);
  if (t) {
    t->ctx = ctx;
    ctx_get(ctx);
  }
  return t;
}
urma_status_t urma_unimport_jetty(urma_target_jetty_t* t) {
  if (!t || !CTX_OP(t->ctx, unimport_jetty)) return URMA_EINVAL;
  urma_context_t* ctx = t->ctx;
  const urma_status_t s = ctx->ops->unimport_jetty(t);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}
urma_status_t urma_bind_jetty(urma_jetty_t* j, urma_target_jetty_t* t) {
  if (!j || !t || !CTX_OP(j->ctx, bind_jetty)) return URMA_EINVAL;
  if (j->remote_jetty) return URMA_EEXIST;
  const urma_status_t s = j->ctx->ops->bind_jetty(j, t);
  if (s == URMA_SUCCESS) j->remote_jetty = t;
  return s;
}
urma_status_t urma_unbind_jetty(urma_jetty_t* j) {
  if (!j || !j->remote_jetty || !CTX_OP(j->ctx, unbind_jetty)) return URMA_EINVAL;
  const urma_status_t s = j->ctx->ops->unbind_jetty(j);
  if (s == URMA_SUCCESS) j->remote_jetty = nullptr;
  return s;
}
urma_status_t urma_advise_jetty(urma_jetty_t* j, urma_target_jetty_t* t) { return (j && t) ? URMA_SUCCESS : URMA_EINVAL; }
urma_status_t urma_unadvise_jetty(urma_jetty_t* j, urma_target_jetty_t* t) {
  return (j && t) ? URMA_SUCCESS : URMA_EINVAL;
}
urma_jetty_grp_t* urma_create_jetty_grp(urma_context_t* ctx, const char* name, uint32_t policy) {
  if (!name || !CTX_OP(ctx, create_jetty_grp)) return nullptr;
  urma_jetty_grp_t* g = ctx->ops->create_jetty_grp(ctx, name, policy);
  if (g) {
    g->ctx = ctx;
    ctx_get(ctx);
  }
  return g;
}
urma_status_t urma_delete_jetty_grp(urma_jetty_grp_t* g) {
  if (!g || !CTX_OP(g->ctx, delete_jetty_grp)) return URMA_EINVAL;
  urma_context_t* ctx = g->ctx;
  const urma_status_t s = ctx->ops->delete_jetty_grp(g);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}

// ================================================================================================ memory
urma_token_id_t* urma_alloc_token_id(urma_context_t* ctx) {
  if (!CTX_OP(ctx, alloc_token_id)) return nullptr;
  urma_token_id_t* t = ctx->ops->alloc_token_id(ctx);
  if (t) {
    t->ctx = ctx;
    ctx_get(ctx);
  }
  return t;
}
urma_status_t urma_free_token_id(urma_token_id_t* t) {
  if (!t || !CTX_OP(t->ctx, free_token_id)) return URMA_EINVAL;
  urma_context_t* ctx = t->ctx;
  const urma_status_t s = ctx->ops->free_token_id(t);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}
urma_target_seg_t* urma_register_seg(urma_context_t* ctx, const urma_seg_cfg_t* cfg) {
  if (!cfg || cfg->va == 0 || cfg->len == 0 || !CTX_OP(ctx, register_seg)) return nullptr;
  if (!access_ok(cfg->access)) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "invalid access flags 0x%x", cfg->access);
    return nullptr;
  }
  if (cfg->token_id && cfg->token_id->ctx != ctx) return nullptr;
  urma_seg_cfg_t c = *cfg;
  bool own = false;
  if (!c.token_id) {  // the reference allocates a token id on behalf of the caller when none is given
    c.token_id = urma_alloc_token_id(ctx);
    if (!c.token_id) return nullptr;
    own = true;
  }
  urma_target_seg_t* t = ctx->ops->register_seg(ctx, &c);
  if (!t) {
    if (own) urma_free_token_id(c.token_id);
    return nullptr;
  }
  t->ctx = ctx;
  t->token_id = c.token_id;
  t->own_token_id = own;
  t->is_import = false;
  t->user_ctx = cfg->user_ctx;
  ctx_get(ctx);
  return t;
}
urma_status_t urma_unregister_seg(urma_target_seg_t* t) {
  if (!t || t->is_import || !CTX_OP(t->ctx, unregister_seg)) return URMA_EINVAL;
  urma_context_t* ctx = t->ctx;
  urma_token_id_t* tok = t->own_token_id ? t->token_id : nullptr;
  const urma_status_t s = ctx->ops->unregister_seg(t);
  if (s == URMA_SUCCESS) {
    if (tok) urma_free_token_id(tok);
    ctx_put(ctx);
  }
  return s;
}
urma_target_seg_t* urma_import_seg(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token,
                                   uint64_t addr, uint32_t flag) {
  if (!seg || seg->len == 0 || !CTX_OP(ctx, import_seg)) return nullptr;
  if (seg->attr & URMA_ACCESS_LOCAL_ONLY) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "segment is local-only and cannot be imported");
    return nullptr;
  }
  urma_target_seg_t* t = ctx->ops->import_seg(ctx, seg, token, addr, flag);
  if (t) {
    t->ctx = ctx;
    t->is_import = true;
    ctx_get(ctx);
  }
  return t;
}
urma_status_t urma_unimport_seg(urma_target_seg_t* t) {
  if (!t || !t->is_import || !CTX_OP(t->ctx, unimport_seg)) return URMA_EINVAL;
  urma_context_t* ctx = t->ctx;
  const urma_status_t s = ctx->ops->unimport_seg(t);
  if (s == URMA_SUCCESS) ctx_put(ctx);
  return s;
}

// ================================================================================================ data plane
urma_status_t urma_post_jfs_wr(urma_jfs_t* jfs, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  if (!jfs || !wr || !bad || !CTX_OP(jfs->ctx, post_jfs_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_POST_JFS);
  return jfs->ctx->ops->post_jfs_wr(jfs, wr, bad);
}
urma_status_t urma_post_jfr_wr(urma_jfr_t* jfr, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  if (!jfr || !wr || !bad || !CTX_OP(jfr->ctx, post_jfr_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_POST_JFR);
  return jfr->ctx->ops->post_jfr_wr(jfr, wr, bad);
}
urma_status_t urma_post_jetty_send_wr(urma_jetty_t* j, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  if (!j || !wr || !bad || !CTX_OP(j->ctx, post_jetty_send_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_POST_JETTY_SEND);
  return j->ctx->ops->post_jetty_send_wr(j, wr, bad);
}
urma_status_t urma_post_jetty_recv_wr(urma_jetty_t* j, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  if (!j || !wr || !bad || !CTX_OP(j->ctx, post_jetty_recv_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_POST_JETTY_RECV);
  return j->ctx->ops->post_jetty_recv_wr(j, wr, bad);
}

static urma_status_t rw_one(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_opcode_t opc, urma_target_seg_t* dst_tseg,
                            urma_target_seg_t* src_tseg, uint64_t dst, uint64_t src, uint32_t len, uint32_t flag,
                            uint64_t user_ctx) {
  if (!jfs || !tjfr || !dst_tseg || !src_tseg || len == 0) return URMA_EINVAL;
  urma_sge_t s{src, len, src_tseg}, d{dst, len, dst_tseg};
  urma_jfs_wr_t wr{};
  wr.opcode = opc;
  wr.flag = flag;
  wr.tjetty = tjfr;
  wr.user_ctx = user_ctx;
  wr.rw.src = urma_sg_t{&s, 1};
  wr.rw.dst = urma_sg_t{&d, 1};
  wr.next = nullptr;
  urma_jfs_wr_t* bad = nullptr;
  if (!CTX_OP(jfs->ctx, post_jfs_wr)) return URMA_FAIL;
  return jfs->ctx->ops->post_jfs_wr(jfs, &wr, &bad);
}
urma_status_t urma_write(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* dst_tseg,
                         urma_target_seg_t* src_tseg, uint64_t dst, uint64_t src, uint32_t len, uint32_t flag,
                         uint64_t user_ctx) {
  PerfScope ps(URMA_PERF_WRITE);
  return rw_one(jfs, tjfr, URMA_OPC_WRITE, dst_tseg, src_tseg, dst, src, len, flag, user_ctx);
}
urma_status_t urma_read(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* dst_tseg,
                        urma_target_seg_t* src_tseg, uint64_t dst, uint64_t src, uint32_t len, uint32_t flag,
                        uint64_t user_ctx) {
  PerfScope ps(URMA_PERF_READ);
  return rw_one(jfs, tjfr, URMA_OPC_READ, dst_tseg, src_tseg, dst, src, len, flag, user_ctx);
}
urma_status_t urma_send(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* src_tseg, uint64_t src,
                        uint32_t len, uint32_t flag, uint64_t user_ctx) {
  if (!jfs || !tjfr || !CTX_OP(jfs->ctx, post_jfs_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_SEND);
  urma_sge_t s{src, len, src_tseg};
  urma_jfs_wr_t wr{};
  wr.opcode = URMA_OPC_SEND;
  wr.flag = flag;
  wr.tjetty = tjfr;
  wr.user_ctx = user_ctx;
  wr.send.src = urma_sg_t{&s, 1};
  urma_jfs_wr_t* bad = nullptr;
  return jfs->ctx->ops->post_jfs_wr(jfs, &wr, &bad);
}
urma_status_t urma_recv(urma_jfr_t* jfr, urma_target_seg_t* recv_tseg, uint64_t buf, uint32_t len, uint64_t user_ctx) {
  if (!jfr || !CTX_OP(jfr->ctx, post_jfr_wr)) return URMA_EINVAL;
  PerfScope ps(URMA_PERF_RECV);
  urma_sge_t s{buf, len, recv_tseg};
  urma_jfr_wr_t wr{};
  wr.src = urma_sg_t{&s, 1};
  wr.user_ctx = user_ctx;
  urma_jfr_wr_t* bad = nullptr;
  return jfr->ctx->ops->post_jfr_wr(jfr, &wr, &bad);
}
int urma_poll_jfc(urma_jfc_t* jfc, int cr_cnt, urma_cr_t* cr) {
  if (!jfc || cr_cnt <= 0 || !cr || !CTX_OP(jfc->ctx, poll_jfc)) return -1;
  PerfScope ps(URMA_PERF_POLL_JFC);
  return jfc->ctx->ops->poll_jfc(jfc, cr_cnt, cr);
}
urma_status_t urma_rearm_jfc(urma_jfc_t* jfc, bool solicited_only) {
  if (!jfc || !CTX_OP(jfc->ctx, rearm_jfc)) return URMA_EINVAL;
  return jfc->ctx->ops->rearm_jfc(jfc, solicited_only);
}
int urma_wait_jfc(urma_jfce_t* jfce, uint32_t jfc_cnt, int time_out, urma_jfc_t* jfc[]) {
  if (!jfce || jfc_cnt == 0 || !jfc || !CTX_OP(jfce->ctx, wait_jfc)) return -1;
  return jfce->ctx->ops->wait_jfc(jfce, jfc_cnt, time_out, jfc);
}
void urma_ack_jfc(urma_jfc_t* jfc[], uint32_t nevents[], uint32_t jfc_cnt) {
  if (!jfc || !nevents || jfc_cnt == 0 || !jfc[0] || !CTX_OP(jfc[0]->ctx, ack_jfc)) return;
  jfc[0]->ctx->ops->ack_jfc(jfc, nevents, jfc_cnt);
}

// ================================================================================================ events / ctl
urma_status_t urma_get_async_event(urma_context_t* ctx, urma_async_event_t* ev) {
  if (!ev || !CTX_OP(ctx, get_async_event)) return URMA_EINVAL;
  return ctx->ops->get_async_event(ctx, ev);
}
void urma_ack_async_event(urma_async_event_t* ev) {
  if (ev && CTX_OP(ev->ctx, ack_async_event)) ev->ctx->ops->ack_async_event(ev);
}
int urma_user_ctl(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out) {
  if (!in || !out || !CTX_OP(ctx, user_ctl)) return -1;
  return ctx->ops->user_ctl(ctx, in, out);
}

}  // extern "C"
