// "cuda_ipc" URMA provider: URMA segments are GPU memory, remote access goes over NVLink through CUDA IPC peer
// mappings. One device ("cuda0", "cuda1", ...) per visible GPU; a context binds to that GPU.
//
//   register_seg   the segment's allocation is exported with cudaIpcGetMemHandle and published (handle, offset inside
//                  the allocation, length, access bits, token) in a small shared-memory directory
//   import_seg     looks the segment up, opens the handle (or uses the pointer directly inside the owning process)
//                  and keeps the mapped address in `mva`
//   WRITE / READ   cudaMemcpyAsync between the local buffer and the mapped remote address on the context's stream
//   atomics        a one-thread kernel doing system-scope atomics on the mapped address; the old value lands in
//                  pinned host memory and is copied to the caller's result buffer when the completion is reaped
//   completion     every request records an event; poll_jfc reaps finished events in order and emits completion
//                  records (token and access violations are reported as URMA_CR_REM_ACCESS_ABORT_ERR at post time)
//   SEND / RECV    every jetty owns a small shared-memory file with a ring of posted receive buffers (device
//                  memory, exported with CUDA IPC when it is posted) and a ring of receive completions. A SEND /
//                  SEND_IMM takes the oldest posted buffer of the target jetty, copies the payload into it with
//                  cudaMemcpyAsync on the sender's stream, and - once the copy's event has fired - writes the
//                  receive completion (length, immediate data, source jetty) into the target's ring, where the
//                  receiver's poll_jfc finds it. No posted buffer = receiver-not-ready error on the sender; a payload
//                  longer than the buffer = length error on both sides. The counterpart of the send path and the
//                  receive queue of the reference's hardware user driver (src/urma/hw/udma/udma_u_jfs.c:819-873,
//                  udma_u_jfr.c).
// This provider takes the place of the reference's hardware user driver (src/urma/hw/udma) for GPUs of one box.
#include <cuda.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "urma_api.h"
#include "urma_provider.h"

namespace {

constexpr uint32_t kDirEntries = 4096;
constexpr uint32_t kDirMagic = 0x43495043;  // "CIPC"

struct DirEntry {
  std::atomic<uint32_t> state;  // 0 free, 1 busy, 2 valid
  uint32_t uasid, token_id, token_val, access, dev, pid;
  uint64_t va, len, alloc_base;
  cudaIpcMemHandle_t handle;
};
struct Dir {
  std::atomic<uint32_t> magic, next_uasid, next_id, pad;
  DirEntry e[kDirEntries];
};
Dir* g_dir = nullptr;
int g_ndev = 0;

Dir* dir() {
  if (g_dir) return g_dir;
  const char* e = getenv("URMA_SHM_DIR");
  const std::string d = (e && *e) ? e : "/dev/shm/umdk_urma_" + std::to_string(getuid());
  mkdir(d.c_str(), 0700);
  const std::string path = d + "/cuda_ipc.dir";
  const int fd = open(path.c_str(), O_RDWR | O_CREAT, 0600);
  if (fd < 0) return nullptr;
  if (ftruncate(fd, sizeof(Dir)) != 0) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, sizeof(Dir), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return nullptr;
  g_dir = static_cast<Dir*>(p);
  uint32_t exp = 0;
  g_dir->magic.compare_exchange_strong(exp, kDirMagic);
  return g_dir;
}

// Base address and size of the allocation that contains `p` (driver entry point resolved through the runtime, so the
// plug-in does not link against libcuda).
bool alloc_range(void* p, void** base, size_t* len) {
  typedef CUresult (*Fn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static Fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<Fn>(f);
  }();
  if (!fn) return false;
  CUdeviceptr b = 0;
  size_t n = 0;
  if (fn(&b, &n, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) return false;
  *base = reinterpret_cast<void*>(b);
  *len = n;
  return true;
}

__global__ void atomic_kernel(unsigned long long* addr, int opcode, unsigned long long operand,
                              unsigned long long cmp, unsigned long long* old_out) {
  unsigned long long old = 0;
  switch (opcode) {
    case URMA_OPC_CAS: old = atomicCAS_system(addr, cmp, operand); break;
    case URMA_OPC_SWAP: old = atomicExch_system(addr, operand); break;
    case URMA_OPC_FADD: old = atomicAdd_system(addr, operand); break;
    case URMA_OPC_FSUB: old = atomicAdd_system(addr, (unsigned long long)(-(long long)operand)); break;
    case URMA_OPC_FAND: old = atomicAnd_system(addr, operand); break;
    case URMA_OPC_FOR: old = atomicOr_system(addr, operand); break;
    case URMA_OPC_FXOR: old = atomicXor_system(addr, operand); break;
    default: break;
  }
  *old_out = old;
}

// ---- two-sided messaging state shared between processes (one file per jetty) ----
constexpr uint32_t kRq = 256;   // posted receive buffers per jetty
constexpr uint32_t kRcq = 512;  // receive completions per jetty
constexpr uint32_t kJettyMagic = 0x544a4355;  // "UCJT"
struct RecvSlot {
  std::atomic<uint32_t> state;  // 0 free, 1 posted
  uint32_t pid, dev, len;
  uint64_t user_ctx, va, alloc_base;
  cudaIpcMemHandle_t handle;
};
struct RecvComp {
  std::atomic<uint32_t> state;  // 0 free, 1 being written, 2 valid
  uint32_t status, len, opcode;
  uint64_t user_ctx, imm;
  urma_jetty_id_t remote;
};
struct JettyShm {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> alive;
  std::atomic<uint64_t> rq_head, rq_tail;   // consumers (senders) advance head with CAS, the owner advances tail
  std::atomic<uint64_t> cq_head, cq_tail;   // producers (senders) reserve at tail with fetch_add, the owner drains head
  RecvSlot rq[kRq];
  RecvComp cq[kRcq];
};

std::string shm_dir() {
  const char* e = getenv("URMA_SHM_DIR");
  const std::string d = (e && *e) ? e : "/dev/shm/umdk_urma_" + std::to_string(getuid());
  mkdir(d.c_str(), 0700);
  return d;
}
std::string jetty_path(uint32_t uasid, uint32_t id) {
  return shm_dir() + "/cuda_jetty_" + std::to_string(uasid) + "_" + std::to_string(id);
}
JettyShm* map_jetty(uint32_t uasid, uint32_t id, bool create) {
  const std::string path = jetty_path(uasid, id);
  const int fd = open(path.c_str(), create ? (O_RDWR | O_CREAT | O_TRUNC) : O_RDWR, 0600);
  if (fd < 0) return nullptr;
  if (create && ftruncate(fd, sizeof(JettyShm)) != 0) {
    close(fd);
    return nullptr;
  }
  struct stat sb{};
  if (fstat(fd, &sb) != 0 || sb.st_size != (off_t)sizeof(JettyShm)) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, sizeof(JettyShm), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return nullptr;
  JettyShm* j = static_cast<JettyShm*>(p);
  if (create) {
    j->alive.store(1);
    j->magic.store(kJettyMagic, std::memory_order_release);
  } else if (j->magic.load(std::memory_order_acquire) != kJettyMagic) {
    munmap(p, sizeof(JettyShm));
    return nullptr;
  }
  return j;
}

// Receive buffers of other processes, opened once per allocation (keyed by the IPC handle bytes).
std::mutex g_ipc_mu;
std::unordered_map<std::string, void*> g_ipc_open;
void* open_remote_alloc(const cudaIpcMemHandle_t& h) {
  const std::string key(reinterpret_cast<const char*>(&h), sizeof(h));
  std::lock_guard<std::mutex> l(g_ipc_mu);
  auto it = g_ipc_open.find(key);
  if (it != g_ipc_open.end()) return it->second;
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  g_ipc_open[key] = p;
  return p;
}

struct CJfc {
  urma_jfc_t pub;
};
struct Req {
  cudaEvent_t ev;
  uint64_t user_ctx;
  uint32_t flag, local_id, len;
  urma_jetty_id_t remote;
  unsigned long long* old_host;  // pinned slot for atomics (or null)
  uint64_t result_addr;          // where the caller wants the old value
  urma_cr_status_t early;        // != SUCCESS: failed at post time, no event
  // SEND: where the receive completion goes once the copy has finished
  JettyShm* rx = nullptr;
  uint64_t rx_user_ctx = 0, imm = 0;
  uint32_t rx_opcode = 0, rx_status = 0;
};
struct CCtx {
  urma_context_t pub;
  int dev;
  cudaStream_t stream;
  std::mutex mu;
  unsigned long long* pinned = nullptr;  // ring of result slots
  uint32_t pinned_next = 0;
  // Completion events are recycled: creating and destroying one per request costs more than a small copy itself.
  std::mutex ev_mu;
  std::vector<cudaEvent_t> ev_free;
};
cudaEvent_t event_get(CCtx* c) {
  {
    std::lock_guard<std::mutex> l(c->ev_mu);
    if (!c->ev_free.empty()) {
      cudaEvent_t e = c->ev_free.back();
      c->ev_free.pop_back();
      return e;
    }
  }
  cudaEvent_t e = nullptr;
  cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
  return e;
}
void event_put(CCtx* c, cudaEvent_t e) {
  if (!e) return;
  {
    std::lock_guard<std::mutex> l(c->ev_mu);
    if (c->ev_free.size() < 4096) {
      c->ev_free.push_back(e);
      return;
    }
  }
  cudaEventDestroy(e);
}
struct CJetty {
  urma_jetty_t pub;
  std::mutex mu;
  std::deque<Req> inflight;
  uint32_t id;
  CJfc* jfc;
  std::atomic<int> state{URMA_JETTY_STATE_READY};
  JettyShm* shm = nullptr;   // this jetty's receive queue and receive-completion ring
  urma_jfc_t* rx_jfc = nullptr;
};
// Direct access from device `from` to memory of device `to` inside this process. Without it a copy between the two
// is staged through host memory by the runtime (tens of GB/s instead of NVLink's hundreds) and a kernel on `from`
// must not touch `to`'s memory at all. Enabled once per pair, the first time a context on `from` is made or a
// segment of `to` is imported; the answer is remembered.
constexpr int kMaxDev = 64;
std::mutex g_peer_mu;
int8_t g_peer[kMaxDev][kMaxDev];   // 0 unknown, 1 direct access works, -1 it does not
bool peer_direct(int from, int to) {
  if (from == to) return true;
  if (from < 0 || to < 0 || from >= kMaxDev || to >= kMaxDev) return false;
  std::lock_guard<std::mutex> l(g_peer_mu);
  if (g_peer[from][to] == 0) {
    int can = 0, cur = -1;
    cudaGetDevice(&cur);
    bool ok = cudaDeviceCanAccessPeer(&can, from, to) == cudaSuccess && can;
    if (ok && cudaSetDevice(from) == cudaSuccess) {
      const cudaError_t e = cudaDeviceEnablePeerAccess(to, 0);
      ok = e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled;
    }
    cudaGetLastError();   // "already enabled" is not an error to carry around
    if (cur >= 0) cudaSetDevice(cur);
    g_peer[from][to] = ok ? 1 : -1;
  }
  return g_peer[from][to] == 1;
}

struct CSeg {
  urma_target_seg_t pub;
  uint32_t token_val;
  bool direct = true;   // kernels of this context's device may touch the segment (false: copies only, staged)
  void* mapped_base = nullptr;  // base returned by cudaIpcOpenMemHandle (imports from another process)
  DirEntry* entry = nullptr;
};
struct CTarget {
  urma_target_jetty_t pub;
  JettyShm* shm = nullptr;   // the remote jetty's rings (null: the jetty has none, SEND is refused)
};
CCtx* C(urma_context_t* c) { return reinterpret_cast<CCtx*>(c->priv); }

urma_jfc_t* op_create_jfc(urma_context_t*, const urma_jfc_cfg_t* cfg) {
  CJfc* j = new CJfc();
  j->pub.cfg = *cfg;
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jfc(urma_jfc_t*, uint32_t, uint32_t) { return URMA_SUCCESS; }
urma_status_t op_delete_jfc(urma_jfc_t* j) {
  delete reinterpret_cast<CJfc*>(j->priv);
  return URMA_SUCCESS;
}
// completion queues of this provider are fed by their jetties; keep the list per JFC
std::mutex g_jmu;
std::unordered_map<urma_jfc_t*, std::vector<CJetty*>> g_jfc_jetties;

urma_jetty_t* op_create_jetty(urma_context_t* ctx, const urma_jetty_cfg_t* cfg) {
  CJetty* j = new CJetty();
  j->id = dir()->next_id.fetch_add(1) + 1;
  j->jfc = reinterpret_cast<CJfc*>(cfg->jfs_cfg.jfc->priv);
  j->pub.jetty_id.eid = ctx->eid;
  j->pub.jetty_id.uasid = ctx->uasid;
  j->pub.jetty_id.id = j->id;
  j->pub.priv = j;
  j->shm = map_jetty(ctx->uasid, j->id, true);
  j->rx_jfc = cfg->jfr_cfg.jfc ? cfg->jfr_cfg.jfc : cfg->jfs_cfg.jfc;
  std::lock_guard<std::mutex> l(g_jmu);
  g_jfc_jetties[cfg->jfs_cfg.jfc].push_back(j);
  if (j->rx_jfc != cfg->jfs_cfg.jfc) g_jfc_jetties[j->rx_jfc].push_back(j);
  return &j->pub;
}
urma_status_t op_modify_jetty(urma_jetty_t* jt, urma_jetty_state_t st) {
  reinterpret_cast<CJetty*>(jt->priv)->state = st;
  return URMA_SUCCESS;
}
urma_status_t op_query_jetty(urma_jetty_t* jt, urma_jetty_cfg_t* cfg, urma_jetty_state_t* st) {
  *cfg = jt->cfg;
  *st = static_cast<urma_jetty_state_t>(reinterpret_cast<CJetty*>(jt->priv)->state.load());
  return URMA_SUCCESS;
}
urma_status_t op_delete_jetty(urma_jetty_t* jt) {
  CJetty* j = reinterpret_cast<CJetty*>(jt->priv);
  {
    std::lock_guard<std::mutex> l(g_jmu);
    for (urma_jfc_t* q : {jt->cfg.jfs_cfg.jfc, j->rx_jfc}) {
      auto& v = g_jfc_jetties[q];
      for (size_t i = 0; i < v.size(); ++i)
        if (v[i] == j) {
          v.erase(v.begin() + i);
          break;
        }
    }
  }
  if (j->shm) {
    j->shm->alive.store(0);
    munmap(j->shm, sizeof(JettyShm));
    unlink(jetty_path(jt->jetty_id.uasid, j->id).c_str());
  }
  for (auto& r : j->inflight)
    if (r.early == URMA_CR_SUCCESS) event_put(reinterpret_cast<CCtx*>(jt->ctx->priv), r.ev);
  delete j;
  return URMA_SUCCESS;
}
urma_target_jetty_t* op_import_jetty(urma_context_t*, const urma_rjetty_t* rj, const urma_token_t*) {
  CTarget* t = new CTarget();
  t->pub.id = rj->jetty_id;
  t->pub.trans_mode = rj->trans_mode;
  t->pub.type = rj->type;
  t->pub.priv = t;
  t->shm = map_jetty(rj->jetty_id.uasid, rj->jetty_id.id, false);
  return &t->pub;
}
urma_status_t op_unimport_jetty(urma_target_jetty_t* t) {
  CTarget* ct = reinterpret_cast<CTarget*>(t->priv);
  if (ct->shm) munmap(ct->shm, sizeof(JettyShm));
  delete ct;
  return URMA_SUCCESS;
}
urma_status_t op_bind(urma_jetty_t*, urma_target_jetty_t*) { return URMA_SUCCESS; }
urma_status_t op_unbind(urma_jetty_t*) { return URMA_SUCCESS; }

urma_token_id_t* op_alloc_token(urma_context_t*) {
  urma_token_id_t* t = new urma_token_id_t();
  t->token_id = dir()->next_id.fetch_add(1) + 1;
  return t;
}
urma_status_t op_free_token(urma_token_id_t* t) {
  delete t;
  return URMA_SUCCESS;
}

urma_target_seg_t* op_register_seg(urma_context_t* ctx, const urma_seg_cfg_t* cfg) {
  CCtx* c = C(ctx);
  cudaSetDevice(c->dev);
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, reinterpret_cast<void*>(cfg->va)) != cudaSuccess ||
      at.type != cudaMemoryTypeDevice) {
    cudaGetLastError();
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "segment must be device memory");
    return nullptr;
  }
  // the IPC handle describes the whole allocation; remember where the segment sits inside it
  void* base = nullptr;
  size_t alloc_len = 0;
  if (!alloc_range(reinterpret_cast<void*>(cfg->va), &base, &alloc_len)) return nullptr;
  DirEntry* e = nullptr;
  for (uint32_t i = 0; i < kDirEntries; ++i) {
    uint32_t exp = 0;
    if (dir()->e[i].state.compare_exchange_strong(exp, 1)) {
      e = &dir()->e[i];
      break;
    }
  }
  if (!e) return nullptr;
  if (cudaIpcGetMemHandle(&e->handle, base) != cudaSuccess) {
    cudaGetLastError();
    e->state = 0;
    return nullptr;
  }
  e->uasid = ctx->uasid;
  e->token_id = cfg->token_id->token_id;
  e->token_val = cfg->token_value.token;
  e->access = cfg->access;
  e->dev = c->dev;
  e->pid = getpid();
  e->va = cfg->va;
  e->len = cfg->len;
  e->alloc_base = reinterpret_cast<uint64_t>(base);
  e->state.store(2, std::memory_order_release);
  CSeg* s = new CSeg();
  s->pub.seg.ubva.eid = ctx->eid;
  s->pub.seg.ubva.uasid = ctx->uasid;
  s->pub.seg.ubva.va = cfg->va;
  s->pub.seg.len = cfg->len;
  s->pub.seg.attr = cfg->access;
  s->pub.seg.token_id = e->token_id;
  s->pub.priv = s;
  s->token_val = cfg->token_value.token;
  s->entry = e;
  return &s->pub;
}
urma_status_t op_unregister_seg(urma_target_seg_t* t) {
  CSeg* s = reinterpret_cast<CSeg*>(t->priv);
  if (s->entry) s->entry->state.store(0);
  delete s;
  return URMA_SUCCESS;
}
urma_target_seg_t* op_import_seg(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token, uint64_t,
                                 uint32_t) {
  CCtx* c = C(ctx);
  DirEntry* e = nullptr;
  for (uint32_t i = 0; i < kDirEntries; ++i) {
    DirEntry& d = dir()->e[i];
    if (d.state.load(std::memory_order_acquire) == 2 && d.uasid == seg->ubva.uasid && d.token_id == seg->token_id) {
      e = &d;
      break;
    }
  }
  if (!e) return nullptr;
  CSeg* s = new CSeg();
  s->pub.seg = *seg;
  s->pub.priv = s;
  s->token_val = token ? token->token : 0;
  s->entry = e;
  cudaSetDevice(c->dev);
  if (e->pid == (uint32_t)getpid()) {
    s->pub.mva = e->va;  // same process: the pointer itself, once this device may reach the owner's memory
    s->direct = peer_direct(c->dev, static_cast<int>(e->dev));
    peer_direct(static_cast<int>(e->dev), c->dev);   // reads come back the other way
  } else {
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, e->handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      delete s;
      return nullptr;
    }
    s->mapped_base = p;
    s->pub.mva = reinterpret_cast<uint64_t>(p) + (e->va - e->alloc_base);
  }
  return &s->pub;
}
urma_status_t op_unimport_seg(urma_target_seg_t* t) {
  CSeg* s = reinterpret_cast<CSeg*>(t->priv);
  if (s->mapped_base) cudaIpcCloseMemHandle(s->mapped_base);
  delete s;
  return URMA_SUCCESS;
}

// validates a remote access against the published registration; returns the mapped address or 0
uint64_t remote_addr(CSeg* s, uint64_t va, uint64_t len, uint32_t need, urma_cr_status_t* st) {
  DirEntry* e = s->entry;
  if (!e || e->state.load() != 2 || e->token_val != s->token_val || (e->access & need) != need) {
    *st = URMA_CR_REM_ACCESS_ABORT_ERR;
    return 0;
  }
  if (va < e->va || va + len > e->va + e->len) {
    *st = URMA_CR_REM_OPERATION_ERR;
    return 0;
  }
  *st = URMA_CR_SUCCESS;
  return s->pub.mva + (va - e->va);
}

urma_status_t op_post_send(urma_jetty_t* jt, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  CCtx* c = C(jt->ctx);
  CJetty* j = reinterpret_cast<CJetty*>(jt->priv);
  cudaSetDevice(c->dev);
  for (urma_jfs_wr_t* w = wr; w; w = w->next) {
    urma_target_jetty_t* tj = w->tjetty ? w->tjetty : jt->remote_jetty;
    if (!tj || j->state.load() != URMA_JETTY_STATE_READY) {
      *bad = w;
      return URMA_EINVAL;
    }
    Req r{};
    r.user_ctx = w->user_ctx;
    r.flag = w->flag;
    r.local_id = j->id;
    r.remote = tj->id;
    r.early = URMA_CR_SUCCESS;
    cudaError_t ce = cudaSuccess;
    switch (w->opcode) {
      case URMA_OPC_WRITE:
      case URMA_OPC_READ: {
        const bool rd = w->opcode == URMA_OPC_READ;
        const urma_sg_t& rem = rd ? w->rw.src : w->rw.dst;
        const urma_sg_t& loc = rd ? w->rw.dst : w->rw.src;
        if (rem.num_sge != 1 || loc.num_sge != 1 || !rem.sge[0].tseg || rem.sge[0].len != loc.sge[0].len) {
          *bad = w;
          return URMA_EINVAL;
        }
        r.len = rem.sge[0].len;
        const uint64_t ra = remote_addr(reinterpret_cast<CSeg*>(rem.sge[0].tseg->priv), rem.sge[0].addr, r.len,
                                        rd ? URMA_ACCESS_READ : URMA_ACCESS_WRITE, &r.early);
        if (r.early == URMA_CR_SUCCESS) {
          void* dst = rd ? reinterpret_cast<void*>(loc.sge[0].addr) : reinterpret_cast<void*>(ra);
          void* src = rd ? reinterpret_cast<void*>(ra) : reinterpret_cast<void*>(loc.sge[0].addr);
          ce = cudaMemcpyAsync(dst, src, r.len, cudaMemcpyDefault, c->stream);
        }
        break;
      }
      case URMA_OPC_CAS:
      case URMA_OPC_SWAP:
      case URMA_OPC_FADD:
      case URMA_OPC_FSUB:
      case URMA_OPC_FAND:
      case URMA_OPC_FOR:
      case URMA_OPC_FXOR: {
        const bool cas = w->opcode == URMA_OPC_CAS || w->opcode == URMA_OPC_SWAP;
        urma_sge_t* d = cas ? w->cas.dst : w->faa.dst;
        urma_sge_t* s = cas ? w->cas.src : w->faa.src;
        if (!d || !d->tseg || d->len != 8 || (d->addr & 7)) {
          *bad = w;
          return URMA_EINVAL;
        }
        r.len = 8;
        uint64_t ra = remote_addr(reinterpret_cast<CSeg*>(d->tseg->priv), d->addr, 8, URMA_ACCESS_ATOMIC, &r.early);
        if (r.early == URMA_CR_SUCCESS && !reinterpret_cast<CSeg*>(d->tseg->priv)->direct) {
          r.early = URMA_CR_REM_UNSUPPORTED_REQ_ERR;   // no direct path between the two GPUs: no kernel may go there
          ra = 0;
        }
        if (r.early == URMA_CR_SUCCESS) {
          {
            std::lock_guard<std::mutex> l(c->mu);
            r.old_host = c->pinned + (c->pinned_next++ % 1024);
          }
          r.result_addr = s ? s->addr : 0;
          atomic_kernel<<<1, 1, 0, c->stream>>>(reinterpret_cast<unsigned long long*>(ra), w->opcode,
                                                cas ? w->cas.swap_data : w->faa.operand, cas ? w->cas.cmp_data : 0,
                                                r.old_host);
          ce = cudaGetLastError();
        }
        break;
      }
      case URMA_OPC_SEND:
      case URMA_OPC_SEND_IMM: {
        CTarget* ct = reinterpret_cast<CTarget*>(tj->priv);
        if (w->send.src.num_sge != 1 || !ct->shm) {
          *bad = w;
          return URMA_EINVAL;
        }
        JettyShm* rx = ct->shm;
        r.len = w->send.src.sge[0].len;
        // take the oldest posted receive buffer of the target (several senders may race for it)
        RecvSlot taken{};
        bool have = false;
        if (rx->alive.load()) {
          for (;;) {
            uint64_t h = rx->rq_head.load(std::memory_order_acquire);
            if (h == rx->rq_tail.load(std::memory_order_acquire)) break;
            RecvSlot& sl = rx->rq[h % kRq];
            if (sl.state.load(std::memory_order_acquire) != 1) break;
            memcpy(&taken.pid, &sl.pid, sizeof(RecvSlot) - offsetof(RecvSlot, pid));
            if (rx->rq_head.compare_exchange_weak(h, h + 1, std::memory_order_acq_rel)) {
              sl.state.store(0, std::memory_order_release);
              have = true;
              break;
            }
          }
        }
        if (!have) {
          r.early = URMA_CR_RNR_RETRY_CNT_EXC_ERR;   // receiver not ready: nothing was consumed on the other side
          break;
        }
        r.rx = rx;
        r.rx_user_ctx = taken.user_ctx;
        r.imm = w->opcode == URMA_OPC_SEND_IMM ? w->send.imm_data : 0;
        r.rx_opcode = w->opcode == URMA_OPC_SEND_IMM ? URMA_CR_OPC_SEND_WITH_IMM : URMA_CR_OPC_SEND;
        r.rx_status = URMA_CR_SUCCESS;
        if (r.len > taken.len) {
          // the message does not fit: both sides learn it, the buffer is spent (as on a NIC)
          r.rx_status = URMA_CR_LOC_LEN_ERR;
          r.early = URMA_CR_REM_RESP_LEN_ERR;
        } else {
          void* dst = nullptr;
          if (taken.pid == (uint32_t)getpid()) {
            dst = reinterpret_cast<void*>(taken.va);
            peer_direct(c->dev, static_cast<int>(taken.dev));   // a copy to another GPU should not go through the host
          } else {
            void* base = open_remote_alloc(taken.handle);
            if (base) dst = static_cast<char*>(base) + (taken.va - taken.alloc_base);
          }
          if (!dst) {
            r.rx_status = URMA_CR_REM_OPERATION_ERR;
            r.early = URMA_CR_REM_OPERATION_ERR;
          } else {
            ce = cudaMemcpyAsync(dst, reinterpret_cast<void*>(w->send.src.sge[0].addr), r.len, cudaMemcpyDefault,
                                 c->stream);
          }
        }
        if (r.early != URMA_CR_SUCCESS) {   // no copy was queued: tell the receiver now
          const uint64_t t = rx->cq_tail.fetch_add(1);
          RecvComp& cc = rx->cq[t % kRcq];
          cc.status = r.rx_status;
          cc.len = 0;
          cc.opcode = r.rx_opcode;
          cc.user_ctx = r.rx_user_ctx;
          cc.imm = r.imm;
          cc.remote = jt->jetty_id;
          cc.state.store(2, std::memory_order_release);
          r.rx = nullptr;
        }
        break;
      }
      case URMA_OPC_NOP: break;
      default:
        *bad = w;
        return URMA_EINVAL;
    }
    if (ce != cudaSuccess) {
      *bad = w;
      return URMA_FAIL;
    }
    if (r.early == URMA_CR_SUCCESS) {
      r.ev = event_get(c);
      cudaEventRecord(r.ev, c->stream);
    }
    std::lock_guard<std::mutex> l(j->mu);
    j->inflight.push_back(r);
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}

urma_status_t op_post_recv(urma_jetty_t* jt, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  CCtx* c = C(jt->ctx);
  CJetty* j = reinterpret_cast<CJetty*>(jt->priv);
  if (!j->shm) {
    *bad = wr;
    return URMA_FAIL;
  }
  cudaSetDevice(c->dev);
  for (urma_jfr_wr_t* w = wr; w; w = w->next) {
    if (w->src.num_sge != 1) {
      *bad = w;
      return URMA_EINVAL;
    }
    void* buf = reinterpret_cast<void*>(w->src.sge[0].addr);
    cudaPointerAttributes at;
    void* base = nullptr;
    size_t alloc_len = 0;
    if (cudaPointerGetAttributes(&at, buf) != cudaSuccess || at.type != cudaMemoryTypeDevice ||
        !alloc_range(buf, &base, &alloc_len)) {
      cudaGetLastError();
      *bad = w;
      return URMA_EINVAL;   // receive buffers of this provider are device memory
    }
    std::lock_guard<std::mutex> l(j->mu);
    const uint64_t t = j->shm->rq_tail.load(std::memory_order_relaxed);
    if (t - j->shm->rq_head.load(std::memory_order_acquire) >= kRq) {
      *bad = w;
      return URMA_EAGAIN;
    }
    RecvSlot& sl = j->shm->rq[t % kRq];
    if (sl.state.load(std::memory_order_acquire) != 0) {   // the sender that took it has not let go of it yet
      *bad = w;
      return URMA_EAGAIN;
    }
    if (cudaIpcGetMemHandle(&sl.handle, base) != cudaSuccess) {
      cudaGetLastError();
      *bad = w;
      return URMA_FAIL;
    }
    sl.pid = getpid();
    sl.dev = c->dev;
    sl.len = w->src.sge[0].len;
    sl.user_ctx = w->user_ctx;
    sl.va = w->src.sge[0].addr;
    sl.alloc_base = reinterpret_cast<uint64_t>(base);
    sl.state.store(1, std::memory_order_release);
    j->shm->rq_tail.store(t + 1, std::memory_order_release);
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}

int op_poll_jfc(urma_jfc_t* jfc, int n, urma_cr_t* cr) {
  static thread_local std::vector<CJetty*> js;   // reused: a poll must not allocate
  {
    std::lock_guard<std::mutex> l(g_jmu);
    js = g_jfc_jetties[jfc];
  }
  int k = 0;
  for (CJetty* j : js) {
    std::lock_guard<std::mutex> l(j->mu);
    while (k < n && !j->inflight.empty()) {
      Req& r = j->inflight.front();
      urma_cr_status_t st = r.early;
      if (st == URMA_CR_SUCCESS) {
        const cudaError_t q = cudaEventQuery(r.ev);
        if (q == cudaErrorNotReady) break;  // completions are delivered in order per jetty
        event_put(C(jfc->ctx), r.ev);
        if (q != cudaSuccess) st = URMA_CR_LOC_OPERATION_ERR;
        if (r.rx) {   // the payload has landed: hand the receiver its completion
          const uint64_t t = r.rx->cq_tail.fetch_add(1);
          RecvComp& cc = r.rx->cq[t % kRcq];
          cc.status = q == cudaSuccess ? (uint32_t)URMA_CR_SUCCESS : (uint32_t)URMA_CR_REM_OPERATION_ERR;
          cc.len = r.len;
          cc.opcode = r.rx_opcode;
          cc.user_ctx = r.rx_user_ctx;
          cc.imm = r.imm;
          cc.remote.eid = j->pub.jetty_id.eid;
          cc.remote.uasid = j->pub.jetty_id.uasid;
          cc.remote.id = j->id;
          cc.state.store(2, std::memory_order_release);
        }
        if (q == cudaSuccess && r.old_host && r.result_addr) {
          // the caller's result buffer may be host or device memory
          cudaMemcpy(reinterpret_cast<void*>(r.result_addr), r.old_host, 8, cudaMemcpyDefault);
        }
      }
      if ((r.flag & URMA_WR_FLAG_COMPLETE_ENABLE) || st != URMA_CR_SUCCESS) {
        cr[k] = urma_cr_t{};
        cr[k].status = st;
        cr[k].user_ctx = r.user_ctx;
        cr[k].completion_len = r.len;
        cr[k].local_id = r.local_id;
        cr[k].remote_id = r.remote;
        ++k;
      }
      j->inflight.pop_front();
    }
    // receive side: completions that senders left in this jetty's ring
    if (j->shm && j->rx_jfc == jfc) {
      while (k < n) {
        const uint64_t h = j->shm->cq_head.load(std::memory_order_relaxed);
        RecvComp& cc = j->shm->cq[h % kRcq];
        if (cc.state.load(std::memory_order_acquire) != 2) break;
        cr[k] = urma_cr_t{};
        cr[k].status = static_cast<urma_cr_status_t>(cc.status);
        cr[k].user_ctx = cc.user_ctx;
        cr[k].opcode = static_cast<urma_cr_opcode_t>(cc.opcode);
        cr[k].flag = URMA_CR_FLAG_RECV;
        cr[k].completion_len = cc.len;
        cr[k].local_id = j->id;
        cr[k].remote_id = cc.remote;
        cr[k].imm_data = cc.imm;
        ++k;
        cc.state.store(0, std::memory_order_release);
        j->shm->cq_head.store(h + 1, std::memory_order_release);
      }
    }
  }
  return k;
}

int op_user_ctl(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out) {
  // opcode 1: out->addr = the context's CUDA stream (so callers can order their kernels against posted copies)
  if (in->opcode == 1) {
    out->addr = reinterpret_cast<uint64_t>(C(ctx)->stream);
    return 0;
  }
  return -1;
}

const urma_ops_t g_ops = {
    "cuda_ipc",
    op_create_jfc, op_modify_jfc, op_delete_jfc, nullptr, nullptr,
    nullptr, nullptr, nullptr, nullptr, nullptr,
    nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
    op_create_jetty, op_modify_jetty, op_query_jetty, nullptr, op_delete_jetty,
    op_import_jetty, op_unimport_jetty, op_bind, op_unbind, nullptr, nullptr,
    op_alloc_token, op_free_token, op_register_seg, op_unregister_seg, op_import_seg, op_unimport_seg,
    nullptr, nullptr, op_post_send, op_post_recv, op_poll_jfc, nullptr, nullptr, nullptr,
    nullptr, nullptr, op_user_ctl,
};

urma_status_t prov_init(const urma_init_attr_t*) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  g_ndev = n;
  return URMA_SUCCESS;
}
urma_status_t prov_uninit(void) { return URMA_SUCCESS; }
int prov_get_devices(urma_device_t* devs, int max) {
  int n = 0;
  for (int i = 0; i < g_ndev && n < max; ++i, ++n) {
    memset(&devs[n], 0, sizeof(urma_device_t));
    snprintf(devs[n].name, sizeof(devs[n].name), "cuda%d", i);
    memcpy(devs[n].eid.raw, "cuda", 4);
    devs[n].eid.raw[15] = static_cast<uint8_t>(i + 1);
    devs[n].priv = reinterpret_cast<void*>(static_cast<intptr_t>(i));
  }
  return n;
}
urma_status_t prov_query(const urma_device_t*, urma_device_attr_t* a) {
  memset(a, 0, sizeof(*a));
  a->max_jfc = a->max_jetty = 65536;
  a->max_seg = kDirEntries;
  a->max_jfc_depth = a->max_jfs_depth = 65536;
  a->max_sge = 1;
  a->max_msg_size = 1ull << 36;
  a->transport_modes = URMA_TM_RM;
  a->port_cnt = 18;  // NVLink 5 links per GPU
  a->atomic_supported = true;
  return URMA_SUCCESS;
}
urma_context_t* prov_create_context(urma_device_t* dev, uint32_t) {
  if (!dir()) return nullptr;
  CCtx* c = new CCtx();
  c->dev = static_cast<int>(reinterpret_cast<intptr_t>(dev->priv));
  if (cudaSetDevice(c->dev) != cudaSuccess || cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaHostAlloc(reinterpret_cast<void**>(&c->pinned), 1024 * 8, cudaHostAllocMapped) != cudaSuccess) {
    cudaGetLastError();
    delete c;
    return nullptr;
  }
  c->pub.ops = &g_ops;
  c->pub.eid = dev->eid;
  c->pub.uasid = dir()->next_uasid.fetch_add(1) + 1;
  c->pub.priv = c;
  c->pub.async_fd = -1;
  return &c->pub;
}
urma_status_t prov_delete_context(urma_context_t* ctx) {
  CCtx* c = C(ctx);
  cudaSetDevice(c->dev);
  cudaStreamSynchronize(c->stream);
  cudaStreamDestroy(c->stream);
  cudaFreeHost(c->pinned);
  for (cudaEvent_t e : c->ev_free) cudaEventDestroy(e);
  delete c;
  return URMA_SUCCESS;
}

const urma_provider_ops_t g_prov = {"cuda_ipc", prov_init,           prov_uninit,        prov_get_devices,
                                    prov_query, prov_create_context, prov_delete_context};
__attribute__((constructor)) void cuda_ipc_provider_ctor() { urma_register_provider_ops(&g_prov); }

}  // namespace
