// UMQ implementation over URMA jetties.
//
// What is kept from the reference (src/urpc/umq): handle-based queues created from an option struct and connected
// by exchanging an opaque bind blob (umq_api.c, umq_ub_private.h:344-349); message buffers handed out by a pool with
// fixed block sizes of 8/16/32/64 KiB, per-thread caches in front of a global pool and a separate path for huge
// requests up to 10 MiB (qbuf/umq_qbuf_pool.c, umq_huge_qbuf_pool.c); the base API (enqueue / dequeue) and the pro
// API (post / poll per direction); control information carried in the immediate data of two-sided messages
// (umq_ub_imm_data.h:20-103); credit-based flow control in which the receiver grants one credit per posted receive
// buffer and returns credits in batches (flow_control/umq_ub_flow_control.c; doc/en/urpc/UMQ Flowcontrol.md);
// io / flow-control / pool statistics and latency records (umq_dfx_api.h).
#include "umq_api.h"

#include <stdlib.h>
#include <string.h>
#include <sys/eventfd.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <algorithm>
#include <deque>
#include <map>
#include <memory>
#include <thread>
#include <mutex>
#include <random>
#include <shared_mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "ub_util.h"
#include "urma_simple.h"
#include "uvs_topo.h"

namespace {

// immediate data layout: [63:56] type, [55:40] credits returned, [39:24] sub-queue the message is for (0 = the
// queue that owns the endpoint), [23:0] message bytes or the cookie of a pull message
// IMM_PULL_REQ: the payload is a PullDesc - the message itself stays in the sender's memory and the receiver fetches
// it with a one-sided read (messages larger than the peer's receive buffers); IMM_PULL_DONE / IMM_PULL_FAIL: the
// receiver is through with the read (low 32 bits = the descriptor's cookie), the sender's buffer completes.
enum ImmType : uint64_t { IMM_IO = 1, IMM_FC_RETURN = 2, IMM_PULL_REQ = 3, IMM_PULL_DONE = 4, IMM_PULL_FAIL = 5 };
struct PullDesc {
  uint32_t magic, cookie, token, len;
  uint64_t addr;
  uint8_t seg[URMA_SIMPLE_SEG_BLOB];
};
constexpr uint32_t kPullMagic = 0x50554c4c;   // "PULL"
inline uint64_t imm_make(ImmType t, uint32_t credits, uint32_t bytes, uint32_t dst_sub = 0) {
  return (uint64_t(t) << 56) | (uint64_t(credits & 0xffff) << 40) | (uint64_t(dst_sub & 0xffff) << 24) |
         (bytes & 0xffffff);
}
inline uint32_t imm_credits(uint64_t imm) { return static_cast<uint32_t>((imm >> 40) & 0xffff); }
inline uint32_t imm_sub(uint64_t imm) { return static_cast<uint32_t>((imm >> 24) & 0xffff); }
inline uint32_t imm_low(uint64_t imm) { return static_cast<uint32_t>(imm & 0xffffff); }

struct Block {
  umq_buf_t meta;  // must be first: umq_buf_t* <-> Block*
  bool huge;
  bool tiny;       // comes from the tiny pool (small control / RPC messages)
  char* mem;
  uint32_t cap;
  uint32_t gen;    // pool generation the block was made in (blocks of an older generation are freed on return)
  Block* fl_prev = nullptr;   // links of the owning queue's in-flight list (under that queue's lock)
  Block* fl_next = nullptr;
  bool in_fl = false;
};
// The blocks an endpoint owns at the moment (posted receives, sends not yet completed), as a list threaded through
// the blocks themselves: every message enters and leaves it once, so it must cost neither an allocation nor a hash.
struct FlightList {
  Block* head = nullptr;
  uint32_t n = 0;
  void insert(Block* b) {
    if (b->in_fl) return;
    b->in_fl = true;
    b->fl_prev = nullptr;
    b->fl_next = head;
    if (head) head->fl_prev = b;
    head = b;
    ++n;
  }
  void erase(Block* b) {
    if (!b->in_fl) return;
    b->in_fl = false;
    if (b->fl_prev) b->fl_prev->fl_next = b->fl_next;
    else head = b->fl_next;
    if (b->fl_next) b->fl_next->fl_prev = b->fl_prev;
    b->fl_prev = b->fl_next = nullptr;
    --n;
  }
  bool empty() const { return n == 0; }
  uint32_t size() const { return n; }
};

// Tiny pool: requests of at most kTinyBytes (headers, acknowledgements, small RPC arguments) are served from blocks
// of that size carved out of large slabs, so that a flood of small messages does not pin one 8-64 KiB block each. It
// has its own free list and per-thread cache and grows slab by slab. Counterpart of the reference's tiny buffer pool
// (src/urpc/umq/qbuf/umq_tiny_qbuf_pool.c).
constexpr uint32_t kTinyBytes = 512;
constexpr uint32_t kTinyPerSlab = 1024;
struct TinyPool {
  std::mutex mu;
  std::vector<Block*> free_list;
  std::vector<char*> slabs;      // data slabs of kTinyPerSlab * kTinyBytes
  std::vector<Block*> desc_slabs;
  uint64_t total = 0, allocs = 0, frees = 0, max_total = 1u << 20;
};
TinyPool g_tiny;

struct Pool {
  std::mutex mu;
  uint32_t block = 8192;
  std::vector<Block*> free_list;
  std::vector<char*> slabs;
  uint64_t total = 0, huge_allocs = 0, alloc_calls = 0, free_calls = 0, failures = 0;
  uint64_t max_total = 0, grown = 0;   // growth cap in blocks; blocks added after pool_init
  bool inited = false;
  std::map<const char*, Block*> by_mem;   // data area -> descriptor (umq_data_to_head)
  uint64_t generation = 0;
};
Pool g_pool;
// Per-thread cache of free blocks. A thread that ends hands its cached blocks back to the global pool (a worker
// thread that polled a queue for a while would otherwise take them with it).
struct ThreadCache {
  std::vector<Block*> v;
  ~ThreadCache();
};
thread_local ThreadCache t_cache_holder;
#define t_cache (t_cache_holder.v)
ThreadCache::~ThreadCache() {
  std::lock_guard<std::mutex> l(g_pool.mu);
  for (Block* b : v) g_pool.free_list.push_back(b);
  v.clear();
}
struct TinyCache {
  std::vector<Block*> v;
  ~TinyCache() {
    std::lock_guard<std::mutex> l(g_tiny.mu);
    for (Block* b : v) g_tiny.free_list.push_back(b);
    v.clear();
  }
};
thread_local TinyCache t_tiny_holder;
#define t_tiny (t_tiny_holder.v)
constexpr size_t kCacheMax = 64;

struct Global {
  std::mutex mu;
  bool inited = false;
  umq_init_cfg_t cfg{};
  urma_context_t* ctx = nullptr;
  std::unordered_map<uint64_t, struct Queue*> queues;
  std::atomic<uint64_t> next_h{1};
  std::atomic<bool> perf_on{false};
  std::mutex perf_mu;
  ub::PerfHist perf[UMQ_PERF_RECORD_MAX];
};
Global g;
ub::Logger g_log("UMQ");

// Asynchronous events (queue went into the error state): a bounded FIFO the application drains with
// umq_async_event_get, like the reference's UMQ_EVENT_QH_ERR (doc/en/urpc/UMQ Abnormal Event.md).
std::mutex g_ev_mu;
std::deque<umq_async_event_t> g_events;
int g_ev_fd = -1;   // created on demand by umq_async_event_fd_get; readable while events are queued
void push_event(umq_async_event_type_t type, uint64_t h, int detail) {
  std::lock_guard<std::mutex> l(g_ev_mu);
  if (g_events.size() >= 1024) g_events.pop_front();
  g_events.push_back(umq_async_event_t{type, h, detail});
  if (g_ev_fd >= 0) {
    const uint64_t one = 1;
    if (write(g_ev_fd, &one, sizeof(one)) < 0) {
      // counter saturated: the fd is readable anyway
    }
  }
}
std::atomic<umq_io_perf_cb_t> g_perf_cb{nullptr};
std::atomic<void*> g_perf_cb_ctx{nullptr};

// Trace: every thread owns a single-producer ring of {start, duration, record point} entries; a flusher thread wakes on
// a timer, drains all rings and appends one text line per entry to the trace file. A full ring drops (and counts)
// new entries instead of blocking the data path. Same shape as the reference's per-thread trace rings flushed by a
// timer (src/urpc/umq/dfx/trace.c:72-526).
struct TraceRec {
  uint64_t t0, dt;
  uint32_t rec, pad;
};
struct TraceRing {
  std::vector<TraceRec> buf;
  std::atomic<uint64_t> head{0}, tail{0};   // head: next slot the owner writes; tail: next slot the flusher reads
  std::atomic<uint64_t> dropped{0};
  uint64_t tid = 0;
};
struct Trace {
  std::atomic<bool> on{false};
  std::mutex mu;                            // guards rings, file, thread
  std::vector<std::shared_ptr<TraceRing>> rings;
  FILE* file = nullptr;
  std::thread flusher;
  std::atomic<bool> stop{false};
  uint32_t interval_ms = 100, ring_entries = 4096;
  std::atomic<uint64_t> generation{0};      // bumped at every start: threads re-register their ring
  std::atomic<uint64_t> written{0};
};
Trace g_trace;
const char* const kRecordNames[UMQ_PERF_RECORD_MAX] = {"enqueue", "dequeue", "post_tx", "poll_rx", "buf_alloc"};

TraceRing* my_trace_ring() {
  thread_local std::shared_ptr<TraceRing> ring;
  thread_local uint64_t ring_gen = 0;
  const uint64_t gen = g_trace.generation.load(std::memory_order_acquire);
  if (!ring || ring_gen != gen) {
    auto r = std::make_shared<TraceRing>();
    r->buf.resize(g_trace.ring_entries);
    r->tid = static_cast<uint64_t>(syscall(SYS_gettid));
    std::lock_guard<std::mutex> l(g_trace.mu);
    if (!g_trace.on.load()) return nullptr;
    g_trace.rings.push_back(r);
    ring = r;
    ring_gen = gen;
  }
  return ring.get();
}

void trace_add(int rec, uint64_t t0, uint64_t dt) {
  TraceRing* r = my_trace_ring();
  if (!r) return;
  const uint64_t h = r->head.load(std::memory_order_relaxed);
  if (h - r->tail.load(std::memory_order_acquire) >= r->buf.size()) {
    r->dropped.fetch_add(1, std::memory_order_relaxed);
    return;
  }
  r->buf[h % r->buf.size()] = TraceRec{t0, dt, static_cast<uint32_t>(rec), 0};
  r->head.store(h + 1, std::memory_order_release);
}

// Caller holds g_trace.mu.
void trace_drain_locked() {
  if (!g_trace.file) return;
  for (auto& r : g_trace.rings) {
    uint64_t t = r->tail.load(std::memory_order_relaxed);
    const uint64_t h = r->head.load(std::memory_order_acquire);
    for (; t < h; ++t) {
      const TraceRec& e = r->buf[t % r->buf.size()];
      fprintf(g_trace.file, "%llu %llu %s %llu\n", (unsigned long long)e.t0, (unsigned long long)r->tid,
              e.rec < UMQ_PERF_RECORD_MAX ? kRecordNames[e.rec] : "?", (unsigned long long)e.dt);
      g_trace.written.fetch_add(1, std::memory_order_relaxed);
    }
    r->tail.store(t, std::memory_order_release);
  }
  fflush(g_trace.file);
}

void trace_flush_loop() {
  while (!g_trace.stop.load()) {
    for (uint32_t slept = 0; slept < g_trace.interval_ms && !g_trace.stop.load(); slept += 5) usleep(5000);
    std::lock_guard<std::mutex> l(g_trace.mu);
    trace_drain_locked();
  }
}

// Call-latency histograms are kept per thread (as the reference keeps its cycle histograms per thread,
// src/urpc/umq/dfx/perf.c): recording takes only the recording thread's own lock, which nobody else holds except a
// reader for the moment of its merge. A restart (umq_stats_perf_start / reset) moves an epoch; a thread clears its
// tables when it next records, and a reader skips tables of an older epoch. A thread that ends leaves its counts in
// the process-wide table.
struct ThreadPerf {
  std::mutex mu;
  uint64_t epoch = 0;
  ub::PerfHist h[UMQ_PERF_RECORD_MAX];
};
std::atomic<uint64_t> g_perf_epoch{1};
std::vector<ThreadPerf*>& perf_threads() {   // under g.perf_mu
  static std::vector<ThreadPerf*>* v = new std::vector<ThreadPerf*>();
  return *v;
}
struct ThreadPerfHolder {
  ThreadPerf* tp = nullptr;
  ThreadPerf* get() {
    if (!tp) {
      tp = new ThreadPerf();
      std::lock_guard<std::mutex> l(g.perf_mu);
      perf_threads().push_back(tp);
    }
    return tp;
  }
  ~ThreadPerfHolder() {
    if (!tp) return;
    std::lock_guard<std::mutex> l(g.perf_mu);
    if (tp->epoch == g_perf_epoch.load())
      for (int i = 0; i < UMQ_PERF_RECORD_MAX; ++i) g.perf[i].merge(tp->h[i]);
    auto& v = perf_threads();
    for (size_t i = 0; i < v.size(); ++i)
      if (v[i] == tp) {
        v[i] = v.back();
        v.pop_back();
        break;
      }
    delete tp;
  }
};
thread_local ThreadPerfHolder t_perf;
inline void perf_record(int rec, uint64_t dt) {
  ThreadPerf* tp = t_perf.get();
  std::lock_guard<std::mutex> l(tp->mu);
  const uint64_t ep = g_perf_epoch.load(std::memory_order_acquire);
  if (tp->epoch != ep) {
    for (auto& h : tp->h) h.reset();
    tp->epoch = ep;
  }
  tp->h[rec].add(dt);
}
// Everything recorded since the last restart, merged into `out[UMQ_PERF_RECORD_MAX]`. Caller holds g.perf_mu.
void perf_collect(ub::PerfHist* out) {
  const uint64_t ep = g_perf_epoch.load(std::memory_order_acquire);
  for (int i = 0; i < UMQ_PERF_RECORD_MAX; ++i) out[i] = g.perf[i];
  for (ThreadPerf* tp : perf_threads()) {
    std::lock_guard<std::mutex> l(tp->mu);
    if (tp->epoch != ep) continue;
    for (int i = 0; i < UMQ_PERF_RECORD_MAX; ++i) out[i].merge(tp->h[i]);
  }
}
// Forgets everything recorded so far. Caller holds g.perf_mu.
void perf_restart() {
  for (auto& h : g.perf) h.reset();
  g_perf_epoch.fetch_add(1, std::memory_order_acq_rel);
}

struct PerfScope {
  int rec;
  uint64_t t0;
  explicit PerfScope(int r)
      : rec(r), t0((g.perf_on.load(std::memory_order_relaxed) || g_trace.on.load(std::memory_order_relaxed) ||
                    g_perf_cb.load(std::memory_order_relaxed))
                       ? ub::now_ns() : 0) {}
  ~PerfScope() {
    if (t0) {
      const uint64_t dt = ub::now_ns() - t0;
      if (g_trace.on.load(std::memory_order_relaxed)) trace_add(rec, t0, dt);
      if (umq_io_perf_cb_t cb = g_perf_cb.load(std::memory_order_relaxed)) cb(rec, dt, g_perf_cb_ctx.load());
      if (g.perf_on.load(std::memory_order_relaxed)) perf_record(rec, dt);
    }
  }
};

struct Queue {
  uint64_t h;
  umq_create_option_t opt;
  const umq_transport_ops_t* tops = nullptr;   // non-null: served by a table entry instead of the URMA code below
  void* tpriv = nullptr;
  urma_simple_ep_t* ep = nullptr;
  urma_target_jetty_t* peer = nullptr;
  std::atomic<int> state{UMQ_STATE_IDLE};
  std::mutex mu;
  std::deque<umq_buf_t*> rx_ready;      // received messages not yet dequeued
  std::deque<umq_buf_t*> tx_done;       // sent buffers whose completion arrived (pro API)
  uint32_t rx_posted = 0;
  FlightList in_flight;  // blocks owned by the endpoint: posted receives, sends not yet completed
  // flow control
  bool fc = false;
  int64_t credits = 0;          // messages we may still send
  uint32_t to_return = 0;       // credits owed to the peer
  uint32_t fc_skip = 0;         // receive buffers consumed by control messages: re-posting them grants nothing
  uint32_t window = 0;
  umq_io_stats_t io{};
  umq_fc_stats_t fcs{};
  bool base_api_tx = true;      // enqueue frees buffers on completion; post hands them back through poll
  // one-sided reads issued with umq_remote_read: completion statuses by read id (ids are odd, see progress())
  std::unordered_map<uint64_t, int> read_done;
  uint64_t next_read = 1;
  std::map<std::string, urma_target_seg_t*> imported;   // peer segments, by blob
  // large-message pull path (a message that does not fit the peer's receive buffers)
  uint32_t peer_rx_buf = 0;     // from the peer's bind information
  uint32_t next_cookie = 1;
  struct PullTx {               // sender: message waiting for the receiver's read
    struct Block* block;
    urma_target_seg_t* seg;
  };
  struct PullRx {               // receiver: read in flight into `block`
    struct Block* block;
    urma_target_seg_t* rseg;
    uint32_t cookie;
  };
  std::unordered_map<uint32_t, PullTx> pull_tx;    // by cookie
  std::unordered_map<uint64_t, PullRx> pull_rx;    // by read id
  // main / sub queues. A sub queue has no endpoint: it receives through its main queue's shared receive buffers
  // (the sender names it in the immediate data) and sends through an endpoint borrowed from the jetty pool.
  // Lock order: a sub queue's `mu`, then a main queue's `mu`; a main queue reaches its subs only through `inbox`.
  Queue* main = nullptr;            // sub queue: the queue whose receive side it shares
  uint32_t sub_id = 0;              // sub queue: its number inside the main queue (travels in the bind information)
  uint32_t peer_sub = 0;            // destination number for what this queue sends (0: the peer is a plain queue)
  std::unordered_map<uint32_t, Queue*> subs;   // main queue: sub queues by number (under mu)
  uint32_t next_sub = 1;
  bool in_pool = false;             // main queue: its endpoint serves the jetty pool
  bool closing = false;             // main queue: being destroyed, takes no new sub queues (under mu)
  struct Event {
    int kind;                       // 0 receive, 1 read done, 2 send done
    int st;
    uint64_t uc;
    uint32_t len;
    uint64_t imm;
  };
  std::mutex inbox_mu;              // leaf lock
  std::vector<Event> inbox;         // completions another queue's progress found for this one
};
constexpr uint64_t kRxPending = 1;   // umq_buf_t::rsvd[1] of a queued receive whose data is still being read

// Every call of the API starts with a look-up by handle, from every thread that drives a queue: the table's mutex
// would be the one lock all of them meet on. A direct-mapped front (handle modulo its size) answers without it. An
// entry is a (tag, pointer) pair that only changes under g.mu: the writer takes the tag down, swaps the pointer,
// puts the new tag up; a reader trusts the pointer only if the tag read the same before and after.
constexpr uint32_t kQHints = 256;
struct QHint {
  std::atomic<uint64_t> h{0};
  std::atomic<Queue*> q{nullptr};
};
QHint g_qhint[kQHints];
void qhint_set(uint64_t h, Queue* q) {   // caller holds g.mu
  QHint& e = g_qhint[h & (kQHints - 1)];
  e.h.store(0, std::memory_order_release);
  e.q.store(q, std::memory_order_release);
  e.h.store(h, std::memory_order_release);
}
void qhint_drop(uint64_t h) {   // caller holds g.mu
  QHint& e = g_qhint[h & (kQHints - 1)];
  if (e.h.load(std::memory_order_relaxed) == h) {
    e.h.store(0, std::memory_order_release);
    e.q.store(nullptr, std::memory_order_release);
  }
}
Queue* find(uint64_t h) {
  QHint& e = g_qhint[h & (kQHints - 1)];
  if (h && e.h.load(std::memory_order_acquire) == h) {
    Queue* q = e.q.load(std::memory_order_acquire);
    if (q && e.h.load(std::memory_order_acquire) == h) return q;
  }
  std::lock_guard<std::mutex> l(g.mu);
  auto it = g.queues.find(h);
  if (it == g.queues.end()) return nullptr;
  qhint_set(h, it->second);
  return it->second;
}
// Hands a completion to the queue with handle `h` if it still exists. The table lock is held across look-up and
// hand-over, so a queue that is being destroyed (erased from the table first, deleted afterwards) either still gets
// the event and frees it with its inbox, or is no longer found.
bool forward_to_handle(uint64_t h, const Queue::Event& e) {
  std::lock_guard<std::mutex> l(g.mu);
  auto it = g.queues.find(h);
  if (it == g.queues.end()) return false;
  std::lock_guard<std::mutex> il(it->second->inbox_mu);
  it->second->inbox.push_back(e);
  return true;
}

// ------------------------------------------------------------------------------------------------ buffers
Block* block_new(uint32_t cap, bool huge) {
  Block* b = static_cast<Block*>(calloc(1, sizeof(Block)));
  if (!b) return nullptr;
  b->mem = static_cast<char*>(malloc(cap));
  if (!b->mem) {
    free(b);
    return nullptr;
  }
  b->cap = cap;
  b->huge = huge;
  return b;
}
std::atomic<uint32_t> g_pool_gen{1};
void block_destroy(Block* b) {   // caller holds g_pool.mu
  g_pool.by_mem.erase(b->mem);
  free(b->mem);
  free(b);
}
void pool_init(uint32_t block, uint64_t bytes) {
  std::lock_guard<std::mutex> l(g_pool.mu);
  if (g_pool.inited && g_pool.block == block) return;
  if (g_pool.inited) {
    // A new umq_init after umq_uninit asks for another block size: start a new generation. Free blocks go now, blocks
    // still held by an application or parked in a thread's cache go when they come back.
    g_pool_gen.fetch_add(1);
    for (Block* b : g_pool.free_list) block_destroy(b);
    g_pool.free_list.clear();
    for (Block* b : t_cache) block_destroy(b);
    t_cache.clear();
    g_pool.total = 0;
    g_pool.grown = 0;
    ++g_pool.generation;
  }
  g_pool.block = block;
  const uint64_t n = bytes / block;
  for (uint64_t i = 0; i < n; ++i) {
    Block* b = block_new(block, false);
    if (!b) break;
    b->gen = g_pool_gen.load();
    g_pool.free_list.push_back(b);
    g_pool.by_mem[b->mem] = b;
    ++g_pool.total;
  }
  g_pool.max_total = n * 16;
  g_pool.inited = true;
}
bool g_tiny_on = true;   // UMQ_TINY_POOL=0 turns it off (every request then takes a full block)
Block* tiny_get() {
  if (!t_tiny.empty()) {
    Block* b = t_tiny.back();
    t_tiny.pop_back();
    return b;
  }
  std::lock_guard<std::mutex> l(g_tiny.mu);
  if (g_tiny.free_list.empty() && g_tiny.total < g_tiny.max_total) {
    char* slab = static_cast<char*>(malloc((size_t)kTinyPerSlab * kTinyBytes));
    Block* descs = static_cast<Block*>(calloc(kTinyPerSlab, sizeof(Block)));
    if (slab && descs) {
      g_tiny.slabs.push_back(slab);
      g_tiny.desc_slabs.push_back(descs);
      for (uint32_t i = 0; i < kTinyPerSlab; ++i) {
        descs[i].tiny = true;
        descs[i].mem = slab + (size_t)i * kTinyBytes;
        descs[i].cap = kTinyBytes;
        g_tiny.free_list.push_back(&descs[i]);
      }
      g_tiny.total += kTinyPerSlab;
      std::lock_guard<std::mutex> lp(g_pool.mu);
      for (uint32_t i = 0; i < kTinyPerSlab; ++i) g_pool.by_mem[descs[i].mem] = &descs[i];
    } else {
      free(slab);
      free(descs);
    }
  }
  for (int i = 0; i < 16 && !g_tiny.free_list.empty(); ++i) {
    t_tiny.push_back(g_tiny.free_list.back());
    g_tiny.free_list.pop_back();
  }
  if (t_tiny.empty()) return nullptr;
  Block* b = t_tiny.back();
  t_tiny.pop_back();
  ++g_tiny.allocs;
  return b;
}
void tiny_put(Block* b) {
  t_tiny.push_back(b);
  if (t_tiny.size() > 128) {
    std::lock_guard<std::mutex> l(g_tiny.mu);
    while (t_tiny.size() > 64) {
      g_tiny.free_list.push_back(t_tiny.back());
      t_tiny.pop_back();
    }
    ++g_tiny.frees;
  }
}

Block* block_get(uint32_t need, bool allow_tiny = false) {
  if (allow_tiny && g_tiny_on && need <= kTinyBytes) {
    if (Block* b = tiny_get()) return b;
  }
  if (need > g_pool.block) {
    if (need > UMQ_MAX_MSG_SIZE) return nullptr;
    Block* b = block_new(need, true);
    std::lock_guard<std::mutex> l(g_pool.mu);
    if (b) {
      ++g_pool.huge_allocs;
      g_pool.by_mem[b->mem] = b;
    } else {
      ++g_pool.failures;
    }
    return b;
  }
  while (!t_cache.empty()) {
    Block* b = t_cache.back();
    t_cache.pop_back();
    if (b->gen == g_pool_gen.load()) return b;
    std::lock_guard<std::mutex> l(g_pool.mu);   // parked here since before the pool was rebuilt
    block_destroy(b);
  }
  std::lock_guard<std::mutex> l(g_pool.mu);
  // refill the thread cache with a small batch
  for (int i = 0; i < 8 && !g_pool.free_list.empty(); ++i) {
    t_cache.push_back(g_pool.free_list.back());
    g_pool.free_list.pop_back();
  }
  // an empty pool grows by a batch, up to 16 times the size it started with (many queues each keep a full receive
  // ring posted; the first size is a floor, not a cap on the number of queues)
  for (int i = 0; t_cache.empty() && i < 8 && g_pool.total < g_pool.max_total; ++i) {
    Block* nb = block_new(g_pool.block, false);
    if (!nb) break;
    nb->gen = g_pool_gen.load();
    g_pool.by_mem[nb->mem] = nb;
    ++g_pool.total;
    ++g_pool.grown;
    t_cache.push_back(nb);
  }
  if (t_cache.empty()) {
    ++g_pool.failures;
    return nullptr;
  }
  Block* b = t_cache.back();
  t_cache.pop_back();
  return b;
}
void block_put(Block* b) {
  if (b->tiny) {
    tiny_put(b);
    return;
  }
  if (b->huge) {
    {
      std::lock_guard<std::mutex> l(g_pool.mu);
      g_pool.by_mem.erase(b->mem);
    }
    free(b->mem);
    free(b);
    return;
  }
  if (b->gen != g_pool_gen.load()) {   // made before the pool was rebuilt with another block size
    std::lock_guard<std::mutex> l(g_pool.mu);
    block_destroy(b);
    return;
  }
  t_cache.push_back(b);
  if (t_cache.size() > kCacheMax) {
    std::lock_guard<std::mutex> l(g_pool.mu);
    while (t_cache.size() > kCacheMax / 2) {
      g_pool.free_list.push_back(t_cache.back());
      t_cache.pop_back();
    }
  }
}
void buf_setup(Block* b, uint64_t h, uint32_t data_size) {
  umq_buf_t* q = &b->meta;
  memset(q, 0, sizeof(*q));
  q->umqh = h;
  q->buf_size = b->cap;
  q->data_size = data_size;
  q->buf_data = b->mem;
}

// ------------------------------------------------------------------------------------------------ rx refill
void refill_rx(Queue* q) {
  while (q->rx_posted < q->opt.rx_depth) {
    Block* b = block_get(q->opt.rx_buf_size);
    if (!b) break;
    buf_setup(b, q->h, 0);
    if (urma_simple_post_recv(q->ep, b->mem, b->cap, reinterpret_cast<uint64_t>(b)) != 0) {
      block_put(b);
      break;
    }
    ++q->rx_posted;
    q->in_flight.insert(b);
    if (q->fc) {
      if (q->fc_skip) --q->fc_skip;
      else ++q->to_return;
    }
  }
}

// -------------------------------------------------------------------------------------------------- jetty pool
// Endpoints of main queues created with UMQ_CREATE_FLAG_SHARE_TRANSPORT. A sub queue borrows one for each message it
// posts (time division at message granularity: any jetty can send to any imported target), so thousands of sub
// queues need only as many jetties as there are main queues. Reference: src/urpc/umq/umq_ub/core/jetty_pool/
// umq_ub_jetty_pool.h:64-102 (shared nodes, availability notification, alloc / free / miss counters).
struct JettyPool {
  std::shared_mutex mu;              // shared: posting through a member; exclusive: members join / leave
  std::vector<Queue*> members;
  std::atomic<uint64_t> allocs{0}, misses{0}, errs{0};
  int efd = -1;                      // counts up whenever a member joins (a jetty became available)
};
JettyPool g_jpool;

// Posts a work request for `q`: on its own endpoint, or - for a sub queue - on a borrowed one. The caller holds
// q->mu (and, for a queue with an endpoint, nothing else).
int q_post(Queue* q, int opcode, urma_target_seg_t* rseg, uint64_t raddr, uint64_t laddr, uint32_t len, uint64_t imm,
           uint64_t uc, int signaled) {
  if (q->ep) return urma_simple_post(q->ep, q->peer, opcode, rseg, raddr, nullptr, laddr, len, imm, uc, signaled);
  static thread_local size_t cursor = 0;   // each thread keeps returning to the member that served it last
  std::shared_lock<std::shared_mutex> pl(g_jpool.mu);
  const size_t n = g_jpool.members.size();
  int rc = URMA_EAGAIN;
  for (size_t k = 0; k <= n; ++k) {
    // the pool's members in turn, the queue's own main queue as the last resort (it need not be a member)
    Queue* m = k < n ? g_jpool.members[(cursor + k) % n] : q->main;
    if (k == n && m->in_pool) break;
    if (m->state.load() == UMQ_STATE_ERR) {
      g_jpool.errs.fetch_add(1, std::memory_order_relaxed);
      continue;
    }
    std::lock_guard<std::mutex> ml(m->mu);
    rc = urma_simple_post(m->ep, q->peer, opcode, rseg, raddr, nullptr, laddr, len, imm, uc, signaled);
    if (rc == 0) {
      if (k < n) cursor = (cursor + k) % n;
      g_jpool.allocs.fetch_add(1, std::memory_order_relaxed);
      return 0;
    }
    g_jpool.misses.fetch_add(1, std::memory_order_relaxed);   // its send queue is full: try the next one
  }
  return rc;
}
// Read ids name the queue that issued the read (a borrowed endpoint's owner sees the completion first).
inline uint64_t read_id(Queue* q) { return (((q->h & 0x7fffffffffull) << 24 | (q->next_read++ & 0xffffff)) << 1) | 1; }
inline uint64_t read_id_owner(uint64_t id) { return (id >> 25) & 0x7fffffffffull; }

void send_credit_return(Queue* q) {
  if (!q->fc || !q->peer || q->to_return == 0) return;
  const uint32_t n = std::min<uint32_t>(q->to_return, 0xffff);
  // zero-length control message; it does not consume a credit on the other side's window accounting
  if (q_post(q, URMA_OPC_SEND_IMM, nullptr, 0, 0, 0, imm_make(IMM_FC_RETURN, n, 0, q->peer_sub), 0, 0) == 0) {
    q->to_return -= n;
    q->fcs.credits_returned += n;
  }
}

// ---------------------------------------------------------------------------------------- large-message pull path
// Sender side of a message that does not fit the peer's receive buffers: the block is registered for remote reads
// and only a descriptor travels. The block stays in flight until the receiver reports the end of its read.
// Reference: the UB_PLUS transport's pull of large messages (src/urpc/umq/umq_ub/core/private/umq_pro_ub.c).
void pull_control(Queue* q, ImmType t, uint32_t cookie) {
  q_post(q, URMA_OPC_SEND_IMM, nullptr, 0, 0, 0, imm_make(t, 0, cookie, q->peer_sub), 0, 0);
}
int pull_send(Queue* q, Block* b, uint32_t piggy) {
  PullDesc d{};
  d.magic = kPullMagic;
  d.cookie = q->next_cookie;
  q->next_cookie = q->next_cookie % 0xffffff + 1;   // 24 bits of the immediate data, never 0
  static thread_local std::mt19937 rng{std::random_device{}()};
  d.token = static_cast<uint32_t>(rng()) | 1u;   // one read permission per message
  d.len = b->meta.data_size;
  d.addr = reinterpret_cast<uint64_t>(b->meta.buf_data);
  urma_target_seg_t* seg = urma_simple_seg_register(g.ctx, b->meta.buf_data, d.len, URMA_ACCESS_READ, d.token, d.seg);
  if (!seg) return UMQ_FAIL;
  Block* db = block_get(sizeof(PullDesc));
  if (!db) {
    urma_unregister_seg(seg);
    return UMQ_ERR_ENOMEM;
  }
  buf_setup(db, q->h, sizeof(PullDesc));
  memcpy(db->mem, &d, sizeof(d));
  db->meta.rsvd[0] = 0;   // the descriptor's own block returns to the pool when its send completes
  const int rc = q_post(q, URMA_OPC_SEND_IMM, nullptr, 0, reinterpret_cast<uint64_t>(db->mem), sizeof(PullDesc),
                        imm_make(IMM_PULL_REQ, piggy, sizeof(PullDesc), q->peer_sub), reinterpret_cast<uint64_t>(db), 1);
  if (rc != 0) {
    block_put(db);
    urma_unregister_seg(seg);
    return rc == URMA_EAGAIN ? UMQ_ERR_EAGAIN : UMQ_FAIL;
  }
  q->in_flight.insert(db);
  q->in_flight.insert(b);
  q->pull_tx[d.cookie] = Queue::PullTx{b, seg};
  ++q->io.pull_tx;
  return UMQ_SUCCESS;
}
// The receiver finished (or gave up) its read: the message's buffer completes like any other send.
void pull_finish_tx(Queue* q, uint64_t imm, uint64_t type) {
  auto it = q->pull_tx.find(imm_low(imm));
  if (it == q->pull_tx.end()) return;
  Block* b = it->second.block;
  urma_unregister_seg(it->second.seg);
  q->pull_tx.erase(it);
  q->in_flight.erase(b);
  b->meta.status = type == IMM_PULL_DONE ? UMQ_BUF_OK : UMQ_BUF_SEND_ERR;
  if (type != IMM_PULL_DONE) ++q->io.tx_errors;
  if (b->meta.rsvd[0]) q->tx_done.push_back(&b->meta);
  else block_put(b);
}
// Receiver side: a descriptor arrived in `db`. The destination block takes the message's place in the receive order
// at once (marked pending: dequeue does not pass it) and the read fills it.
void pull_start_rx(Queue* q, Block* db, uint32_t len) {
  PullDesc d;
  if (len < sizeof(d)) {
    ++q->io.rx_errors;
    return;
  }
  memcpy(&d, db->mem, sizeof(d));
  if (d.magic != kPullMagic || d.len == 0 || d.len > UMQ_MAX_MSG_SIZE) {
    ++q->io.rx_errors;
    return;
  }
  Block* dst = block_get(d.len);
  urma_target_seg_t* rseg = dst ? urma_simple_seg_import(g.ctx, d.seg, d.token) : nullptr;
  const uint64_t id = read_id(q);
  if (!dst || !rseg ||
      q_post(q, URMA_OPC_READ, rseg, d.addr, reinterpret_cast<uint64_t>(dst->mem), d.len, 0, id, 1) != 0) {
    if (rseg) urma_unimport_seg(rseg);
    if (dst) block_put(dst);
    ++q->io.rx_errors;
    pull_control(q, IMM_PULL_FAIL, d.cookie);
    return;
  }
  buf_setup(dst, q->h, d.len);
  dst->meta.total_data_size = d.len;
  dst->meta.rsvd[1] = kRxPending;
  q->rx_ready.push_back(&dst->meta);
  q->pull_rx[id] = Queue::PullRx{dst, rseg, d.cookie};
}
// Completion of a read. False when the id is not one of the pull path's.
bool pull_finish_rx(Queue* q, uint64_t id, int status) {
  auto it = q->pull_rx.find(id);
  if (it == q->pull_rx.end()) return false;
  Queue::PullRx r = it->second;
  q->pull_rx.erase(it);
  urma_unimport_seg(r.rseg);
  r.block->meta.rsvd[1] = 0;
  if (status == 0) {
    r.block->meta.status = UMQ_BUF_OK;
    ++q->io.rx_msgs;
    ++q->io.pull_rx;
    q->io.rx_bytes += r.block->meta.data_size;
  } else {   // the message is lost: its place in the order is given up
    ++q->io.rx_errors;
    for (auto p = q->rx_ready.begin(); p != q->rx_ready.end(); ++p)
      if (*p == &r.block->meta) {
        q->rx_ready.erase(p);
        break;
      }
    block_put(r.block);
  }
  pull_control(q, status == 0 ? IMM_PULL_DONE : IMM_PULL_FAIL, r.cookie);
  return true;
}

// One completion, applied to the queue it belongs to. Caller holds q->mu.
void handle_event(Queue* q, const Queue::Event& e) {
  if (e.kind == 0) {   // a message arrived in block e.uc
    Block* b = reinterpret_cast<Block*>(e.uc);
    const uint64_t type = e.imm >> 56;
    const uint32_t credits = imm_credits(e.imm);
    if (credits) {
      q->credits += credits;
      q->fcs.credits_granted += credits;
    }
    if ((type == IMM_PULL_DONE || type == IMM_PULL_FAIL) && e.st == 0) pull_finish_tx(q, e.imm, type);
    if (type == IMM_FC_RETURN || type == IMM_PULL_DONE || type == IMM_PULL_FAIL || e.st != 0) {
      if (e.st != 0) ++q->io.rx_errors;
      else if (q->ep) ++q->fc_skip;
      block_put(b);  // control message or failed receive: the buffer goes straight back
      return;
    }
    if (!q->ep && q->fc) ++q->to_return;   // sub queue: the main queue re-posts the buffer, the credit is ours to give
    if (type == IMM_PULL_REQ) {   // a descriptor: fetch the message it names, keep its place in the order
      pull_start_rx(q, b, e.len);
      block_put(b);
      return;
    }
    b->meta.umqh = q->h;
    b->meta.data_size = e.len;
    b->meta.total_data_size = e.len;
    b->meta.status = UMQ_BUF_OK;
    q->rx_ready.push_back(&b->meta);
    ++q->io.rx_msgs;
    q->io.rx_bytes += e.len;
  } else if (e.kind == 1) {
    // a one-sided read: one of the pull path's, or one the application issued with umq_remote_read
    if (!pull_finish_rx(q, e.uc, e.st)) q->read_done[e.uc] = e.st;
  } else {
    Block* b = reinterpret_cast<Block*>(e.uc);
    q->in_flight.erase(b);
    b->meta.status = e.st == 0 ? UMQ_BUF_OK : UMQ_BUF_SEND_ERR;
    if (e.st != 0) {
      ++q->io.tx_errors;
      if (q->state.exchange(UMQ_STATE_ERR) != UMQ_STATE_ERR) {
        g_log.log(ub::kLogErr, "queue %llu (%s): send completed with status %d, queue set to ERR",
                  (unsigned long long)q->h, q->opt.name, e.st);
        push_event(UMQ_EVENT_QH_ERR, q->h, e.st);
      }
    }
    if (b->meta.rsvd[0]) q->tx_done.push_back(&b->meta);  // pro API: hand back through poll(TX)
    else block_put(b);
  }
}
// Hands a completion to another queue (found while polling this one's endpoint). False: that queue is gone.
bool forward_event(Queue* to, const Queue::Event& e) {
  if (!to) return false;
  std::lock_guard<std::mutex> l(to->inbox_mu);
  to->inbox.push_back(e);
  return true;
}

// Drains the completion queue of the endpoint; caller holds q->mu. What belongs to this queue is applied at once,
// what belongs to a sub queue (or to a queue that borrowed the endpoint) goes to that queue's inbox. A sub queue
// drives its main queue's endpoint first and then empties its own inbox.
void progress(Queue* q) {
  if (!q->ep) {
    if (q->main) {
      std::lock_guard<std::mutex> ml(q->main->mu);
      progress(q->main);
    }
    if (!q->in_flight.empty() || !q->pull_rx.empty()) {
      // work of this queue is outstanding on borrowed endpoints: their completions surface only when the owner's
      // completion queue is polled, and the owner may be idle
      std::shared_lock<std::shared_mutex> pl(g_jpool.mu);
      for (Queue* m : g_jpool.members) {
        if (m == q->main) continue;
        std::unique_lock<std::mutex> ml(m->mu, std::try_to_lock);   // busy = its own thread is polling it right now
        if (ml.owns_lock()) progress(m);
      }
    }
    std::vector<Queue::Event> evs;
    {
      std::lock_guard<std::mutex> l(q->inbox_mu);
      evs.swap(q->inbox);
    }
    for (auto& e : evs) handle_event(q, e);
    if (q->fc && q->to_return >= std::max<uint32_t>(1, q->window / 4)) send_credit_return(q);
    return;
  }
  int st[32];
  uint64_t uc[32], imm[32];
  uint32_t len[32], flag[32];
  for (;;) {
    const int n = urma_simple_poll(q->ep, 32, st, uc, len, imm, flag);
    if (n <= 0) break;
    for (int i = 0; i < n; ++i) {
      Queue::Event e{0, st[i], uc[i], len[i], imm[i]};
      if (flag[i] & URMA_CR_FLAG_RECV) {
        Block* b = reinterpret_cast<Block*>(uc[i]);
        --q->rx_posted;
        q->in_flight.erase(b);
        const uint32_t dst = imm_sub(imm[i]);
        if (dst == 0) {
          handle_event(q, e);
          continue;
        }
        // for a sub queue: the buffer that replaces this one grants nothing to this queue's own peer
        if (q->fc) ++q->fc_skip;
        auto it = q->subs.find(dst);
        if (it == q->subs.end() || !forward_event(it->second, e)) {
          ++q->io.rx_errors;   // nobody of that number (any more)
          block_put(b);
        }
      } else if (uc[i] & 1) {   // reads carry odd ids (buffer descriptors are aligned, so their low bit is 0)
        e.kind = 1;
        const uint64_t owner = read_id_owner(uc[i]);
        if (owner == (q->h & 0x7fffffffffull)) handle_event(q, e);
        else forward_to_handle(owner, e);
      } else if (uc[i] != 0) {
        e.kind = 2;
        Block* b = reinterpret_cast<Block*>(uc[i]);
        if (b->meta.umqh == q->h) handle_event(q, e);
        else if (!forward_to_handle(b->meta.umqh, e)) block_put(b);   // its queue was destroyed
      }
    }
  }
  {   // completions that the owner of another endpoint found for this queue
    std::vector<Queue::Event> evs;
    {
      std::lock_guard<std::mutex> l(q->inbox_mu);
      evs.swap(q->inbox);
    }
    for (auto& e : evs) handle_event(q, e);
  }
  refill_rx(q);
  if (q->fc && q->to_return >= std::max<uint32_t>(1, q->window / 4)) send_credit_return(q);
}

int send_one(Queue* q, umq_buf_t* buf, bool pro) {
  if (q->state.load() != UMQ_STATE_READY || !q->peer) return UMQ_ERR_ESTATE;
  if (buf->data_size > q->opt.rx_buf_size && buf->data_size > g_pool.block) {
    // the peer's receive buffers are at least one block; larger messages need a matching rx_buf_size
  }
  if (q->fc && q->credits <= 0) {
    progress(q);
    if (q->credits <= 0) {
      ++q->fcs.stalls;
      ++q->io.tx_eagain;
      return UMQ_ERR_EAGAIN;
    }
  }
  Block* b = reinterpret_cast<Block*>(buf);
  b->meta.rsvd[0] = pro ? 1 : 0;
  uint32_t piggy = 0;
  if (q->fc && q->to_return) {
    piggy = std::min<uint32_t>(q->to_return, 0xffff);
  }
  b->meta.umqh = q->h;   // the completion finds its queue by this (the endpoint may be a borrowed one)
  if (q->peer_rx_buf && buf->data_size > q->peer_rx_buf) {   // does not fit over there: the peer pulls it
    const int prc = pull_send(q, b, piggy);
    if (prc != UMQ_SUCCESS) {
      ++q->io.tx_eagain;
      return prc;
    }
    if (piggy) {
      q->fcs.credits_returned += piggy;
      q->to_return -= piggy;
    }
    if (q->fc) --q->credits;
    ++q->io.tx_msgs;
    q->io.tx_bytes += buf->data_size;
    return UMQ_SUCCESS;
  }
  const int rc = q_post(q, URMA_OPC_SEND_IMM, nullptr, 0, reinterpret_cast<uint64_t>(buf->buf_data), buf->data_size,
                        imm_make(IMM_IO, piggy, buf->data_size, q->peer_sub), reinterpret_cast<uint64_t>(b), 1);
  if (rc != 0) {
    ++q->io.tx_eagain;
    return rc == URMA_EAGAIN ? UMQ_ERR_EAGAIN : UMQ_FAIL;
  }
  q->in_flight.insert(b);
  if (piggy) {
    q->fcs.credits_returned += piggy;
    q->to_return -= piggy;
  }
  if (q->fc) --q->credits;
  ++q->io.tx_msgs;
  q->io.tx_bytes += buf->data_size;
  return UMQ_SUCCESS;
}

struct BindBlob {
  uint32_t magic, rx_buf_size, rx_depth, fc;
  uint8_t jetty[URMA_SIMPLE_JETTY_BLOB];
  uint32_t token;
  uint32_t sub_id;   // 0: a queue with its own endpoint; else the sub queue's number inside the queue that owns `jetty`
};

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------------------ transports
// In-process transport (mode IPC): queues bound to each other inside one process pass buffers by pointer.
struct LocalQ {
  uint64_t h;
  std::mutex mu;
  std::deque<umq_buf_t*> rx;
  uint64_t peer = 0;
  uint32_t depth = 128;
};
std::mutex g_local_mu;
std::unordered_map<uint64_t, LocalQ*> g_local;
int local_create(uint64_t h, const umq_create_option_t* opt, void** priv) {
  LocalQ* q = new LocalQ();
  q->h = h;
  q->depth = opt->rx_depth ? opt->rx_depth : 128;
  std::lock_guard<std::mutex> l(g_local_mu);
  g_local[h] = q;
  *priv = q;
  return UMQ_SUCCESS;
}
void local_destroy(void* p) {
  LocalQ* q = static_cast<LocalQ*>(p);
  {
    std::lock_guard<std::mutex> l(g_local_mu);
    g_local.erase(q->h);
  }
  for (umq_buf_t* b : q->rx) umq_buf_free(b);
  delete q;
}
uint32_t local_bind_info(void* p, uint8_t* out, uint32_t size) {
  if (size < 16) return 0;
  const uint64_t magic = 0x4c4f43414c514831ull;
  memcpy(out, &magic, 8);
  memcpy(out + 8, &static_cast<LocalQ*>(p)->h, 8);
  return 16;
}
int local_bind(void* p, const uint8_t* info, uint32_t size) {
  uint64_t magic = 0, peer = 0;
  if (size < 16) return UMQ_ERR_EINVAL;
  memcpy(&magic, info, 8);
  memcpy(&peer, info + 8, 8);
  if (magic != 0x4c4f43414c514831ull) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_local_mu);
  if (!g_local.count(peer)) return UMQ_ERR_EINVAL;   // the peer must live in this process
  static_cast<LocalQ*>(p)->peer = peer;
  return UMQ_SUCCESS;
}
int local_unbind(void* p) {
  static_cast<LocalQ*>(p)->peer = 0;
  return UMQ_SUCCESS;
}
int local_send(void* p, umq_buf_t* b) {
  LocalQ* q = static_cast<LocalQ*>(p);
  LocalQ* peer = nullptr;
  {
    std::lock_guard<std::mutex> l(g_local_mu);
    auto it = g_local.find(q->peer);
    if (it == g_local.end()) return UMQ_ERR_ESTATE;
    peer = it->second;
    std::lock_guard<std::mutex> lp(peer->mu);
    if (peer->rx.size() >= peer->depth) return UMQ_ERR_EAGAIN;   // the receiver's ring is full: back-pressure
    b->umqh = peer->h;
    peer->rx.push_back(b);
  }
  return UMQ_SUCCESS;
}
umq_buf_t* local_recv(void* p) {
  LocalQ* q = static_cast<LocalQ*>(p);
  std::lock_guard<std::mutex> l(q->mu);
  if (q->rx.empty()) return nullptr;
  umq_buf_t* b = q->rx.front();
  q->rx.pop_front();
  return b;
}
const umq_transport_ops_t g_local_ops = {"ipc-local", local_create, local_destroy, local_bind_info, local_bind,
                                         local_unbind,  local_send,   local_recv};
constexpr int kMaxModes = 8;
struct TransportTable {
  std::mutex mu;
  const umq_transport_ops_t* ops[kMaxModes] = {nullptr};   // null at index UB: the built-in URMA transport
  TransportTable() { ops[UMQ_TRANS_MODE_IPC] = &g_local_ops; }
};
TransportTable& transports() {
  static TransportTable t;
  return t;
}

int umq_transport_register(umq_trans_mode_t mode, const umq_transport_ops_t* ops) {
  if ((int)mode < 0 || (int)mode >= kMaxModes) return UMQ_ERR_EINVAL;
  if (ops && (!ops->create || !ops->destroy || !ops->bind_info_get || !ops->bind || !ops->send || !ops->recv))
    return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(transports().mu);
  transports().ops[mode] = ops;   // null restores the built-in URMA transport for that mode
  return UMQ_SUCCESS;
}
const char* umq_transport_name(umq_trans_mode_t mode) {
  if ((int)mode < 0 || (int)mode >= kMaxModes) return nullptr;
  std::lock_guard<std::mutex> l(transports().mu);
  return transports().ops[mode] ? transports().ops[mode]->name : "urma";
}

int umq_init(const umq_init_cfg_t* cfg) {
  std::lock_guard<std::mutex> l(g.mu);
  if (g.inited) return UMQ_SUCCESS;
  if (cfg) g.cfg = *cfg;
  const uint32_t kb = g.cfg.block_size_kb ? g.cfg.block_size_kb : 8;
  if (kb != 8 && kb != 16 && kb != 32 && kb != 64) {
    g_log.log(ub::kLogErr, "umq_init: block size %u KB is not one of 8 / 16 / 32 / 64", kb);
    return UMQ_ERR_EINVAL;
  }
  g.ctx = urma_simple_open(g.cfg.dev_name[0] ? g.cfg.dev_name : "shm0");
  if (!g.ctx) {
    g_log.log(ub::kLogErr, "umq_init: device %s cannot be opened", g.cfg.dev_name[0] ? g.cfg.dev_name : "shm0");
    return UMQ_FAIL;
  }
  pool_init(kb * 1024, g.cfg.pool_bytes ? g.cfg.pool_bytes : (64ull << 20));
  if (const char* e = getenv("UMQ_TINY_POOL")) g_tiny_on = !(e[0] == '0');
  g.inited = true;
  return UMQ_SUCCESS;
}

void umq_uninit(void) {
  std::vector<uint64_t> hs;
  {
    std::lock_guard<std::mutex> l(g.mu);
    if (!g.inited) return;
    for (auto& kv : g.queues)
      if (!kv.second->tops && !kv.second->ep) hs.push_back(kv.first);   // sub queues before their main queues
    for (auto& kv : g.queues)
      if (kv.second->tops || kv.second->ep) hs.push_back(kv.first);
  }
  for (uint64_t h : hs) umq_destroy(h);
  std::lock_guard<std::mutex> l(g.mu);
  urma_simple_close(g.ctx);
  g.ctx = nullptr;
  g.inited = false;
}

uint64_t umq_create(const umq_create_option_t* opt) {
  if (!opt || !g.inited) {
    g_log.log(ub::kLogErr, "umq_create: %s", !opt ? "no options given" : "umq_init has not run");
    return UMQ_INVALID_HANDLE;
  }
  Queue* q = new Queue();
  q->opt = *opt;
  if (!q->opt.rx_depth) q->opt.rx_depth = 128;
  if (!q->opt.tx_depth) q->opt.tx_depth = 128;
  if (!q->opt.rx_buf_size) q->opt.rx_buf_size = g_pool.block;
  if (!q->opt.tx_buf_size) q->opt.tx_buf_size = g_pool.block;
  if (q->opt.rx_buf_size > UMQ_MAX_MSG_SIZE) {
    delete q;
    return UMQ_INVALID_HANDLE;
  }
  {
    const int mode = q->opt.transport ? (int)q->opt.transport - 1 : (int)g.cfg.trans_mode;
    if (mode < 0 || mode >= kMaxModes) {
      delete q;
      return UMQ_INVALID_HANDLE;
    }
    std::lock_guard<std::mutex> l(transports().mu);
    q->tops = transports().ops[mode];
  }
  if (q->tops) {
    q->h = g.next_h.fetch_add(1);
    if (q->tops->create(q->h, &q->opt, &q->tpriv) != UMQ_SUCCESS) {
      delete q;
      return UMQ_INVALID_HANDLE;
    }
    std::lock_guard<std::mutex> l(g.mu);
    g.queues[q->h] = q;
    return q->h;
  }
  q->fc = (g.cfg.feature & UMQ_FEATURE_FLOW_CONTROL) != 0;
  if (opt->create_flag & UMQ_CREATE_FLAG_SUB) {
    // no endpoint: receives through the main queue's buffers, sends through the jetty pool
    Queue* m = find(opt->share_rq_umqh);
    if (!m || !m->ep || !(m->opt.create_flag & UMQ_CREATE_FLAG_MAIN)) {
      g_log.log(ub::kLogErr, "umq_create: share_rq_umqh does not name a main queue");
      delete q;
      return UMQ_INVALID_HANDLE;
    }
    q->main = m;
    q->opt.rx_buf_size = m->opt.rx_buf_size;
    q->h = g.next_h.fetch_add(1);
    {
      std::lock_guard<std::mutex> l(m->mu);
      if (m->subs.size() >= 0xfffe || m->closing) {
        delete q;
        return UMQ_INVALID_HANDLE;
      }
      do {
        q->sub_id = m->next_sub;
        m->next_sub = m->next_sub % 0xffff + 1;
      } while (m->subs.count(q->sub_id));
      m->subs[q->sub_id] = q;
    }
    std::lock_guard<std::mutex> l(g.mu);
    g.queues[q->h] = q;
    return q->h;
  }
  // the jetty must hold the data messages plus the occasional credit-return message
  q->ep = urma_simple_ep_create(g.ctx, q->opt.rx_depth + q->opt.tx_depth + 16, opt->token,
                                opt->mode == UMQ_MODE_INTERRUPT);
  if (!q->ep) {
    delete q;
    return UMQ_INVALID_HANDLE;
  }
  q->h = g.next_h.fetch_add(1);
  {
    std::lock_guard<std::mutex> l(q->mu);
    refill_rx(q);
    q->to_return = 0;  // the initial window travels in the bind blob
  }
  {
    std::lock_guard<std::mutex> l(g.mu);
    g.queues[q->h] = q;
  }
  if ((opt->create_flag & UMQ_CREATE_FLAG_MAIN) && (opt->create_flag & UMQ_CREATE_FLAG_SHARE_TRANSPORT)) {
    std::unique_lock<std::shared_mutex> pl(g_jpool.mu);
    g_jpool.members.push_back(q);
    q->in_pool = true;
    if (g_jpool.efd >= 0) {   // a jetty became available
      const uint64_t one = 1;
      if (write(g_jpool.efd, &one, sizeof(one)) < 0) {
        // counter saturated: readable anyway
      }
    }
  }
  return q->h;
}

int umq_destroy(uint64_t h) {
  Queue* q;
  {
    std::lock_guard<std::mutex> l(g.mu);
    auto it = g.queues.find(h);
    if (it == g.queues.end()) return UMQ_ERR_EINVAL;
    q = it->second;
  }
  if (!q->tops && q->ep) {
    // A main queue goes after its sub queues. (The queue's lock is taken without the table lock: progress() looks
    // queues up in the table while it holds a queue's lock.)
    std::lock_guard<std::mutex> ql(q->mu);
    if (!q->subs.empty()) return UMQ_ERR_ESTATE;
    q->closing = true;   // no new sub queue attaches from here on
  }
  {
    std::lock_guard<std::mutex> l(g.mu);
    if (!g.queues.erase(h)) return UMQ_ERR_EINVAL;   // somebody else destroyed it in between
    qhint_drop(h);
  }
  if (!q->tops && q->in_pool) {
    std::unique_lock<std::shared_mutex> pl(g_jpool.mu);   // waits for posts that borrowed the endpoint
    auto& v = g_jpool.members;
    v.erase(std::remove(v.begin(), v.end(), q), v.end());
  }
  if (!q->tops && !q->ep) {   // sub queue
    {
      std::lock_guard<std::mutex> ml(q->main->mu);
      q->main->subs.erase(q->sub_id);
    }
    for (auto& e : q->inbox)
      if (e.kind != 1) block_put(reinterpret_cast<Block*>(e.uc));
    for (auto& kv : q->pull_tx) urma_unregister_seg(kv.second.seg);
    for (auto* b : q->rx_ready) block_put(reinterpret_cast<Block*>(b));
    for (auto* b : q->tx_done) block_put(reinterpret_cast<Block*>(b));
    if (q->peer) urma_unimport_jetty(q->peer);
    // blocks still in flight complete on the endpoint that carried them; its owner returns them to the pool when
    // it finds that their queue is gone
    delete q;
    return UMQ_SUCCESS;
  }
  if (q->tops) {
    q->tops->destroy(q->tpriv);
    delete q;
    return UMQ_SUCCESS;
  }
  // the endpoint goes first: a pull read that is still running must not land in a block that is back in the pool
  urma_simple_ep_destroy(q->ep);
  for (auto& kv : q->pull_rx) urma_unimport_seg(kv.second.rseg);
  for (auto& kv : q->pull_tx) urma_unregister_seg(kv.second.seg);   // their blocks are in in_flight
  for (auto* b : q->rx_ready) block_put(reinterpret_cast<Block*>(b));
  for (auto* b : q->tx_done) block_put(reinterpret_cast<Block*>(b));
  for (auto& kv : q->imported) urma_unimport_seg(kv.second);
  if (q->peer) urma_unimport_jetty(q->peer);
  // the endpoint is gone: nothing can complete into the blocks it still held (posted receives, unfinished sends)
  while (Block* b = q->in_flight.head) {
    q->in_flight.erase(b);
    block_put(b);
  }
  delete q;
  return UMQ_SUCCESS;
}

uint32_t umq_bind_info_get(uint64_t h, uint8_t* out, uint32_t size) {
  Queue* q = find(h);
  if (q && q->tops) return out ? q->tops->bind_info_get(q->tpriv, out, size) : 0;
  if (!q || !out || size < sizeof(BindBlob)) return 0;
  BindBlob b{};
  b.magic = 0x554d5142;
  b.rx_buf_size = q->opt.rx_buf_size;
  b.rx_depth = q->opt.rx_depth;
  b.fc = q->fc;
  b.token = q->ep ? q->opt.token : q->main->opt.token;
  b.sub_id = q->sub_id;
  urma_simple_ep_blob(q->ep ? q->ep : q->main->ep, b.jetty);
  memcpy(out, &b, sizeof(b));
  return sizeof(b);
}

int umq_bind(uint64_t h, const uint8_t* info, uint32_t size) {
  Queue* q = find(h);
  if (q && q->tops) {
    const int rc = info ? q->tops->bind(q->tpriv, info, size) : UMQ_ERR_EINVAL;
    if (rc == UMQ_SUCCESS) q->state = UMQ_STATE_READY;
    return rc;
  }
  if (!q || !info || size < sizeof(BindBlob)) return UMQ_ERR_EINVAL;
  BindBlob b;
  memcpy(&b, info, sizeof(b));
  if (b.magic != 0x554d5142) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  if (q->peer) return UMQ_ERR_ESTATE;
  q->peer = urma_simple_ep_import(g.ctx, b.jetty, b.token);
  if (!q->peer) return UMQ_FAIL;
  q->fc = q->fc && b.fc;
  q->peer_sub = b.sub_id;
  q->peer_rx_buf = b.rx_buf_size;
  q->window = b.rx_depth;
  q->credits = b.rx_depth;  // one credit per receive buffer the peer has posted
  q->fcs.window = b.rx_depth;
  q->state = UMQ_STATE_READY;
  return UMQ_SUCCESS;
}

int umq_unbind(uint64_t h) {
  Queue* q = find(h);
  if (!q) return UMQ_ERR_EINVAL;
  if (q->tops) {
    q->state = UMQ_STATE_IDLE;
    return q->tops->unbind ? q->tops->unbind(q->tpriv) : UMQ_SUCCESS;
  }
  std::lock_guard<std::mutex> l(q->mu);
  if (!q->peer) return UMQ_ERR_ESTATE;
  urma_unimport_jetty(q->peer);
  q->peer = nullptr;
  q->state = UMQ_STATE_IDLE;
  return UMQ_SUCCESS;
}

int umq_state_set(uint64_t h, umq_state_t s) {
  Queue* q = find(h);
  if (!q) return UMQ_ERR_EINVAL;
  const int old = q->state.exchange(s);
  if (s == UMQ_STATE_ERR && old != UMQ_STATE_ERR) push_event(UMQ_EVENT_QH_ERR, h, 0);
  g_log.log(ub::kLogInfo, "queue %llu (%s): state %d -> %d", (unsigned long long)h, q->opt.name, old, (int)s);
  return UMQ_SUCCESS;
}
umq_state_t umq_state_get(uint64_t h) {
  Queue* q = find(h);
  return q ? static_cast<umq_state_t>(q->state.load()) : UMQ_STATE_ERR;
}

umq_buf_t* umq_buf_alloc(uint32_t request_size, uint32_t num, uint64_t h) {
  PerfScope ps(UMQ_PERF_BUF_ALLOC);
  if (num == 0 || num > UMQ_BATCH_SIZE) return nullptr;
  {
    std::lock_guard<std::mutex> l(g_pool.mu);
    ++g_pool.alloc_calls;
  }
  umq_buf_t *head = nullptr, *tail = nullptr;
  for (uint32_t i = 0; i < num; ++i) {
    // application buffers of tiny size come from the tiny pool; receive buffers (posted by the queue itself) and
    // anything larger come from the block pool
    Block* b = block_get(request_size ? request_size : 1, true);
    if (!b) {
      if (head) umq_buf_free(head);
      return nullptr;
    }
    buf_setup(b, h, request_size);
    if (!head) head = &b->meta;
    else tail->qbuf_next = &b->meta;
    tail = &b->meta;
  }
  head->total_data_size = request_size * num;
  return head;
}

void umq_buf_free(umq_buf_t* qbuf) {
  {
    std::lock_guard<std::mutex> l(g_pool.mu);
    ++g_pool.free_calls;
  }
  while (qbuf) {
    umq_buf_t* nx = qbuf->qbuf_next;
    block_put(reinterpret_cast<Block*>(qbuf));
    qbuf = nx;
  }
}

int umq_buf_headroom_reset(umq_buf_t* qbuf, uint16_t headroom) {
  if (!qbuf || headroom > 512) return UMQ_ERR_EINVAL;
  Block* b = reinterpret_cast<Block*>(qbuf);
  if (headroom >= b->cap) return UMQ_ERR_EINVAL;
  qbuf->headroom_size = headroom;
  qbuf->buf_data = b->mem + headroom;
  qbuf->buf_size = b->cap - headroom;
  if (qbuf->data_size > qbuf->buf_size) qbuf->data_size = qbuf->buf_size;
  return UMQ_SUCCESS;
}

int umq_buf_reset(umq_buf_t* qbuf) {
  if (!qbuf) return UMQ_ERR_EINVAL;
  Block* b = reinterpret_cast<Block*>(qbuf);
  qbuf->headroom_size = 0;
  qbuf->buf_data = b->mem;
  qbuf->buf_size = b->cap;
  qbuf->data_size = 0;
  qbuf->status = 0;
  return UMQ_SUCCESS;
}

static int plugin_send_chain(Queue* q, umq_buf_t* qbuf, umq_buf_t** bad) {
  if (q->state.load() != UMQ_STATE_READY) return UMQ_ERR_ESTATE;
  for (umq_buf_t* b = qbuf; b;) {
    umq_buf_t* nx = b->qbuf_next;
    b->qbuf_next = nullptr;
    const uint32_t n = b->data_size;
    const int rc = q->tops->send(q->tpriv, b);
    if (rc != UMQ_SUCCESS) {
      b->qbuf_next = nx;
      if (bad) *bad = b;
      return rc;
    }
    ++q->io.tx_msgs;
    q->io.tx_bytes += n;
    b = nx;
  }
  if (bad) *bad = nullptr;
  return UMQ_SUCCESS;
}

int umq_enqueue(uint64_t h, umq_buf_t* qbuf, umq_buf_t** bad) {
  PerfScope ps(UMQ_PERF_ENQUEUE);
  Queue* q = find(h);
  if (!q || !qbuf) return UMQ_ERR_EINVAL;
  if (!(g.cfg.feature & UMQ_FEATURE_API_BASE) && g.cfg.feature) return UMQ_ERR_EINVAL;
  if (q->tops) return plugin_send_chain(q, qbuf, bad);
  std::lock_guard<std::mutex> l(q->mu);
  for (umq_buf_t* b = qbuf; b;) {
    umq_buf_t* nx = b->qbuf_next;
    b->qbuf_next = nullptr;
    const int rc = send_one(q, b, false);
    if (rc != UMQ_SUCCESS) {
      b->qbuf_next = nx;
      if (bad) *bad = b;
      return rc;
    }
    b = nx;
  }
  if (bad) *bad = nullptr;
  progress(q);
  return UMQ_SUCCESS;
}

umq_buf_t* umq_dequeue(uint64_t h) {
  PerfScope ps(UMQ_PERF_DEQUEUE);
  Queue* q = find(h);
  if (!q) return nullptr;
  if (q->tops) {
    umq_buf_t* b = q->tops->recv(q->tpriv);
    if (b) {
      ++q->io.rx_msgs;
      q->io.rx_bytes += b->data_size;
    }
    return b;
  }
  std::lock_guard<std::mutex> l(q->mu);
  progress(q);
  if (q->rx_ready.empty() || q->rx_ready.front()->rsvd[1] == kRxPending) return nullptr;   // head still being read
  umq_buf_t* b = q->rx_ready.front();
  q->rx_ready.pop_front();
  return b;
}

int umq_post(uint64_t h, umq_buf_t* qbuf, umq_io_direction_t dir, umq_buf_t** bad) {
  PerfScope ps(UMQ_PERF_POST_TX);
  Queue* q = find(h);
  if (!q || !qbuf) return UMQ_ERR_EINVAL;
  if (q->tops) {
    if (dir == UMQ_IO_RX) {   // such transports own their receive side: buffers offered for it are simply returned
      umq_buf_free(qbuf);
      if (bad) *bad = nullptr;
      return UMQ_SUCCESS;
    }
    return plugin_send_chain(q, qbuf, bad);
  }
  if (dir == UMQ_IO_RX && !q->ep) return UMQ_ERR_EINVAL;   // a sub queue's receive buffers are its main queue's
  std::lock_guard<std::mutex> l(q->mu);
  if (dir == UMQ_IO_RX) {
    // application-provided receive buffers (instead of the automatic refill)
    for (umq_buf_t* b = qbuf; b;) {
      umq_buf_t* nx = b->qbuf_next;
      b->qbuf_next = nullptr;
      Block* blk = reinterpret_cast<Block*>(b);
      if (urma_simple_post_recv(q->ep, b->buf_data, b->buf_size, reinterpret_cast<uint64_t>(blk)) != 0) {
        b->qbuf_next = nx;
        if (bad) *bad = b;
        return UMQ_ERR_EAGAIN;
      }
      ++q->rx_posted;
      q->in_flight.insert(blk);
      if (q->fc) ++q->to_return;
      b = nx;
    }
    if (bad) *bad = nullptr;
    return UMQ_SUCCESS;
  }
  for (umq_buf_t* b = qbuf; b;) {
    umq_buf_t* nx = b->qbuf_next;
    b->qbuf_next = nullptr;
    const int rc = send_one(q, b, true);
    if (rc != UMQ_SUCCESS) {
      b->qbuf_next = nx;
      if (bad) *bad = b;
      return rc;
    }
    b = nx;
  }
  if (bad) *bad = nullptr;
  return UMQ_SUCCESS;
}

int umq_poll(uint64_t h, umq_io_direction_t dir, umq_buf_t** bufs, uint32_t max) {
  PerfScope ps(UMQ_PERF_POLL_RX);
  Queue* q = find(h);
  if (!q || !bufs || max == 0) return UMQ_ERR_EINVAL;
  if (q->tops) {
    uint32_t n = 0;
    while (dir == UMQ_IO_RX && n < max) {
      umq_buf_t* b = q->tops->recv(q->tpriv);
      if (!b) break;
      bufs[n++] = b;
    }
    return static_cast<int>(n);
  }
  std::lock_guard<std::mutex> l(q->mu);
  progress(q);
  std::deque<umq_buf_t*>& src = dir == UMQ_IO_RX ? q->rx_ready : q->tx_done;
  uint32_t n = 0;
  while (n < max && !src.empty() && src.front()->rsvd[1] != kRxPending) {   // a message still being read waits
    bufs[n++] = src.front();
    src.pop_front();
  }
  return static_cast<int>(n);
}

// The endpoint whose completion channel wakes the queue: its own, or its main queue's.
static urma_simple_ep_t* event_ep(Queue* q) { return q->ep ? q->ep : (q->main ? q->main->ep : nullptr); }
int umq_rearm_interrupt(uint64_t h, int, umq_io_direction_t) {
  Queue* q = find(h);
  if (!q || !event_ep(q)) return UMQ_ERR_EINVAL;
  return urma_rearm_jfc(urma_simple_ep_jfc(event_ep(q)), false) == URMA_SUCCESS ? UMQ_SUCCESS : UMQ_FAIL;
}
int umq_wait_interrupt(uint64_t h, int timeout_ms) {
  Queue* q = find(h);
  if (!q || !event_ep(q)) return UMQ_ERR_EINVAL;
  urma_jfc_t* jfc = urma_simple_ep_jfc(event_ep(q));
  if (!jfc->cfg.jfce) return UMQ_ERR_EINVAL;
  urma_jfc_t* fired[1];
  return urma_wait_jfc(jfc->cfg.jfce, 1, timeout_ms, fired);
}
void umq_ack_interrupt(uint64_t h, uint32_t nevents) {
  Queue* q = find(h);
  if (!q || !event_ep(q)) return;
  urma_jfc_t* jfc = urma_simple_ep_jfc(event_ep(q));
  urma_ack_jfc(&jfc, &nevents, 1);
}
int umq_interrupt_fd_get(uint64_t h) {
  Queue* q = find(h);
  if (!q || !event_ep(q)) return -1;
  urma_jfc_t* jfc = urma_simple_ep_jfc(event_ep(q));
  return jfc->cfg.jfce ? jfc->cfg.jfce->fd : -1;
}

int umq_stats_io_get(uint64_t h, umq_io_stats_t* out) {
  Queue* q = find(h);
  if (!q || !out) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  *out = q->io;
  return UMQ_SUCCESS;
}
int umq_stats_flow_control_get(uint64_t h, umq_fc_stats_t* out) {
  Queue* q = find(h);
  if (!q || !out) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  q->fcs.credits_local = q->credits > 0 ? q->credits : 0;
  q->fcs.credits_remote = q->to_return;
  *out = q->fcs;
  return UMQ_SUCCESS;
}
int umq_stats_qbuf_pool_get(umq_qbuf_stats_t* out) {
  if (!out) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_pool.mu);
  out->block_size = g_pool.block;
  out->blocks_total = g_pool.total;
  out->blocks_free = g_pool.free_list.size();
  out->huge_allocs = g_pool.huge_allocs;
  out->alloc_calls = g_pool.alloc_calls;
  out->free_calls = g_pool.free_calls;
  out->alloc_failures = g_pool.failures;
  return UMQ_SUCCESS;
}
int umq_stats_perf_start(void) {
  std::lock_guard<std::mutex> l(g.perf_mu);
  perf_restart();
  g.perf_on = true;
  return UMQ_SUCCESS;
}
int umq_stats_perf_stop(void) {
  g.perf_on = false;
  return UMQ_SUCCESS;
}
int umq_stats_perf_get(umq_perf_entry_t* e) {
  if (!e) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g.perf_mu);
  static ub::PerfHist all[UMQ_PERF_RECORD_MAX];   // (under the lock; too large for the stack of a small thread)
  perf_collect(all);
  for (int i = 0; i < UMQ_PERF_RECORD_MAX; ++i) {
    e[i].count = all[i].count();
    e[i].avg_ns = static_cast<uint64_t>(all[i].mean());
    e[i].min_ns = all[i].min();
    e[i].max_ns = all[i].max();
    e[i].p99_ns = all[i].quantile(0.99);
  }
  return UMQ_SUCCESS;
}
// ---------------------------------------------------------------------------------------------- buffer list helpers
int umq_buf_split(umq_buf_t* head, umq_buf_t* node) {
  if (!head || !node || head == node) return UMQ_ERR_EINVAL;
  uint32_t before = 0;
  umq_buf_t* prev = nullptr;
  for (umq_buf_t* b = head; b; prev = b, b = b->qbuf_next) {
    if (b == node) {
      prev->qbuf_next = nullptr;
      uint32_t after = 0;
      for (umq_buf_t* x = node; x; x = x->qbuf_next) after += x->data_size;
      head->total_data_size = before;
      node->total_data_size = after;
      return UMQ_SUCCESS;
    }
    before += b->data_size;
  }
  return UMQ_ERR_EINVAL;  // node is not on the list
}
// A list may hold several messages back to back; the first buffer of each carries the message's total_data_size.
// Frees the buffers of the first message and returns the first buffer of the next one (NULL if there is none).
umq_buf_t* umq_buf_break_and_free(umq_buf_t* qbuf) {
  if (!qbuf) return nullptr;
  uint32_t left = qbuf->total_data_size;
  umq_buf_t* b = qbuf;
  umq_buf_t* last = nullptr;
  do {
    left -= b->data_size < left ? b->data_size : left;
    last = b;
    b = b->qbuf_next;
  } while (b && left > 0);
  last->qbuf_next = nullptr;
  umq_buf_free(qbuf);
  return b;
}
umq_buf_t* umq_data_to_head(void* data) {
  if (!data) return nullptr;
  // the data area of a pooled block starts right after its descriptor + headroom; walk the pool's arenas
  std::lock_guard<std::mutex> l(g_pool.mu);
  const char* p = static_cast<const char*>(data);
  auto it = g_pool.by_mem.upper_bound(p);
  if (it == g_pool.by_mem.begin()) return nullptr;
  --it;
  Block* b = it->second;
  return (p >= b->mem && p < b->mem + b->cap) ? &b->meta : nullptr;
}
void umq_notify(uint64_t h) {
  // sends are handed to the device at enqueue time, so there is nothing deferred to flush: make progress instead,
  // which returns credits and completes finished sends
  Queue* q = find(h);
  if (!q) return;
  std::lock_guard<std::mutex> l(q->mu);
  progress(q);
}

// ---------------------------------------------------------------------------------------------- memory by reference
// A sender registers memory and ships its description inside a message; the receiver pulls the bytes with a
// one-sided read over the queue's own endpoint. This is what carries large RPC arguments by reference (the DMA table
// of the reference's request header and urpc_ref_read, src/urpc/framework/lib/datapath/dp.c:1333-1452).
struct MemSeg {
  urma_target_seg_t* seg;
  uint8_t blob[URMA_SIMPLE_SEG_BLOB];
};
static std::mutex g_seg_mu;
static std::map<uint64_t, MemSeg> g_segs;
static uint64_t g_seg_next = 1;
uint64_t umq_mem_seg_register(void* va, uint64_t len, uint32_t token, uint8_t* blob, uint32_t blob_cap) {
  if (!g.inited || !va || !len || !blob || blob_cap < URMA_SIMPLE_SEG_BLOB) return 0;
  MemSeg m;
  m.seg = urma_simple_seg_register(g.ctx, va, len, URMA_ACCESS_READ, token, m.blob);
  if (!m.seg) return 0;
  memcpy(blob, m.blob, URMA_SIMPLE_SEG_BLOB);
  std::lock_guard<std::mutex> l(g_seg_mu);
  const uint64_t h = g_seg_next++;
  g_segs[h] = m;
  return h;
}
int umq_mem_seg_unregister(uint64_t seg_h) {
  std::lock_guard<std::mutex> l(g_seg_mu);
  auto it = g_segs.find(seg_h);
  if (it == g_segs.end()) return UMQ_ERR_EINVAL;
  urma_unregister_seg(it->second.seg);
  g_segs.erase(it);
  return UMQ_SUCCESS;
}
int umq_remote_read(uint64_t h, const uint8_t* seg_blob, uint32_t token, uint64_t remote_addr, void* local,
                    uint32_t len, int timeout_ms) {
  Queue* q = find(h);
  if (!q || !q->ep || !seg_blob || !local || !len) return UMQ_ERR_EINVAL;   // queues with an endpoint of their own
  uint64_t id;
  {
    std::lock_guard<std::mutex> l(q->mu);
    if (!q->peer) return UMQ_ERR_ESTATE;
    const std::string key(reinterpret_cast<const char*>(seg_blob), URMA_SIMPLE_SEG_BLOB);
    urma_target_seg_t*& rseg = q->imported[key];
    if (!rseg) rseg = urma_simple_seg_import(g.ctx, seg_blob, token);
    if (!rseg) {
      q->imported.erase(key);
      return UMQ_ERR_EINVAL;
    }
    id = read_id(q);
    if (urma_simple_post(q->ep, q->peer, URMA_OPC_READ, rseg, remote_addr, nullptr, reinterpret_cast<uint64_t>(local),
                         len, 0, id, 1) != 0)
      return UMQ_FAIL;
  }
  const uint64_t deadline = ub::now_ns() + uint64_t(timeout_ms > 0 ? timeout_ms : 5000) * 1000000ull;
  for (;;) {
    {
      std::lock_guard<std::mutex> l(q->mu);
      progress(q);
      auto it = q->read_done.find(id);
      if (it != q->read_done.end()) {
        const int st = it->second;
        q->read_done.erase(it);
        return st == 0 ? UMQ_SUCCESS : UMQ_FAIL;   // a refused read (bad token, out of range) completes in error
      }
    }
    if (ub::now_ns() > deadline) return UMQ_ERR_EAGAIN;
    sched_yield();
  }
}

// ---------------------------------------------------------------------------------------------- queries
int umq_cfg_get(uint64_t h, umq_cfg_get_t* cfg) {
  Queue* q = find(h);
  if (!q || !cfg) return UMQ_ERR_EINVAL;
  cfg->create_option = q->opt;
  cfg->state = static_cast<umq_state_t>(q->state.load());
  cfg->feature = g.cfg.feature;
  cfg->trans_mode = g.cfg.trans_mode;
  cfg->block_size = g_pool.block;
  return UMQ_SUCCESS;
}
int umq_info_get(uint64_t h, umq_info_t* info) {
  Queue* q = find(h);
  if (!q || !info) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  memset(info, 0, sizeof(*info));
  info->umqh = h;
  snprintf(info->name, sizeof(info->name), "%s", q->opt.name);
  info->state = static_cast<umq_state_t>(q->state.load());
  info->bound = q->peer != nullptr;
  info->rx_posted = q->rx_posted;
  info->rx_ready = static_cast<uint32_t>(q->rx_ready.size());
  info->tx_in_flight = static_cast<uint32_t>(q->in_flight.size()) - (q->rx_posted < q->in_flight.size() ? q->rx_posted : 0);
  info->credits = q->credits;
  info->io = q->io;
  return UMQ_SUCCESS;
}
int umq_log_config_get(int* level) {
  if (!level) return UMQ_ERR_EINVAL;
  *level = g_log.level();
  return UMQ_SUCCESS;
}
int umq_dev_info_get(const char* dev_name, umq_trans_mode_t mode, umq_dev_info_t* out) {
  if (!dev_name || !out) return UMQ_ERR_EINVAL;
  urma_device_t* d = urma_get_device_by_name(dev_name);
  if (!d) return UMQ_ERR_EINVAL;
  memset(out, 0, sizeof(*out));
  snprintf(out->dev_name, sizeof(out->dev_name), "%s", d->name);
  memcpy(out->eid, d->eid.raw, sizeof(out->eid));
  out->trans_mode = mode;
  urma_device_attr_t a;
  if (urma_query_device(d, &a) == URMA_SUCCESS) {
    out->max_msg_size = a.max_msg_size;
    out->port_cnt = a.port_cnt;
  }
  return UMQ_SUCCESS;
}
umq_dev_info_t* umq_dev_info_list_get(umq_trans_mode_t mode, int* dev_num) {
  if (!dev_num) return nullptr;
  int n = 0;
  urma_device_t** list = urma_get_device_list(&n);
  if (!list || n <= 0) {
    *dev_num = 0;
    return nullptr;
  }
  umq_dev_info_t* out = static_cast<umq_dev_info_t*>(calloc(n, sizeof(umq_dev_info_t)));
  int k = 0;
  for (int i = 0; i < n && out; ++i)
    if (umq_dev_info_get(list[i]->name, mode, &out[k]) == UMQ_SUCCESS) ++k;
  urma_free_device_list(list);
  *dev_num = k;
  return out;
}
void umq_dev_info_list_free(umq_trans_mode_t, umq_dev_info_t* list) { free(list); }
int umq_dev_add(const char* dev_name) {
  // queues are created on the device named at umq_init; another device only has to exist to be usable by a later
  // umq_init, so adding one is a presence check
  return dev_name && urma_get_device_by_name(dev_name) ? UMQ_SUCCESS : UMQ_ERR_EINVAL;
}
int umq_get_route_list(const umq_route_key_t* key, umq_trans_mode_t, umq_route_list_t* out) {
  if (!key || !out) return UMQ_ERR_EINVAL;
  memset(out, 0, sizeof(*out));
  urma_eid_t src, dst;
  memcpy(src.raw, key->src_eid, sizeof(src.raw));
  memcpy(dst.raw, key->dst_eid, sizeof(dst.raw));
  uvs_path_set_t ps;
  if (uvs_get_path_set(&src, &dst, UVS_RTP, &ps) != 0) {
    if (uvs_discover_local_topology() <= 0 || uvs_get_path_set(&src, &dst, UVS_RTP, &ps) != 0) return UMQ_FAIL;
  }
  out->route_num = ps.path_count < UMQ_MAX_ROUTES ? ps.path_count : UMQ_MAX_ROUTES;
  for (uint32_t i = 0; i < out->route_num; ++i) {
    memcpy(out->routes[i].src_port_eid, ps.paths[i].src_eid.raw, 16);
    memcpy(out->routes[i].dst_port_eid, ps.paths[i].dst_eid.raw, 16);
  }
  return UMQ_SUCCESS;
}
int umq_mempool_state_get(uint64_t, uint32_t mempool_id, umq_mempool_state_t* out) {
  if (!out || mempool_id > 1) return UMQ_ERR_EINVAL;   // pool 0: blocks, pool 1: tiny buffers
  if (mempool_id == 1) {
    std::lock_guard<std::mutex> l(g_tiny.mu);
    out->block_size = kTinyBytes;
    out->blocks_total = g_tiny.total;
    out->blocks_free = g_tiny.free_list.size();
    out->registered = g_tiny_on ? 1 : 0;
    out->generation = g_tiny.slabs.size();
    return UMQ_SUCCESS;
  }
  std::lock_guard<std::mutex> l(g_pool.mu);
  out->block_size = g_pool.block;
  out->blocks_total = g_pool.total;
  out->blocks_free = g_pool.free_list.size();
  out->registered = g_pool.total != 0;
  out->generation = g_pool.generation;
  return UMQ_SUCCESS;
}
int umq_mempool_state_refresh(uint64_t, uint32_t mempool_id) {
  if (mempool_id != 0) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_pool.mu);
  ++g_pool.generation;   // users compare generations to learn that the pool was looked at again
  return UMQ_SUCCESS;
}
int umq_user_ctl(uint64_t h, umq_user_ctl_in_t* in, umq_user_ctl_out_t* out) {
  Queue* q = find(h);
  if (!q || !in) return UMQ_ERR_EINVAL;
  switch (in->opcode) {
    case UMQ_USER_CTL_PROGRESS: {   // run the completion path now; out->value = messages ready to dequeue
      std::lock_guard<std::mutex> l(q->mu);
      progress(q);
      if (out) out->value = q->rx_ready.size();
      return UMQ_SUCCESS;
    }
    case UMQ_USER_CTL_RETURN_CREDITS: {   // push owed credits back to the peer without waiting for the batch size
      std::lock_guard<std::mutex> l(q->mu);
      if (out) out->value = q->to_return;
      send_credit_return(q);
      return UMQ_SUCCESS;
    }
    default: return UMQ_ERR_EINVAL;
  }
}
int umq_interrupt_fd_list_get(uint64_t h, umq_io_direction_t, int* fds, uint32_t max) {
  const int fd = umq_interrupt_fd_get(h);
  if (fd < 0 || !fds || max == 0) return UMQ_FAIL;
  fds[0] = fd;   // one completion channel serves both directions
  return 1;
}
int umq_get_cq_event(uint64_t h, umq_io_direction_t) { return umq_wait_interrupt(h, 0); }
int umq_async_event_fd_get(void) {
  std::lock_guard<std::mutex> l(g_ev_mu);
  if (g_ev_fd < 0) g_ev_fd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  return g_ev_fd;
}
int umq_get_async_event(umq_async_event_t* ev) { return umq_async_event_get(ev); }
void umq_ack_async_event(umq_async_event_t*) {}   // events are copied out and hold nothing

// ---------------------------------------------------------------------------------------------- statistics helpers
int umq_stats_io_reset(uint64_t h) {
  Queue* q = find(h);
  if (!q) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  q->io = umq_io_stats_t{};
  return UMQ_SUCCESS;
}
int umq_stats_perf_reset(void) {
  std::lock_guard<std::mutex> l(g.perf_mu);
  perf_restart();
  return UMQ_SUCCESS;
}
int umq_io_stats_to_str(const umq_io_stats_t* s, char* buf, uint32_t len) {
  if (!s || !buf || !len) return UMQ_ERR_EINVAL;
  return snprintf(buf, len, "tx %llu msgs %llu B, rx %llu msgs %llu B, tx_errors %llu, rx_errors %llu, tx_eagain %llu",
                  (unsigned long long)s->tx_msgs, (unsigned long long)s->tx_bytes, (unsigned long long)s->rx_msgs,
                  (unsigned long long)s->rx_bytes, (unsigned long long)s->tx_errors, (unsigned long long)s->rx_errors,
                  (unsigned long long)s->tx_eagain);
}
int umq_flow_control_stats_to_str(const umq_fc_stats_t* s, char* buf, uint32_t len) {
  if (!s || !buf || !len) return UMQ_ERR_EINVAL;
  return snprintf(buf, len, "window %llu, credits local %llu remote %llu, granted %llu, returned %llu, stalls %llu",
                  (unsigned long long)s->window, (unsigned long long)s->credits_local,
                  (unsigned long long)s->credits_remote, (unsigned long long)s->credits_granted,
                  (unsigned long long)s->credits_returned, (unsigned long long)s->stalls);
}
int umq_qbuf_pool_stats_to_str(const umq_qbuf_stats_t* s, char* buf, uint32_t len) {
  if (!s || !buf || !len) return UMQ_ERR_EINVAL;
  return snprintf(buf, len, "block %llu B, blocks %llu total %llu free, huge %llu, alloc %llu, free %llu, failures %llu",
                  (unsigned long long)s->block_size, (unsigned long long)s->blocks_total,
                  (unsigned long long)s->blocks_free, (unsigned long long)s->huge_allocs,
                  (unsigned long long)s->alloc_calls, (unsigned long long)s->free_calls,
                  (unsigned long long)s->alloc_failures);
}
int umq_stats_perf_to_str(char* buf, uint32_t len) {
  if (!buf || !len) return UMQ_ERR_EINVAL;
  umq_perf_entry_t e[UMQ_PERF_RECORD_MAX];
  umq_stats_perf_get(e);
  int off = 0;
  for (int i = 0; i < UMQ_PERF_RECORD_MAX && off < (int)len; ++i)
    off += snprintf(buf + off, len - off, "%-10s count %llu avg %llu ns min %llu max %llu p99 %llu\n", kRecordNames[i],
                    (unsigned long long)e[i].count, (unsigned long long)e[i].avg_ns, (unsigned long long)e[i].min_ns,
                    (unsigned long long)e[i].max_ns, (unsigned long long)e[i].p99_ns);
  return off;
}
int umq_stats_trace_start(const char* path) { return umq_trace_start(path, 0, 0); }
int umq_stats_trace_stop(void) { return umq_trace_stop(); }
// transport-level (URMA data-plane) latency sampling, passed through to the URMA perf sampler
int umq_stats_tp_perf_start(void) { return urma_start_perf() == URMA_SUCCESS ? UMQ_SUCCESS : UMQ_FAIL; }
int umq_stats_tp_perf_stop(void) { return urma_stop_perf() == URMA_SUCCESS ? UMQ_SUCCESS : UMQ_FAIL; }
int umq_stats_tp_perf_info_get(char* buf, uint32_t* len) {
  if (!buf || !len) return UMQ_ERR_EINVAL;
  return urma_get_perf_info(nullptr, buf, len) == URMA_SUCCESS ? UMQ_SUCCESS : UMQ_FAIL;
}

// ---------------------------------------------------------------------------------------------- plug-in locks
// Applications with their own threading runtime (coroutines, user-level threads) may supply the lock and
// thread-key primitives; the library's own structures keep using std::mutex, and the registered primitives guard the
// application-visible critical sections reached through umq_external_lock / unlock.
static umq_external_mutex_ops_t g_ext_mutex{};
static umq_external_rwlock_ops_t g_ext_rwlock{};
static umq_external_thread_key_ops_t g_ext_key{};
int umq_external_mutex_lock_ops_register(const umq_external_mutex_ops_t* ops) {
  if (ops && (!ops->create || !ops->lock || !ops->unlock || !ops->destroy)) return UMQ_ERR_EINVAL;
  g_ext_mutex = ops ? *ops : umq_external_mutex_ops_t{};
  return UMQ_SUCCESS;
}
int umq_external_rwlock_ops_register(const umq_external_rwlock_ops_t* ops) {
  if (ops && (!ops->create || !ops->rdlock || !ops->wrlock || !ops->unlock || !ops->destroy)) return UMQ_ERR_EINVAL;
  g_ext_rwlock = ops ? *ops : umq_external_rwlock_ops_t{};
  return UMQ_SUCCESS;
}
int umq_external_thread_key_ops_register(const umq_external_thread_key_ops_t* ops) {
  if (ops && (!ops->create || !ops->set || !ops->get || !ops->destroy)) return UMQ_ERR_EINVAL;
  g_ext_key = ops ? *ops : umq_external_thread_key_ops_t{};
  return UMQ_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- transport pool
// A transport pool groups the completion channels of several queues behind one eventfd, so that one thread can
// sleep on many queues (the reference's time-division jetty pool serves the same purpose for many connections).
struct TpPool {
  int efd = -1;
  std::vector<uint64_t> queues;
  uint64_t wakeups = 0;
};
static std::mutex g_tpp_mu;
static std::map<uint64_t, TpPool> g_tp_pools;
static uint64_t g_tpp_next = 1;
uint64_t umq_transport_pool_resource_create(void) {
  std::lock_guard<std::mutex> l(g_tpp_mu);
  TpPool p;
  p.efd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  if (p.efd < 0) return 0;
  const uint64_t id = g_tpp_next++;
  g_tp_pools[id] = p;
  return id;
}
int umq_transport_pool_resource_modify(uint64_t pool, uint64_t umqh, int add) {
  if (!find(umqh)) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_tpp_mu);
  auto it = g_tp_pools.find(pool);
  if (it == g_tp_pools.end()) return UMQ_ERR_EINVAL;
  auto& v = it->second.queues;
  auto pos = std::find(v.begin(), v.end(), umqh);
  if (add) {
    if (pos != v.end()) return UMQ_ERR_EINVAL;
    v.push_back(umqh);
  } else {
    if (pos == v.end()) return UMQ_ERR_EINVAL;
    v.erase(pos);
  }
  return UMQ_SUCCESS;
}
int umq_transport_pool_resource_destroy(uint64_t pool) {
  std::lock_guard<std::mutex> l(g_tpp_mu);
  auto it = g_tp_pools.find(pool);
  if (it == g_tp_pools.end()) return UMQ_ERR_EINVAL;
  close(it->second.efd);
  g_tp_pools.erase(it);
  return UMQ_SUCCESS;
}
int umq_transport_pool_eventfd_get(uint64_t pool) {
  std::lock_guard<std::mutex> l(g_tpp_mu);
  auto it = g_tp_pools.find(pool);
  return it == g_tp_pools.end() ? -1 : it->second.efd;
}
// Polls the member queues once; returns how many have messages ready and signals the pool's eventfd if any has.
int umq_jetty_pool_stats_get(umq_jetty_pool_stats_t* out) {
  if (!out) return UMQ_ERR_EINVAL;
  memset(out, 0, sizeof(*out));
  {
    std::shared_lock<std::shared_mutex> pl(g_jpool.mu);
    out->total_num = g_jpool.members.size();
    for (Queue* m : g_jpool.members) out->err_num += m->state.load() == UMQ_STATE_ERR;
  }
  out->acc_alloc_num = out->acc_free_num = g_jpool.allocs.load();
  out->acc_miss_num = g_jpool.misses.load();
  std::lock_guard<std::mutex> l(g.mu);
  for (auto& kv : g.queues) out->sub_queues += !kv.second->tops && !kv.second->ep;
  return UMQ_SUCCESS;
}
int umq_jetty_pool_eventfd_get(void) {
  std::unique_lock<std::shared_mutex> pl(g_jpool.mu);
  if (g_jpool.efd < 0) g_jpool.efd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  return g_jpool.efd;
}
int umq_stats_transport_pool_get(uint64_t pool, umq_transport_pool_stats_t* out) {
  std::vector<uint64_t> qs;
  int efd;
  {
    std::lock_guard<std::mutex> l(g_tpp_mu);
    auto it = g_tp_pools.find(pool);
    if (it == g_tp_pools.end() || !out) return UMQ_ERR_EINVAL;
    qs = it->second.queues;
    efd = it->second.efd;
  }
  uint32_t ready = 0;
  for (uint64_t h : qs) {
    Queue* q = find(h);
    if (!q) continue;
    std::lock_guard<std::mutex> l(q->mu);
    progress(q);
    if (!q->rx_ready.empty()) ++ready;
  }
  std::lock_guard<std::mutex> l(g_tpp_mu);
  auto it = g_tp_pools.find(pool);
  if (it == g_tp_pools.end()) return UMQ_ERR_EINVAL;
  if (ready) {
    const uint64_t one = 1;
    if (write(efd, &one, sizeof(one)) > 0) ++it->second.wakeups;
  }
  out->queues = static_cast<uint32_t>(qs.size());
  out->queues_ready = ready;
  out->wakeups = it->second.wakeups;
  return UMQ_SUCCESS;
}
int umq_transport_pool_stats_to_str(const umq_transport_pool_stats_t* s, char* buf, uint32_t len) {
  if (!s || !buf || !len) return UMQ_ERR_EINVAL;
  return snprintf(buf, len, "queues %u, ready %u, wakeups %llu", s->queues, s->queues_ready,
                  (unsigned long long)s->wakeups);
}

int umq_log_config_set(int level, umq_log_cb_t cb) {
  if (level < 0 || level > 4) return UMQ_ERR_EINVAL;
  g_log.configure(level, cb);
  return UMQ_SUCCESS;
}
int umq_io_perf_callback_register(umq_io_perf_cb_t cb, void* ctx) {
  g_perf_cb_ctx = ctx;
  g_perf_cb = cb;
  return UMQ_SUCCESS;
}
int umq_async_event_get(umq_async_event_t* ev) {
  if (!ev) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_ev_mu);
  if (g_events.empty()) return UMQ_ERR_EAGAIN;
  *ev = g_events.front();
  g_events.pop_front();
  return UMQ_SUCCESS;
}
int umq_trace_start(const char* path, uint32_t flush_interval_ms, uint32_t ring_entries) {
  if (!path || !*path) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g_trace.mu);
  if (g_trace.on.load()) return UMQ_ERR_EINVAL;
  g_trace.file = fopen(path, "w");
  if (!g_trace.file) return UMQ_FAIL;
  fprintf(g_trace.file, "# start_ns tid record duration_ns\n");
  g_trace.interval_ms = flush_interval_ms ? flush_interval_ms : 100;
  g_trace.ring_entries = ring_entries ? ring_entries : 4096;
  g_trace.rings.clear();
  g_trace.written = 0;
  g_trace.stop = false;
  g_trace.generation.fetch_add(1, std::memory_order_release);
  g_trace.on = true;
  g_trace.flusher = std::thread(trace_flush_loop);
  return UMQ_SUCCESS;
}
int umq_trace_stop(void) {
  std::thread t;
  {
    std::lock_guard<std::mutex> l(g_trace.mu);
    if (!g_trace.on.load()) return UMQ_ERR_EINVAL;
    g_trace.on = false;
    g_trace.stop = true;
    t = std::move(g_trace.flusher);
  }
  if (t.joinable()) t.join();
  std::lock_guard<std::mutex> l(g_trace.mu);
  trace_drain_locked();
  if (g_trace.file) fclose(g_trace.file);
  g_trace.file = nullptr;
  return UMQ_SUCCESS;
}
int umq_trace_stats(uint64_t* written, uint64_t* dropped) {
  std::lock_guard<std::mutex> l(g_trace.mu);
  uint64_t d = 0;
  for (auto& r : g_trace.rings) d += r->dropped.load();
  if (written) *written = g_trace.written.load();
  if (dropped) *dropped = d;
  return UMQ_SUCCESS;
}
int umq_info_to_str(uint64_t h, char* buf, uint32_t len) {
  Queue* q = find(h);
  if (!q || !buf || len == 0) return UMQ_ERR_EINVAL;
  std::lock_guard<std::mutex> l(q->mu);
  return snprintf(buf, len,
                  "umq %llu name=%s state=%d rx_depth=%u tx_depth=%u rx_buf=%u fc=%d credits=%lld owed=%u "
                  "tx=%llu/%lluB rx=%llu/%lluB",
                  (unsigned long long)q->h, q->opt.name, q->state.load(), q->opt.rx_depth, q->opt.tx_depth,
                  q->opt.rx_buf_size, (int)q->fc, (long long)q->credits, q->to_return,
                  (unsigned long long)q->io.tx_msgs, (unsigned long long)q->io.tx_bytes,
                  (unsigned long long)q->io.rx_msgs, (unsigned long long)q->io.rx_bytes);
}

}  // extern "C"
