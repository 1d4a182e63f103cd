// "shm" URMA provider: a software NIC per context, connected through POSIX shared memory. It gives the whole
// northbound API real semantics (one-sided write/read, atomics, two-sided send/recv with immediate data, completion
// and event queues, tokens and access checks, error completions on timeouts) between threads and between processes
// of one host, with no special hardware. It plays the role that the reference's hardware user driver plays
// (src/urma/hw/udma: udma_u_jfs.c post_sq_wr / udma_u_jfc.c poll) and doubles as the fake device that the
// reference's unit tests build with link-time mocks (test/urma/include/urma_hw_mock.h).
//
// Wire model: every context owns an "inbox" in a shared-memory file: four bounded multi-producer rings. Initiators
// write request messages (header + up to 4 KiB of payload per slot, gathered straight into the slot; larger transfers
// are fragmented) into the ring that the target jetty's number selects; whoever executes the target's inbox runs them
// against the target process's memory after checking segment token, bounds and access rights, and answers into the
// ring of the initiator that the asking send queue's number selects; executing those answers turns them into
// completion records. Requests in flight live in a lock-free table and carry a deadline, so a dead peer produces
// URMA_CR_ACK_TIMEOUT_ERR rather than a hang.
//
// Who executes an inbox: an application thread that polls an empty completion queue does it itself, inside the poll
// (a message is then copied once, by the thread that is about to read it), and the context's own thread does it
// whenever nobody has polled for a few microseconds (requests of peers must progress while the application sleeps
// on a completion event or computes). Rings are executed concurrently, one consumer each; the operations that free
// a queue wait until no message is being handled. A context that has been quiet for a while costs no processor time:
// its thread sleeps on a futex word in the inbox file and the next sender wakes it.
#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <linux/futex.h>
#include <sys/eventfd.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "ub_util.h"
#include "urma_api.h"
#include "urma_provider.h"

namespace {

constexpr uint32_t kSlotPayload = 4096;
constexpr uint32_t kRings = 4;          // rings per inbox (power of two)
constexpr uint32_t kRingSlots = 256;   // slots per ring (power of two)
constexpr uint32_t kMaxCtx = 256;
constexpr uint32_t kRegMagic = 0x55524d41;  // "URMA"

enum MsgType : uint32_t { MSG_WRITE = 1, MSG_READ, MSG_ATOMIC, MSG_SEND, MSG_RESP, MSG_RESP_DATA, MSG_PROBE };
enum MsgFlag : uint32_t { F_FIRST = 1, F_LAST = 2, F_IMM = 4, F_WANT_ACK = 8 };

struct MsgHdr {
  uint32_t type, opcode, flags, status;
  uint32_t src_uasid, src_jetty, dst_jetty, token_id;
  uint32_t token_val, len, total_len, frag_off;
  uint64_t remote_va, wr_id, operand, cmp;
  uint8_t src_eid[16];
};
struct Slot {
  std::atomic<uint64_t> seq;
  MsgHdr h;
  uint8_t payload[kSlotPayload];
};
// An inbox is several rings. A message goes to the ring that its queue's number selects (requests: the target
// jetty; answers: the send queue that asked), so everything whose order matters shares a ring, while the rings can be
// executed by different threads at the same time - what several receive queues do for a NIC.
struct Ring {
  std::atomic<uint64_t> enq;
  char pad0[56];
  std::atomic<uint64_t> deq;
  char pad1[56];
  Slot slots[kRingSlots];
};
struct Inbox {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> owner_pid;
  // 1 while the owner's thread sleeps because nothing has arrived for a while: whoever publishes a message then
  // wakes it (a futex on this word, which works between processes because the file is mapped shared). An idle
  // context costs no processor time this way, and its first message is not left waiting for a timer.
  std::atomic<uint32_t> sleeping;
  char pad[52];
  Ring ring[kRings];
};
static_assert(sizeof(std::atomic<uint32_t>) == sizeof(uint32_t), "the futex word is a plain 32-bit word");
// No fence between publishing the message and reading the word: a full barrier here would drain the store buffer
// after every payload copy (measured: a sixth of the pipelined send rate). The read may therefore be served while
// the publishing store is still on its way, at the very moment the owner decides to sleep - which is why the owner
// looks at its rings once more a few microseconds after it announced the sleep (see nic_loop): by then every store
// issued before this read is visible to it.
inline void wake_owner(Inbox* box) {
  __asm__ __volatile__("" ::: "memory");   // the compiler keeps the order; the processor may not (see above)
  if (box->sleeping.load(std::memory_order_relaxed) && box->sleeping.exchange(0, std::memory_order_acq_rel))
    syscall(SYS_futex, reinterpret_cast<uint32_t*>(&box->sleeping), FUTEX_WAKE, 1, nullptr, nullptr, 0);
}
inline Ring* ring_of(Inbox* in, uint32_t queue_id) { return &in->ring[queue_id & (kRings - 1)]; }
struct CtxSlot {
  std::atomic<uint32_t> uasid;  // 0 = free
  std::atomic<uint32_t> pid;
  std::atomic<uint64_t> heartbeat_ns;
};
struct DevReg {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> next_uasid;
  std::atomic<uint32_t> next_jetty;
  std::atomic<uint32_t> next_token;
  CtxSlot ctx[kMaxCtx];
};

std::string shm_dir() {
  const char* e = getenv("URMA_SHM_DIR");
  if (e && *e) return e;
  return "/dev/shm/umdk_urma_" + std::to_string(getuid());
}

void* map_file(const std::string& path, size_t bytes, bool create, bool* created = nullptr) {
  int fd = open(path.c_str(), O_RDWR | (create ? O_CREAT : 0), 0600);
  if (fd < 0) return nullptr;
  struct stat st;
  if (fstat(fd, &st) != 0) {
    close(fd);
    return nullptr;
  }
  if (static_cast<size_t>(st.st_size) < bytes) {
    if (!create || ftruncate(fd, bytes) != 0) {
      close(fd);
      return nullptr;
    }
    if (created) *created = true;
  }
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  return p == MAP_FAILED ? nullptr : p;
}

// Vyukov bounded queue, multi-producer side. Returns the reserved slot or nullptr when the ring is full.
Slot* ring_reserve(Ring* in, uint64_t* pos_out) {
  uint64_t pos = in->enq.load(std::memory_order_relaxed);
  for (;;) {
    Slot* s = &in->slots[pos & (kRingSlots - 1)];
    const uint64_t seq = s->seq.load(std::memory_order_acquire);
    const int64_t dif = static_cast<int64_t>(seq) - static_cast<int64_t>(pos);
    if (dif == 0) {
      if (in->enq.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
        *pos_out = pos;
        return s;
      }
    } else if (dif < 0) {
      return nullptr;
    } else {
      pos = in->enq.load(std::memory_order_relaxed);
    }
  }
}
void ring_publish(Slot* s, uint64_t pos) { s->seq.store(pos + 1, std::memory_order_release); }

struct Device {
  std::string name;
  urma_eid_t eid;
  DevReg* reg = nullptr;
};
// (never destroyed: a context that the application left open still has its thread running while the process exits)
std::vector<Device>& g_devs = *new std::vector<Device>();
std::mutex g_mu;

using ub::cpu_relax;
// The queues below are touched for a few dozen nanoseconds at a time by an application thread and a NIC thread that
// both poll: a mutex that puts the loser to sleep costs more than the whole critical section, so they spin (and
// give the core away when the holder seems to have been descheduled).
class SpinLock {
 public:
  void lock() {
    for (uint32_t n = 0;; ++n) {
      if (!f_.load(std::memory_order_relaxed) && !f_.exchange(true, std::memory_order_acquire)) return;
      if ((n & 255) == 255) sched_yield();
      else cpu_relax();
    }
  }
  void unlock() { f_.store(false, std::memory_order_release); }

 private:
  std::atomic<bool> f_{false};
};

struct SegReg {
  uint64_t va, len;
  uint32_t access, token_val;
};
struct SgeList {  // a scatter / gather list held by value (no allocation on the data path)
  urma_sge_t sge[URMA_MAX_SGE];
  uint32_t n = 0;
  void assign(const urma_sge_t* src, uint32_t cnt) {
    n = cnt > URMA_MAX_SGE ? URMA_MAX_SGE : cnt;
    for (uint32_t i = 0; i < n; ++i) sge[i] = src[i];
  }
  uint32_t bytes() const {
    uint32_t t = 0;
    for (uint32_t i = 0; i < n; ++i) t += sge[i].len;
    return t;
  }
};
struct RecvWr {
  SgeList sges;
  uint64_t user_ctx;
};
struct Unexpected {
  std::vector<uint8_t> data;
  uint64_t imm;
  bool has_imm;
  uint32_t src_uasid, src_jetty;
  uint64_t wr_id;
  urma_eid_t src_eid;
  bool want_ack;
};
struct ShmJfce {
  urma_jfce_t pub;
  int efd;
  std::mutex mu;
  std::deque<urma_jfc_t*> fired;
};
struct ShmJfc {
  urma_jfc_t pub;
  SpinLock mu;
  std::vector<urma_cr_t> ring;      // cfg.depth records
  uint32_t head = 0, tail = 0;      // under mu: next to pop / next to push (free-running)
  std::atomic<uint32_t> count{0};   // lets a poller see "empty" without taking the lock
  bool armed = false;
  uint32_t overflow = 0;
  std::atomic<uint32_t> empty_polls{0};   // consecutive polls that found nothing (a hint; races between pollers are harmless)
};
constexpr uint32_t kInlineAfterEmptyPolls = 3;
struct ShmCtx;
struct RecvQueue {  // a JFR, or the receive half of a jetty
  uint32_t id;
  ShmJfc* jfc;
  uint32_t depth;
  uint32_t token_val;
  SpinLock mu;
  // posted receive requests: a ring of `depth` entries made once (a request is 200 bytes of scatter list; a deque
  // would allocate for nearly every one)
  std::vector<RecvWr> ring;
  uint32_t head = 0, tail = 0;   // free-running, under mu
  bool posted_empty() const { return head == tail; }
  uint32_t posted_size() const { return tail - head; }
  RecvWr& posted_front() { return ring[head % ring.size()]; }
  void posted_pop() { ++head; }
  void posted_push(const RecvWr& w) { ring[tail++ % ring.size()] = w; }
  std::deque<Unexpected> unexpected;
  std::atomic<int> state{URMA_JETTY_STATE_READY};
};
struct SendQueue {
  uint32_t id;
  ShmJfc* jfc;
  uint32_t depth;
  std::atomic<int> state{URMA_JETTY_STATE_READY};
  std::atomic<uint32_t> inflight{0};
  uint32_t err_timeout_ms = 2000;
};
struct ShmJfs {
  urma_jfs_t pub;
  SendQueue sq;
};
struct ShmJfr {
  urma_jfr_t pub;
  RecvQueue rq;
};
struct ShmJetty {
  urma_jetty_t pub;
  SendQueue sq;
  RecvQueue own_rq;
  RecvQueue* rq;  // own_rq or a shared JFR's queue
};
struct Pending {
  SendQueue* sq;
  uint64_t user_ctx;
  uint32_t flag;
  urma_opcode_t opcode;
  SgeList local;  // destination of READ data / atomic old value
  uint32_t total = 0, received = 0;
  uint64_t deadline_ns;
  urma_jetty_id_t remote;
};
struct Reasm {
  std::vector<uint8_t> data;   // staging, used only when no receive request was posted when the message began
  uint32_t got = 0;
  bool direct = false;         // fragments go straight into `wr`'s buffers
  RecvWr wr;
};
constexpr uint32_t kPendSlots = 4096;  // power of two
constexpr uint64_t kPendBusy = ~0ull;
struct PendSlot {
  std::atomic<uint64_t> id{0};
  Pending p;
};
constexpr uint32_t kPeerHints = 64;  // power of two
struct PeerHint {
  std::atomic<uint32_t> uasid{0};
  std::atomic<Inbox*> in{nullptr};
};
struct ShmCtx {
  urma_context_t pub;
  Device* dev;
  Inbox* inbox = nullptr;
  std::string inbox_path;
  int reg_slot = -1;
  std::thread nic;
  std::atomic<bool> stop{false};
  std::mutex mu;  // guards the tables below
  // Held shared by whoever handles messages (they may touch queues they looked up under `mu` after dropping `mu`)
  // and exclusively by the delete operations while they free a queue: an object is never freed under a handler's
  // feet. `deleters` makes the handlers step aside for a waiting delete (a reader-preferring lock would starve it).
  std::shared_mutex life_mu;
  std::atomic<int> deleters{0};
  std::atomic<bool> ring_busy[kRings] = {};   // ring r is being executed
  std::unordered_map<uint32_t, SegReg> segs;
  std::unordered_map<uint32_t, RecvQueue*> rqs;
  // Requests that wait for their answer. A request id names its slot (id modulo the table size); the slot's `id`
  // word is the whole protocol: 0 = free, kPendBusy = a thread is filling or emptying it, anything else = the
  // request that lives there. The posting thread claims and fills, whoever ends the request (the NIC thread on the
  // answer, the deadline scan, a flush, a failed post) claims it back with one compare-and-swap, so no two threads
  // ever complete one request and none of them takes a lock. An id whose slot is still held by a request 4096 ids
  // older goes to `pending_more` under `pend_mu` instead.
  PendSlot pend[kPendSlots];
  std::mutex pend_mu;
  std::unordered_map<uint64_t, Pending> pending_more;
  std::atomic<uint32_t> pending_more_n{0};
  std::atomic<uint64_t> next_wr{1};
  std::unordered_map<uint32_t, Inbox*> peers;
  PeerHint peer_hint[kPeerHints];   // lock-free front of `peers` (mappings live until the context goes)
  std::map<std::pair<uint32_t, uint64_t>, Reasm> reasm;
  std::deque<urma_async_event_t> events;
  int event_fd = -1;
  std::atomic<uint64_t> app_poll_ticks{0};   // fast_ticks() of the last poll of an empty completion queue
  bool inline_poll = true;              // URMA_SHM_INLINE_POLL=0: only the context's own thread executes the inbox
  std::atomic<bool> drop_tx{false};  // fault injection: outgoing requests vanish (a dead link)
  // Answers that did not fit into a full peer inbox. The NIC thread never blocks on a full ring (two NIC threads
  // answering into each other's full inbox would deadlock); it parks the answer here and retries later.
  struct Deferred {
    uint32_t uasid;
    uint32_t queue;   // selects the ring of the peer's inbox
    MsgHdr h;
    std::vector<uint8_t> payload;
  };
  SpinLock deferred_mu;
  std::deque<Deferred> deferred;            // under deferred_mu
  std::atomic<uint32_t> deferred_n{0};      // its size, readable without the lock
};

// ---------------------------------------------------------------------------------------------- helpers
void push_cr(ShmJfc* jfc, const urma_cr_t& cr) {
  if (!jfc) return;
  ShmJfce* ce = nullptr;
  {
    std::lock_guard<SpinLock> l(jfc->mu);
    const uint32_t cap = static_cast<uint32_t>(jfc->ring.size());
    if (jfc->tail - jfc->head >= cap) {
      ++jfc->overflow;
      return;
    }
    jfc->ring[jfc->tail++ % cap] = cr;
    jfc->count.store(jfc->tail - jfc->head, std::memory_order_release);
    if (jfc->armed && jfc->pub.cfg.jfce) {
      jfc->armed = false;
      ce = reinterpret_cast<ShmJfce*>(jfc->pub.cfg.jfce->priv);
    }
  }
  if (ce) {
    {
      std::lock_guard<std::mutex> l(ce->mu);
      ce->fired.push_back(&jfc->pub);
    }
    uint64_t one = 1;
    if (write(ce->efd, &one, sizeof(one)) < 0) {
    }
  }
}

Inbox* peer_inbox(ShmCtx* c, uint32_t uasid) {
  if (uasid == c->pub.uasid) return c->inbox;
  PeerHint& hint = c->peer_hint[uasid & (kPeerHints - 1)];
  if (hint.uasid.load(std::memory_order_acquire) == uasid) {
    // `in` and `uasid` are two words: a writer that replaces the pair may be between its two stores, so the pair
    // counts only if the tag still reads the same after the pointer was taken
    Inbox* in = hint.in.load(std::memory_order_acquire);
    if (in && hint.uasid.load(std::memory_order_acquire) == uasid) return in;
  }
  std::lock_guard<std::mutex> l(c->mu);
  Inbox* in = nullptr;
  auto it = c->peers.find(uasid);
  if (it != c->peers.end()) {
    in = it->second;
  } else {
    const std::string path = shm_dir() + "/inbox_" + c->dev->name + "_" + std::to_string(uasid);
    in = static_cast<Inbox*>(map_file(path, sizeof(Inbox), false));
    if (in && in->magic.load() != kRegMagic) {
      munmap(in, sizeof(Inbox));
      in = nullptr;
    }
    if (in) c->peers[uasid] = in;
  }
  if (in) {   // writers are serialised by c->mu; the tag is taken down while the pair changes
    hint.uasid.store(0, std::memory_order_release);
    hint.in.store(in, std::memory_order_release);
    hint.uasid.store(uasid, std::memory_order_release);
  }
  return in;
}

// Blocks (bounded) until a slot is free in the target inbox. Returns false if the ring stayed full.
Slot* reserve_wait(Ring* in, uint64_t* pos, uint32_t timeout_ms) {
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    if (Slot* s = ring_reserve(in, pos)) return s;
    if ((spins & 63) == 63) {
      const uint64_t now = ub::now_ns();
      if (!t0) t0 = now;
      if (now - t0 > uint64_t(timeout_ms) * 1000000ull) return nullptr;
      sched_yield();
    } else {
      cpu_relax();
    }
  }
}
bool send_msg(Inbox* box, Ring* in, const MsgHdr& h, const void* payload, uint32_t timeout_ms = 2000) {
  uint64_t pos;
  Slot* s = reserve_wait(in, &pos, timeout_ms);
  if (!s) return false;
  s->h = h;
  if (h.len && payload) memcpy(s->payload, payload, h.len);
  ring_publish(s, pos);
  wake_owner(box);
  return true;
}
// Copies up to kSlotPayload bytes of a gather list into `dst`, continuing at (*si, *so); returns the bytes copied.
uint32_t gather_frag(const urma_sg_t& src, uint32_t* si, uint32_t* so, uint8_t* dst) {
  uint32_t n = 0;
  while (n < kSlotPayload && *si < src.num_sge) {
    const uint32_t take = std::min(kSlotPayload - n, src.sge[*si].len - *so);
    if (take) memcpy(dst + n, reinterpret_cast<void*>(src.sge[*si].addr + *so), take);
    n += take;
    *so += take;
    if (*so == src.sge[*si].len) {
      ++*si;
      *so = 0;
    }
  }
  return n;
}

// scatter `len` bytes at `src` into an SGE list starting at byte offset `off`
void scatter(const SgeList& sges, uint32_t off, const uint8_t* src, uint32_t len) {
  for (uint32_t i = 0; i < sges.n; ++i) {
    const urma_sge_t& g = sges.sge[i];
    if (len == 0) break;
    if (off >= g.len) {
      off -= g.len;
      continue;
    }
    const uint32_t n = std::min(len, g.len - off);
    memcpy(reinterpret_cast<void*>(g.addr + off), src, n);
    src += n;
    len -= n;
    off = 0;
  }
}
uint32_t sg_len(const urma_sg_t& sg) {
  uint32_t n = 0;
  for (uint32_t i = 0; i < sg.num_sge; ++i) n += sg.sge[i].len;
  return n;
}

urma_cr_status_t check_seg(ShmCtx* c, const MsgHdr& h, uint32_t need, uint64_t len) {
  std::lock_guard<std::mutex> l(c->mu);
  auto it = c->segs.find(h.token_id);
  if (it == c->segs.end()) return URMA_CR_REM_ACCESS_ABORT_ERR;
  const SegReg& s = it->second;
  if (s.token_val != h.token_val) return URMA_CR_REM_ACCESS_ABORT_ERR;
  if ((s.access & need) != need) return URMA_CR_REM_ACCESS_ABORT_ERR;
  if (h.remote_va < s.va || h.remote_va + len > s.va + s.len) return URMA_CR_REM_OPERATION_ERR;
  return URMA_CR_SUCCESS;
}

void reply(ShmCtx* c, const MsgHdr& req, uint32_t type, urma_cr_status_t st, uint64_t operand = 0,
           const void* payload = nullptr, uint32_t len = 0, uint32_t off = 0, uint32_t flags = F_LAST) {
  Inbox* in = peer_inbox(c, req.src_uasid);
  if (!in) return;
  MsgHdr r{};
  r.type = type;
  r.opcode = req.opcode;
  r.flags = flags;
  r.status = st;
  r.src_uasid = c->pub.uasid;
  r.wr_id = req.wr_id;
  r.operand = operand;
  r.len = len;
  r.frag_off = off;
  // answers go to the ring of the send queue that asked: its completions keep their order
  if (c->deferred_n.load(std::memory_order_acquire) == 0) {
    uint64_t pos;
    if (Slot* s = ring_reserve(ring_of(in, req.src_jetty), &pos)) {
      s->h = r;
      if (len && payload) memcpy(s->payload, payload, len);
      ring_publish(s, pos);
      wake_owner(in);
      return;
    }
  }
  ShmCtx::Deferred d;
  d.uasid = req.src_uasid;
  d.queue = req.src_jetty;
  d.h = r;
  if (len && payload) d.payload.assign(static_cast<const uint8_t*>(payload), static_cast<const uint8_t*>(payload) + len);
  std::lock_guard<SpinLock> l(c->deferred_mu);
  c->deferred.push_back(std::move(d));
  c->deferred_n.store(static_cast<uint32_t>(c->deferred.size()), std::memory_order_release);
}

// Retries parked answers in order; stops at the first one that still does not fit.
void flush_deferred(ShmCtx* c) {
  std::lock_guard<SpinLock> l(c->deferred_mu);
  while (!c->deferred.empty()) {
    ShmCtx::Deferred& d = c->deferred.front();
    Inbox* in = peer_inbox(c, d.uasid);
    if (in) {
      uint64_t pos;
      Slot* s = ring_reserve(ring_of(in, d.queue), &pos);
      if (!s) break;
      s->h = d.h;
      if (!d.payload.empty()) memcpy(s->payload, d.payload.data(), d.payload.size());
      ring_publish(s, pos);
      wake_owner(in);
    }
    c->deferred.pop_front();
  }
  c->deferred_n.store(static_cast<uint32_t>(c->deferred.size()), std::memory_order_release);
}

// Completes one receive request with `len` bytes at `data` (null: the bytes are in the buffer already, a message
// reassembled in place); `m` carries who sent them (its own data is not used).
void finish_recv(ShmCtx* c, RecvQueue* rq, const RecvWr& wr, const uint8_t* data, uint32_t len, const Unexpected& m) {
  urma_cr_t cr{};
  cr.user_ctx = wr.user_ctx;
  cr.flag = URMA_CR_FLAG_RECV;
  cr.local_id = rq->id;
  cr.remote_id.eid = m.src_eid;
  cr.remote_id.uasid = m.src_uasid;
  cr.remote_id.id = m.src_jetty;
  cr.imm_data = m.imm;
  cr.opcode = m.has_imm ? URMA_CR_OPC_SEND_WITH_IMM : URMA_CR_OPC_SEND;
  urma_cr_status_t st = URMA_CR_SUCCESS;
  if (len > wr.sges.bytes()) {
    st = URMA_CR_LOC_LEN_ERR;
  } else {
    if (data) scatter(wr.sges, 0, data, len);
    cr.completion_len = len;
  }
  cr.status = st;
  push_cr(rq->jfc, cr);
  if (m.want_ack) {
    MsgHdr req{};
    req.src_uasid = m.src_uasid;
    req.src_jetty = m.src_jetty;
    req.wr_id = m.wr_id;
    req.opcode = URMA_OPC_SEND;
    reply(c, req, MSG_RESP, st == URMA_CR_SUCCESS ? URMA_CR_SUCCESS : URMA_CR_REM_RESP_LEN_ERR);
  }
}

// Delivers a complete incoming message into a posted receive buffer, or parks it until one is posted.
void deliver(ShmCtx* c, RecvQueue* rq, Unexpected&& u) {
  RecvWr wr;
  {
    std::lock_guard<SpinLock> l(rq->mu);
    if (rq->posted_empty()) {
      rq->unexpected.push_back(std::move(u));
      return;
    }
    wr = rq->posted_front();
    rq->posted_pop();
  }
  finish_recv(c, rq, wr, u.data.data(), static_cast<uint32_t>(u.data.size()), u);
}

// ---- the table of requests in flight
bool pend_put(ShmCtx* c, uint64_t id, const Pending& p) {
  PendSlot& e = c->pend[id & (kPendSlots - 1)];
  uint64_t free_word = 0;
  if (e.id.load(std::memory_order_relaxed) == 0 &&
      e.id.compare_exchange_strong(free_word, kPendBusy, std::memory_order_acquire)) {
    e.p = p;
    e.id.store(id, std::memory_order_release);
    return true;
  }
  std::lock_guard<std::mutex> l(c->pend_mu);
  c->pending_more[id] = p;
  c->pending_more_n.fetch_add(1, std::memory_order_release);
  return true;
}
// Takes the request out of the table; false when somebody else already ended it (or it never existed).
bool pend_take(ShmCtx* c, uint64_t id, Pending* out) {
  PendSlot& e = c->pend[id & (kPendSlots - 1)];
  for (;;) {
    uint64_t cur = e.id.load(std::memory_order_acquire);
    if (cur == id) {
      if (!e.id.compare_exchange_strong(cur, kPendBusy, std::memory_order_acquire)) continue;
      *out = e.p;
      e.id.store(0, std::memory_order_release);
      return true;
    }
    if (cur == kPendBusy) {   // being filled (not ours: ours was published before its message left) or being
      cpu_relax();            // read for a data fragment by the NIC thread, which puts it back at once
      continue;
    }
    break;
  }
  if (c->pending_more_n.load(std::memory_order_acquire) == 0) return false;
  std::lock_guard<std::mutex> l(c->pend_mu);
  auto it = c->pending_more.find(id);
  if (it == c->pending_more.end()) return false;
  *out = it->second;
  c->pending_more.erase(it);
  c->pending_more_n.fetch_sub(1, std::memory_order_release);
  return true;
}
// Runs `fn(Pending&)` on the request while it stays in the table (data fragments of a READ land this way).
template <typename F>
bool pend_with(ShmCtx* c, uint64_t id, F fn) {
  PendSlot& e = c->pend[id & (kPendSlots - 1)];
  for (;;) {
    uint64_t cur = e.id.load(std::memory_order_acquire);
    if (cur == id) {
      if (!e.id.compare_exchange_strong(cur, kPendBusy, std::memory_order_acquire)) continue;
      fn(e.p);
      e.id.store(id, std::memory_order_release);
      return true;
    }
    if (cur != kPendBusy) break;
    cpu_relax();
  }
  if (c->pending_more_n.load(std::memory_order_acquire) == 0) return false;
  std::lock_guard<std::mutex> l(c->pend_mu);
  auto it = c->pending_more.find(id);
  if (it == c->pending_more.end()) return false;
  fn(it->second);
  return true;
}
// Ids of the requests for which `pred(Pending&)` holds (a snapshot: each id still has to be taken).
template <typename F>
std::vector<uint64_t> pend_select(ShmCtx* c, F pred) {
  std::vector<uint64_t> ids;
  for (uint32_t i = 0; i < kPendSlots; ++i) {
    PendSlot& e = c->pend[i];
    uint64_t cur = e.id.load(std::memory_order_acquire);
    if (cur == 0 || cur == kPendBusy) continue;
    const uint64_t id = cur;
    if (!e.id.compare_exchange_strong(cur, kPendBusy, std::memory_order_acquire)) continue;
    const bool hit = pred(e.p);
    e.id.store(id, std::memory_order_release);
    if (hit) ids.push_back(id);
  }
  if (c->pending_more_n.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> l(c->pend_mu);
    for (auto& kv : c->pending_more)
      if (pred(kv.second)) ids.push_back(kv.first);
  }
  return ids;
}
uint32_t pend_count(ShmCtx* c) {
  uint32_t n = c->pending_more_n.load();
  for (uint32_t i = 0; i < kPendSlots; ++i) n += c->pend[i].id.load(std::memory_order_relaxed) != 0;
  return n;
}

void complete_pending(ShmCtx* c, uint64_t wr_id, urma_cr_status_t st, uint64_t operand, bool have_operand) {
  Pending p;
  if (!pend_take(c, wr_id, &p)) return;
  if (have_operand && p.local.n && st == URMA_CR_SUCCESS)
    scatter(p.local, 0, reinterpret_cast<const uint8_t*>(&operand), 8);
  p.sq->inflight.fetch_sub(1);
  if ((p.flag & URMA_WR_FLAG_COMPLETE_ENABLE) || st != URMA_CR_SUCCESS) {
    urma_cr_t cr{};
    cr.status = st;
    cr.user_ctx = p.user_ctx;
    cr.local_id = p.sq->id;
    cr.remote_id = p.remote;
    cr.completion_len = p.total;
    push_cr(p.sq->jfc, cr);
  }
  if (st != URMA_CR_SUCCESS) p.sq->state = URMA_JETTY_STATE_ERROR;
}

void handle(ShmCtx* c, Slot* s) {
  const MsgHdr& h = s->h;
  switch (h.type) {
    case MSG_WRITE: {
      urma_cr_status_t st = check_seg(c, h, URMA_ACCESS_WRITE, h.len);
      if (st == URMA_CR_SUCCESS && h.len) memcpy(reinterpret_cast<void*>(h.remote_va), s->payload, h.len);
      if (h.flags & F_LAST) {
        if (st == URMA_CR_SUCCESS && (h.flags & F_IMM)) {  // WRITE_IMM / WRITE_NOTIFY consume a receive WR
          RecvQueue* rq = nullptr;
          {
            std::lock_guard<std::mutex> l(c->mu);
            auto it = c->rqs.find(h.dst_jetty);
            if (it != c->rqs.end()) rq = it->second;
          }
          if (rq) {
            RecvWr wr;
            bool have = false;
            {
              std::lock_guard<SpinLock> l(rq->mu);
              if (!rq->posted_empty()) {
                wr = rq->posted_front();
                rq->posted_pop();
                have = true;
              }
            }
            if (have) {
              urma_cr_t cr{};
              cr.user_ctx = wr.user_ctx;
              cr.flag = URMA_CR_FLAG_RECV;
              cr.opcode = URMA_CR_OPC_WRITE_WITH_IMM;
              cr.imm_data = h.operand;
              cr.completion_len = h.total_len;
              cr.local_id = rq->id;
              cr.remote_id.uasid = h.src_uasid;
              cr.remote_id.id = h.src_jetty;
              memcpy(cr.remote_id.eid.raw, h.src_eid, 16);
              push_cr(rq->jfc, cr);
            } else {
              st = URMA_CR_RNR_RETRY_CNT_EXC_ERR;
            }
          } else {
            st = URMA_CR_REM_OPERATION_ERR;
          }
        }
        reply(c, h, MSG_RESP, st);
      } else if (st != URMA_CR_SUCCESS) {
        reply(c, h, MSG_RESP, st);
      }
      break;
    }
    case MSG_READ: {
      urma_cr_status_t st = check_seg(c, h, URMA_ACCESS_READ, h.total_len);
      if (st != URMA_CR_SUCCESS) {
        reply(c, h, MSG_RESP, st);
        break;
      }
      uint32_t off = 0;
      while (off < h.total_len) {
        const uint32_t n = std::min(kSlotPayload, h.total_len - off);
        reply(c, h, MSG_RESP_DATA, URMA_CR_SUCCESS, 0, reinterpret_cast<void*>(h.remote_va + off), n, off,
              off + n == h.total_len ? F_LAST : 0);
        off += n;
      }
      break;
    }
    case MSG_ATOMIC: {
      urma_cr_status_t st = check_seg(c, h, URMA_ACCESS_ATOMIC, 8);
      uint64_t old = 0;
      if (st == URMA_CR_SUCCESS && (h.remote_va & 7)) st = URMA_CR_REM_OPERATION_ERR;
      if (st == URMA_CR_SUCCESS) {
        uint64_t* p = reinterpret_cast<uint64_t*>(h.remote_va);
        switch (h.opcode) {
          case URMA_OPC_CAS: {
            uint64_t exp = h.cmp;
            __atomic_compare_exchange_n(p, &exp, h.operand, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
            old = exp;
            break;
          }
          case URMA_OPC_SWAP: old = __atomic_exchange_n(p, h.operand, __ATOMIC_SEQ_CST); break;
          case URMA_OPC_FADD: old = __atomic_fetch_add(p, h.operand, __ATOMIC_SEQ_CST); break;
          case URMA_OPC_FSUB: old = __atomic_fetch_sub(p, h.operand, __ATOMIC_SEQ_CST); break;
          case URMA_OPC_FAND: old = __atomic_fetch_and(p, h.operand, __ATOMIC_SEQ_CST); break;
          case URMA_OPC_FOR: old = __atomic_fetch_or(p, h.operand, __ATOMIC_SEQ_CST); break;
          case URMA_OPC_FXOR: old = __atomic_fetch_xor(p, h.operand, __ATOMIC_SEQ_CST); break;
          default: st = URMA_CR_REM_UNSUPPORTED_REQ_ERR;
        }
      }
      reply(c, h, MSG_RESP, st, old);
      break;
    }
    case MSG_SEND: {
      RecvQueue* rq = nullptr;
      {
        std::lock_guard<std::mutex> l(c->mu);
        auto it = c->rqs.find(h.dst_jetty);
        if (it != c->rqs.end()) rq = it->second;
      }
      if (!rq || rq->state.load() != URMA_JETTY_STATE_READY || rq->token_val != h.token_val) {
        if (h.flags & F_LAST) reply(c, h, MSG_RESP, rq ? URMA_CR_REM_ACCESS_ABORT_ERR : URMA_CR_REM_OPERATION_ERR);
        break;
      }
      if ((h.flags & (F_FIRST | F_LAST)) == (F_FIRST | F_LAST)) {
        // the whole message is in this slot: straight into the posted buffer, no reassembly and no staging copy
        Unexpected u;
        u.imm = h.operand;
        u.has_imm = (h.flags & F_IMM) != 0;
        u.src_uasid = h.src_uasid;
        u.src_jetty = h.src_jetty;
        u.wr_id = h.wr_id;
        u.want_ack = true;
        memcpy(u.src_eid.raw, h.src_eid, 16);
        RecvWr wr;
        bool have = false;
        {
          std::lock_guard<SpinLock> l(rq->mu);
          if (!rq->posted_empty()) {
            wr = rq->posted_front();
            rq->posted_pop();
            have = true;
          } else {
            u.data.assign(s->payload, s->payload + h.len);
            rq->unexpected.push_back(std::move(u));
          }
        }
        if (have) finish_recv(c, rq, wr, s->payload, h.len, u);
        break;
      }
      const auto key = std::make_pair(h.src_uasid, h.wr_id);
      Reasm* r;
      {
        std::lock_guard<std::mutex> l(c->mu);
        r = &c->reasm[key];
      }
      if (h.flags & F_FIRST) {
        // a receive request that is already posted takes the fragments as they come (no staging copy); its turn in
        // the queue is the moment the message begins
        std::lock_guard<SpinLock> l(rq->mu);
        if (!rq->posted_empty()) {
          r->wr = rq->posted_front();
          rq->posted_pop();
          r->direct = true;
        }
      }
      if (r->direct) {
        if (h.len && uint64_t(h.frag_off) + h.len <= r->wr.sges.bytes()) scatter(r->wr.sges, h.frag_off, s->payload, h.len);
      } else {
        if (h.flags & F_FIRST) r->data.resize(h.total_len);
        if (h.frag_off + h.len <= r->data.size() && h.len) memcpy(r->data.data() + h.frag_off, s->payload, h.len);
      }
      if (h.flags & F_LAST) {
        Unexpected u;
        u.imm = h.operand;
        u.has_imm = (h.flags & F_IMM) != 0;
        u.src_uasid = h.src_uasid;
        u.src_jetty = h.src_jetty;
        u.wr_id = h.wr_id;
        u.want_ack = true;
        memcpy(u.src_eid.raw, h.src_eid, 16);
        const bool direct = r->direct;
        const RecvWr wr = r->wr;
        if (!direct) u.data = std::move(r->data);
        {
          std::lock_guard<std::mutex> l(c->mu);
          c->reasm.erase(key);
        }
        if (direct) finish_recv(c, rq, wr, nullptr, h.total_len, u);   // too long for the buffer: nothing was copied
        else deliver(c, rq, std::move(u));
      }
      break;
    }
    case MSG_RESP: complete_pending(c, h.wr_id, static_cast<urma_cr_status_t>(h.status), h.operand,
                                    h.opcode >= URMA_OPC_CAS && h.opcode <= URMA_OPC_FXOR); break;
    case MSG_RESP_DATA: {
      const bool known = pend_with(c, h.wr_id, [&](Pending& p) {
        scatter(p.local, h.frag_off, s->payload, h.len);
        p.received += h.len;
      });
      if (known && (h.flags & F_LAST)) complete_pending(c, h.wr_id, URMA_CR_SUCCESS, 0, false);
      break;
    }
    case MSG_PROBE: reply(c, h, MSG_RESP, URMA_CR_SUCCESS); break;
    default: break;
  }
}

// Executes up to `budget` messages of the context's inbox. Each ring has one consumer at a time (a flag taken with
// a try); different rings are executed by different threads at once, all of them holding the lifetime lock shared -
// the operations that free a queue take it exclusively and so wait until no message is being handled. A thread that
// finds a ring taken moves on to the next: somebody else is doing that work.
inline bool ring_ready(Ring* in) {
  const uint64_t pos = in->deq.load(std::memory_order_relaxed);
  return in->slots[pos & (kRingSlots - 1)].seq.load(std::memory_order_acquire) == pos + 1;
}
int consume(ShmCtx* c, int budget) {
  // a look without taking anything: most polls find every ring empty
  uint32_t ready = 0;
  for (uint32_t r = 0; r < kRings; ++r) ready |= ring_ready(&c->inbox->ring[r]) ? 1u << r : 0;
  if (!ready && c->deferred_n.load(std::memory_order_acquire) == 0) return 0;
  if (c->deleters.load(std::memory_order_acquire)) return 0;   // let a waiting delete through
  std::shared_lock<std::shared_mutex> life(c->life_mu, std::try_to_lock);
  if (!life.owns_lock()) return 0;
  if (c->deferred_n.load(std::memory_order_acquire)) flush_deferred(c);
  int done = 0;
  static thread_local uint32_t first = 0;   // successive calls of a thread start at different rings
  ++first;
  for (uint32_t k = 0; k < kRings && done < budget; ++k) {
    const uint32_t ri = (first + k) & (kRings - 1);
    if (!(ready >> ri & 1)) continue;
    Ring* in = &c->inbox->ring[ri];
    if (c->ring_busy[ri].exchange(true, std::memory_order_acquire)) continue;
    while (done < budget) {
      const uint64_t pos = in->deq.load(std::memory_order_relaxed);
      Slot* s = &in->slots[pos & (kRingSlots - 1)];
      if (s->seq.load(std::memory_order_acquire) != pos + 1) break;
      handle(c, s);
      in->deq.store(pos + 1, std::memory_order_relaxed);
      s->seq.store(pos + kRingSlots, std::memory_order_release);
      ++done;
    }
    c->ring_busy[ri].store(false, std::memory_order_release);
  }
  return done;
}
// Taken by the operations that free a queue or a completion queue.
struct LifeExclusive {
  ShmCtx* c;
  explicit LifeExclusive(ShmCtx* c_) : c(c_) {
    c->deleters.fetch_add(1, std::memory_order_acq_rel);
    c->life_mu.lock();
  }
  ~LifeExclusive() {
    c->life_mu.unlock();
    c->deleters.fetch_sub(1, std::memory_order_acq_rel);
  }
};

// A cheap clock for "did the application poll just now": the cycle counter.
inline uint64_t fast_ticks() { return ub::cycles(); }
uint64_t ticks_per_us() {
  static const uint64_t v = [] {
    const uint64_t n0 = ub::now_ns(), t0 = fast_ticks();
    while (ub::now_ns() - n0 < 200000) cpu_relax();
    const uint64_t per = (fast_ticks() - t0) * 1000 / (ub::now_ns() - n0);
    return per ? per : 1;
  }();
  return v;
}

// The context's own thread. An application that polls its completion queues executes the inbox itself, inside the
// poll (see op_poll_jfc): the message is then copied once, by the thread that is about to read it, instead of being
// copied by this thread on another core first. Every such poll leaves a time stamp; while the last one is younger
// than a few microseconds this thread stays out of the way, and the moment the application stops polling (it sleeps
// on a completion event, computes, or only ever posts) it executes the inbox as a NIC would, so requests of peers
// progress in any case.
void nic_loop(ShmCtx* c) {
  urma_log_set_thread_tag("shm-nic");
  uint32_t idle = 0, deferred_rounds = 0;
  uint64_t last_scan = ub::now_ns();
  const uint64_t defer_ticks = 3 * ticks_per_us();
  while (!c->stop.load(std::memory_order_relaxed)) {
    const bool app_drives =
        c->inline_poll && fast_ticks() - c->app_poll_ticks.load(std::memory_order_relaxed) < defer_ticks;
    if (app_drives) {
      // stays close for a while (the application may stop polling any moment), then stops burning a core for an
      // application that evidently polls all the time: it looks in every 50 us
      if (++deferred_rounds < 2000) {
        for (int i = 0; i < 8; ++i) cpu_relax();
        if ((deferred_rounds & 1023) != 0) continue;   // the periodic work below still runs now and then
      } else {
        usleep(50);
      }
    } else if (deferred_rounds = 0, consume(c, 64) > 0) {
      idle = 0;
      continue;
    } else if (++idle < 4000) {
      if ((idle & 63) == 0) sched_yield();
      else cpu_relax();
    } else if (idle < 5000) {
      usleep(50);   // quiet for a moment only: look in often (about 50 ms of this before the deep sleep below)
    } else {
      // nothing for a while: sleep until a sender wakes this thread (or 5 ms pass: heartbeat, deadlines).
      // The word goes up first and the rings are looked at once more, so a message published in between is not
      // slept over; a sender that finds the word up takes it down and wakes.
      Inbox* box = c->inbox;
      box->sleeping.store(1, std::memory_order_seq_cst);
      bool pending = c->deferred_n.load(std::memory_order_acquire) != 0;
      for (uint32_t r = 0; r < kRings && !pending; ++r) pending = ring_ready(&box->ring[r]);
      if (!pending) {
        // a short first wait and a second look: a sender that read the word just before it went up does not wake
        // us, and its message may not have been visible at the first look
        const timespec brief{0, 20000};
        syscall(SYS_futex, reinterpret_cast<uint32_t*>(&box->sleeping), FUTEX_WAIT, 1, &brief, nullptr, 0);
        for (uint32_t r = 0; r < kRings && !pending; ++r) pending = ring_ready(&box->ring[r]);
        if (!pending && box->sleeping.load(std::memory_order_relaxed)) {
          const timespec ts{0, 5000000};
          syscall(SYS_futex, reinterpret_cast<uint32_t*>(&box->sleeping), FUTEX_WAIT, 1, &ts, nullptr, 0);
        }
      }
      box->sleeping.store(0, std::memory_order_seq_cst);
      if (pending) idle = 0;
    }
    const uint64_t now = ub::now_ns();
    if (now - last_scan > 20000000ull) {  // every 20 ms: heartbeat + request deadlines
      last_scan = now;
      if (c->reg_slot >= 0) c->dev->reg->ctx[c->reg_slot].heartbeat_ns.store(now);
      for (uint64_t id : pend_select(c, [now](Pending& p) { return now > p.deadline_ns; }))
        complete_pending(c, id, URMA_CR_ACK_TIMEOUT_ERR, 0, false);
    }
  }
}

ShmCtx* C(urma_context_t* ctx) { return reinterpret_cast<ShmCtx*>(ctx->priv); }

// ---------------------------------------------------------------------------------------------- ops: queues
urma_jfc_t* op_create_jfc(urma_context_t*, const urma_jfc_cfg_t* cfg) {
  ShmJfc* j = new ShmJfc();
  j->pub.cfg = *cfg;
  j->pub.priv = j;
  j->ring.resize(cfg->depth ? cfg->depth : 1);
  static std::atomic<uint32_t> ids{1};
  j->pub.id = ids++;
  return &j->pub;
}
urma_status_t op_modify_jfc(urma_jfc_t*, uint32_t, uint32_t) { return URMA_SUCCESS; }
urma_status_t op_delete_jfc(urma_jfc_t* jfc) {
  LifeExclusive life(C(jfc->ctx));
  delete reinterpret_cast<ShmJfc*>(jfc->priv);
  return URMA_SUCCESS;
}
urma_jfce_t* op_create_jfce(urma_context_t*) {
  ShmJfce* e = new ShmJfce();
  e->efd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  e->pub.fd = e->efd;
  e->pub.priv = e;
  return &e->pub;
}
urma_status_t op_delete_jfce(urma_jfce_t* jfce) {
  ShmJfce* e = reinterpret_cast<ShmJfce*>(jfce->priv);
  close(e->efd);
  delete e;
  return URMA_SUCCESS;
}

uint32_t new_jetty_id(ShmCtx* c, uint32_t want) {
  if (want) return want;
  return c->dev->reg->next_jetty.fetch_add(1) + 1;
}
void fill_id(ShmCtx* c, urma_jetty_id_t* id, uint32_t n) {
  id->eid = c->pub.eid;
  id->uasid = c->pub.uasid;
  id->id = n;
}

urma_jfs_t* op_create_jfs(urma_context_t* ctx, const urma_jfs_cfg_t* cfg) {
  ShmCtx* c = C(ctx);
  ShmJfs* j = new ShmJfs();
  j->sq.id = new_jetty_id(c, 0);
  j->sq.jfc = reinterpret_cast<ShmJfc*>(cfg->jfc->priv);
  j->sq.depth = cfg->depth;
  if (cfg->err_timeout) j->sq.err_timeout_ms = 100u << cfg->err_timeout;
  fill_id(c, &j->pub.jfs_id, j->sq.id);
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jfs(urma_jfs_t* jfs, urma_jetty_state_t st) {
  reinterpret_cast<ShmJfs*>(jfs->priv)->sq.state = st;
  return URMA_SUCCESS;
}
urma_status_t op_query_jfs(urma_jfs_t* jfs, urma_jfs_cfg_t* cfg, urma_jetty_state_t* st) {
  *cfg = jfs->cfg;
  *st = static_cast<urma_jetty_state_t>(reinterpret_cast<ShmJfs*>(jfs->priv)->sq.state.load());
  return URMA_SUCCESS;
}
int flush_sq(ShmCtx* c, SendQueue* sq, int cr_cnt, urma_cr_t* cr) {
  int n = 0;
  for (uint64_t id : pend_select(c, [sq](Pending& p) { return p.sq == sq; })) {
    if (n >= cr_cnt) break;
    Pending p;
    if (!pend_take(c, id, &p)) continue;
    sq->inflight.fetch_sub(1);
    cr[n] = urma_cr_t{};
    cr[n].status = URMA_CR_WR_FLUSH_ERR;
    cr[n].user_ctx = p.user_ctx;
    cr[n].local_id = sq->id;
    ++n;
  }
  return n;
}
int op_flush_jfs(urma_jfs_t* jfs, int cr_cnt, urma_cr_t* cr) {
  return flush_sq(C(jfs->ctx), &reinterpret_cast<ShmJfs*>(jfs->priv)->sq, cr_cnt, cr);
}
urma_status_t op_delete_jfs(urma_jfs_t* jfs) {
  ShmJfs* j = reinterpret_cast<ShmJfs*>(jfs->priv);
  urma_cr_t tmp[16];
  while (flush_sq(C(jfs->ctx), &j->sq, 16, tmp) == 16) {
  }
  LifeExclusive life(C(jfs->ctx));
  delete j;
  return URMA_SUCCESS;
}

void rq_init(ShmCtx* c, RecvQueue* rq, const urma_jfr_cfg_t* cfg) {
  rq->id = new_jetty_id(c, cfg->id);
  rq->jfc = reinterpret_cast<ShmJfc*>(cfg->jfc->priv);
  rq->depth = cfg->depth;
  rq->ring.resize(cfg->depth ? cfg->depth : 1);
  rq->token_val = cfg->token_value.token;
  std::lock_guard<std::mutex> l(c->mu);
  c->rqs[rq->id] = rq;
}
void rq_fini(ShmCtx* c, RecvQueue* rq) {
  std::lock_guard<std::mutex> l(c->mu);
  c->rqs.erase(rq->id);
}
urma_jfr_t* op_create_jfr(urma_context_t* ctx, const urma_jfr_cfg_t* cfg) {
  ShmCtx* c = C(ctx);
  ShmJfr* j = new ShmJfr();
  rq_init(c, &j->rq, cfg);
  fill_id(c, &j->pub.jfr_id, j->rq.id);
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jfr(urma_jfr_t* jfr, urma_jetty_state_t st, uint32_t) {
  reinterpret_cast<ShmJfr*>(jfr->priv)->rq.state = st;
  return URMA_SUCCESS;
}
urma_status_t op_query_jfr(urma_jfr_t* jfr, urma_jfr_cfg_t* cfg, urma_jetty_state_t* st) {
  *cfg = jfr->cfg;
  *st = static_cast<urma_jetty_state_t>(reinterpret_cast<ShmJfr*>(jfr->priv)->rq.state.load());
  return URMA_SUCCESS;
}
urma_status_t op_delete_jfr(urma_jfr_t* jfr) {
  ShmJfr* j = reinterpret_cast<ShmJfr*>(jfr->priv);
  rq_fini(C(jfr->ctx), &j->rq);
  LifeExclusive life(C(jfr->ctx));
  delete j;
  return URMA_SUCCESS;
}

struct ShmTarget {
  urma_target_jetty_t pub;
  uint32_t token_val;
};
urma_target_jetty_t* op_import(urma_context_t* ctx, const urma_rjetty_t* rj, const urma_token_t* token) {
  ShmCtx* c = C(ctx);
  if (memcmp(rj->jetty_id.eid.raw, c->pub.eid.raw, 16) != 0) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "remote jetty is on another device (EID mismatch)");
    return nullptr;
  }
  if (!peer_inbox(c, rj->jetty_id.uasid)) {
    urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "no context with uasid %u on %s", rj->jetty_id.uasid,
             c->dev->name.c_str());
    return nullptr;
  }
  ShmTarget* t = new ShmTarget();
  t->pub.id = rj->jetty_id;
  t->pub.trans_mode = rj->trans_mode;
  t->pub.type = rj->type;
  t->pub.priv = t;
  t->token_val = token ? token->token : 0;
  return &t->pub;
}
urma_status_t op_unimport(urma_target_jetty_t* t) {
  delete reinterpret_cast<ShmTarget*>(t->priv);
  return URMA_SUCCESS;
}

urma_jetty_t* op_create_jetty(urma_context_t* ctx, const urma_jetty_cfg_t* cfg) {
  ShmCtx* c = C(ctx);
  ShmJetty* j = new ShmJetty();
  const uint32_t id = new_jetty_id(c, cfg->id);
  j->sq.id = id;
  j->sq.jfc = reinterpret_cast<ShmJfc*>(cfg->jfs_cfg.jfc->priv);
  j->sq.depth = cfg->jfs_cfg.depth;
  if (cfg->jfs_cfg.err_timeout) j->sq.err_timeout_ms = 100u << cfg->jfs_cfg.err_timeout;
  if (cfg->shared_jfr) {
    j->rq = &reinterpret_cast<ShmJfr*>(cfg->shared_jfr->priv)->rq;
  } else {
    urma_jfr_cfg_t rc = cfg->jfr_cfg;
    rc.id = id;
    rq_init(c, &j->own_rq, &rc);
    j->rq = &j->own_rq;
  }
  fill_id(c, &j->pub.jetty_id, id);
  j->pub.priv = j;
  return &j->pub;
}
urma_status_t op_modify_jetty(urma_jetty_t* jt, urma_jetty_state_t st) {
  ShmJetty* j = reinterpret_cast<ShmJetty*>(jt->priv);
  j->sq.state = st;
  if (j->rq == &j->own_rq) j->own_rq.state = st;
  return URMA_SUCCESS;
}
urma_status_t op_query_jetty(urma_jetty_t* jt, urma_jetty_cfg_t* cfg, urma_jetty_state_t* st) {
  *cfg = jt->cfg;
  *st = static_cast<urma_jetty_state_t>(reinterpret_cast<ShmJetty*>(jt->priv)->sq.state.load());
  return URMA_SUCCESS;
}
int op_flush_jetty(urma_jetty_t* jt, int n, urma_cr_t* cr) {
  return flush_sq(C(jt->ctx), &reinterpret_cast<ShmJetty*>(jt->priv)->sq, n, cr);
}
urma_status_t op_delete_jetty(urma_jetty_t* jt) {
  ShmJetty* j = reinterpret_cast<ShmJetty*>(jt->priv);
  urma_cr_t tmp[16];
  while (flush_sq(C(jt->ctx), &j->sq, 16, tmp) == 16) {
  }
  if (j->rq == &j->own_rq) rq_fini(C(jt->ctx), &j->own_rq);
  LifeExclusive life(C(jt->ctx));
  delete j;
  return URMA_SUCCESS;
}
urma_status_t op_bind(urma_jetty_t*, urma_target_jetty_t*) { return URMA_SUCCESS; }
urma_status_t op_unbind(urma_jetty_t*) { return URMA_SUCCESS; }
urma_jetty_grp_t* op_create_grp(urma_context_t* ctx, const char* name, uint32_t policy) {
  urma_jetty_grp_t* g = new urma_jetty_grp_t();
  snprintf(g->name, sizeof(g->name), "%s", name);
  g->policy = policy;
  fill_id(C(ctx), &g->id, new_jetty_id(C(ctx), 0));
  return g;
}
urma_status_t op_delete_grp(urma_jetty_grp_t* g) {
  delete g;
  return URMA_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- ops: memory
urma_token_id_t* op_alloc_token(urma_context_t* ctx) {
  urma_token_id_t* t = new urma_token_id_t();
  t->token_id = C(ctx)->dev->reg->next_token.fetch_add(1) + 1;
  return t;
}
urma_status_t op_free_token(urma_token_id_t* t) {
  delete t;
  return URMA_SUCCESS;
}
struct ShmSeg {
  urma_target_seg_t pub;
  uint32_t token_val;
};
urma_target_seg_t* op_register_seg(urma_context_t* ctx, const urma_seg_cfg_t* cfg) {
  ShmCtx* c = C(ctx);
  ShmSeg* s = new ShmSeg();
  s->pub.seg.ubva.eid = c->pub.eid;
  s->pub.seg.ubva.uasid = c->pub.uasid;
  s->pub.seg.ubva.va = cfg->va;
  s->pub.seg.len = cfg->len;
  s->pub.seg.attr = cfg->access;
  s->pub.seg.token_id = cfg->token_id->token_id;
  s->pub.priv = s;
  s->token_val = cfg->token_value.token;
  std::lock_guard<std::mutex> l(c->mu);
  if (c->segs.count(s->pub.seg.token_id)) {
    delete s;
    return nullptr;  // one registration per token id
  }
  c->segs[s->pub.seg.token_id] = SegReg{cfg->va, cfg->len, cfg->access, cfg->token_value.token};
  return &s->pub;
}
urma_status_t op_unregister_seg(urma_target_seg_t* t) {
  ShmCtx* c = C(t->ctx);
  {
    std::lock_guard<std::mutex> l(c->mu);
    c->segs.erase(t->seg.token_id);
  }
  delete reinterpret_cast<ShmSeg*>(t->priv);
  return URMA_SUCCESS;
}
urma_target_seg_t* op_import_seg(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token, uint64_t,
                                 uint32_t) {
  ShmCtx* c = C(ctx);
  if (memcmp(seg->ubva.eid.raw, c->pub.eid.raw, 16) != 0) return nullptr;
  ShmSeg* s = new ShmSeg();
  s->pub.seg = *seg;
  s->pub.priv = s;
  s->token_val = token ? token->token : 0;
  return &s->pub;
}
urma_status_t op_unimport_seg(urma_target_seg_t* t) {
  delete reinterpret_cast<ShmSeg*>(t->priv);
  return URMA_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- ops: data plane
bool local_ok(const urma_sge_t& g) { return g.addr != 0 || g.len == 0; }

urma_status_t post_one(ShmCtx* c, SendQueue* sq, urma_target_jetty_t* bound, urma_jfs_wr_t* wr) {
  if (sq->state.load() != URMA_JETTY_STATE_READY) return URMA_FAIL;
  urma_target_jetty_t* tj = wr->tjetty ? wr->tjetty : bound;
  if (!tj) return URMA_EINVAL;
  if (sq->inflight.load() >= sq->depth) return URMA_EAGAIN;
  Inbox* box = peer_inbox(c, tj->id.uasid);
  if (!box) return URMA_FAIL;
  Ring* in = ring_of(box, tj->id.id);   // everything for one target jetty travels through one ring, in order
  const uint64_t id = c->next_wr.fetch_add(1);
  Pending p;
  p.sq = sq;
  p.user_ctx = wr->user_ctx;
  p.flag = wr->flag;
  p.opcode = wr->opcode;
  p.deadline_ns = ub::now_ns() + uint64_t(sq->err_timeout_ms) * 1000000ull;
  p.remote = tj->id;
  MsgHdr h{};
  h.opcode = wr->opcode;
  h.src_uasid = c->pub.uasid;
  h.src_jetty = sq->id;
  h.dst_jetty = tj->id.id;
  h.wr_id = id;
  memcpy(h.src_eid, c->pub.eid.raw, 16);
  auto add_pending = [&]() {
    sq->inflight.fetch_add(1);
    pend_put(c, id, p);
  };
  auto fail_pending = [&]() {
    Pending gone;
    if (pend_take(c, id, &gone)) sq->inflight.fetch_sub(1);
  };
  // One fragment: the slot is reserved first and the gather list is copied straight into it.
  auto send_frag = [&](const urma_sg_t& src, uint32_t* si, uint32_t* so, uint32_t off, uint32_t total, uint32_t extra,
                       uint64_t va) -> int {   // bytes sent, or -1 when the peer's ring stayed full
    if (c->drop_tx.load(std::memory_order_relaxed)) {
      uint8_t sink[kSlotPayload];
      return static_cast<int>(gather_frag(src, si, so, sink));
    }
    uint64_t pos;
    Slot* s = reserve_wait(in, &pos, sq->err_timeout_ms);
    if (!s) return -1;
    const uint32_t n = gather_frag(src, si, so, s->payload);
    h.len = n;
    h.frag_off = off;
    h.remote_va = va;
    h.flags = (off == 0 ? F_FIRST : 0) | (off + n == total ? F_LAST : 0) | extra;
    s->h = h;
    ring_publish(s, pos);
    wake_owner(box);
    return static_cast<int>(n);
  };
  switch (wr->opcode) {
    case URMA_OPC_WRITE:
    case URMA_OPC_WRITE_IMM:
    case URMA_OPC_WRITE_NOTIFY: {
      const urma_sg_t &src = wr->rw.src, &dst = wr->rw.dst;
      if (dst.num_sge != 1 || src.num_sge == 0 || src.num_sge > URMA_MAX_SGE || !dst.sge[0].tseg) return URMA_EINVAL;
      const uint32_t total = sg_len(src);
      if (total != dst.sge[0].len) return URMA_EINVAL;
      ShmSeg* rs = reinterpret_cast<ShmSeg*>(dst.sge[0].tseg->priv);
      h.type = MSG_WRITE;
      h.token_id = dst.sge[0].tseg->seg.token_id;
      h.token_val = rs->token_val;
      h.total_len = total;
      h.operand = wr->rw.notify_data;
      p.total = total;
      add_pending();
      uint32_t off = 0, si = 0, so = 0;
      do {
        const int n = send_frag(src, &si, &so, off, total, wr->opcode != URMA_OPC_WRITE ? F_IMM : 0,
                                dst.sge[0].addr + off);
        if (n < 0) {
          fail_pending();
          return URMA_EAGAIN;
        }
        off += static_cast<uint32_t>(n);
      } while (off < total);
      return URMA_SUCCESS;
    }
    case URMA_OPC_READ: {
      const urma_sg_t &src = wr->rw.src, &dst = wr->rw.dst;  // src = remote, dst = local
      if (src.num_sge != 1 || dst.num_sge == 0 || dst.num_sge > URMA_MAX_SGE || !src.sge[0].tseg) return URMA_EINVAL;
      const uint32_t total = src.sge[0].len;
      if (total != sg_len(dst)) return URMA_EINVAL;
      ShmSeg* rs = reinterpret_cast<ShmSeg*>(src.sge[0].tseg->priv);
      h.type = MSG_READ;
      h.token_id = src.sge[0].tseg->seg.token_id;
      h.token_val = rs->token_val;
      h.total_len = total;
      h.remote_va = src.sge[0].addr;
      p.total = total;
      p.local.assign(dst.sge, dst.num_sge);
      add_pending();
      if (!c->drop_tx.load() && !send_msg(box, in, h, nullptr, sq->err_timeout_ms)) {
        fail_pending();
        return URMA_EAGAIN;
      }
      return URMA_SUCCESS;
    }
    case URMA_OPC_CAS:
    case URMA_OPC_SWAP:
    case URMA_OPC_FADD:
    case URMA_OPC_FSUB:
    case URMA_OPC_FAND:
    case URMA_OPC_FOR:
    case URMA_OPC_FXOR: {
      const bool cas = wr->opcode == URMA_OPC_CAS || wr->opcode == URMA_OPC_SWAP;
      urma_sge_t* d = cas ? wr->cas.dst : wr->faa.dst;
      urma_sge_t* s = cas ? wr->cas.src : wr->faa.src;
      if (!d || !d->tseg || d->len != 8) return URMA_EINVAL;
      ShmSeg* rs = reinterpret_cast<ShmSeg*>(d->tseg->priv);
      h.type = MSG_ATOMIC;
      h.token_id = d->tseg->seg.token_id;
      h.token_val = rs->token_val;
      h.remote_va = d->addr;
      h.operand = cas ? wr->cas.swap_data : wr->faa.operand;
      h.cmp = cas ? wr->cas.cmp_data : 0;
      p.total = 8;
      if (s && s->addr) p.local.assign(s, 1);
      add_pending();
      if (!c->drop_tx.load() && !send_msg(box, in, h, nullptr, sq->err_timeout_ms)) {
        fail_pending();
        return URMA_EAGAIN;
      }
      return URMA_SUCCESS;
    }
    case URMA_OPC_SEND:
    case URMA_OPC_SEND_IMM:
    case URMA_OPC_SEND_INVALIDATE: {
      const urma_sg_t& src = wr->send.src;
      if (src.num_sge > URMA_MAX_SGE) return URMA_EINVAL;
      const uint32_t total = sg_len(src);
      h.type = MSG_SEND;
      h.token_val = reinterpret_cast<ShmTarget*>(tj->priv)->token_val;
      h.total_len = total;
      h.operand = wr->send.imm_data;
      p.total = total;
      add_pending();
      uint32_t off = 0, si = 0, so = 0;
      do {
        const int n = send_frag(src, &si, &so, off, total, wr->opcode == URMA_OPC_SEND_IMM ? F_IMM : 0, 0);
        if (n < 0) {
          fail_pending();
          return URMA_EAGAIN;
        }
        off += static_cast<uint32_t>(n);
      } while (off < total);
      return URMA_SUCCESS;
    }
    case URMA_OPC_NOP: {
      h.type = MSG_PROBE;
      add_pending();
      if (!c->drop_tx.load() && !send_msg(box, in, h, nullptr, sq->err_timeout_ms)) {
        fail_pending();
        return URMA_EAGAIN;
      }
      return URMA_SUCCESS;
    }
    default: return URMA_EINVAL;
  }
}

urma_status_t post_send_list(ShmCtx* c, SendQueue* sq, urma_target_jetty_t* bound, urma_jfs_wr_t* wr,
                             urma_jfs_wr_t** bad) {
  for (urma_jfs_wr_t* w = wr; w; w = w->next) {
    const urma_status_t s = post_one(c, sq, bound, w);
    if (s != URMA_SUCCESS) {
      *bad = w;
      return s;
    }
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}
urma_status_t post_recv_list(ShmCtx* c, RecvQueue* rq, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  for (urma_jfr_wr_t* w = wr; w; w = w->next) {
    if (rq->state.load() != URMA_JETTY_STATE_READY || w->src.num_sge > URMA_MAX_SGE) {
      *bad = w;
      return URMA_EINVAL;
    }
    RecvWr r;
    r.user_ctx = w->user_ctx;
    r.sges.assign(w->src.sge, w->src.num_sge);
    Unexpected u;
    bool have = false;
    {
      std::lock_guard<SpinLock> l(rq->mu);
      if (rq->posted_size() >= rq->depth) {
        *bad = w;
        return URMA_EAGAIN;
      }
      rq->posted_push(r);
      if (!rq->unexpected.empty()) {
        u = std::move(rq->unexpected.front());
        rq->unexpected.pop_front();
        have = true;
      }
    }
    if (have) deliver(c, rq, std::move(u));
  }
  *bad = nullptr;
  return URMA_SUCCESS;
}
urma_status_t op_post_jfs(urma_jfs_t* jfs, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  return post_send_list(C(jfs->ctx), &reinterpret_cast<ShmJfs*>(jfs->priv)->sq, nullptr, wr, bad);
}
urma_status_t op_post_jfr(urma_jfr_t* jfr, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  return post_recv_list(C(jfr->ctx), &reinterpret_cast<ShmJfr*>(jfr->priv)->rq, wr, bad);
}
urma_status_t op_post_jetty_send(urma_jetty_t* jt, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad) {
  return post_send_list(C(jt->ctx), &reinterpret_cast<ShmJetty*>(jt->priv)->sq, jt->remote_jetty, wr, bad);
}
urma_status_t op_post_jetty_recv(urma_jetty_t* jt, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad) {
  return post_recv_list(C(jt->ctx), reinterpret_cast<ShmJetty*>(jt->priv)->rq, wr, bad);
}
int op_poll_jfc(urma_jfc_t* jfc, int n, urma_cr_t* cr) {
  ShmJfc* j = reinterpret_cast<ShmJfc*>(jfc->priv);
  if (j->count.load(std::memory_order_acquire) == 0) {
    // nothing completed yet: do the NIC's work on this thread (requests and answers waiting in the inbox), which is
    // what fills this queue; still nothing -> the common answer of a polling loop, without a lock
    // (only a thread that has found the queue empty several times in a row is waiting for something; one that
    // finds completions most of the time is part of a pipelined flow, which the context's own thread serves in
    // parallel)
    ShmCtx* c = C(jfc->ctx);
    if (!c->inline_poll || j->empty_polls.fetch_add(1, std::memory_order_relaxed) + 1 < kInlineAfterEmptyPolls) return 0;
    c->app_poll_ticks.store(fast_ticks(), std::memory_order_relaxed);
    if (consume(c, 32) == 0 || j->count.load(std::memory_order_acquire) == 0) return 0;
  }
  j->empty_polls.store(0, std::memory_order_relaxed);
  std::lock_guard<SpinLock> l(j->mu);
  const uint32_t cap = static_cast<uint32_t>(j->ring.size());
  int k = 0;
  while (k < n && j->head != j->tail) cr[k++] = j->ring[j->head++ % cap];
  j->count.store(j->tail - j->head, std::memory_order_release);
  return k;
}
urma_status_t op_rearm_jfc(urma_jfc_t* jfc, bool) {
  ShmJfc* j = reinterpret_cast<ShmJfc*>(jfc->priv);
  ShmJfce* ce = nullptr;
  {
    std::lock_guard<SpinLock> l(j->mu);
    if (j->head != j->tail && jfc->cfg.jfce) ce = reinterpret_cast<ShmJfce*>(jfc->cfg.jfce->priv);  // fire at once
    else j->armed = true;
  }
  if (ce) {
    {
      std::lock_guard<std::mutex> l(ce->mu);
      ce->fired.push_back(jfc);
    }
    uint64_t one = 1;
    if (write(ce->efd, &one, sizeof(one)) < 0) {
    }
  }
  return URMA_SUCCESS;
}
int op_wait_jfc(urma_jfce_t* jfce, uint32_t cnt, int timeout_ms, urma_jfc_t* out[]) {
  ShmJfce* e = reinterpret_cast<ShmJfce*>(jfce->priv);
  for (;;) {
    {
      std::lock_guard<std::mutex> l(e->mu);
      if (!e->fired.empty()) {
        uint32_t k = 0;
        while (k < cnt && !e->fired.empty()) {
          out[k++] = e->fired.front();
          e->fired.pop_front();
        }
        return static_cast<int>(k);
      }
    }
    pollfd pfd{e->efd, POLLIN, 0};
    const int r = poll(&pfd, 1, timeout_ms);
    if (r == 0) return 0;
    if (r < 0 && errno != EINTR) return -1;
    uint64_t v;
    if (read(e->efd, &v, sizeof(v)) < 0) {
    }
  }
}
void op_ack_jfc(urma_jfc_t*[], uint32_t[], uint32_t) {}

urma_status_t op_get_async_event(urma_context_t* ctx, urma_async_event_t* ev) {
  ShmCtx* c = C(ctx);
  std::lock_guard<std::mutex> l(c->mu);
  if (c->events.empty()) return URMA_EAGAIN;
  *ev = c->events.front();
  c->events.pop_front();
  uint64_t v;
  if (read(c->event_fd, &v, sizeof(v)) < 0) {
  }
  return URMA_SUCCESS;
}
void op_ack_async_event(urma_async_event_t*) {}

// user_ctl opcodes of this provider: 1 = number of pending requests, 2 = inject an async event (in->addr = type),
// 3 = peer liveness: in->addr = uasid, out->rsv = age of the peer's heartbeat in ms (or 0xffffffff if unknown),
// 4 = fault injection: in->addr != 0 makes every outgoing request vanish (requests then end with
//     URMA_CR_ACK_TIMEOUT_ERR after the send queue's error timeout), 0 restores the link
int op_user_ctl(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out) {
  ShmCtx* c = C(ctx);
  switch (in->opcode) {
    case 1: {
      out->rsv = pend_count(c);
      return 0;
    }
    case 2: {
      urma_async_event_t ev{};
      ev.ctx = ctx;
      ev.event_type = static_cast<urma_async_event_type_t>(in->addr);
      {
        std::lock_guard<std::mutex> l(c->mu);
        c->events.push_back(ev);
      }
      uint64_t one = 1;
      if (write(c->event_fd, &one, sizeof(one)) < 0) {
      }
      return 0;
    }
    case 3: {
      out->rsv = 0xffffffffu;
      for (uint32_t i = 0; i < kMaxCtx; ++i) {
        if (c->dev->reg->ctx[i].uasid.load() == static_cast<uint32_t>(in->addr)) {
          const uint64_t hb = c->dev->reg->ctx[i].heartbeat_ns.load();
          const uint64_t now = ub::now_ns();
          out->rsv = static_cast<uint32_t>((now > hb ? now - hb : 0) / 1000000ull);
        }
      }
      return 0;
    }
    case 4: c->drop_tx = in->addr != 0; return 0;
    default: return -1;
  }
}

const urma_ops_t g_ops = {
    "shm",           op_create_jfc,   op_modify_jfc,   op_delete_jfc,     op_create_jfce,     op_delete_jfce,
    op_create_jfs,   op_modify_jfs,   op_query_jfs,    op_flush_jfs,      op_delete_jfs,      op_create_jfr,
    op_modify_jfr,   op_query_jfr,    op_delete_jfr,   op_import,         op_unimport,        op_create_jetty,
    op_modify_jetty, op_query_jetty,  op_flush_jetty,  op_delete_jetty,   op_import,          op_unimport,
    op_bind,         op_unbind,       op_create_grp,   op_delete_grp,     op_alloc_token,     op_free_token,
    op_register_seg, op_unregister_seg, op_import_seg, op_unimport_seg,   op_post_jfs,        op_post_jfr,
    op_post_jetty_send, op_post_jetty_recv, op_poll_jfc, op_rearm_jfc,    op_wait_jfc,        op_ack_jfc,
    op_get_async_event, op_ack_async_event, op_user_ctl,
};

// ---------------------------------------------------------------------------------------------- provider ops
urma_status_t prov_init(const urma_init_attr_t*) {
  std::lock_guard<std::mutex> l(g_mu);
  if (!g_devs.empty()) return URMA_SUCCESS;
  const std::string dir = shm_dir();
  mkdir(dir.c_str(), 0700);
  int n = 2;
  if (const char* e = getenv("URMA_SHM_DEVICES")) n = std::max(1, std::min(8, atoi(e)));
  for (int i = 0; i < n; ++i) {
    Device d;
    d.name = "shm" + std::to_string(i);
    memset(d.eid.raw, 0, 16);
    memcpy(d.eid.raw, "umdk", 4);
    const uint32_t uid = getuid();
    memcpy(d.eid.raw + 8, &uid, 4);
    d.eid.raw[15] = static_cast<uint8_t>(i + 1);
    bool created = false;
    d.reg = static_cast<DevReg*>(map_file(dir + "/dev_" + d.name + ".reg", sizeof(DevReg), true, &created));
    if (!d.reg) return URMA_FAIL;
    uint32_t exp = 0;
    d.reg->magic.compare_exchange_strong(exp, kRegMagic);
    g_devs.push_back(d);
  }
  return URMA_SUCCESS;
}
urma_status_t prov_uninit(void) { return URMA_SUCCESS; }
int prov_get_devices(urma_device_t* devs, int max) {
  std::lock_guard<std::mutex> l(g_mu);
  int n = 0;
  for (auto& d : g_devs) {
    if (n >= max) break;
    memset(&devs[n], 0, sizeof(urma_device_t));
    snprintf(devs[n].name, sizeof(devs[n].name), "%s", d.name.c_str());
    devs[n].eid = d.eid;
    devs[n].priv = &d;
    ++n;
  }
  return n;
}
urma_status_t prov_query(const urma_device_t*, urma_device_attr_t* a) {
  memset(a, 0, sizeof(*a));
  a->max_jfc = a->max_jfs = a->max_jfr = a->max_jetty = 65536;
  a->max_seg = 1u << 20;
  a->max_jfc_depth = a->max_jfs_depth = a->max_jfr_depth = 65536;
  a->max_sge = URMA_MAX_SGE;
  a->max_msg_size = 1ull << 30;
  a->transport_modes = URMA_TM_RM | URMA_TM_RC | URMA_TM_UM;
  a->port_cnt = 1;
  a->atomic_supported = true;
  return URMA_SUCCESS;
}
urma_context_t* prov_create_context(urma_device_t* dev, uint32_t eid_index) {
  Device* d = static_cast<Device*>(dev->priv);
  if (eid_index != 0) return nullptr;
  ShmCtx* c = new ShmCtx();
  c->dev = d;
  c->pub.ops = &g_ops;
  c->pub.eid = d->eid;
  c->pub.eid_index = 0;
  c->pub.priv = c;
  uint32_t uasid = d->reg->next_uasid.fetch_add(1) + 1;
  c->pub.uasid = uasid;
  const uint64_t now = ub::now_ns();
  for (uint32_t i = 0; i < kMaxCtx; ++i) {
    uint32_t exp = 0;
    CtxSlot& s = d->reg->ctx[i];
    // reuse free slots and slots whose owner stopped beating for 10 s
    const uint32_t cur = s.uasid.load();
    if (cur != 0 && now - s.heartbeat_ns.load() > 10000000000ull) exp = cur;
    if (s.uasid.compare_exchange_strong(exp, uasid)) {
      s.pid = getpid();
      s.heartbeat_ns = now;
      c->reg_slot = static_cast<int>(i);
      break;
    }
  }
  c->inbox_path = shm_dir() + "/inbox_" + d->name + "_" + std::to_string(uasid);
  unlink(c->inbox_path.c_str());
  c->inbox = static_cast<Inbox*>(map_file(c->inbox_path, sizeof(Inbox), true));
  if (!c->inbox) {
    delete c;
    return nullptr;
  }
  for (uint32_t r = 0; r < kRings; ++r) {
    for (uint32_t i = 0; i < kRingSlots; ++i) c->inbox->ring[r].slots[i].seq.store(i);
    c->inbox->ring[r].enq = 0;
    c->inbox->ring[r].deq = 0;
  }
  c->inbox->owner_pid = getpid();
  c->inbox->sleeping.store(0);
  c->inbox->magic.store(kRegMagic, std::memory_order_release);
  c->event_fd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC | EFD_SEMAPHORE);
  c->pub.async_fd = c->event_fd;
  if (const char* e = getenv("URMA_SHM_INLINE_POLL")) c->inline_poll = e[0] != '0';
  ticks_per_us();   // calibrated before the first thread needs it
  c->nic = std::thread(nic_loop, c);
  return &c->pub;
}
urma_status_t prov_delete_context(urma_context_t* ctx) {
  ShmCtx* c = C(ctx);
  c->stop = true;
  if (c->nic.joinable()) c->nic.join();
  if (c->reg_slot >= 0) c->dev->reg->ctx[c->reg_slot].uasid.store(0);
  c->inbox->magic.store(0);
  munmap(c->inbox, sizeof(Inbox));
  unlink(c->inbox_path.c_str());
  for (auto& kv : c->peers) munmap(kv.second, sizeof(Inbox));
  close(c->event_fd);
  delete c;
  return URMA_SUCCESS;
}

const urma_provider_ops_t g_prov = {"shm",      prov_init,           prov_uninit,        prov_get_devices,
                                    prov_query, prov_create_context, prov_delete_context};

__attribute__((constructor)) void shm_provider_ctor() { urma_register_provider_ops(&g_prov); }

}  // namespace
