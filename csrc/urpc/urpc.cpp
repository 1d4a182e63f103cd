// URPC framework: function calls over UMQ queues with a TCP control plane.
//
// Kept from the reference (src/urpc/framework): a client "channel" is attached to a server through a TCP handshake
// that exchanges queue information (lib/control/ip/ip_handshaker.c:329-371); requests carry a packed header with
// function id, request id and client channel (protocol/protocol.h); `urpc_func_call` records a pending entry with a
// deadline and optionally blocks (lib/datapath/dp.c:352-535); the server polls its queues, executes the registered
// function and returns the response (dp.c:1258-1322, 1897-2002); the client matches responses to pending entries
// (dp.c:1333-1452); request timeouts and keepalive probes with a callback on peer loss
// (lib/manager/keepalive_probe.c, keepalive_task.c); counters and a call-latency record (lib/control/dfx).
#include "urpc_api.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <sys/eventfd.h>
#include <unistd.h>

#include <algorithm>
#include <set>
#include <string>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <optional>
#include <thread>
#include <unordered_map>
#include <vector>

#include "ub_secure.h"
#include "ub_util.h"
#include "umq_api.h"
#include "urpc_proto.h"
#include "urpc_util.h"

namespace {

using urpc_proto::Head;
constexpr uint32_t kHelloMagic = 0x55525043;  // "URPC"

struct Hello {
  uint32_t magic, version, blob_len, channel;
  uint8_t blob[UMQ_BIND_INFO_SIZE];
  uint32_t sealed;        // response: 1 = data_key is valid and every payload must be sealed with it
  uint8_t data_key[32];   // only ever sent inside the TLS channel
  uint32_t n_extra;       // request: LaneHello records that follow; response: lanes the server made (same number)
};
struct LaneHello {
  uint32_t blob_len;
  uint8_t blob[UMQ_BIND_INFO_SIZE];
};

struct Pending {
  uint64_t func_id, user_ctx, t0, deadline;
  uint32_t lane_id = 0;     // the lane that carried the request (its response returns there)
  bool want_ack = false, acked = false;
  bool sync = false;
  bool done = false;
  int status = 0;
  // A synchronous caller waits inside urpc_func_call with its answer buffer at hand: the answer is copied straight
  // there by whichever thread polls the channel (under the channel's lock), once.
  void* sync_buf = nullptr;
  uint32_t sync_cap = 0, rsp_len = 0;
};
struct Ready {
  urpc_poll_event_t ev;
  uint64_t func_id, user_ctx;
  uint32_t req_id;
  int status;
  umq_buf_t* buf;  // owns the payload (may be null)
};
// Payload sealing of one connection (channel on the client, session on the server): AES-256-GCM under a random key
// that the server hands over inside the TLS handshake exchange. The 32-byte message header travels in clear as
// additional authenticated data and carries the sender's message counter (bytes 20..27), which is the nonce.
constexpr uint8_t kFlagSealed = 0x80;
struct Sealer {
  std::mutex mu;
  // Held from the moment a message takes its counter until it sits in the queue, so that several threads replying
  // on one lane (deferred urpc_func_return calls, the poll thread's inline replies) enqueue in counter order.
  std::mutex tx_order;
  std::unique_ptr<ub::AeadCipher> tx, rx;
  uint64_t tx_nonce = 0, rx_last = 0;
  // Replay window: bit i set = counter (rx_last - i) has been accepted. A message older than the window, or one
  // whose bit is set, is dropped; a late one inside the window is still accepted once.
  uint64_t rx_seen = 0;
  bool replay_check(uint64_t nonce) const {
    if (nonce == 0) return false;
    if (nonce > rx_last) return true;
    const uint64_t d = rx_last - nonce;
    return d < 64 && !((rx_seen >> d) & 1);
  }
  void replay_accept(uint64_t nonce) {
    if (nonce > rx_last) {
      const uint64_t d = nonce - rx_last;
      rx_seen = d >= 64 ? 0 : (rx_seen << d);
      rx_seen |= 1;
      rx_last = nonce;
    } else {
      rx_seen |= 1ull << (rx_last - nonce);
    }
  }
  // One key serves every queue pair of a session: the salt names the lane and the direction, so no two senders ever
  // share a (key, nonce) pair, and each lane keeps its own replay counter.
  void set(const uint8_t key[32], bool is_server, uint32_t lane = 0) {
    tx.reset(new ub::AeadCipher(key, 2 * lane + (is_server ? 1u : 0u)));
    rx.reset(new ub::AeadCipher(key, 2 * lane + (is_server ? 0u : 1u)));
    tx_nonce = rx_last = rx_seen = 0;
  }
  void clear() {
    tx.reset();
    rx.reset();
    tx_nonce = rx_last = rx_seen = 0;
  }
  bool on() const { return tx != nullptr; }
};

// A further queue pair of a channel / session beside the first one (the reference's several queues per channel,
// src/urpc/include/framework/urpc_framework_api.h urpc_channel_queue_add / _pair). On the client it is always a queue
// from urpc_queue_create; on the server it is made during the attach.
struct Lane {
  uint32_t id = 0;        // 1.. per attach, never handed out twice: the id is part of the sealing salt, so a queue
                          // that joins later can never repeat a (key, counter) pair of one that left
  uint64_t umqh = 0;
  Sealer seal;
  std::atomic<bool> closing{false};   // leaving: no new request is sent on it / taken from it
  std::atomic<int> users{0};          // server: poll passes working on the queue right now
};
using LanePtr = std::shared_ptr<Lane>;
constexpr uint32_t kMaxLanes = 16;      // queue pairs of one channel at any time
constexpr uint32_t kMaxLaneId = 255;    // lane ids of one attach (8 bits of the deferred-request cookie)

struct Channel {
  uint32_t id;
  uint64_t umqh = 0;
  std::vector<LanePtr> extra;                 // the further lanes, in the order they joined
  uint32_t next_lane_id = 1;
  uint32_t rr = 0;                            // round-robin cursor of urpc_func_call over the lanes
  urpc_proto::Negotiated proto;               // version and capabilities agreed at attach time
  uint8_t data_key[32] = {0};                 // sealing key of this attach (lanes that join later derive from it)
  bool sealed = false;
  std::mutex ctl_mu;                          // one control exchange at a time
  uint32_t ctl_seq = 0;
  std::vector<uint8_t> rxbuf;                 // control bytes read so far (under ctl_mu)
  int tcp = -1;
  std::unique_ptr<ub::SecureConn> conn;
  Sealer seal;
  std::atomic<bool> attached{false};
  std::atomic<bool> lost{false};
  std::mutex mu;
  std::unordered_map<uint32_t, Pending> pending;
  uint64_t next_deadline_scan = 0;   // under mu
  std::deque<Ready> ready;
  uint32_t next_req = 1;
  uint32_t ka_outstanding = 0;
  uint32_t timeout_ms = 0;          // 0 = the library default
  bool user_queue = false;          // umqh came from urpc_queue_create (not destroyed with the channel)
  std::string server_ip;
  uint16_t server_port = 0;
};
// Lane index of a queue inside a channel (0 = the first queue), -1 when the channel does not hold it.
int channel_lane(Channel* ch, uint64_t qh) {
  if (ch->umqh == qh) return 0;
  for (size_t i = 0; i < ch->extra.size(); ++i)
    if (ch->extra[i]->umqh == qh) return static_cast<int>(i + 1);
  return -1;
}
struct Session {
  uint64_t umqh;
  std::vector<LanePtr> extra;   // guarded by lanes_mu once the session is published
  std::mutex lanes_mu;
  int tcp;
  uint32_t id;
  std::unique_ptr<ub::SecureConn> conn;
  std::mutex conn_wmu;          // writers of the control connection (task answers, notices)
  Sealer seal;
  urpc_proto::Negotiated proto;
  uint8_t data_key[32] = {0};
  bool sealed = false;
  std::atomic<bool> closed{false};    // detached or connection lost: its queues are no longer polled
  std::atomic<int> users{0};          // poll passes inside the session right now
  std::mutex cancel_mu;
  std::set<uint32_t> cancelled;       // deferred requests the client gave up on
  std::vector<uint8_t> rxbuf;         // control bytes read so far (engine thread only)
};
// Lane of a session by id (0 = the first queue pair). Null when it has left.
struct LaneRef {
  uint64_t umqh = 0;
  Sealer* seal = nullptr;
  LanePtr keep;
};
bool session_lane(Session* s, uint32_t lane_id, LaneRef* out) {
  if (lane_id == 0) {
    out->umqh = s->umqh;
    out->seal = &s->seal;
    return !s->closed.load();
  }
  std::lock_guard<std::mutex> l(s->lanes_mu);
  for (auto& ln : s->extra)
    if (ln->id == lane_id && !ln->closing.load()) {
      out->umqh = ln->umqh;
      out->seal = &ln->seal;
      out->keep = ln;
      return !s->closed.load();
    }
  return false;
}
struct Func {
  urpc_func_t fn;
  void* ctx;
};

struct Global {
  std::mutex mu;
  bool inited = false;
  urpc_config_t cfg{};
  std::map<uint32_t, Channel*> channels;
  uint32_t next_ch = 0;
  std::vector<Session*> sessions;
  std::unordered_map<uint64_t, Func> funcs;
  int listen_fd = -1;
  std::thread accept_thr, ka_thr;
  std::atomic<bool> stop{false};
  urpc_keepalive_cb_t ka_cb = nullptr;
  void* ka_ctx = nullptr;
  urpc_stats_t stats{};
  ub::PerfHist lat;
  std::mutex lat_mu;   // guards `lat`
  std::mutex stat_mu;
  int admin_fd = -1;
  std::string admin_path;
  std::thread admin_thr;
  std::atomic<bool> admin_stop{false};
  std::unordered_map<std::string, uint64_t> func_names;   // registered names -> function ids
  std::deque<urpc_async_event_t> events;
  int event_fd = -1;
  ub::PskConfig psk;
  ub::PskConfig server_psk;   // the key in force when the server was started
  bool psk_set = false;   // urpc_set_psk was called: the environment is not consulted
};
Global g;
ub::Logger g_log("URPC");
std::atomic<urpc_perf_recorder_t> g_recorder{nullptr};
std::atomic<void*> g_recorder_ctx{nullptr};
// Arguments by reference: entries appended to a request, each describing registered client memory.
constexpr uint8_t kFlagRefs = 0x40;
struct RefEntry {
  uint64_t addr;
  uint32_t len, token;
  uint8_t blob[UMQ_SEG_BLOB_SIZE];
};
struct CurrentReq {
  uint64_t umqh;
  const RefEntry* refs;
  uint32_t nrefs;
};
thread_local CurrentReq* t_current = nullptr;
thread_local uint64_t t_call_queue = 0;   // queue the request urpc_func_call sends next must use (0 = round robin)
thread_local uint8_t t_call_flags = 0;   // extra header flags for the request urpc_func_call sends next
struct MemSeg {
  void* va;
  uint64_t len;
  uint32_t token;
  uint64_t umq_h;   // 0 while remote access is disabled
  uint8_t blob[UMQ_SEG_BLOB_SIZE];
};
std::mutex g_mem_mu;
std::map<uint64_t, MemSeg> g_mem;
uint64_t g_mem_next = 1;
thread_local bool g_lookup_call = false;   // set by urpc_func_id_get around its own call of the lookup function
std::atomic<urpc_func_poll_cb_t> g_poll_cb{nullptr};
std::atomic<urpc_ctrl_cb_t> g_ctrl_cb{nullptr};
void push_event(urpc_async_event_type_t type, uint32_t chid, int detail) {
  std::lock_guard<std::mutex> l(g.stat_mu);
  if (g.events.size() >= 1024) g.events.pop_front();
  g.events.push_back(urpc_async_event_t{type, chid, detail});
  if (g.event_fd >= 0) {
    const uint64_t one = 1;
    if (write(g.event_fd, &one, sizeof(one)) < 0) {
      // saturated counter: still readable
    }
  }
}
// Counters are bumped from every thread that sends or polls: relaxed atomic adds, no lock (readers take a snapshot
// that may be a few events apart between fields, which is all statistics need).
inline void stat_add(uint64_t& field, uint64_t n = 1) { __atomic_fetch_add(&field, n, __ATOMIC_RELAXED); }
inline void record(urpc_perf_point_t pt, uint64_t ns) {
  if (urpc_perf_recorder_t cb = g_recorder.load(std::memory_order_relaxed)) cb(pt, ns, g_recorder_ctx.load());
}

bool read_full(int fd, void* buf, size_t n, int timeout_ms = 5000) {
  uint8_t* p = static_cast<uint8_t*>(buf);
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    if (poll(&pf, 1, timeout_ms) <= 0) return false;
    const ssize_t r = read(fd, p, n);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}
bool write_full(int fd, const void* buf, size_t n) {
  const uint8_t* p = static_cast<const uint8_t*>(buf);
  while (n) {
    const ssize_t r = write(fd, p, n);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}

uint64_t make_queue(const char* name, const urpc_queue_cfg_t* cfg = nullptr) {
  umq_create_option_t o{};
  snprintf(o.name, sizeof(o.name), "%s", name);
  o.rx_depth = cfg && cfg->rx_depth ? cfg->rx_depth : 128;
  o.tx_depth = cfg && cfg->tx_depth ? cfg->tx_depth : 128;
  o.rx_buf_size = cfg && cfg->rx_buf_size ? cfg->rx_buf_size : 64 * 1024;
  if (cfg && cfg->interrupt) o.mode = UMQ_MODE_INTERRUPT;
  o.token = 0x75727063;
  return umq_create(&o);
}

// Queues one message: the 32-byte envelope `head` (already laid out for its kind; the size word and the sealed
// flag are filled in here, they sit at the same place in every layout) followed by the payload.
constexpr uint8_t kFlagKeepalive = 0x20;   // version 2 response head: answer to a keepalive probe
int send_frame(uint64_t umqh, urpc_req_head_t head, const urpc_sge_t* sg, uint32_t nsg, const void* flat,
               uint32_t flat_len, Sealer* seal) {
  uint32_t total = flat_len;
  for (uint32_t i = 0; i < nsg; ++i) total += sg[i].len;
  const bool sealed = seal && seal->on();
  const uint32_t tag = sealed ? (uint32_t)ub::AeadCipher::kTagBytes : 0u;
  umq_buf_t* b = umq_buf_alloc(sizeof(urpc_req_head_t) + total + tag, 1, umqh);
  if (!b) return URPC_ERR_EAGAIN;
  if (sealed) head.bytes[1] |= kFlagSealed;
  if ((head.bytes[0] & 0xf) != URPC_MSG_ACK) urpc_proto::put_le(head.bytes + 16, total, 4);
  memcpy(b->buf_data, head.bytes, sizeof(head.bytes));
  char* p = b->buf_data + sizeof(urpc_req_head_t);
  for (uint32_t i = 0; i < nsg; ++i) {
    memcpy(p, sg[i].addr, sg[i].len);
    p += sg[i].len;
  }
  if (flat_len) memcpy(p, flat, flat_len);
  std::unique_lock<std::mutex> order;
  if (sealed) order = std::unique_lock<std::mutex>(seal->tx_order);
  if (sealed) {
    // seal in place: header (with the message counter) authenticated, payload encrypted, tag appended
    std::lock_guard<std::mutex> l(seal->mu);
    uint8_t* hb = reinterpret_cast<uint8_t*>(b->buf_data);
    const uint64_t nonce = ++seal->tx_nonce;
    urpc_proto::put_le(hb + 20, nonce, 8);
    uint8_t* body = hb + sizeof(urpc_req_head_t);
    std::vector<uint8_t> ct(total + tag);
    if (!seal->tx->seal(nonce, hb, sizeof(urpc_req_head_t), body, total, ct.data())) {
      umq_buf_free(b);
      return URPC_FAIL;
    }
    memcpy(body, ct.data(), ct.size());
  }
  b->data_size = sizeof(urpc_req_head_t) + total + tag;
  umq_buf_t* bad = nullptr;
  const uint64_t deadline = ub::now_ns() + 2000000000ull;
  for (;;) {
    const int rc = umq_enqueue(umqh, b, &bad);
    if (rc == UMQ_SUCCESS) break;
    if (rc != UMQ_ERR_EAGAIN || ub::now_ns() > deadline) {
      umq_buf_free(b);
      return rc == UMQ_ERR_EAGAIN ? URPC_ERR_EAGAIN : URPC_FAIL;
    }
    sched_yield();
  }
  if (order.owns_lock()) order.unlock();
  stat_add(g.stats.bytes_tx, total);
  return URPC_SUCCESS;
}
int send_msg(uint64_t umqh, const Head& h, const urpc_sge_t* sg, uint32_t nsg, const void* flat, uint32_t flat_len,
             Sealer* seal = nullptr) {
  urpc_req_head_t head;
  urpc_proto::encode(h, &head);
  return send_frame(umqh, head, sg, nsg, flat, flat_len, seal);
}
// A response in the layout of the negotiated version. `req_flags` are the flags of the request being answered:
// a version-2 response to a request that asked for an acknowledgement is ACK_AND_RSP unless the acknowledgement
// already went out by itself (`acked_separately`).
int send_rsp(uint64_t umqh, Sealer* seal, uint8_t version, const Head& req, int status, const void* rsp, uint32_t len,
             bool acked_separately = false, bool keepalive = false) {
  urpc_req_head_t head;
  if (version >= 2) {
    urpc_proto::RspHead r{};
    r.version = version;
    r.type = ((req.flags & 1) && !acked_separately) ? URPC_MSG_ACK_AND_RSP : URPC_MSG_RSP;
    r.flags = keepalive ? kFlagKeepalive : 0;
    r.req_id_range = 1;
    r.req_id = req.req_id;
    r.channel = req.channel;
    r.status = static_cast<int8_t>(status);
    urpc_proto::encode_rsp(r, &head);
  } else {
    Head rh{version, URPC_MSG_RSP, 0, req.func_id, req.req_id, req.channel, 0, static_cast<int8_t>(status)};
    urpc_proto::encode(rh, &head);
  }
  return send_frame(umqh, head, nullptr, 0, rsp, len, seal);
}
int send_ack(uint64_t umqh, Sealer* seal, uint8_t version, const Head& req) {
  urpc_req_head_t head;
  urpc_proto::encode_ack(urpc_proto::AckHead{version, 1, req.req_id, req.channel}, &head);
  return send_frame(umqh, head, nullptr, 0, nullptr, 0, seal);
}

// Checks and removes the seal of a received message in place. False = drop it: sealed without a key, clear although a
// key is set, replayed counter, or bad tag.
bool open_msg(umq_buf_t* b, Sealer* seal) {
  const bool sealed = b->data_size >= sizeof(urpc_req_head_t) && (static_cast<uint8_t>(b->buf_data[1]) & kFlagSealed);
  if (!seal || !seal->on()) return !sealed;
  if (!sealed || b->data_size < sizeof(urpc_req_head_t) + ub::AeadCipher::kTagBytes) return false;
  std::lock_guard<std::mutex> l(seal->mu);
  uint8_t* hb = reinterpret_cast<uint8_t*>(b->buf_data);
  const uint64_t nonce = urpc_proto::get_le(hb + 20, 8);
  if (!seal->replay_check(nonce)) return false;
  const size_t n_sealed = b->data_size - sizeof(urpc_req_head_t);
  std::vector<uint8_t> pt(n_sealed);
  if (!seal->rx->open(nonce, hb, sizeof(urpc_req_head_t), hb + sizeof(urpc_req_head_t), n_sealed, pt.data())) return false;
  seal->replay_accept(nonce);
  memcpy(hb + sizeof(urpc_req_head_t), pt.data(), n_sealed - ub::AeadCipher::kTagBytes);
  b->data_size -= ub::AeadCipher::kTagBytes;
  return true;
}

// Drains the channel's queue: responses complete pending calls, expired calls time out. Caller holds ch->mu.
void channel_progress(Channel* ch) {
  for (size_t lane = 0; lane <= ch->extra.size();) {
    const uint64_t q = lane ? ch->extra[lane - 1]->umqh : ch->umqh;
    Sealer* seal = lane ? &ch->extra[lane - 1]->seal : &ch->seal;
    umq_buf_t* b = umq_dequeue(q);
    if (!b) {
      ++lane;
      continue;
    }
    // one envelope, three layouts: the type nibble says which
    const urpc_req_head_t* raw = reinterpret_cast<const urpc_req_head_t*>(b->buf_data);
    const bool framed = b->data_size >= sizeof(urpc_req_head_t);
    const uint8_t type = framed ? (raw->bytes[0] & 0xf) : 0xff;
    const uint8_t version = framed ? (raw->bytes[0] >> 4) : 0;
    urpc_proto::RspHead r{};
    urpc_proto::AckHead ack{};
    bool ok = framed && version == ch->proto.version && open_msg(b, seal);
    bool keepalive = false;
    if (ok && type == URPC_MSG_ACK) {
      ok = version >= 2 && urpc_proto::decode_ack(raw, &ack);
    } else if (ok && version >= 2) {
      ok = urpc_proto::decode_rsp(raw, &r);
      keepalive = (r.flags & kFlagKeepalive) != 0;
    } else if (ok) {   // version 1: responses use the request layout
      Head h;
      ok = urpc_proto::decode(raw, &h) && h.type == URPC_MSG_RSP;
      r.req_id = h.req_id;
      r.status = h.status;
      r.total_size = h.total_size;
      keepalive = h.func_id == URPC_FUNC_ID_KEEPALIVE;
    }
    if (!ok) {
      if (framed) stat_add(g.stats.errors);
      umq_buf_free(b);
      continue;
    }
    if (type == URPC_MSG_ACK) {   // the server has the request(s) and will answer later
      for (uint32_t k = 0; k < ack.req_id_range; ++k) {
        auto it = ch->pending.find(ack.req_id + k);
        if (it == ch->pending.end() || it->second.acked) continue;
        it->second.acked = true;
        if (!it->second.sync && it->second.want_ack)
          ch->ready.push_back(Ready{URPC_POLL_ACK, it->second.func_id, it->second.user_ctx, it->first, 0, nullptr});
      }
      umq_buf_free(b);
      continue;
    }
    stat_add(g.stats.bytes_rx, r.total_size);
    if (keepalive) {
      ch->ka_outstanding = 0;
      umq_buf_free(b);
      continue;
    }
    auto it = ch->pending.find(r.req_id);
    if (it == ch->pending.end()) {  // late answer of a call that already timed out or was cancelled
      umq_buf_free(b);
      continue;
    }
    Pending& p = it->second;
    {
      const uint64_t took = ub::now_ns() - p.t0;
      stat_add(g.stats.responses);
      {
        std::lock_guard<std::mutex> l(g.lat_mu);
        g.lat.add(took);
      }
      record(URPC_PERF_CALL_TO_RESPONSE, took);
    }
    if (p.sync) {
      p.rsp_len = b->data_size - static_cast<uint32_t>(sizeof(urpc_req_head_t));
      if (p.sync_buf && p.rsp_len)
        memcpy(p.sync_buf, b->buf_data + sizeof(urpc_req_head_t), std::min(p.rsp_len, p.sync_cap));
      p.status = r.status;
      p.done = true;
      umq_buf_free(b);
    } else {
      ch->ready.push_back(Ready{URPC_POLL_RSP, p.func_id, p.user_ctx, r.req_id, r.status, b});
      ch->pending.erase(it);
    }
  }
  // deadlines are whole milliseconds: the table of calls in flight is walked at most once per millisecond, not on
  // every poll of a busy channel
  const uint64_t now = ub::now_ns();
  if (now < ch->next_deadline_scan) return;
  ch->next_deadline_scan = now + 1000000ull;
  for (auto it = ch->pending.begin(); it != ch->pending.end();) {
    Pending& p = it->second;
    if (!p.done && now > p.deadline) {
      stat_add(g.stats.timeouts);
      if (p.sync) {
        p.status = URPC_ERR_TIMEOUT;
        p.done = true;
        ++it;
      } else {
        ch->ready.push_back(Ready{URPC_POLL_TIMEOUT, p.func_id, p.user_ctx, it->first, URPC_ERR_TIMEOUT, nullptr});
        it = ch->pending.erase(it);
      }
    } else {
      ++it;
    }
  }
}

// The key in force: the one given to urpc_set_psk, else URPC_PSK / URPC_PSK_ID from the environment (a malformed
// environment key yields a key nobody else has, so that connections fail instead of running in clear text).
ub::PskConfig current_psk() {
  std::lock_guard<std::mutex> l(g.mu);
  if (!g.psk_set) {
    bool bad = false;
    g.psk = ub::PskConfig::from_env("URPC", &bad);
    if (bad) {
      g.psk.key.assign(32, 0);
      ub::random_bytes(g.psk.key.data(), g.psk.key.size());
    }
    g.psk_set = true;
  }
  return g.psk;
}

// The version word this process advertises. URPC_PROTO_MAX / URPC_PROTO_MIN narrow the range (an operator pins a
// mixed fleet to the old protocol during an upgrade; tests use them to stand in for an older or newer build).
uint32_t my_version_word() {
  uint32_t hi = urpc_proto::kVersion, lo = urpc_proto::kVersionMin;
  if (const char* e = getenv("URPC_PROTO_MAX")) hi = static_cast<uint32_t>(atoi(e));
  if (const char* e = getenv("URPC_PROTO_MIN")) lo = static_cast<uint32_t>(atoi(e));
  if (hi < 1 || hi > 255) hi = urpc_proto::kVersion;
  if (lo < 1 || lo > hi) lo = hi < urpc_proto::kVersionMin ? hi : urpc_proto::kVersionMin;
  if (hi == 1) return 1;   // exactly what a version-1 build sends
  return urpc_proto::pack_version(static_cast<uint8_t>(hi), static_cast<uint8_t>(lo), urpc_proto::kCapsAll);
}

// ------------------------------------------------------------------------------------------ control task engine
// One thread serves the control connections of all sessions. A control message becomes a task: an object in a slab
// with an id, a step counter and a deadline. A step either finishes the task (the answer goes out) or asks to be
// run again after a pause; the pause is a timer on the wheel, so a task that has to wait (for poll passes to leave a
// queue that is being retired) never blocks the messages of other sessions. Reference: the asynchronous task
// engine of the IP control plane (src/urpc/framework/lib/control/ip/task_engine.c) drives attach / detach / queue
// changes as multi-step tasks in the same way.
struct CtlTask {
  uint32_t id = 0;
  Session* s = nullptr;
  uint16_t opcode = 0;
  uint32_t seq = 0;
  int step = 0;
  uint64_t deadline_ms = 0;
  uint32_t timer = 0;
  std::vector<uint8_t> payload, answer;
  LanePtr lane;
};
struct Engine {
  std::mutex mu;                       // watch list and run queue
  std::vector<Session*> watched;
  std::deque<uint64_t> runq;           // slab handles of tasks ready for their next step
  urpc_util::Slab<CtlTask> tasks{32};
  urpc_util::IdGen ids{1, 4096};
  std::unique_ptr<urpc_util::TimerWheel> wheel;   // made when the engine starts: its clock begins at that moment
  std::thread thr;
  std::atomic<bool> stop{false};
  bool running = false;
  urpc_ctl_stats_t st{};
  std::mutex st_mu;
};
Engine g_eng;
constexpr uint64_t kTaskDeadlineMs = 3000;
uint64_t now_ms() { return ub::now_ns() / 1000000ull; }

void ctl_answer(Session* s, uint16_t opcode, uint32_t seq, int status, const void* payload, uint32_t len) {
  urpc_proto::CtlHead h{urpc_proto::kCtlMagic, opcode, urpc_proto::kCtlAnswer, seq, status, len};
  std::lock_guard<std::mutex> l(s->conn_wmu);
  if (!s->conn) return;
  if (s->conn->write_full(&h, sizeof(h)) && len) s->conn->write_full(payload, len);
}
// Server -> client notice (no answer expected).
void ctl_notice(Session* s, uint16_t opcode, const void* payload, uint32_t len) {
  urpc_proto::CtlHead h{urpc_proto::kCtlMagic, opcode, 0, 0, 0, len};
  std::lock_guard<std::mutex> l(s->conn_wmu);
  if (!s->conn || s->closed.load()) return;
  if (s->conn->write_full(&h, sizeof(h)) && len) s->conn->write_full(payload, len);
  std::lock_guard<std::mutex> l2(g_eng.st_mu);
  ++g_eng.st.notices_sent;
}

enum StepResult { kStepDone = 0, kStepAgain = 1 };
// Retiring a session: stop polling it, wait until no poll pass is inside, then free its queues. The Session object
// stays in the table (ids are positions) with no queues.
StepResult step_retire(CtlTask& t, int* status) {
  Session* s = t.s;
  if (t.step == 0) {
    s->closed = true;
    t.step = 1;
  }
  if (s->users.load() > 0 && now_ms() < t.deadline_ms) return kStepAgain;
  {
    std::lock_guard<std::mutex> l(s->lanes_mu);
    for (auto& ln : s->extra) {
      umq_unbind(ln->umqh);
      umq_destroy(ln->umqh);
    }
    s->extra.clear();
  }
  if (s->umqh) {
    umq_unbind(s->umqh);
    umq_destroy(s->umqh);
    s->umqh = 0;
  }
  if (urpc_ctrl_cb_t cb = g_ctrl_cb.load()) cb(URPC_CTRL_DETACH, s->id, 0);
  {
    std::lock_guard<std::mutex> l(g_eng.st_mu);
    ++g_eng.st.sessions_retired;
  }
  *status = URPC_SUCCESS;
  return kStepDone;
}
StepResult step_queue_add(CtlTask& t, int* status) {
  Session* s = t.s;
  uint32_t lane_id = 0, blob_len = 0;
  if (t.payload.size() < 8) {
    *status = URPC_ERR_EINVAL;
    return kStepDone;
  }
  memcpy(&lane_id, t.payload.data(), 4);
  memcpy(&blob_len, t.payload.data() + 4, 4);
  if (lane_id == 0 || lane_id > kMaxLaneId || blob_len > UMQ_BIND_INFO_SIZE || t.payload.size() < 8 + blob_len ||
      !(s->proto.caps & urpc_proto::kCapLiveQueues)) {
    *status = URPC_ERR_EINVAL;
    return kStepDone;
  }
  {
    std::lock_guard<std::mutex> l(s->lanes_mu);
    bool clash = s->extra.size() + 1 >= kMaxLanes;
    for (auto& ln : s->extra) clash = clash || ln->id >= lane_id;   // ids only grow: a salt is never used twice
    if (clash) {
      *status = URPC_ERR_EINVAL;
      return kStepDone;
    }
  }
  const uint64_t lq = make_queue("urpc-srv");
  if (!lq || umq_bind(lq, t.payload.data() + 8, blob_len) != UMQ_SUCCESS) {
    if (lq) umq_destroy(lq);
    *status = URPC_FAIL;
    return kStepDone;
  }
  LanePtr ln(new Lane());
  ln->id = lane_id;
  ln->umqh = lq;
  if (s->sealed) ln->seal.set(s->data_key, true, lane_id);
  t.answer.resize(UMQ_BIND_INFO_SIZE);
  t.answer.resize(umq_bind_info_get(lq, t.answer.data(), UMQ_BIND_INFO_SIZE));
  {
    std::lock_guard<std::mutex> l(s->lanes_mu);
    s->extra.push_back(ln);   // published: the next poll pass takes requests from it
  }
  *status = URPC_SUCCESS;
  return kStepDone;
}
StepResult step_queue_rm(CtlTask& t, int* status) {
  Session* s = t.s;
  if (t.step == 0) {
    uint32_t lane_id = 0;
    if (t.payload.size() >= 4) memcpy(&lane_id, t.payload.data(), 4);
    {
      std::lock_guard<std::mutex> l(s->lanes_mu);
      for (auto& ln : s->extra)
        if (ln->id == lane_id && lane_id != 0) t.lane = ln;
    }
    if (!t.lane) {
      *status = URPC_ERR_EINVAL;
      return kStepDone;
    }
    t.lane->closing = true;   // poll passes that start from now on leave the queue alone
    t.step = 1;
  }
  if (t.lane->users.load() > 0 && now_ms() < t.deadline_ms) return kStepAgain;   // a pass is still inside
  {
    std::lock_guard<std::mutex> l(s->lanes_mu);
    s->extra.erase(std::remove(s->extra.begin(), s->extra.end(), t.lane), s->extra.end());
  }
  umq_unbind(t.lane->umqh);
  umq_destroy(t.lane->umqh);
  t.lane.reset();
  *status = URPC_SUCCESS;
  return kStepDone;
}
StepResult step_task_cancel(CtlTask& t, int* status) {
  uint32_t req_id = 0;
  if (t.payload.size() >= 4) memcpy(&req_id, t.payload.data(), 4);
  std::lock_guard<std::mutex> l(t.s->cancel_mu);
  if (t.s->cancelled.size() >= 1024) t.s->cancelled.erase(t.s->cancelled.begin());
  t.s->cancelled.insert(req_id);
  *status = URPC_SUCCESS;
  return kStepDone;
}

void engine_enqueue(uint64_t h) {
  std::lock_guard<std::mutex> l(g_eng.mu);
  g_eng.runq.push_back(h);
}
// Creates the task of one control message (opcode 0 = the connection ended: retire without an answer).
void engine_new_task(Session* s, uint16_t opcode, uint32_t seq, std::vector<uint8_t> payload) {
  CtlTask* t = nullptr;
  const uint64_t h = g_eng.tasks.acquire(&t);
  uint32_t id = 0;
  if (!g_eng.ids.alloc(&id)) {   // more live tasks than ids: refuse instead of queueing without bound
    g_eng.tasks.release(h);
    if (opcode) ctl_answer(s, opcode, seq, URPC_ERR_EAGAIN, nullptr, 0);
    return;
  }
  t->id = id;
  t->s = s;
  t->opcode = opcode;
  t->seq = seq;
  t->payload = std::move(payload);
  t->deadline_ms = now_ms() + kTaskDeadlineMs;
  t->timer = g_eng.wheel->create([h] { engine_enqueue(h); });
  {
    std::lock_guard<std::mutex> l(g_eng.st_mu);
    ++g_eng.st.tasks_started;
  }
  engine_enqueue(h);
}
void engine_run_task(uint64_t h) {
  CtlTask* t = g_eng.tasks.get(h);
  if (!t) return;
  int status = URPC_FAIL;
  StepResult r = kStepDone;
  switch (t->opcode) {
    case 0:
    case urpc_proto::kCtlDetach: r = step_retire(*t, &status); break;
    case urpc_proto::kCtlQueueAdd: r = step_queue_add(*t, &status); break;
    case urpc_proto::kCtlQueueRm: r = step_queue_rm(*t, &status); break;
    case urpc_proto::kCtlTaskCancel: r = step_task_cancel(*t, &status); break;
    default: status = URPC_ERR_EINVAL; break;
  }
  if (r == kStepAgain) {
    g_eng.wheel->start(t->timer, g_eng.wheel->tick_ms());
    return;
  }
  const bool late = now_ms() >= t->deadline_ms;
  if (t->opcode) ctl_answer(t->s, t->opcode, t->seq, status, t->answer.data(), static_cast<uint32_t>(t->answer.size()));
  {
    std::lock_guard<std::mutex> l(g_eng.st_mu);
    if (status == URPC_SUCCESS) ++g_eng.st.tasks_done;
    else ++g_eng.st.tasks_failed;
    if (late) ++g_eng.st.tasks_timed_out;
  }
  g_eng.wheel->destroy(t->timer);
  g_eng.ids.free(t->id);
  g_eng.tasks.release(h);
}
// Reads what the control connection holds without ever waiting for more: bytes collect in the session's buffer
// until a whole message is there. False = the connection ended (or sent something that is not a control message).
bool engine_read(Session* s) {
  for (;;) {
    uint8_t tmp[512];
    size_t want = sizeof(urpc_proto::CtlHead);
    if (s->rxbuf.size() >= sizeof(urpc_proto::CtlHead)) {
      urpc_proto::CtlHead h;
      memcpy(&h, s->rxbuf.data(), sizeof(h));
      if (h.magic != urpc_proto::kCtlMagic || h.len > urpc_proto::kCtlMaxPayload) return false;
      want = sizeof(h) + h.len;
      if (s->rxbuf.size() >= want) {
        std::vector<uint8_t> payload(s->rxbuf.begin() + sizeof(h), s->rxbuf.begin() + want);
        s->rxbuf.erase(s->rxbuf.begin(), s->rxbuf.begin() + want);
        if (s->proto.version < 2) return false;   // a version-1 peer has no control messages
        engine_new_task(s, h.opcode, h.seq, std::move(payload));
        continue;
      }
    }
    // one byte at a time would be slow, a blocking read of the rest could stall every other session: read what is
    // there (pending() for decrypted bytes, poll() for the socket), never more than the message still needs
    pollfd pf{s->tcp, POLLIN, 0};
    if (!s->conn->pending() && poll(&pf, 1, 0) <= 0) return true;
    size_t n = want - s->rxbuf.size();
    if (n > sizeof(tmp)) n = sizeof(tmp);
    // a TLS record may carry less than the message needs; one byte is always safe, the rest only when buffered
    if (!s->conn->read_full(tmp, 1, 200)) return false;
    s->rxbuf.push_back(tmp[0]);
    while (--n > 0 && s->conn->pending()) {
      if (!s->conn->read_full(tmp, 1, 200)) return false;
      s->rxbuf.push_back(tmp[0]);
    }
  }
}
void engine_loop() {
  while (!g_eng.stop.load()) {
    std::vector<Session*> ss;
    {
      std::lock_guard<std::mutex> l(g_eng.mu);
      ss = g_eng.watched;
    }
    std::vector<pollfd> pfs;
    for (Session* s : ss) pfs.push_back(pollfd{s->tcp, POLLIN, 0});
    bool buffered = false;
    for (Session* s : ss) buffered = buffered || (s->conn && s->conn->pending());
    if (pfs.empty()) usleep(g_eng.wheel->tick_ms() * 1000);
    else poll(pfs.data(), pfs.size(), buffered ? 0 : static_cast<int>(g_eng.wheel->tick_ms()));
    for (size_t i = 0; i < ss.size(); ++i) {
      Session* s = ss[i];
      if (!(pfs[i].revents & (POLLIN | POLLHUP | POLLERR)) && !s->conn->pending()) continue;
      if (engine_read(s)) continue;
      {   // the connection is gone: stop watching, retire the session
        std::lock_guard<std::mutex> l(g_eng.mu);
        g_eng.watched.erase(std::remove(g_eng.watched.begin(), g_eng.watched.end(), s), g_eng.watched.end());
      }
      if (!s->closed.load()) engine_new_task(s, 0, 0, {});
    }
    g_eng.wheel->run(now_ms());
    for (;;) {
      uint64_t h = 0;
      {
        std::lock_guard<std::mutex> l(g_eng.mu);
        if (g_eng.runq.empty()) break;
        h = g_eng.runq.front();
        g_eng.runq.pop_front();
      }
      engine_run_task(h);
    }
  }
}
void engine_watch(Session* s) {
  std::lock_guard<std::mutex> l(g_eng.mu);
  g_eng.watched.push_back(s);
  if (!g_eng.running) {
    g_eng.stop = false;
    g_eng.wheel.reset(new urpc_util::TimerWheel(5, now_ms()));
    g_eng.thr = std::thread(engine_loop);
    g_eng.running = true;
  }
}
void engine_stop() {
  {
    std::lock_guard<std::mutex> l(g_eng.mu);
    if (!g_eng.running) return;
    g_eng.stop = true;
  }
  g_eng.thr.join();
  std::lock_guard<std::mutex> l(g_eng.mu);
  g_eng.running = false;
  g_eng.watched.clear();
  g_eng.runq.clear();
}

// ---------------------------------------------------------------------------------- control messages, client side
// What the server sends without being asked (today: the function table changed) becomes an asynchronous event.
void ctl_handle_notice(Channel* ch, const urpc_proto::CtlHead& h, const std::vector<uint8_t>& payload) {
  if (h.opcode == urpc_proto::kCtlFuncChange && payload.size() >= 12) {
    uint32_t added = 0;
    memcpy(&added, payload.data() + 8, 4);
    push_event(URPC_EVENT_FUNC_CHANGED, ch->id, static_cast<int>(added));
  }
}
// Reads one whole control message if the connection has (or, within `wait_ms`, gets) one. 1 = message, 0 = none
// yet, -1 = the connection ended. Caller holds ch->ctl_mu.
int ctl_read_one(Channel* ch, urpc_proto::CtlHead* h, std::vector<uint8_t>* payload, int wait_ms) {
  const uint64_t deadline = now_ms() + static_cast<uint64_t>(wait_ms);
  for (;;) {
    if (ch->rxbuf.size() >= sizeof(*h)) {
      memcpy(h, ch->rxbuf.data(), sizeof(*h));
      if (h->magic != urpc_proto::kCtlMagic || h->len > urpc_proto::kCtlMaxPayload) return -1;
      if (ch->rxbuf.size() >= sizeof(*h) + h->len) {
        payload->assign(ch->rxbuf.begin() + sizeof(*h), ch->rxbuf.begin() + sizeof(*h) + h->len);
        ch->rxbuf.erase(ch->rxbuf.begin(), ch->rxbuf.begin() + sizeof(*h) + h->len);
        return 1;
      }
    }
    if (!ch->conn) return -1;
    if (!ch->conn->pending()) {
      const uint64_t now = now_ms();
      pollfd pf{ch->tcp, POLLIN, 0};
      if (poll(&pf, 1, now >= deadline ? 0 : static_cast<int>(deadline - now)) <= 0) return 0;
    }
    uint8_t byte;
    if (!ch->conn->read_full(&byte, 1, 200)) return -1;
    ch->rxbuf.push_back(byte);
  }
}
// One request / answer exchange on the channel's control connection. Notices that arrive in between are handled.
int ctl_call(Channel* ch, uint16_t opcode, const void* payload, uint32_t len, std::vector<uint8_t>* answer,
             int timeout_ms) {
  std::lock_guard<std::mutex> l(ch->ctl_mu);
  if (!ch->conn) return URPC_ERR_SESSION_CLOSE;
  urpc_proto::CtlHead h{urpc_proto::kCtlMagic, opcode, 0, ++ch->ctl_seq, 0, len};
  if (!ch->conn->write_full(&h, sizeof(h)) || (len && !ch->conn->write_full(payload, len)))
    return URPC_ERR_SESSION_CLOSE;
  const uint64_t deadline = now_ms() + static_cast<uint64_t>(timeout_ms);
  for (;;) {
    const uint64_t now = now_ms();
    if (now >= deadline) return URPC_ERR_TIMEOUT;
    urpc_proto::CtlHead rh;
    std::vector<uint8_t> rp;
    const int rc = ctl_read_one(ch, &rh, &rp, static_cast<int>(deadline - now));
    if (rc < 0) return URPC_ERR_SESSION_CLOSE;
    if (rc == 0) continue;
    if (!(rh.flags & urpc_proto::kCtlAnswer)) {
      ctl_handle_notice(ch, rh, rp);
      continue;
    }
    if (rh.seq != h.seq) continue;   // answer of an exchange that was given up earlier
    if (answer) answer->swap(rp);
    return rh.status;
  }
}
// Picks up notices while nobody is in an exchange (called from the channel's progress path).
void ctl_drain_notices(Channel* ch) {
  if (ch->proto.version < 2 || !ch->attached.load()) return;
  std::unique_lock<std::mutex> l(ch->ctl_mu, std::try_to_lock);
  if (!l.owns_lock() || !ch->conn) return;
  for (int i = 0; i < 8; ++i) {
    urpc_proto::CtlHead rh;
    std::vector<uint8_t> rp;
    if (ctl_read_one(ch, &rh, &rp, 0) != 1) return;
    if (!(rh.flags & urpc_proto::kCtlAnswer)) ctl_handle_notice(ch, rh, rp);
  }
}

void accept_loop() {
  while (!g.stop.load()) {
    pollfd pf{g.listen_fd, POLLIN, 0};
    if (poll(&pf, 1, 100) <= 0) continue;
    const int fd = accept(g.listen_fd, nullptr, nullptr);
    if (fd < 0) continue;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    Hello hello;
    std::string err;
    std::unique_ptr<ub::SecureConn> conn = ub::SecureConn::server(fd, g.server_psk, 3000, &err);
    if (!conn) {  // wrong key, clear-text client, or a client that stalled in the handshake
      g_log.log(ub::kLogWarn, "connection refused in the secure handshake: %s", err.c_str());
      std::lock_guard<std::mutex> l(g.stat_mu);
      stat_add(g.stats.errors);
      close(fd);
      continue;
    }
    if (!conn->read_full(&hello, sizeof(hello), 5000) || hello.magic != kHelloMagic) {
      conn.reset();
      close(fd);
      continue;
    }
    const urpc_proto::Negotiated nego = urpc_proto::negotiate(my_version_word(), hello.version);
    if (nego.version == 0) {   // nothing in common: say so (version word 0) instead of just hanging up
      g_log.log(ub::kLogWarn, "attach refused: peer speaks protocol %u..%u, this side %u..%u",
                (hello.version >> 8) & 0xff ? (hello.version >> 8) & 0xff : hello.version & 0xff, hello.version & 0xff,
                (my_version_word() >> 8) & 0xff, my_version_word() & 0xff);
      Hello no{};
      no.magic = kHelloMagic;
      conn->write_full(&no, sizeof(no));
      conn.reset();
      close(fd);
      std::lock_guard<std::mutex> l(g.stat_mu);
      stat_add(g.stats.errors);
      continue;
    }
    // one server queue per queue of the client's channel; the session is published only when all are bound
    std::vector<LaneHello> lane_req(hello.n_extra < kMaxLanes ? hello.n_extra : 0), lane_rsp(lane_req.size());
    bool ok = hello.n_extra < kMaxLanes;
    for (size_t i = 0; ok && i < lane_req.size(); ++i)
      ok = conn->read_full(&lane_req[i], sizeof(LaneHello), 5000) && lane_req[i].blob_len <= UMQ_BIND_INFO_SIZE;
    const uint64_t q = ok ? make_queue("urpc-srv") : 0;
    Hello rsp{};
    rsp.magic = kHelloMagic;
    // the chosen version; a version-1 client compares the whole word with 1, so no capability bits for it
    rsp.version = nego.version >= 2 ? urpc_proto::pack_version(nego.version, nego.version, nego.caps) : nego.version;
    rsp.n_extra = static_cast<uint32_t>(lane_req.size());
    Session* s = new Session();
    s->proto = nego;
    ok = ok && q && umq_bind(q, hello.blob, hello.blob_len) == UMQ_SUCCESS;
    for (size_t i = 0; ok && i < lane_req.size(); ++i) {
      const uint64_t lq = make_queue("urpc-srv");
      if (!lq) {
        ok = false;
        break;
      }
      s->extra.emplace_back(new Lane());
      s->extra.back()->umqh = lq;
      s->extra.back()->id = static_cast<uint32_t>(i + 1);
      ok = umq_bind(lq, lane_req[i].blob, lane_req[i].blob_len) == UMQ_SUCCESS;
      lane_rsp[i].blob_len = umq_bind_info_get(lq, lane_rsp[i].blob, sizeof(lane_rsp[i].blob));
    }
    if (ok && conn->encrypted()) {
      ok = ub::random_bytes(rsp.data_key, sizeof(rsp.data_key));
      if (ok) {
        rsp.sealed = 1;
        s->sealed = true;
        memcpy(s->data_key, rsp.data_key, sizeof(s->data_key));
        s->seal.set(rsp.data_key, true, 0);
        for (size_t i = 0; i < s->extra.size(); ++i) s->extra[i]->seal.set(rsp.data_key, true, static_cast<uint32_t>(i + 1));
      }
    }
    if (!ok) {
      if (q) umq_destroy(q);
      for (auto& ln : s->extra) umq_destroy(ln->umqh);
      delete s;
      conn.reset();
      close(fd);
      continue;
    }
    rsp.blob_len = umq_bind_info_get(q, rsp.blob, sizeof(rsp.blob));
    s->umqh = q;
    s->tcp = fd;
    s->id = 0;
    {
      std::lock_guard<std::mutex> l(g.mu);
      s->id = static_cast<uint32_t>(g.sessions.size());
      rsp.channel = s->id;
      g.sessions.push_back(s);
    }
    s->conn = std::move(conn);
    if (urpc_ctrl_cb_t cb = g_ctrl_cb.load()) cb(URPC_CTRL_ATTACH, s->id, hello.channel);
    bool sent = s->conn->write_full(&rsp, sizeof(rsp));
    for (size_t i = 0; sent && i < lane_rsp.size(); ++i) sent = s->conn->write_full(&lane_rsp[i], sizeof(LaneHello));
    // from here on the control connection belongs to the task engine: control messages of the client, and its end
    // of file (a client that went away, also one that left during the handshake) retires the session
    engine_watch(s);
  }
}

void keepalive_loop() {
  const uint32_t interval = g.cfg.keepalive_interval_ms;
  const uint32_t limit = g.cfg.keepalive_miss_limit ? g.cfg.keepalive_miss_limit : 3;
  while (!g.stop.load()) {
    for (uint32_t slept = 0; slept < interval && !g.stop.load(); slept += 10) usleep(10000);
    std::vector<Channel*> chs;
    {
      std::lock_guard<std::mutex> l(g.mu);
      for (auto& kv : g.channels) chs.push_back(kv.second);
    }
    for (Channel* ch : chs) {
      if (!ch->attached.load() || ch->lost.load()) continue;
      ctl_drain_notices(ch);
      bool lost = false;
      {
        std::lock_guard<std::mutex> l(ch->mu);
        channel_progress(ch);
        if (ch->ka_outstanding >= limit) {
          lost = true;
        } else {
          Head h{ch->proto.version, URPC_MSG_REQ, 1, URPC_FUNC_ID_KEEPALIVE, 0, ch->id, 0, 0};
          send_msg(ch->umqh, h, nullptr, 0, nullptr, 0, &ch->seal);
          ++ch->ka_outstanding;
          std::lock_guard<std::mutex> l2(g.stat_mu);
          stat_add(g.stats.keepalive_sent);
        }
      }
      if (lost) {
        ch->lost = true;
        stat_add(g.stats.keepalive_lost);
        g_log.log(ub::kLogWarn, "channel %u: peer missed %u keepalive probes, marked lost", ch->id, limit);
        push_event(URPC_EVENT_CHANNEL_LOST, ch->id, (int)limit);
        if (g.ka_cb) g.ka_cb(ch->id, 0, g.ka_ctx);
      }
    }
  }
}

// caller holds g.mu
Channel* get_channel_unlocked(uint32_t id) {
  auto it = g.channels.find(id);
  return it == g.channels.end() ? nullptr : it->second;
}
Channel* get_channel(uint32_t id) {
  std::lock_guard<std::mutex> l(g.mu);
  auto it = g.channels.find(id);
  return it == g.channels.end() ? nullptr : it->second;
}

}  // namespace

extern "C" {

int urpc_set_psk(const char* key_hex, const char* identity) {
  ub::PskConfig cfg;
  if (key_hex && *key_hex) {
    if (!ub::PskConfig::parse_hex(key_hex, &cfg.key) || cfg.key.size() < 16 || cfg.key.size() > 64) return URPC_ERR_EINVAL;
  }
  if (identity && *identity) cfg.identity = identity;
  std::lock_guard<std::mutex> l(g.mu);
  g.psk = cfg;
  g.psk_set = true;
  return URPC_SUCCESS;
}

int urpc_set_tls_files(const char* ca_file, const char* cert_file, const char* key_file) {
  const bool any = (ca_file && *ca_file) || (cert_file && *cert_file) || (key_file && *key_file);
  const bool all = ca_file && *ca_file && cert_file && *cert_file && key_file && *key_file;
  if (any && !all) return URPC_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g.mu);
  g.psk.ca_file = all ? ca_file : "";
  g.psk.cert_file = all ? cert_file : "";
  g.psk.key_file = all ? key_file : "";
  g.psk_set = true;
  return URPC_SUCCESS;
}

int urpc_init(const urpc_config_t* cfg) {
  std::lock_guard<std::mutex> l(g.mu);
  if (g.inited) return URPC_SUCCESS;
  if (cfg) g.cfg = *cfg;
  if (!g.cfg.default_timeout_ms) g.cfg.default_timeout_ms = 5000;
  umq_init_cfg_t uc{};
  uc.feature = UMQ_FEATURE_API_BASE | UMQ_FEATURE_STATS | UMQ_FEATURE_FLOW_CONTROL;
  uc.block_size_kb = 64;
  snprintf(uc.dev_name, sizeof(uc.dev_name), "%s", g.cfg.dev_name);
  if (umq_init(&uc) != UMQ_SUCCESS) return URPC_FAIL;
  g.stop = false;
  g.inited = true;
  if (g.cfg.keepalive_interval_ms) g.ka_thr = std::thread(keepalive_loop);
  if (const char* p = getenv("URPC_ADMIN_SOCKET")) urpc_admin_start(p);
  return URPC_SUCCESS;
}

void urpc_uninit(void) {
  {
    std::lock_guard<std::mutex> l(g.mu);
    if (!g.inited) return;
    g.stop = true;
  }
  if (g.accept_thr.joinable()) g.accept_thr.join();
  if (g.ka_thr.joinable()) g.ka_thr.join();
  engine_stop();
  urpc_admin_stop();
  std::lock_guard<std::mutex> l(g.mu);
  if (g.listen_fd >= 0) close(g.listen_fd);
  g.listen_fd = -1;
  for (auto& kv : g.channels) {
    kv.second->conn.reset();
    if (kv.second->tcp >= 0) close(kv.second->tcp);
    if (kv.second->umqh) umq_destroy(kv.second->umqh);
    delete kv.second;
  }
  g.channels.clear();
  for (Session* s : g.sessions) {
    s->conn.reset();
    if (s->tcp >= 0) close(s->tcp);
    if (s->umqh) umq_destroy(s->umqh);
    for (auto& ln : s->extra) umq_destroy(ln->umqh);
    delete s;
  }
  g.sessions.clear();
  g.funcs.clear();
  umq_uninit();
  g.inited = false;
}

int urpc_server_start(const char* ip, uint16_t port) {
  if (!g.inited) return URPC_FAIL;
  const int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return URPC_FAIL;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  a.sin_addr.s_addr = ip && *ip ? inet_addr(ip) : htonl(INADDR_LOOPBACK);
  if (bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || listen(fd, 64) != 0) {
    close(fd);
    return URPC_FAIL;
  }
  socklen_t len = sizeof(a);
  getsockname(fd, reinterpret_cast<sockaddr*>(&a), &len);
  g.server_psk = current_psk();
  g.listen_fd = fd;
  g.accept_thr = std::thread(accept_loop);
  return ntohs(a.sin_port);
}

// Tells every attached version-2 client that the function table changed. Caller holds g.mu.
static void notify_func_change(uint64_t func_id, uint32_t added) {
  uint8_t payload[12];
  memcpy(payload, &func_id, 8);
  memcpy(payload + 8, &added, 4);
  for (Session* s : g.sessions)
    if (s->proto.version >= 2 && !s->closed.load()) ctl_notice(s, urpc_proto::kCtlFuncChange, payload, sizeof(payload));
}
int urpc_func_register(uint64_t func_id, urpc_func_t fn, void* ctx) {
  if (!fn || func_id >= URPC_FUNC_ID_LOOKUP) return URPC_ERR_EINVAL;   // the two top ids are reserved
  std::lock_guard<std::mutex> l(g.mu);
  if (g.funcs.count(func_id)) return URPC_ERR_EINVAL;
  g.funcs[func_id] = Func{fn, ctx};
  notify_func_change(func_id, 1);
  return URPC_SUCCESS;
}
int urpc_func_unregister(uint64_t func_id) {
  std::lock_guard<std::mutex> l(g.mu);
  if (!g.funcs.erase(func_id)) return URPC_ERR_FUNC_NOT_FOUND;
  notify_func_change(func_id, 0);
  return URPC_SUCCESS;
}
int urpc_ctl_stats_get(urpc_ctl_stats_t* out) {
  if (!out) return URPC_ERR_EINVAL;
  {
    std::lock_guard<std::mutex> l(g_eng.st_mu);
    *out = g_eng.st;
  }
  out->tasks_live = g_eng.tasks.live();
  std::lock_guard<std::mutex> l(g_eng.mu);
  out->timers_armed = g_eng.wheel ? g_eng.wheel->armed_count() : 0;
  return URPC_SUCCESS;
}

int urpc_server_poll(urpc_poll_msg_t* msgs, int max) { return urpc_server_poll_shard(0, 1, msgs, max); }
int urpc_server_poll_shard(uint32_t shard, uint32_t nshards, urpc_poll_msg_t* msgs, int max) {
  if (nshards == 0 || shard >= nshards) return URPC_ERR_EINVAL;
  static thread_local std::vector<Session*> ss;
  ss.clear();
  {
    std::lock_guard<std::mutex> l(g.mu);
    for (Session* s : g.sessions)
      if (s->id % nshards == shard) ss.push_back(s);
  }
  int n = 0;
  static thread_local std::vector<uint8_t> rsp(64 * 1024);
  for (Session* s : ss) {
   // a session that is being retired, or a queue pair that is leaving, is not touched: the engine frees the queues
   // once `users` shows that no pass is inside
   struct Guard {
     std::atomic<int>* c;
     explicit Guard(std::atomic<int>* c_) : c(c_) { c->fetch_add(1); }
     ~Guard() { c->fetch_sub(1); }
   };
   Guard in_session(&s->users);
   if (s->closed.load()) continue;
   // (a poll pass allocates nothing: the list is a per-thread vector that keeps its storage, a guard lives on the
   // stack)
   static thread_local std::vector<LanePtr> lanes;
   lanes.clear();
   lanes.emplace_back();   // slot 0 stands for the first queue pair
   {
     std::lock_guard<std::mutex> l(s->lanes_mu);
     lanes.insert(lanes.end(), s->extra.begin(), s->extra.end());
   }
   for (size_t li = 0; li < lanes.size(); ++li) {   // every queue pair of the session in turn
    Lane* ln = lanes[li].get();
    std::optional<Guard> in_lane;
    if (ln) {
      in_lane.emplace(&ln->users);
      if (ln->closing.load()) continue;
    }
    const uint32_t lane = ln ? ln->id : 0;
    const uint64_t lq = ln ? ln->umqh : s->umqh;
    Sealer* lseal = ln ? &ln->seal : &s->seal;
    for (int budget = 0; budget < 64; ++budget) {
      umq_buf_t* b = umq_dequeue(lq);
      if (!b) break;
      Head h;
      if (b->data_size < sizeof(urpc_req_head_t) ||
          !urpc_proto::decode(reinterpret_cast<urpc_req_head_t*>(b->buf_data), &h) || h.type != URPC_MSG_REQ ||
          h.version != s->proto.version || !open_msg(b, lseal)) {
        if (b->data_size >= sizeof(urpc_req_head_t)) {  // a request that fails the seal check is dropped and counted
          std::lock_guard<std::mutex> l(g.stat_mu);
          stat_add(g.stats.errors);
        }
        umq_buf_free(b);
        continue;
      }
      const char* args = b->buf_data + sizeof(urpc_req_head_t);
      uint32_t alen = b->data_size - sizeof(urpc_req_head_t);
      uint32_t nrefs = 0;
      if (h.flags & kFlagRefs) {   // [inline args][reference table][count]: the handler sees the inline part only
        if (alen >= 4) memcpy(&nrefs, args + alen - 4, 4);
        if (nrefs == 0 || nrefs > URPC_MAX_REFS || alen < 4 + nrefs * sizeof(RefEntry)) {
          std::lock_guard<std::mutex> l(g.stat_mu);
          stat_add(g.stats.errors);
          umq_buf_free(b);
          continue;
        }
        alen -= 4 + nrefs * sizeof(RefEntry);
      }
      CurrentReq cur{lq, reinterpret_cast<const RefEntry*>(args + alen), nrefs};
      const uint8_t ver = s->proto.version;
      if (h.func_id == URPC_FUNC_ID_KEEPALIVE) {
        send_rsp(lq, lseal, ver, h, 0, nullptr, 0, false, true);
        umq_buf_free(b);
        continue;
      }
      if (h.func_id == URPC_FUNC_ID_LOOKUP) {   // name -> function id
        uint64_t id = 0;
        int lst = 0;
        {
          std::lock_guard<std::mutex> l(g.mu);
          auto it = g.func_names.find(std::string(args, strnlen(args, alen)));
          if (it != g.func_names.end()) id = it->second;
          else lst = URPC_ERR_FUNC_NOT_FOUND;
        }
        send_rsp(lq, lseal, ver, h, lst, &id, sizeof(id));
        umq_buf_free(b);
        continue;
      }
      Func f{nullptr, nullptr};
      {
        std::lock_guard<std::mutex> l(g.mu);
        auto it = g.funcs.find(h.func_id);
        if (it != g.funcs.end()) f = it->second;
      }
      stat_add(g.stats.requests_served);
      stat_add(g.stats.bytes_rx, alen);
      if (f.fn) {
        uint32_t rlen = static_cast<uint32_t>(rsp.size());
        const uint64_t e0 = ub::now_ns();
        t_current = &cur;   // urpc_ref_read(NULL, ...) inside the handler reads this request's references
        const int st = f.fn(args, alen, rsp.data(), &rlen, f.ctx);
        t_current = nullptr;
        const uint64_t e1 = ub::now_ns();
        record(URPC_PERF_FUNC_EXEC, e1 - e0);
        send_rsp(lq, lseal, ver, h, st, rsp.data(), rlen > rsp.size() ? 0 : rlen);
        record(URPC_PERF_FUNC_RETURN, ub::now_ns() - e1);
        umq_buf_free(b);
      } else if (msgs && n < max) {
        // the answer comes later, from the application: acknowledge now if the caller asked for it
        if ((h.flags & 1) && ver >= 2 && (s->proto.caps & urpc_proto::kCapAck)) send_ack(lq, lseal, ver, h);
        msgs[n].event = URPC_POLL_REQ;
        msgs[n].func_id = h.func_id;
        msgs[n].req_id = h.req_id;
        msgs[n].user_ctx = (uint64_t(s->id) << 32) | (uint64_t(lane) << 24) | (h.channel & 0xffffff);
        msgs[n].data = const_cast<char*>(args);
        msgs[n].len = alen;
        msgs[n].status = 0;
        msgs[n].priv = b;
        ++n;
      } else {
        send_rsp(lq, lseal, ver, h, URPC_ERR_FUNC_NOT_FOUND, nullptr, 0);
        umq_buf_free(b);
      }
    }
   }
   lanes.clear();   // the pass holds no lane beyond its own end
  }
  return n;
}

int urpc_func_return(const urpc_poll_msg_t* req, const void* rsp, uint32_t len, int status) {
  if (!req) return URPC_ERR_EINVAL;
  const uint32_t sid = static_cast<uint32_t>(req->user_ctx >> 32);
  Session* s = nullptr;
  {
    std::lock_guard<std::mutex> l(g.mu);
    if (sid < g.sessions.size()) s = g.sessions[sid];
  }
  if (!s) return URPC_ERR_EINVAL;
  {   // the client gave the call up (control message TASK_CANCEL): nothing is sent
    std::lock_guard<std::mutex> l(s->cancel_mu);
    if (s->cancelled.erase(req->req_id)) return URPC_ERR_CANCELED;
  }
  // the request's own head still sits in its buffer: its flags say whether an acknowledgement was asked for (and,
  // between version-2 peers, has been sent when the request was handed to the application)
  Head rq{};
  rq.func_id = req->func_id;
  rq.req_id = req->req_id;
  rq.channel = static_cast<uint32_t>(req->user_ctx & 0xffffff);
  if (req->priv) rq.flags = static_cast<uint8_t>(static_cast<umq_buf_t*>(req->priv)->buf_data[1]);
  const uint32_t lane = static_cast<uint32_t>(req->user_ctx >> 24) & 0xff;   // answer on the lane of the request
  LaneRef lr;
  if (!session_lane(s, lane, &lr)) return URPC_ERR_SESSION_CLOSE;
  const bool acked = (rq.flags & 1) && s->proto.version >= 2 && (s->proto.caps & urpc_proto::kCapAck);
  return send_rsp(lr.umqh, lr.seal, s->proto.version, rq, status, rsp, len, acked);
}

int urpc_channel_create(void) {
  if (!g.inited) return URPC_FAIL;
  Channel* ch = new Channel();
  ch->umqh = make_queue("urpc-cli");
  if (!ch->umqh) {
    delete ch;
    return URPC_FAIL;
  }
  std::lock_guard<std::mutex> l(g.mu);
  ch->id = g.next_ch++;
  g.channels[ch->id] = ch;
  return static_cast<int>(ch->id);
}

int urpc_channel_server_attach(uint32_t chid, const char* ip, uint16_t port) {
  Channel* ch = get_channel(chid);
  if (!ch || ch->attached.load()) return URPC_ERR_EINVAL;
  const int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return URPC_FAIL;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  a.sin_addr.s_addr = ip && *ip ? inet_addr(ip) : htonl(INADDR_LOOPBACK);
  if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
    close(fd);
    return URPC_FAIL;
  }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  std::string err;
  std::unique_ptr<ub::SecureConn> conn = ub::SecureConn::client(fd, current_psk(), 3000, &err);
  if (!conn) {
    close(fd);
    return URPC_FAIL;
  }
  Hello hello{};
  hello.magic = kHelloMagic;
  hello.version = my_version_word();
  hello.channel = chid;
  hello.blob_len = umq_bind_info_get(ch->umqh, hello.blob, sizeof(hello.blob));
  hello.n_extra = static_cast<uint32_t>(ch->extra.size());
  // every further queue of the channel travels with the hello, so the server publishes a complete session
  bool ok = conn->write_full(&hello, sizeof(hello));
  for (size_t i = 0; ok && i < ch->extra.size(); ++i) {
    LaneHello lh{};
    lh.blob_len = umq_bind_info_get(ch->extra[i]->umqh, lh.blob, sizeof(lh.blob));
    ok = conn->write_full(&lh, sizeof(lh));
  }
  Hello rsp;
  ok = ok && conn->read_full(&rsp, sizeof(rsp), 5000) && rsp.magic == kHelloMagic;
  // the answer names the version to use: one number from a version-1 server, version + capabilities otherwise;
  // it must lie inside what this side offered
  urpc_proto::Negotiated nego;
  if (ok) {
    nego.version = static_cast<uint8_t>(rsp.version & 0xff);
    nego.caps = (rsp.version >> 16) & (my_version_word() >> 16);
    const uint32_t mine = my_version_word();
    const uint8_t lo = (mine >> 8) & 0xff ? (mine >> 8) & 0xff : mine & 0xff;
    if (nego.version == 0 || nego.version > (mine & 0xff) || nego.version < lo) {
      g_log.log(ub::kLogWarn, "channel %u: no protocol version in common with the server", chid);
      conn.reset();
      close(fd);
      return URPC_ERR_VERSION;
    }
    if (nego.version < 2) nego.caps = 0;
  }
  ok = ok && !(conn->encrypted() && !rsp.sealed) && rsp.n_extra == hello.n_extra &&
       umq_bind(ch->umqh, rsp.blob, rsp.blob_len) == UMQ_SUCCESS;
  size_t bound = 0;
  for (; ok && bound < ch->extra.size(); ++bound) {
    LaneHello lr;
    ok = conn->read_full(&lr, sizeof(lr), 5000) && umq_bind(ch->extra[bound]->umqh, lr.blob, lr.blob_len) == UMQ_SUCCESS;
    if (!ok) break;
  }
  if (!ok) {
    for (size_t i = 0; i < bound; ++i) umq_unbind(ch->extra[i]->umqh);
    conn.reset();
    close(fd);
    return URPC_FAIL;
  }
  for (size_t lane = 0; lane <= ch->extra.size(); ++lane) {
    Sealer& sl = lane ? ch->extra[lane - 1]->seal : ch->seal;
    if (lane) {
      ch->extra[lane - 1]->id = static_cast<uint32_t>(lane);
      ch->extra[lane - 1]->closing = false;
    }
    std::lock_guard<std::mutex> l(sl.mu);
    if (rsp.sealed) sl.set(rsp.data_key, false, static_cast<uint32_t>(lane));
    else sl.clear();
  }
  ch->next_lane_id = static_cast<uint32_t>(ch->extra.size() + 1);
  ch->proto = nego;
  ch->sealed = rsp.sealed != 0;
  memcpy(ch->data_key, rsp.data_key, sizeof(ch->data_key));
  ch->rxbuf.clear();
  ch->conn = std::move(conn);
  ch->tcp = fd;
  ch->server_ip = ip && *ip ? ip : "127.0.0.1";
  ch->server_port = port;
  ch->lost = false;
  ch->attached = true;
  return URPC_SUCCESS;
}

int urpc_channel_server_detach(uint32_t chid) {
  Channel* ch = get_channel(chid);
  if (!ch || !ch->attached.load()) return URPC_ERR_EINVAL;
  // version 2: say goodbye, so that the server retires the session now (it would notice the closed connection
  // anyway, a little later); the answer is not needed to go on
  if (ch->proto.version >= 2 && !ch->lost.load()) ctl_call(ch, urpc_proto::kCtlDetach, nullptr, 0, nullptr, 500);
  std::lock_guard<std::mutex> l(ch->mu);
  ch->attached = false;
  ch->proto = urpc_proto::Negotiated();
  umq_unbind(ch->umqh);
  for (auto& ln : ch->extra) umq_unbind(ln->umqh);
  {
    std::lock_guard<std::mutex> cl(ch->ctl_mu);
    ch->conn.reset();
    if (ch->tcp >= 0) close(ch->tcp);
    ch->tcp = -1;
    ch->rxbuf.clear();
  }
  for (auto& kv : ch->pending)
    if (!kv.second.sync)
      ch->ready.push_back(Ready{URPC_POLL_ERR, kv.second.func_id, kv.second.user_ctx, kv.first,
                                URPC_ERR_SESSION_CLOSE, nullptr});
  ch->pending.clear();
  return URPC_SUCCESS;
}

int urpc_channel_destroy(uint32_t chid) {
  Channel* ch;
  {
    std::lock_guard<std::mutex> l(g.mu);
    auto it = g.channels.find(chid);
    if (it == g.channels.end()) return URPC_ERR_EINVAL;
    ch = it->second;
    g.channels.erase(it);
  }
  ch->conn.reset();
  if (ch->tcp >= 0) close(ch->tcp);
  for (auto& r : ch->ready)
    if (r.buf) umq_buf_free(r.buf);
  if (!ch->user_queue) umq_destroy(ch->umqh);   // a queue from urpc_queue_create stays with its creator
  delete ch;
  return URPC_SUCCESS;
}

int urpc_func_call(uint32_t chid, const urpc_call_wr_t* wr, const urpc_call_option_t* opt) {
  Channel* ch = get_channel(chid);
  if (!ch || !wr || wr->func_id >= URPC_FUNC_ID_KEEPALIVE) return URPC_ERR_EINVAL;
  if (wr->func_id == URPC_FUNC_ID_LOOKUP && !g_lookup_call) return URPC_ERR_EINVAL;
  if (!ch->attached.load() || ch->lost.load()) return URPC_ERR_SESSION_CLOSE;
  const uint32_t tmo = opt && opt->timeout_ms ? opt->timeout_ms : (ch->timeout_ms ? ch->timeout_ms : g.cfg.default_timeout_ms);
  uint32_t req_id;
  {
    std::lock_guard<std::mutex> l(ch->mu);
    req_id = ch->next_req++;
    Pending p;
    p.func_id = wr->func_id;
    p.user_ctx = wr->user_ctx;
    p.t0 = ub::now_ns();
    p.deadline = p.t0 + uint64_t(tmo) * 1000000ull;
    p.sync = opt && opt->sync;
    if (p.sync) {
      p.sync_buf = opt->rsp_buf;
      p.sync_cap = opt->rsp_buf ? opt->rsp_buf_len : 0;
    }
    // version 1 always set the bit (and nobody acted on it); version 2 sets it when the caller wants the event
    p.want_ack = opt && opt->want_ack && (ch->proto.caps & urpc_proto::kCapAck);
    const uint8_t ackbit = (ch->proto.version < 2 || p.want_ack) ? 1 : 0;
    Head h{ch->proto.version, URPC_MSG_REQ, static_cast<uint8_t>(ackbit | t_call_flags), wr->func_id, req_id, chid, 0, 0};
    // the queue the caller named (urpc_func_call_on), else the lanes in turn (one that is leaving takes no more)
    size_t lane = ch->extra.empty() ? 0 : ch->rr++ % (ch->extra.size() + 1);
    for (size_t tries = 0; lane && ch->extra[lane - 1]->closing.load() && tries <= ch->extra.size(); ++tries)
      lane = ch->rr++ % (ch->extra.size() + 1);
    if (lane && ch->extra[lane - 1]->closing.load()) lane = 0;
    if (t_call_queue) {
      lane = ch->extra.size() + 1;
      if (ch->umqh == t_call_queue) lane = 0;
      for (size_t i = 0; i < ch->extra.size(); ++i)
        if (ch->extra[i]->umqh == t_call_queue && !ch->extra[i]->closing.load()) lane = i + 1;
    }
    if (lane && lane <= ch->extra.size()) p.lane_id = ch->extra[lane - 1]->id;
    ch->pending[req_id] = std::move(p);
    const int rc = lane > ch->extra.size()
                       ? URPC_ERR_EINVAL
                       : send_msg(lane ? ch->extra[lane - 1]->umqh : ch->umqh, h, wr->args, wr->num_args, nullptr, 0,
                                  lane ? &ch->extra[lane - 1]->seal : &ch->seal);
    record(URPC_PERF_FUNC_CALL, ub::now_ns() - ch->pending[req_id].t0);
    if (rc != URPC_SUCCESS) {
      ch->pending.erase(req_id);
      stat_add(g.stats.errors);
      return rc;
    }
    stat_add(g.stats.calls);
  }
  if (!(opt && opt->sync)) return static_cast<int>(req_id);
  for (uint32_t spins = 0;; ++spins) {
    {
      std::lock_guard<std::mutex> l(ch->mu);
      channel_progress(ch);
      auto it = ch->pending.find(req_id);
      if (it == ch->pending.end()) return URPC_FAIL;
      if (it->second.done) {
        const int st = it->second.status;
        if (st == 0 && opt->rsp_len) *opt->rsp_len = it->second.rsp_len;   // (the bytes are in rsp_buf already)
        ch->pending.erase(it);
        return st;
      }
    }
    if (ch->lost.load()) {
      std::lock_guard<std::mutex> l(ch->mu);
      ch->pending.erase(req_id);
      return URPC_ERR_SESSION_CLOSE;
    }
    // an answer usually takes microseconds: poll tightly for that long before giving the core away between polls
    if (spins < 256) ub::cpu_relax();
    else sched_yield();
  }
}

int urpc_func_poll(uint32_t chid, urpc_poll_msg_t* msgs, int max) {
  Channel* ch = get_channel(chid);
  if (!ch || !msgs || max <= 0) return URPC_ERR_EINVAL;
  ctl_drain_notices(ch);
  std::lock_guard<std::mutex> l(ch->mu);
  if (ch->attached.load()) channel_progress(ch);
  int n = 0;
  while (n < max && !ch->ready.empty()) {
    Ready r = ch->ready.front();
    ch->ready.pop_front();
    msgs[n].event = r.ev;
    msgs[n].func_id = r.func_id;
    msgs[n].req_id = r.req_id;
    msgs[n].user_ctx = r.user_ctx;
    msgs[n].status = r.status;
    msgs[n].priv = r.buf;
    msgs[n].data = r.buf ? r.buf->buf_data + sizeof(urpc_req_head_t) : nullptr;
    msgs[n].len = r.buf ? r.buf->data_size - sizeof(urpc_req_head_t) : 0;
    if (urpc_func_poll_cb_t cb = g_poll_cb.load()) cb(chid, &msgs[n]);
    ++n;
  }
  return n;
}

void urpc_msg_release(urpc_poll_msg_t* msg) {
  if (msg && msg->priv) {
    umq_buf_free(static_cast<umq_buf_t*>(msg->priv));
    msg->priv = nullptr;
    msg->data = nullptr;
  }
}

int urpc_keepalive_callback_register(urpc_keepalive_cb_t cb, void* ctx) {
  g.ka_cb = cb;
  g.ka_ctx = ctx;
  return URPC_SUCCESS;
}

int urpc_channel_task_cancel(uint32_t chid, uint32_t req_id) {
  Channel* ch = get_channel(chid);
  if (!ch) return URPC_ERR_EINVAL;
  {
    std::lock_guard<std::mutex> l(ch->mu);
    if (!ch->pending.erase(req_id)) return URPC_ERR_EINVAL;
  }
  // the server drops its deferred copy too (when it knows how); a peer without the capability just answers late
  // and the answer is discarded here
  if (ch->attached.load() && (ch->proto.caps & urpc_proto::kCapTaskCancel))
    ctl_call(ch, urpc_proto::kCtlTaskCancel, &req_id, sizeof(req_id), nullptr, 1000);
  return URPC_SUCCESS;
}

// ---------------------------------------------------------------------------------------------- management socket
static std::string admin_report(const std::string& cmd) {
  char line[512];
  std::string r;
  if (cmd == "version") {
    r = "urpc 1.0 (umdk_b200), protocol versions " + std::to_string((int)urpc_proto::kVersionMin) + ".." +
        std::to_string((int)urpc_proto::kVersion) + "\n";
  } else if (cmd == "stats") {
    urpc_stats_t s{};
    urpc_stats_get(&s);
    snprintf(line, sizeof(line),
             "calls %llu\nresponses %llu\ntimeouts %llu\nerrors %llu\nrequests_served %llu\nkeepalive_sent %llu\n"
             "keepalive_lost %llu\nbytes_tx %llu\nbytes_rx %llu\n",
             (unsigned long long)s.calls, (unsigned long long)s.responses, (unsigned long long)s.timeouts,
             (unsigned long long)s.errors, (unsigned long long)s.requests_served, (unsigned long long)s.keepalive_sent,
             (unsigned long long)s.keepalive_lost, (unsigned long long)s.bytes_tx, (unsigned long long)s.bytes_rx);
    r = line;
  } else if (cmd == "perf") {
    uint64_t c = 0, avg = 0, p99 = 0;
    urpc_perf_get(&c, &avg, &p99);
    snprintf(line, sizeof(line), "call_to_response count %llu avg_ns %llu p99_ns %llu\n", (unsigned long long)c,
             (unsigned long long)avg, (unsigned long long)p99);
    r = line;
  } else if (cmd == "channels") {
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.channels) {
      Channel* ch = kv.second;
      std::lock_guard<std::mutex> cl(ch->mu);
      snprintf(line, sizeof(line), "channel %u attached %d lost %d pending %zu ready %zu next_req %u\n", ch->id,
               (int)ch->attached.load(), (int)ch->lost.load(), ch->pending.size(), ch->ready.size(), ch->next_req);
      r += line;
    }
    if (r.empty()) r = "(no channels)\n";
  } else if (cmd == "sessions") {
    std::lock_guard<std::mutex> l(g.mu);
    for (Session* s : g.sessions) {
      size_t lanes = 1;
      {
        std::lock_guard<std::mutex> ll(s->lanes_mu);
        lanes += s->extra.size();
      }
      snprintf(line, sizeof(line), "session %u tcp_fd %d queue %llx control %s payload %s proto %u caps 0x%x lanes %zu %s\n",
               s->id, s->tcp, (unsigned long long)s->umqh, s->conn ? s->conn->cipher() : "none",
               s->seal.on() ? "sealed" : "clear", s->proto.version, s->proto.caps, lanes,
               s->closed.load() ? "retired" : "live");
      r += line;
    }
    if (r.empty()) r = "(no sessions)\n";
  } else if (cmd == "tasks") {
    urpc_ctl_stats_t t{};
    urpc_ctl_stats_get(&t);
    snprintf(line, sizeof(line),
             "tasks_started %llu\ntasks_done %llu\ntasks_failed %llu\ntasks_timed_out %llu\nnotices_sent %llu\n"
             "sessions_retired %llu\ntasks_live %u\ntimers_armed %u\n",
             (unsigned long long)t.tasks_started, (unsigned long long)t.tasks_done, (unsigned long long)t.tasks_failed,
             (unsigned long long)t.tasks_timed_out, (unsigned long long)t.notices_sent,
             (unsigned long long)t.sessions_retired, t.tasks_live, t.timers_armed);
    r = line;
  } else if (cmd == "funcs") {
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.funcs) {
      snprintf(line, sizeof(line), "func 0x%llx\n", (unsigned long long)kv.first);
      r += line;
    }
    if (r.empty()) r = "(no functions)\n";
  } else {
    r = "unknown command; try: version stats perf channels sessions tasks funcs\n";
  }
  return r;
}

static void admin_loop() {
  while (!g.admin_stop.load()) {
    pollfd pf{g.admin_fd, POLLIN, 0};
    if (poll(&pf, 1, 100) <= 0) continue;
    const int c = accept(g.admin_fd, nullptr, nullptr);
    if (c < 0) continue;
    char buf[128] = {0};
    pollfd pc{c, POLLIN, 0};
    if (poll(&pc, 1, 1000) > 0) {
      const ssize_t n = read(c, buf, sizeof(buf) - 1);
      if (n > 0) {
        std::string cmd(buf, n);
        while (!cmd.empty() && (cmd.back() == '\n' || cmd.back() == '\r' || cmd.back() == ' ')) cmd.pop_back();
        const std::string rep = admin_report(cmd);
        write_full(c, rep.data(), rep.size());
      }
    }
    close(c);
  }
}

int urpc_admin_start(const char* path) {
  if (!path || !*path || strlen(path) >= sizeof(sockaddr_un::sun_path)) return URPC_ERR_EINVAL;
  if (g.admin_fd >= 0) return URPC_FAIL;
  const int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (fd < 0) return URPC_FAIL;
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  snprintf(a.sun_path, sizeof(a.sun_path), "%s", path);
  unlink(path);
  if (bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || listen(fd, 4) != 0) {
    close(fd);
    return URPC_FAIL;
  }
  g.admin_fd = fd;
  g.admin_path = path;
  g.admin_stop = false;
  g.admin_thr = std::thread(admin_loop);
  return URPC_SUCCESS;
}
void urpc_admin_stop(void) {
  if (g.admin_fd < 0) return;
  g.admin_stop = true;
  if (g.admin_thr.joinable()) g.admin_thr.join();
  close(g.admin_fd);
  g.admin_fd = -1;
  unlink(g.admin_path.c_str());
}
int urpc_admin_query(const char* command, char* out, uint32_t cap) {
  if (!command || !out || cap == 0) return URPC_ERR_EINVAL;
  const std::string rep = admin_report(command);
  const uint32_t n = std::min<uint32_t>(cap - 1, (uint32_t)rep.size());
  memcpy(out, rep.data(), n);
  out[n] = 0;
  return (int)n;
}

int urpc_stats_get(urpc_stats_t* out) {
  if (!out) return URPC_ERR_EINVAL;
  const uint64_t* src = reinterpret_cast<const uint64_t*>(&g.stats);
  uint64_t* dst = reinterpret_cast<uint64_t*>(out);
  static_assert(sizeof(urpc_stats_t) % sizeof(uint64_t) == 0, "urpc_stats_t is a row of 64-bit counters");
  for (size_t i = 0; i < sizeof(urpc_stats_t) / sizeof(uint64_t); ++i) dst[i] = __atomic_load_n(src + i, __ATOMIC_RELAXED);
  return URPC_SUCCESS;
}
uint64_t urpc_mem_seg_register(void* va, uint64_t len) {
  if (!va || !len) return 0;
  MemSeg m{va, len, 0, 0, {0}};
  ub::random_bytes(&m.token, sizeof(m.token));
  m.umq_h = umq_mem_seg_register(va, len, m.token, m.blob, sizeof(m.blob));
  if (!m.umq_h) return 0;
  std::lock_guard<std::mutex> l(g_mem_mu);
  const uint64_t h = g_mem_next++;
  g_mem[h] = m;
  return h;
}
int urpc_mem_seg_unregister(uint64_t mem_h) {
  std::lock_guard<std::mutex> l(g_mem_mu);
  auto it = g_mem.find(mem_h);
  if (it == g_mem.end()) return URPC_ERR_EINVAL;
  if (it->second.umq_h) umq_mem_seg_unregister(it->second.umq_h);
  g_mem.erase(it);
  return URPC_SUCCESS;
}
int urpc_mem_seg_token_get(uint64_t mem_h, uint32_t* token) {
  std::lock_guard<std::mutex> l(g_mem_mu);
  auto it = g_mem.find(mem_h);
  if (it == g_mem.end() || !token) return URPC_ERR_EINVAL;
  *token = it->second.token;
  return URPC_SUCCESS;
}
int urpc_mem_seg_remote_access_disable(uint64_t mem_h) {
  std::lock_guard<std::mutex> l(g_mem_mu);
  auto it = g_mem.find(mem_h);
  if (it == g_mem.end()) return URPC_ERR_EINVAL;
  if (it->second.umq_h) umq_mem_seg_unregister(it->second.umq_h);   // descriptions already sent stop working
  it->second.umq_h = 0;
  return URPC_SUCCESS;
}
int urpc_mem_seg_remote_access_enable(uint64_t mem_h) {
  std::lock_guard<std::mutex> l(g_mem_mu);
  auto it = g_mem.find(mem_h);
  if (it == g_mem.end()) return URPC_ERR_EINVAL;
  MemSeg& m = it->second;
  if (m.umq_h) return URPC_SUCCESS;
  ub::random_bytes(&m.token, sizeof(m.token));   // a fresh token: old descriptions stay dead
  m.umq_h = umq_mem_seg_register(m.va, m.len, m.token, m.blob, sizeof(m.blob));
  return m.umq_h ? URPC_SUCCESS : URPC_FAIL;
}
int urpc_func_call_ref(uint32_t chid, const urpc_call_wr_t* wr, const urpc_mem_ref_t* refs, uint32_t num_refs,
                       const urpc_call_option_t* opt) {
  if (!wr || !refs || num_refs == 0 || num_refs > URPC_MAX_REFS) return URPC_ERR_EINVAL;
  // the table rides behind the inline arguments as one more scatter element
  std::vector<uint8_t> table(num_refs * sizeof(RefEntry) + 4);
  {
    std::lock_guard<std::mutex> l(g_mem_mu);
    for (uint32_t i = 0; i < num_refs; ++i) {
      auto it = g_mem.find(refs[i].mem_h);
      if (it == g_mem.end() || !it->second.umq_h) return URPC_ERR_EINVAL;
      const MemSeg& m = it->second;
      const uint64_t base = reinterpret_cast<uint64_t>(m.va);
      if (refs[i].addr < base || refs[i].addr + refs[i].len > base + m.len) return URPC_ERR_EINVAL;
      RefEntry e{refs[i].addr, refs[i].len, m.token, {0}};
      memcpy(e.blob, m.blob, sizeof(e.blob));
      memcpy(table.data() + i * sizeof(RefEntry), &e, sizeof(e));
    }
  }
  memcpy(table.data() + num_refs * sizeof(RefEntry), &num_refs, 4);
  std::vector<urpc_sge_t> sg(wr->args, wr->args + wr->num_args);
  sg.push_back(urpc_sge_t{table.data(), static_cast<uint32_t>(table.size())});
  urpc_call_wr_t w2 = *wr;
  w2.args = sg.data();
  w2.num_args = static_cast<uint32_t>(sg.size());
  t_call_flags = kFlagRefs;
  const int rc = urpc_func_call(chid, &w2, opt);
  t_call_flags = 0;
  return rc;
}
static const CurrentReq* req_of(const urpc_poll_msg_t* req, CurrentReq* tmp) {
  if (!req) return t_current;
  // a request taken with urpc_server_poll: the table sits behind the inline arguments in the same buffer
  umq_buf_t* b = static_cast<umq_buf_t*>(req->priv);
  if (!b || req->event != URPC_POLL_REQ) return nullptr;
  Head h;
  if (!urpc_proto::decode(reinterpret_cast<urpc_req_head_t*>(b->buf_data), &h) || !(h.flags & kFlagRefs)) return nullptr;
  const char* args = b->buf_data + sizeof(urpc_req_head_t);
  const uint32_t all = b->data_size - sizeof(urpc_req_head_t);
  uint32_t n = 0;
  memcpy(&n, args + all - 4, 4);
  Session* s = nullptr;
  {
    std::lock_guard<std::mutex> l(g.mu);
    const uint32_t sid = static_cast<uint32_t>(req->user_ctx >> 32);
    if (sid < g.sessions.size()) s = g.sessions[sid];
  }
  const uint32_t lane = static_cast<uint32_t>(req->user_ctx >> 24) & 0xff;
  LaneRef lr;
  if (!s || n == 0 || n > URPC_MAX_REFS || !session_lane(s, lane, &lr)) return nullptr;
  *tmp = CurrentReq{lr.umqh, reinterpret_cast<const RefEntry*>(args + all - 4 - n * sizeof(RefEntry)), n};
  return tmp;
}
int urpc_ref_count(const urpc_poll_msg_t* req) {
  CurrentReq tmp;
  const CurrentReq* c = req_of(req, &tmp);
  return c ? static_cast<int>(c->nrefs) : 0;
}
int urpc_ref_len(const urpc_poll_msg_t* req, uint32_t idx, uint32_t* len) {
  CurrentReq tmp;
  const CurrentReq* c = req_of(req, &tmp);
  if (!c || idx >= c->nrefs || !len) return URPC_ERR_EINVAL;
  RefEntry e;
  memcpy(&e, &c->refs[idx], sizeof(e));
  *len = e.len;
  return URPC_SUCCESS;
}
int urpc_ref_read(const urpc_poll_msg_t* req, uint32_t idx, uint64_t offset, void* buf, uint32_t len) {
  CurrentReq tmp;
  const CurrentReq* c = req_of(req, &tmp);
  if (!c || idx >= c->nrefs || !buf || !len) return URPC_ERR_EINVAL;
  RefEntry e;
  memcpy(&e, &c->refs[idx], sizeof(e));
  if (offset + len > e.len) return URPC_ERR_EINVAL;
  const int rc = umq_remote_read(c->umqh, e.blob, e.token, e.addr + offset, buf, len, 3000);
  return rc == UMQ_SUCCESS ? URPC_SUCCESS : (rc == UMQ_ERR_EAGAIN ? URPC_ERR_TIMEOUT : URPC_FAIL);
}

int urpc_perf_recorder_unregister(void) {
  g_recorder = nullptr;
  g_recorder_ctx = nullptr;
  return URPC_SUCCESS;
}
int urpc_log_config_get(int* level) {
  if (!level) return URPC_ERR_EINVAL;
  *level = g_log.level();
  return URPC_SUCCESS;
}
uint32_t urpc_hdr_size_get(urpc_hdr_type_t type, uint16_t) {
  // requests, acknowledgements and responses share one fixed 32-byte header here; a sealed message adds a tag
  (void)type;
  return sizeof(urpc_req_head_t);
}
int urpc_ssl_config_set(const urpc_ssl_config_t* cfg) {
  if (!cfg) return URPC_ERR_EINVAL;
  return urpc_set_psk(cfg->enable ? cfg->psk_hex : "", cfg->psk_identity);
}
int urpc_func_name_register(uint64_t func_id, const char* name) {
  if (!name || !*name || func_id >= URPC_FUNC_ID_LOOKUP) return URPC_ERR_EINVAL;
  std::lock_guard<std::mutex> l(g.mu);
  if (!g.funcs.count(func_id)) return URPC_ERR_FUNC_NOT_FOUND;
  g.func_names[name] = func_id;
  return URPC_SUCCESS;
}
uint64_t urpc_func_id_get(uint32_t chid, const char* name) {
  if (!name || !*name) return 0;
  {   // a function of this process
    std::lock_guard<std::mutex> l(g.mu);
    auto it = g.func_names.find(name);
    if (it != g.func_names.end() && !get_channel_unlocked(chid)) return it->second;
  }
  uint64_t id = 0;
  uint32_t rlen = 0;
  urpc_sge_t sge{const_cast<char*>(name), static_cast<uint32_t>(strlen(name) + 1)};
  urpc_call_wr_t wr{URPC_FUNC_ID_LOOKUP, &sge, 1, 0};
  urpc_call_option_t opt{0, 1, &id, sizeof(id), &rlen};
  g_lookup_call = true;
  const int rc = urpc_func_call(chid, &wr, &opt);
  g_lookup_call = false;
  return rc == 0 && rlen == sizeof(id) ? id : 0;
}
// Runs a registered function in this process, without a channel: the same handler a remote caller would reach.
int urpc_func_exec(uint64_t func_id, urpc_sge_t* args, uint32_t num_args, void* rsp, uint32_t* rsp_len) {
  Func f{nullptr, nullptr};
  {
    std::lock_guard<std::mutex> l(g.mu);
    auto it = g.funcs.find(func_id);
    if (it != g.funcs.end()) f = it->second;
  }
  if (!f.fn) return URPC_ERR_FUNC_NOT_FOUND;
  if (!rsp || !rsp_len || (!args && num_args)) return URPC_ERR_EINVAL;
  std::vector<char> flat;
  for (uint32_t i = 0; i < num_args; ++i)
    flat.insert(flat.end(), static_cast<char*>(args[i].addr), static_cast<char*>(args[i].addr) + args[i].len);
  const uint64_t t0 = ub::now_ns();
  const int st = f.fn(flat.data(), static_cast<uint32_t>(flat.size()), rsp, rsp_len, f.ctx);
  record(URPC_PERF_FUNC_EXEC, ub::now_ns() - t0);
  return st;
}
// The same on a helper thread; `done(status, rsp, rsp_len, user_ctx)` runs there when the handler returns.
int urpc_func_async_exec(uint64_t func_id, urpc_sge_t* args, uint32_t num_args, urpc_async_exec_cb_t done,
                         void* user_ctx) {
  {
    std::lock_guard<std::mutex> l(g.mu);
    if (!g.funcs.count(func_id)) return URPC_ERR_FUNC_NOT_FOUND;
  }
  if (!done || (!args && num_args)) return URPC_ERR_EINVAL;
  std::vector<char> flat;
  for (uint32_t i = 0; i < num_args; ++i)
    flat.insert(flat.end(), static_cast<char*>(args[i].addr), static_cast<char*>(args[i].addr) + args[i].len);
  std::thread([func_id, flat, done, user_ctx]() mutable {
    std::vector<char> rsp(64 * 1024);
    uint32_t rlen = static_cast<uint32_t>(rsp.size());
    urpc_sge_t sge{flat.data(), static_cast<uint32_t>(flat.size())};
    const int st = urpc_func_exec(func_id, &sge, 1, rsp.data(), &rlen);
    done(st, rsp.data(), rlen, user_ctx);
  }).detach();
  return URPC_SUCCESS;
}
int urpc_func_poll_cb_register(urpc_func_poll_cb_t cb) {
  if (!cb) return URPC_ERR_EINVAL;
  g_poll_cb = cb;
  return URPC_SUCCESS;
}
int urpc_func_poll_cb_unregister(void) {
  g_poll_cb = nullptr;
  return URPC_SUCCESS;
}
int urpc_func_poll_wait(uint32_t chid, urpc_poll_msg_t* msgs, int max, int timeout_ms) {
  const uint64_t deadline = ub::now_ns() + uint64_t(timeout_ms < 0 ? 0 : timeout_ms) * 1000000ull;
  for (;;) {
    const int n = urpc_func_poll(chid, msgs, max);
    if (n != 0 || ub::now_ns() >= deadline) return n;
    usleep(50);
  }
}
int urpc_ctrl_msg_cb_register(urpc_ctrl_cb_t cb) {
  g_ctrl_cb = cb;
  return URPC_SUCCESS;
}
int urpc_async_event_get(urpc_async_event_t* events, int num) {
  if (!events || num <= 0) return URPC_ERR_EINVAL;
  {   // notices of the servers (function table changes) sit on the control connections until somebody reads them
    std::vector<Channel*> chs;
    {
      std::lock_guard<std::mutex> l(g.mu);
      for (auto& kv : g.channels) chs.push_back(kv.second);
    }
    for (Channel* ch : chs) ctl_drain_notices(ch);
  }
  std::lock_guard<std::mutex> l(g.stat_mu);
  int n = 0;
  while (n < num && !g.events.empty()) {
    events[n++] = g.events.front();
    g.events.pop_front();
  }
  if (g.events.empty() && g.event_fd >= 0) {
    uint64_t drained;
    if (read(g.event_fd, &drained, sizeof(drained)) < 0) {
      // nothing pending
    }
  }
  return n;
}
int urpc_async_event_fd_get(void) {
  std::lock_guard<std::mutex> l(g.stat_mu);
  if (g.event_fd < 0) g.event_fd = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  return g.event_fd;
}
int urpc_channel_cfg_get(uint32_t chid, urpc_channel_cfg_t* cfg) {
  Channel* ch = get_channel(chid);
  if (!ch || !cfg) return URPC_ERR_EINVAL;
  std::lock_guard<std::mutex> l(ch->mu);
  cfg->timeout_ms = ch->timeout_ms ? ch->timeout_ms : g.cfg.default_timeout_ms;
  cfg->attached = ch->attached.load();
  cfg->lost = ch->lost.load();
  cfg->sealed = ch->seal.on();
  cfg->proto_version = ch->attached.load() ? ch->proto.version : 0;
  cfg->proto_caps = ch->attached.load() ? ch->proto.caps : 0;
  cfg->pending_calls = static_cast<uint32_t>(ch->pending.size());
  snprintf(cfg->server_ip, sizeof(cfg->server_ip), "%s", ch->server_ip.c_str());
  cfg->server_port = ch->server_port;
  return URPC_SUCCESS;
}
int urpc_channel_cfg_set(uint32_t chid, const urpc_channel_cfg_t* cfg) {
  Channel* ch = get_channel(chid);
  if (!ch || !cfg) return URPC_ERR_EINVAL;
  std::lock_guard<std::mutex> l(ch->mu);
  ch->timeout_ms = cfg->timeout_ms;   // the only settable field; the rest of the structure reports state
  return URPC_SUCCESS;
}
int urpc_channel_server_refresh(uint32_t chid) {
  Channel* ch = get_channel(chid);
  if (!ch || ch->server_port == 0) return URPC_ERR_EINVAL;
  const std::string ip = ch->server_ip;
  const uint16_t port = ch->server_port;
  if (ch->attached.load()) urpc_channel_server_detach(chid);
  const int rc = urpc_channel_server_attach(chid, ip.c_str(), port);
  if (rc == URPC_SUCCESS) push_event(URPC_EVENT_CHANNEL_REFRESHED, chid, 0);
  return rc;
}
// A queue of a channel is its UMQ handle: the queue calls below take the handles urpc_channel_queue_query returns
// (lane order; at most `max` are written, the return value is the number the channel holds).
int urpc_channel_queue_query(uint32_t chid, uint64_t* qh, uint32_t max) {
  Channel* ch = get_channel(chid);
  if (!ch || !qh || max == 0) return URPC_ERR_EINVAL;
  std::lock_guard<std::mutex> l(ch->mu);
  qh[0] = ch->umqh;
  for (size_t i = 0; i < ch->extra.size() && i + 1 < max; ++i) qh[i + 1] = ch->extra[i]->umqh;
  return static_cast<int>(ch->extra.size() + 1);
}
// Explicit queues: created on their own, given to a channel before it attaches (the channel then uses it instead of
// the queue it made for itself), taken back after a detach.
static std::mutex g_q_mu;
static std::map<uint64_t, urpc_queue_cfg_t> g_user_queues;   // queues made by urpc_queue_create -> their cfg
uint64_t urpc_queue_create(const urpc_queue_cfg_t* cfg) {
  if (!g.inited) return 0;
  const uint64_t q = make_queue("urpc-user", cfg);
  if (!q) return 0;
  std::lock_guard<std::mutex> l(g_q_mu);
  g_user_queues[q] = cfg ? *cfg : urpc_queue_cfg_t{128, 128, 64 * 1024, 0};
  return q;
}
int urpc_queue_destroy(uint64_t qh) {
  {
    std::lock_guard<std::mutex> l(g_q_mu);
    if (!g_user_queues.erase(qh)) return URPC_ERR_EINVAL;
  }
  {   // a queue that a channel still uses cannot go away
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.channels)
      if (channel_lane(kv.second, qh) >= 0) {
        std::lock_guard<std::mutex> l2(g_q_mu);
        g_user_queues[qh] = urpc_queue_cfg_t{};
        return URPC_ERR_EAGAIN;
      }
  }
  return umq_destroy(qh) == UMQ_SUCCESS ? URPC_SUCCESS : URPC_FAIL;
}
int urpc_queue_cfg_get(uint64_t qh, urpc_queue_cfg_t* cfg) {
  umq_cfg_get_t c;
  if (!cfg || umq_cfg_get(qh, &c) != UMQ_SUCCESS) return URPC_ERR_EINVAL;
  cfg->rx_depth = c.create_option.rx_depth;
  cfg->tx_depth = c.create_option.tx_depth;
  cfg->rx_buf_size = c.create_option.rx_buf_size;
  cfg->interrupt = c.create_option.mode == UMQ_MODE_INTERRUPT;
  return URPC_SUCCESS;
}
int urpc_queue_cfg_set(uint64_t qh, const urpc_queue_cfg_t* cfg) {
  // depths and buffer size are fixed when the queue is created: only a matching configuration is accepted
  urpc_queue_cfg_t cur;
  if (!cfg || urpc_queue_cfg_get(qh, &cur) != URPC_SUCCESS) return URPC_ERR_EINVAL;
  return (cfg->rx_depth == cur.rx_depth && cfg->tx_depth == cur.tx_depth && cfg->rx_buf_size == cur.rx_buf_size)
             ? URPC_SUCCESS : URPC_ERR_EINVAL;
}
int urpc_queue_modify(uint64_t qh, urpc_queue_status_t status) {
  const umq_state_t st = status == URPC_QUEUE_READY ? UMQ_STATE_READY
                         : (status == URPC_QUEUE_IDLE ? UMQ_STATE_IDLE : UMQ_STATE_ERR);
  return umq_state_set(qh, st) == UMQ_SUCCESS ? URPC_SUCCESS : URPC_ERR_EINVAL;
}
int urpc_queue_rx_post(uint64_t qh, uint32_t) {
  // receive buffers are posted and re-posted by the queue itself; this runs its completion path, which does that
  umq_user_ctl_in_t in{UMQ_USER_CTL_PROGRESS, 0};
  umq_user_ctl_out_t out{};
  return umq_user_ctl(qh, &in, &out) == UMQ_SUCCESS ? URPC_SUCCESS : URPC_ERR_EINVAL;
}
int urpc_channel_queue_add(uint32_t chid, uint64_t qh) {
  Channel* ch = get_channel(chid);
  {
    std::lock_guard<std::mutex> l(g_q_mu);
    if (!g_user_queues.count(qh)) return URPC_ERR_EINVAL;
  }
  if (!ch) return URPC_ERR_EINVAL;
  {   // one queue serves one channel
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.channels)
      if (channel_lane(kv.second, qh) >= 0) return URPC_ERR_EINVAL;
  }
  if (ch->attached.load()) {
    // Live channel: pair the queue with a new server queue through the control connection, then let calls use it.
    // Needs a peer that negotiated version 2 with the capability; an older peer changes queues only while detached.
    if (!(ch->proto.caps & urpc_proto::kCapLiveQueues) || ch->lost.load()) return URPC_ERR_EINVAL;
    LanePtr ln(new Lane());
    {
      std::lock_guard<std::mutex> l(ch->mu);
      if (ch->extra.size() + 1 >= kMaxLanes || ch->next_lane_id > kMaxLaneId) return URPC_ERR_EINVAL;
      ln->id = ch->next_lane_id++;
    }
    ln->umqh = qh;
    std::vector<uint8_t> msg(8 + UMQ_BIND_INFO_SIZE), answer;
    const uint32_t blob_len = umq_bind_info_get(qh, msg.data() + 8, UMQ_BIND_INFO_SIZE);
    memcpy(msg.data(), &ln->id, 4);
    memcpy(msg.data() + 4, &blob_len, 4);
    const int rc = ctl_call(ch, urpc_proto::kCtlQueueAdd, msg.data(), 8 + blob_len, &answer, 3000);
    if (rc != URPC_SUCCESS) return rc;
    if (umq_bind(qh, answer.data(), static_cast<uint32_t>(answer.size())) != UMQ_SUCCESS) {
      ctl_call(ch, urpc_proto::kCtlQueueRm, &ln->id, 4, nullptr, 3000);   // undo the server half
      return URPC_FAIL;
    }
    if (ch->sealed) ln->seal.set(ch->data_key, false, ln->id);
    std::lock_guard<std::mutex> l(ch->mu);
    ch->extra.push_back(ln);
    return URPC_SUCCESS;
  }
  std::lock_guard<std::mutex> l(ch->mu);
  if (!ch->user_queue) {   // the first explicit queue takes the place of the one the channel made for itself
    umq_destroy(ch->umqh);
    ch->umqh = qh;
    ch->user_queue = true;
    return URPC_SUCCESS;
  }
  if (ch->extra.size() + 1 >= kMaxLanes) return URPC_ERR_EINVAL;
  ch->extra.emplace_back(new Lane());
  ch->extra.back()->umqh = qh;
  return URPC_SUCCESS;
}
int urpc_channel_queue_rm(uint32_t chid, uint64_t qh) {
  Channel* ch = get_channel(chid);
  if (!ch) return URPC_ERR_EINVAL;
  if (ch->attached.load()) {
    // Live channel: stop sending on the lane, wait for the calls in flight on it (their answers return on the same
    // lane), have the server retire its half, then unbind. The first queue pair carries the keepalive probes and
    // stays for the whole attach.
    if (!(ch->proto.caps & urpc_proto::kCapLiveQueues)) return URPC_ERR_EINVAL;
    LanePtr ln;
    {
      std::lock_guard<std::mutex> l(ch->mu);
      const int lane = channel_lane(ch, qh);
      if (lane <= 0) return URPC_ERR_EINVAL;
      ln = ch->extra[lane - 1];
      if (ln->closing.exchange(true)) return URPC_ERR_EINVAL;   // already leaving
    }
    const uint64_t deadline = now_ms() + (ch->timeout_ms ? ch->timeout_ms : g.cfg.default_timeout_ms) + 100;
    for (;;) {
      size_t inflight = 0;
      {
        std::lock_guard<std::mutex> l(ch->mu);
        channel_progress(ch);
        for (auto& kv : ch->pending) inflight += kv.second.lane_id == ln->id && !kv.second.done;
      }
      if (inflight == 0 || now_ms() > deadline || ch->lost.load()) break;
      usleep(200);
    }
    const int rc = ctl_call(ch, urpc_proto::kCtlQueueRm, &ln->id, 4, nullptr, 4000);
    std::lock_guard<std::mutex> l(ch->mu);
    umq_unbind(ln->umqh);
    ch->extra.erase(std::remove(ch->extra.begin(), ch->extra.end(), ln), ch->extra.end());
    return rc == URPC_ERR_SESSION_CLOSE ? URPC_SUCCESS : rc;   // a server that is gone has nothing left to retire
  }
  std::lock_guard<std::mutex> l(ch->mu);
  const int lane = channel_lane(ch, qh);
  if (lane < 0 || !ch->user_queue) return URPC_ERR_EINVAL;
  if (lane > 0) {
    ch->extra.erase(ch->extra.begin() + (lane - 1));
    return URPC_SUCCESS;
  }
  if (!ch->extra.empty()) {   // the next lane moves up
    ch->umqh = ch->extra.front()->umqh;
    ch->extra.erase(ch->extra.begin());
    return URPC_SUCCESS;
  }
  const uint64_t own = make_queue("urpc-cli");
  if (!own) return URPC_FAIL;
  ch->umqh = own;
  ch->user_queue = false;
  return URPC_SUCCESS;
}
// Pairing a local queue with the server's happens during attach; these report / undo it for one channel.
int urpc_channel_queue_pair(uint32_t chid, uint64_t local_qh) {
  Channel* ch = get_channel(chid);
  if (!ch || channel_lane(ch, local_qh) < 0) return URPC_ERR_EINVAL;
  return ch->attached.load() ? URPC_SUCCESS : URPC_ERR_SESSION_CLOSE;
}
int urpc_channel_queue_unpair(uint32_t chid, uint64_t local_qh) {
  Channel* ch = get_channel(chid);
  if (!ch || channel_lane(ch, local_qh) < 0) return URPC_ERR_EINVAL;
  return urpc_channel_server_detach(chid);
}
// urpc_func_call on one named queue of the channel instead of the lanes in turn.
int urpc_func_call_on(uint32_t chid, uint64_t qh, const urpc_call_wr_t* wr, const urpc_call_option_t* opt) {
  if (!qh) return URPC_ERR_EINVAL;
  t_call_queue = qh;
  const int rc = urpc_func_call(chid, wr, opt);
  t_call_queue = 0;
  return rc;
}
// Allocator plug-in for the copies the library makes of responses to synchronous calls.
static urpc_allocator_t g_alloc{};
int urpc_allocator_register(const urpc_allocator_t* a) {
  if (!a || !a->alloc || !a->free) return URPC_ERR_EINVAL;
  g_alloc = *a;
  return URPC_SUCCESS;
}
int urpc_allocator_unregister(void) {
  g_alloc = urpc_allocator_t{};
  return URPC_SUCCESS;
}
void* urpc_rsp_copy(const void* data, uint32_t len) {
  void* p = g_alloc.alloc ? g_alloc.alloc(len ? len : 1) : malloc(len ? len : 1);
  if (p && len) memcpy(p, data, len);
  return p;
}
void urpc_rsp_free(void* p) {
  if (g_alloc.free) g_alloc.free(p);
  else free(p);
}

int urpc_queue_status_query(uint64_t qh, urpc_queue_status_t* status) {
  if (!status) return URPC_ERR_EINVAL;
  const umq_state_t st = umq_state_get(qh);
  *status = st == UMQ_STATE_READY ? URPC_QUEUE_READY : (st == UMQ_STATE_IDLE ? URPC_QUEUE_IDLE : URPC_QUEUE_ERROR);
  return URPC_SUCCESS;
}
int urpc_queue_interrupt_fd_get(uint64_t qh) { return umq_interrupt_fd_get(qh); }
static const char* const kQueueStatNames[] = {"tx_msgs", "tx_bytes", "rx_msgs", "rx_bytes"};
static const char* const kQueueErrNames[] = {"tx_errors", "rx_errors", "tx_eagain"};
int urpc_queue_stats_get(uint64_t qh, uint64_t* stats, int len) {
  umq_io_stats_t io;
  if (!stats || len < 4 || umq_stats_io_get(qh, &io) != UMQ_SUCCESS) return URPC_ERR_EINVAL;
  stats[0] = io.tx_msgs;
  stats[1] = io.tx_bytes;
  stats[2] = io.rx_msgs;
  stats[3] = io.rx_bytes;
  return 4;
}
const char* urpc_queue_stats_name_get(int type) { return type >= 0 && type < 4 ? kQueueStatNames[type] : nullptr; }
int urpc_queue_error_stats_get(uint64_t qh, uint64_t* stats, int len) {
  umq_io_stats_t io;
  if (!stats || len < 3 || umq_stats_io_get(qh, &io) != UMQ_SUCCESS) return URPC_ERR_EINVAL;
  stats[0] = io.tx_errors;
  stats[1] = io.rx_errors;
  stats[2] = io.tx_eagain;
  return 3;
}
const char* urpc_queue_error_stats_name_get(int type) { return type >= 0 && type < 3 ? kQueueErrNames[type] : nullptr; }
int urpc_error_stats_get(uint64_t* stats, int len) {
  if (!stats || len < 3) return URPC_ERR_EINVAL;
  stats[0] = __atomic_load_n(&g.stats.errors, __ATOMIC_RELAXED);
  stats[1] = __atomic_load_n(&g.stats.timeouts, __ATOMIC_RELAXED);
  stats[2] = __atomic_load_n(&g.stats.keepalive_lost, __ATOMIC_RELAXED);
  return 3;
}

int urpc_perf_recorder_register(urpc_perf_recorder_t cb, void* ctx) {
  g_recorder_ctx = ctx;
  g_recorder = cb;
  return URPC_SUCCESS;
}
int urpc_log_config_set(int level, urpc_log_cb_t cb) {
  if (level < 0 || level > 4) return URPC_ERR_EINVAL;
  g_log.configure(level, cb);
  return URPC_SUCCESS;
}
int urpc_perf_get(uint64_t* count, uint64_t* avg_ns, uint64_t* p99_ns) {
  std::lock_guard<std::mutex> l(g.lat_mu);
  if (count) *count = g.lat.count();
  if (avg_ns) *avg_ns = static_cast<uint64_t>(g.lat.mean());
  if (p99_ns) *p99_ns = g.lat.quantile(0.99);
  return URPC_SUCCESS;
}

}  // extern "C"

// Self-checks of the header-only units (timer wheel, slab, id generator) and of the head codecs / negotiation.
// 0 = all passed, else the source line of the first check that failed. Exported for the test-suite.
extern "C" URPC_EXPORT int urpc_units_selftest(void) {
#define UNIT_CHECK(c) \
  do {                \
    if (!(c)) return __LINE__; \
  } while (0)
  {   // id generator: lowest free after the last one, no reuse at once, double free reported
    urpc_util::IdGen ids(10, 4);
    uint32_t a, b, c, d, e;
    UNIT_CHECK(ids.alloc(&a) && ids.alloc(&b) && ids.alloc(&c) && ids.alloc(&d));
    UNIT_CHECK(a == 10 && b == 11 && c == 12 && d == 13 && !ids.alloc(&e) && ids.in_use() == 4);
    UNIT_CHECK(ids.free(11) && !ids.free(11) && !ids.free(99) && ids.in_use() == 3);
    UNIT_CHECK(ids.alloc(&e) && e == 11);
    UNIT_CHECK(ids.free(10) && ids.free(12) && ids.alloc(&e) && e == 12);   // hint moved past 11
  }
  {   // slab: stable pointers, stale handles do not resolve, growth by chunks
    urpc_util::Slab<std::vector<int>> slab(2);
    std::vector<int>* p1 = nullptr;
    std::vector<int>* p2 = nullptr;
    std::vector<int>* p3 = nullptr;
    const uint64_t h1 = slab.acquire(&p1), h2 = slab.acquire(&p2), h3 = slab.acquire(&p3);
    p1->assign(3, 7);
    UNIT_CHECK(slab.live() == 3 && slab.capacity() == 4 && slab.get(h1) == p1 && slab.get(h2) == p2);
    UNIT_CHECK(slab.release(h2) && !slab.release(h2) && slab.get(h2) == nullptr && slab.live() == 2);
    std::vector<int>* p4 = nullptr;
    const uint64_t h4 = slab.acquire(&p4);
    UNIT_CHECK(p4 == p2 && h4 != h2 && slab.get(h2) == nullptr && slab.get(h4) == p4 && p4->empty());
    UNIT_CHECK(slab.get(h1)->size() == 3 && slab.get(h3) == p3);
  }
  {   // timer wheel: one-shot order, periodic re-arm, restart, stop, far wheel (beyond one turn of 256 ticks)
    urpc_util::TimerWheel w(10, 1000);
    std::vector<int> fired;
    const uint32_t t1 = w.create([&] { fired.push_back(1); });
    const uint32_t t2 = w.create([&] { fired.push_back(2); });
    const uint32_t t3 = w.create([&] { fired.push_back(3); });
    const uint32_t t4 = w.create([&] { fired.push_back(4); });
    UNIT_CHECK(w.start(t1, 30) && w.start(t2, 20) && w.start(t3, 5000) && w.start(t4, 25, true));
    UNIT_CHECK(w.run(1010) == 0 && fired.empty());
    UNIT_CHECK(w.run(1030) == 3 && fired == (std::vector<int>{2, 1, 4}));   // t4 rounds 25 ms up to 3 ticks
    UNIT_CHECK(w.armed(t4) && !w.armed(t1) && w.armed_count() == 2);
    UNIT_CHECK(w.run(1060) == 1 && fired.back() == 4);                       // periodic: again after 3 ticks
    UNIT_CHECK(w.stop(t4) && !w.stop(t4));
    UNIT_CHECK(w.start(t1, 40) && w.start(t1, 100));                         // restart moves it
    UNIT_CHECK(w.run(1120) == 0 && w.run(1160) == 1 && fired.back() == 1);
    UNIT_CHECK(w.run(5990) == 0 && w.run(6000) == 1 && fired.back() == 3);   // 500 ticks away: far wheel
    UNIT_CHECK(w.destroy(t2) && !w.start(t2, 10));
    const uint32_t t5 = w.create([&] { fired.push_back(5); });
    UNIT_CHECK(t5 == t2);                                                    // slot reused
    UNIT_CHECK(w.start(t5, 256 * 10 * 300) && w.armed(t5));                  // more than one turn of the far wheel
    UNIT_CHECK(w.run(6000 + 256 * 10 * 299) == 0 && w.run(6000 + 256 * 10 * 300) == 1 && fired.back() == 5);
  }
  {   // heads: every layout survives its codec, and the kinds do not decode as one another
    urpc_req_head_t raw;
    urpc_proto::AckHead a{2, 3, 0x01020304, 0xabcdef}, a2{};
    urpc_proto::encode_ack(a, &raw);
    UNIT_CHECK(urpc_proto::decode_ack(&raw, &a2) && a2.version == 2 && a2.req_id_range == 3 &&
               a2.req_id == 0x01020304 && a2.channel == 0xabcdef);
    urpc_proto::RspHead r{2, URPC_MSG_ACK_AND_RSP, 0x20, 1, 0xdeadbeef, 77, 0x123456, 4096, -38}, r2{};
    UNIT_CHECK(!urpc_proto::decode_rsp(&raw, &r2));   // an ACK is not a response
    urpc_proto::encode_rsp(r, &raw);
    UNIT_CHECK(urpc_proto::decode_rsp(&raw, &r2) && r2.type == URPC_MSG_ACK_AND_RSP && r2.flags == 0x20 &&
               r2.function_defined == 0xdeadbeef && r2.req_id == 77 && r2.channel == 0x123456 &&
               r2.total_size == 4096 && r2.status == -38 && r2.req_id_range == 1);
    UNIT_CHECK(!urpc_proto::decode_ack(&raw, &a2));
    Head h{2, URPC_MSG_REQ, 1, 0x0000123456789abcull, 9, 5, 100, 0}, h2{};
    urpc_proto::encode(h, &raw);
    UNIT_CHECK(urpc_proto::decode(&raw, &h2) && h2.func_id == 0x123456789abcull && h2.req_id == 9 && h2.version == 2);
    raw.bytes[0] = static_cast<uint8_t>((9 << 4) | URPC_MSG_REQ);
    UNIT_CHECK(!urpc_proto::decode(&raw, &h2));       // a version nobody speaks
  }
  {   // negotiation: newest common version, capabilities only from version 2 on, old peers send the plain number
    using urpc_proto::negotiate;
    using urpc_proto::pack_version;
    const uint32_t v2 = pack_version(2, 1, urpc_proto::kCapsAll);
    UNIT_CHECK(negotiate(v2, v2).version == 2 && negotiate(v2, v2).caps == urpc_proto::kCapsAll);
    UNIT_CHECK(negotiate(v2, 1).version == 1 && negotiate(v2, 1).caps == 0);
    UNIT_CHECK(negotiate(1, v2).version == 1);
    UNIT_CHECK(negotiate(pack_version(2, 2, urpc_proto::kCapsAll), 1).version == 0);   // needs 2, peer only 1
    UNIT_CHECK(negotiate(pack_version(3, 2, 0xffff), pack_version(2, 1, urpc_proto::kCapAck)).version == 2);
    UNIT_CHECK(negotiate(pack_version(3, 2, 0xffff), pack_version(2, 1, urpc_proto::kCapAck)).caps == urpc_proto::kCapAck);
    UNIT_CHECK(negotiate(pack_version(3, 3, 0), v2).version == 0);
  }
#undef UNIT_CHECK
  return 0;
}
