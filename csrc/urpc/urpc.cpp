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
#include <string>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

#include "ub_secure.h"
#include "ub_util.h"
#include "umq_api.h"
#include "urpc_proto.h"

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
  bool sync = false;
  bool done = false;
  int status = 0;
  std::vector<uint8_t> rsp;
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
  uint64_t umqh = 0;
  Sealer seal;
};
constexpr uint32_t kMaxLanes = 16;

struct Channel {
  uint32_t id;
  uint64_t umqh = 0;
  std::vector<std::unique_ptr<Lane>> extra;   // lanes 1..n
  uint32_t rr = 0;                            // round-robin cursor of urpc_func_call over the lanes
  int tcp = -1;
  std::unique_ptr<ub::SecureConn> conn;
  Sealer seal;
  std::atomic<bool> attached{false};
  std::atomic<bool> lost{false};
  std::mutex mu;
  std::unordered_map<uint32_t, Pending> pending;
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
  std::vector<std::unique_ptr<Lane>> extra;   // fixed before the session is published
  int tcp;
  uint32_t id;
  std::unique_ptr<ub::SecureConn> conn;
  Sealer seal;
};
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

int send_msg(uint64_t umqh, const Head& h, const urpc_sge_t* sg, uint32_t nsg, const void* flat, uint32_t flat_len,
             Sealer* seal = nullptr) {
  uint32_t total = flat_len;
  for (uint32_t i = 0; i < nsg; ++i) total += sg[i].len;
  const bool sealed = seal && seal->on();
  const uint32_t tag = sealed ? (uint32_t)ub::AeadCipher::kTagBytes : 0u;
  umq_buf_t* b = umq_buf_alloc(sizeof(urpc_req_head_t) + total + tag, 1, umqh);
  if (!b) return URPC_ERR_EAGAIN;
  Head hh = h;
  hh.total_size = total;
  if (sealed) hh.flags |= kFlagSealed;
  urpc_proto::encode(hh, reinterpret_cast<urpc_req_head_t*>(b->buf_data));
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
  std::lock_guard<std::mutex> l(g.stat_mu);
  g.stats.bytes_tx += total;
  return URPC_SUCCESS;
}

// Checks and removes the seal of a received message in place. False = drop it: sealed without a key, clear although a
// key is set, replayed counter, or bad tag.
bool open_msg(umq_buf_t* b, const Head& h, Sealer* seal) {
  const bool sealed = (h.flags & kFlagSealed) != 0;
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
    Head h;
    if (b->data_size < sizeof(urpc_req_head_t) ||
        !urpc_proto::decode(reinterpret_cast<urpc_req_head_t*>(b->buf_data), &h) ||
        (h.type != URPC_MSG_RSP && h.type != URPC_MSG_ACK_AND_RSP) || !open_msg(b, h, seal)) {
      if (b->data_size >= sizeof(urpc_req_head_t)) {
        std::lock_guard<std::mutex> l(g.stat_mu);
        ++g.stats.errors;
      }
      umq_buf_free(b);
      continue;
    }
    {
      std::lock_guard<std::mutex> l(g.stat_mu);
      g.stats.bytes_rx += h.total_size;
    }
    if (h.func_id == URPC_FUNC_ID_KEEPALIVE) {
      ch->ka_outstanding = 0;
      umq_buf_free(b);
      continue;
    }
    auto it = ch->pending.find(h.req_id);
    if (it == ch->pending.end()) {  // late answer of a call that already timed out or was cancelled
      umq_buf_free(b);
      continue;
    }
    Pending& p = it->second;
    {
      std::lock_guard<std::mutex> l(g.stat_mu);
      ++g.stats.responses;
      g.lat.add(ub::now_ns() - p.t0);
      record(URPC_PERF_CALL_TO_RESPONSE, ub::now_ns() - p.t0);
    }
    if (p.sync) {
      p.rsp.assign(b->buf_data + sizeof(urpc_req_head_t), b->buf_data + b->data_size);
      p.status = h.status;
      p.done = true;
      umq_buf_free(b);
    } else {
      ch->ready.push_back(Ready{URPC_POLL_RSP, p.func_id, p.user_ctx, h.req_id, h.status, b});
      ch->pending.erase(it);
    }
  }
  const uint64_t now = ub::now_ns();
  for (auto it = ch->pending.begin(); it != ch->pending.end();) {
    Pending& p = it->second;
    if (!p.done && now > p.deadline) {
      {
        std::lock_guard<std::mutex> l(g.stat_mu);
        ++g.stats.timeouts;
      }
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
      ++g.stats.errors;
      close(fd);
      continue;
    }
    if (!conn->read_full(&hello, sizeof(hello), 5000) || hello.magic != kHelloMagic ||
        hello.version != urpc_proto::kVersion) {
      conn.reset();
      close(fd);
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
    rsp.version = urpc_proto::kVersion;
    rsp.n_extra = static_cast<uint32_t>(lane_req.size());
    Session* s = new Session();
    ok = ok && q && umq_bind(q, hello.blob, hello.blob_len) == UMQ_SUCCESS;
    for (size_t i = 0; ok && i < lane_req.size(); ++i) {
      const uint64_t lq = make_queue("urpc-srv");
      if (!lq) {
        ok = false;
        break;
      }
      s->extra.emplace_back(new Lane());
      s->extra.back()->umqh = lq;
      ok = umq_bind(lq, lane_req[i].blob, lane_req[i].blob_len) == UMQ_SUCCESS;
      lane_rsp[i].blob_len = umq_bind_info_get(lq, lane_rsp[i].blob, sizeof(lane_rsp[i].blob));
    }
    if (ok && conn->encrypted()) {
      ok = ub::random_bytes(rsp.data_key, sizeof(rsp.data_key));
      if (ok) {
        rsp.sealed = 1;
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
    // a client that went away during the handshake leaves a session that never receives a request
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
      bool lost = false;
      {
        std::lock_guard<std::mutex> l(ch->mu);
        channel_progress(ch);
        if (ch->ka_outstanding >= limit) {
          lost = true;
        } else {
          Head h{urpc_proto::kVersion, URPC_MSG_REQ, 1, URPC_FUNC_ID_KEEPALIVE, 0, ch->id, 0, 0};
          send_msg(ch->umqh, h, nullptr, 0, nullptr, 0, &ch->seal);
          ++ch->ka_outstanding;
          std::lock_guard<std::mutex> l2(g.stat_mu);
          ++g.stats.keepalive_sent;
        }
      }
      if (lost) {
        ch->lost = true;
        {
          std::lock_guard<std::mutex> l(g.stat_mu);
          ++g.stats.keepalive_lost;
        }
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
    umq_destroy(s->umqh);
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

int urpc_func_register(uint64_t func_id, urpc_func_t fn, void* ctx) {
  if (!fn || func_id >= URPC_FUNC_ID_LOOKUP) return URPC_ERR_EINVAL;   // the two top ids are reserved
  std::lock_guard<std::mutex> l(g.mu);
  if (g.funcs.count(func_id)) return URPC_ERR_EINVAL;
  g.funcs[func_id] = Func{fn, ctx};
  return URPC_SUCCESS;
}
int urpc_func_unregister(uint64_t func_id) {
  std::lock_guard<std::mutex> l(g.mu);
  return g.funcs.erase(func_id) ? URPC_SUCCESS : URPC_ERR_FUNC_NOT_FOUND;
}

int urpc_server_poll(urpc_poll_msg_t* msgs, int max) {
  std::vector<Session*> ss;
  {
    std::lock_guard<std::mutex> l(g.mu);
    ss = g.sessions;
  }
  int n = 0;
  static thread_local std::vector<uint8_t> rsp(64 * 1024);
  for (Session* s : ss)
   for (size_t lane = 0; lane <= s->extra.size(); ++lane) {   // every queue pair of the session in turn
    const uint64_t lq = lane ? s->extra[lane - 1]->umqh : s->umqh;
    Sealer* lseal = lane ? &s->extra[lane - 1]->seal : &s->seal;
    for (int budget = 0; budget < 64; ++budget) {
      umq_buf_t* b = umq_dequeue(lq);
      if (!b) break;
      Head h;
      if (b->data_size < sizeof(urpc_req_head_t) ||
          !urpc_proto::decode(reinterpret_cast<urpc_req_head_t*>(b->buf_data), &h) || h.type != URPC_MSG_REQ ||
          !open_msg(b, h, lseal)) {
        if (b->data_size >= sizeof(urpc_req_head_t)) {  // a request that fails the seal check is dropped and counted
          std::lock_guard<std::mutex> l(g.stat_mu);
          ++g.stats.errors;
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
          ++g.stats.errors;
          umq_buf_free(b);
          continue;
        }
        alen -= 4 + nrefs * sizeof(RefEntry);
      }
      CurrentReq cur{lq, reinterpret_cast<const RefEntry*>(args + alen), nrefs};
      Head rh{urpc_proto::kVersion, URPC_MSG_RSP, 0, h.func_id, h.req_id, h.channel, 0, 0};
      if (h.func_id == URPC_FUNC_ID_KEEPALIVE) {
        send_msg(lq, rh, nullptr, 0, nullptr, 0, lseal);
        umq_buf_free(b);
        continue;
      }
      if (h.func_id == URPC_FUNC_ID_LOOKUP) {   // name -> function id
        uint64_t id = 0;
        {
          std::lock_guard<std::mutex> l(g.mu);
          auto it = g.func_names.find(std::string(args, strnlen(args, alen)));
          if (it != g.func_names.end()) id = it->second;
          else rh.status = static_cast<int8_t>(URPC_ERR_FUNC_NOT_FOUND);
        }
        send_msg(lq, rh, nullptr, 0, &id, sizeof(id), lseal);
        umq_buf_free(b);
        continue;
      }
      Func f{nullptr, nullptr};
      {
        std::lock_guard<std::mutex> l(g.mu);
        auto it = g.funcs.find(h.func_id);
        if (it != g.funcs.end()) f = it->second;
      }
      {
        std::lock_guard<std::mutex> l(g.stat_mu);
        ++g.stats.requests_served;
        g.stats.bytes_rx += alen;
      }
      if (f.fn) {
        uint32_t rlen = static_cast<uint32_t>(rsp.size());
        const uint64_t e0 = ub::now_ns();
        t_current = &cur;   // urpc_ref_read(NULL, ...) inside the handler reads this request's references
        const int st = f.fn(args, alen, rsp.data(), &rlen, f.ctx);
        t_current = nullptr;
        const uint64_t e1 = ub::now_ns();
        record(URPC_PERF_FUNC_EXEC, e1 - e0);
        rh.status = static_cast<int8_t>(st);
        send_msg(lq, rh, nullptr, 0, rsp.data(), rlen > rsp.size() ? 0 : rlen, lseal);
        record(URPC_PERF_FUNC_RETURN, ub::now_ns() - e1);
        umq_buf_free(b);
      } else if (msgs && n < max) {
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
        rh.status = static_cast<int8_t>(URPC_ERR_FUNC_NOT_FOUND);
        send_msg(lq, rh, nullptr, 0, nullptr, 0, lseal);
        umq_buf_free(b);
      }
    }
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
  Head rh{urpc_proto::kVersion, URPC_MSG_RSP, 0, req->func_id, req->req_id,
          static_cast<uint32_t>(req->user_ctx & 0xffffff), 0, static_cast<int8_t>(status)};
  const uint32_t lane = static_cast<uint32_t>(req->user_ctx >> 24) & 0xff;   // answer on the lane of the request
  if (lane > s->extra.size()) return URPC_ERR_EINVAL;
  return send_msg(lane ? s->extra[lane - 1]->umqh : s->umqh, rh, nullptr, 0, rsp, len,
                  lane ? &s->extra[lane - 1]->seal : &s->seal);
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
  hello.version = urpc_proto::kVersion;
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
  ok = ok && conn->read_full(&rsp, sizeof(rsp), 5000) && rsp.magic == kHelloMagic &&
       !(conn->encrypted() && !rsp.sealed) && rsp.n_extra == hello.n_extra &&
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
    std::lock_guard<std::mutex> l(sl.mu);
    if (rsp.sealed) sl.set(rsp.data_key, false, static_cast<uint32_t>(lane));
    else sl.clear();
  }
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
  std::lock_guard<std::mutex> l(ch->mu);
  ch->attached = false;
  umq_unbind(ch->umqh);
  for (auto& ln : ch->extra) umq_unbind(ln->umqh);
  ch->conn.reset();
  if (ch->tcp >= 0) close(ch->tcp);
  ch->tcp = -1;
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
    ch->pending[req_id] = std::move(p);
    Head h{urpc_proto::kVersion, URPC_MSG_REQ, static_cast<uint8_t>(1 | t_call_flags), wr->func_id, req_id, chid, 0, 0};
    // the queue the caller named (urpc_func_call_on), else the lanes in turn
    size_t lane = ch->extra.empty() ? 0 : ch->rr++ % (ch->extra.size() + 1);
    if (t_call_queue) {
      lane = ch->extra.size() + 1;
      if (ch->umqh == t_call_queue) lane = 0;
      for (size_t i = 0; i < ch->extra.size(); ++i)
        if (ch->extra[i]->umqh == t_call_queue) lane = i + 1;
    }
    const int rc = lane > ch->extra.size()
                       ? URPC_ERR_EINVAL
                       : send_msg(lane ? ch->extra[lane - 1]->umqh : ch->umqh, h, wr->args, wr->num_args, nullptr, 0,
                                  lane ? &ch->extra[lane - 1]->seal : &ch->seal);
    record(URPC_PERF_FUNC_CALL, ub::now_ns() - ch->pending[req_id].t0);
    if (rc != URPC_SUCCESS) {
      ch->pending.erase(req_id);
      std::lock_guard<std::mutex> l2(g.stat_mu);
      ++g.stats.errors;
      return rc;
    }
    std::lock_guard<std::mutex> l2(g.stat_mu);
    ++g.stats.calls;
  }
  if (!(opt && opt->sync)) return static_cast<int>(req_id);
  for (;;) {
    {
      std::lock_guard<std::mutex> l(ch->mu);
      channel_progress(ch);
      auto it = ch->pending.find(req_id);
      if (it == ch->pending.end()) return URPC_FAIL;
      if (it->second.done) {
        const int st = it->second.status;
        if (st == 0 && opt->rsp_buf) {
          const uint32_t n = std::min<uint32_t>(opt->rsp_buf_len, it->second.rsp.size());
          memcpy(opt->rsp_buf, it->second.rsp.data(), n);
          if (opt->rsp_len) *opt->rsp_len = static_cast<uint32_t>(it->second.rsp.size());
        }
        ch->pending.erase(it);
        return st;
      }
    }
    if (ch->lost.load()) {
      std::lock_guard<std::mutex> l(ch->mu);
      ch->pending.erase(req_id);
      return URPC_ERR_SESSION_CLOSE;
    }
    sched_yield();
  }
}

int urpc_func_poll(uint32_t chid, urpc_poll_msg_t* msgs, int max) {
  Channel* ch = get_channel(chid);
  if (!ch || !msgs || max <= 0) return URPC_ERR_EINVAL;
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
  std::lock_guard<std::mutex> l(ch->mu);
  return ch->pending.erase(req_id) ? URPC_SUCCESS : URPC_ERR_EINVAL;
}

// ---------------------------------------------------------------------------------------------- management socket
static std::string admin_report(const std::string& cmd) {
  char line[512];
  std::string r;
  if (cmd == "version") {
    r = "urpc 1.0 (umdk_b200), protocol version " + std::to_string((int)urpc_proto::kVersion) + "\n";
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
      snprintf(line, sizeof(line), "session %u tcp_fd %d queue %llx control %s payload %s\n", s->id, s->tcp,
               (unsigned long long)s->umqh, s->conn ? s->conn->cipher() : "none", s->seal.on() ? "sealed" : "clear");
      r += line;
    }
    if (r.empty()) r = "(no sessions)\n";
  } else if (cmd == "funcs") {
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.funcs) {
      snprintf(line, sizeof(line), "func 0x%llx\n", (unsigned long long)kv.first);
      r += line;
    }
    if (r.empty()) r = "(no functions)\n";
  } else {
    r = "unknown command; try: version stats perf channels sessions funcs\n";
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
  std::lock_guard<std::mutex> l(g.stat_mu);
  *out = g.stats;
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
  if (!s || n == 0 || n > URPC_MAX_REFS || lane > s->extra.size()) return nullptr;
  *tmp = CurrentReq{lane ? s->extra[lane - 1]->umqh : s->umqh, reinterpret_cast<const RefEntry*>(args + all - 4 - n * sizeof(RefEntry)), n};
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
  if (!ch || ch->attached.load()) return URPC_ERR_EINVAL;   // queues change hands only while detached
  {   // one queue serves one channel
    std::lock_guard<std::mutex> l(g.mu);
    for (auto& kv : g.channels)
      if (channel_lane(kv.second, qh) >= 0) return URPC_ERR_EINVAL;
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
  if (!ch || ch->attached.load()) return URPC_ERR_EINVAL;
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
  std::lock_guard<std::mutex> l(g.stat_mu);
  stats[0] = g.stats.errors;
  stats[1] = g.stats.timeouts;
  stats[2] = g.stats.keepalive_lost;
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
  std::lock_guard<std::mutex> l(g.stat_mu);
  if (count) *count = g.lat.count();
  if (avg_ns) *avg_ns = static_cast<uint64_t>(g.lat.mean());
  if (p99_ns) *p99_ns = g.lat.quantile(0.99);
  return URPC_SUCCESS;
}

}  // extern "C"
