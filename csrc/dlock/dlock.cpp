// DLock server and client.
//
// Kept from the reference (src/ulock/dlock/lib): two server threads - a control thread serving TCP requests
// (client init / get_lock / release / heartbeat / object create, server/dlock_server.cpp:53-95) and a command thread
// that busy-polls the URMA completion queue, applies lock commands to the lock memory and replies
// (dlock_server.cpp:1536-1595, 1248-1308); per-type state machines in the lock memory (lock_memory.cpp:205-698:
// ATOMIC = exclusive owner + lease, RW = writer or reader count + lease, FAIR = ticket lock served in FIFO order);
// leases that expire so a crashed holder cannot block others forever; clients keep a cache of the locks they hold
// and push it to a restarted server, which answers DLOCK_NOT_READY until enough clients have re-registered
// (dlock_server.cpp:2685-2890, DLock User Guide :218-236); 64-bit atomic objects accessed with one-sided URMA
// fetch-add / compare-swap on a server segment (common/jetty_mgr.cpp:518-527); debug counters.
// Security (the reference's ssl_connection.cpp and dlock_cipher.cpp): with a pre-shared key configured (dlock_set_psk or
// DLOCK_PSK / DLOCK_PSK_ID in the environment) the control channel runs TLS 1.3 PSK with TLS_AES_256_GCM_SHA384, the
// server hands each client a random 256-bit data key inside that channel, and every lock command and reply on the
// URMA data channel is sealed with AES-256-GCM under that key (client id in clear as the key selector, a message
// counter as the nonce, replayed or unsealed commands refused).
#include "dlock_api.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "ub_secure.h"
#include "ub_util.h"
#include "urma_simple.h"

namespace {

constexpr uint32_t kMagic = 0x444c4f43;  // "DLOC"
enum CtlOp : uint32_t { C_INIT = 1, C_REINIT, C_DEINIT, C_HEARTBEAT, C_GET_LOCK, C_RELEASE_LOCK, C_OBJ_CREATE,
                        C_OBJ_GET, C_OBJ_DESTROY, C_UPDATE_LOCK, C_REINIT_DONE, C_OBJ_RELEASE };
struct CtlMsg {
  uint32_t magic, op;
  int32_t client_id, status;
  int32_t id;          // lock id / object id
  uint32_t type;       // lock type / op
  uint64_t value;      // object init / lease remaining
  char name[DLOCK_NAME_LEN];
  uint8_t ep_blob[URMA_SIMPLE_JETTY_BLOB];
  uint8_t seg_blob[URMA_SIMPLE_SEG_BLOB];
  uint32_t epoch;      // server incarnation
  uint32_t secure;     // init reply: 1 = data_key is valid and commands must be sealed
  uint8_t data_key[32];
};
struct CmdMsg {  // data plane
  uint32_t magic, seq;
  int32_t client_id, lock_id;
  uint32_t op, expire_ms;
  int32_t status;
  uint32_t epoch;
};

// What travels on the data channel: the command itself, or its sealed form.
struct CmdWire {
  int32_t client_id;   // in clear: selects the key on the server
  uint32_t sealed;     // 0 = body holds a plain CmdMsg, 1 = AES-256-GCM ciphertext + tag
  uint64_t nonce;      // sender's message counter, never reused under one key
  uint8_t body[sizeof(CmdMsg) + ub::AeadCipher::kTagBytes];
};
constexpr uint32_t kDirToServer = 0, kDirToClient = 1;  // nonce salts: the two directions never share a nonce

struct DataKey {
  std::unique_ptr<ub::AeadCipher> tx, rx;
  uint64_t tx_nonce = 0, rx_last = 0;
  void set(const uint8_t key[32], bool is_server) {
    tx.reset(new ub::AeadCipher(key, is_server ? kDirToClient : kDirToServer));
    rx.reset(new ub::AeadCipher(key, is_server ? kDirToServer : kDirToClient));
    tx_nonce = rx_last = 0;
  }
  bool on() const { return tx != nullptr; }
};

void pack_cmd(CmdWire* w, const CmdMsg& m, DataKey* k) {
  w->client_id = m.client_id;
  if (k && k->on()) {
    w->sealed = 1;
    w->nonce = ++k->tx_nonce;
    k->tx->seal(w->nonce, w, 16, &m, sizeof(m), w->body);
  } else {
    w->sealed = 0;
    w->nonce = 0;
    memcpy(w->body, &m, sizeof(m));
  }
}
// False when the message must be dropped: sealed without a key, unsealed although a key is set, bad tag, replay.
bool unpack_cmd(const CmdWire& w, CmdMsg* m, DataKey* k) {
  if (!k || !k->on()) {
    if (w.sealed) return false;
    memcpy(m, w.body, sizeof(*m));
    return true;
  }
  if (!w.sealed || w.nonce <= k->rx_last) return false;
  if (!k->rx->open(w.nonce, &w, 16, w.body, sizeof(w.body), m)) return false;
  k->rx_last = w.nonce;
  return m->client_id == w.client_id;
}

std::mutex g_psk_mu;
ub::PskConfig g_psk;
bool g_psk_loaded = false, g_psk_bad = false;
// The key in force: the one set with dlock_set_psk, else the environment's. *bad: the environment's key is malformed.
ub::PskConfig current_psk(bool* bad) {
  std::lock_guard<std::mutex> l(g_psk_mu);
  if (!g_psk_loaded) {
    g_psk = ub::PskConfig::from_env("DLOCK", &g_psk_bad);
    g_psk_loaded = true;
  }
  *bad = g_psk_bad;
  return g_psk;
}

// ------------------------------------------------------------------------------------------------ lock memory
struct LockEntry {
  bool used = false;
  dlock_type_t type = DLOCK_ATOMIC;
  std::string name;
  int refs = 0;
  // ATOMIC / RW writer
  int32_t owner = -1;
  uint64_t owner_expiry = 0;
  // RW readers
  std::map<int32_t, uint64_t> readers;  // client -> expiry
  // FAIR
  uint32_t next_ticket = 0, now_serving = 0;
  std::map<int32_t, uint32_t> tickets;  // waiting client -> ticket
};

struct LockMemory {
  std::vector<LockEntry> locks;
  std::unordered_map<std::string, int32_t> by_name;
  dlock_debug_stats_t st{};

  void expire(LockEntry& e, uint64_t now) {
    if (e.owner >= 0 && now > e.owner_expiry) {
      e.owner = -1;
      ++st.expired_takeover;
      if (e.type == DLOCK_FAIR) ++e.now_serving;
    }
    for (auto it = e.readers.begin(); it != e.readers.end();)
      it = now > it->second ? e.readers.erase(it) : std::next(it);
  }

  int apply(int32_t client, int32_t id, uint32_t op, uint32_t expire_ms) {
    if (id < 0 || id >= (int32_t)locks.size() || !locks[id].used) return DLOCK_LOCK_NOT_FOUND;
    LockEntry& e = locks[id];
    const uint64_t now = ub::now_ns();
    const uint64_t lease = now + uint64_t(expire_ms ? expire_ms : 10000) * 1000000ull;
    expire(e, now);
    switch (op) {
      case DLOCK_LOCK_EXCLUSIVE:
        if (e.owner == client) return DLOCK_ALREADY_LOCKED;
        if (e.type == DLOCK_FAIR) {
          auto it = e.tickets.find(client);
          if (it == e.tickets.end()) it = e.tickets.emplace(client, e.next_ticket++).first;
          if (e.owner >= 0 || it->second != e.now_serving) {
            ++st.trylock_busy;
            return DLOCK_EAGAIN;
          }
          e.tickets.erase(it);
          e.owner = client;
          e.owner_expiry = lease;
          ++st.trylock_ok;
          return DLOCK_SUCCESS;
        }
        if (e.owner >= 0 || !e.readers.empty()) {
          ++st.trylock_busy;
          return DLOCK_EAGAIN;
        }
        e.owner = client;
        e.owner_expiry = lease;
        ++st.trylock_ok;
        return DLOCK_SUCCESS;
      case DLOCK_LOCK_SHARED:
        if (e.type != DLOCK_RW) return DLOCK_EINVAL;
        if (e.owner >= 0) {
          ++st.trylock_busy;
          return DLOCK_EAGAIN;
        }
        e.readers[client] = lease;
        ++st.trylock_ok;
        return DLOCK_SUCCESS;
      case DLOCK_UNLOCK:
        if (e.owner == client) {
          e.owner = -1;
          if (e.type == DLOCK_FAIR) ++e.now_serving;
          ++st.unlock_ok;
          return DLOCK_SUCCESS;
        }
        if (e.readers.erase(client)) {
          ++st.unlock_ok;
          return DLOCK_SUCCESS;
        }
        if (e.type == DLOCK_FAIR && e.tickets.count(client)) {  // give up a queued ticket
          const uint32_t t = e.tickets[client];
          e.tickets.erase(client);
          if (t == e.now_serving && e.owner < 0) ++e.now_serving;
          ++st.unlock_ok;
          return DLOCK_SUCCESS;
        }
        ++st.unlock_fail;
        return DLOCK_NOT_OWNER;
      case DLOCK_EXTEND:
        if (e.owner == client) {
          e.owner_expiry = lease;
          ++st.extend_ok;
          return DLOCK_SUCCESS;
        }
        if (e.readers.count(client)) {
          e.readers[client] = lease;
          ++st.extend_ok;
          return DLOCK_SUCCESS;
        }
        return DLOCK_NOT_OWNER;
      default: return DLOCK_EINVAL;
    }
  }
  // a ticket whose owner vanished must not stall the queue: skip tickets of clients that no longer wait
  void drop_client(int32_t client) {
    for (auto& e : locks) {
      if (!e.used) continue;
      if (e.owner == client) {
        e.owner = -1;
        if (e.type == DLOCK_FAIR) ++e.now_serving;
      }
      e.readers.erase(client);
      auto it = e.tickets.find(client);
      if (it != e.tickets.end()) {
        const uint32_t t = it->second;
        e.tickets.erase(it);
        if (t == e.now_serving && e.owner < 0) ++e.now_serving;
      }
    }
  }
};

// ------------------------------------------------------------------------------------------------ server
struct SrvClient {
  int32_t id;
  int fd;
  std::unique_ptr<ub::SecureConn> conn;
  DataKey key;
  urma_target_jetty_t* ep = nullptr;
  uint64_t last_seen;
  bool alive = true;
  bool reinit_done = false;
};
struct Server {
  dlock_server_cfg_t cfg;
  int listen_fd = -1;
  uint16_t port = 0;
  uint32_t epoch;
  std::thread ctl, cmd;
  std::atomic<bool> stop{false};
  std::mutex mu;
  LockMemory mem;
  ub::PskConfig psk;
  std::vector<SrvClient*> clients;
  urma_context_t* ctx = nullptr;
  urma_simple_ep_t* ep = nullptr;
  std::vector<uint64_t> objects;
  std::vector<char> obj_used;
  std::unordered_map<std::string, int32_t> obj_by_name;
  urma_target_seg_t* obj_seg = nullptr;
  uint8_t obj_blob[URMA_SIMPLE_SEG_BLOB];
  std::vector<CmdWire> rx;  // receive ring
  std::deque<CmdWire*> tx_free;
  std::vector<CmdWire> tx;
  bool recovering = false;
  uint32_t recovered_clients = 0;
  uint64_t recovery_deadline = 0;
};
std::mutex g_srv_mu;
std::map<int, Server*> g_servers;
int g_next_server = 1;

void srv_handle_ctl(Server* s, SrvClient* c, const CtlMsg& in) {
  CtlMsg out = in;
  out.status = DLOCK_SUCCESS;
  out.epoch = s->epoch;
  std::lock_guard<std::mutex> l(s->mu);
  ++s->mem.st.control_msgs;
  c->last_seen = ub::now_ns();
  switch (in.op) {
    case C_HEARTBEAT: ++s->mem.st.heartbeat; break;
    case C_REINIT_DONE: {
      // this client has pushed all its locks; when every connected client has said so, recovery is over at once
      c->reinit_done = true;
      bool all = true;
      for (auto* o : s->clients) all &= !o->alive || o->reinit_done;
      if (all && s->recovered_clients >= s->cfg.recovery_client_num) s->recovering = false;
      break;
    }
    case C_OBJ_RELEASE:
      if (in.id < 0 || in.id >= (int32_t)s->obj_used.size() || !s->obj_used[in.id]) out.status = DLOCK_LOCK_NOT_FOUND;
      break;   // the object stays until it is destroyed; the client only drops its handle
    case C_GET_LOCK: {
      const std::string name(in.name, strnlen(in.name, DLOCK_NAME_LEN));
      auto it = s->mem.by_name.find(name);
      if (it != s->mem.by_name.end()) {
        if (s->mem.locks[it->second].type != (dlock_type_t)in.type) {
          out.status = DLOCK_EINVAL;
          break;
        }
        out.id = it->second;
        ++s->mem.locks[it->second].refs;
        break;
      }
      int32_t id = -1;
      for (size_t i = 0; i < s->mem.locks.size(); ++i)
        if (!s->mem.locks[i].used) {
          id = (int32_t)i;
          break;
        }
      if (id < 0) {
        if (s->mem.locks.size() >= s->cfg.max_locks) {
          out.status = DLOCK_SERVER_FULL;
          break;
        }
        id = (int32_t)s->mem.locks.size();
        s->mem.locks.emplace_back();
      }
      LockEntry& e = s->mem.locks[id];
      e = LockEntry();
      e.used = true;
      e.type = (dlock_type_t)in.type;
      e.name = name;
      e.refs = 1;
      s->mem.by_name[name] = id;
      out.id = id;
      break;
    }
    case C_RELEASE_LOCK: {
      if (in.id < 0 || in.id >= (int32_t)s->mem.locks.size() || !s->mem.locks[in.id].used) {
        out.status = DLOCK_LOCK_NOT_FOUND;
        break;
      }
      LockEntry& e = s->mem.locks[in.id];
      if (--e.refs <= 0) {
        s->mem.by_name.erase(e.name);
        e = LockEntry();
      }
      break;
    }
    case C_UPDATE_LOCK: {  // recovery: the client reports a lock it holds (name, type, mode, remaining lease)
      const std::string name(in.name, strnlen(in.name, DLOCK_NAME_LEN));
      int32_t id;
      auto it = s->mem.by_name.find(name);
      if (it == s->mem.by_name.end()) {
        id = (int32_t)s->mem.locks.size();
        s->mem.locks.emplace_back();
        s->mem.locks[id].used = true;
        s->mem.locks[id].type = (dlock_type_t)(in.type & 0xff);
        s->mem.locks[id].name = name;
        s->mem.by_name[name] = id;
      } else {
        id = it->second;
      }
      LockEntry& e = s->mem.locks[id];
      ++e.refs;
      const uint64_t lease = ub::now_ns() + in.value * 1000000ull;
      if ((in.type >> 8) == DLOCK_LOCK_SHARED) e.readers[c->id] = lease;
      else if ((in.type >> 8) == DLOCK_LOCK_EXCLUSIVE) {
        e.owner = c->id;
        e.owner_expiry = lease;
      }
      ++s->mem.st.recovered_locks;
      out.id = id;
      break;
    }
    case C_OBJ_CREATE: {
      const std::string name(in.name, strnlen(in.name, DLOCK_NAME_LEN));
      if (s->obj_by_name.count(name)) {
        out.status = DLOCK_ALREADY_LOCKED;
        out.id = s->obj_by_name[name];
        break;
      }
      int32_t id = -1;
      for (size_t i = 0; i < s->obj_used.size(); ++i)
        if (!s->obj_used[i]) {
          id = (int32_t)i;
          break;
        }
      if (id < 0) {
        out.status = DLOCK_SERVER_FULL;
        break;
      }
      s->obj_used[id] = 1;
      __atomic_store_n(&s->objects[id], in.value, __ATOMIC_SEQ_CST);
      s->obj_by_name[name] = id;
      ++s->mem.st.objects;
      out.id = id;
      break;
    }
    case C_OBJ_GET: {
      const std::string name(in.name, strnlen(in.name, DLOCK_NAME_LEN));
      auto it = s->obj_by_name.find(name);
      if (it == s->obj_by_name.end()) out.status = DLOCK_LOCK_NOT_FOUND;
      else out.id = it->second;
      break;
    }
    case C_OBJ_DESTROY: {
      if (in.id < 0 || in.id >= (int32_t)s->obj_used.size() || !s->obj_used[in.id]) {
        out.status = DLOCK_LOCK_NOT_FOUND;
        break;
      }
      s->obj_used[in.id] = 0;
      for (auto it = s->obj_by_name.begin(); it != s->obj_by_name.end(); ++it)
        if (it->second == in.id) {
          s->obj_by_name.erase(it);
          break;
        }
      break;
    }
    case C_DEINIT:
      s->mem.drop_client(c->id);
      c->alive = false;
      break;
    default: out.status = DLOCK_EINVAL;
  }
  c->conn->write_full(&out, sizeof(out));
}

void srv_ctl_loop(Server* s) {
  while (!s->stop.load()) {
    std::vector<pollfd> pfs;
    pfs.push_back(pollfd{s->listen_fd, POLLIN, 0});
    std::vector<SrvClient*> cs;
    {
      std::lock_guard<std::mutex> l(s->mu);
      for (auto* c : s->clients)
        if (c->alive) {
          pfs.push_back(pollfd{c->fd, POLLIN, 0});
          cs.push_back(c);
        }
    }
    bool buffered = false;  // decrypted bytes waiting inside a TLS object do not show up in poll()
    for (auto* c : cs) buffered |= c->conn->pending();
    if (poll(pfs.data(), pfs.size(), buffered ? 0 : 50) <= 0 && !buffered) continue;
    if (pfs[0].revents & POLLIN) {
      const int fd = accept(s->listen_fd, nullptr, nullptr);
      if (fd >= 0) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        CtlMsg m;
        std::string err;
        std::unique_ptr<ub::SecureConn> conn = ub::SecureConn::server(fd, s->psk, 3000, &err);
        if (!conn) {
          std::lock_guard<std::mutex> l(s->mu);
          ++s->mem.st.tls_rejected;
          close(fd);
        } else if (conn->read_full(&m, sizeof(m), 3000) && m.magic == kMagic && (m.op == C_INIT || m.op == C_REINIT)) {
          std::lock_guard<std::mutex> l(s->mu);
          CtlMsg out = m;
          out.epoch = s->epoch;
          if (s->clients.size() >= s->cfg.max_clients) {
            out.status = DLOCK_SERVER_FULL;
            conn->write_full(&out, sizeof(out));
            conn.reset();
            close(fd);
          } else {
            SrvClient* c = new SrvClient();
            c->id = m.op == C_REINIT && m.client_id >= 0 ? m.client_id : (int32_t)s->clients.size() + 1000 * (int32_t)(s->epoch & 0xff);
            c->fd = fd;
            out.secure = 0;
            if (conn->encrypted() && ub::random_bytes(out.data_key, sizeof(out.data_key))) {
              out.secure = 1;
              c->key.set(out.data_key, true);
            }
            c->last_seen = ub::now_ns();
            c->ep = urma_simple_ep_import(s->ctx, m.ep_blob, 0x646c);
            s->clients.push_back(c);
            ++s->mem.st.clients;
            if (m.op == C_REINIT && s->recovering) ++s->recovered_clients;
            out.client_id = c->id;
            out.status = c->ep ? DLOCK_SUCCESS : DLOCK_FAIL;
            urma_simple_ep_blob(s->ep, out.ep_blob);
            memcpy(out.seg_blob, s->obj_blob, sizeof(out.seg_blob));
            if (conn->encrypted() && !out.secure) out.status = DLOCK_FAIL;  // no randomness for a data key
            conn->write_full(&out, sizeof(out));
            c->conn = std::move(conn);
          }
        } else {
          conn.reset();
          close(fd);
        }
      }
    }
    for (size_t i = 1; i < pfs.size(); ++i) {
      SrvClient* c = cs[i - 1];
      if (pfs[i].revents & (POLLHUP | POLLERR)) {
        std::lock_guard<std::mutex> l(s->mu);
        c->alive = false;  // connection lost: the client's leases run out on their own
        continue;
      }
      if ((pfs[i].revents & POLLIN) || c->conn->pending()) {
        CtlMsg m;
        if (!c->conn->read_full(&m, sizeof(m), 1000) || m.magic != kMagic) {
          std::lock_guard<std::mutex> l(s->mu);
          c->alive = false;
          continue;
        }
        srv_handle_ctl(s, c, m);
      }
    }
  }
}

void srv_cmd_loop(Server* s) {
  int st[32];
  uint64_t uc[32], imm[32];
  uint32_t len[32], flag[32];
  uint32_t idle = 0;
  while (!s->stop.load()) {
    const int n = urma_simple_poll(s->ep, 32, st, uc, len, imm, flag);
    if (n <= 0) {
      // the next command usually follows within microseconds: poll tightly first, then offer the core, then sleep
      if (++idle > 4000) usleep(50);
      else if (idle > 200) sched_yield();
      else ub::cpu_relax();
      continue;
    }
    idle = 0;
    for (int i = 0; i < n; ++i) {
      if (!(flag[i] & URMA_CR_FLAG_RECV)) {
        if (uc[i]) {
          std::lock_guard<std::mutex> l(s->mu);
          s->tx_free.push_back(reinterpret_cast<CmdWire*>(uc[i]));
        }
        continue;
      }
      CmdWire* wire = reinterpret_cast<CmdWire*>(uc[i]);
      CmdMsg cmd{};
      CmdMsg* in = &cmd;
      CmdMsg reply{};
      urma_target_jetty_t* dst = nullptr;
      SrvClient* from = nullptr;
      {
        std::lock_guard<std::mutex> l(s->mu);
        ++s->mem.st.data_msgs;
        for (auto* c : s->clients)
          if (c->id == wire->client_id && c->alive) from = c;
        // a command that does not open under its sender's key (or comes in clear to a secured server) is dropped
        if (st[i] != 0 || !from || !unpack_cmd(*wire, &cmd, &from->key)) {
          ++s->mem.st.sealed_rejected;
          urma_simple_post_recv(s->ep, wire, sizeof(CmdWire), reinterpret_cast<uint64_t>(wire));
          continue;
        }
        reply = cmd;
        if (s->recovering) {
          if (s->recovered_clients >= s->cfg.recovery_client_num || ub::now_ns() > s->recovery_deadline)
            s->recovering = false;
        }
        if (st[i] != 0 || in->magic != kMagic) reply.status = DLOCK_EINVAL;
        else if (s->recovering) reply.status = DLOCK_NOT_READY;
        else reply.status = s->mem.apply(in->client_id, in->lock_id, in->op, in->expire_ms);
        reply.epoch = s->epoch;
        dst = from->ep;
      }
      urma_simple_post_recv(s->ep, wire, sizeof(CmdWire), reinterpret_cast<uint64_t>(wire));
      if (!dst) continue;
      CmdWire* out = nullptr;
      {
        std::lock_guard<std::mutex> l(s->mu);
        if (!s->tx_free.empty()) {
          out = s->tx_free.front();
          s->tx_free.pop_front();
        }
      }
      if (!out) continue;  // reply ring exhausted: the client retries after its timeout
      {
        std::lock_guard<std::mutex> l(s->mu);
        pack_cmd(out, reply, &from->key);
      }
      if (urma_simple_post(s->ep, dst, URMA_OPC_SEND, nullptr, 0, nullptr, reinterpret_cast<uint64_t>(out),
                           sizeof(CmdWire), 0, reinterpret_cast<uint64_t>(out), 1) != 0) {
        std::lock_guard<std::mutex> l(s->mu);
        s->tx_free.push_back(out);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ client
struct HeldLock {
  std::string name;
  dlock_type_t type;
  int mode;  // -1 none, DLOCK_LOCK_EXCLUSIVE, DLOCK_LOCK_SHARED
  uint64_t expiry_ns;
};
struct Client {
  int32_t id = -1;
  int fd = -1;
  std::unique_ptr<ub::SecureConn> conn;
  DataKey key;
  uint32_t epoch = 0;
  urma_context_t* ctx = nullptr;
  urma_simple_ep_t* ep = nullptr;
  urma_target_jetty_t* srv = nullptr;
  urma_target_seg_t* objseg = nullptr;
  uint64_t obj_va = 0;
  std::mutex mu;
  uint32_t seq = 1;
  CmdMsg tx;
  CmdWire tx_wire, rx[8];
  bool async_pending = false;   // a lock_request_async is outstanding
  dlock_lock_req_t async_req{};
  uint64_t async_deadline = 0;
  uint64_t result;
  std::map<int32_t, HeldLock> locks;  // lock id -> description and state (the recovery cache)
  dlock_debug_stats_t st{};
};
std::mutex g_cli_mu;
std::map<int, Client*> g_clients;
int g_next_client = 1;

const char* g_default_dev_name();

Client* cli(int handle) {
  std::lock_guard<std::mutex> l(g_cli_mu);
  auto it = g_clients.find(handle);
  return it == g_clients.end() ? nullptr : it->second;
}

int ctl_call(Client* c, CtlMsg* m) {
  m->magic = kMagic;
  m->client_id = c->id;
  ++c->st.control_msgs;
  if (!c->conn || !c->conn->write_full(m, sizeof(*m)) || !c->conn->read_full(m, sizeof(*m), 3000))
    return DLOCK_BAD_RESPONSE;
  if (m->epoch != c->epoch) return DLOCK_BAD_RESPONSE;
  return m->status;
}

int connect_server(Client* c, const char* ip, uint16_t port, bool reinit) {
  const int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return DLOCK_FAIL;
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(port);
  a.sin_addr.s_addr = ip && *ip ? inet_addr(ip) : htonl(INADDR_LOOPBACK);
  if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
    close(fd);
    return DLOCK_BAD_RESPONSE;
  }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  bool bad_key = false;
  const ub::PskConfig psk = current_psk(&bad_key);
  if (bad_key) {
    close(fd);
    return DLOCK_EINVAL;
  }
  std::string err;
  std::unique_ptr<ub::SecureConn> conn = ub::SecureConn::client(fd, psk, 3000, &err);
  if (!conn) {
    close(fd);
    return DLOCK_BAD_RESPONSE;  // the server refused the key, speaks no TLS, or is gone
  }
  CtlMsg m{};
  m.magic = kMagic;
  m.op = reinit ? C_REINIT : C_INIT;
  m.client_id = c->id;
  urma_simple_ep_blob(c->ep, m.ep_blob);
  if (!conn->write_full(&m, sizeof(m)) || !conn->read_full(&m, sizeof(m), 3000) || m.status != DLOCK_SUCCESS ||
      (conn->encrypted() && !m.secure)) {
    conn.reset();
    close(fd);
    return m.status ? m.status : DLOCK_BAD_RESPONSE;
  }
  c->conn.reset();
  if (c->fd >= 0) close(c->fd);
  c->fd = fd;
  c->conn = std::move(conn);
  if (m.secure) c->key.set(m.data_key, false);
  else c->key = DataKey();
  c->id = m.client_id;
  c->epoch = m.epoch;
  if (c->srv) urma_unimport_jetty(c->srv);
  if (c->objseg) urma_unimport_seg(c->objseg);
  c->srv = urma_simple_ep_import(c->ctx, m.ep_blob, 0x646c);
  c->objseg = urma_simple_seg_import(c->ctx, m.seg_blob, 0x6f626a);
  if (!c->srv || !c->objseg) return DLOCK_FAIL;
  c->obj_va = c->objseg->seg.ubva.va;
  return DLOCK_SUCCESS;
}

// Data channel: a request is one sealed (or plain) command sent to the server; its reply is matched by sequence number.
int data_send(Client* c, int32_t lock_id, uint32_t op, uint32_t expire_ms) {
  c->tx = CmdMsg{kMagic, c->seq++, c->id, lock_id, op, expire_ms, 0, c->epoch};
  ++c->st.data_msgs;
  pack_cmd(&c->tx_wire, c->tx, &c->key);
  if (urma_simple_post(c->ep, c->srv, URMA_OPC_SEND, nullptr, 0, nullptr, reinterpret_cast<uint64_t>(&c->tx_wire),
                       sizeof(CmdWire), 0, 0, 0) != 0)
    return DLOCK_BAD_RESPONSE;
  return DLOCK_SUCCESS;
}
// Polls for the reply of the last data_send until `deadline_ns`. DLOCK_ASYNC_AGAIN = nothing yet.
int data_poll(Client* c, uint64_t deadline_ns) {
  int st[4];
  uint64_t uc[4], imm[4];
  uint32_t len[4], flag[4];
  uint32_t spins = 0;
  do {
    const int n = urma_simple_poll(c->ep, 4, st, uc, len, imm, flag);
    for (int i = 0; i < n; ++i) {
      if (!(flag[i] & URMA_CR_FLAG_RECV)) {
        if (st[i] != 0) return DLOCK_BAD_RESPONSE;
        continue;
      }
      CmdWire* r = reinterpret_cast<CmdWire*>(uc[i]);
      CmdMsg got{};
      const bool opened = unpack_cmd(*r, &got, &c->key);
      urma_simple_post_recv(c->ep, r, sizeof(CmdWire), reinterpret_cast<uint64_t>(r));
      if (opened && got.magic == kMagic && got.seq == c->tx.seq) {
        if (got.epoch != c->epoch) return DLOCK_BAD_RESPONSE;
        return got.status;
      }
    }
    if (n <= 0) {   // an answer takes a microsecond or two: a system call between polls would double that
      if (++spins < 400) ub::cpu_relax();
      else sched_yield();
    }
  } while (ub::now_ns() < deadline_ns);
  return DLOCK_ASYNC_AGAIN;
}
// one request/response exchange on the data channel
int data_call(Client* c, int32_t lock_id, uint32_t op, uint32_t expire_ms) {
  if (c->async_pending) return DLOCK_EASYNC;  // the reply slot belongs to the outstanding asynchronous request
  const int rc = data_send(c, lock_id, op, expire_ms);
  if (rc != DLOCK_SUCCESS) return rc;
  const int got = data_poll(c, ub::now_ns() + 1500000000ull);
  return got == DLOCK_ASYNC_AGAIN ? DLOCK_BAD_RESPONSE : got;  // no answer: the server is gone or was restarted
}

}  // namespace

extern "C" {

int dlock_server_start(const dlock_server_cfg_t* cfg, int* server_id, uint16_t* port_out) {
  if (!cfg || !server_id) return DLOCK_EINVAL;
  Server* s = new Server();
  s->cfg = *cfg;
  bool bad_key = false;
  s->psk = current_psk(&bad_key);
  if (bad_key) {  // a malformed key must not silently leave the server in clear text
    delete s;
    return DLOCK_EINVAL;
  }
  if (!s->cfg.max_clients) s->cfg.max_clients = 1000;
  if (!s->cfg.max_locks) s->cfg.max_locks = 51200;
  if (!s->cfg.max_objects) s->cfg.max_objects = 4096;
  if (!s->cfg.recovery_timeout_ms) s->cfg.recovery_timeout_ms = 3000;
  s->epoch = static_cast<uint32_t>(ub::now_ns() >> 10) | 1u;
  s->ctx = urma_simple_open(cfg->dev_name[0] ? cfg->dev_name : "shm0");
  if (!s->ctx) {
    delete s;
    return DLOCK_FAIL;
  }
  s->ep = urma_simple_ep_create(s->ctx, 1024, 0x646c, 0);
  s->objects.assign(s->cfg.max_objects, 0);
  s->obj_used.assign(s->cfg.max_objects, 0);
  s->obj_seg = urma_simple_seg_register(s->ctx, s->objects.data(), s->objects.size() * 8,
                                        URMA_ACCESS_READ | URMA_ACCESS_WRITE | URMA_ACCESS_ATOMIC, 0x6f626a,
                                        s->obj_blob);
  if (!s->ep || !s->obj_seg) {
    delete s;
    return DLOCK_FAIL;
  }
  s->rx.resize(512);
  for (auto& m : s->rx) urma_simple_post_recv(s->ep, &m, sizeof(CmdWire), reinterpret_cast<uint64_t>(&m));
  s->tx.resize(512);
  for (auto& m : s->tx) s->tx_free.push_back(&m);
  s->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(cfg->port);
  a.sin_addr.s_addr = cfg->ip[0] ? inet_addr(cfg->ip) : htonl(INADDR_LOOPBACK);
  if (bind(s->listen_fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || listen(s->listen_fd, 128) != 0) {
    close(s->listen_fd);
    delete s;
    return DLOCK_FAIL;
  }
  socklen_t len = sizeof(a);
  getsockname(s->listen_fd, reinterpret_cast<sockaddr*>(&a), &len);
  s->port = ntohs(a.sin_port);
  if (port_out) *port_out = s->port;
  if (s->cfg.recovery_client_num) {
    s->recovering = true;
    s->recovery_deadline = ub::now_ns() + uint64_t(s->cfg.recovery_timeout_ms) * 1000000ull;
  }
  s->ctl = std::thread(srv_ctl_loop, s);
  s->cmd = std::thread(srv_cmd_loop, s);
  std::lock_guard<std::mutex> l(g_srv_mu);
  *server_id = g_next_server++;
  g_servers[*server_id] = s;
  return DLOCK_SUCCESS;
}

int dlock_server_stop(int server_id) {
  Server* s;
  {
    std::lock_guard<std::mutex> l(g_srv_mu);
    auto it = g_servers.find(server_id);
    if (it == g_servers.end()) return DLOCK_EINVAL;
    s = it->second;
    g_servers.erase(it);
  }
  s->stop = true;
  s->ctl.join();
  s->cmd.join();
  close(s->listen_fd);
  for (auto* c : s->clients) {
    c->conn.reset();
    close(c->fd);
    if (c->ep) urma_unimport_jetty(c->ep);
    delete c;
  }
  urma_unregister_seg(s->obj_seg);
  urma_simple_ep_destroy(s->ep);
  urma_simple_close(s->ctx);
  delete s;
  return DLOCK_SUCCESS;
}

int dlock_set_psk(const char* key_hex, const char* identity) {
  ub::PskConfig cfg;
  if (key_hex && *key_hex) {
    if (!ub::PskConfig::parse_hex(key_hex, &cfg.key) || cfg.key.size() < 16 || cfg.key.size() > 64) return DLOCK_EINVAL;
  }
  if (identity && *identity) cfg.identity = identity;
  std::lock_guard<std::mutex> l(g_psk_mu);
  g_psk = cfg;
  g_psk_loaded = true;
  g_psk_bad = false;
  return DLOCK_SUCCESS;
}

int dlock_set_tls_files(const char* ca_file, const char* cert_file, const char* key_file) {
  const bool any = (ca_file && *ca_file) || (cert_file && *cert_file) || (key_file && *key_file);
  const bool all = ca_file && *ca_file && cert_file && *cert_file && key_file && *key_file;
  if (any && !all) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(g_psk_mu);
  if (!g_psk_loaded) g_psk = ub::PskConfig();
  g_psk.ca_file = all ? ca_file : "";
  g_psk.cert_file = all ? cert_file : "";
  g_psk.key_file = all ? key_file : "";
  g_psk_loaded = true;
  g_psk_bad = false;
  return DLOCK_SUCCESS;
}

int dlock_get_server_debug_stats(int server_id, dlock_debug_stats_t* out) {
  std::lock_guard<std::mutex> l(g_srv_mu);
  auto it = g_servers.find(server_id);
  if (it == g_servers.end() || !out) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l2(it->second->mu);
  *out = it->second->mem.st;
  return DLOCK_SUCCESS;
}

int dlock_client_init(int* client_id, const char* ip, uint16_t port) {
  if (!client_id) return DLOCK_EINVAL;
  Client* c = new Client();
  c->ctx = urma_simple_open(g_default_dev_name());
  c->ep = c->ctx ? urma_simple_ep_create(c->ctx, 64, 0x646c, 0) : nullptr;
  if (!c->ep) {
    delete c;
    return DLOCK_FAIL;
  }
  for (auto& m : c->rx) urma_simple_post_recv(c->ep, &m, sizeof(CmdWire), reinterpret_cast<uint64_t>(&m));
  const int rc = connect_server(c, ip, port, false);
  if (rc != DLOCK_SUCCESS) {
    urma_simple_ep_destroy(c->ep);
    urma_simple_close(c->ctx);
    delete c;
    return rc;
  }
  std::lock_guard<std::mutex> l(g_cli_mu);
  *client_id = g_next_client++;
  g_clients[*client_id] = c;
  return DLOCK_SUCCESS;
}

int dlock_client_reinit(int handle, const char* ip, uint16_t port) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  return connect_server(c, ip, port, true);
}

int dlock_client_deinit(int handle) {
  Client* c;
  {
    std::lock_guard<std::mutex> l(g_cli_mu);
    auto it = g_clients.find(handle);
    if (it == g_clients.end()) return DLOCK_CLIENT_NOT_INIT;
    c = it->second;
    g_clients.erase(it);
  }
  CtlMsg m{};
  m.op = C_DEINIT;
  ctl_call(c, &m);
  c->conn.reset();
  close(c->fd);
  if (c->srv) urma_unimport_jetty(c->srv);
  if (c->objseg) urma_unimport_seg(c->objseg);
  urma_simple_ep_destroy(c->ep);
  urma_simple_close(c->ctx);
  delete c;
  return DLOCK_SUCCESS;
}

int dlock_client_heartbeat(int handle, uint32_t) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  CtlMsg m{};
  m.op = C_HEARTBEAT;
  ++c->st.heartbeat;
  return ctl_call(c, &m);
}

int dlock_get_lock(int handle, const dlock_lock_desc_t* d, int32_t* lock_id) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  if (!d || !lock_id) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(c->mu);
  CtlMsg m{};
  m.op = C_GET_LOCK;
  m.type = d->type;
  memcpy(m.name, d->name, DLOCK_NAME_LEN);
  const int rc = ctl_call(c, &m);
  if (rc == DLOCK_SUCCESS) {
    *lock_id = m.id;
    c->locks[m.id] = HeldLock{std::string(d->name, strnlen(d->name, DLOCK_NAME_LEN)), d->type, -1, 0};
  }
  return rc;
}

int dlock_release_lock(int handle, int32_t lock_id) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  CtlMsg m{};
  m.op = C_RELEASE_LOCK;
  m.id = lock_id;
  const int rc = ctl_call(c, &m);
  if (rc == DLOCK_SUCCESS) c->locks.erase(lock_id);
  return rc;
}

int dlock_batch_get_lock(int handle, uint32_t n, const dlock_lock_desc_t* descs, int32_t* ids) {
  if (n == 0 || n > DLOCK_MAX_BATCH || !descs || !ids) return DLOCK_EINVAL;
  for (uint32_t i = 0; i < n; ++i) {
    const int rc = dlock_get_lock(handle, &descs[i], &ids[i]);
    if (rc != DLOCK_SUCCESS) return rc;
  }
  return DLOCK_SUCCESS;
}

int dlock_trylock(int handle, const dlock_lock_req_t* req) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  if (!req || (req->op != DLOCK_LOCK_EXCLUSIVE && req->op != DLOCK_LOCK_SHARED)) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(c->mu);
  const int rc = data_call(c, req->lock_id, req->op, req->expire_ms);
  if (rc == DLOCK_SUCCESS) {
    ++c->st.trylock_ok;
    auto it = c->locks.find(req->lock_id);
    if (it != c->locks.end()) {
      it->second.mode = req->op;
      it->second.expiry_ns = ub::now_ns() + uint64_t(req->expire_ms ? req->expire_ms : 10000) * 1000000ull;
    }
  } else if (rc == DLOCK_EAGAIN) {
    ++c->st.trylock_busy;
  }
  return rc;
}

int dlock_lock(int handle, const dlock_lock_req_t* req, uint32_t timeout_ms) {
  const uint64_t deadline = ub::now_ns() + uint64_t(timeout_ms) * 1000000ull;
  for (;;) {
    const int rc = dlock_trylock(handle, req);
    if (rc != DLOCK_EAGAIN && rc != DLOCK_NOT_READY) return rc;
    if (ub::now_ns() > deadline) {
      if (rc == DLOCK_EAGAIN) dlock_unlock(handle, req->lock_id);  // leave a fair lock's queue
      return DLOCK_TIMEOUT;
    }
    usleep(200);
  }
}

int dlock_unlock(int handle, int32_t lock_id) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  const int rc = data_call(c, lock_id, DLOCK_UNLOCK, 0);
  if (rc == DLOCK_SUCCESS) {
    ++c->st.unlock_ok;
    auto it = c->locks.find(lock_id);
    if (it != c->locks.end()) it->second.mode = -1;
  } else {
    ++c->st.unlock_fail;
  }
  return rc;
}

int dlock_lock_extend(int handle, int32_t lock_id, uint32_t expire_ms) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  const int rc = data_call(c, lock_id, DLOCK_EXTEND, expire_ms);
  if (rc == DLOCK_SUCCESS) {
    ++c->st.extend_ok;
    auto it = c->locks.find(lock_id);
    if (it != c->locks.end()) it->second.expiry_ns = ub::now_ns() + uint64_t(expire_ms) * 1000000ull;
  }
  return rc;
}

int dlock_batch_trylock(int handle, uint32_t n, const dlock_lock_req_t* reqs, int* results) {
  if (n == 0 || n > DLOCK_MAX_BATCH || !reqs || !results) return DLOCK_EINVAL;
  int worst = DLOCK_SUCCESS;
  for (uint32_t i = 0; i < n; ++i) {
    results[i] = dlock_trylock(handle, &reqs[i]);
    if (results[i] != DLOCK_SUCCESS) worst = results[i];
  }
  return worst;
}
int dlock_batch_unlock(int handle, uint32_t n, const int32_t* ids, int* results) {
  if (n == 0 || n > DLOCK_MAX_BATCH || !ids || !results) return DLOCK_EINVAL;
  int worst = DLOCK_SUCCESS;
  for (uint32_t i = 0; i < n; ++i) {
    results[i] = dlock_unlock(handle, ids[i]);
    if (results[i] != DLOCK_SUCCESS) worst = results[i];
  }
  return worst;
}

int dlock_batch_lock_extend(int handle, uint32_t n, const dlock_lock_req_t* reqs, int* results) {
  if (n == 0 || n > DLOCK_MAX_BATCH || !reqs || !results) return DLOCK_EINVAL;
  int worst = DLOCK_SUCCESS;
  for (uint32_t i = 0; i < n; ++i) {
    results[i] = dlock_lock_extend(handle, reqs[i].lock_id, reqs[i].expire_ms);
    if (results[i] != DLOCK_SUCCESS) worst = results[i];
  }
  return worst;
}
int dlock_batch_release_lock(int handle, uint32_t n, const int32_t* ids) {
  if (n == 0 || n > DLOCK_MAX_BATCH || !ids) return DLOCK_EINVAL;
  int worst = DLOCK_SUCCESS;
  for (uint32_t i = 0; i < n; ++i) {
    const int rc = dlock_release_lock(handle, ids[i]);
    if (rc != DLOCK_SUCCESS) worst = rc;
  }
  return worst;
}

// Asynchronous lock request: the command goes out, the caller does other work and collects the answer later. One
// request may be outstanding per client (the reference's rule, dlock_client_api.h:341-389).
int dlock_lock_request_async(int handle, const dlock_lock_req_t* req) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  if (!req) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(c->mu);
  if (c->async_pending) return DLOCK_EASYNC;
  const int rc = data_send(c, req->lock_id, req->op, req->expire_ms);
  if (rc != DLOCK_SUCCESS) return rc;
  c->async_pending = true;
  c->async_req = *req;
  c->async_deadline = ub::now_ns() + 5000000000ull;
  return DLOCK_SUCCESS;
}
int dlock_lock_result_check(int handle, int* result) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  if (!result) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(c->mu);
  if (!c->async_pending) return DLOCK_NO_ASYNC;
  const int rc = data_poll(c, ub::now_ns() + 100000ull);   // a short look, never a long wait
  if (rc == DLOCK_ASYNC_AGAIN) {
    if (ub::now_ns() < c->async_deadline) return DLOCK_ASYNC_AGAIN;
    c->async_pending = false;
    return DLOCK_TIMEOUT;
  }
  c->async_pending = false;
  *result = rc;
  const dlock_lock_req_t& r = c->async_req;
  auto it = c->locks.find(r.lock_id);
  if (rc == DLOCK_SUCCESS && it != c->locks.end()) {
    if (r.op == DLOCK_LOCK_EXCLUSIVE || r.op == DLOCK_LOCK_SHARED) {
      ++c->st.trylock_ok;
      it->second.mode = r.op;
      it->second.expiry_ns = ub::now_ns() + uint64_t(r.expire_ms ? r.expire_ms : 10000) * 1000000ull;
    } else if (r.op == DLOCK_UNLOCK) {
      ++c->st.unlock_ok;
      it->second.mode = -1;
    } else if (r.op == DLOCK_EXTEND) {
      ++c->st.extend_ok;
      it->second.expiry_ns = ub::now_ns() + uint64_t(r.expire_ms) * 1000000ull;
    }
  } else if (rc == DLOCK_EAGAIN) {
    ++c->st.trylock_busy;
  }
  return rc;
}

int dlock_client_reinit_done(int handle) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  CtlMsg m{};
  m.op = C_REINIT_DONE;
  return ctl_call(c, &m);
}
int dlock_clear_client_debug_stats(int handle) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  c->st = dlock_debug_stats_t{};
  return DLOCK_SUCCESS;
}
int dlock_clear_server_debug_stats(int server_id) {
  std::lock_guard<std::mutex> l(g_srv_mu);
  auto it = g_servers.find(server_id);
  if (it == g_servers.end()) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l2(it->second->mu);
  const uint64_t clients = it->second->mem.st.clients, objects = it->second->mem.st.objects;
  it->second->mem.st = dlock_debug_stats_t{};
  it->second->mem.st.clients = clients;     // gauges, not event counters
  it->second->mem.st.objects = objects;
  return DLOCK_SUCCESS;
}

// Library contexts (the reference's dclient_lib_init / dserver_lib_init): defaults for the instances created
// afterwards, and a tear-down that leaves no instance behind.
static std::mutex g_lib_mu;
static int g_client_lib = 0, g_server_lib = 0;
static char g_default_dev[64] = "shm0";
}  // extern "C"
namespace {
const char* g_default_dev_name() { return g_default_dev; }
}  // namespace
extern "C" {
int dlock_client_lib_init(const dlock_lib_cfg_t* cfg) {
  std::lock_guard<std::mutex> l(g_lib_mu);
  if (cfg) {
    if (cfg->dev_name[0]) snprintf(g_default_dev, sizeof(g_default_dev), "%s", cfg->dev_name);
    if (cfg->psk_hex[0] && dlock_set_psk(cfg->psk_hex, cfg->psk_identity) != DLOCK_SUCCESS) return DLOCK_EINVAL;
  }
  ++g_client_lib;
  return DLOCK_SUCCESS;
}
void dlock_client_lib_deinit(void) {
  std::vector<int> ids;
  {
    std::lock_guard<std::mutex> l(g_lib_mu);
    if (g_client_lib > 0) --g_client_lib;
    if (g_client_lib > 0) return;
    std::lock_guard<std::mutex> l2(g_cli_mu);
    for (auto& kv : g_clients) ids.push_back(kv.first);
  }
  for (int id : ids) dlock_client_deinit(id);
}
int dlock_server_lib_init(const dlock_lib_cfg_t* cfg) {
  std::lock_guard<std::mutex> l(g_lib_mu);
  if (cfg) {
    if (cfg->dev_name[0]) snprintf(g_default_dev, sizeof(g_default_dev), "%s", cfg->dev_name);
    if (cfg->psk_hex[0] && dlock_set_psk(cfg->psk_hex, cfg->psk_identity) != DLOCK_SUCCESS) return DLOCK_EINVAL;
  }
  ++g_server_lib;
  return DLOCK_SUCCESS;
}
void dlock_server_lib_deinit(void) {
  std::vector<int> ids;
  {
    std::lock_guard<std::mutex> l(g_lib_mu);
    if (g_server_lib > 0) --g_server_lib;
    if (g_server_lib > 0) return;
    std::lock_guard<std::mutex> l2(g_srv_mu);
    for (auto& kv : g_servers) ids.push_back(kv.first);
  }
  for (int id : ids) dlock_server_stop(id);
}

int dlock_update_all_locks(int handle) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  std::map<int32_t, HeldLock> fresh;
  const uint64_t now = ub::now_ns();
  for (auto& kv : c->locks) {
    CtlMsg m{};
    m.op = C_UPDATE_LOCK;
    const bool held = kv.second.mode >= 0 && kv.second.expiry_ns > now;
    m.type = (uint32_t)kv.second.type | (uint32_t)((held ? kv.second.mode : 0xff) << 8);
    m.value = held ? (kv.second.expiry_ns - now) / 1000000ull : 0;
    snprintf(m.name, sizeof(m.name), "%s", kv.second.name.c_str());
    const int rc = ctl_call(c, &m);
    if (rc != DLOCK_SUCCESS) return rc;
    HeldLock h = kv.second;
    if (!held) h.mode = -1;
    fresh[m.id] = h;  // lock ids are assigned anew by the restarted server
    ++c->st.recovered_locks;
  }
  c->locks.swap(fresh);
  return DLOCK_SUCCESS;
}

int dlock_get_client_debug_stats(int handle, dlock_debug_stats_t* out) {
  Client* c = cli(handle);
  if (!c || !out) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  *out = c->st;
  return DLOCK_SUCCESS;
}

static int obj_ctl(int handle, uint32_t op, const char* name, uint64_t init, int32_t id_in, int32_t* id_out) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  std::lock_guard<std::mutex> l(c->mu);
  CtlMsg m{};
  m.op = op;
  m.value = init;
  m.id = id_in;
  if (name) snprintf(m.name, sizeof(m.name), "%s", name);
  const int rc = ctl_call(c, &m);
  if (id_out && (rc == DLOCK_SUCCESS || rc == DLOCK_ALREADY_LOCKED)) *id_out = m.id;
  return rc;
}
int dlock_umo_atomic64_create(int h, const char* name, uint64_t init, int32_t* id) {
  return name && id ? obj_ctl(h, C_OBJ_CREATE, name, init, 0, id) : DLOCK_EINVAL;
}
int dlock_umo_atomic64_get(int h, const char* name, int32_t* id) {
  return name && id ? obj_ctl(h, C_OBJ_GET, name, 0, 0, id) : DLOCK_EINVAL;
}
int dlock_umo_atomic64_destroy(int h, int32_t id) { return obj_ctl(h, C_OBJ_DESTROY, nullptr, 0, id, nullptr); }
int dlock_umo_atomic64_release(int h, int32_t id) { return obj_ctl(h, C_OBJ_RELEASE, nullptr, 0, id, nullptr); }

static int obj_atomic(int handle, int opcode, int32_t id, uint64_t operand, uint64_t cmp, uint64_t* old) {
  Client* c = cli(handle);
  if (!c) return DLOCK_CLIENT_NOT_INIT;
  if (id < 0) return DLOCK_EINVAL;
  std::lock_guard<std::mutex> l(c->mu);
  ++c->st.object_ops;
  int rc;
  if (opcode == URMA_OPC_READ) {
    rc = urma_simple_post(c->ep, c->srv, URMA_OPC_READ, c->objseg, c->obj_va + 8ull * id, nullptr,
                          reinterpret_cast<uint64_t>(&c->result), 8, 0, 1, 1);
  } else {
    rc = urma_simple_atomic(c->ep, c->srv, opcode, c->objseg, c->obj_va + 8ull * id, operand, cmp, &c->result, 1);
  }
  if (rc != 0) return DLOCK_BAD_RESPONSE;
  int st[4];
  uint64_t uc[4];
  uint32_t flag[4];
  const uint64_t deadline = ub::now_ns() + 3000000000ull;
  while (ub::now_ns() < deadline) {
    const int n = urma_simple_poll(c->ep, 4, st, uc, nullptr, nullptr, flag);
    for (int i = 0; i < n; ++i)
      if (!(flag[i] & URMA_CR_FLAG_RECV) && uc[i] == 1) {
        if (st[i] != 0) return DLOCK_BAD_RESPONSE;
        if (old) *old = c->result;
        return DLOCK_SUCCESS;
      }
    if (n <= 0) sched_yield();
  }
  return DLOCK_BAD_RESPONSE;
}
int dlock_umo_atomic64_faa(int h, int32_t id, uint64_t add, uint64_t* old) {
  return obj_atomic(h, URMA_OPC_FADD, id, add, 0, old);
}
int dlock_umo_atomic64_cas(int h, int32_t id, uint64_t cmp, uint64_t swap, uint64_t* old) {
  return obj_atomic(h, URMA_OPC_CAS, id, swap, cmp, old);
}
int dlock_umo_atomic64_get_snapshot(int h, int32_t id, uint64_t* value) {
  return obj_atomic(h, URMA_OPC_READ, id, 0, 0, value);
}

}  // extern "C"
