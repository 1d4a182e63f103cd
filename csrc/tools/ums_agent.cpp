// ums_agent: token agent of the UMS sockets (one per host).
//
//   ums_agent [--config FILE] [--sock PATH] [--ip ADDR] [--port N] [--syslog] [--insecure]
//
// Local UMS endpoints talk to it over a Unix stream socket (PUT / DEL / GET / STATS records of ums_agent_proto.h);
// agents talk to each other over TLS 1.3 (pre-shared key or certificates, the secure layer of the host libraries) and
// answer only GET. A GET that names a peer "ip:port" is forwarded to that agent over a pooled connection. The daemon
// refuses to start without a key or certificates unless --insecure is given. SIGTERM / SIGINT end it cleanly (the
// Unix socket is removed).
//
// Config file: `key = value` lines, `#` comments. Keys: sock, ip, port, psk, psk_id, tls_ca, tls_cert, tls_key,
// max_tokens, peer_timeout_ms, pool_idle_ms, log_level (0 errors .. 4 debug). Command-line options come last. The key
// may also come from UMS_AGENT_PSK / UMS_AGENT_PSK_ID or UMS_AGENT_TLS_CA / _CERT / _KEY in the environment.
//
// Same role as the reference daemon: main loop and signal handling (src/usock/ums/ums_agent/ums_agent_main.c),
// configuration (ums_agent_config.c), token proxy (ums_agent_token_proxy.c), TLS connections and their pool
// (ums_agent_tls_conn.c), syslog logging (ums_agent_log.c). The local side is a Unix socket instead of netlink.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <signal.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/epoll.h>
#include <sys/signalfd.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <syslog.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "ub_secure.h"
#include "ub_util.h"
#include "ums_agent_proto.h"

namespace {

struct Config {
  std::string sock = UMS_AGENT_DEFAULT_SOCK;
  std::string ip = "127.0.0.1";
  int port = 0;   // 0 = any free port (printed at start)
  ub::PskConfig sec;
  uint32_t max_tokens = 65536;
  int peer_timeout_ms = 3000;
  int pool_idle_ms = 60000;
  int log_level = ub::kLogNotice;
  bool use_syslog = false;
  bool insecure = false;
};

ub::Logger g_log("UMS_AGENT");
std::atomic<bool> g_stop{false};

void syslog_sink(int lvl, const char* msg) {
  static const int prio[] = {3 /*err*/, 4 /*warning*/, 5 /*notice*/, 6 /*info*/, 7 /*debug*/};
  syslog(prio[lvl < 0 ? 0 : (lvl > 4 ? 4 : lvl)], "%s", msg);
}

std::string trim(const std::string& s) {
  const size_t a = s.find_first_not_of(" \t\r\n");
  if (a == std::string::npos) return "";
  return s.substr(a, s.find_last_not_of(" \t\r\n") - a + 1);
}

// False (with a message) on an unknown key or a value that does not parse: a daemon must not run on a half-read file.
bool set_key(Config* c, const std::string& k, const std::string& v, std::string* err) {
  auto num = [&](long lo, long hi, long* out) {
    char* end = nullptr;
    const long x = strtol(v.c_str(), &end, 10);
    if (v.empty() || *end || x < lo || x > hi) {
      *err = "bad value for " + k + ": '" + v + "'";
      return false;
    }
    *out = x;
    return true;
  };
  long x = 0;
  if (k == "sock") c->sock = v;
  else if (k == "ip") c->ip = v;
  else if (k == "port") { if (!num(0, 65535, &x)) return false; c->port = static_cast<int>(x); }
  else if (k == "psk") {
    if (!ub::PskConfig::parse_hex(v.c_str(), &c->sec.key) || c->sec.key.size() < 16 || c->sec.key.size() > 64) {
      c->sec.key.clear();
      *err = "psk must be 32..128 hex digits";
      return false;
    }
  }
  else if (k == "psk_id") c->sec.identity = v;
  else if (k == "tls_ca") c->sec.ca_file = v;
  else if (k == "tls_cert") c->sec.cert_file = v;
  else if (k == "tls_key") c->sec.key_file = v;
  else if (k == "max_tokens") { if (!num(1, 1 << 24, &x)) return false; c->max_tokens = static_cast<uint32_t>(x); }
  else if (k == "peer_timeout_ms") { if (!num(10, 600000, &x)) return false; c->peer_timeout_ms = static_cast<int>(x); }
  else if (k == "pool_idle_ms") { if (!num(0, 86400000, &x)) return false; c->pool_idle_ms = static_cast<int>(x); }
  else if (k == "log_level") { if (!num(0, 4, &x)) return false; c->log_level = static_cast<int>(x); }
  else {
    *err = "unknown key '" + k + "'";
    return false;
  }
  return true;
}

bool load_config(Config* c, const char* path, std::string* err) {
  FILE* f = fopen(path, "r");
  if (!f) {
    *err = std::string("cannot open ") + path;
    return false;
  }
  char line[1024];
  int no = 0;
  bool ok = true;
  while (ok && fgets(line, sizeof(line), f)) {
    ++no;
    std::string s(line);
    const size_t hash = s.find('#');
    if (hash != std::string::npos) s.resize(hash);
    s = trim(s);
    if (s.empty()) continue;
    const size_t eq = s.find('=');
    if (eq == std::string::npos) {
      *err = "line " + std::to_string(no) + ": expected key = value";
      ok = false;
      break;
    }
    if (!set_key(c, trim(s.substr(0, eq)), trim(s.substr(eq + 1)), err)) {
      *err = "line " + std::to_string(no) + ": " + *err;
      ok = false;
    }
  }
  fclose(f);
  return ok;
}

// ---------------------------------------------------------------------------------------------- token table
struct Stats {
  std::atomic<uint64_t> puts{0}, dels{0}, gets_local{0}, gets_forwarded{0}, gets_served{0}, misses{0}, peer_errors{0},
      tls_accepted{0}, tls_rejected{0}, pool_connects{0}, pool_reuses{0};
};
Stats g_st;

class TokenTable {
 public:
  explicit TokenTable(uint32_t cap) : cap_(cap) {}
  int put(uint64_t id, const uint8_t* v, uint32_t n) {
    std::lock_guard<std::mutex> l(mu_);
    if (!map_.count(id) && map_.size() >= cap_) return UMS_AGENT_EFULL;
    map_[id].assign(v, v + n);
    return UMS_AGENT_OK;
  }
  int del(uint64_t id) {
    std::lock_guard<std::mutex> l(mu_);
    return map_.erase(id) ? UMS_AGENT_OK : UMS_AGENT_ENOENT;
  }
  int get(uint64_t id, uint8_t* v, uint32_t* n) {
    std::lock_guard<std::mutex> l(mu_);
    auto it = map_.find(id);
    if (it == map_.end()) return UMS_AGENT_ENOENT;
    memcpy(v, it->second.data(), it->second.size());
    *n = static_cast<uint32_t>(it->second.size());
    return UMS_AGENT_OK;
  }
  size_t size() {
    std::lock_guard<std::mutex> l(mu_);
    return map_.size();
  }

 private:
  std::mutex mu_;
  uint32_t cap_;
  std::unordered_map<uint64_t, std::vector<uint8_t>> map_;
};

// ---------------------------------------------------------------------------------------------- connections to peers
struct PeerConn {
  int fd = -1;
  std::unique_ptr<ub::SecureConn> conn;
  uint64_t last_used_ns = 0;
  ~PeerConn() {
    conn.reset();
    if (fd >= 0) close(fd);
  }
};

class PeerPool {
 public:
  PeerPool(const Config& c) : cfg_(c) {}
  // One GET at the agent `peer` ("ip:port"); reuses the pooled connection and reconnects once when it has gone stale.
  int fetch(const std::string& peer, ums_agent_msg_t* m) {
    std::lock_guard<std::mutex> l(mu_);
    reap_idle();
    for (int attempt = 0; attempt < 2; ++attempt) {
      auto it = pool_.find(peer);
      const bool fresh = it == pool_.end();
      if (fresh) {
        std::unique_ptr<PeerConn> pc = dial(peer);
        if (!pc) return UMS_AGENT_EPEER;
        it = pool_.emplace(peer, std::move(pc)).first;
        ++g_st.pool_connects;
      } else {
        ++g_st.pool_reuses;
      }
      ums_agent_msg_t q = *m;
      memset(q.peer, 0, sizeof(q.peer));
      ums_agent_msg_t r;
      if (it->second->conn->write_full(&q, sizeof(q)) && it->second->conn->read_full(&r, sizeof(r), cfg_.peer_timeout_ms) &&
          r.magic == UMS_AGENT_MAGIC && r.len <= UMS_AGENT_MAX_VALUE) {
        it->second->last_used_ns = ub::now_ns();
        *m = r;
        return static_cast<int>(r.status);
      }
      pool_.erase(it);       // broken: a pooled connection gets one more try on a new one
      if (fresh) break;
    }
    return UMS_AGENT_EPEER;
  }
  size_t size() {
    std::lock_guard<std::mutex> l(mu_);
    return pool_.size();
  }

 private:
  void reap_idle() {
    if (cfg_.pool_idle_ms <= 0) return;
    const uint64_t now = ub::now_ns();
    for (auto it = pool_.begin(); it != pool_.end();)
      it = now - it->second->last_used_ns > uint64_t(cfg_.pool_idle_ms) * 1000000ull ? pool_.erase(it) : std::next(it);
  }
  std::unique_ptr<PeerConn> dial(const std::string& peer) {
    const size_t colon = peer.rfind(':');
    if (colon == std::string::npos) return nullptr;
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(static_cast<uint16_t>(atoi(peer.c_str() + colon + 1)));
    if (inet_pton(AF_INET, peer.substr(0, colon).c_str(), &a.sin_addr) != 1 || a.sin_port == 0) return nullptr;
    std::unique_ptr<PeerConn> pc(new PeerConn());
    pc->fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (pc->fd < 0) return nullptr;
    timeval tv{cfg_.peer_timeout_ms / 1000, (cfg_.peer_timeout_ms % 1000) * 1000};
    setsockopt(pc->fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    if (connect(pc->fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
      g_log.log(ub::kLogWarn, "peer %s: connect failed: %s", peer.c_str(), strerror(errno));
      return nullptr;
    }
    int one = 1;
    setsockopt(pc->fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    std::string err;
    pc->conn = ub::SecureConn::client(pc->fd, cfg_.sec, cfg_.peer_timeout_ms, &err);
    if (!pc->conn) {
      g_log.log(ub::kLogWarn, "peer %s: TLS handshake failed: %s", peer.c_str(), err.c_str());
      return nullptr;
    }
    pc->last_used_ns = ub::now_ns();
    g_log.log(ub::kLogInfo, "peer %s: connected (%s)", peer.c_str(), pc->conn->cipher());
    return pc;
  }
  const Config& cfg_;
  std::mutex mu_;
  std::map<std::string, std::unique_ptr<PeerConn>> pool_;
};

// ---------------------------------------------------------------------------------------------- agent
struct Agent {
  Config cfg;
  TokenTable table;
  PeerPool pool;
  int tls_fd = -1, unix_fd = -1;
  int tls_port = 0;
  std::atomic<int> serving{0};
  explicit Agent(const Config& c) : cfg(c), table(c.max_tokens), pool(cfg) {}
};

// One inbound agent connection: TLS handshake, then GET records until the peer hangs up or the daemon stops.
void serve_peer(Agent* ag, int fd) {
  ++ag->serving;
  std::string err;
  std::unique_ptr<ub::SecureConn> conn = ub::SecureConn::server(fd, ag->cfg.sec, ag->cfg.peer_timeout_ms, &err);
  if (!conn) {
    ++g_st.tls_rejected;
    g_log.log(ub::kLogWarn, "inbound agent connection refused: %s", err.c_str());
  } else {
    ++g_st.tls_accepted;
    while (!g_stop.load()) {
      if (!conn->pending()) {   // wait in short steps so that a stop request is seen
        pollfd pf{fd, POLLIN, 0};
        if (poll(&pf, 1, 500) <= 0) continue;
      }
      ums_agent_msg_t m;
      if (!conn->read_full(&m, sizeof(m), ag->cfg.peer_timeout_ms)) break;   // hung up, or stalled inside a record
      ums_agent_msg_t r{};
      r.magic = UMS_AGENT_MAGIC;
      r.op = m.op;
      r.token_id = m.token_id;
      if (m.magic != UMS_AGENT_MAGIC || m.op != UMS_AGENT_GET) {
        r.status = UMS_AGENT_EINVAL;   // other agents may only read
      } else {
        r.status = static_cast<uint32_t>(ag->table.get(m.token_id, r.value, &r.len));
        ++g_st.gets_served;
        if (r.status != UMS_AGENT_OK) ++g_st.misses;
      }
      if (!conn->write_full(&r, sizeof(r))) break;
    }
  }
  conn.reset();
  close(fd);
  --ag->serving;
}

void tls_accept_loop(Agent* ag) {
  while (!g_stop.load()) {
    pollfd pf{ag->tls_fd, POLLIN, 0};
    if (poll(&pf, 1, 200) <= 0) continue;
    const int fd = accept4(ag->tls_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (fd < 0) continue;
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    std::thread(serve_peer, ag, fd).detach();
  }
}

void handle_local(Agent* ag, const ums_agent_msg_t& m, ums_agent_msg_t* r) {
  memset(r, 0, sizeof(*r));
  r->magic = UMS_AGENT_MAGIC;
  r->op = m.op;
  r->token_id = m.token_id;
  if (m.magic != UMS_AGENT_MAGIC || m.len > UMS_AGENT_MAX_VALUE) {
    r->status = UMS_AGENT_EINVAL;
    return;
  }
  switch (m.op) {
    case UMS_AGENT_PUT:
      r->status = m.len ? static_cast<uint32_t>(ag->table.put(m.token_id, m.value, m.len)) : UMS_AGENT_EINVAL;
      ++g_st.puts;
      break;
    case UMS_AGENT_DEL:
      r->status = static_cast<uint32_t>(ag->table.del(m.token_id));
      ++g_st.dels;
      break;
    case UMS_AGENT_GET: {
      const std::string peer(m.peer, strnlen(m.peer, sizeof(m.peer)));
      if (peer.empty()) {
        r->status = static_cast<uint32_t>(ag->table.get(m.token_id, r->value, &r->len));
        ++g_st.gets_local;
      } else {
        // The forward runs inside the main loop: a peer that does not answer holds up the other local requests for
        // at most peer_timeout_ms (connect, handshake and reply each have that limit). Inbound agent connections are
        // served by their own threads, so two agents that ask each other at the same time do not wait on one another.
        ums_agent_msg_t q = m;
        const int st = ag->pool.fetch(peer, &q);
        ++g_st.gets_forwarded;
        r->status = static_cast<uint32_t>(st);
        if (st == UMS_AGENT_OK) {
          r->len = q.len;
          memcpy(r->value, q.value, q.len);
        } else if (st == UMS_AGENT_EPEER) {
          ++g_st.peer_errors;
        }
      }
      if (r->status == UMS_AGENT_ENOENT) ++g_st.misses;
      break;
    }
    case UMS_AGENT_STATS: {
      char text[UMS_AGENT_MAX_VALUE];
      const int n = snprintf(text, sizeof(text), "tok %zu put %llu del %llu get %llu fwd %llu srv %llu miss %llu perr %llu tls %llu/%llu pool %zu/%llu/%llu",
                             ag->table.size(), (unsigned long long)g_st.puts.load(), (unsigned long long)g_st.dels.load(),
                             (unsigned long long)g_st.gets_local.load(), (unsigned long long)g_st.gets_forwarded.load(),
                             (unsigned long long)g_st.gets_served.load(), (unsigned long long)g_st.misses.load(),
                             (unsigned long long)g_st.peer_errors.load(), (unsigned long long)g_st.tls_accepted.load(),
                             (unsigned long long)g_st.tls_rejected.load(), ag->pool.size(),
                             (unsigned long long)g_st.pool_connects.load(), (unsigned long long)g_st.pool_reuses.load());
      r->len = static_cast<uint32_t>(n < 0 ? 0 : (n >= (int)sizeof(text) ? sizeof(text) - 1 : n));
      memcpy(r->value, text, r->len);
      break;
    }
    default:
      r->status = UMS_AGENT_EINVAL;
  }
}

int fail(const char* what) {
  fprintf(stderr, "ums_agent: %s\n", what);
  return 1;
}

}  // namespace

int main(int argc, char** argv) {
  Config cfg;
  std::string err;
  bool bad_env = false;
  cfg.sec = ub::PskConfig::from_env("UMS_AGENT", &bad_env);
  if (bad_env) return fail("malformed UMS_AGENT_PSK or incomplete UMS_AGENT_TLS_* in the environment");
  for (int i = 1; i < argc; ++i)   // the file first, so that options override it
    if (!strcmp(argv[i], "--config") && i + 1 < argc && !load_config(&cfg, argv[i + 1], &err)) return fail(err.c_str());
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--config") && i + 1 < argc) ++i;
    else if (!strcmp(argv[i], "--sock") && i + 1 < argc) cfg.sock = argv[++i];
    else if (!strcmp(argv[i], "--ip") && i + 1 < argc) cfg.ip = argv[++i];
    else if (!strcmp(argv[i], "--port") && i + 1 < argc) cfg.port = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--syslog")) cfg.use_syslog = true;
    else if (!strcmp(argv[i], "--insecure")) cfg.insecure = true;
    else return fail("usage: ums_agent [--config FILE] [--sock PATH] [--ip ADDR] [--port N] [--syslog] [--insecure]");
  }
  const int files = !cfg.sec.ca_file.empty() + !cfg.sec.cert_file.empty() + !cfg.sec.key_file.empty();
  if (files != 0 && files != 3) return fail("tls_ca, tls_cert and tls_key go together");
  if (!cfg.sec.enabled() && !cfg.insecure) return fail("no key or certificates configured (give --insecure to run in the clear)");
  if (cfg.use_syslog) openlog("ums_agent", LOG_PID, LOG_DAEMON);
  g_log.configure(cfg.log_level, cfg.use_syslog ? syslog_sink : nullptr);

  // signals arrive through a descriptor of the main loop; blocked here so that every thread inherits the mask
  sigset_t mask;
  sigemptyset(&mask);
  sigaddset(&mask, SIGTERM);
  sigaddset(&mask, SIGINT);
  pthread_sigmask(SIG_BLOCK, &mask, nullptr);
  signal(SIGPIPE, SIG_IGN);
  const int sig_fd = signalfd(-1, &mask, SFD_CLOEXEC | SFD_NONBLOCK);

  Agent ag(cfg);
  ag.tls_fd = socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  int one = 1;
  setsockopt(ag.tls_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(static_cast<uint16_t>(cfg.port));
  if (inet_pton(AF_INET, cfg.ip.c_str(), &a.sin_addr) != 1) return fail("bad listen address");
  if (bind(ag.tls_fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0 || listen(ag.tls_fd, 64) != 0)
    return fail("cannot listen on the agent port");
  socklen_t alen = sizeof(a);
  getsockname(ag.tls_fd, reinterpret_cast<sockaddr*>(&a), &alen);
  ag.tls_port = ntohs(a.sin_port);

  sockaddr_un ua{};
  ua.sun_family = AF_UNIX;
  if (cfg.sock.size() >= sizeof(ua.sun_path)) return fail("socket path too long");
  snprintf(ua.sun_path, sizeof(ua.sun_path), "%s", cfg.sock.c_str());
  unlink(cfg.sock.c_str());
  ag.unix_fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
  if (bind(ag.unix_fd, reinterpret_cast<sockaddr*>(&ua), sizeof(ua)) != 0 || listen(ag.unix_fd, 64) != 0)
    return fail("cannot listen on the local socket");
  chmod(cfg.sock.c_str(), 0600);   // token values are for this user's endpoints only

  std::thread tls_thr(tls_accept_loop, &ag);
  const int ep = epoll_create1(EPOLL_CLOEXEC);
  auto watch = [&](int fd) {
    epoll_event ev{};
    ev.events = EPOLLIN;
    ev.data.fd = fd;
    epoll_ctl(ep, EPOLL_CTL_ADD, fd, &ev);
  };
  watch(ag.unix_fd);
  watch(sig_fd);
  printf("ums_agent: listening on %s:%d, local socket %s, %s\n", cfg.ip.c_str(), ag.tls_port, cfg.sock.c_str(),
         cfg.sec.use_certs() ? "certificates" : (cfg.sec.enabled() ? "pre-shared key" : "CLEAR TEXT"));
  fflush(stdout);
  g_log.log(ub::kLogNotice, "started: port %d, socket %s", ag.tls_port, cfg.sock.c_str());

  std::unordered_map<int, std::vector<uint8_t>> partial;   // local connections -> bytes of the record so far
  while (!g_stop.load()) {
    epoll_event evs[32];
    const int n = epoll_wait(ep, evs, 32, 500);
    for (int i = 0; i < n; ++i) {
      const int fd = evs[i].data.fd;
      if (fd == sig_fd) {
        signalfd_siginfo si;
        if (read(sig_fd, &si, sizeof(si)) == sizeof(si)) {
          g_log.log(ub::kLogNotice, "signal %u: stopping", si.ssi_signo);
          g_stop = true;
        }
      } else if (fd == ag.unix_fd) {
        const int c = accept4(ag.unix_fd, nullptr, nullptr, SOCK_CLOEXEC | SOCK_NONBLOCK);
        if (c >= 0) {
          watch(c);
          partial[c];
        }
      } else {
        std::vector<uint8_t>& buf = partial[fd];
        uint8_t tmp[sizeof(ums_agent_msg_t)];
        const ssize_t r = recv(fd, tmp, sizeof(ums_agent_msg_t) - buf.size(), 0);
        bool drop = r == 0 || (r < 0 && errno != EAGAIN && errno != EINTR);
        if (r > 0) buf.insert(buf.end(), tmp, tmp + r);
        if (buf.size() == sizeof(ums_agent_msg_t)) {
          ums_agent_msg_t m, rsp;
          memcpy(&m, buf.data(), sizeof(m));
          buf.clear();
          handle_local(&ag, m, &rsp);
          // replies are one small record: a local client that does not read it is dropped, not waited for
          if (send(fd, &rsp, sizeof(rsp), MSG_NOSIGNAL) != (ssize_t)sizeof(rsp)) drop = true;
        }
        if (drop) {
          epoll_ctl(ep, EPOLL_CTL_DEL, fd, nullptr);
          close(fd);
          partial.erase(fd);
        }
      }
    }
  }
  tls_thr.join();
  for (int i = 0; i < 100 && ag.serving.load() > 0; ++i) usleep(10000);   // inbound connections see g_stop within 0.5 s
  for (auto& kv : partial) close(kv.first);
  close(ag.unix_fd);
  close(ag.tls_fd);
  close(ep);
  close(sig_fd);
  unlink(cfg.sock.c_str());
  g_log.log(ub::kLogNotice, "stopped");
  if (cfg.use_syslog) closelog();
  printf("ums_agent: stopped\n");
  return 0;
}
