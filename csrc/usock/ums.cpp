// UMS implementation (see ums.h).
#include "ums.h"
#include "ums_agent_proto.h"

#include "ub_secure.h"
#include "ub_util.h"
#include "ums_shm.h"

#include <arpa/inet.h>
#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <memory>
#include <mutex>
#include <vector>
#include <string>
#include <thread>
#include <unordered_map>

namespace {

using namespace ums_shm;

// The real libc entry points. When the preload shim is active, plain calls from this library would be interposed by
// the shim and come straight back here, so the library always goes through RTLD_NEXT.
struct Libc {
  int (*socket)(int, int, int);
  int (*listen)(int, int);
  int (*accept)(int, struct sockaddr*, socklen_t*);
  int (*connect)(int, const struct sockaddr*, socklen_t);
  ssize_t (*send)(int, const void*, size_t, int);
  ssize_t (*recv)(int, void*, size_t, int);
  int (*shutdown)(int, int);
  int (*close)(int);
  Libc() {
    // Resolve directly inside libc: this library may sit after libc in the lookup order (it is pulled in as a
    // dependency of the preload shim), in which case RTLD_NEXT would find nothing.
    void* h = dlopen("libc.so.6", RTLD_LAZY | RTLD_NOLOAD);
    if (!h) h = dlopen("libc.so.6", RTLD_LAZY);
    auto sym = [&](const char* n) {
      void* p = h ? dlsym(h, n) : nullptr;
      return p ? p : dlsym(RTLD_NEXT, n);
    };
    socket = reinterpret_cast<decltype(socket)>(sym("socket"));
    listen = reinterpret_cast<decltype(listen)>(sym("listen"));
    accept = reinterpret_cast<decltype(accept)>(sym("accept"));
    connect = reinterpret_cast<decltype(connect)>(sym("connect"));
    send = reinterpret_cast<decltype(send)>(sym("send"));
    recv = reinterpret_cast<decltype(recv)>(sym("recv"));
    shutdown = reinterpret_cast<decltype(shutdown)>(sym("shutdown"));
    close = reinterpret_cast<decltype(close)>(sym("close"));
  }
};
const Libc& libc() {
  static const Libc l;
  return l;
}

constexpr uint32_t kNoSlot = 0xffffffffu;
struct Clc {
  uint32_t magic;
  uint32_t accept;  // reply: 1 = accelerated, 0 = declined
  uint32_t slot;    // kNoSlot: shm_name is a file for this connection alone; else a link file and the slot in it
  uint32_t first;   // 1: this is the link's first connection (the server confirms the link)
  char shm_name[64];
  uint64_t nonce;   // with a pre-shared key: random per message
  uint8_t tag[16];  // AES-256-GCM tag over everything above (key derived from UMS_PSK), else zero
};
constexpr size_t kClcSigned = offsetof(Clc, tag);

// Handshake authentication. The reference's ums_agent carries the ring tokens of two hosts over a TLS connection of
// its own (ums_agent_tls_conn.c, ums_agent_token_proxy.c); here both ends are on one host and the token is the name
// of the ring file, so the handshake message itself is authenticated with a key derived from a pre-shared secret
// (UMS_PSK, hex). A message whose tag does not verify is treated like a peer that declined: the connection stays on
// TCP and is counted in conns_auth_fail.
struct ClcAuth {
  bool on = false, bad = false;
  uint8_t key[32];
  ClcAuth() {
    const ub::PskConfig cfg = ub::PskConfig::from_env("UMS", &bad);
    on = cfg.enabled() && ub::derive_key(cfg, "ums-clc", "ums", 3, key);
  }
};
const ClcAuth& clc_auth() {
  static const ClcAuth a;
  return a;
}
void clc_sign(Clc* m, bool from_server) {
  memset(m->tag, 0, sizeof(m->tag));
  m->nonce = 0;
  const ClcAuth& a = clc_auth();
  if (!a.on) return;
  ub::random_bytes(&m->nonce, sizeof(m->nonce));
  ub::AeadCipher c(a.key, from_server ? 1u : 0u);
  c.seal(m->nonce, m, kClcSigned, nullptr, 0, m->tag);
}
bool clc_verify(const Clc& m, bool from_server) {
  const ClcAuth& a = clc_auth();
  if (a.bad) return false;          // a malformed key never authenticates anything
  if (!a.on) return true;
  ub::AeadCipher c(a.key, from_server ? 1u : 0u);
  uint8_t none = 0;
  return c.open(m.nonce, &m, kClcSigned, m.tag, sizeof(m.tag), &none);
}

// Token exchange through the agents (ums_agent): with UMS_AGENT_SOCK and UMS_AGENT_ADDR (the "ip:port" other agents
// reach this host's agent on) a connecting endpoint stores the ring name with its agent and sends only
// "@<token id>@<agent address>"; the accepting endpoint has its own agent fetch the name over the agents' TLS
// connection. The name itself never travels on the application's connection
// (the reference: ums_agent_token_proxy.c, token request on connection setup).
bool agent_mode_tx() {
  const char* s = getenv("UMS_AGENT_SOCK");
  const char* a = getenv("UMS_AGENT_ADDR");
  return s && *s && a && *a && strlen(a) < 40;
}
// Replaces an "@id@addr" reference by the ring name; false when it cannot be resolved.
bool agent_resolve(char name[64]) {
  if (name[0] != '@') return true;
  const char* s = getenv("UMS_AGENT_SOCK");
  if (!s || !*s) return false;
  char* end = nullptr;
  const uint64_t id = strtoull(name + 1, &end, 16);
  if (!end || *end != '@' || !end[1]) return false;
  char value[UMS_AGENT_MAX_VALUE];
  uint32_t len = sizeof(value);
  if (ums_agent_get(nullptr, end + 1, id, value, &len) != 0 || len == 0 || len >= 64) return false;
  memcpy(name, value, len);
  name[len] = 0;
  return true;
}

// One mapped link file (see ums_shm.h). `owner` = this process created it (the connecting side).
struct Link {
  std::string name, path, group;
  LinkShm* shm = nullptr;
  bool owner = false;
  uint32_t local_conns = 0;
  uint64_t empty_since_ms = 0;
  uint32_t test_sent = 0;
  std::atomic<uint32_t> test_acked{0};
  std::atomic<bool> confirmed{false};
  bool deleted_by_peer = false;
};
// Receive moderation of one connection: how long recv busy-polls before it sleeps on the descriptor. The budget
// moves between fixed levels according to how the last samples ended, like the moderation profiles of the
// reference's dynamic interrupt moderation (src/usock/ums/kmod/ums/dim/ums_dim.c).
struct Dim {
  std::atomic<uint32_t> level{2};
  std::atomic<uint32_t> samples{0}, slept{0}, late{0};
};
constexpr uint32_t kDimSpins[5] = {0, 500, 4000, 16000, 64000};
struct Conn {
  bool accelerated = false;
  bool listener = false;
  uint16_t port = 0;
  ConnShm* shm = nullptr;
  Ring* tx = nullptr;
  Ring* rx = nullptr;
  std::string shm_path;
  bool owner = false;
  std::shared_ptr<Link> link;   // set when the connection lives in a slot of a link
  uint32_t slot = kNoSlot;
  std::shared_ptr<Dim> dim;
};
// Heap-allocated on first use and never destroyed: the preload shim can call into this library before its static
// constructors ran (during process start-up) and after its destructors ran (during exit).
struct State {
  std::mutex mu;
  std::unordered_map<int, Conn> conns;
  // Moves whenever `conns` changes (under mu). A thread keeps a copy of the connection it used last together with
  // the value it saw: while the two agree the copy is the table's entry, and send / recv need no lock at all.
  std::atomic<uint64_t> conns_gen{1};
  ums_stats_t stats{};
  std::unordered_map<std::string, std::shared_ptr<Link>> links;                 // every mapped link, by role ("c:" created here, "s:" accepted here) and name
  std::unordered_map<std::string, std::vector<std::shared_ptr<Link>>> groups;   // links this process owns, by server
};
State& state() {
  static State* s = new State();
  return *s;
}
#define g_mu (state().mu)
#define g_conns (state().conns)
#define g_links (state().links)
#define g_groups (state().groups)
#define g_stats (state().stats)
// Counters are bumped from every thread that sends or receives: relaxed atomic adds, never under a lock of their own.
inline void stat_add(uint64_t& f, uint64_t n = 1) { __atomic_fetch_add(&f, n, __ATOMIC_RELAXED); }
std::atomic<uint64_t> g_seq{1};

std::string dir() {
  const char* e = getenv("UMS_SHM_DIR");
  std::string d = (e && *e) ? e : "/dev/shm/ums_" + std::to_string(getuid());
  mkdir(d.c_str(), 0700);
  return d;
}
std::string listen_marker(uint16_t port) { return dir() + "/listen_" + std::to_string(port); }

// How long an accepted loopback connection may stay silent before it is taken for an ordinary TCP client
// (UMS_PEEK_MS, default 50: a UMS client sends its handshake right after connect()).
int peek_limit_ms() {
  static const int v = [] {
    const char* e = getenv("UMS_PEEK_MS");
    const int x = e ? atoi(e) : 50;
    return x < 0 ? 0 : (x > 2000 ? 2000 : x);
  }();
  return v;
}

bool rd_full(int fd, void* b, size_t n, int tmo_ms) {
  char* p = static_cast<char*>(b);
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    if (poll(&pf, 1, tmo_ms) <= 0) return false;
    const ssize_t r = libc().recv(fd, p, n, 0);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}
bool wr_full(int fd, const void* b, size_t n) {
  const char* p = static_cast<const char*>(b);
  while (n) {
    const ssize_t r = libc().send(fd, p, n, MSG_NOSIGNAL);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}

Conn* find(int fd) {
  auto it = g_conns.find(fd);
  return it == g_conns.end() ? nullptr : &it->second;
}
inline void conns_changed() { state().conns_gen.fetch_add(1, std::memory_order_release); }   // caller holds g_mu
// The data calls' view of a descriptor: known = the table has it. Served from the calling thread's copy while the
// table has not changed since the copy was made.
struct ConnView {
  int fd = -1;
  uint64_t gen = 0;
  bool known = false;
  Conn c;
};
const ConnView& lookup(int fd) {
  static thread_local ConnView v;
  const uint64_t gen = state().conns_gen.load(std::memory_order_acquire);
  if (v.fd == fd && v.gen == gen) return v;
  std::lock_guard<std::mutex> l(g_mu);
  v.gen = state().conns_gen.load(std::memory_order_relaxed);
  v.fd = fd;
  Conn* p = find(fd);
  v.known = p != nullptr;
  v.c = p ? *p : Conn();
  return v;
}

size_t ring_write(Ring* r, const char* src, size_t n) {
  const uint64_t prod = r->prod.load(std::memory_order_relaxed);
  const uint64_t cons = r->cons.load(std::memory_order_acquire);
  const size_t space = kRingBytes - static_cast<size_t>(prod - cons);
  const size_t k = n < space ? n : space;
  if (k == 0) return 0;
  const size_t off = prod % kRingBytes;
  const size_t first = k < kRingBytes - off ? k : kRingBytes - off;
  memcpy(r->data + off, src, first);
  memcpy(r->data, src + first, k - first);
  r->prod.store(prod + k, std::memory_order_release);
  return k;
}
size_t ring_read(Ring* r, char* dst, size_t n, bool peek) {
  const uint64_t cons = r->cons.load(std::memory_order_relaxed);
  const uint64_t prod = r->prod.load(std::memory_order_acquire);
  const size_t avail = static_cast<size_t>(prod - cons);
  const size_t k = n < avail ? n : avail;
  if (k == 0) return 0;
  const size_t off = cons % kRingBytes;
  const size_t first = k < kRingBytes - off ? k : kRingBytes - off;
  memcpy(dst, r->data + off, first);
  memcpy(dst + first, r->data, k - first);
  if (!peek) r->cons.store(cons + k, std::memory_order_release);
  return k;
}

bool nonblocking(int fd) { return (fcntl(fd, F_GETFL) & O_NONBLOCK) != 0; }

}  // namespace

extern "C" {

// One receive that found the ring empty has ended: by catching data while polling (late = in the second half of the
// budget) or by going to sleep. Every 32 samples the level moves: mostly sleeps -> poll less (the peer is slow, the
// cycles are wasted), mostly late catches -> poll longer (a little more patience saves the sleep and the doorbell).
void dim_sample(Dim* d, uint32_t level, bool caught, bool late) {
  if (!caught) d->slept.fetch_add(1, std::memory_order_relaxed);
  else if (late) d->late.fetch_add(1, std::memory_order_relaxed);
  if (d->samples.fetch_add(1, std::memory_order_relaxed) + 1 < 32) return;
  const uint32_t slept = d->slept.exchange(0), lt = d->late.exchange(0);
  d->samples.store(0);
  uint32_t next = level;
  if (slept >= 24 && level > 0) next = level - 1;
  else if (slept + lt >= 12 && slept < 12 && level < 4) next = level + 1;
  if (next != level && d->level.compare_exchange_strong(level, next)) {
    if (next > level) stat_add(g_stats.dim_up);
    else stat_add(g_stats.dim_down);
  }
}

// ------------------------------------------------------------------------------------------------ link groups
uint64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
bool link_groups_on() {
  static const bool v = [] {
    const char* e = getenv("UMS_LINK_GROUP");
    return !(e && e[0] == '0');
  }();
  return v;
}
// How long a link without connections is kept for the next connection before its file is removed.
uint64_t linger_ms() {
  static const uint64_t v = [] {
    const char* e = getenv("UMS_LINK_LINGER_MS");
    const long x = e ? atol(e) : 1000;
    return static_cast<uint64_t>(x < 0 ? 0 : x);
  }();
  return v;
}
// Maps a link file. create: make it (exclusive) and write the header; else it must be a regular file of this user
// and of exactly the link size that carries the link magic.
std::shared_ptr<Link> link_map(const std::string& name, bool create) {
  const std::string path = dir() + "/" + name;
  const int fd = create ? ::open(path.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600) : ::open(path.c_str(), O_RDWR | O_NOFOLLOW);
  if (fd < 0) return nullptr;
  void* p = MAP_FAILED;
  if (create) {
    if (ftruncate(fd, sizeof(LinkShm)) == 0) p = mmap(nullptr, sizeof(LinkShm), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  } else {
    struct stat sb{};
    if (fstat(fd, &sb) == 0 && S_ISREG(sb.st_mode) && sb.st_uid == geteuid() && sb.st_size == (off_t)sizeof(LinkShm))
      p = mmap(nullptr, sizeof(LinkShm), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  }
  libc().close(fd);
  if (p == MAP_FAILED) {
    if (create) unlink(path.c_str());
    return nullptr;
  }
  LinkShm* shm = static_cast<LinkShm*>(p);
  if (create) {   // a new file is all zero: cursors, bitmaps and state start from there
    shm->magic = kLinkMagic;
    shm->version = 1;
    shm->owner_pid = static_cast<uint32_t>(getpid());
    shm->slots = kLinkSlots;
  } else if (shm->magic != kLinkMagic || shm->slots != kLinkSlots) {
    munmap(p, sizeof(LinkShm));
    return nullptr;
  }
  auto l = std::make_shared<Link>();
  l->name = name;
  l->path = path;
  l->shm = shm;
  l->owner = create;
  return l;
}
// Control messages. One process is the only producer of a ring (serialised by g_mu, which the caller holds).
bool llc_push(Link* l, uint32_t type, uint32_t flags, uint32_t seq, uint32_t slot, const char* name = nullptr) {
  LlcRing& r = l->owner ? l->shm->llc_c2s : l->shm->llc_s2c;
  const uint64_t prod = r.prod.load(std::memory_order_relaxed);
  if (prod - r.cons.load(std::memory_order_acquire) >= kLlcEntries) return false;   // the peer is not reading
  LlcMsg& m = r.msg[prod % kLlcEntries];
  m.type = type;
  m.flags = flags;
  m.seq = seq;
  m.slot = slot;
  memset(m.name, 0, sizeof(m.name));
  if (name) snprintf(m.name, sizeof(m.name), "%s", name);
  r.prod.store(prod + 1, std::memory_order_release);
  stat_add(g_stats.llc_tx);
  return true;
}
bool llc_has_input(Link* l) {
  LlcRing& r = l->owner ? l->shm->llc_s2c : l->shm->llc_c2s;
  return r.prod.load(std::memory_order_acquire) != r.cons.load(std::memory_order_relaxed);
}
// Handles what the peer put on this side's control ring. Caller holds g_mu.
void llc_progress(Link* l) {
  LlcRing& r = l->owner ? l->shm->llc_s2c : l->shm->llc_c2s;
  for (;;) {
    const uint64_t cons = r.cons.load(std::memory_order_relaxed);
    if (cons == r.prod.load(std::memory_order_acquire)) return;
    const LlcMsg m = r.msg[cons % kLlcEntries];
    r.cons.store(cons + 1, std::memory_order_release);
    stat_add(g_stats.llc_rx);
    const bool rsp = (m.flags & kLlcResponse) != 0;
    switch (m.type) {
      case LLC_CONFIRM_LINK:
        if (!rsp) llc_push(l, LLC_CONFIRM_LINK, kLlcResponse, m.seq, 0);
        l->confirmed = true;
        l->shm->state.store(LINK_ACTIVE);
        break;
      case LLC_ADD_LINK:   // a further link of the group: map it now, its first connection finds it ready
        if (!rsp && !l->owner) {
          char nm[sizeof(m.name) + 1] = {0};
          memcpy(nm, m.name, sizeof(m.name));
          if (!strchr(nm, '/') && !g_links.count(std::string("s:") + nm)) {
            if (auto nl = link_map(nm, false)) {
              nl->group = l->group;
              nl->empty_since_ms = now_ms();
              g_links[std::string("s:") + nm] = nl;
              stat_add(g_stats.links_created);
            }
          }
          llc_push(l, LLC_ADD_LINK, kLlcResponse, m.seq, 0);
        }
        break;
      case LLC_DELETE_LINK:
        if (!l->owner) l->deleted_by_peer = true;
        break;
      case LLC_TEST_LINK:
        if (!rsp) {
          llc_push(l, LLC_TEST_LINK, kLlcResponse, m.seq, 0);
        } else {
          l->test_acked = m.seq;
          stat_add(g_stats.link_tests_ok);
        }
        break;
      default: break;   // DELETE_CONN is a notice
    }
  }
}
// Frees links that have had no connection for the linger time. Caller holds g_mu.
void reap_links() {
  const uint64_t now = now_ms();
  for (auto it = g_links.begin(); it != g_links.end();) {
    Link* l = it->second.get();
    bool drop = false;
    if (l->local_conns == 0) {
      if (l->owner) {
        drop = now - l->empty_since_ms >= linger_ms();
        if (drop) {
          l->shm->state.store(LINK_DELETED);
          llc_push(l, LLC_DELETE_LINK, 0, 0, 0);
          unlink(l->path.c_str());
        }
      } else {
        llc_progress(l);
        drop = l->deleted_by_peer || l->shm->state.load() == LINK_DELETED || access(l->path.c_str(), F_OK) != 0;
      }
    }
    if (!drop) {
      ++it;
      continue;
    }
    for (auto& g : g_groups) {
      auto& v = g.second;
      for (size_t i = 0; i < v.size(); ++i)
        if (v[i].get() == l) {
          v.erase(v.begin() + i);
          break;
        }
    }
    munmap(l->shm, sizeof(LinkShm));
    l->shm = nullptr;
    stat_add(g_stats.links_freed);
    it = g_links.erase(it);
  }
}
// Client side: a slot for a new connection to the server named by `key`, on an existing link of the group or on a
// new one. Caller holds g_mu.
std::shared_ptr<Link> link_pick(const std::string& key, uint64_t salt, uint32_t* slot, uint32_t* first) {
  reap_links();
  auto& grp = g_groups[key];
  for (auto& l : grp) {
    if (l->shm->state.load() == LINK_DELETED) continue;
    const uint32_t used = l->shm->slot_used.load();
    const uint32_t done = l->shm->closed_c.load() & l->shm->closed_s.load();   // both sides closed: reusable
    for (uint32_t i = 0; i < kLinkSlots; ++i) {
      const uint32_t bit = 1u << i;
      if ((used & bit) && !(done & bit)) continue;
      ConnShm& c = l->shm->conn[i];
      for (Ring* r : {&c.c2s, &c.s2c}) {
        r->prod.store(0);
        r->cons.store(0);
        r->closed.store(0);
        r->waiter.store(0);
      }
      l->shm->closed_c.fetch_and(~bit);
      l->shm->closed_s.fetch_and(~bit);
      l->shm->slot_used.fetch_or(bit);
      *slot = i;
      *first = l->confirmed.load() ? 0 : 1;
      return l;
    }
  }
  // every slot of every link is taken (or there is no link yet): one more link for the group
  char name[64];
  snprintf(name, sizeof(name), "lg_%d_%llu_%016llx", getpid(), (unsigned long long)g_seq.fetch_add(1),
           (unsigned long long)salt);
  auto l = link_map(name, true);
  if (!l) return nullptr;
  l->group = grp.empty() ? l->name : grp.front()->group;
  snprintf(l->shm->group, sizeof(l->shm->group), "%s", l->group.c_str());
  if (!grp.empty() && grp.front()->confirmed.load() && l->name.size() < sizeof(LlcMsg::name))
    llc_push(grp.front().get(), LLC_ADD_LINK, 0, 0, 0, l->name.c_str());   // announce it on the group's first link
  grp.push_back(l);
  g_links["c:" + l->name] = l;
  static const bool cleanup_registered = [] {
    // a process that exits with connections still open must not leave its link files behind
    atexit([] {
      std::lock_guard<std::mutex> lk(g_mu);
      for (auto& kv : g_links)
        if (kv.second->owner && kv.second->shm) {
          kv.second->shm->state.store(LINK_DELETED);
          unlink(kv.second->path.c_str());
        }
    });
    return true;
  }();
  (void)cleanup_registered;
  stat_add(g_stats.links_created);
  l->shm->slot_used.fetch_or(1u);
  *slot = 0;
  *first = 1;
  return l;
}
// Identity of the listener behind a loopback port: what its marker file holds (pid and a random token), so that a
// restarted server is a new peer and gets new links.
std::string server_key(uint16_t port) {
  char buf[96] = {0};
  const int fd = ::open(listen_marker(port).c_str(), O_RDONLY);
  if (fd >= 0) {
    const ssize_t n = pread(fd, buf, sizeof(buf) - 1, 0);   // (not read(): see ums_adopt_listener)
    if (n < 0) buf[0] = 0;
    libc().close(fd);
  }
  return std::to_string(port) + ":" + buf;
}

int ums_socket(int domain, int type, int protocol) {
  const int fd = libc().socket(domain, type, protocol);
  if (fd >= 0 && (domain == AF_INET || domain == AF_INET6) && (type & 0xf) == SOCK_STREAM) {
    std::lock_guard<std::mutex> l(g_mu);
    g_conns[fd] = Conn();
    conns_changed();
  }
  return fd;
}
int ums_bind(int fd, const struct sockaddr* addr, socklen_t len) { return ::bind(fd, addr, len); }

int ums_adopt_listener(int fd) {
  sockaddr_in a{};
  socklen_t l = sizeof(a);
  if (getsockname(fd, reinterpret_cast<sockaddr*>(&a), &l) != 0) return -1;
  // (random numbers are drawn before the lock is taken: the generator may open and close files, and under the
  // preload shim close() comes back into this library)
  uint64_t tok = 0;
  ub::random_bytes(&tok, sizeof(tok));
  std::lock_guard<std::mutex> lk(g_mu);
  Conn& c = g_conns[fd];
  conns_changed();
  c.listener = true;
  c.port = ntohs(a.sin_port);
  const int m = ::open(listen_marker(c.port).c_str(), O_CREAT | O_WRONLY | O_TRUNC, 0600);  // "this port speaks UMS"
  if (m >= 0) {   // who is listening: clients group their links by it
    char id[64];
    const int n = snprintf(id, sizeof(id), "%d:%016llx", getpid(), (unsigned long long)tok);
    // pwrite, not write: the preload shim routes write() back into this library, which would take the lock again
    if (pwrite(m, id, n, 0) < 0) {
      // an empty marker still says that the port speaks UMS
    }
    libc().close(m);
  }
  return 0;
}
int ums_listen(int fd, int backlog) {
  const int rc = libc().listen(fd, backlog);
  if (rc == 0) ums_adopt_listener(fd);
  return rc;
}

int ums_adopt_accepted(int listen_fd, int fd) {
  {
    std::lock_guard<std::mutex> l(g_mu);
    Conn* lc = find(listen_fd);
    if (!lc || !lc->listener) return 0;
  }
  // Server side of the handshake: a UMS client speaks first, but an ordinary TCP client (or a UMS client on another
  // host, which never sends the handshake) does not. So nothing is consumed until the stream is known to start with
  // the handshake magic: only loopback peers are candidates, their first bytes are PEEKED with a short limit, and
  // anything else leaves the byte stream untouched and falls back to TCP at once.
  Clc in{};
  Conn c;
  bool candidate = false;
  {
    sockaddr_storage ps{};
    socklen_t pl = sizeof(ps);
    if (getpeername(fd, reinterpret_cast<sockaddr*>(&ps), &pl) == 0 && ps.ss_family == AF_INET)
      candidate = (ntohl(reinterpret_cast<sockaddr_in*>(&ps)->sin_addr.s_addr) >> 24) == 127;
  }
  if (candidate) {
    candidate = false;
    const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(peek_limit_ms());
    for (;;) {
      uint32_t magic = 0;
      const ssize_t r = libc().recv(fd, &magic, sizeof(magic), MSG_PEEK | MSG_DONTWAIT);
      if (r == (ssize_t)sizeof(magic)) {
        candidate = magic == kClcMagic;
        break;
      }
      if (r == 0 || (r < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) break;
      if (r > 0 && memcmp(&magic, &kClcMagic, (size_t)r) != 0) break;   // already differs: not a handshake
      const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(t_end - std::chrono::steady_clock::now());
      if (left.count() <= 0) break;
      pollfd pf{fd, POLLIN, 0};
      if (r > 0) {
        // a partial magic is pending: POLLIN would return at once, so just yield briefly
        std::this_thread::sleep_for(std::chrono::microseconds(200));
      } else if (poll(&pf, 1, (int)left.count()) <= 0) {
        break;
      }
    }
  }
  if (candidate && rd_full(fd, &in, sizeof(in), 2000) && in.magic == kClcMagic) {
    Clc out{};
    out.magic = kClcMagic;
    in.shm_name[sizeof(in.shm_name) - 1] = 0;
    const bool trusted = clc_verify(in, false) && agent_resolve(in.shm_name) && !strchr(in.shm_name, '/');
    if (!trusted) {
      std::lock_guard<std::mutex> l(g_mu);
      stat_add(g_stats.conns_auth_fail);
    }
    const std::string path = dir() + "/" + in.shm_name;
    if (trusted && in.slot != kNoSlot) {   // a slot of a link: the link is mapped once, however many connections
      std::lock_guard<std::mutex> l(g_mu);
      reap_links();
      std::shared_ptr<Link> lk;
      // (both ends may live in one process: each role has its own mapping and its own entry)
      auto it = g_links.find(std::string("s:") + in.shm_name);
      if (it != g_links.end()) lk = it->second;
      else if ((lk = link_map(in.shm_name, false))) {
        lk->group = std::string(lk->shm->group, strnlen(lk->shm->group, sizeof(lk->shm->group)));
        g_links["s:" + lk->name] = lk;
        stat_add(g_stats.links_created);
      }
      if (lk && !lk->owner && in.slot < kLinkSlots && (lk->shm->slot_used.load() & (1u << in.slot)) &&
          lk->shm->state.load() != LINK_DELETED) {
        lk->shm->peer_pid.store(static_cast<uint32_t>(getpid()));
        if (!lk->confirmed.load()) llc_push(lk.get(), LLC_CONFIRM_LINK, 0, 1, in.slot);   // before the answer goes out
        llc_progress(lk.get());
        ++lk->local_conns;
        lk->shm->conns_total.fetch_add(1);
        out.accept = 1;
        out.slot = in.slot;
        c.accelerated = true;
        c.link = lk;
        c.slot = in.slot;
        c.shm = &lk->shm->conn[in.slot];
        c.tx = &c.shm->s2c;
        c.rx = &c.shm->c2s;
        c.dim = std::make_shared<Dim>();
        stat_add(g_stats.conns_on_links);
      }
    }
    const int sfd = (trusted && in.slot == kNoSlot) ? ::open(path.c_str(), O_RDWR | O_NOFOLLOW) : -1;
    void* p = MAP_FAILED;
    if (sfd >= 0) {
      // the ring file must be what a client of this user created: a regular file of exactly the ring size
      struct stat sb{};
      if (fstat(sfd, &sb) == 0 && S_ISREG(sb.st_mode) && sb.st_uid == geteuid() &&
          sb.st_size == (off_t)sizeof(ConnShm))
        p = mmap(nullptr, sizeof(ConnShm), PROT_READ | PROT_WRITE, MAP_SHARED, sfd, 0);
      libc().close(sfd);
    }
    if (p != MAP_FAILED) {
      out.accept = 1;
      out.slot = kNoSlot;
      c.accelerated = true;
      c.shm = static_cast<ConnShm*>(p);
      c.tx = &c.shm->s2c;
      c.rx = &c.shm->c2s;
      c.shm_path = path;
      c.dim = std::make_shared<Dim>();
    }
    clc_sign(&out, true);
    wr_full(fd, &out, sizeof(out));
  }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  std::lock_guard<std::mutex> l(g_mu);
  if (c.accelerated) stat_add(g_stats.conns_ums);
  else stat_add(g_stats.conns_fallback);
  g_conns[fd] = c;
  conns_changed();
  return c.accelerated ? 1 : 0;
}
int ums_accept(int fd, struct sockaddr* addr, socklen_t* len) {
  const int nfd = libc().accept(fd, addr, len);
  if (nfd >= 0) ums_adopt_accepted(fd, nfd);
  return nfd;
}

int ums_adopt_connected(int fd, const struct sockaddr* peer) {
  Conn c;
  const sockaddr_in* a = reinterpret_cast<const sockaddr_in*>(peer);
  bool try_ums = false;
  if (peer->sa_family == AF_INET && ntohl(a->sin_addr.s_addr) >> 24 == 127) {
    // same host: accelerate only if the listener announced itself, otherwise stay on plain TCP without touching
    // the byte stream (the peer may be an ordinary TCP server)
    try_ums = access(listen_marker(ntohs(a->sin_port)).c_str(), F_OK) == 0;
  }
  if (try_ums) {
    Clc out{};
    out.magic = kClcMagic;
    out.slot = kNoSlot;
    std::shared_ptr<Link> lk;
    void* p = MAP_FAILED;
    std::string path;
    if (link_groups_on()) {   // a slot on a link to that server (an existing link, or a new one for the group)
      uint64_t salt = 0;   // for the name of a new link file, drawn outside the lock (see ums_adopt_listener)
      ub::random_bytes(&salt, sizeof(salt));
      const std::string key = server_key(ntohs(a->sin_port));
      std::lock_guard<std::mutex> l(g_mu);
      lk = link_pick(key, salt, &out.slot, &out.first);
      if (lk) {
        ++lk->local_conns;
        snprintf(out.shm_name, sizeof(out.shm_name), "%s", lk->name.c_str());
      }
    }
    if (!lk) {   // a file for this connection alone
      out.slot = kNoSlot;
      uint64_t salt = 0;   // unguessable ring names: another local process cannot name a connection's ring file
      ub::random_bytes(&salt, sizeof(salt));
      snprintf(out.shm_name, sizeof(out.shm_name), "conn_%d_%llu_%016llx", getpid(),
               (unsigned long long)g_seq.fetch_add(1), (unsigned long long)salt);
      path = dir() + "/" + out.shm_name;
      const int sfd = ::open(path.c_str(), O_CREAT | O_RDWR | O_TRUNC, 0600);
      if (sfd >= 0 && ftruncate(sfd, sizeof(ConnShm)) == 0)
        p = mmap(nullptr, sizeof(ConnShm), PROT_READ | PROT_WRITE, MAP_SHARED, sfd, 0);
      if (sfd >= 0) libc().close(sfd);
    }
    uint64_t token_id = 0;
    bool token_stored = false;
    if (agent_mode_tx()) {   // the name goes to the agent, the message carries a reference to it
      ub::random_bytes(&token_id, sizeof(token_id));
      token_stored = ums_agent_put(nullptr, token_id, out.shm_name, static_cast<uint32_t>(strlen(out.shm_name))) == 0;
      if (token_stored)
        snprintf(out.shm_name, sizeof(out.shm_name), "@%llx@%s", (unsigned long long)token_id, getenv("UMS_AGENT_ADDR"));
      else
        out.shm_name[0] = 0;   // agent wanted but unreachable: the name is not sent in the clear; the peer declines
    }
    clc_sign(&out, false);
    const bool was_nb = nonblocking(fd);
    if (was_nb) fcntl(fd, F_SETFL, fcntl(fd, F_GETFL) & ~O_NONBLOCK);
    Clc in{};
    const bool answered = (lk || p != MAP_FAILED) && wr_full(fd, &out, sizeof(out)) &&
                          rd_full(fd, &in, sizeof(in), 2000) && in.magic == kClcMagic;
    const bool trusted = answered && clc_verify(in, true);
    if (token_stored) ums_agent_del(nullptr, token_id);   // one connection, one use
    if (answered && !trusted) {
      std::lock_guard<std::mutex> l(g_mu);
      stat_add(g_stats.conns_auth_fail);
    }
    if (trusted && in.accept && lk && in.slot == out.slot) {
      c.accelerated = true;
      c.link = lk;
      c.slot = out.slot;
      c.shm = &lk->shm->conn[out.slot];
      c.tx = &c.shm->c2s;
      c.rx = &c.shm->s2c;
      c.dim = std::make_shared<Dim>();
      std::lock_guard<std::mutex> l(g_mu);
      llc_progress(lk.get());   // the server's CONFIRM LINK came before its answer: reply, the link is ACTIVE
      stat_add(g_stats.conns_on_links);
    } else if (trusted && in.accept && !lk) {
      c.accelerated = true;
      c.shm = static_cast<ConnShm*>(p);
      c.tx = &c.shm->c2s;
      c.rx = &c.shm->s2c;
      c.shm_path = path;
      c.owner = true;
      c.dim = std::make_shared<Dim>();
    } else if (lk) {   // declined: the slot goes back
      std::lock_guard<std::mutex> l(g_mu);
      lk->shm->slot_used.fetch_and(~(1u << out.slot));
      if (--lk->local_conns == 0) lk->empty_since_ms = now_ms();
    } else if (p != MAP_FAILED) {
      munmap(p, sizeof(ConnShm));
      unlink(path.c_str());
    }
    if (was_nb) fcntl(fd, F_SETFL, fcntl(fd, F_GETFL) | O_NONBLOCK);
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  }
  std::lock_guard<std::mutex> l(g_mu);
  if (c.accelerated) stat_add(g_stats.conns_ums);
  else stat_add(g_stats.conns_fallback);
  g_conns[fd] = c;
  conns_changed();
  return c.accelerated ? 1 : 0;
}
int ums_connect(int fd, const struct sockaddr* addr, socklen_t len) {
  const int rc = libc().connect(fd, addr, len);
  if (rc == 0) ums_adopt_connected(fd, addr);
  return rc;
}

ssize_t ums_send(int fd, const void* buf, size_t n, int flags) {
  const ConnView& view = lookup(fd);
  const Conn& c = view.c;
  if (!c.accelerated) {
    if (view.known) stat_add(g_stats.bytes_tx_tcp, n);
    return libc().send(fd, buf, n, flags);
  }
  if (c.link && llc_has_input(c.link.get())) {   // control messages of the link are served from inside data calls
    std::lock_guard<std::mutex> l(g_mu);
    llc_progress(c.link.get());
  }
  if (c.tx->closed.load()) {
    errno = EPIPE;
    return -1;
  }
  const char* p = static_cast<const char*>(buf);
  size_t sent = 0;
  // (whether the descriptor is non-blocking is a system call to find out: asked only when the call would wait)
  int nb_state = (flags & MSG_DONTWAIT) ? 1 : -1;
  auto nb_now = [&]() {
    if (nb_state < 0) nb_state = nonblocking(fd) ? 1 : 0;
    return nb_state == 1;
  };
  uint32_t spins = 0;
  while (sent < n) {
    const uint64_t before = c.tx->prod.load(std::memory_order_relaxed);
    const size_t k = ring_write(c.tx, p + sent, n - sent);
    if (k) {
      sent += k;
      // The reader may have gone to sleep on the TCP descriptor if it had consumed everything that was published
      // before this write. Checking AFTER publishing closes the lost-wakeup window.
      std::atomic_thread_fence(std::memory_order_seq_cst);
      (void)before;
      if (c.tx->waiter.load(std::memory_order_relaxed)) {  // one byte makes the peer's descriptor readable
        const char bell = 1;
        if (libc().send(fd, &bell, 1, MSG_NOSIGNAL | MSG_DONTWAIT) < 0 && errno != EAGAIN && errno != EWOULDBLOCK) {
          if (sent) break;
          return -1;
        }
        stat_add(g_stats.doorbells);
      }
      spins = 0;
      continue;
    }
    if (nb_now()) {
      if (sent) break;
      errno = EAGAIN;
      return -1;
    }
    // ring full: wait for the reader; give up if the peer closed its TCP side
    if (++spins > 2000) {
      pollfd pf{fd, 0, 0};
      poll(&pf, 1, 1);
      if (pf.revents & (POLLHUP | POLLERR)) {
        errno = EPIPE;
        return sent ? (ssize_t)sent : -1;
      }
      stat_add(g_stats.tx_waits);
    } else {
      sched_yield();
    }
  }
  stat_add(g_stats.bytes_tx_ring, sent);
  return static_cast<ssize_t>(sent);
}

ssize_t ums_recv(int fd, void* buf, size_t n, int flags) {
  const ConnView& view = lookup(fd);
  const Conn& c = view.c;
  if (!c.accelerated) {
    const ssize_t r = libc().recv(fd, buf, n, flags);
    if (r > 0) stat_add(g_stats.bytes_rx_tcp, r);
    return r;
  }
  int nb_state = (flags & MSG_DONTWAIT) ? 1 : -1;   // found out (a system call) only when the ring is empty
  for (;;) {
    if (c.link && llc_has_input(c.link.get())) {
      std::lock_guard<std::mutex> l(g_mu);
      llc_progress(c.link.get());
    }
    size_t k = ring_read(c.rx, static_cast<char*>(buf), n, flags & MSG_PEEK);
    if (!k && nb_state < 0) nb_state = nonblocking(fd) ? 1 : 0;
    const bool nb = nb_state == 1;
    if (!k && !nb) {
      // short busy-poll before sleeping: a request/response partner usually answers within microseconds, and the
      // answer is then picked up without a system call on either side
      // The budget adapts (c.dim): polling that keeps ending in a sleep is shortened, polling that catches the data
      // only near the end of its budget is lengthened.
      const uint32_t level = c.dim ? c.dim->level.load(std::memory_order_relaxed) : 2;
      const uint32_t budget = kDimSpins[level];
      uint32_t spin = 0;
      for (; spin < budget && !k; ++spin) {
        ub::cpu_relax();
        k = ring_read(c.rx, static_cast<char*>(buf), n, flags & MSG_PEEK);
      }
      if (c.dim) dim_sample(c.dim.get(), level, k != 0, k != 0 && spin > budget / 2);
    }
    if (!k) {
      // announce that we are going to wait on the descriptor, then look once more (no lost wake-up)
      c.rx->waiter.store(1, std::memory_order_relaxed);
      std::atomic_thread_fence(std::memory_order_seq_cst);
      k = ring_read(c.rx, static_cast<char*>(buf), n, flags & MSG_PEEK);
    }
    if (k) {
      if (c.rx->waiter.load(std::memory_order_relaxed)) c.rx->waiter.store(0, std::memory_order_relaxed);
      stat_add(g_stats.bytes_rx_ring, k);
      return static_cast<ssize_t>(k);
    }
    // nothing in the ring: consume doorbells (or learn that the peer closed)
    char bells[64];
    const ssize_t r = libc().recv(fd, bells, sizeof(bells), nb ? MSG_DONTWAIT : 0);
    if (r == 0) {
      // orderly shutdown of the peer: deliver what is still in the ring, then end of stream
      const size_t k2 = ring_read(c.rx, static_cast<char*>(buf), n, flags & MSG_PEEK);
      return static_cast<ssize_t>(k2);
    }
    if (r < 0) {
      if (errno == EINTR) continue;
      if ((errno == EAGAIN || errno == EWOULDBLOCK) && c.rx->prod.load() != c.rx->cons.load()) continue;
      return -1;
    }
  }
}

int ums_shutdown(int fd, int how) {
  {
    std::lock_guard<std::mutex> l(g_mu);
    Conn* p = find(fd);
    if (p && p->accelerated && (how == SHUT_WR || how == SHUT_RDWR)) p->tx->closed = 1;
  }
  return libc().shutdown(fd, how);
}

int ums_close(int fd) {
  Conn c;
  bool known = false;
  {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_conns.find(fd);
    if (it != g_conns.end()) {
      c = it->second;
      known = true;
      g_conns.erase(it);
      conns_changed();
    }
  }
  if (known) {
    if (c.listener) unlink(listen_marker(c.port).c_str());
    if (c.accelerated && c.link) {
      // the slot becomes reusable once both sides have closed; the link itself lingers for the next connection
      c.tx->closed = 1;
      std::lock_guard<std::mutex> l(g_mu);
      Link* lk = c.link.get();
      if (lk->shm) {
        (lk->owner ? lk->shm->closed_c : lk->shm->closed_s).fetch_or(1u << c.slot);
        llc_push(lk, LLC_DELETE_CONN, 0, 0, c.slot);
        llc_progress(lk);
        if (lk->local_conns && --lk->local_conns == 0) lk->empty_since_ms = now_ms();
      }
      reap_links();
    } else if (c.accelerated) {
      c.tx->closed = 1;
      munmap(c.shm, sizeof(ConnShm));
      if (c.owner) unlink(c.shm_path.c_str());
    }
  }
  return libc().close(fd);
}

int ums_is_accelerated(int fd) {
  std::lock_guard<std::mutex> l(g_mu);
  Conn* p = find(fd);
  return p ? (p->accelerated ? 1 : 0) : -1;
}
int ums_owns(int fd) {
  std::lock_guard<std::mutex> l(g_mu);
  return find(fd) != nullptr;
}
void ums_get_stats(ums_stats_t* out) {
  std::lock_guard<std::mutex> l(g_mu);
  reap_links();
  __atomic_store_n(&g_stats.links_active, g_links.size(), __ATOMIC_RELAXED);
  const uint64_t* src = reinterpret_cast<const uint64_t*>(&g_stats);
  uint64_t* dst = reinterpret_cast<uint64_t*>(out);
  static_assert(sizeof(ums_stats_t) % sizeof(uint64_t) == 0, "ums_stats_t is a row of 64-bit counters");
  for (size_t i = 0; i < sizeof(ums_stats_t) / sizeof(uint64_t); ++i) dst[i] = __atomic_load_n(src + i, __ATOMIC_RELAXED);
}
int ums_link_test(int fd, int timeout_ms) {
  std::shared_ptr<Link> lk;
  uint32_t seq = 0;
  {
    std::lock_guard<std::mutex> l(g_mu);
    Conn* p = find(fd);
    if (!p || !p->accelerated || !p->link) return -1;
    lk = p->link;
    seq = ++lk->test_sent;
    if (!llc_push(lk.get(), LLC_TEST_LINK, 0, seq, p->slot)) return -1;
    if (p->tx->waiter.load()) {   // the peer sleeps in recv on this connection: wake it, it looks at the control ring
      const char bell = 1;
      if (libc().send(fd, &bell, 1, MSG_NOSIGNAL | MSG_DONTWAIT) > 0) stat_add(g_stats.doorbells);
    }
  }
  const uint64_t deadline = now_ms() + static_cast<uint64_t>(timeout_ms > 0 ? timeout_ms : 0);
  for (;;) {
    {
      std::lock_guard<std::mutex> l(g_mu);
      if (lk->shm) llc_progress(lk.get());
    }
    if (lk->test_acked.load() >= seq) return 0;
    if (now_ms() >= deadline) return -1;
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}
int ums_conn_info(int fd, ums_conn_info_t* out) {
  if (!out) return -1;
  std::lock_guard<std::mutex> l(g_mu);
  Conn* p = find(fd);
  if (!p || !p->accelerated) return -1;
  memset(out, 0, sizeof(*out));
  out->slot = p->slot;
  out->dim_level = p->dim ? p->dim->level.load() : 0;
  if (p->link) {
    snprintf(out->link, sizeof(out->link), "%s", p->link->name.c_str());
    out->link_conns = p->link->local_conns;
    out->link_state = p->link->shm ? p->link->shm->state.load() : (uint32_t)LINK_DELETED;
  }
  return 0;
}

}  // extern "C"
