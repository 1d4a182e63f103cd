// urma_perftest: latency and bandwidth of URMA verbs (write / read / send / atomic) between two endpoints.
//   urma_perftest [--stress THREADS] [--dev shm0|bond0|cudaN] [--peer-dev cudaM] [--mem cudaN] [--op write|read|send|faa|cas] [--size N] [--iters N]
//                 [--depth N] [--duration SEC] [--jettys N] [--cq-mod N] [--rate-limit MB/s]
//     --dev cudaN  the buffers live in the memory of GPU N (allocated through the CUDA runtime, loaded at run time);
//                  --peer-dev cudaM puts the second endpoint of the in-process mode on GPU M (default: the same GPU)
//     --duration   run the pipelined part for a time instead of a number of operations
//     --jettys     N endpoint pairs driven round-robin (in-process mode)
//     --cq-mod     ask for a completion only on every N-th operation (completion moderation)
//     --rate-limit pace the pipelined part to this many MB/s
//   urma_perftest --server PORT         waits for one client, serves its one-sided and two-sided traffic
//   urma_perftest --client HOST PORT    measures against a server in another process
// Without --server/--client both endpoints live in this process. Option names follow the reference's tool
// (src/urma/tools/urma_perftest, doc/en/urma/URMA User Guide.md:1690-1740: test type, message size, iterations,
// queue depth, out-of-band TCP exchange of segment and jetty information).
#include <arpa/inet.h>
#include <dlfcn.h>
#include <netinet/in.h>
#include <sched.h>
#include <stdio.h>
#include <sys/select.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <string>
#include <thread>
#include <vector>

#include "ub_util.h"
#include "urma_simple.h"

struct Blob {
  uint8_t ep[URMA_SIMPLE_JETTY_BLOB];
  uint8_t seg[URMA_SIMPLE_SEG_BLOB];
};
static int fail(const char* w) {
  fprintf(stderr, "urma_perftest: FAILED: %s\n", w);
  return 1;
}
static bool xfer(int fd, void* b, size_t n, bool tx) {
  char* p = (char*)b;
  while (n) {
    const ssize_t r = tx ? write(fd, p, n) : read(fd, p, n);
    if (r <= 0) return false;
    p += r;
    n -= r;
  }
  return true;
}
// Buffers: host memory, or - for the cudaN devices - memory of that GPU. The tool is a plain host program: the CUDA
// runtime is loaded when (and only when) a GPU device is named.
struct GpuRt {
  int (*set_device)(int) = nullptr;
  int (*malloc_)(void**, size_t) = nullptr;
  int (*memset_)(void*, int, size_t) = nullptr;
  int (*sync)() = nullptr;
  int (*memcpy_)(void*, const void*, size_t, int) = nullptr;
  bool load() {
    if (malloc_) return true;
    void* h = nullptr;
    for (const char* n : {"libcudart.so.12", "libcudart.so.13", "libcudart.so"})
      if ((h = dlopen(n, RTLD_NOW | RTLD_GLOBAL))) break;
    if (!h) return false;
    set_device = reinterpret_cast<int (*)(int)>(dlsym(h, "cudaSetDevice"));
    malloc_ = reinterpret_cast<int (*)(void**, size_t)>(dlsym(h, "cudaMalloc"));
    memset_ = reinterpret_cast<int (*)(void*, int, size_t)>(dlsym(h, "cudaMemset"));
    sync = reinterpret_cast<int (*)()>(dlsym(h, "cudaDeviceSynchronize"));
    memcpy_ = reinterpret_cast<int (*)(void*, const void*, size_t, int)>(dlsym(h, "cudaMemcpy"));
    return set_device && malloc_ && memset_ && sync && memcpy_;
  }
};
static GpuRt g_rt;
// -1 for a device that is not a GPU, else the GPU's index.
static int gpu_index(const std::string& dev) { return dev.rfind("cuda", 0) == 0 ? atoi(dev.c_str() + 4) : -1; }
// Host buffers live until the program ends (endpoints may still reference them while it winds down) and are
// released then; GPU buffers go with the CUDA context.
static std::vector<void*>& host_bufs() {
  static std::vector<void*> v;
  return v;
}
static uint8_t* alloc_buf(const std::string& dev, size_t bytes, int fill) {
  const int gi = gpu_index(dev);
  if (gi < 0) {
    uint8_t* p = static_cast<uint8_t*>(malloc(bytes));
    if (p) {
      memset(p, fill, bytes);
      if (host_bufs().empty())
        atexit([] {
          for (void* q : host_bufs()) free(q);
          host_bufs().clear();
        });
      host_bufs().push_back(p);
    }
    return p;
  }
  void* p = nullptr;
  if (!g_rt.load() || g_rt.set_device(gi) != 0 || g_rt.malloc_(&p, bytes) != 0 || g_rt.memset_(p, fill, bytes) != 0 ||
      g_rt.sync() != 0)
    return nullptr;
  return static_cast<uint8_t*>(p);
}

// The first `bytes` of a buffer as host memory (a copy for GPU buffers).
static std::vector<uint8_t> host_copy(const std::string& dev, const uint8_t* p, size_t bytes) {
  std::vector<uint8_t> out(bytes);
  if (gpu_index(dev) < 0) memcpy(out.data(), p, bytes);
  else if (g_rt.sync() != 0 || g_rt.memcpy_(out.data(), p, bytes, 4 /* cudaMemcpyDefault */) != 0) out.clear();
  return out;
}

static int wait_n(urma_simple_ep_t* ep, int want, int* bad) {
  int st[64];
  uint64_t uc[64];
  uint32_t fl[64];
  int got = 0;
  const uint64_t deadline = ub::now_ns() + 10000000000ull;
  while (got < want && ub::now_ns() < deadline) {
    const int n = urma_simple_poll(ep, std::min(64, want - got), st, uc, nullptr, nullptr, fl);
    for (int i = 0; i < n; ++i)
      if (st[i] != 0) ++*bad;
    if (n > 0) got += n;
    else sched_yield();
  }
  return got;
}

// --stress N: N threads at once between two contexts of this process, each with an endpoint pair of its own. Every
// round a thread sends a message of its own length and pattern (one slot up to several fragments) and receives it on
// the other side, writes a slice of the shared segment and reads it back, and adds to one shared counter. All data is
// checked; the counter must end at threads x rounds. What runs concurrently underneath: the posting threads, the two
// contexts' own threads, and the same application threads executing the inboxes from inside their polls.
static int stress(const std::string& dev, uint32_t threads, uint32_t rounds, uint32_t size) {
  urma_context_t* ca = urma_simple_open(dev.c_str());
  urma_context_t* cb = urma_simple_open(dev.c_str());
  if (!ca || !cb) return fail("open device (stress)");
  const uint32_t max_msg = size * 3 + 17;
  const uint32_t slice = max_msg;
  const uint64_t seg_bytes = uint64_t(slice) * threads + 64;
  std::vector<uint8_t> seg_mem(seg_bytes, 0);
  uint8_t seg_blob[URMA_SIMPLE_SEG_BLOB];
  urma_target_seg_t* seg = urma_simple_seg_register(cb, seg_mem.data(), seg_bytes, 14, 7, seg_blob);
  urma_target_seg_t* rseg = seg ? urma_simple_seg_import(ca, seg_blob, 7) : nullptr;
  if (!seg || !rseg) return fail("segment (stress)");
  const uint64_t counter_off = uint64_t(slice) * threads;   // 8-byte aligned below
  const uint64_t counter_va = (rseg->seg.ubva.va + counter_off + 7) & ~7ull;
  std::atomic<int> failed{0};
  std::atomic<uint32_t> ready{0};
  auto worker = [&](uint32_t t) {
    auto bail = [&](const char* what) {
      fprintf(stderr, "urma_perftest: stress thread %u: %s\n", t, what);
      ++failed;
    };
    urma_simple_ep_t* a = urma_simple_ep_create(ca, 32, 1, 0);
    urma_simple_ep_t* b = urma_simple_ep_create(cb, 32, 1, 0);
    if (!a || !b) return bail("endpoints");
    uint8_t blob[URMA_SIMPLE_JETTY_BLOB];
    urma_simple_ep_blob(b, blob);
    urma_target_jetty_t* tb = urma_simple_ep_import(ca, blob, 1);
    if (!tb) return bail("import");
    constexpr uint32_t kRecv = 4;
    std::vector<std::vector<uint8_t>> rbuf(kRecv, std::vector<uint8_t>(max_msg));
    for (uint32_t i = 0; i < kRecv; ++i)
      if (urma_simple_post_recv(b, rbuf[i].data(), max_msg, i) != 0) return bail("post_recv");
    std::vector<uint8_t> out(max_msg), back(max_msg);
    ++ready;
    while (ready.load() < threads && !failed.load()) sched_yield();   // everybody starts together
    auto wait_one = [&](urma_simple_ep_t* ep, bool want_recv, uint64_t* uc, uint32_t* len, uint64_t* imm) {
      const uint64_t deadline = ub::now_ns() + 20000000000ull;
      while (ub::now_ns() < deadline && !failed.load()) {
        int st;
        uint32_t fl;
        const int n = urma_simple_poll(ep, 1, &st, uc, len, imm, &fl);
        if (n == 1) {
          if (st != 0) return false;
          if (((fl & URMA_CR_FLAG_RECV) != 0) == want_recv) return true;
        }
      }
      return false;
    };
    for (uint32_t i = 0; i < rounds && !failed.load(); ++i) {
      // lengths walk through: tiny, one slot, just over a slot, several fragments
      const uint32_t lens[4] = {1 + (i + t) % 97, size, size + 1 + (i % 7), max_msg - (i % 13)};
      const uint32_t len = lens[(i + t) & 3];
      for (uint32_t k = 0; k < len; ++k) out[k] = (uint8_t)(k * 31 + i * 7 + t * 13 + 1);
      uint64_t uc = 0, imm = 0;
      uint32_t got = 0;
      if (urma_simple_post(a, tb, URMA_OPC_SEND_IMM, nullptr, 0, nullptr, (uint64_t)out.data(), len, (uint64_t(t) << 32) | i, i, 1) != 0)
        return bail("post send");
      if (!wait_one(b, true, &uc, &got, &imm)) return bail("receive completion");
      if (got != len || imm != ((uint64_t(t) << 32) | i) || uc >= kRecv || memcmp(rbuf[uc].data(), out.data(), len))
        return bail("received data differs");
      if (urma_simple_post_recv(b, rbuf[uc].data(), max_msg, uc) != 0) return bail("re-post receive");
      if (!wait_one(a, false, &uc, &got, &imm)) return bail("send completion");
      // one-sided: write this thread's slice, read it back
      const uint64_t va = rseg->seg.ubva.va + uint64_t(slice) * t;
      if (urma_simple_post(a, tb, URMA_OPC_WRITE, rseg, va, nullptr, (uint64_t)out.data(), len, 0, i, 1) != 0 ||
          !wait_one(a, false, &uc, &got, &imm))
        return bail("write");
      memset(back.data(), 0, len);
      if (urma_simple_post(a, tb, URMA_OPC_READ, rseg, va, nullptr, (uint64_t)back.data(), len, 0, i, 1) != 0 ||
          !wait_one(a, false, &uc, &got, &imm))
        return bail("read");
      if (memcmp(back.data(), out.data(), len)) return bail("read back differs from what was written");
      uint64_t old = 0;
      if (urma_simple_atomic(a, tb, URMA_OPC_FADD, rseg, counter_va, 1, 0, &old, i) != 0 ||
          !wait_one(a, false, &uc, &got, &imm))
        return bail("fetch-add");
    }
    urma_unimport_jetty(tb);
    urma_simple_ep_destroy(a);
    urma_simple_ep_destroy(b);
  };
  const uint64_t t0 = ub::now_ns();
  std::vector<std::thread> th;
  for (uint32_t t = 0; t < threads; ++t) th.emplace_back(worker, t);
  for (auto& x : th) x.join();
  const double sec = (ub::now_ns() - t0) * 1e-9;
  uint64_t total = 0;
  memcpy(&total, seg_mem.data() + (counter_va - rseg->seg.ubva.va), 8);
  if (failed.load() == 0 && total != uint64_t(threads) * rounds) {
    fprintf(stderr, "urma_perftest: shared counter is %llu, expected %llu\n", (unsigned long long)total,
            (unsigned long long)threads * rounds);
    ++failed;
  }
  printf("stress dev=%s threads=%u rounds=%u size=%u: %.0f operations/s in total, %s\n", dev.c_str(), threads, rounds,
         size, 4.0 * threads * rounds / sec, failed.load() ? "FAILED" : "all data verified");
  urma_unimport_seg(rseg);
  urma_unregister_seg(seg);
  if (urma_simple_close(ca) != 0 || urma_simple_close(cb) != 0) return fail("contexts still had objects at the end");
  if (failed.load()) return fail("stress");
  printf("urma_perftest: OK\n");
  return 0;
}

int main(int argc, char** argv) {
  std::string dev = "shm0", peer_dev, op = "write", host = "127.0.0.1", mem;
  uint32_t size = 4096, iters = 20000, depth = 64;
  int server = -1, client = -1;
  uint32_t jettys = 1, cq_mod = 1;
  double duration = 0, rate_mbs = 0;
  uint32_t stress_threads = 0;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--stress") && i + 1 < argc) stress_threads = std::max(1, atoi(argv[++i]));
    else
    if (!strcmp(argv[i], "--duration") && i + 1 < argc) duration = atof(argv[++i]);
    else if (!strcmp(argv[i], "--jettys") && i + 1 < argc) jettys = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--cq-mod") && i + 1 < argc) cq_mod = std::max(1, atoi(argv[++i]));
    else if (!strcmp(argv[i], "--rate-limit") && i + 1 < argc) rate_mbs = atof(argv[++i]);
    else if (!strcmp(argv[i], "--dev") && i + 1 < argc) dev = argv[++i];
    else if (!strcmp(argv[i], "--peer-dev") && i + 1 < argc) peer_dev = argv[++i];
    else if (!strcmp(argv[i], "--mem") && i + 1 < argc) mem = argv[++i];
    else if (!strcmp(argv[i], "--op") && i + 1 < argc) op = argv[++i];
    else if (!strcmp(argv[i], "--size") && i + 1 < argc) size = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--depth") && i + 1 < argc) depth = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--server") && i + 1 < argc) server = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--client") && i + 2 < argc) {
      host = argv[++i];
      client = atoi(argv[++i]);
    }
  }
  if (stress_threads) {
    if (gpu_index(dev) >= 0) return fail("--stress runs on host devices");
    return stress(dev, stress_threads, iters, size);
  }
  urma_context_t* ctx = urma_simple_open(dev.c_str());
  if (!ctx) return fail("open device");
  const uint32_t seg_bytes = std::max<uint32_t>(size, 4096) * 2;
  if (peer_dev.empty()) peer_dev = dev;
  if ((gpu_index(dev) >= 0) != (gpu_index(peer_dev) >= 0)) return fail("--dev and --peer-dev must both be GPUs or both not");
  // (named like the vectors they replace: .data() is the buffer, in host or GPU memory)
  struct Buf {
    uint8_t* p = nullptr;
    uint8_t* data() const { return p; }
  };
  // where the buffers live: with the device by default; --mem cudaN puts them on a GPU whatever the device is called
  // (a bond device whose paths are cudaN devices)
  const std::string mem_a_dev = mem.empty() ? dev : mem, mem_b_dev = mem.empty() ? peer_dev : mem;
  Buf mem_a{alloc_buf(mem_a_dev, seg_bytes, 1)}, mem_b{alloc_buf(mem_b_dev, seg_bytes, 2)};
  if (!mem_a.p || !mem_b.p) return fail("buffer allocation (for cudaN: is the CUDA runtime library on the loader path?)");
  urma_simple_ep_t* ea = urma_simple_ep_create(ctx, depth * 2, 1, 0);
  Blob mine{}, peer{};
  urma_target_seg_t* seg_a = urma_simple_seg_register(ctx, mem_a.data(), seg_bytes, 14, 1, mine.seg);
  if (!ea || !seg_a) return fail("endpoint / segment");
  urma_simple_ep_blob(ea, mine.ep);
  urma_simple_ep_t* eb = nullptr;
  urma_context_t* ctx_b = nullptr;
  urma_target_seg_t* seg_b_reg = nullptr;
  int tcp = -1;
  if (server >= 0 || client >= 0) {
    if (server >= 0) {
      const int ls = socket(AF_INET, SOCK_STREAM, 0);
      int one = 1;
      setsockopt(ls, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
      sockaddr_in a{};
      a.sin_family = AF_INET;
      a.sin_port = htons(server);
      a.sin_addr.s_addr = htonl(INADDR_ANY);
      if (bind(ls, (sockaddr*)&a, sizeof(a)) || listen(ls, 1)) return fail("listen");
      printf("urma_perftest server ready on port %d\n", server);
      fflush(stdout);
      tcp = accept(ls, nullptr, nullptr);
      close(ls);
    } else {
      tcp = socket(AF_INET, SOCK_STREAM, 0);
      sockaddr_in a{};
      a.sin_family = AF_INET;
      a.sin_port = htons(client);
      a.sin_addr.s_addr = inet_addr(host.c_str());
      if (connect(tcp, (sockaddr*)&a, sizeof(a))) return fail("connect");
    }
    if (!xfer(tcp, &mine, sizeof(mine), true) || !xfer(tcp, &peer, sizeof(peer), false)) return fail("exchange");
  } else {
    ctx_b = urma_simple_open(peer_dev.c_str());
    eb = urma_simple_ep_create(ctx_b, depth * 2, 1, 0);
    urma_target_seg_t* seg_b = urma_simple_seg_register(ctx_b, mem_b.data(), seg_bytes, 14, 1, peer.seg);
    seg_b_reg = seg_b;
    if (!eb || !seg_b) return fail("second endpoint");
    urma_simple_ep_blob(eb, peer.ep);
  }
  // extra endpoint pairs for --jettys (in-process mode): pair j = (ex_a[j], ex_b[j]), same segments
  std::vector<urma_simple_ep_t*> ex_a, ex_b;
  std::vector<urma_target_jetty_t*> ex_t;
  if (eb) {
    for (uint32_t j = 1; j < jettys; ++j) {
      urma_simple_ep_t* a2 = urma_simple_ep_create(ctx, depth * 2, 1, 0);
      urma_simple_ep_t* b2 = urma_simple_ep_create(ctx_b, depth * 2, 1, 0);
      if (!a2 || !b2) return fail("extra endpoints");
      uint8_t blob[URMA_SIMPLE_JETTY_BLOB];
      urma_simple_ep_blob(b2, blob);
      urma_target_jetty_t* t2 = urma_simple_ep_import(ctx, blob, 1);
      if (!t2) return fail("import of an extra endpoint");
      ex_a.push_back(a2);
      ex_b.push_back(b2);
      ex_t.push_back(t2);
    }
  } else {
    jettys = 1;
  }
  urma_target_jetty_t* tj = urma_simple_ep_import(ctx, peer.ep, 1);
  urma_target_seg_t* rseg = urma_simple_seg_import(ctx, peer.seg, 1);
  if (!tj || !rseg) return fail("import");
  const uint64_t rva = rseg->seg.ubva.va;
  if (server >= 0) {  // passive side: keep receives posted until the client says goodbye
    std::vector<Buf> rb(depth);
    for (uint32_t i = 0; i < depth; ++i) {
      rb[i].p = alloc_buf(mem_a_dev, size, 0);
      if (!rb[i].p) return fail("receive buffer allocation");
      urma_simple_post_recv(ea, rb[i].data(), size, i);
    }
    char bye;
    for (;;) {
      int st[32];
      uint64_t uc[32];
      uint32_t fl[32];
      const int n = urma_simple_poll(ea, 32, st, uc, nullptr, nullptr, fl);
      for (int i = 0; i < n; ++i)
        if (fl[i] & URMA_CR_FLAG_RECV) urma_simple_post_recv(ea, rb[uc[i]].data(), size, uc[i]);
      {
        fd_set s;
        FD_ZERO(&s);
        FD_SET(tcp, &s);
        timeval tv{0, n > 0 ? 0 : 200};
        if (select(tcp + 1, &s, nullptr, nullptr, &tv) > 0 && read(tcp, &bye, 1) <= 1) break;
      }
    }
    printf("urma_perftest server: done\n");
    return 0;
  }
  int opc = URMA_OPC_WRITE;
  bool atomic = false, two_sided = false;
  if (op == "read") opc = URMA_OPC_READ;
  else if (op == "send") {
    opc = URMA_OPC_SEND;
    two_sided = true;
  } else if (op == "faa") {
    opc = URMA_OPC_FADD;
    atomic = true;
    size = 8;
  } else if (op == "cas") {
    opc = URMA_OPC_CAS;
    atomic = true;
    size = 8;
  }
  std::vector<Buf> rb;
  if (two_sided && eb) {
    rb.resize(depth * 2);
    for (uint32_t i = 0; i < depth * 2; ++i) {
      rb[i].p = alloc_buf(mem_b_dev, size, 0);
      if (!rb[i].p) return fail("receive buffer allocation");
      urma_simple_post_recv(eb, rb[i].data(), size, i);
    }
  }
  auto post = [&](uint64_t id) {
    if (atomic) return urma_simple_atomic(ea, tj, opc, rseg, rva, 1, 0, nullptr, id);
    return urma_simple_post(ea, tj, opc, two_sided ? nullptr : rseg, rva, nullptr, (uint64_t)mem_a.data(), size, 0, id, 1);
  };
  int bad = 0;
  // latency: one operation at a time
  const uint32_t lat_iters = std::min<uint32_t>(iters, 5000);
  ub::PerfHist h;
  for (uint32_t i = 0; i < lat_iters; ++i) {
    const uint64_t t0 = ub::now_ns();
    if (post(i) != 0) return fail("post");
    if (wait_n(ea, 1, &bad) != 1) return fail("completion timeout");
    h.add(ub::now_ns() - t0);
    if (two_sided && eb) {
      int st;
      uint64_t uc;
      uint32_t fl;
      while (urma_simple_poll(eb, 1, &st, &uc, nullptr, nullptr, &fl) == 1)
        if (fl & URMA_CR_FLAG_RECV) urma_simple_post_recv(eb, rb[uc].data(), size, uc);
    }
  }
  // bandwidth / rate: keep `depth` operations in flight on every endpoint pair
  std::vector<urma_simple_ep_t*> all_a{ea}, all_b{eb};
  std::vector<urma_target_jetty_t*> all_t{tj};
  for (size_t j = 0; j < ex_a.size(); ++j) {
    all_a.push_back(ex_a[j]);
    all_b.push_back(ex_b[j]);
    all_t.push_back(ex_t[j]);
  }
  if (two_sided && eb) {
    for (size_t j = 1; j < all_b.size(); ++j)
      for (uint32_t i = 0; i < depth * 2; ++i) urma_simple_post_recv(all_b[j], rb[i].data(), size, i);
  }
  std::vector<uint64_t> sent(jettys, 0), done(jettys, 0);
  std::vector<char> last_sig(jettys, 1), flushed(jettys, 0);
  uint64_t total_sent = 0, total_done = 0;
  const uint64_t t0 = ub::now_ns();
  const uint64_t t_end = duration > 0 ? t0 + (uint64_t)(duration * 1e9) : 0;
  auto more = [&]() { return t_end ? ub::now_ns() < t_end : total_sent < iters; };
  auto paced = [&]() {  // true while the byte budget of --rate-limit allows another operation
    if (rate_mbs <= 0) return true;
    return total_sent * (double)size <= rate_mbs * 1e6 * ((ub::now_ns() - t0) * 1e-9);
  };
  while (more() || total_done < total_sent) {
    for (uint32_t j = 0; j < jettys; ++j) {
      while (more() && paced() && sent[j] - done[j] < depth) {
        // completion moderation: only every cq_mod-th operation of a pair asks for a completion, which then stands
        // for the cq_mod operations up to it (the last operation of the run always asks)
        const bool sig = ((sent[j] + 1) % cq_mod) == 0 || atomic;
        int rc;
        if (atomic) rc = urma_simple_atomic(all_a[j], all_t[j], opc, rseg, rva, 1, 0, nullptr, sent[j]);
        else rc = urma_simple_post(all_a[j], all_t[j], opc, two_sided ? nullptr : rseg, rva, nullptr,
                                   (uint64_t)mem_a.data(), size, 0, sent[j], sig ? 1 : 0);
        if (rc == URMA_EAGAIN) break;
        if (rc != 0) return fail("post (pipelined)");
        ++sent[j];
        ++total_sent;
        last_sig[j] = sig;
      }
    }
    bool progressed = false;
    for (uint32_t j = 0; j < jettys; ++j) {
      int st[64];
      uint64_t uc[64];
      uint32_t fl[64];
      const int n = urma_simple_poll(all_a[j], 64, st, uc, nullptr, nullptr, fl);
      for (int i = 0; i < n; ++i) {
        if (st[i] != 0) ++bad;
        const uint64_t upto = uc[i] + 1;          // operations are completed in order on one endpoint
        if (upto > done[j]) {
          total_done += upto - done[j];
          done[j] = upto;
        }
        progressed = true;
      }
      if (two_sided && all_b[j]) {
        const int m = urma_simple_poll(all_b[j], 64, st, uc, nullptr, nullptr, fl);
        for (int i = 0; i < m; ++i)
          if (fl[i] & URMA_CR_FLAG_RECV) urma_simple_post_recv(all_b[j], rb[uc[i]].data(), size, uc[i]);
      }
    }
    if (!more()) {
      // flush the tail: operations after the last signalled one complete silently, so one more signalled operation
      // per pair is posted, whose completion stands for everything before it
      for (uint32_t j = 0; j < jettys; ++j) {
        if (done[j] < sent[j] && !last_sig[j] && !flushed[j]) {
          if (urma_simple_post(all_a[j], all_t[j], opc, two_sided ? nullptr : rseg, rva, nullptr,
                               (uint64_t)mem_a.data(), size, 0, sent[j], 1) == 0) {
            ++sent[j];
            ++total_sent;
            flushed[j] = true;
          }
        }
      }
    }
    if (!progressed) {
      if (ub::now_ns() - t0 > (uint64_t)((duration > 0 ? duration : 0) * 1e9) + 20000000000ull)
        return fail("completion timeout (pipelined)");
      sched_yield();
    }
  }
  iters = (uint32_t)total_done;
  const double sec = (ub::now_ns() - t0) * 1e-9;
  printf("%s dev=%s size=%u depth=%u jettys=%u cq_mod=%u: latency avg %.2f us p99 %.2f us min %.2f us | %.0f ops/s, %.2f MB/s | errors %d\n",
         op.c_str(), dev.c_str(), size, depth, jettys, cq_mod, h.mean() / 1e3, h.quantile(0.99) / 1e3, h.min() / 1e3, iters / sec,
         iters * (double)size / sec / 1e6, bad);
  if (tcp >= 0) {
    char bye = 'q';
    if (write(tcp, &bye, 1) < 0) {
    }
    close(tcp);
  }
  bool data_ok = true;
  if (!two_sided && !atomic && opc == URMA_OPC_WRITE && eb) {   // a write must have carried the source buffer over
    const std::vector<uint8_t> ha = host_copy(mem_a_dev, mem_a.data(), size), hb = host_copy(mem_b_dev, mem_b.data(), size);
    data_ok = ha.size() == size && hb.size() == size && memcmp(ha.data(), hb.data(), size) == 0;
  }
  // tear down in the reverse order of the bring-up (imports, endpoints, segments, contexts)
  for (auto* t : ex_t) urma_unimport_jetty(t);
  urma_unimport_jetty(tj);
  urma_unimport_seg(rseg);
  for (auto* e : ex_a) urma_simple_ep_destroy(e);
  for (auto* e : ex_b) urma_simple_ep_destroy(e);
  urma_simple_ep_destroy(ea);
  if (eb) urma_simple_ep_destroy(eb);
  urma_unregister_seg(seg_a);
  if (seg_b_reg) urma_unregister_seg(seg_b_reg);
  if (ctx_b) urma_simple_close(ctx_b);
  urma_simple_close(ctx);
  if (bad) return fail("completions with error status");
  if (!data_ok) return fail("written data differs");
  printf("urma_perftest: OK\n");
  return 0;
}
