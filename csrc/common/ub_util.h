// Small header-only utilities shared by the host libraries: intrusive list, chained hash map, bitmap, string
// builder, hashing, clocks and a log-bucket latency histogram. Same roles as the reference's src/urma/common
// (ub_list.h, ub_hmap.h, ub_bitmap.h, ub_hash.h, ub_dstring.h, ub_get_clock.h) and the percentile tables of
// src/urma/lib/urma/core/urma_perf.c, written from scratch as C++17.
#pragma once
#include <cstdlib>
#include <cstdio>
#include <cstdarg>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <syslog.h>
#include <time.h>

#include <atomic>
#include <string>
#include <vector>

namespace ub {

// ---------------------------------------------------------------- intrusive list
struct ListNode {
  ListNode* prev;
  ListNode* next;
  ListNode() : prev(this), next(this) {}
  bool empty() const { return next == this; }
  void push_back(ListNode* n) {
    n->prev = prev;
    n->next = this;
    prev->next = n;
    prev = n;
  }
  void push_front(ListNode* n) {
    n->next = next;
    n->prev = this;
    next->prev = n;
    next = n;
  }
  static void remove(ListNode* n) {
    n->prev->next = n->next;
    n->next->prev = n->prev;
    n->prev = n->next = n;
  }
  ListNode* pop_front() {
    if (empty()) return nullptr;
    ListNode* n = next;
    remove(n);
    return n;
  }
  size_t size() const {
    size_t c = 0;
    for (const ListNode* n = next; n != this; n = n->next) ++c;
    return c;
  }
};
#define UB_CONTAINER_OF(ptr, type, member) \
  (reinterpret_cast<type*>(reinterpret_cast<char*>(ptr) - offsetof(type, member)))

// ---------------------------------------------------------------- hashing
inline uint32_t hash_bytes(const void* data, size_t n, uint32_t seed = 0x9747b28c) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint32_t h = seed ^ 2166136261u;
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 16777619u;
  }
  h ^= h >> 15;
  h *= 0x85ebca6bu;
  h ^= h >> 13;
  return h;
}
inline uint32_t hash_u64(uint64_t v) {
  v ^= v >> 33;
  v *= 0xff51afd7ed558ccdULL;
  v ^= v >> 33;
  v *= 0xc4ceb9fe1a85ec53ULL;
  v ^= v >> 33;
  return static_cast<uint32_t>(v);
}

// ---------------------------------------------------------------- chained hash map with intrusive nodes
struct HmapNode {
  HmapNode* next = nullptr;
  uint32_t hash = 0;
};
class Hmap {
 public:
  explicit Hmap(size_t buckets = 64) : buckets_(round_pow2(buckets), nullptr) {}
  void insert(HmapNode* n, uint32_t hash) {
    if (count_ > buckets_.size() * 2) grow();
    n->hash = hash;
    HmapNode*& head = buckets_[hash & (buckets_.size() - 1)];
    n->next = head;
    head = n;
    ++count_;
  }
  bool remove(HmapNode* n) {
    HmapNode** pp = &buckets_[n->hash & (buckets_.size() - 1)];
    for (; *pp; pp = &(*pp)->next) {
      if (*pp == n) {
        *pp = n->next;
        n->next = nullptr;
        --count_;
        return true;
      }
    }
    return false;
  }
  HmapNode* first_with_hash(uint32_t hash) const {
    for (HmapNode* n = buckets_[hash & (buckets_.size() - 1)]; n; n = n->next)
      if (n->hash == hash) return n;
    return nullptr;
  }
  static HmapNode* next_with_hash(HmapNode* n) {
    for (HmapNode* m = n->next; m; m = m->next)
      if (m->hash == n->hash) return m;
    return nullptr;
  }
  size_t count() const { return count_; }
  template <typename F>
  void for_each(F f) const {
    for (HmapNode* head : buckets_)
      for (HmapNode* n = head; n;) {
        HmapNode* nx = n->next;
        f(n);
        n = nx;
      }
  }

 private:
  static size_t round_pow2(size_t v) {
    size_t p = 1;
    while (p < v) p <<= 1;
    return p;
  }
  void grow() {
    std::vector<HmapNode*> nb(buckets_.size() * 4, nullptr);
    for (HmapNode* head : buckets_)
      for (HmapNode* n = head; n;) {
        HmapNode* nx = n->next;
        HmapNode*& h = nb[n->hash & (nb.size() - 1)];
        n->next = h;
        h = n;
        n = nx;
      }
    buckets_.swap(nb);
  }
  std::vector<HmapNode*> buckets_;
  size_t count_ = 0;
};

// ---------------------------------------------------------------- bitmap
class Bitmap {
 public:
  explicit Bitmap(size_t bits = 0) { resize(bits); }
  void resize(size_t bits) {
    bits_ = bits;
    words_.assign((bits + 63) / 64, 0);
  }
  size_t size() const { return bits_; }
  bool test(size_t i) const { return i < bits_ && ((words_[i >> 6] >> (i & 63)) & 1u); }
  void set(size_t i) {
    if (i < bits_) words_[i >> 6] |= (uint64_t(1) << (i & 63));
  }
  void clear(size_t i) {
    if (i < bits_) words_[i >> 6] &= ~(uint64_t(1) << (i & 63));
  }
  // index of the first zero bit, set it; returns -1 when full
  long alloc() {
    for (size_t w = 0; w < words_.size(); ++w) {
      if (~words_[w]) {
        const int b = __builtin_ctzll(~words_[w]);
        const size_t i = w * 64 + b;
        if (i >= bits_) return -1;
        words_[w] |= (uint64_t(1) << b);
        return static_cast<long>(i);
      }
    }
    return -1;
  }
  size_t popcount() const {
    size_t c = 0;
    for (uint64_t w : words_) c += __builtin_popcountll(w);
    return c;
  }

 private:
  size_t bits_ = 0;
  std::vector<uint64_t> words_;
};

// ---------------------------------------------------------------- string builder
class DString {
 public:
  void printf(const char* fmt, ...) __attribute__((format(printf, 2, 3))) {
    va_list ap;
    va_start(ap, fmt);
    char buf[1024];
    const int n = vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (n < 0) return;
    if (static_cast<size_t>(n) < sizeof(buf)) {
      s_.append(buf, n);
    } else {
      std::string big(n + 1, '\0');
      va_start(ap, fmt);
      vsnprintf(&big[0], big.size(), fmt, ap);
      va_end(ap);
      s_.append(big.c_str(), n);
    }
  }
  void puts(const char* s) { s_ += s; }
  const char* c_str() const { return s_.c_str(); }
  const std::string& str() const { return s_; }
  void clear() { s_.clear(); }

 private:
  std::string s_;
};

// ---------------------------------------------------------------- clocks
inline uint64_t now_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return uint64_t(ts.tv_sec) * 1000000000ull + ts.tv_nsec;
}
inline uint64_t cycles() {
#if defined(__x86_64__)
  uint32_t lo, hi;
  __asm__ __volatile__("rdtsc" : "=a"(lo), "=d"(hi));
  return (uint64_t(hi) << 32) | lo;
#elif defined(__aarch64__)
  uint64_t v;
  __asm__ __volatile__("mrs %0, cntvct_el0" : "=r"(v));
  return v;
#else
  return now_ns();
#endif
}

// One step of a polling loop: tells the core that this is a spin-wait (frees the pipeline for the sibling thread,
// avoids the memory-order mis-speculation penalty on leaving the loop).
inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#elif defined(__aarch64__)
  __asm__ __volatile__("yield");
#endif
}

// ---------------------------------------------------------------- latency histogram (log2 buckets x 8 sub-buckets)
class PerfHist {
 public:
  static constexpr int kSub = 8;
  static constexpr int kBuckets = 64 * kSub;
  void add(uint64_t ns) {
    const int idx = bucket_of(ns);
    ++b_[idx];
    ++n_;
    sum_ += ns;
    if (ns < min_) min_ = ns;
    if (ns > max_) max_ = ns;
  }
  void reset() { *this = PerfHist(); }
  void merge(const PerfHist& o) {
    for (int i = 0; i < kBuckets; ++i) b_[i] += o.b_[i];
    n_ += o.n_;
    sum_ += o.sum_;
    if (o.min_ < min_) min_ = o.min_;
    if (o.max_ > max_) max_ = o.max_;
  }
  uint64_t count() const { return n_; }
  uint64_t min() const { return n_ ? min_ : 0; }
  uint64_t max() const { return max_; }
  double mean() const { return n_ ? double(sum_) / double(n_) : 0.0; }
  // upper bound of the bucket that holds quantile q in [0,1]
  uint64_t quantile(double q) const {
    if (!n_) return 0;
    const uint64_t target = static_cast<uint64_t>(q * double(n_ - 1)) + 1;
    uint64_t run = 0;
    for (int i = 0; i < kBuckets; ++i) {
      run += b_[i];
      if (run >= target) return bucket_hi(i) < max_ ? bucket_hi(i) : max_;
    }
    return max_;
  }

 private:
  static int bucket_of(uint64_t v) {
    if (v < kSub) return static_cast<int>(v);
    const int msb = 63 - __builtin_clzll(v);
    const int sub = static_cast<int>((v >> (msb - 3)) & (kSub - 1));
    const int idx = (msb - 2) * kSub + sub;
    return idx < kBuckets ? idx : kBuckets - 1;
  }
  static uint64_t bucket_hi(int idx) {
    if (idx < kSub) return idx;
    const int msb = idx / kSub + 2;
    const int sub = idx % kSub;
    return (uint64_t(1) << msb) + (uint64_t(sub + 1) << (msb - 3)) - 1;
  }
  uint64_t b_[kBuckets] = {0};
  uint64_t n_ = 0, sum_ = 0, min_ = ~0ull, max_ = 0;
};

// Leveled logger shared by the queue / RPC libraries: one instance per component, default sink stderr, optional user
// callback, level from the component's API or from <TAG>_LOG_LEVEL (0 = error ... 4 = debug). Same controls as the
// reference's *_log_config_set calls (src/urpc/include/umq/umq_api.h, urpc_framework_api.h).
enum LogLevel : int { kLogErr = 0, kLogWarn = 1, kLogNotice = 2, kLogInfo = 3, kLogDebug = 4 };
typedef void (*log_cb_t)(int level, const char* msg);
class Logger {
 public:
  explicit Logger(const char* tag) : tag_(tag) {
    char name[64];
    snprintf(name, sizeof(name), "%s_LOG_LEVEL", tag);
    if (const char* e = getenv(name)) level_ = atoi(e);
    snprintf(name, sizeof(name), "%s_LOG_SYSLOG", tag);
    if (const char* e = getenv(name)) to_syslog_ = atoi(e) != 0;
  }
  void configure(int level, log_cb_t cb) {
    level_ = level;
    cb_ = cb;
  }
  int level() const { return level_; }
  void log(int lvl, const char* fmt, ...) __attribute__((format(printf, 3, 4))) {
    if (lvl > level_) return;
    char msg[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    log_cb_t cb = cb_;
    if (cb) {
      cb(lvl, msg);
    } else {
      static const char* const names[] = {"ERR", "WARN", "NOTICE", "INFO", "DEBUG"};
      static const int prio[] = {LOG_ERR, LOG_WARNING, LOG_NOTICE, LOG_INFO, LOG_DEBUG};
      const int l = lvl < 0 ? 0 : (lvl > 4 ? 4 : lvl);
      if (to_syslog_)  // same "[TAG][LEVEL]" prefix as on stderr: the packaged rsyslog rules route on it
        syslog(prio[l], "[%s][%s] %s", tag_, names[l], msg);
      else
        fprintf(stderr, "[%s][%s] %s\n", tag_, names[l], msg);
    }
  }

 private:
  const char* tag_;
  std::atomic<int> level_{kLogWarn};
  std::atomic<log_cb_t> cb_{nullptr};
  bool to_syslog_ = false;
};

}  // namespace ub
