// Small building blocks of the RPC library's control plane: a timer wheel with one-shot and periodic timers, a slab
// of fixed-size objects addressed by (index, generation) handles, and an id generator that hands out the lowest free
// number of a range. The control-plane task engine keeps its tasks in a Slab, names them with IdGen and puts their
// deadlines and waits on a TimerWheel; the pieces are header-only and have no other dependency.
//
// Same roles as the reference's utility units (src/urpc/util/urpc_timer.h:34-47 timing wheel with create / start /
// restart / delete and a periodic flag, src/urpc/util/urpc_slab.h object slab, src/urpc/util/urpc_id_generator.h
// bitmap id generator).
#pragma once
#include <stdint.h>

#include <functional>
#include <mutex>
#include <utility>
#include <vector>

namespace urpc_util {

// ---------------------------------------------------------------------------------------------------- id generator
// Ids min..min+count-1. alloc() prefers the id after the one handed out last (so a freed id is not reused at once,
// which keeps a late message that still names the old owner from reaching a new one), and wraps around.
class IdGen {
 public:
  IdGen(uint32_t min, uint32_t count) : min_(min), n_(count), used_((count + 63) / 64, 0) {}
  bool alloc(uint32_t* id) {
    std::lock_guard<std::mutex> l(mu_);
    if (in_use_ == n_) return false;
    for (uint32_t k = 0; k < n_; ++k) {
      const uint32_t i = (hint_ + k) % n_;
      if (!(used_[i / 64] >> (i % 64) & 1)) {
        used_[i / 64] |= 1ull << (i % 64);
        hint_ = (i + 1) % n_;
        ++in_use_;
        *id = min_ + i;
        return true;
      }
    }
    return false;
  }
  bool free(uint32_t id) {
    std::lock_guard<std::mutex> l(mu_);
    if (id < min_ || id - min_ >= n_) return false;
    const uint32_t i = id - min_;
    if (!(used_[i / 64] >> (i % 64) & 1)) return false;   // double free is reported, not ignored
    used_[i / 64] &= ~(1ull << (i % 64));
    --in_use_;
    return true;
  }
  uint32_t in_use() {
    std::lock_guard<std::mutex> l(mu_);
    return in_use_;
  }

 private:
  const uint32_t min_, n_;
  std::mutex mu_;
  std::vector<uint64_t> used_;
  uint32_t hint_ = 0, in_use_ = 0;
};

// ------------------------------------------------------------------------------------------------------------ slab
// Objects live in chunks that never move, so a pointer stays valid until its object is released. A handle packs the
// slot index with the slot's generation: a handle kept after release() no longer resolves (get() returns null)
// even when the slot has been handed out again.
template <typename T>
class Slab {
 public:
  explicit Slab(uint32_t chunk_objs = 64) : per_(chunk_objs ? chunk_objs : 64) {}
  ~Slab() {
    for (auto& c : chunks_) delete[] c;
  }
  Slab(const Slab&) = delete;
  Slab& operator=(const Slab&) = delete;

  uint64_t acquire(T** out) {
    std::lock_guard<std::mutex> l(mu_);
    if (free_.empty()) {
      Slot* c = new Slot[per_];
      const uint32_t base = static_cast<uint32_t>(chunks_.size()) * per_;
      chunks_.push_back(c);
      for (uint32_t i = per_; i-- > 0;) free_.push_back(base + i);
    }
    const uint32_t idx = free_.back();
    free_.pop_back();
    Slot& s = slot(idx);
    s.live = true;
    s.obj = T();
    ++live_;
    if (out) *out = &s.obj;
    return (uint64_t(s.gen) << 32) | idx;
  }
  T* get(uint64_t h) {
    std::lock_guard<std::mutex> l(mu_);
    const uint32_t idx = static_cast<uint32_t>(h);
    if (idx >= chunks_.size() * per_) return nullptr;
    Slot& s = slot(idx);
    return (s.live && s.gen == static_cast<uint32_t>(h >> 32)) ? &s.obj : nullptr;
  }
  bool release(uint64_t h) {
    std::lock_guard<std::mutex> l(mu_);
    const uint32_t idx = static_cast<uint32_t>(h);
    if (idx >= chunks_.size() * per_) return false;
    Slot& s = slot(idx);
    if (!s.live || s.gen != static_cast<uint32_t>(h >> 32)) return false;
    s.live = false;
    s.obj = T();   // drop what the object owned
    ++s.gen;
    free_.push_back(idx);
    --live_;
    return true;
  }
  uint32_t live() {
    std::lock_guard<std::mutex> l(mu_);
    return live_;
  }
  uint32_t capacity() {
    std::lock_guard<std::mutex> l(mu_);
    return static_cast<uint32_t>(chunks_.size()) * per_;
  }

 private:
  struct Slot {
    T obj{};
    uint32_t gen = 1;
    bool live = false;
  };
  Slot& slot(uint32_t idx) { return chunks_[idx / per_][idx % per_]; }
  const uint32_t per_;
  std::mutex mu_;
  std::vector<Slot*> chunks_;
  std::vector<uint32_t> free_;
  uint32_t live_ = 0;
};

// ----------------------------------------------------------------------------------------------------- timer wheel
// Two wheels of 256 slots: the near one turns once per 256 ticks, the far one holds what is further away and is
// emptied into the near wheel one slot per near-wheel turn. Timers are created once and started / restarted / stopped
// many times (the usual life of a keepalive or a retry timer); a periodic timer re-arms itself after it ran.
// run(now_ms) is called by ONE thread and runs the callbacks outside the lock; everything else is thread-safe.
class TimerWheel {
 public:
  using Fn = std::function<void()>;
  explicit TimerWheel(uint32_t tick_ms = 10, uint64_t start_ms = 0)
      : tick_(tick_ms ? tick_ms : 10), now_tick_(start_ms / (tick_ms ? tick_ms : 10)), near_(kSlots), far_(kSlots) {}

  uint32_t create(Fn fn) {
    std::lock_guard<std::mutex> l(mu_);
    uint32_t id = 0;
    for (; id < timers_.size(); ++id)
      if (!timers_[id].exists) break;
    if (id == timers_.size()) timers_.emplace_back();
    Timer& t = timers_[id];
    t = Timer();
    t.exists = true;
    t.fn = std::move(fn);
    return id + 1;
  }
  // Arms (or re-arms) the timer to fire `delay_ms` from the wheel's present time; at least one tick.
  bool start(uint32_t id, uint64_t delay_ms, bool periodic = false) {
    std::lock_guard<std::mutex> l(mu_);
    Timer* t = find(id);
    if (!t) return false;
    unlink(id - 1);
    t->period_ticks = ticks_of(delay_ms);
    t->periodic = periodic;
    link(id - 1, now_tick_ + t->period_ticks);
    return true;
  }
  bool stop(uint32_t id) {
    std::lock_guard<std::mutex> l(mu_);
    Timer* t = find(id);
    if (!t) return false;
    const bool was = t->armed;
    unlink(id - 1);
    return was;
  }
  bool destroy(uint32_t id) {
    std::lock_guard<std::mutex> l(mu_);
    Timer* t = find(id);
    if (!t) return false;
    unlink(id - 1);
    *t = Timer();
    return true;
  }
  bool armed(uint32_t id) {
    std::lock_guard<std::mutex> l(mu_);
    Timer* t = find(id);
    return t && t->armed;
  }
  // Advances the wheel to `now_ms` and runs every timer that became due, in order of its tick. Returns how many ran.
  int run(uint64_t now_ms) {
    int ran = 0;
    const uint64_t target = now_ms / tick_;
    for (;;) {
      std::vector<std::pair<uint32_t, Fn>> due;
      {
        std::lock_guard<std::mutex> l(mu_);
        if (now_tick_ >= target) break;
        ++now_tick_;
        if (now_tick_ % kSlots == 0) cascade();
        std::vector<uint32_t>& s = near_[now_tick_ % kSlots];
        std::vector<uint32_t> keep;
        for (uint32_t idx : s) {
          Timer& t = timers_[idx];
          if (!t.exists || !t.armed || t.slot_is_far) continue;
          if (t.expire > now_tick_) {   // belongs to a later turn (placed while the far wheel was bypassed)
            keep.push_back(idx);
            continue;
          }
          t.armed = false;
          due.emplace_back(idx, t.fn);
        }
        s.swap(keep);
        for (auto& d : due) {
          Timer& t = timers_[d.first];
          if (t.periodic) link(d.first, now_tick_ + t.period_ticks);
        }
      }
      for (auto& d : due)
        if (d.second) d.second();
      ran += static_cast<int>(due.size());
    }
    return ran;
  }
  uint32_t tick_ms() const { return tick_; }
  uint32_t armed_count() {
    std::lock_guard<std::mutex> l(mu_);
    uint32_t n = 0;
    for (auto& t : timers_) n += t.exists && t.armed;
    return n;
  }

 private:
  static constexpr uint32_t kSlots = 256;
  struct Timer {
    Fn fn;
    uint64_t expire = 0, period_ticks = 0;
    bool exists = false, armed = false, periodic = false, slot_is_far = false;
  };
  Timer* find(uint32_t id) {
    if (id == 0 || id > timers_.size() || !timers_[id - 1].exists) return nullptr;
    return &timers_[id - 1];
  }
  uint64_t ticks_of(uint64_t ms) const {
    const uint64_t t = (ms + tick_ - 1) / tick_;
    return t ? t : 1;
  }
  void link(uint32_t idx, uint64_t expire) {
    Timer& t = timers_[idx];
    t.expire = expire;
    t.armed = true;
    // same turn of the near wheel as now -> near; otherwise wait in the far wheel, by turn number
    t.slot_is_far = expire / kSlots != now_tick_ / kSlots;
    if (t.slot_is_far) far_[(expire / kSlots) % kSlots].push_back(idx);
    else near_[expire % kSlots].push_back(idx);
  }
  void unlink(uint32_t idx) {
    Timer& t = timers_[idx];
    if (!t.armed) return;
    std::vector<uint32_t>& s = t.slot_is_far ? far_[(t.expire / kSlots) % kSlots] : near_[t.expire % kSlots];
    for (size_t i = 0; i < s.size(); ++i)
      if (s[i] == idx) {
        s[i] = s.back();
        s.pop_back();
        break;
      }
    t.armed = false;
  }
  // A new turn of the near wheel begins: move this turn's timers out of the far wheel.
  void cascade() {
    const uint64_t turn = now_tick_ / kSlots;
    std::vector<uint32_t>& f = far_[turn % kSlots];
    std::vector<uint32_t> later;
    for (uint32_t idx : f) {
      Timer& t = timers_[idx];
      if (!t.exists || !t.armed || !t.slot_is_far) continue;
      if (t.expire / kSlots != turn) {   // a full turn of the far wheel further on
        later.push_back(idx);
        continue;
      }
      t.slot_is_far = false;
      near_[t.expire % kSlots].push_back(idx);
    }
    f.swap(later);
  }
  const uint32_t tick_;
  std::mutex mu_;
  uint64_t now_tick_;
  std::vector<Timer> timers_;
  std::vector<std::vector<uint32_t>> near_, far_;
};

}  // namespace urpc_util
