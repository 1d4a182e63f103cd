// Hashed timing wheel for the bond provider's deferred work: the pause before a stored work request is resent on
// another path (so that a burst of failures does not hammer the survivors) and the schedule of failback probes.
// Tasks hang in `slots` buckets of `tick_ms` each; a task further away than one turn of the wheel carries the number of
// turns left. `advance()` is called by one thread (the bond context's timer thread) and runs what has become due
// outside the lock; `schedule()` and `cancel()` may be called from any thread. Every scheduled task runs exactly once:
// executed when due, or cancelled (by `cancel` or by the destructor) - the callback is told which.
// Same contract as the reference's timing wheel (src/urma/lib/urma/bond/utils/bondp_timewheel.h:26-66).
#pragma once
#include <stdint.h>

#include <functional>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace bond {

class TimeWheel {
 public:
  enum Reason { kExecuted = 0, kCanceled = 1 };
  using Fn = std::function<void(Reason)>;

  explicit TimeWheel(uint32_t tick_ms = 10, uint32_t slots = 256)
      : tick_ms_(tick_ms ? tick_ms : 10), slots_(slots ? slots : 256), wheel_(slots_ ? slots_ : 256) {}
  ~TimeWheel() {
    std::vector<Fn> left;
    {
      std::lock_guard<std::mutex> l(mu_);
      for (auto& s : wheel_)
        for (auto& t : s) left.push_back(std::move(t.fn));
      for (auto& s : wheel_) s.clear();
      index_.clear();
    }
    for (auto& f : left) f(kCanceled);
  }

  // Runs `fn` after `delay_ms` (at least one tick). Returns the task id (never 0).
  uint64_t schedule(uint64_t delay_ms, Fn fn) {
    std::lock_guard<std::mutex> l(mu_);
    uint64_t ticks = (delay_ms + tick_ms_ - 1) / tick_ms_;
    if (ticks == 0) ticks = 1;
    const uint32_t slot = static_cast<uint32_t>((cursor_ + ticks) % slots_);
    Task t;
    t.id = ++next_id_;
    t.turns = (ticks - 1) / slots_;
    t.fn = std::move(fn);
    wheel_[slot].push_back(std::move(t));
    index_[next_id_] = slot;
    return next_id_;
  }

  // True when the task was still pending (its callback has then been called with kCanceled).
  bool cancel(uint64_t id) {
    Fn fn;
    {
      std::lock_guard<std::mutex> l(mu_);
      auto it = index_.find(id);
      if (it == index_.end()) return false;
      auto& s = wheel_[it->second];
      for (auto t = s.begin(); t != s.end(); ++t)
        if (t->id == id) {
          fn = std::move(t->fn);
          s.erase(t);
          break;
        }
      index_.erase(it);
    }
    if (fn) fn(kCanceled);
    return static_cast<bool>(fn);
  }

  // Moves the wheel forward by `ticks` ticks and runs everything that became due. Returns how many tasks ran.
  int advance(uint32_t ticks = 1) {
    int ran = 0;
    for (uint32_t k = 0; k < ticks; ++k) {
      std::vector<Fn> due;
      {
        std::lock_guard<std::mutex> l(mu_);
        cursor_ = (cursor_ + 1) % slots_;
        auto& s = wheel_[cursor_];
        for (auto t = s.begin(); t != s.end();) {
          if (t->turns == 0) {
            due.push_back(std::move(t->fn));
            index_.erase(t->id);
            t = s.erase(t);
          } else {
            --t->turns;
            ++t;
          }
        }
      }
      for (auto& f : due) f(kExecuted);
      ran += static_cast<int>(due.size());
    }
    return ran;
  }

  size_t pending() {
    std::lock_guard<std::mutex> l(mu_);
    return index_.size();
  }
  uint32_t tick_ms() const { return tick_ms_; }

 private:
  struct Task {
    uint64_t id = 0;
    uint64_t turns = 0;
    Fn fn;
  };
  const uint32_t tick_ms_, slots_;
  std::mutex mu_;
  std::vector<std::list<Task>> wheel_;
  std::unordered_map<uint64_t, uint32_t> index_;
  uint64_t cursor_ = 0, next_id_ = 0;
};

}  // namespace bond
