// Sliding window over message sequence numbers: accepts each number once, tolerates reordering inside the window,
// rejects duplicates and numbers that fell behind the window. Used by the bond provider to drop the second copy of a
// message that was re-sent on another path after its first copy had in fact arrived (same purpose as the reference's
// src/urma/lib/urma/bond/utils/bondp_slide_window.h:36-49).
#pragma once
#include <stdint.h>

namespace bond {

class SlideWindow {
 public:
  static constexpr uint32_t kBits = 1024;
  // Returns true when `msn` is new (and records it), false for a duplicate or a too-old number.
  bool accept(uint32_t msn) {
    if (!started_) {
      started_ = true;
      base_ = msn;
    }
    const int32_t d = static_cast<int32_t>(msn - base_);
    if (d < 0) return false;  // behind the window: treated as already seen
    if (static_cast<uint32_t>(d) >= kBits) {
      // slide forward so that msn becomes the newest element of the window
      const uint32_t shift = static_cast<uint32_t>(d) - kBits + 1;
      if (shift >= kBits) {
        for (auto& w : bits_) w = 0;
      } else {
        for (uint32_t i = 0; i < shift; ++i) clear((base_ + i) % kBits);
      }
      base_ += shift;
    }
    const uint32_t slot = msn % kBits;
    if (test(slot)) return false;
    set(slot);
    // advance the base over the contiguous prefix of seen numbers (keeps the window as far forward as possible)
    while (test(base_ % kBits) && static_cast<int32_t>(msn - base_) > static_cast<int32_t>(kBits / 2)) {
      clear(base_ % kBits);
      ++base_;
    }
    return true;
  }
  uint32_t base() const { return base_; }

 private:
  bool test(uint32_t i) const { return (bits_[i >> 6] >> (i & 63)) & 1u; }
  void set(uint32_t i) { bits_[i >> 6] |= (uint64_t(1) << (i & 63)); }
  void clear(uint32_t i) { bits_[i >> 6] &= ~(uint64_t(1) << (i & 63)); }
  uint64_t bits_[kBits / 64] = {0};
  uint32_t base_ = 0;
  bool started_ = false;
};

}  // namespace bond
