// Shared-memory layout of one accelerated UMS connection (one file per connection in the UMS directory) and the
// name of the handshake magic. Shared by the library and by ums_admin, which maps the files read-only.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>

namespace ums_shm {

constexpr uint32_t kClcMagic = 0x554d5331;  // "UMS1"
constexpr size_t kRingBytes = 1 << 20;      // per direction

struct Ring {
  std::atomic<uint64_t> prod;
  char pad0[56];
  std::atomic<uint64_t> cons;
  char pad1[56];
  std::atomic<uint32_t> closed;  // producer side shut down
  std::atomic<uint32_t> waiter;  // the consumer is (about to be) asleep on its descriptor: ring the doorbell
  char pad2[56];
  char data[kRingBytes];
};
struct ConnShm {
  Ring c2s;  // client -> server
  Ring s2c;
};

}  // namespace ums_shm
