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

// A link: one shared-memory file that carries up to kLinkSlots connections between the same two processes plus a
// pair of small control rings (LLC messages). The connecting process creates the file and hands out the slots; all
// links between two processes form a link group (a second link is added when the first one's slots are used up).
// Counterpart of the reference's link groups with up to 32 connections per link and of its link-layer control
// messages (src/usock/ums/kmod/ums/cm/ums_core.c, cm/ums_llc.c: CONFIRM LINK, ADD LINK, DELETE LINK, TEST LINK).
constexpr uint32_t kLinkMagic = 0x554d534c;  // "UMSL"
constexpr uint32_t kLinkSlots = 32;
constexpr uint32_t kLlcEntries = 64;
enum LlcType : uint32_t {
  LLC_CONFIRM_LINK = 1,  // server -> client on a link's first connection; the answer makes the link ACTIVE
  LLC_ADD_LINK = 2,      // client -> server on an existing link: `name` is a further link of the group
  LLC_DELETE_LINK = 3,   // client -> server: the link's file is going away
  LLC_TEST_LINK = 4,     // either side: answered with the same seq (liveness of the peer's UMS layer)
  LLC_DELETE_CONN = 5,   // either side: the connection in `slot` was closed here
};
constexpr uint32_t kLlcResponse = 1;
struct LlcMsg {
  uint32_t type, flags, seq, slot;
  char name[48];
};
struct LlcRing {
  std::atomic<uint64_t> prod;
  char pad0[56];
  std::atomic<uint64_t> cons;
  char pad1[56];
  LlcMsg msg[kLlcEntries];
};
enum LinkState : uint32_t { LINK_CREATED = 0, LINK_ACTIVE = 1, LINK_DELETED = 2 };
struct LinkShm {
  uint32_t magic, version, owner_pid, slots;
  std::atomic<uint32_t> peer_pid;
  std::atomic<uint32_t> state;       // LinkState
  std::atomic<uint32_t> slot_used;   // bit per slot: handed out by the owner, cleared by whoever closes last
  std::atomic<uint32_t> closed_c;    // bit per slot: the client side closed the connection
  std::atomic<uint32_t> closed_s;    // ... the server side
  std::atomic<uint32_t> conns_total; // connections this link has carried
  char group[64];                    // name of the group's first link
  char pad[24];
  LlcRing llc_c2s, llc_s2c;
  ConnShm conn[kLinkSlots];
};

}  // namespace ums_shm
