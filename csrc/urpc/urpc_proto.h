// Wire header of URPC messages with explicit, endianness-independent packing.
// byte 0      version (high nibble) | message type (low nibble)
// byte 1      flags: bit0 ack requested, bit1 function-defined, bits 2..7 DMA descriptor count
// bytes 2..7  function id (48 bit, little endian)
// bytes 8..11 request id
// bytes 12..14 client channel (24 bit)    byte 15 status (responses)
// bytes 16..19 total size of the arguments / response
// bytes 20..27 message counter of a sealed message, bytes 28..31 reserved
//
// Protocol version 2 keeps that 32-byte envelope for every message (the counter of a sealed message has to sit at
// one place) and defines, inside it, one layout per message kind - the request head above plus
//   ACK head   byte 0 version|type(ACK)  byte 1 reserved  bytes 2..3 request-id range (how many consecutive ids,
//              starting at `request id`, this acknowledgement covers)  bytes 8..11 first request id
//              bytes 12..14 client channel
//   RSP head   byte 0 version|type(RSP or ACK_AND_RSP)  byte 1 flags  bytes 2..3 request-id range
//              bytes 4..7 function-defined word  bytes 8..11 request id  bytes 12..14 client channel  byte 15 status
//              bytes 16..19 response size
// (reference: src/urpc/framework/protocol/protocol.h urpc_req_head / urpc_ack_head / urpc_rsp_head), and a set of
// control messages that travel on the channel's control connection after the attach (CtlHead below; reference:
// the urpc_ctl_opcode set of the same file). Version 1 peers know the request layout only, no acknowledgements and
// no control messages after the attach; the attach negotiates the version both sides then use (see Negotiation).
#pragma once
#include <stdint.h>
#include <string.h>

#include "urpc_api.h"

namespace urpc_proto {
constexpr uint8_t kVersionMin = 1;   // oldest protocol this build still speaks
constexpr uint8_t kVersion = 2;      // newest
struct Head {
  uint8_t version, type, flags;
  uint64_t func_id;
  uint32_t req_id, channel, total_size;
  int8_t status;
};
inline void put_le(uint8_t* p, uint64_t v, int n) {
  for (int i = 0; i < n; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}
inline uint64_t get_le(const uint8_t* p, int n) {
  uint64_t v = 0;
  for (int i = 0; i < n; ++i) v |= uint64_t(p[i]) << (8 * i);
  return v;
}
inline void encode(const Head& h, urpc_req_head_t* out) {
  memset(out->bytes, 0, sizeof(out->bytes));
  out->bytes[0] = static_cast<uint8_t>((h.version << 4) | (h.type & 0xf));
  out->bytes[1] = h.flags;
  put_le(out->bytes + 2, h.func_id & 0xFFFFFFFFFFFFull, 6);
  put_le(out->bytes + 8, h.req_id, 4);
  put_le(out->bytes + 12, h.channel & 0xFFFFFF, 3);
  out->bytes[15] = static_cast<uint8_t>(h.status);
  put_le(out->bytes + 16, h.total_size, 4);
}
inline bool decode(const urpc_req_head_t* in, Head* h) {
  h->version = in->bytes[0] >> 4;
  h->type = in->bytes[0] & 0xf;
  h->flags = in->bytes[1];
  h->func_id = get_le(in->bytes + 2, 6);
  h->req_id = static_cast<uint32_t>(get_le(in->bytes + 8, 4));
  h->channel = static_cast<uint32_t>(get_le(in->bytes + 12, 3));
  h->status = static_cast<int8_t>(in->bytes[15]);
  h->total_size = static_cast<uint32_t>(get_le(in->bytes + 16, 4));
  return h->version >= kVersionMin && h->version <= kVersion;
}

// ---------------------------------------------------------------------------------------------- ACK / RSP layouts
struct AckHead {
  uint8_t version;
  uint16_t req_id_range;
  uint32_t req_id, channel;
};
inline void encode_ack(const AckHead& a, urpc_req_head_t* out) {
  memset(out->bytes, 0, sizeof(out->bytes));
  out->bytes[0] = static_cast<uint8_t>((a.version << 4) | URPC_MSG_ACK);
  put_le(out->bytes + 2, a.req_id_range, 2);
  put_le(out->bytes + 8, a.req_id, 4);
  put_le(out->bytes + 12, a.channel & 0xFFFFFF, 3);
}
inline bool decode_ack(const urpc_req_head_t* in, AckHead* a) {
  if ((in->bytes[0] & 0xf) != URPC_MSG_ACK) return false;
  a->version = in->bytes[0] >> 4;
  a->req_id_range = static_cast<uint16_t>(get_le(in->bytes + 2, 2));
  a->req_id = static_cast<uint32_t>(get_le(in->bytes + 8, 4));
  a->channel = static_cast<uint32_t>(get_le(in->bytes + 12, 3));
  return a->version >= 2 && a->version <= kVersion && a->req_id_range >= 1;
}
struct RspHead {
  uint8_t version, type, flags;
  uint16_t req_id_range;
  uint32_t function_defined, req_id, channel, total_size;
  int8_t status;
};
inline void encode_rsp(const RspHead& r, urpc_req_head_t* out) {
  memset(out->bytes, 0, sizeof(out->bytes));
  out->bytes[0] = static_cast<uint8_t>((r.version << 4) | (r.type & 0xf));
  out->bytes[1] = r.flags;
  put_le(out->bytes + 2, r.req_id_range, 2);
  put_le(out->bytes + 4, r.function_defined, 4);
  put_le(out->bytes + 8, r.req_id, 4);
  put_le(out->bytes + 12, r.channel & 0xFFFFFF, 3);
  out->bytes[15] = static_cast<uint8_t>(r.status);
  put_le(out->bytes + 16, r.total_size, 4);
}
inline bool decode_rsp(const urpc_req_head_t* in, RspHead* r) {
  r->version = in->bytes[0] >> 4;
  r->type = in->bytes[0] & 0xf;
  if (r->type != URPC_MSG_RSP && r->type != URPC_MSG_ACK_AND_RSP) return false;
  r->flags = in->bytes[1];
  r->req_id_range = static_cast<uint16_t>(get_le(in->bytes + 2, 2));
  r->function_defined = static_cast<uint32_t>(get_le(in->bytes + 4, 4));
  r->req_id = static_cast<uint32_t>(get_le(in->bytes + 8, 4));
  r->channel = static_cast<uint32_t>(get_le(in->bytes + 12, 3));
  r->status = static_cast<int8_t>(in->bytes[15]);
  r->total_size = static_cast<uint32_t>(get_le(in->bytes + 16, 4));
  return r->version >= kVersionMin && r->version <= kVersion;
}

// ------------------------------------------------------------------------------------------------- negotiation
// The attach hello carries, in its 32-bit version word, the newest version the sender speaks (bits 0..7), the oldest
// (bits 8..15) and its capability bits (16..31). A version-1 build put the plain number 1 there: oldest = 0 reads as
// "only `newest`", capabilities none. The answer carries the chosen version (the newest both speak) and the
// capabilities both have; 0 = no common version, the attach fails on both sides.
// (reference: src/urpc/framework/lib/control/cp_vers_compat.c keeps old and new peers attachable the same way.)
constexpr uint32_t kCapLiveQueues = 1u << 0;   // queues may join / leave an attached channel (control messages)
constexpr uint32_t kCapAck = 1u << 1;          // the server acknowledges deferred requests that ask for it
constexpr uint32_t kCapTaskCancel = 1u << 2;   // a cancelled call is also dropped on the server
constexpr uint32_t kCapsAll = kCapLiveQueues | kCapAck | kCapTaskCancel;
inline uint32_t pack_version(uint8_t newest, uint8_t oldest, uint32_t caps) {
  return uint32_t(newest) | (uint32_t(oldest) << 8) | ((caps & 0xffff) << 16);
}
struct Negotiated {
  uint8_t version = 0;   // 0 = none in common
  uint32_t caps = 0;
};
inline Negotiated negotiate(uint32_t mine, uint32_t theirs) {
  auto newest = [](uint32_t w) { return uint8_t(w & 0xff); };
  auto oldest = [](uint32_t w) { return uint8_t((w >> 8) & 0xff) ? uint8_t((w >> 8) & 0xff) : uint8_t(w & 0xff); };
  Negotiated n;
  const uint8_t hi = newest(mine) < newest(theirs) ? newest(mine) : newest(theirs);
  const uint8_t lo = oldest(mine) > oldest(theirs) ? oldest(mine) : oldest(theirs);
  if (hi == 0 || hi < lo) return n;
  n.version = hi;
  n.caps = hi >= 2 ? ((mine >> 16) & (theirs >> 16)) : 0;   // version 1 has no optional parts
  return n;
}

// ------------------------------------------------------------------------------------------- control messages
// Sent on the control connection of an attached channel (version >= 2). A request and its answer share `seq`; the
// answer has kCtlAnswer set and carries the outcome in `status` (0 or a negative URPC_ERR_* value).
constexpr uint32_t kCtlMagic = 0x4354524c;   // "CTRL"
constexpr uint16_t kCtlAnswer = 1;
constexpr uint32_t kCtlMaxPayload = 4096;
enum CtlOpcode : uint16_t {
  kCtlQueueAdd = 1,      // payload: lane id (u32), bind blob length (u32), blob; answer: the server queue's blob
  kCtlQueueRm = 2,       // payload: lane id (u32)
  kCtlTaskCancel = 3,    // payload: request id (u32): a deferred request not yet answered is dropped
  kCtlDetach = 4,        // no payload: the session is retired at once instead of when the connection drops
  kCtlFuncChange = 5,    // server -> client notice, no answer: the function table changed (payload: u64 id, u32 added)
};
struct CtlHead {
  uint32_t magic;
  uint16_t opcode, flags;
  uint32_t seq;
  int32_t status;
  uint32_t len;
};
static_assert(sizeof(CtlHead) == 20, "control head is 20 bytes on the wire");
}  // namespace urpc_proto
