// Wire header of URPC messages with explicit, endianness-independent packing.
// byte 0      version (high nibble) | message type (low nibble)
// byte 1      flags: bit0 ack requested, bit1 function-defined, bits 2..7 DMA descriptor count
// bytes 2..7  function id (48 bit, little endian)
// bytes 8..11 request id
// bytes 12..14 client channel (24 bit)    byte 15 status (responses)
// bytes 16..19 total size of the arguments / response
// bytes 20..31 reserved
#pragma once
#include <stdint.h>
#include <string.h>

#include "urpc_api.h"

namespace urpc_proto {
constexpr uint8_t kVersion = 1;
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
  return h->version == kVersion;
}
}  // namespace urpc_proto
