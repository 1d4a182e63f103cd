/* Command messages of the URMA control path as type-length-value records.
 *
 * In the reference every control call crosses into the kernel as one command whose arguments are a list of typed
 * attributes (src/urma/lib/urma/core/urma_cmd_tlv.c: command header + attribute array, each attribute with a type, a
 * field size and an element count). Here the "other side" is the device registry that the user-space providers and
 * the admin tool share (urma_admin_cmd_exec in urma_eid_table.cpp); the wire form is kept: a command is
 *   header  { magic u32, command u32, n_attrs u32, total_bytes u32 }
 *   attr    { type u16, flags u16, len u32, value[len] padded to 8 bytes } ...
 * Values are little-endian scalars, strings without terminator, or opaque byte arrays. A decoder rejects truncated
 * input, attributes that run past the end, and duplicate scalar attributes. */
#ifndef UMDK_URMA_CMD_TLV_H
#define UMDK_URMA_CMD_TLV_H

#include <stdint.h>
#include <string.h>

#include <string>
#include <vector>

namespace urma_tlv {

constexpr uint32_t kMagic = 0x564c5455; /* "UTLV" */

enum Command : uint32_t {
  CMD_EID_ADD = 1,
  CMD_EID_DEL = 2,
  CMD_EID_SHOW = 3,
  CMD_EID_MODE = 4,   /* static / dynamic EID assignment of a device */
  CMD_NS_MODE = 5,    /* exclusive / shared device visibility between namespaces */
  CMD_SHARING = 6,    /* a device may / may not be opened by several processes at once */
  CMD_SYSTEM_SHOW = 7,
  CMD_REPLY = 100,
};
enum AttrType : uint16_t {
  ATTR_DEV_NAME = 1,   /* string */
  ATTR_EID = 2,        /* 16 bytes */
  ATTR_EID_INDEX = 3,  /* u32 */
  ATTR_FLAG = 4,       /* u32 */
  ATTR_NS = 5,         /* u64: namespace id (inode of the caller's network namespace) */
  ATTR_STATUS = 6,     /* i32 (replies) */
  ATTR_TEXT = 7,       /* string (replies) */
};

struct Attr {
  uint16_t type = 0, flags = 0;
  std::vector<uint8_t> value;
};

class Encoder {
 public:
  explicit Encoder(uint32_t command) : command_(command) {}
  Encoder& put_bytes(uint16_t type, const void* p, size_t n) {
    Attr a;
    a.type = type;
    a.value.assign(static_cast<const uint8_t*>(p), static_cast<const uint8_t*>(p) + n);
    attrs_.push_back(std::move(a));
    return *this;
  }
  Encoder& put_u32(uint16_t type, uint32_t v) { return put_bytes(type, &v, 4); }
  Encoder& put_u64(uint16_t type, uint64_t v) { return put_bytes(type, &v, 8); }
  Encoder& put_i32(uint16_t type, int32_t v) { return put_bytes(type, &v, 4); }
  Encoder& put_str(uint16_t type, const std::string& s) { return put_bytes(type, s.data(), s.size()); }
  std::vector<uint8_t> finish() const {
    std::vector<uint8_t> out(16);
    for (const Attr& a : attrs_) {
      const uint32_t len = static_cast<uint32_t>(a.value.size());
      const size_t at = out.size();
      out.resize(at + 8 + ((len + 7) & ~7u));
      memcpy(&out[at], &a.type, 2);
      memcpy(&out[at + 2], &a.flags, 2);
      memcpy(&out[at + 4], &len, 4);
      if (len) memcpy(&out[at + 8], a.value.data(), len);
    }
    const uint32_t n = static_cast<uint32_t>(attrs_.size()), total = static_cast<uint32_t>(out.size());
    memcpy(&out[0], &kMagic, 4);
    memcpy(&out[4], &command_, 4);
    memcpy(&out[8], &n, 4);
    memcpy(&out[12], &total, 4);
    return out;
  }

 private:
  uint32_t command_;
  std::vector<Attr> attrs_;
};

class Decoder {
 public:
  /* false when the buffer is not a well-formed command */
  bool parse(const uint8_t* p, size_t n) {
    attrs_.clear();
    if (!p || n < 16) return false;
    uint32_t magic, cnt, total;
    memcpy(&magic, p, 4);
    memcpy(&command_, p + 4, 4);
    memcpy(&cnt, p + 8, 4);
    memcpy(&total, p + 12, 4);
    if (magic != kMagic || total != n || cnt > 1024) return false;
    size_t at = 16;
    for (uint32_t i = 0; i < cnt; ++i) {
      if (at + 8 > n) return false;
      Attr a;
      uint32_t len;
      memcpy(&a.type, p + at, 2);
      memcpy(&a.flags, p + at + 2, 2);
      memcpy(&len, p + at + 4, 4);
      const size_t padded = (static_cast<size_t>(len) + 7) & ~size_t(7);
      if (len > n || at + 8 + padded > n) return false;
      for (const Attr& o : attrs_)
        if (o.type == a.type) return false;
      a.value.assign(p + at + 8, p + at + 8 + len);
      attrs_.push_back(std::move(a));
      at += 8 + padded;
    }
    return at == n;
  }
  uint32_t command() const { return command_; }
  const Attr* find(uint16_t type) const {
    for (const Attr& a : attrs_)
      if (a.type == type) return &a;
    return nullptr;
  }
  bool get_u32(uint16_t type, uint32_t* v) const {
    const Attr* a = find(type);
    if (!a || a->value.size() != 4) return false;
    memcpy(v, a->value.data(), 4);
    return true;
  }
  bool get_u64(uint16_t type, uint64_t* v) const {
    const Attr* a = find(type);
    if (!a || a->value.size() != 8) return false;
    memcpy(v, a->value.data(), 8);
    return true;
  }
  bool get_i32(uint16_t type, int32_t* v) const { return get_u32(type, reinterpret_cast<uint32_t*>(v)); }
  bool get_str(uint16_t type, std::string* s) const {
    const Attr* a = find(type);
    if (!a) return false;
    s->assign(a->value.begin(), a->value.end());
    return true;
  }

 private:
  uint32_t command_ = 0;
  std::vector<Attr> attrs_;
};

}  // namespace urma_tlv
#endif
