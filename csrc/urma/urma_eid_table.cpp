// EID table and system-wide device settings, shared by every process of the box through one file in the URMA state
// directory, and the executor of the admin commands that change them.
//
// The reference keeps these in its kernel core and drives them from `urma_admin` over netlink: EID add / delete / mode
// (src/urma/tools/urma_admin/admin_cmd_eid.c), namespace mode and device sharing (admin_cmd_system.c). Here a device
// can carry up to 8 extra EIDs beside the one its provider reports (index 0); `urma_get_eid_list` shows them and
// `urma_create_context(dev, index)` gives the context that EID. Commands arrive as TLV messages (urma_cmd_tlv.h) so
// that the tool, tests and other front ends all speak one format; the reply is a TLV message with a status and text.
#include <fcntl.h>
#include <signal.h>
#include <stdio.h>
#include <sys/file.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <mutex>
#include <string>

#include "urma_api.h"
#include "urma_cmd_tlv.h"

namespace {

constexpr uint32_t kDevs = 64, kEidsPerDev = 8;
struct DevRec {
  char name[64];
  uint32_t used, eid_mode /* 0 static, 1 dynamic */, sharing /* 1 = several processes may open it */;
  uint32_t owner_pid; /* the process that holds an exclusive device (0 = nobody) */
  uint32_t eid_valid[kEidsPerDev];
  uint8_t eid[kEidsPerDev][16];
  uint64_t eid_ns[kEidsPerDev];
};
struct Table {
  uint32_t magic, ns_mode /* 0 exclusive, 1 shared */;
  DevRec dev[kDevs];
};
constexpr uint32_t kMagic = 0x44494555;  // "UEID"
constexpr int URMA_ENODEV = 19, URMA_ENOENT = 2;   // errno values the status enum has no name for

Table* g_tab = nullptr;
int g_fd = -1;
std::mutex g_mu;

Table* table() {
  std::lock_guard<std::mutex> l(g_mu);
  if (g_tab) return g_tab;
  const char* e = getenv("URMA_SHM_DIR");
  const std::string d = (e && *e) ? e : "/dev/shm/umdk_urma_" + std::to_string(getuid());
  mkdir(d.c_str(), 0700);
  const int fd = open((d + "/eid_table").c_str(), O_RDWR | O_CREAT, 0600);
  if (fd < 0) return nullptr;
  if (ftruncate(fd, sizeof(Table)) != 0) {
    close(fd);
    return nullptr;
  }
  void* p = mmap(nullptr, sizeof(Table), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  if (p == MAP_FAILED) {
    close(fd);
    return nullptr;
  }
  g_fd = fd;
  g_tab = static_cast<Table*>(p);
  flock(fd, LOCK_EX);
  if (g_tab->magic != kMagic) {
    memset(g_tab, 0, sizeof(Table));
    g_tab->ns_mode = 1;
    g_tab->magic = kMagic;
  }
  flock(fd, LOCK_UN);
  return g_tab;
}
struct FileLock {
  FileLock() { if (g_fd >= 0) flock(g_fd, LOCK_EX); }
  ~FileLock() { if (g_fd >= 0) flock(g_fd, LOCK_UN); }
};
DevRec* dev_rec(Table* t, const std::string& name, bool create) {
  DevRec* free_slot = nullptr;
  for (DevRec& d : t->dev) {
    if (d.used && name == d.name) return &d;
    if (!d.used && !free_slot) free_slot = &d;
  }
  if (!create || !free_slot || name.empty() || name.size() >= sizeof(free_slot->name)) return nullptr;
  memset(free_slot, 0, sizeof(*free_slot));
  memcpy(free_slot->name, name.data(), name.size());
  free_slot->used = 1;
  free_slot->sharing = 1;
  return free_slot;
}
bool device_exists(const std::string& name) { return urma_get_device_by_name(name.c_str()) != nullptr; }

std::vector<uint8_t> reply(int32_t status, const std::string& text) {
  return urma_tlv::Encoder(urma_tlv::CMD_REPLY).put_i32(urma_tlv::ATTR_STATUS, status)
      .put_str(urma_tlv::ATTR_TEXT, text).finish();
}

}  // namespace

// Extra EIDs of a device for urma_get_eid_list / urma_create_context. Returns how many were written (index i + 1).
extern "C" URMA_EXPORT int urma_eid_table_get(const char* dev_name, urma_eid_info_t* out, int max) {
  Table* t = table();
  if (!t || !dev_name) return 0;
  FileLock fl;
  DevRec* d = dev_rec(t, dev_name, false);
  if (!d) return 0;
  int n = 0;
  for (uint32_t i = 0; i < kEidsPerDev && n < max; ++i)
    if (d->eid_valid[i]) {
      memcpy(out[n].eid.raw, d->eid[i], 16);
      out[n].eid_index = i + 1;
      ++n;
    }
  return n;
}
// 1 when several processes may open the device (the default), 0 when the admin made it exclusive.
extern "C" URMA_EXPORT int urma_eid_table_sharing(const char* dev_name) {
  Table* t = table();
  if (!t || !dev_name) return 1;
  FileLock fl;
  DevRec* d = dev_rec(t, dev_name, false);
  return d ? (int)d->sharing : 1;
}

// A process opens a context on the device: always allowed on a shared device; on an exclusive one only while no other
// live process holds it. Returns 1 when the context may be created.
extern "C" URMA_EXPORT int urma_eid_table_claim(const char* dev_name) {
  Table* t = table();
  if (!t || !dev_name) return 1;
  FileLock fl;
  DevRec* d = dev_rec(t, dev_name, false);
  if (!d || d->sharing) return 1;
  const uint32_t me = static_cast<uint32_t>(getpid());
  if (d->owner_pid == 0 || d->owner_pid == me || kill(static_cast<pid_t>(d->owner_pid), 0) != 0) {
    d->owner_pid = me;
    return 1;
  }
  return 0;
}

// Executes one TLV command; the TLV reply is written to `out` (up to *out_len bytes, *out_len = bytes written).
// Returns 0 when a reply was produced (its status attribute says whether the command worked), -1 on a malformed
// command or a reply buffer that is too small.
extern "C" URMA_EXPORT int urma_admin_cmd_exec(const uint8_t* cmd, uint32_t len, uint8_t* out, uint32_t* out_len) {
  urma_tlv::Decoder d;
  if (!out || !out_len || !d.parse(cmd, len)) return -1;
  Table* t = table();
  std::vector<uint8_t> r;
  if (!t) {
    r = reply(-URMA_FAIL, "no state directory");
  } else {
    FileLock fl;
    std::string dev;
    d.get_str(urma_tlv::ATTR_DEV_NAME, &dev);
    uint32_t idx = 0, flag = 0;
    const bool have_idx = d.get_u32(urma_tlv::ATTR_EID_INDEX, &idx);
    d.get_u32(urma_tlv::ATTR_FLAG, &flag);
    switch (d.command()) {
      case urma_tlv::CMD_EID_ADD: {
        const urma_tlv::Attr* e = d.find(urma_tlv::ATTR_EID);
        uint64_t ns = 0;
        d.get_u64(urma_tlv::ATTR_NS, &ns);
        if (!device_exists(dev)) r = reply(-URMA_ENODEV, "no such device: " + dev);
        else if (!e || e->value.size() != 16) r = reply(-URMA_EINVAL, "an EID is 16 bytes");
        else {
          DevRec* rec = dev_rec(t, dev, true);
          int slot = -1;
          if (rec && have_idx) slot = (idx >= 1 && idx <= kEidsPerDev && !rec->eid_valid[idx - 1]) ? (int)idx - 1 : -1;
          else if (rec)
            for (uint32_t i = 0; i < kEidsPerDev && slot < 0; ++i)
              if (!rec->eid_valid[i]) slot = (int)i;
          bool dup = false;
          for (uint32_t i = 0; rec && i < kEidsPerDev; ++i)
            dup |= rec->eid_valid[i] && !memcmp(rec->eid[i], e->value.data(), 16);
          if (!rec || slot < 0) r = reply(-URMA_EAGAIN, "no free EID index (1..8) on " + dev);
          else if (dup) r = reply(-URMA_EEXIST, "EID already present on " + dev);
          else if (rec->eid_mode == 1 && have_idx) r = reply(-URMA_EINVAL, dev + " assigns EID indexes dynamically");
          else {
            memcpy(rec->eid[slot], e->value.data(), 16);
            rec->eid_ns[slot] = ns;
            rec->eid_valid[slot] = 1;
            r = reply(0, "eid index " + std::to_string(slot + 1));
          }
        }
        break;
      }
      case urma_tlv::CMD_EID_DEL: {
        DevRec* rec = dev_rec(t, dev, false);
        if (!rec || !have_idx || idx < 1 || idx > kEidsPerDev || !rec->eid_valid[idx - 1])
          r = reply(-URMA_ENOENT, "no such EID index");
        else {
          rec->eid_valid[idx - 1] = 0;
          r = reply(0, "deleted");
        }
        break;
      }
      case urma_tlv::CMD_EID_MODE: {
        if (!device_exists(dev)) r = reply(-URMA_ENODEV, "no such device: " + dev);
        else {
          DevRec* rec = dev_rec(t, dev, true);
          if (!rec) r = reply(-URMA_EAGAIN, "device table full");
          else {
            rec->eid_mode = flag ? 1 : 0;
            r = reply(0, flag ? "dynamic" : "static");
          }
        }
        break;
      }
      case urma_tlv::CMD_SHARING: {
        if (!device_exists(dev)) r = reply(-URMA_ENODEV, "no such device: " + dev);
        else {
          DevRec* rec = dev_rec(t, dev, true);
          if (!rec) r = reply(-URMA_EAGAIN, "device table full");
          else {
            rec->sharing = flag ? 1 : 0;
            rec->owner_pid = 0;
            r = reply(0, flag ? "shared" : "exclusive");
          }
        }
        break;
      }
      case urma_tlv::CMD_NS_MODE:
        t->ns_mode = flag ? 1 : 0;
        r = reply(0, flag ? "shared" : "exclusive");
        break;
      case urma_tlv::CMD_EID_SHOW:
      case urma_tlv::CMD_SYSTEM_SHOW: {
        std::string s;
        char line[256];
        if (d.command() == urma_tlv::CMD_SYSTEM_SHOW) {
          snprintf(line, sizeof(line), "namespace mode: %s\n", t->ns_mode ? "shared" : "exclusive");
          s += line;
        }
        for (DevRec& rec : t->dev) {
          if (!rec.used || (!dev.empty() && dev != rec.name)) continue;
          snprintf(line, sizeof(line), "%s: eid mode %s, %s\n", rec.name, rec.eid_mode ? "dynamic" : "static",
                   rec.sharing ? "shared" : "exclusive");
          s += line;
          for (uint32_t i = 0; i < kEidsPerDev; ++i)
            if (rec.eid_valid[i]) {
              urma_eid_t e;
              memcpy(e.raw, rec.eid[i], 16);
              char txt[64];
              urma_eid_to_str(&e, txt, sizeof(txt));
              snprintf(line, sizeof(line), "  [%u] %s ns %llu\n", i + 1, txt, (unsigned long long)rec.eid_ns[i]);
              s += line;
            }
        }
        r = reply(0, s);
        break;
      }
      default: r = reply(-URMA_EINVAL, "unknown command");
    }
  }
  if (r.size() > *out_len) return -1;
  memcpy(out, r.data(), r.size());
  *out_len = static_cast<uint32_t>(r.size());
  return 0;
}
