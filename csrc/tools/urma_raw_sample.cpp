// urma_raw_sample: the bring-up sequence of the URMA API without the urma_simple wrapper, as a program that talks
// to itself: two contexts on one device, a jetty and a registered segment on each side, the identifiers handed over
// in memory (a real pair of programs sends them over TCP), then a write, a read, a send into a posted receive and a
// fetch-add, each checked. It is the program that docs/migration_from_verbs.md walks through; the canonical
// client/server sample of the reference has the same steps (src/urma/tools/urma_sample).
//   urma_raw_sample [--dev shm0]
#include <stdio.h>
#include <string.h>

#include <vector>

#include "urma_api.h"

static int fail(const char* what) {
  fprintf(stderr, "urma_raw_sample: FAILED: %s\n", what);
  return 1;
}
struct Side {
  urma_context_t* ctx = nullptr;
  urma_jfc_t* jfc = nullptr;
  urma_jetty_t* jetty = nullptr;
  urma_target_seg_t* seg = nullptr;
  std::vector<uint8_t> mem;
};
static bool make_side(Side* s, urma_device_t* dev, uint32_t jetty_token, uint32_t seg_token) {
  s->ctx = urma_create_context(dev, 0);
  if (!s->ctx) return false;
  urma_jfc_cfg_t cc{};
  cc.depth = 64;
  s->jfc = urma_create_jfc(s->ctx, &cc);
  urma_jetty_cfg_t jc{};
  jc.jfs_cfg.depth = 16;
  jc.jfs_cfg.trans_mode = URMA_TM_RM;
  jc.jfs_cfg.jfc = s->jfc;
  jc.jfr_cfg.depth = 16;
  jc.jfr_cfg.trans_mode = URMA_TM_RM;
  jc.jfr_cfg.jfc = s->jfc;
  jc.jfr_cfg.token_value.token = jetty_token;   // senders must present it
  s->jetty = s->jfc ? urma_create_jetty(s->ctx, &jc) : nullptr;
  s->mem.assign(8192, 0);
  urma_seg_cfg_t sc{};
  sc.va = reinterpret_cast<uint64_t>(s->mem.data());
  sc.len = s->mem.size();
  sc.access = URMA_ACCESS_READ | URMA_ACCESS_WRITE | URMA_ACCESS_ATOMIC;
  sc.token_value.token = seg_token;
  s->seg = urma_register_seg(s->ctx, &sc);
  return s->jetty && s->seg;
}
// Waits for one completion on `jfc`; the record must be a success of the expected kind.
static bool reap(urma_jfc_t* jfc, bool recv_side, urma_cr_t* cr) {
  for (int spins = 0; spins < 200000000; ++spins) {
    if (urma_poll_jfc(jfc, 1, cr) == 1)
      return cr->status == URMA_CR_SUCCESS && ((cr->flag & URMA_CR_FLAG_RECV) != 0) == recv_side;
  }
  return false;
}

int main(int argc, char** argv) {
  const char* dev_name = "shm0";
  for (int i = 1; i + 1 < argc; ++i)
    if (!strcmp(argv[i], "--dev")) dev_name = argv[i + 1];
  urma_init_attr_t ia{};
  if (urma_init(&ia) != URMA_SUCCESS) return fail("urma_init");
  urma_device_t* dev = urma_get_device_by_name(dev_name);
  if (!dev) return fail("no such device");
  Side a, b;
  if (!make_side(&a, dev, 0x1111, 0x2222) || !make_side(&b, dev, 0x3333, 0x4444)) return fail("bring-up");

  // what the two sides exchange out of band: b's jetty id and segment (and the token values, agreed beforehand)
  urma_rjetty_t rj{};
  rj.jetty_id = b.jetty->jetty_id;
  rj.trans_mode = URMA_TM_RM;
  rj.type = 1;   // a jetty
  urma_token_t jt{0x3333}, st{0x4444}, wrong{0x9999};
  urma_target_jetty_t* tj = urma_import_jetty(a.ctx, &rj, &jt);
  urma_target_seg_t* rseg = urma_import_seg(a.ctx, &b.seg->seg, &st, 0, 0);
  if (!tj || !rseg) return fail("import");

  urma_cr_t cr{};
  urma_jfs_wr_t wr{}, *bad = nullptr;
  // ---- write 1000 bytes into b's segment at offset 100
  for (int i = 0; i < 1000; ++i) a.mem[i] = static_cast<uint8_t>(i * 3 + 1);
  urma_sge_t src{reinterpret_cast<uint64_t>(a.mem.data()), 1000, a.seg};
  urma_sge_t dst{rseg->seg.ubva.va + 100, 1000, rseg};
  wr.opcode = URMA_OPC_WRITE;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.user_ctx = 42;
  wr.rw.src.sge = &src;
  wr.rw.src.num_sge = 1;
  wr.rw.dst.sge = &dst;
  wr.rw.dst.num_sge = 1;
  if (urma_post_jetty_send_wr(a.jetty, &wr, &bad) != URMA_SUCCESS || !reap(a.jfc, false, &cr) || cr.user_ctx != 42)
    return fail("write");
  if (memcmp(b.mem.data() + 100, a.mem.data(), 1000)) return fail("written bytes");
  // ---- read them back into a's buffer at offset 4096
  urma_sge_t rsrc{rseg->seg.ubva.va + 100, 1000, rseg};
  urma_sge_t rdst{reinterpret_cast<uint64_t>(a.mem.data() + 4096), 1000, a.seg};
  wr = urma_jfs_wr_t{};
  wr.opcode = URMA_OPC_READ;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.rw.src.sge = &rsrc;
  wr.rw.src.num_sge = 1;
  wr.rw.dst.sge = &rdst;
  wr.rw.dst.num_sge = 1;
  if (urma_post_jetty_send_wr(a.jetty, &wr, &bad) != URMA_SUCCESS || !reap(a.jfc, false, &cr)) return fail("read");
  if (memcmp(a.mem.data() + 4096, a.mem.data(), 1000)) return fail("read bytes");
  // ---- two-sided: b posts a receive, a sends 64 bytes with immediate data
  urma_sge_t rbuf{reinterpret_cast<uint64_t>(b.mem.data() + 2048), 256, b.seg};
  urma_jfr_wr_t rwr{}, *rbad = nullptr;
  rwr.src.sge = &rbuf;
  rwr.src.num_sge = 1;
  rwr.user_ctx = 7;
  if (urma_post_jetty_recv_wr(b.jetty, &rwr, &rbad) != URMA_SUCCESS) return fail("post receive");
  urma_sge_t ssrc{reinterpret_cast<uint64_t>(a.mem.data()), 64, a.seg};
  wr = urma_jfs_wr_t{};
  wr.opcode = URMA_OPC_SEND_IMM;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.send.src.sge = &ssrc;
  wr.send.src.num_sge = 1;
  wr.send.imm_data = 0xabcdef0123ull;
  if (urma_post_jetty_send_wr(a.jetty, &wr, &bad) != URMA_SUCCESS) return fail("send");
  if (!reap(b.jfc, true, &cr) || cr.user_ctx != 7 || cr.completion_len != 64 || cr.imm_data != 0xabcdef0123ull ||
      cr.remote_id.id != a.jetty->jetty_id.id)
    return fail("receive completion");
  if (memcmp(b.mem.data() + 2048, a.mem.data(), 64) || !reap(a.jfc, false, &cr)) return fail("sent bytes");
  // ---- fetch-add on an 8-byte word of b's segment; the old value comes back into a's buffer
  memset(b.mem.data() + 4096, 0, 8);
  b.mem[4096] = 5;
  urma_sge_t adst{rseg->seg.ubva.va + 4096, 8, rseg};
  urma_sge_t aold{reinterpret_cast<uint64_t>(a.mem.data() + 6000), 8, a.seg};
  wr = urma_jfs_wr_t{};
  wr.opcode = URMA_OPC_FADD;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.faa.dst = &adst;
  wr.faa.src = &aold;
  wr.faa.operand = 10;
  if (urma_post_jetty_send_wr(a.jetty, &wr, &bad) != URMA_SUCCESS || !reap(a.jfc, false, &cr)) return fail("fetch-add");
  uint64_t now_there = 0, was = 0;
  memcpy(&now_there, b.mem.data() + 4096, 8);
  memcpy(&was, a.mem.data() + 6000, 8);
  if (now_there != 15 || was != 5) return fail("fetch-add values");
  // ---- the wrong token: the import succeeds, the first access is refused
  urma_target_seg_t* forged = urma_import_seg(a.ctx, &b.seg->seg, &wrong, 0, 0);
  if (!forged) return fail("import with another token value");
  urma_sge_t fdst{forged->seg.ubva.va, 8, forged};
  urma_sge_t fsrc{reinterpret_cast<uint64_t>(a.mem.data()), 8, a.seg};
  wr = urma_jfs_wr_t{};
  wr.opcode = URMA_OPC_WRITE;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.rw.src.sge = &fsrc;
  wr.rw.src.num_sge = 1;
  wr.rw.dst.sge = &fdst;
  wr.rw.dst.num_sge = 1;
  if (urma_post_jetty_send_wr(a.jetty, &wr, &bad) != URMA_SUCCESS) return fail("post with the wrong token");
  bool refused = false;
  for (int spins = 0; spins < 200000000 && !refused; ++spins)
    if (urma_poll_jfc(a.jfc, 1, &cr) == 1) refused = cr.status == URMA_CR_REM_ACCESS_ABORT_ERR;
  if (!refused) return fail("a wrong token value must end in URMA_CR_REM_ACCESS_ABORT_ERR");

  // tear-down in reverse order; a context with objects left refuses to go
  if (urma_delete_context(a.ctx) != URMA_EAGAIN) return fail("a context with live objects must not be deleted");
  urma_unimport_seg(forged);
  urma_unimport_seg(rseg);
  urma_unimport_jetty(tj);
  for (Side* s : {&a, &b}) {
    urma_unregister_seg(s->seg);
    urma_delete_jetty(s->jetty);
    urma_delete_jfc(s->jfc);
    if (urma_delete_context(s->ctx) != URMA_SUCCESS) return fail("delete context");
  }
  urma_uninit();
  printf("urma_raw_sample: OK (write, read, send with immediate data, fetch-add, token check on %s)\n", dev_name);
  return 0;
}
