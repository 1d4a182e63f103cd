// Flat convenience layer over the URMA API (see urma_simple.h).
#include "urma_simple.h"

#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "ub_util.h"

struct urma_simple_ep {
  urma_context_t* ctx;
  urma_jfce_t* jfce;
  urma_jfc_t* jfc;
  urma_jetty_t* jetty;
  int interrupt_mode;
};

extern "C" {

urma_context_t* urma_simple_open(const char* dev_name) {
  static std::once_flag once;
  std::call_once(once, [] {
    urma_init_attr_t attr{};
    urma_init(&attr);
  });
  urma_device_t* dev = urma_get_device_by_name(dev_name ? dev_name : "shm0");
  if (!dev) return nullptr;
  return urma_create_context(dev, 0);
}
int urma_simple_close(urma_context_t* ctx) { return urma_delete_context(ctx); }

urma_simple_ep_t* urma_simple_ep_create(urma_context_t* ctx, uint32_t depth, uint32_t recv_token, int interrupt_mode) {
  if (!ctx || depth == 0) return nullptr;
  urma_simple_ep_t* ep = new urma_simple_ep();
  ep->ctx = ctx;
  ep->interrupt_mode = interrupt_mode;
  ep->jfce = urma_create_jfce(ctx);
  urma_jfc_cfg_t cc{};
  cc.depth = depth * 2;
  cc.jfce = ep->jfce;
  ep->jfc = urma_create_jfc(ctx, &cc);
  urma_jetty_cfg_t jc{};
  jc.jfs_cfg.depth = depth;
  jc.jfs_cfg.trans_mode = URMA_TM_RM;
  jc.jfs_cfg.jfc = ep->jfc;
  jc.jfs_cfg.max_sge = 1;
  jc.jfr_cfg.depth = depth;
  jc.jfr_cfg.trans_mode = URMA_TM_RM;
  jc.jfr_cfg.jfc = ep->jfc;
  jc.jfr_cfg.token_value.token = recv_token;
  ep->jetty = ep->jfc ? urma_create_jetty(ctx, &jc) : nullptr;
  if (!ep->jfc || !ep->jetty) {
    urma_simple_ep_destroy(ep);
    return nullptr;
  }
  if (!ep->jfce) ep->interrupt_mode = 0;  // devices without event channels (bond) are polled
  if (ep->interrupt_mode) urma_rearm_jfc(ep->jfc, false);
  return ep;
}
int urma_simple_ep_recover(urma_simple_ep_t* ep) {
  if (!ep || !ep->jetty) return -1;
  urma_cr_t cr[16];
  int flushed = 0, n;
  while ((n = urma_flush_jetty(ep->jetty, 16, cr)) > 0) flushed += n;
  if (urma_modify_jetty(ep->jetty, URMA_JETTY_STATE_READY) != URMA_SUCCESS) return -1;
  return flushed;
}
int urma_simple_ep_destroy(urma_simple_ep_t* ep) {
  if (!ep) return -1;
  if (ep->jetty) urma_delete_jetty(ep->jetty);
  if (ep->jfc) urma_delete_jfc(ep->jfc);
  if (ep->jfce) urma_delete_jfce(ep->jfce);
  delete ep;
  return 0;
}
void urma_simple_ep_blob(urma_simple_ep_t* ep, uint8_t out[URMA_SIMPLE_JETTY_BLOB]) {
  memset(out, 0, URMA_SIMPLE_JETTY_BLOB);
  memcpy(out, &ep->jetty->jetty_id, sizeof(urma_jetty_id_t));
}
urma_target_jetty_t* urma_simple_ep_import(urma_context_t* ctx, const uint8_t blob[URMA_SIMPLE_JETTY_BLOB],
                                           uint32_t token) {
  urma_rjetty_t rj{};
  memcpy(&rj.jetty_id, blob, sizeof(urma_jetty_id_t));
  rj.trans_mode = URMA_TM_RM;
  rj.type = 1;
  urma_token_t t{token};
  return urma_import_jetty(ctx, &rj, &t);
}
urma_jetty_t* urma_simple_ep_jetty(urma_simple_ep_t* ep) { return ep->jetty; }
urma_jfc_t* urma_simple_ep_jfc(urma_simple_ep_t* ep) { return ep->jfc; }

urma_target_seg_t* urma_simple_seg_register(urma_context_t* ctx, void* va, uint64_t len, uint32_t access,
                                            uint32_t token, uint8_t blob_out[URMA_SIMPLE_SEG_BLOB]) {
  urma_seg_cfg_t cfg{};
  cfg.va = reinterpret_cast<uint64_t>(va);
  cfg.len = len;
  cfg.access = access;
  cfg.token_value.token = token;
  urma_target_seg_t* t = urma_register_seg(ctx, &cfg);
  if (t && blob_out) {
    memset(blob_out, 0, URMA_SIMPLE_SEG_BLOB);
    static_assert(sizeof(urma_seg_t) <= URMA_SIMPLE_SEG_BLOB, "segment descriptor blob too small");
    memcpy(blob_out, &t->seg, sizeof(urma_seg_t));
  }
  return t;
}
urma_target_seg_t* urma_simple_seg_import(urma_context_t* ctx, const uint8_t blob[URMA_SIMPLE_SEG_BLOB],
                                          uint32_t token) {
  urma_seg_t seg;
  memcpy(&seg, blob, sizeof(seg));
  urma_token_t t{token};
  return urma_import_seg(ctx, &seg, &t, 0, 0);
}

int urma_simple_post(urma_simple_ep_t* ep, urma_target_jetty_t* peer, int opcode, urma_target_seg_t* rseg,
                     uint64_t raddr, urma_target_seg_t* lseg, uint64_t laddr, uint32_t len, uint64_t imm,
                     uint64_t user_ctx, int signaled) {
  if (!ep || !peer) return URMA_EINVAL;
  urma_sge_t l{laddr, len, lseg}, r{raddr, len, rseg};
  urma_jfs_wr_t wr{};
  wr.opcode = static_cast<urma_opcode_t>(opcode);
  wr.flag = signaled ? URMA_WR_FLAG_COMPLETE_ENABLE : 0;
  wr.tjetty = peer;
  wr.user_ctx = user_ctx;
  switch (opcode) {
    case URMA_OPC_WRITE:
    case URMA_OPC_WRITE_IMM:
    case URMA_OPC_WRITE_NOTIFY:
      wr.rw.src = urma_sg_t{&l, 1};
      wr.rw.dst = urma_sg_t{&r, 1};
      wr.rw.notify_data = imm;
      break;
    case URMA_OPC_READ:
      wr.rw.src = urma_sg_t{&r, 1};
      wr.rw.dst = urma_sg_t{&l, 1};
      break;
    case URMA_OPC_SEND:
    case URMA_OPC_SEND_IMM:
      wr.send.src = urma_sg_t{&l, 1};
      wr.send.imm_data = imm;
      break;
    case URMA_OPC_NOP: break;
    default: return URMA_EINVAL;
  }
  urma_jfs_wr_t* bad = nullptr;
  return urma_post_jetty_send_wr(ep->jetty, &wr, &bad);
}

int urma_simple_atomic(urma_simple_ep_t* ep, urma_target_jetty_t* peer, int opcode, urma_target_seg_t* rseg,
                       uint64_t raddr, uint64_t operand, uint64_t compare, uint64_t* result, uint64_t user_ctx) {
  if (!ep || !peer || !rseg) return URMA_EINVAL;
  urma_sge_t d{raddr, 8, rseg}, s{reinterpret_cast<uint64_t>(result), 8, nullptr};
  urma_jfs_wr_t wr{};
  wr.opcode = static_cast<urma_opcode_t>(opcode);
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = peer;
  wr.user_ctx = user_ctx;
  if (opcode == URMA_OPC_CAS || opcode == URMA_OPC_SWAP) {
    wr.cas.dst = &d;
    wr.cas.src = result ? &s : nullptr;
    wr.cas.cmp_data = compare;
    wr.cas.swap_data = operand;
  } else {
    wr.faa.dst = &d;
    wr.faa.src = result ? &s : nullptr;
    wr.faa.operand = operand;
  }
  urma_jfs_wr_t* bad = nullptr;
  return urma_post_jetty_send_wr(ep->jetty, &wr, &bad);
}

int urma_simple_post_recv(urma_simple_ep_t* ep, void* buf, uint32_t len, uint64_t user_ctx) {
  if (!ep) return URMA_EINVAL;
  urma_sge_t s{reinterpret_cast<uint64_t>(buf), len, nullptr};
  urma_jfr_wr_t wr{};
  wr.src = urma_sg_t{&s, 1};
  wr.user_ctx = user_ctx;
  urma_jfr_wr_t* bad = nullptr;
  return urma_post_jetty_recv_wr(ep->jetty, &wr, &bad);
}

int urma_simple_poll(urma_simple_ep_t* ep, int max, int* status, uint64_t* user_ctx, uint32_t* len, uint64_t* imm,
                     uint32_t* flag) {
  if (!ep || max <= 0) return -1;
  if (max > 64) max = 64;
  urma_cr_t cr[64];
  const int n = urma_poll_jfc(ep->jfc, max, cr);
  for (int i = 0; i < n; ++i) {
    if (status) status[i] = cr[i].status;
    if (user_ctx) user_ctx[i] = cr[i].user_ctx;
    if (len) len[i] = cr[i].completion_len;
    if (imm) imm[i] = cr[i].imm_data;
    if (flag) flag[i] = cr[i].flag;
  }
  return n;
}

int urma_simple_wait(urma_simple_ep_t* ep, int want, int timeout_ms, int max, int* status, uint64_t* user_ctx,
                     uint32_t* len, uint64_t* imm, uint32_t* flag) {
  if (!ep || want <= 0 || max < want) return -1;
  int got = 0;
  const uint64_t deadline = ub::now_ns() + uint64_t(timeout_ms) * 1000000ull;
  while (got < want) {
    const int n = urma_simple_poll(ep, max - got, status ? status + got : nullptr, user_ctx ? user_ctx + got : nullptr,
                                   len ? len + got : nullptr, imm ? imm + got : nullptr, flag ? flag + got : nullptr);
    if (n < 0) return n;
    got += n;
    if (got >= want) break;
    const uint64_t now = ub::now_ns();
    if (now >= deadline) break;
    if (ep->interrupt_mode) {
      urma_jfc_t* fired[1];
      urma_rearm_jfc(ep->jfc, false);
      const int left_ms = static_cast<int>((deadline - now) / 1000000ull) + 1;
      const int r = urma_wait_jfc(ep->jfce, 1, left_ms, fired);
      if (r > 0) {
        uint32_t one = 1;
        urma_ack_jfc(fired, &one, 1);
      }
    } else {
      sched_yield();
    }
  }
  return got;
}

}  // extern "C"
