// urma_ext_selftest: exercises the extended control plane of the URMA API on a loopback device -
// two-phase creation (an allocated jetty refuses work until it is activated), options, batch deletion, asynchronous
// import / bind through a notifier, peer descriptions, transport-path attributes and addressing helpers.
//   urma_ext_selftest [device]      (default shm0)
#include <stdio.h>
#include <string.h>

#include <vector>

#include "urma_api.h"
#include "urma_simple.h"

static int g_line = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) {                                                           \
      fprintf(stderr, "urma_ext_selftest: FAILED at line %d: %s\n", __LINE__, #cond); \
      return 1;                                                              \
    }                                                                        \
    g_line = __LINE__;                                                       \
  } while (0)

static int g_loc_logs = 0;
static void loc_log(int, const char* function, int line, const char* message) {
  if (function && line > 0 && message) ++g_loc_logs;
}
static urma_status_t g_advise_status = URMA_FAIL;
static void advise_cb(urma_status_t s, void* arg) {
  g_advise_status = s;
  *static_cast<int*>(arg) = 1;
}

int main(int argc, char** argv) {
  const char* dev = argc > 1 ? argv[1] : "shm0";
  urma_context_t* ctx = urma_simple_open(dev);
  CHECK(ctx);

  // ---- two-phase creation ----
  urma_jfc_cfg_t cc{};
  cc.depth = 64;
  urma_jfc_t* jfc = nullptr;
  CHECK(urma_alloc_jfc(ctx, &cc, &jfc) == URMA_SUCCESS && jfc);
  uint32_t u32 = 0;
  uint64_t u64 = 0x1234;
  CHECK(urma_get_jfc_opt(jfc, URMA_OPT_DEPTH, &u32, sizeof(u32)) == URMA_SUCCESS && u32 == 64);
  CHECK(urma_get_jfc_opt(jfc, URMA_OPT_STATE, &u32, sizeof(u32)) == URMA_SUCCESS && u32 == 0);
  CHECK(urma_set_jfc_opt(jfc, URMA_OPT_USER_CTX, &u64, sizeof(u64)) == URMA_SUCCESS);
  u32 = 4;
  CHECK(urma_set_jfc_opt(jfc, URMA_OPT_MODERATE_COUNT, &u32, sizeof(u32)) == URMA_SUCCESS);
  CHECK(urma_set_jfc_opt(jfc, URMA_OPT_DEPTH, &u32, sizeof(u32)) == URMA_ENOPERM);      // fixed at allocation
  CHECK(urma_set_jfc_opt(jfc, URMA_OPT_USER_CTX, &u64, 2) == URMA_EINVAL);              // short buffer
  CHECK(urma_active_jfc(jfc) == URMA_SUCCESS);
  CHECK(urma_set_jfc_opt(jfc, URMA_OPT_USER_CTX, &u64, sizeof(u64)) == URMA_ENOPERM);   // too late
  CHECK(urma_get_jfc_opt(jfc, URMA_OPT_USER_CTX, &u64, sizeof(u64)) == URMA_SUCCESS && u64 == 0x1234);
  CHECK(urma_active_jfc(jfc) == URMA_EINVAL);                                            // already active

  urma_jetty_cfg_t jc{};
  jc.jfs_cfg.depth = 32;
  jc.jfs_cfg.trans_mode = URMA_TM_RM;
  jc.jfs_cfg.jfc = jfc;
  jc.jfs_cfg.max_sge = 1;
  jc.jfr_cfg.depth = 32;
  jc.jfr_cfg.trans_mode = URMA_TM_RM;
  jc.jfr_cfg.jfc = jfc;
  urma_jetty_t* jetty = nullptr;
  CHECK(urma_alloc_jetty(ctx, &jc, &jetty) == URMA_SUCCESS && jetty);
  CHECK(urma_get_jetty_opt(jetty, URMA_OPT_STATE, &u32, sizeof(u32)) == URMA_SUCCESS && u32 == URMA_JETTY_STATE_RESET);
  uint8_t prio = 3;
  CHECK(urma_set_jetty_opt(jetty, URMA_OPT_PRIORITY, &prio, sizeof(prio)) == URMA_SUCCESS);
  prio = 0;
  CHECK(urma_get_jetty_opt(jetty, URMA_OPT_PRIORITY, &prio, sizeof(prio)) == URMA_SUCCESS && prio == 3);

  // a peer description of the jetty, imported back on the same context
  urma_rjetty_t* rj = nullptr;
  uint32_t rlen = 0;
  CHECK(urma_get_rjetty(jetty, &rj, &rlen) == URMA_SUCCESS && rj && rlen == sizeof(urma_rjetty_t));
  CHECK(rj->jetty_id.id == jetty->jetty_id.id);
  urma_token_t tok{};
  urma_notifier_t* nf = urma_create_notifier(ctx);
  CHECK(nf && nf->fd >= 0);
  urma_notify_t ev[4];
  CHECK(urma_wait_notify(nf, 4, ev, 10) == 0);                                           // nothing yet
  urma_target_jetty_t* tj = urma_import_jetty_async(nf, rj, &tok, 77, 1000);
  CHECK(tj);
  CHECK(urma_wait_notify(nf, 4, ev, 1000) == 1);
  CHECK(ev[0].type == URMA_IMPORT_JETTY_NOTIFY && ev[0].status == URMA_SUCCESS && ev[0].user_ctx == 77 &&
        ev[0].tjetty == tj);
  CHECK(urma_ack_notify(ctx, 1, ev) == URMA_SUCCESS);
  urma_put_rjetty(rj);

  // while only allocated, the jetty refuses work requests; after activation the same request goes through
  std::vector<uint8_t> mem(8192, 7);
  urma_seg_cfg_t sc{};
  sc.va = reinterpret_cast<uint64_t>(mem.data());
  sc.len = mem.size();
  sc.access = 14;
  urma_target_seg_t* seg = urma_register_seg(ctx, &sc);
  CHECK(seg);
  urma_seg_t* seg_desc = nullptr;
  uint32_t seg_size = 0;
  CHECK(urma_get_seg_ctx(seg, &seg_desc, &seg_size) == URMA_SUCCESS && seg_size == sizeof(urma_seg_t));
  urma_target_seg_t* rseg = urma_import_seg(ctx, seg_desc, &tok, 0, 0);
  CHECK(rseg);
  urma_put_seg_ctx(seg_desc);
  urma_jfs_wr_t wr{};
  wr.opcode = URMA_OPC_WRITE;
  wr.flag = URMA_WR_FLAG_COMPLETE_ENABLE;
  wr.tjetty = tj;
  wr.user_ctx = 5;
  urma_sge_t src{reinterpret_cast<uint64_t>(mem.data()), 64, seg};
  urma_sge_t dst{reinterpret_cast<uint64_t>(mem.data()) + 4096, 64, rseg};
  wr.rw.src.sge = &src;
  wr.rw.src.num_sge = 1;
  wr.rw.dst.sge = &dst;
  wr.rw.dst.num_sge = 1;
  urma_jfs_wr_t* bad = nullptr;
  CHECK(urma_post_jetty_send_wr(jetty, &wr, &bad) != URMA_SUCCESS);                     // still in RESET
  CHECK(urma_active_jetty(jetty) == URMA_SUCCESS);
  CHECK(urma_get_jetty_opt(jetty, URMA_OPT_STATE, &u32, sizeof(u32)) == URMA_SUCCESS && u32 == URMA_JETTY_STATE_READY);
  mem[4096] = 0;
  CHECK(urma_post_jetty_send_wr(jetty, &wr, &bad) == URMA_SUCCESS);
  urma_cr_t cr;
  int polled = 0;
  for (int spin = 0; spin < 2000000 && polled == 0; ++spin) polled = urma_poll_jfc(jfc, 1, &cr);
  CHECK(polled == 1 && cr.status == URMA_CR_SUCCESS && cr.user_ctx == 5 && mem[4096] == 7);
  CHECK(urma_get_tpn(jetty) == 0);                                                       // not bound: shared path

  // ---- transport paths and addressing ----
  urma_get_tp_cfg_t tc{};
  tc.trans_mode = URMA_TM_RM;
  tc.local_eid = ctx->eid;
  tc.peer_eid = ctx->eid;
  urma_tp_info_t tp[2];
  uint32_t ntp = 2;
  CHECK(urma_get_tp_list(ctx, &tc, &ntp, tp) == URMA_SUCCESS && ntp == 1 && tp[0].tp_handle != 0);
  urma_tp_info_t tp2[1];
  uint32_t ntp2 = 1;
  CHECK(urma_get_tp_list(ctx, &tc, &ntp2, tp2) == URMA_SUCCESS && tp2[0].tp_handle == tp[0].tp_handle);   // stable
  urma_tp_attr_value_t av{};
  av.ttl = 9;
  av.sl = 2;
  CHECK(urma_set_tp_attr(ctx, tp[0].tp_handle, 2, URMA_TP_ATTR_TTL | URMA_TP_ATTR_SL, &av) == URMA_SUCCESS);
  CHECK(urma_set_tp_attr(ctx, tp[0].tp_handle, 1, URMA_TP_ATTR_TTL | URMA_TP_ATTR_SL, &av) == URMA_EINVAL);  // count
  CHECK(urma_set_tp_attr(ctx, 0xdead, 1, URMA_TP_ATTR_TTL, &av) == URMA_EINVAL);
  uint8_t acnt = 0;
  uint32_t abits = 0;
  urma_tp_attr_value_t got{};
  CHECK(urma_get_tp_attr(ctx, tp[0].tp_handle, &acnt, &abits, &got) == URMA_SUCCESS);
  CHECK(got.ttl == 9 && got.sl == 2 && (abits & URMA_TP_ATTR_SL) && acnt == __builtin_popcount(abits));
  urma_tp_cfg_t mcfg{URMA_TM_RM, ctx->eid, ctx->eid};
  urma_tp_attr_t mattr{};
  mattr.mtu = 1024;
  CHECK(urma_modify_tp(ctx, 0, &mcfg, &mattr, 16u) == 0 && mattr.mtu == 1024 && mattr.state == 1);
  urma_import_jetty_ex_cfg_t ex{tp[0].tp_handle, 0, 0};
  urma_rjetty_t rj2{jetty->jetty_id, URMA_TM_RM, 1};
  urma_target_jetty_t* tj2 = urma_import_jetty_ex(ctx, &rj2, &tok, &ex);
  CHECK(tj2);
  ex.tp_handle = 0xbad;
  CHECK(urma_import_jetty_ex(ctx, &rj2, &tok, &ex) == nullptr);                         // unknown path
  CHECK(urma_unimport_jetty_async(tj2) == URMA_SUCCESS);

  uint32_t naddr = 0;
  urma_net_addr_info_t* addrs = urma_get_net_addr_list(ctx, &naddr);
  CHECK(addrs && naddr == 1);
  urma_eid_t back;
  CHECK(urma_get_eid_by_ip(ctx, &addrs[0].netaddr, &back) == URMA_SUCCESS && memcmp(&back, &ctx->eid, sizeof(back)) == 0);
  urma_net_addr_t ip;
  CHECK(urma_get_ip_by_eid(ctx, &ctx->eid, &ip) == URMA_SUCCESS && memcmp(&ip, &addrs[0].netaddr, sizeof(ip)) == 0);
  uint8_t smac[6], dmac[6];
  CHECK(urma_get_smac(ctx, smac) == URMA_SUCCESS && urma_get_dmac(ctx, &ip, dmac) == URMA_SUCCESS);
  CHECK(memcmp(smac, dmac, 6) == 0 && (smac[0] & 3) == 2);
  urma_free_net_addr_list(addrs);

  // ---- context option, logging with source location, advise callback ----
  CHECK(urma_set_context_opt(ctx, URMA_OPT_CTX_LOG_TAG, "selftest", 9) == URMA_SUCCESS);
  CHECK(strcmp(urma_log_get_thread_tag(), "selftest") == 0);
  CHECK(urma_register_loc_log_func(loc_log) == URMA_SUCCESS);
  urma_log(URMA_VLOG_LEVEL_ERR, __func__, __LINE__, "a message for the location callback");
  CHECK(g_loc_logs == 1);
  CHECK(urma_register_loc_log_func(nullptr) == URMA_SUCCESS);
  urma_token_id_flag_t tf{};
  tf.bs.multi_seg = 1;
  urma_token_id_t* tid = urma_alloc_token_id_ex(ctx, tf);
  CHECK(tid && urma_free_token_id(tid) == URMA_SUCCESS);

  // ---- standalone JFS / JFR in two phases, advise, batch deletion ----
  // (multipath devices expose jetties only, no standalone send / receive queues)
  if (strncmp(dev, "bond", 4) != 0) {
    urma_jfs_cfg_t sc2 = jc.jfs_cfg;
    urma_jfr_cfg_t rc2 = jc.jfr_cfg;
    urma_jfs_t* jfs = nullptr;
    urma_jfr_t* jfr = nullptr;
    CHECK(urma_alloc_jfs(ctx, &sc2, &jfs) == URMA_SUCCESS && urma_alloc_jfr(ctx, &rc2, &jfr) == URMA_SUCCESS);
    u32 = 8;
    CHECK(urma_set_jfr_opt(jfr, URMA_OPT_RX_THRESHOLD, &u32, sizeof(u32)) == URMA_SUCCESS);
    CHECK(urma_active_jfs(jfs) == URMA_SUCCESS && urma_active_jfr(jfr) == URMA_SUCCESS);
    CHECK(urma_get_jfr_opt(jfr, URMA_OPT_STATE, &u32, sizeof(u32)) == URMA_SUCCESS && u32 == URMA_JETTY_STATE_READY);
    urma_rjfr_t rjfr{jfr->jfr_id, URMA_TM_RM, 0};
    urma_target_jetty_t* tjfr = urma_import_jfr_ex(ctx, &rjfr, &tok, nullptr);
    CHECK(tjfr);
    int called = 0;
    CHECK(urma_advise_jfr_async(jfs, tjfr, advise_cb, &called) == URMA_SUCCESS && called == 1);
    CHECK(urma_unimport_jfr(tjfr) == URMA_SUCCESS);
    CHECK(urma_deactive_jfs(jfs) == URMA_SUCCESS && urma_deactive_jfs(jfs) == URMA_EINVAL);
    CHECK(urma_free_jfs(jfs) == URMA_SUCCESS && urma_free_jfr(jfr) == URMA_SUCCESS);
  }

  urma_jfc_cfg_t bc{};
  bc.depth = 8;
  urma_jfc_t* batch[3] = {urma_create_jfc(ctx, &bc), urma_create_jfc(ctx, &bc), nullptr};
  urma_jfc_t* bad_jfc = reinterpret_cast<urma_jfc_t*>(1);
  CHECK(batch[0] && batch[1]);
  CHECK(urma_delete_jfc_batch(batch, 3, &bad_jfc) == URMA_EINVAL && bad_jfc == nullptr);   // stops at the null entry
  // the first two are gone; a completion queue still in use is reported as the bad one
  urma_jfc_t* busy[1] = {jfc};
  CHECK(urma_delete_jfc_batch(busy, 1, &bad_jfc) != URMA_SUCCESS && bad_jfc == jfc);

  // ---- tear-down in reference order ----
  CHECK(urma_unimport_seg(rseg) == URMA_SUCCESS && urma_unregister_seg(seg) == URMA_SUCCESS);
  CHECK(urma_unimport_jetty(tj) == URMA_SUCCESS);
  CHECK(urma_delete_notifier(nf) == URMA_SUCCESS);
  urma_jetty_t* jb[1] = {jetty};
  urma_jetty_t* bad_jetty = nullptr;
  CHECK(urma_delete_jetty_batch(jb, 1, &bad_jetty) == URMA_SUCCESS && bad_jetty == nullptr);
  CHECK(urma_deactive_jfc(jfc) == URMA_SUCCESS);
  CHECK(urma_free_jfc(jfc) == URMA_SUCCESS);
  urma_simple_close(ctx);
  printf("urma_ext_selftest: OK (%s)\n", dev);
  return 0;
}
