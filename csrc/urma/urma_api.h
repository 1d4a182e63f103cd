/* URMA northbound API. Function names and argument order follow the reference's
 * src/urma/lib/urma/core/include/urma_api.h (init :27-33, devices :42-89, context :97-112, JFC :120-198,
 * JFS :206-304, JFR :312-460, Jetty :472-735, jetty group :747-754, JFCE :761-768, async events :776-783,
 * token id :790-807, segments :816-857, post WR :866-893, write/read/send/recv :908-952,
 * poll/rearm/wait/ack :962-994, user_ctl :1001-1011, logging :1018-1057) and urma_perf.h:60-74. */
#ifndef UMDK_URMA_API_H
#define UMDK_URMA_API_H

#include "urma_types.h"

#ifdef __cplusplus
extern "C" {
#endif
#define URMA_EXPORT __attribute__((visibility("default")))

/* lifecycle */
URMA_EXPORT urma_status_t urma_init(const urma_init_attr_t* attr);
URMA_EXPORT urma_status_t urma_uninit(void);
/* devices */
URMA_EXPORT urma_device_t** urma_get_device_list(int* num_devices);
URMA_EXPORT void urma_free_device_list(urma_device_t** list);
URMA_EXPORT urma_device_t* urma_get_device_by_name(const char* name);
URMA_EXPORT urma_device_t* urma_get_device_by_eid(urma_eid_t eid);
URMA_EXPORT urma_status_t urma_query_device(urma_device_t* dev, urma_device_attr_t* attr);
URMA_EXPORT urma_eid_info_t* urma_get_eid_list(urma_device_t* dev, uint32_t* cnt);
URMA_EXPORT void urma_free_eid_list(urma_eid_info_t* list);
URMA_EXPORT int urma_str_to_eid(const char* s, urma_eid_t* eid);
URMA_EXPORT void urma_eid_to_str(const urma_eid_t* eid, char* buf, size_t len);
/* context */
URMA_EXPORT urma_context_t* urma_create_context(urma_device_t* dev, uint32_t eid_index);
URMA_EXPORT urma_status_t urma_delete_context(urma_context_t* ctx);
URMA_EXPORT uint32_t urma_get_uasid(urma_context_t* ctx);
/* JFC / JFCE */
URMA_EXPORT urma_jfc_t* urma_create_jfc(urma_context_t* ctx, const urma_jfc_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_modify_jfc(urma_jfc_t* jfc, uint32_t moderate_count, uint32_t moderate_period);
URMA_EXPORT urma_status_t urma_delete_jfc(urma_jfc_t* jfc);
URMA_EXPORT urma_jfce_t* urma_create_jfce(urma_context_t* ctx);
URMA_EXPORT urma_status_t urma_delete_jfce(urma_jfce_t* jfce);
/* JFS */
URMA_EXPORT urma_jfs_t* urma_create_jfs(urma_context_t* ctx, const urma_jfs_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_modify_jfs(urma_jfs_t* jfs, urma_jetty_state_t state);
URMA_EXPORT urma_status_t urma_query_jfs(urma_jfs_t* jfs, urma_jfs_cfg_t* cfg, urma_jetty_state_t* state);
URMA_EXPORT int urma_flush_jfs(urma_jfs_t* jfs, int cr_cnt, urma_cr_t* cr);
URMA_EXPORT urma_status_t urma_delete_jfs(urma_jfs_t* jfs);
/* JFR */
URMA_EXPORT urma_jfr_t* urma_create_jfr(urma_context_t* ctx, const urma_jfr_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_modify_jfr(urma_jfr_t* jfr, urma_jetty_state_t state, uint32_t rx_threshold);
URMA_EXPORT urma_status_t urma_query_jfr(urma_jfr_t* jfr, urma_jfr_cfg_t* cfg, urma_jetty_state_t* state);
URMA_EXPORT urma_status_t urma_delete_jfr(urma_jfr_t* jfr);
URMA_EXPORT urma_target_jetty_t* urma_import_jfr(urma_context_t* ctx, const urma_rjfr_t* rjfr,
                                                 const urma_token_t* token);
URMA_EXPORT urma_status_t urma_unimport_jfr(urma_target_jetty_t* tjfr);
URMA_EXPORT urma_status_t urma_advise_jfr(urma_jfs_t* jfs, urma_target_jetty_t* tjfr);
URMA_EXPORT urma_status_t urma_unadvise_jfr(urma_jfs_t* jfs, urma_target_jetty_t* tjfr);
/* Jetty */
URMA_EXPORT urma_jetty_t* urma_create_jetty(urma_context_t* ctx, const urma_jetty_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_modify_jetty(urma_jetty_t* jetty, urma_jetty_state_t state);
URMA_EXPORT urma_status_t urma_query_jetty(urma_jetty_t* jetty, urma_jetty_cfg_t* cfg, urma_jetty_state_t* state);
URMA_EXPORT int urma_flush_jetty(urma_jetty_t* jetty, int cr_cnt, urma_cr_t* cr);
URMA_EXPORT urma_status_t urma_delete_jetty(urma_jetty_t* jetty);
URMA_EXPORT urma_target_jetty_t* urma_import_jetty(urma_context_t* ctx, const urma_rjetty_t* rjetty,
                                                   const urma_token_t* token);
URMA_EXPORT urma_status_t urma_unimport_jetty(urma_target_jetty_t* tjetty);
URMA_EXPORT urma_status_t urma_bind_jetty(urma_jetty_t* jetty, urma_target_jetty_t* tjetty);
URMA_EXPORT urma_status_t urma_unbind_jetty(urma_jetty_t* jetty);
URMA_EXPORT urma_status_t urma_advise_jetty(urma_jetty_t* jetty, urma_target_jetty_t* tjetty);
URMA_EXPORT urma_status_t urma_unadvise_jetty(urma_jetty_t* jetty, urma_target_jetty_t* tjetty);
URMA_EXPORT urma_jetty_grp_t* urma_create_jetty_grp(urma_context_t* ctx, const char* name, uint32_t policy);
URMA_EXPORT urma_status_t urma_delete_jetty_grp(urma_jetty_grp_t* grp);
/* token ids and segments */
URMA_EXPORT urma_token_id_t* urma_alloc_token_id(urma_context_t* ctx);
URMA_EXPORT urma_status_t urma_free_token_id(urma_token_id_t* token_id);
URMA_EXPORT urma_target_seg_t* urma_register_seg(urma_context_t* ctx, const urma_seg_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_unregister_seg(urma_target_seg_t* tseg);
URMA_EXPORT urma_target_seg_t* urma_import_seg(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token,
                                               uint64_t addr, uint32_t flag);
URMA_EXPORT urma_status_t urma_unimport_seg(urma_target_seg_t* tseg);
/* data plane */
URMA_EXPORT urma_status_t urma_post_jfs_wr(urma_jfs_t* jfs, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad_wr);
URMA_EXPORT urma_status_t urma_post_jfr_wr(urma_jfr_t* jfr, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad_wr);
URMA_EXPORT urma_status_t urma_post_jetty_send_wr(urma_jetty_t* jetty, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad_wr);
URMA_EXPORT urma_status_t urma_post_jetty_recv_wr(urma_jetty_t* jetty, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad_wr);
URMA_EXPORT urma_status_t urma_write(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* dst_tseg,
                                     urma_target_seg_t* src_tseg, uint64_t dst, uint64_t src, uint32_t len,
                                     uint32_t flag, uint64_t user_ctx);
URMA_EXPORT urma_status_t urma_read(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* dst_tseg,
                                    urma_target_seg_t* src_tseg, uint64_t dst, uint64_t src, uint32_t len,
                                    uint32_t flag, uint64_t user_ctx);
URMA_EXPORT urma_status_t urma_send(urma_jfs_t* jfs, urma_target_jetty_t* tjfr, urma_target_seg_t* src_tseg,
                                    uint64_t src, uint32_t len, uint32_t flag, uint64_t user_ctx);
URMA_EXPORT urma_status_t urma_recv(urma_jfr_t* jfr, urma_target_seg_t* recv_tseg, uint64_t buf, uint32_t len,
                                    uint64_t user_ctx);
URMA_EXPORT int urma_poll_jfc(urma_jfc_t* jfc, int cr_cnt, urma_cr_t* cr);
URMA_EXPORT urma_status_t urma_rearm_jfc(urma_jfc_t* jfc, bool solicited_only);
URMA_EXPORT int urma_wait_jfc(urma_jfce_t* jfce, uint32_t jfc_cnt, int time_out, urma_jfc_t* jfc[]);
URMA_EXPORT void urma_ack_jfc(urma_jfc_t* jfc[], uint32_t nevents[], uint32_t jfc_cnt);
/* async events, user control */
URMA_EXPORT urma_status_t urma_get_async_event(urma_context_t* ctx, urma_async_event_t* event);
URMA_EXPORT void urma_ack_async_event(urma_async_event_t* event);
URMA_EXPORT int urma_user_ctl(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out);
/* logging */
URMA_EXPORT urma_status_t urma_register_log_func(urma_log_cb_t func);
URMA_EXPORT urma_status_t urma_unregister_log_func(void);
URMA_EXPORT urma_vlog_level_t urma_log_get_level(void);
URMA_EXPORT void urma_log_set_level(urma_vlog_level_t level);
URMA_EXPORT void urma_log_set_thread_tag(const char* tag);
URMA_EXPORT void urma_log(int level, const char* func, int line, const char* fmt, ...)
    __attribute__((format(printf, 4, 5)));
URMA_EXPORT urma_status_t urma_register_loc_log_func(urma_loc_log_cb func);
URMA_EXPORT const char* urma_log_get_thread_tag(void);

/* ---- extended control plane (urma_ext.cpp; same names as the reference's urma_api.h) ---- */
/* Two-phase creation: urma_alloc_* creates the object in the RESET state (it refuses work requests), options may be
 * read and, where marked rw in urma_opt_name_t, changed; urma_active_* makes it READY; urma_deactive_* takes it back
 * to RESET; urma_free_* deletes it. */
URMA_EXPORT urma_status_t urma_alloc_jfc(urma_context_t* ctx, urma_jfc_cfg_t* cfg, urma_jfc_t** jfc);
URMA_EXPORT urma_status_t urma_set_jfc_opt(urma_jfc_t* jfc, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_get_jfc_opt(urma_jfc_t* jfc, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_active_jfc(urma_jfc_t* jfc);
URMA_EXPORT urma_status_t urma_deactive_jfc(urma_jfc_t* jfc);
URMA_EXPORT urma_status_t urma_free_jfc(urma_jfc_t* jfc);
URMA_EXPORT urma_status_t urma_alloc_jfs(urma_context_t* ctx, urma_jfs_cfg_t* cfg, urma_jfs_t** jfs);
URMA_EXPORT urma_status_t urma_set_jfs_opt(urma_jfs_t* jfs, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_get_jfs_opt(urma_jfs_t* jfs, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_active_jfs(urma_jfs_t* jfs);
URMA_EXPORT urma_status_t urma_deactive_jfs(urma_jfs_t* jfs);
URMA_EXPORT urma_status_t urma_free_jfs(urma_jfs_t* jfs);
URMA_EXPORT urma_status_t urma_alloc_jfr(urma_context_t* ctx, urma_jfr_cfg_t* cfg, urma_jfr_t** jfr);
URMA_EXPORT urma_status_t urma_set_jfr_opt(urma_jfr_t* jfr, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_get_jfr_opt(urma_jfr_t* jfr, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_active_jfr(urma_jfr_t* jfr);
URMA_EXPORT urma_status_t urma_deactive_jfr(urma_jfr_t* jfr);
URMA_EXPORT urma_status_t urma_free_jfr(urma_jfr_t* jfr);
URMA_EXPORT urma_status_t urma_alloc_jetty(urma_context_t* ctx, urma_jetty_cfg_t* cfg, urma_jetty_t** jetty);
URMA_EXPORT urma_status_t urma_set_jetty_opt(urma_jetty_t* jetty, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_get_jetty_opt(urma_jetty_t* jetty, uint64_t opt, void* buf, uint32_t len);
URMA_EXPORT urma_status_t urma_active_jetty(urma_jetty_t* jetty);
URMA_EXPORT urma_status_t urma_deactive_jetty(urma_jetty_t* jetty);
URMA_EXPORT urma_status_t urma_free_jetty(urma_jetty_t* jetty);
/* Batch deletion: stops at the first failure and reports it in *bad (NULL when all were deleted). */
URMA_EXPORT urma_status_t urma_delete_jfc_batch(urma_jfc_t** arr, int num, urma_jfc_t** bad);
URMA_EXPORT urma_status_t urma_delete_jfs_batch(urma_jfs_t** arr, int num, urma_jfs_t** bad);
URMA_EXPORT urma_status_t urma_delete_jfr_batch(urma_jfr_t** arr, int num, urma_jfr_t** bad);
URMA_EXPORT urma_status_t urma_delete_jetty_batch(urma_jetty_t** arr, int num, urma_jetty_t** bad);
/* Import / bind with an explicit transport path, and their asynchronous forms: the call returns at once and the
 * outcome arrives as a urma_notify_t on the notifier (on one box the work itself completes immediately). */
URMA_EXPORT urma_target_jetty_t* urma_import_jetty_ex(urma_context_t* ctx, urma_rjetty_t* rjetty,
                                                      urma_token_t* token_value, urma_import_jetty_ex_cfg_t* cfg);
URMA_EXPORT urma_target_jetty_t* urma_import_jfr_ex(urma_context_t* ctx, urma_rjfr_t* rjfr, urma_token_t* token_value,
                                                    urma_import_jfr_ex_cfg_t* cfg);
URMA_EXPORT urma_status_t urma_bind_jetty_ex(urma_jetty_t* jetty, urma_target_jetty_t* tjetty,
                                             urma_bind_jetty_ex_cfg_t* cfg);
URMA_EXPORT urma_notifier_t* urma_create_notifier(urma_context_t* ctx);
URMA_EXPORT urma_status_t urma_delete_notifier(urma_notifier_t* notifier);
URMA_EXPORT urma_target_jetty_t* urma_import_jetty_async(urma_notifier_t* notifier, const urma_rjetty_t* rjetty,
                                                         const urma_token_t* token_value, uint64_t user_ctx,
                                                         int timeout);
URMA_EXPORT urma_status_t urma_unimport_jetty_async(urma_target_jetty_t* tjetty);
URMA_EXPORT urma_status_t urma_bind_jetty_async(urma_notifier_t* notifier, urma_jetty_t* jetty,
                                                urma_target_jetty_t* tjetty, uint64_t user_ctx, int timeout);
URMA_EXPORT urma_status_t urma_unbind_jetty_async(urma_jetty_t* jetty);
URMA_EXPORT urma_status_t urma_advise_jfr_async(urma_jfs_t* jfs, urma_target_jetty_t* tjfr,
                                                urma_advise_async_cb_func cb_fun, void* cb_arg);
URMA_EXPORT int urma_wait_notify(urma_notifier_t* notifier, uint32_t cnt, urma_notify_t* notify, int timeout);
URMA_EXPORT urma_status_t urma_ack_notify(urma_context_t* ctx, uint32_t cnt, urma_notify_t* notify);
/* Descriptions that can be sent to a peer: heap copies, released with the matching put call. */
URMA_EXPORT urma_status_t urma_get_rjetty(urma_jetty_t* jetty, urma_rjetty_t** rjetty, uint32_t* length);
URMA_EXPORT void urma_put_rjetty(urma_rjetty_t* rjetty);
URMA_EXPORT urma_status_t urma_get_seg_ctx(urma_target_seg_t* tseg, urma_seg_t** seg, uint32_t* size);
URMA_EXPORT void urma_put_seg_ctx(urma_seg_t* seg);
URMA_EXPORT urma_token_id_t* urma_alloc_token_id_ex(urma_context_t* ctx, urma_token_id_flag_t flag);
URMA_EXPORT urma_status_t urma_set_context_opt(urma_context_t* ctx, urma_opt_name_t opt_name, const void* opt_value,
                                               size_t opt_len);
/* Transport paths: one per (local EID, peer EID, transport mode); attributes are kept per path. */
URMA_EXPORT int urma_get_tpn(urma_jetty_t* jetty);
URMA_EXPORT urma_status_t urma_get_tp_list(urma_context_t* ctx, urma_get_tp_cfg_t* cfg, uint32_t* tp_cnt,
                                           urma_tp_info_t* tp_list);
URMA_EXPORT urma_status_t urma_set_tp_attr(const urma_context_t* ctx, const uint64_t tp_handle,
                                           const uint8_t tp_attr_cnt, const uint32_t tp_attr_bitmap,
                                           const urma_tp_attr_value_t* tp_attr);
URMA_EXPORT urma_status_t urma_get_tp_attr(const urma_context_t* ctx, const uint64_t tp_handle, uint8_t* tp_attr_cnt,
                                           uint32_t* tp_attr_bitmap, urma_tp_attr_value_t* tp_attr);
URMA_EXPORT int urma_modify_tp(urma_context_t* ctx, uint32_t tpn, urma_tp_cfg_t* cfg, urma_tp_attr_t* attr,
                               urma_tp_attr_mask_t mask);
/* Addressing: every EID of this box has a synthetic IPv6 address (the EID itself) and MAC (its last 6 bytes). */
URMA_EXPORT urma_net_addr_info_t* urma_get_net_addr_list(urma_context_t* ctx, uint32_t* cnt);
URMA_EXPORT void urma_free_net_addr_list(urma_net_addr_info_t* net_addr_list);
URMA_EXPORT urma_status_t urma_get_eid_by_ip(const urma_context_t* ctx, const urma_net_addr_t* net_addr,
                                             urma_eid_t* eid);
URMA_EXPORT urma_status_t urma_get_ip_by_eid(const urma_context_t* ctx, const urma_eid_t* eid,
                                             urma_net_addr_t* net_addr);
URMA_EXPORT urma_status_t urma_get_smac(const urma_context_t* ctx, uint8_t* mac);
URMA_EXPORT urma_status_t urma_get_dmac(const urma_context_t* ctx, const urma_net_addr_t* net_addr, uint8_t* mac);

/* perf sampling of the data-plane calls */
typedef enum urma_perf_op {
  URMA_PERF_WRITE = 0, URMA_PERF_READ, URMA_PERF_SEND, URMA_PERF_RECV, URMA_PERF_POST_JFS, URMA_PERF_POST_JFR,
  URMA_PERF_POST_JETTY_SEND, URMA_PERF_POST_JETTY_RECV, URMA_PERF_POLL_JFC, URMA_PERF_OP_MAX
} urma_perf_op_t;
typedef struct urma_perf_entry {
  uint64_t count, min_ns, max_ns, avg_ns, p90_ns, p99_ns, p9999_ns;
} urma_perf_entry_t;
URMA_EXPORT urma_status_t urma_start_perf(void);
URMA_EXPORT urma_status_t urma_stop_perf(void);
URMA_EXPORT urma_status_t urma_get_perf_info(urma_perf_entry_t* entries /* [URMA_PERF_OP_MAX] */, char* text,
                                             uint32_t* text_len);

#ifdef __cplusplus
}
#endif
#endif
