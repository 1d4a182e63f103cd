/* Southbound (provider) interface of URMA: a device driver fills one `urma_ops_t` per context and registers a
 * `urma_provider_ops_t` from a library constructor. The core dispatches every northbound call through these tables
 * after validating arguments and handling reference counts. Same role as the reference's
 * src/urma/lib/urma/core/include/urma_provider.h (urma_ops_t / urma_provider_ops_t / urma_register_provider_ops);
 * the set of entries is the subset this project's providers implement. An entry may be NULL: the core then returns
 * URMA_FAIL / NULL for that call. */
#ifndef UMDK_URMA_PROVIDER_H
#define UMDK_URMA_PROVIDER_H

#include "urma_types.h"

#ifndef URMA_EXPORT
#define URMA_EXPORT __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct urma_ops {
  const char* name;
  /* completion queues / event channels */
  urma_jfc_t* (*create_jfc)(urma_context_t* ctx, const urma_jfc_cfg_t* cfg);
  urma_status_t (*modify_jfc)(urma_jfc_t* jfc, uint32_t moderate_count, uint32_t moderate_period);
  urma_status_t (*delete_jfc)(urma_jfc_t* jfc);
  urma_jfce_t* (*create_jfce)(urma_context_t* ctx);
  urma_status_t (*delete_jfce)(urma_jfce_t* jfce);
  /* send / receive queues */
  urma_jfs_t* (*create_jfs)(urma_context_t* ctx, const urma_jfs_cfg_t* cfg);
  urma_status_t (*modify_jfs)(urma_jfs_t* jfs, urma_jetty_state_t state);
  urma_status_t (*query_jfs)(urma_jfs_t* jfs, urma_jfs_cfg_t* cfg, urma_jetty_state_t* state);
  int (*flush_jfs)(urma_jfs_t* jfs, int cr_cnt, urma_cr_t* cr);
  urma_status_t (*delete_jfs)(urma_jfs_t* jfs);
  urma_jfr_t* (*create_jfr)(urma_context_t* ctx, const urma_jfr_cfg_t* cfg);
  urma_status_t (*modify_jfr)(urma_jfr_t* jfr, urma_jetty_state_t state, uint32_t rx_threshold);
  urma_status_t (*query_jfr)(urma_jfr_t* jfr, urma_jfr_cfg_t* cfg, urma_jetty_state_t* state);
  urma_status_t (*delete_jfr)(urma_jfr_t* jfr);
  urma_target_jetty_t* (*import_jfr)(urma_context_t* ctx, const urma_rjfr_t* rjfr, const urma_token_t* token);
  urma_status_t (*unimport_jfr)(urma_target_jetty_t* tjfr);
  urma_jetty_t* (*create_jetty)(urma_context_t* ctx, const urma_jetty_cfg_t* cfg);
  urma_status_t (*modify_jetty)(urma_jetty_t* jetty, urma_jetty_state_t state);
  urma_status_t (*query_jetty)(urma_jetty_t* jetty, urma_jetty_cfg_t* cfg, urma_jetty_state_t* state);
  int (*flush_jetty)(urma_jetty_t* jetty, int cr_cnt, urma_cr_t* cr);
  urma_status_t (*delete_jetty)(urma_jetty_t* jetty);
  urma_target_jetty_t* (*import_jetty)(urma_context_t* ctx, const urma_rjetty_t* rjetty, const urma_token_t* token);
  urma_status_t (*unimport_jetty)(urma_target_jetty_t* tjetty);
  urma_status_t (*bind_jetty)(urma_jetty_t* jetty, urma_target_jetty_t* tjetty);
  urma_status_t (*unbind_jetty)(urma_jetty_t* jetty);
  urma_jetty_grp_t* (*create_jetty_grp)(urma_context_t* ctx, const char* name, uint32_t policy);
  urma_status_t (*delete_jetty_grp)(urma_jetty_grp_t* grp);
  /* memory */
  urma_token_id_t* (*alloc_token_id)(urma_context_t* ctx);
  urma_status_t (*free_token_id)(urma_token_id_t* token_id);
  urma_target_seg_t* (*register_seg)(urma_context_t* ctx, const urma_seg_cfg_t* cfg);
  urma_status_t (*unregister_seg)(urma_target_seg_t* tseg);
  urma_target_seg_t* (*import_seg)(urma_context_t* ctx, const urma_seg_t* seg, const urma_token_t* token,
                                   uint64_t addr, uint32_t flag);
  urma_status_t (*unimport_seg)(urma_target_seg_t* tseg);
  /* data plane */
  urma_status_t (*post_jfs_wr)(urma_jfs_t* jfs, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad_wr);
  urma_status_t (*post_jfr_wr)(urma_jfr_t* jfr, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad_wr);
  urma_status_t (*post_jetty_send_wr)(urma_jetty_t* jetty, urma_jfs_wr_t* wr, urma_jfs_wr_t** bad_wr);
  urma_status_t (*post_jetty_recv_wr)(urma_jetty_t* jetty, urma_jfr_wr_t* wr, urma_jfr_wr_t** bad_wr);
  int (*poll_jfc)(urma_jfc_t* jfc, int cr_cnt, urma_cr_t* cr);
  urma_status_t (*rearm_jfc)(urma_jfc_t* jfc, bool solicited_only);
  int (*wait_jfc)(urma_jfce_t* jfce, uint32_t jfc_cnt, int time_out_ms, urma_jfc_t* jfc[]);
  void (*ack_jfc)(urma_jfc_t* jfc[], uint32_t nevents[], uint32_t jfc_cnt);
  /* events / misc */
  urma_status_t (*get_async_event)(urma_context_t* ctx, urma_async_event_t* event);
  void (*ack_async_event)(urma_async_event_t* event);
  int (*user_ctl)(urma_context_t* ctx, urma_user_ctl_in_t* in, urma_user_ctl_out_t* out);
} urma_ops_t;

typedef struct urma_provider_ops {
  const char* name;
  urma_status_t (*init)(const urma_init_attr_t* attr);
  urma_status_t (*uninit)(void);
  /* fills up to `max` devices, returns how many exist */
  int (*get_devices)(urma_device_t* devs, int max);
  urma_status_t (*query_device)(const urma_device_t* dev, urma_device_attr_t* attr);
  urma_context_t* (*create_context)(urma_device_t* dev, uint32_t eid_index);
  urma_status_t (*delete_context)(urma_context_t* ctx);
} urma_provider_ops_t;

/* Called by providers (typically from a constructor of a liburma-*.so plug-in, or statically for built-ins). */
URMA_EXPORT int urma_register_provider_ops(const urma_provider_ops_t* ops);
URMA_EXPORT int urma_unregister_provider_ops(const urma_provider_ops_t* ops);

#ifdef __cplusplus
}
#endif
#endif
