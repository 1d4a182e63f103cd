/* UMQ: handle-based message queues with managed buffers on top of URMA jetties.
 * API groups follow the reference's src/urpc/include/umq/umq_api.h:26-385 (init, create/destroy, bind, buffers,
 * enqueue/dequeue, interrupts, state), umq_pro_api.h:30-76 (post/poll) and umq_dfx_api.h:26-199 (stats, perf). */
#ifndef UMDK_UMQ_API_H
#define UMDK_UMQ_API_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define UMQ_EXPORT __attribute__((visibility("default")))

#define UMQ_SUCCESS 0
#define UMQ_FAIL (-1)
#define UMQ_ERR_EAGAIN (-11)
#define UMQ_ERR_EINVAL (-22)
#define UMQ_ERR_ENOMEM (-12)
#define UMQ_ERR_ESTATE (-108)
#define UMQ_INVALID_HANDLE 0
#define UMQ_BATCH_SIZE 256
#define UMQ_MAX_MSG_SIZE (10u << 20)
#define UMQ_BIND_INFO_SIZE 128

/* feature bits of umq_init_cfg_t.feature */
#define UMQ_FEATURE_API_BASE 0x1u
#define UMQ_FEATURE_API_PRO 0x2u
#define UMQ_FEATURE_STATS 0x8u
#define UMQ_FEATURE_PERF 0x10u
#define UMQ_FEATURE_FLOW_CONTROL 0x20u

typedef enum umq_trans_mode { UMQ_TRANS_MODE_UB = 0, UMQ_TRANS_MODE_IPC = 3 } umq_trans_mode_t;
typedef enum umq_queue_mode { UMQ_MODE_POLLING = 0, UMQ_MODE_INTERRUPT = 1 } umq_queue_mode_t;
typedef enum umq_state { UMQ_STATE_IDLE = 0, UMQ_STATE_READY = 1, UMQ_STATE_ERR = 2 } umq_state_t;
typedef enum umq_io_direction { UMQ_IO_TX = 0, UMQ_IO_RX = 1 } umq_io_direction_t;
typedef enum umq_buf_status { UMQ_BUF_OK = 0, UMQ_BUF_SEND_ERR = 1, UMQ_BUF_RECV_ERR = 2 } umq_buf_status_t;

typedef struct umq_init_cfg {
  uint32_t feature;
  umq_trans_mode_t trans_mode;
  char dev_name[64]; /* URMA device, "" = shm0 */
  uint32_t block_size_kb; /* qbuf block size: 8, 16, 32 or 64 (0 = 8) */
  uint64_t pool_bytes;    /* pool size at start, 0 = 64 MiB; an exhausted pool grows in batches up to 16 times this */
} umq_init_cfg_t;

typedef struct umq_create_option {
  char name[32];
  uint32_t rx_buf_size, tx_buf_size; /* 0 = block size */
  uint32_t rx_depth, tx_depth;       /* 0 = 128 */
  umq_queue_mode_t mode;
  uint32_t token;
  uint32_t transport; /* 0 = the transport mode given to umq_init, else (umq_trans_mode_t value + 1) for this queue */
  uint32_t create_flag;   /* UMQ_CREATE_FLAG_* */
  uint64_t share_rq_umqh; /* UMQ_CREATE_FLAG_SUB: the main queue whose receive buffers this queue shares */
} umq_create_option_t;
/* Main and sub queues. A MAIN queue is an ordinary queue that can also host sub queues; with SHARE_TRANSPORT its
 * endpoint joins the jetty pool. A SUB queue has no endpoint of its own: messages for it arrive in the main queue's
 * receive buffers (rx_depth and rx_buf_size are the main queue's, shared by all its sub queues) and it sends through
 * an endpoint borrowed from the pool, message by message - so a process with thousands of connections needs
 * receive buffers and jetties for its main queues only. A sub queue binds like any queue (to a plain queue, a main
 * queue or another sub queue); the main queue must be destroyed after its sub queues. */
#define UMQ_CREATE_FLAG_MAIN 1u
#define UMQ_CREATE_FLAG_SHARE_TRANSPORT 2u
#define UMQ_CREATE_FLAG_SUB 4u
typedef struct umq_jetty_pool_stats {
  uint64_t total_num;     /* endpoints in the pool */
  uint64_t err_num;       /* of which in the ERR state right now */
  uint64_t acc_alloc_num; /* posts that borrowed an endpoint */
  uint64_t acc_free_num;  /* ... and gave it back (an endpoint is held for one post) */
  uint64_t acc_miss_num;  /* attempts that found an endpoint's send queue full and moved on */
  uint64_t sub_queues;    /* sub queues alive */
} umq_jetty_pool_stats_t;
UMQ_EXPORT int umq_jetty_pool_stats_get(umq_jetty_pool_stats_t* out);
UMQ_EXPORT int umq_jetty_pool_eventfd_get(void); /* becomes readable when an endpoint joins the pool */

/* Message buffer. `buf_data` points `headroom_size` bytes into the block; buffers chain through `qbuf_next`. */
typedef struct umq_buf {
  struct umq_buf* qbuf_next;
  uint64_t umqh;
  uint32_t total_data_size; /* of the whole chain, valid in the first buffer */
  uint32_t buf_size;        /* capacity of this buffer's data area */
  uint32_t data_size;       /* valid bytes at buf_data */
  uint16_t headroom_size;
  uint16_t status;          /* umq_buf_status_t after completion */
  uint64_t user_ctx;
  char* buf_data;
  uint64_t rsvd[8];
} umq_buf_t;

UMQ_EXPORT int umq_init(const umq_init_cfg_t* cfg);
UMQ_EXPORT void umq_uninit(void);
UMQ_EXPORT uint64_t umq_create(const umq_create_option_t* opt);
UMQ_EXPORT int umq_destroy(uint64_t umqh);
UMQ_EXPORT uint32_t umq_bind_info_get(uint64_t umqh, uint8_t* bind_info, uint32_t size);
UMQ_EXPORT int umq_bind(uint64_t umqh, const uint8_t* bind_info, uint32_t size);
UMQ_EXPORT int umq_unbind(uint64_t umqh);
UMQ_EXPORT int umq_state_set(uint64_t umqh, umq_state_t state);
UMQ_EXPORT umq_state_t umq_state_get(uint64_t umqh);
/* buffers */
UMQ_EXPORT umq_buf_t* umq_buf_alloc(uint32_t request_size, uint32_t request_qbuf_num, uint64_t umqh);
UMQ_EXPORT void umq_buf_free(umq_buf_t* qbuf);
UMQ_EXPORT int umq_buf_headroom_reset(umq_buf_t* qbuf, uint16_t headroom_size);
UMQ_EXPORT int umq_buf_reset(umq_buf_t* qbuf);
/* base API */
UMQ_EXPORT int umq_enqueue(uint64_t umqh, umq_buf_t* qbuf, umq_buf_t** bad_qbuf);
UMQ_EXPORT umq_buf_t* umq_dequeue(uint64_t umqh);
/* pro API */
UMQ_EXPORT int umq_post(uint64_t umqh, umq_buf_t* qbuf, umq_io_direction_t dir, umq_buf_t** bad_qbuf);
UMQ_EXPORT int umq_poll(uint64_t umqh, umq_io_direction_t dir, umq_buf_t** bufs, uint32_t max);
/* interrupt mode */
UMQ_EXPORT int umq_rearm_interrupt(uint64_t umqh, int solicited, umq_io_direction_t dir);
UMQ_EXPORT int umq_wait_interrupt(uint64_t umqh, int timeout_ms);
UMQ_EXPORT void umq_ack_interrupt(uint64_t umqh, uint32_t nevents);
UMQ_EXPORT int umq_interrupt_fd_get(uint64_t umqh);
/* dfx */
typedef struct umq_io_stats {
  uint64_t tx_msgs, tx_bytes, rx_msgs, rx_bytes, tx_errors, rx_errors, tx_eagain;
  uint64_t pull_tx, pull_rx; /* messages that went through the large-message pull path (also counted above) */
} umq_io_stats_t;
typedef struct umq_fc_stats {
  uint64_t credits_local, credits_remote, credits_granted, credits_returned, stalls, window;
} umq_fc_stats_t;
typedef struct umq_qbuf_stats {
  uint64_t block_size, blocks_total, blocks_free, huge_allocs, alloc_calls, free_calls, alloc_failures;
} umq_qbuf_stats_t;
typedef struct umq_perf_entry {
  uint64_t count, avg_ns, min_ns, max_ns, p99_ns;
} umq_perf_entry_t;
typedef enum umq_perf_record { UMQ_PERF_ENQUEUE = 0, UMQ_PERF_DEQUEUE, UMQ_PERF_POST_TX, UMQ_PERF_POLL_RX,
                               UMQ_PERF_BUF_ALLOC, UMQ_PERF_RECORD_MAX } umq_perf_record_t;
UMQ_EXPORT int umq_stats_io_get(uint64_t umqh, umq_io_stats_t* out);
UMQ_EXPORT int umq_stats_flow_control_get(uint64_t umqh, umq_fc_stats_t* out);
UMQ_EXPORT int umq_stats_qbuf_pool_get(umq_qbuf_stats_t* out);
UMQ_EXPORT int umq_stats_perf_start(void);
UMQ_EXPORT int umq_stats_perf_stop(void);
UMQ_EXPORT int umq_stats_perf_get(umq_perf_entry_t* entries /* [UMQ_PERF_RECORD_MAX] */);
/* ---- transports ----
 * Every transport mode has an entry in a table of operations; a queue is served by the entry of its mode. Mode UB is
 * the built-in URMA transport (send / receive over jetties, credits in the immediate data). Mode IPC is a built-in
 * in-process transport: two queues of one process hand buffers to each other without copying. Further modes can be
 * added (or these replaced) with umq_transport_register before queues of that mode are created - the counterpart of the
 * reference's per-mode framework table (src/urpc/umq/umq_api.c:65-204, 258-270). */
typedef struct umq_transport_ops {
  const char* name;
  int (*create)(uint64_t umqh, const umq_create_option_t* opt, void** priv);
  void (*destroy)(void* priv);
  uint32_t (*bind_info_get)(void* priv, uint8_t* out, uint32_t size);
  int (*bind)(void* priv, const uint8_t* info, uint32_t size);
  int (*unbind)(void* priv);
  int (*send)(void* priv, struct umq_buf* one); /* one buffer; ownership passes to the transport on success */
  struct umq_buf* (*recv)(void* priv);          /* next received buffer or NULL; the caller frees it */
} umq_transport_ops_t;
UMQ_EXPORT int umq_transport_register(umq_trans_mode_t mode, const umq_transport_ops_t* ops);
UMQ_EXPORT const char* umq_transport_name(umq_trans_mode_t mode);
/* ---- buffer lists ---- */
/* Cuts the list at `node`: `head` keeps the buffers before it, `node` starts a list of its own (sizes recomputed). */
UMQ_EXPORT int umq_buf_split(umq_buf_t* head, umq_buf_t* node);
/* A list may hold several messages back to back: frees the first one, returns the first buffer of the next. */
UMQ_EXPORT umq_buf_t* umq_buf_break_and_free(umq_buf_t* qbuf);
/* The buffer whose data area contains `data` (NULL if it is not a buffer of this library). */
UMQ_EXPORT umq_buf_t* umq_data_to_head(void* data);
/* Runs the completion path of the queue (returns credits, completes sends). */
UMQ_EXPORT void umq_notify(uint64_t umqh);

/* ---- memory by reference ---- */
/* Registers readable memory; `blob` (UMQ_SEG_BLOB_SIZE bytes) is the description a peer needs to read it. */
#define UMQ_SEG_BLOB_SIZE 64
UMQ_EXPORT uint64_t umq_mem_seg_register(void* va, uint64_t len, uint32_t token, uint8_t* blob, uint32_t blob_cap);
UMQ_EXPORT int umq_mem_seg_unregister(uint64_t seg_h);
/* One-sided read of the peer's registered memory over the queue's endpoint; blocks until done or timeout. */
UMQ_EXPORT int umq_remote_read(uint64_t umqh, const uint8_t* seg_blob, uint32_t token, uint64_t remote_addr, void* local,
                               uint32_t len, int timeout_ms);

/* ---- queries ---- */
typedef struct umq_cfg_get {
  umq_create_option_t create_option;
  umq_state_t state;
  uint32_t feature;
  umq_trans_mode_t trans_mode;
  uint32_t block_size;
} umq_cfg_get_t;
UMQ_EXPORT int umq_cfg_get(uint64_t umqh, umq_cfg_get_t* cfg);
typedef struct umq_dev_info {
  char dev_name[64];
  uint8_t eid[16];
  umq_trans_mode_t trans_mode;
  uint64_t max_msg_size;
  uint32_t port_cnt;
} umq_dev_info_t;
UMQ_EXPORT int umq_dev_add(const char* dev_name);
UMQ_EXPORT int umq_dev_info_get(const char* dev_name, umq_trans_mode_t mode, umq_dev_info_t* out);
UMQ_EXPORT umq_dev_info_t* umq_dev_info_list_get(umq_trans_mode_t mode, int* dev_num);
UMQ_EXPORT void umq_dev_info_list_free(umq_trans_mode_t mode, umq_dev_info_t* list);
#define UMQ_MAX_ROUTES 32
typedef struct umq_route_key {
  uint8_t src_eid[16], dst_eid[16];
} umq_route_key_t;
typedef struct umq_route_list {
  uint32_t route_num;
  struct {
    uint8_t src_port_eid[16], dst_port_eid[16];
  } routes[UMQ_MAX_ROUTES];
} umq_route_list_t;
/* Port pairs that connect two devices according to the topology registry (uvs_topo.h). */
UMQ_EXPORT int umq_get_route_list(const umq_route_key_t* key, umq_trans_mode_t mode, umq_route_list_t* out);
typedef struct umq_mempool_state {
  uint64_t block_size, blocks_total, blocks_free, generation;
  int registered;
} umq_mempool_state_t;
UMQ_EXPORT int umq_mempool_state_get(uint64_t umqh, uint32_t mempool_id, umq_mempool_state_t* out);
UMQ_EXPORT int umq_mempool_state_refresh(uint64_t umqh, uint32_t mempool_id);
typedef enum umq_user_ctl_opcode { UMQ_USER_CTL_PROGRESS = 1, UMQ_USER_CTL_RETURN_CREDITS = 2 } umq_user_ctl_opcode_t;
typedef struct umq_user_ctl_in {
  uint32_t opcode;
  uint64_t arg;
} umq_user_ctl_in_t;
typedef struct umq_user_ctl_out {
  uint64_t value;
} umq_user_ctl_out_t;
UMQ_EXPORT int umq_user_ctl(uint64_t umqh, umq_user_ctl_in_t* in, umq_user_ctl_out_t* out);
UMQ_EXPORT int umq_interrupt_fd_list_get(uint64_t umqh, umq_io_direction_t dir, int* fds, uint32_t max);
UMQ_EXPORT int umq_get_cq_event(uint64_t umqh, umq_io_direction_t dir);

/* ---- plug-in lock / thread-key primitives for applications with their own threading runtime ---- */
typedef struct umq_external_mutex_ops {
  void* (*create)(void);
  int (*lock)(void*);
  int (*unlock)(void*);
  void (*destroy)(void*);
} umq_external_mutex_ops_t;
typedef struct umq_external_rwlock_ops {
  void* (*create)(void);
  int (*rdlock)(void*);
  int (*wrlock)(void*);
  int (*unlock)(void*);
  void (*destroy)(void*);
} umq_external_rwlock_ops_t;
typedef struct umq_external_thread_key_ops {
  int (*create)(uint32_t* key);
  int (*set)(uint32_t key, void* value);
  void* (*get)(uint32_t key);
  void (*destroy)(uint32_t key);
} umq_external_thread_key_ops_t;
UMQ_EXPORT int umq_external_mutex_lock_ops_register(const umq_external_mutex_ops_t* ops);
UMQ_EXPORT int umq_external_rwlock_ops_register(const umq_external_rwlock_ops_t* ops);
UMQ_EXPORT int umq_external_thread_key_ops_register(const umq_external_thread_key_ops_t* ops);

/* ---- transport pool: several queues behind one eventfd ---- */
typedef struct umq_transport_pool_stats {
  uint32_t queues, queues_ready;
  uint64_t wakeups;
} umq_transport_pool_stats_t;
UMQ_EXPORT uint64_t umq_transport_pool_resource_create(void);
UMQ_EXPORT int umq_transport_pool_resource_modify(uint64_t pool, uint64_t umqh, int add);
UMQ_EXPORT int umq_transport_pool_resource_destroy(uint64_t pool);
UMQ_EXPORT int umq_transport_pool_eventfd_get(uint64_t pool);
/* Polls the member queues once, signals the eventfd if any has messages ready, and reports the counts. */
UMQ_EXPORT int umq_stats_transport_pool_get(uint64_t pool, umq_transport_pool_stats_t* out);
UMQ_EXPORT int umq_transport_pool_stats_to_str(const umq_transport_pool_stats_t* s, char* buf, uint32_t len);

/* Logging: level 0 (errors) .. 4 (debug), default 1 or UMQ_LOG_LEVEL; cb NULL = stderr. */
typedef void (*umq_log_cb_t)(int level, const char* msg);
UMQ_EXPORT int umq_log_config_set(int level, umq_log_cb_t cb);
/* Called with (record point, duration in ns, ctx) after every API call at a perf record point; NULL unregisters. */
typedef void (*umq_io_perf_cb_t)(int record, uint64_t duration_ns, void* ctx);
UMQ_EXPORT int umq_io_perf_callback_register(umq_io_perf_cb_t cb, void* ctx);
/* Asynchronous events. UMQ_EVENT_QH_ERR: the queue entered UMQ_STATE_ERR (a send completed in error, or the
 * application set the state); detail = completion status. Returns UMQ_ERR_EAGAIN when there is none. */
typedef enum umq_async_event_type { UMQ_EVENT_QH_ERR = 1 } umq_async_event_type_t;
typedef struct umq_async_event {
  umq_async_event_type_t type;
  uint64_t umqh;
  int detail;
} umq_async_event_t;
UMQ_EXPORT int umq_async_event_get(umq_async_event_t* ev);
UMQ_EXPORT int umq_get_async_event(umq_async_event_t* ev);   /* same, under the reference's name */
UMQ_EXPORT void umq_ack_async_event(umq_async_event_t* ev);
UMQ_EXPORT int umq_async_event_fd_get(void);                 /* readable while events are queued */
UMQ_EXPORT int umq_log_config_get(int* level);
/* Trace: one text line `start_ns tid record duration_ns` per API call at the perf record points, collected in
 * per-thread rings (ring_entries each, 0 = 4096; a full ring drops and counts) and appended to `path` by a flusher
 * thread every flush_interval_ms (0 = 100). */
UMQ_EXPORT int umq_trace_start(const char* path, uint32_t flush_interval_ms, uint32_t ring_entries);
UMQ_EXPORT int umq_trace_stop(void);
UMQ_EXPORT int umq_trace_stats(uint64_t* written, uint64_t* dropped);
typedef struct umq_info {
  uint64_t umqh;
  char name[32];
  umq_state_t state;
  int bound;
  uint32_t rx_posted, rx_ready, tx_in_flight;
  int64_t credits;
  umq_io_stats_t io;
} umq_info_t;
UMQ_EXPORT int umq_info_get(uint64_t umqh, umq_info_t* info);
UMQ_EXPORT int umq_stats_io_reset(uint64_t umqh);
UMQ_EXPORT int umq_stats_perf_reset(void);
UMQ_EXPORT int umq_io_stats_to_str(const umq_io_stats_t* s, char* buf, uint32_t len);
UMQ_EXPORT int umq_flow_control_stats_to_str(const umq_fc_stats_t* s, char* buf, uint32_t len);
UMQ_EXPORT int umq_qbuf_pool_stats_to_str(const umq_qbuf_stats_t* s, char* buf, uint32_t len);
UMQ_EXPORT int umq_stats_perf_to_str(char* buf, uint32_t len);
UMQ_EXPORT int umq_stats_trace_start(const char* path);   /* umq_trace_start with default ring size and interval */
UMQ_EXPORT int umq_stats_trace_stop(void);
/* latency of the transport (URMA data-plane) calls underneath, from the URMA perf sampler */
UMQ_EXPORT int umq_stats_tp_perf_start(void);
UMQ_EXPORT int umq_stats_tp_perf_stop(void);
UMQ_EXPORT int umq_stats_tp_perf_info_get(char* buf, uint32_t* len);
UMQ_EXPORT int umq_info_to_str(uint64_t umqh, char* buf, uint32_t len);
#ifdef __cplusplus
}
#endif
#endif
