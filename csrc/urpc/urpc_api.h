/* URPC: remote function calls over UMQ queues. API shape follows the reference's
 * src/urpc/include/framework/urpc_framework_api.h:29-638 (init, server start, channels, queues, function
 * registration, call / poll / return, keepalive, statistics); wire headers follow the field list of
 * src/urpc/framework/protocol/protocol.h (version, message type, ack bit, 48-bit function id, request id,
 * 24-bit client channel, total size, DMA descriptor count). */
#ifndef UMDK_URPC_API_H
#define UMDK_URPC_API_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define URPC_EXPORT __attribute__((visibility("default")))

#define URPC_SUCCESS 0
#define URPC_FAIL (-1)
#define URPC_ERR_EINVAL (-22)
#define URPC_ERR_EAGAIN (-11)
#define URPC_ERR_TIMEOUT (-110)
#define URPC_ERR_SESSION_CLOSE (-104)
#define URPC_ERR_FUNC_NOT_FOUND (-38)
#define URPC_ERR_VERSION (-71)   /* no protocol version in common with the peer */
#define URPC_ERR_CANCELED (-125) /* the client cancelled the request this answer belongs to */

typedef enum urpc_role { URPC_ROLE_SERVER = 0, URPC_ROLE_CLIENT = 1, URPC_ROLE_SERVER_CLIENT = 2 } urpc_role_t;
typedef enum urpc_msg_type { URPC_MSG_REQ = 0, URPC_MSG_ACK = 1, URPC_MSG_RSP = 2, URPC_MSG_ACK_AND_RSP = 3,
                             URPC_MSG_READ = 4 } urpc_msg_type_t;
/* URPC_POLL_ACK: the server took a request that asked for an acknowledgement (want_ack) and will answer it later;
 * the call stays pending. Only between peers that negotiated protocol version 2. */
typedef enum urpc_poll_event { URPC_POLL_REQ = 1, URPC_POLL_RSP = 2, URPC_POLL_ERR = 3, URPC_POLL_TIMEOUT = 4,
                               URPC_POLL_ACK = 5 } urpc_poll_event_t;

#define URPC_FUNC_ID_KEEPALIVE 0xFFFFFFFFFFFFull /* reserved 48-bit id */
#define URPC_FUNC_ID_LOOKUP 0xFFFFFFFFFFFEull    /* reserved: function name -> id (urpc_func_id_get) */

typedef struct urpc_config {
  urpc_role_t role;
  char dev_name[64];
  uint32_t keepalive_interval_ms; /* 0 = off */
  uint32_t keepalive_miss_limit;  /* peer declared lost after this many unanswered probes (default 3) */
  uint32_t default_timeout_ms;    /* request timeout (default 5000) */
} urpc_config_t;

/* Wire header, 32 bytes, little endian bit packing done by hand (endianness-safe accessors in urpc_proto.h). */
typedef struct urpc_req_head {
  uint8_t bytes[32];
} urpc_req_head_t;

typedef struct urpc_sge {
  void* addr;
  uint32_t len;
} urpc_sge_t;

typedef struct urpc_call_wr {
  uint64_t func_id;
  urpc_sge_t* args;
  uint32_t num_args;
  uint64_t user_ctx;
} urpc_call_wr_t;

typedef struct urpc_call_option {
  uint32_t timeout_ms; /* 0 = default */
  int sync;            /* 1: block until the response (or timeout) and copy it to rsp_buf */
  void* rsp_buf;
  uint32_t rsp_buf_len;
  uint32_t* rsp_len;
  int want_ack;        /* 1: ask the server to acknowledge the request when it defers the answer (URPC_POLL_ACK) */
} urpc_call_option_t;

typedef struct urpc_poll_msg {
  urpc_poll_event_t event;
  uint64_t func_id;
  uint32_t req_id;
  uint64_t user_ctx;  /* client side: the call's user_ctx */
  void* data;         /* request arguments (server) or response payload (client); valid until urpc_msg_release */
  uint32_t len;
  int status;
  void* priv;
} urpc_poll_msg_t;

/* Handler of a registered function: fills rsp (capacity *rsp_len) and sets *rsp_len. Return value = status. */
typedef int (*urpc_func_t)(const void* args, uint32_t len, void* rsp, uint32_t* rsp_len, void* ctx);
typedef void (*urpc_keepalive_cb_t)(uint32_t chid, int alive, void* ctx);

/* Security: a pre-shared key (hex, 16..64 bytes) makes the connection handshake run inside TLS 1.3 PSK
 * (TLS_AES_256_GCM_SHA384) and seals every request / response payload with AES-256-GCM under a per-connection key
 * the server hands out in that handshake. Empty key = off. Without a call the key comes from URPC_PSK /
 * URPC_PSK_ID in the environment. Call before urpc_server_start / urpc_channel_server_attach. */
URPC_EXPORT int urpc_set_psk(const char* key_hex, const char* identity);
/* Certificates instead of a shared key (they take precedence): PEM files of the CA, of this process's certificate chain
 * and of its private key; the handshake is then TLS 1.3 with mutual authentication. Three empty strings switch it off.
 * Environment: URPC_TLS_CA / URPC_TLS_CERT / URPC_TLS_KEY. */
URPC_EXPORT int urpc_set_tls_files(const char* ca_file, const char* cert_file, const char* key_file);
URPC_EXPORT int urpc_init(const urpc_config_t* cfg);
URPC_EXPORT void urpc_uninit(void);
/* server */
URPC_EXPORT int urpc_server_start(const char* ip, uint16_t port); /* returns the bound port (> 0) or < 0 */
URPC_EXPORT int urpc_func_register(uint64_t func_id, urpc_func_t fn, void* ctx);
URPC_EXPORT int urpc_func_unregister(uint64_t func_id);
/* Polls every attached client: executes registered functions and returns their results (auto mode), or hands the
 * request to the caller when no function is registered. Returns the number of messages written to msgs. */
URPC_EXPORT int urpc_server_poll(urpc_poll_msg_t* msgs, int max);
/* The same for one share of the clients: thread k of n server threads calls it with (k, n) and serves the sessions
 * whose number is k modulo n, so the threads never meet on a queue. */
URPC_EXPORT int urpc_server_poll_shard(uint32_t shard, uint32_t nshards, urpc_poll_msg_t* msgs, int max);
URPC_EXPORT int urpc_func_return(const urpc_poll_msg_t* req, const void* rsp, uint32_t len, int status);
/* client */
URPC_EXPORT int urpc_channel_create(void); /* returns channel id >= 0 */
URPC_EXPORT int urpc_channel_server_attach(uint32_t chid, const char* ip, uint16_t port);
URPC_EXPORT int urpc_channel_server_detach(uint32_t chid);
URPC_EXPORT int urpc_channel_destroy(uint32_t chid);
URPC_EXPORT int urpc_func_call(uint32_t chid, const urpc_call_wr_t* wr, const urpc_call_option_t* opt);
URPC_EXPORT int urpc_func_poll(uint32_t chid, urpc_poll_msg_t* msgs, int max);
URPC_EXPORT void urpc_msg_release(urpc_poll_msg_t* msg);
URPC_EXPORT int urpc_keepalive_callback_register(urpc_keepalive_cb_t cb, void* ctx);
URPC_EXPORT int urpc_channel_task_cancel(uint32_t chid, uint32_t req_id);
/* dfx */
typedef struct urpc_stats {
  uint64_t calls, responses, timeouts, errors, requests_served, keepalive_sent, keepalive_lost, bytes_tx, bytes_rx;
} urpc_stats_t;
URPC_EXPORT int urpc_stats_get(urpc_stats_t* out);
URPC_EXPORT int urpc_perf_get(uint64_t* count, uint64_t* avg_ns, uint64_t* p99_ns); /* call -> response latency */
/* User recorder: called with (record point, nanoseconds, ctx) at the points below; NULL unregisters.
 * FUNC_CALL = time inside urpc_func_call until the request is queued, CALL_TO_RESPONSE = request queued until its
 * response is matched, FUNC_EXEC = the registered handler on the server, FUNC_RETURN = sending the response. */
typedef enum urpc_perf_point { URPC_PERF_FUNC_CALL = 0, URPC_PERF_CALL_TO_RESPONSE, URPC_PERF_FUNC_EXEC,
                               URPC_PERF_FUNC_RETURN, URPC_PERF_POINT_MAX } urpc_perf_point_t;
typedef void (*urpc_perf_recorder_t)(urpc_perf_point_t point, uint64_t ns, void* ctx);
URPC_EXPORT int urpc_perf_recorder_register(urpc_perf_recorder_t cb, void* ctx);
/* Logging: level 0 (errors) .. 4 (debug), default 1 or URPC_LOG_LEVEL; cb NULL = stderr. */
typedef void (*urpc_log_cb_t)(int level, const char* msg);
URPC_EXPORT int urpc_log_config_set(int level, urpc_log_cb_t cb);
/* Arguments by reference: register memory once, pass (handle, address, length) with a call, and let the server pull
 * the bytes it wants with one-sided reads instead of receiving them inline. Inside a registered handler pass
 * req = NULL ("the request being handled"); for requests taken with urpc_server_poll pass the message. */
#define URPC_MAX_REFS 16
typedef struct urpc_mem_ref {
  uint64_t mem_h;
  uint64_t addr;
  uint32_t len;
} urpc_mem_ref_t;
URPC_EXPORT uint64_t urpc_mem_seg_register(void* va, uint64_t len); /* 0 on failure */
URPC_EXPORT int urpc_mem_seg_unregister(uint64_t mem_h);
URPC_EXPORT int urpc_mem_seg_token_get(uint64_t mem_h, uint32_t* token);
URPC_EXPORT int urpc_mem_seg_remote_access_disable(uint64_t mem_h); /* descriptions already sent stop working */
URPC_EXPORT int urpc_mem_seg_remote_access_enable(uint64_t mem_h);
URPC_EXPORT int urpc_func_call_ref(uint32_t chid, const urpc_call_wr_t* wr, const urpc_mem_ref_t* refs,
                                   uint32_t num_refs, const urpc_call_option_t* opt);
URPC_EXPORT int urpc_ref_count(const urpc_poll_msg_t* req);
URPC_EXPORT int urpc_ref_len(const urpc_poll_msg_t* req, uint32_t idx, uint32_t* len);
URPC_EXPORT int urpc_ref_read(const urpc_poll_msg_t* req, uint32_t idx, uint64_t offset, void* buf, uint32_t len);
URPC_EXPORT int urpc_perf_recorder_unregister(void);
URPC_EXPORT int urpc_log_config_get(int* level);
typedef enum urpc_hdr_type { URPC_HDR_REQ = 0, URPC_HDR_ACK = 1, URPC_HDR_RSP = 2 } urpc_hdr_type_t;
URPC_EXPORT uint32_t urpc_hdr_size_get(urpc_hdr_type_t type, uint16_t flag);
typedef struct urpc_ssl_config {
  int enable;
  char psk_hex[132];
  char psk_identity[64];
} urpc_ssl_config_t;
URPC_EXPORT int urpc_ssl_config_set(const urpc_ssl_config_t* cfg); /* urpc_set_psk from a structure */
/* Function names: the server gives a registered function a name, a client looks the id up over its channel. */
URPC_EXPORT int urpc_func_name_register(uint64_t func_id, const char* name);
URPC_EXPORT uint64_t urpc_func_id_get(uint32_t chid, const char* name); /* 0 = unknown */
/* Local execution of a registered function (same handler a remote caller reaches), inline or on a helper thread. */
URPC_EXPORT int urpc_func_exec(uint64_t func_id, urpc_sge_t* args, uint32_t num_args, void* rsp, uint32_t* rsp_len);
typedef void (*urpc_async_exec_cb_t)(int status, const void* rsp, uint32_t rsp_len, void* user_ctx);
URPC_EXPORT int urpc_func_async_exec(uint64_t func_id, urpc_sge_t* args, uint32_t num_args, urpc_async_exec_cb_t done,
                                     void* user_ctx);
typedef void (*urpc_func_poll_cb_t)(uint32_t chid, const urpc_poll_msg_t* msg);
URPC_EXPORT int urpc_func_poll_cb_register(urpc_func_poll_cb_t cb); /* called for every message urpc_func_poll returns */
URPC_EXPORT int urpc_func_poll_cb_unregister(void);
URPC_EXPORT int urpc_func_poll_wait(uint32_t chid, urpc_poll_msg_t* msgs, int max, int timeout_ms);
typedef enum urpc_ctrl_msg_type { URPC_CTRL_ATTACH = 1, URPC_CTRL_DETACH = 2 } urpc_ctrl_msg_type_t;
typedef void (*urpc_ctrl_cb_t)(urpc_ctrl_msg_type_t type, uint32_t session, uint32_t client_channel);
URPC_EXPORT int urpc_ctrl_msg_cb_register(urpc_ctrl_cb_t cb); /* server: a client attached / detached */
/* FUNC_CHANGED: the attached server registered (detail 1) or unregistered (detail 0) a function. */
typedef enum urpc_async_event_type { URPC_EVENT_CHANNEL_LOST = 1, URPC_EVENT_CHANNEL_REFRESHED = 2,
                                     URPC_EVENT_FUNC_CHANGED = 3 } urpc_async_event_type_t;
typedef struct urpc_async_event {
  urpc_async_event_type_t type;
  uint32_t chid;
  int detail;
} urpc_async_event_t;
URPC_EXPORT int urpc_async_event_get(urpc_async_event_t* events, int num);
URPC_EXPORT int urpc_async_event_fd_get(void);
typedef struct urpc_channel_cfg {
  uint32_t timeout_ms; /* settable: request timeout of this channel (0 = library default) */
  int attached, lost, sealed;
  int proto_version;   /* negotiated at attach time (0 while detached) */
  uint32_t proto_caps; /* capability bits both sides have */
  uint32_t pending_calls;
  char server_ip[64];
  uint16_t server_port;
} urpc_channel_cfg_t;
URPC_EXPORT int urpc_channel_cfg_get(uint32_t chid, urpc_channel_cfg_t* cfg);
URPC_EXPORT int urpc_channel_cfg_set(uint32_t chid, const urpc_channel_cfg_t* cfg);
URPC_EXPORT int urpc_channel_server_refresh(uint32_t chid); /* detach + attach to the same server: new queue pair */
/* Queues: a channel's queue is a UMQ handle; these calls report on it. */
typedef enum urpc_queue_status { URPC_QUEUE_IDLE = 0, URPC_QUEUE_READY = 1, URPC_QUEUE_ERROR = 2 } urpc_queue_status_t;
typedef struct urpc_queue_cfg {
  uint32_t rx_depth, tx_depth, rx_buf_size; /* 0 = 128, 128, 64 KiB */
  int interrupt;                            /* completion events instead of polling */
} urpc_queue_cfg_t;
/* Explicit queues: created on their own and given to a channel. Before the attach the first one replaces the queue
 * the channel made for itself and the others become further queue pairs; on an ATTACHED channel (protocol version 2)
 * urpc_channel_queue_add pairs the queue with a new server queue through a control message and calls start to use
 * it at once, urpc_channel_queue_rm waits for the calls in flight on it, retires the pair and hands the queue
 * back. Depths and sizes are fixed at creation. */
/* Control-plane task engine of the server (one thread, asynchronous multi-step tasks): counters for dfx. */
typedef struct urpc_ctl_stats {
  uint64_t tasks_started, tasks_done, tasks_failed, tasks_timed_out, notices_sent, sessions_retired;
  uint32_t tasks_live, timers_armed;
} urpc_ctl_stats_t;
URPC_EXPORT int urpc_ctl_stats_get(urpc_ctl_stats_t* out);
URPC_EXPORT uint64_t urpc_queue_create(const urpc_queue_cfg_t* cfg); /* 0 on failure */
URPC_EXPORT int urpc_queue_destroy(uint64_t qh);
URPC_EXPORT int urpc_queue_cfg_get(uint64_t qh, urpc_queue_cfg_t* cfg);
URPC_EXPORT int urpc_queue_cfg_set(uint64_t qh, const urpc_queue_cfg_t* cfg);
URPC_EXPORT int urpc_queue_modify(uint64_t qh, urpc_queue_status_t status);
URPC_EXPORT int urpc_queue_rx_post(uint64_t qh, uint32_t num);
// A channel holds up to 16 queues. The first explicit queue replaces the one the channel made for itself, each further
// one becomes another lane; all of them are paired with queues of the server during the attach. urpc_func_call spreads
// requests over the lanes in turn, urpc_func_call_on names the lane; the response returns on the lane of its request.
URPC_EXPORT int urpc_func_call_on(uint32_t chid, uint64_t qh, const urpc_call_wr_t* wr, const urpc_call_option_t* opt);
URPC_EXPORT int urpc_channel_queue_add(uint32_t chid, uint64_t qh);
URPC_EXPORT int urpc_channel_queue_rm(uint32_t chid, uint64_t qh);
URPC_EXPORT int urpc_channel_queue_pair(uint32_t chid, uint64_t local_qh);
URPC_EXPORT int urpc_channel_queue_unpair(uint32_t chid, uint64_t local_qh);
typedef struct urpc_allocator {
  void* (*alloc)(size_t);
  void (*free)(void*);
} urpc_allocator_t;
/* Allocator for the copies handed out by urpc_rsp_copy (a response kept beyond urpc_msg_release). */
URPC_EXPORT int urpc_allocator_register(const urpc_allocator_t* a);
URPC_EXPORT int urpc_allocator_unregister(void);
URPC_EXPORT void* urpc_rsp_copy(const void* data, uint32_t len);
URPC_EXPORT void urpc_rsp_free(void* p);
URPC_EXPORT int urpc_channel_queue_query(uint32_t chid, uint64_t* qh, uint32_t max);
URPC_EXPORT int urpc_queue_status_query(uint64_t qh, urpc_queue_status_t* status);
URPC_EXPORT int urpc_queue_interrupt_fd_get(uint64_t qh);
URPC_EXPORT int urpc_queue_stats_get(uint64_t qh, uint64_t* stats, int len);       /* 4 counters */
URPC_EXPORT const char* urpc_queue_stats_name_get(int type);
URPC_EXPORT int urpc_queue_error_stats_get(uint64_t qh, uint64_t* stats, int len); /* 3 counters */
URPC_EXPORT const char* urpc_queue_error_stats_name_get(int type);
URPC_EXPORT int urpc_error_stats_get(uint64_t* stats, int len);                    /* errors, timeouts, peers lost */
/* Management socket: a unix-domain stream socket at `path` that answers one text command per connection
 * ("version", "stats", "perf", "channels", "sessions", "funcs") with a text report; `urpc_admin` is its client.
 * Also started by urpc_init when the environment names a path in URPC_ADMIN_SOCKET. */
URPC_EXPORT int urpc_admin_start(const char* path);
URPC_EXPORT void urpc_admin_stop(void);
/* the same reports without a socket; returns the number of bytes written (truncated to cap - 1) or < 0 */
URPC_EXPORT int urpc_admin_query(const char* command, char* out, uint32_t cap);
#ifdef __cplusplus
}
#endif
#endif
