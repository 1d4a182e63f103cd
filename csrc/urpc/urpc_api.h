/* URPC: remote function calls over UMQ queues. API shape follows the reference's
 * src/urpc/include/framework/urpc_framework_api.h:29-638 (init, server start, channels, queues, function
 * registration, call / poll / return, keepalive, statistics); wire headers follow the field list of
 * src/urpc/framework/protocol/protocol.h (version, message type, ack bit, 48-bit function id, request id,
 * 24-bit client channel, total size, DMA descriptor count). */
#ifndef UMDK_URPC_API_H
#define UMDK_URPC_API_H
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

typedef enum urpc_role { URPC_ROLE_SERVER = 0, URPC_ROLE_CLIENT = 1, URPC_ROLE_SERVER_CLIENT = 2 } urpc_role_t;
typedef enum urpc_msg_type { URPC_MSG_REQ = 0, URPC_MSG_ACK = 1, URPC_MSG_RSP = 2, URPC_MSG_ACK_AND_RSP = 3,
                             URPC_MSG_READ = 4 } urpc_msg_type_t;
typedef enum urpc_poll_event { URPC_POLL_REQ = 1, URPC_POLL_RSP = 2, URPC_POLL_ERR = 3, URPC_POLL_TIMEOUT = 4 }
    urpc_poll_event_t;

#define URPC_FUNC_ID_KEEPALIVE 0xFFFFFFFFFFFFull /* reserved 48-bit id */

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
URPC_EXPORT int urpc_init(const urpc_config_t* cfg);
URPC_EXPORT void urpc_uninit(void);
/* server */
URPC_EXPORT int urpc_server_start(const char* ip, uint16_t port); /* returns the bound port (> 0) or < 0 */
URPC_EXPORT int urpc_func_register(uint64_t func_id, urpc_func_t fn, void* ctx);
URPC_EXPORT int urpc_func_unregister(uint64_t func_id);
/* Polls every attached client: executes registered functions and returns their results (auto mode), or hands the
 * request to the caller when no function is registered. Returns the number of messages written to msgs. */
URPC_EXPORT int urpc_server_poll(urpc_poll_msg_t* msgs, int max);
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
