/* DLock: distributed locks and 64-bit atomic objects served from one process, with a TCP control channel and an
 * URMA data channel. API shape follows the reference's src/ulock/dlock/lib/include/dlock_client_api.h:25-512,
 * dlock_server_api.h:25-62 and dlock_types.h:20-140 (lock kinds ATOMIC / RW / FAIR, operations, batch limit 31,
 * status codes, debug statistics). */
#ifndef UMDK_DLOCK_API_H
#define UMDK_DLOCK_API_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
#define DLOCK_EXPORT __attribute__((visibility("default")))
#define DLOCK_MAX_BATCH 31
#define DLOCK_NAME_LEN 64

typedef enum dlock_status {
  DLOCK_SUCCESS = 0,
  DLOCK_DONE = 1,
  DLOCK_FAIL = -1,
  DLOCK_EINVAL = -22,
  DLOCK_EAGAIN = 0x1000,          /* lock is held by someone else */
  DLOCK_ALREADY_LOCKED = 0x1001,
  DLOCK_NOT_OWNER = 0x1002,
  DLOCK_LOCK_NOT_FOUND = 0x1003,
  DLOCK_TIMEOUT = 0x1004,
  DLOCK_CLIENT_NOT_INIT = 0x2000,
  DLOCK_BAD_RESPONSE = 0x2001,    /* server unreachable or restarted: call dlock_client_reinit */
  DLOCK_NOT_READY = 0x2002,       /* server is still recovering lock state from its clients */
  DLOCK_SERVER_FULL = 0x2003,
  DLOCK_EASYNC = 0x2004,          /* an asynchronous request is outstanding: collect it first */
  DLOCK_NO_ASYNC = 0x2005,        /* dlock_lock_result_check without a request */
  DLOCK_ASYNC_AGAIN = 0x2006,     /* the answer has not arrived yet: check again */
} dlock_status_t;

typedef enum dlock_type { DLOCK_ATOMIC = 0, DLOCK_RW = 1, DLOCK_FAIR = 2 } dlock_type_t;
typedef enum dlock_op { DLOCK_LOCK_EXCLUSIVE = 0, DLOCK_LOCK_SHARED = 1, DLOCK_UNLOCK = 2, DLOCK_EXTEND = 3 } dlock_op_t;

typedef struct dlock_server_cfg {
  char ip[32];
  uint16_t port;                 /* 0 = pick one */
  uint32_t max_clients;          /* default 1000 */
  uint32_t max_locks;            /* default 51200 */
  uint32_t max_objects;          /* default 4096 */
  uint32_t recovery_client_num;  /* > 0: start in recovery mode and wait for this many clients to re-register */
  uint32_t recovery_timeout_ms;  /* default 3000 */
  char dev_name[64];
} dlock_server_cfg_t;

typedef struct dlock_lock_desc {
  char name[DLOCK_NAME_LEN];
  dlock_type_t type;
} dlock_lock_desc_t;

typedef struct dlock_lock_req {
  int32_t lock_id;
  dlock_op_t op;
  uint32_t expire_ms; /* lease: the lock may be taken over after this time unless extended */
} dlock_lock_req_t;

typedef struct dlock_debug_stats {
  uint64_t trylock_ok, trylock_busy, unlock_ok, unlock_fail, extend_ok, expired_takeover, heartbeat, recovered_locks,
      control_msgs, data_msgs, objects, object_ops, clients,
      tls_rejected,    /* control connections refused: TLS handshake failed (wrong key, clear-text client) */
      sealed_rejected; /* data-channel commands dropped: unknown sender, bad seal, replay, or clear text to a secured server */
} dlock_debug_stats_t;

/* Security: a pre-shared key (hex, 16..64 bytes) switches the control channel to TLS 1.3 PSK and seals the data
 * channel with AES-256-GCM; an empty key switches both off. Applies to servers started and clients initialised
 * afterwards. Without a call the key comes from DLOCK_PSK / DLOCK_PSK_ID in the environment. */
DLOCK_EXPORT int dlock_set_psk(const char* key_hex, const char* identity);
/* Certificates instead of a shared key (they take precedence): PEM files of the CA that signs the peers, of this
 * process's certificate chain and of its private key. The control channel then runs TLS 1.3 with mutual
 * authentication (a peer without a certificate of that CA is refused) and the data channel is sealed as with a key.
 * Three empty strings switch it off. Environment: DLOCK_TLS_CA / DLOCK_TLS_CERT / DLOCK_TLS_KEY. */
DLOCK_EXPORT int dlock_set_tls_files(const char* ca_file, const char* cert_file, const char* key_file);

/* server */
DLOCK_EXPORT int dlock_server_start(const dlock_server_cfg_t* cfg, int* server_id, uint16_t* port_out);
DLOCK_EXPORT int dlock_server_stop(int server_id);
DLOCK_EXPORT int dlock_get_server_debug_stats(int server_id, dlock_debug_stats_t* out);
/* client */
DLOCK_EXPORT int dlock_client_init(int* client_id, const char* server_ip, uint16_t port);
DLOCK_EXPORT int dlock_client_reinit(int client_id, const char* server_ip, uint16_t port);
DLOCK_EXPORT int dlock_client_deinit(int client_id);
DLOCK_EXPORT int dlock_client_heartbeat(int client_id, uint32_t timeout_ms);
DLOCK_EXPORT int dlock_get_lock(int client_id, const dlock_lock_desc_t* desc, int32_t* lock_id);
DLOCK_EXPORT int dlock_release_lock(int client_id, int32_t lock_id);
DLOCK_EXPORT int dlock_batch_get_lock(int client_id, uint32_t n, const dlock_lock_desc_t* descs, int32_t* lock_ids);
DLOCK_EXPORT int dlock_trylock(int client_id, const dlock_lock_req_t* req);
DLOCK_EXPORT int dlock_lock(int client_id, const dlock_lock_req_t* req, uint32_t timeout_ms);
DLOCK_EXPORT int dlock_unlock(int client_id, int32_t lock_id);
DLOCK_EXPORT int dlock_lock_extend(int client_id, int32_t lock_id, uint32_t expire_ms);
DLOCK_EXPORT int dlock_batch_trylock(int client_id, uint32_t n, const dlock_lock_req_t* reqs, int* results);
DLOCK_EXPORT int dlock_batch_unlock(int client_id, uint32_t n, const int32_t* lock_ids, int* results);
DLOCK_EXPORT int dlock_update_all_locks(int client_id); /* after reinit: push held locks to the new server */
DLOCK_EXPORT int dlock_client_reinit_done(int client_id); /* after update_all_locks: this client is fully back */
DLOCK_EXPORT int dlock_batch_lock_extend(int client_id, uint32_t n, const dlock_lock_req_t* reqs, int* results);
DLOCK_EXPORT int dlock_batch_release_lock(int client_id, uint32_t n, const int32_t* lock_ids);
/* One asynchronous lock / unlock / extend per client: send now, collect the status later with result_check
 * (DLOCK_ASYNC_AGAIN until the answer is there, DLOCK_TIMEOUT after 5 s). */
DLOCK_EXPORT int dlock_lock_request_async(int client_id, const dlock_lock_req_t* req);
DLOCK_EXPORT int dlock_lock_result_check(int client_id, int* result);
DLOCK_EXPORT int dlock_clear_client_debug_stats(int client_id);
DLOCK_EXPORT int dlock_clear_server_debug_stats(int server_id);
/* Library contexts: defaults (URMA device, pre-shared key) for instances created afterwards; the last deinit stops
 * every instance that is still running. */
typedef struct dlock_lib_cfg {
  char dev_name[64];
  char psk_hex[132];
  char psk_identity[64];
} dlock_lib_cfg_t;
DLOCK_EXPORT int dlock_client_lib_init(const dlock_lib_cfg_t* cfg);
DLOCK_EXPORT void dlock_client_lib_deinit(void);
DLOCK_EXPORT int dlock_server_lib_init(const dlock_lib_cfg_t* cfg);
DLOCK_EXPORT void dlock_server_lib_deinit(void);
DLOCK_EXPORT int dlock_get_client_debug_stats(int client_id, dlock_debug_stats_t* out);
/* 64-bit atomic objects (one-sided URMA atomics on the server's object segment) */
DLOCK_EXPORT int dlock_umo_atomic64_create(int client_id, const char* name, uint64_t init, int32_t* obj_id);
DLOCK_EXPORT int dlock_umo_atomic64_get(int client_id, const char* name, int32_t* obj_id);
DLOCK_EXPORT int dlock_umo_atomic64_destroy(int client_id, int32_t obj_id);
DLOCK_EXPORT int dlock_umo_atomic64_release(int client_id, int32_t obj_id); /* drop the handle, keep the object */
DLOCK_EXPORT int dlock_umo_atomic64_faa(int client_id, int32_t obj_id, uint64_t add, uint64_t* old);
DLOCK_EXPORT int dlock_umo_atomic64_cas(int client_id, int32_t obj_id, uint64_t cmp, uint64_t swap, uint64_t* old);
DLOCK_EXPORT int dlock_umo_atomic64_get_snapshot(int client_id, int32_t obj_id, uint64_t* value);
#ifdef __cplusplus
}
#endif
#endif
