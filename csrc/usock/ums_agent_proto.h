// Token agent of the UMS sockets: wire format and the client calls of the library.
//
// A UMS endpoint publishes the token that protects its ring (an opaque value of up to 128 bytes) to the agent of its
// own host and hands the peer only a token id; the peer asks ITS agent for the value, and that agent fetches it from
// the first one over a TLS connection. Applications therefore never send token values over their own connection.
// Same role as the reference's ums_agent (src/usock/ums/ums_agent/ums_agent_token_proxy.c: token requests from the
// local side, ums_agent_tls_conn.c: pooled TLS connections between agents); the local side talks to the agent over a
// Unix stream socket here, where the reference's kernel module uses netlink (ums_agent_nl.c).
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UMS_AGENT_MAGIC 0x554d5341u /* "UMSA" */
#define UMS_AGENT_MAX_VALUE 128
#define UMS_AGENT_DEFAULT_SOCK "/tmp/ums_agent.sock"

enum ums_agent_op {
  UMS_AGENT_PUT = 1,   /* store token_id -> value in the local table */
  UMS_AGENT_DEL = 2,   /* forget token_id */
  UMS_AGENT_GET = 3,   /* peer empty: local table; peer "ip:port": ask that agent */
  UMS_AGENT_STATS = 4, /* value <- text report */
};

enum ums_agent_status {
  UMS_AGENT_OK = 0,
  UMS_AGENT_ENOENT = 1,  /* unknown token id */
  UMS_AGENT_EPEER = 2,   /* the peer agent cannot be reached or refused the TLS handshake */
  UMS_AGENT_EINVAL = 3,
  UMS_AGENT_EFULL = 4,   /* token table full */
};

/* One fixed-size record in each direction, on the Unix socket and between agents. */
typedef struct ums_agent_msg {
  uint32_t magic;
  uint32_t op;
  uint64_t token_id;
  uint32_t status; /* replies */
  uint32_t len;    /* bytes of value in use */
  char peer[64];   /* GET through the local agent: "ip:port" of the agent that holds the token */
  uint8_t value[UMS_AGENT_MAX_VALUE];
} ums_agent_msg_t;

#define UMS_AGENT_EXPORT __attribute__((visibility("default")))
/* Client calls: `sock` is the agent's Unix socket path (NULL = $UMS_AGENT_SOCK, else the default). They return 0, a
 * positive ums_agent_status from the agent, or -1 when the agent cannot be reached. */
UMS_AGENT_EXPORT int ums_agent_put(const char* sock, uint64_t token_id, const void* value, uint32_t len);
UMS_AGENT_EXPORT int ums_agent_del(const char* sock, uint64_t token_id);
UMS_AGENT_EXPORT int ums_agent_get(const char* sock, const char* peer, uint64_t token_id, void* value, uint32_t* len);
UMS_AGENT_EXPORT int ums_agent_stats(const char* sock, char* text, uint32_t cap);

#ifdef __cplusplus
}
#endif
