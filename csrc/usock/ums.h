/* UMS: stream sockets whose payload travels through shared-memory ring buffers instead of the TCP stack, with a
 * TCP connection kept for the handshake, for readiness notification (so poll/select/epoll keep working on the file
 * descriptor) and as the transparent fallback when the peer does not speak UMS.
 * User-space counterpart of the reference's kernel module (src/usock/ums/kmod/ums: CLC handshake over TCP then a
 * ring-buffer data path with producer/consumer cursors, io/ums_cdc.h:34-83; fallback to TCP when negotiation is
 * declined, ums_mod.c:269-432) and of its LD_PRELOAD shim (src/usock/ums/tools/ums-preload.c:77-100). */
#ifndef UMDK_UMS_H
#define UMDK_UMS_H
#include <stddef.h>
#include <stdint.h>
#include <sys/socket.h>
#include <sys/types.h>
#ifdef __cplusplus
extern "C" {
#endif
#define UMS_EXPORT __attribute__((visibility("default")))

UMS_EXPORT int ums_socket(int domain, int type, int protocol);
UMS_EXPORT int ums_bind(int fd, const struct sockaddr* addr, socklen_t len);
UMS_EXPORT int ums_listen(int fd, int backlog);
UMS_EXPORT int ums_accept(int fd, struct sockaddr* addr, socklen_t* len);
UMS_EXPORT int ums_connect(int fd, const struct sockaddr* addr, socklen_t len);
UMS_EXPORT ssize_t ums_send(int fd, const void* buf, size_t n, int flags);
UMS_EXPORT ssize_t ums_recv(int fd, void* buf, size_t n, int flags);
UMS_EXPORT int ums_shutdown(int fd, int how);
UMS_EXPORT int ums_close(int fd);
/* 1 if the connection uses the shared-memory data path, 0 if it fell back to TCP, -1 if fd is unknown */
UMS_EXPORT int ums_is_accelerated(int fd);

typedef struct ums_stats {
  uint64_t conns_ums, conns_fallback, bytes_tx_ring, bytes_rx_ring, bytes_tx_tcp, bytes_rx_tcp, doorbells, tx_waits;
  uint64_t conns_auth_fail; /* handshakes refused because the peer's message did not verify under UMS_PSK */
  /* link groups: connections between the same two processes share link files of 32 slots each */
  uint64_t links_created, links_freed, links_active, conns_on_links;
  uint64_t llc_tx, llc_rx, link_tests_ok; /* control messages on the links' LLC rings */
  /* receive moderation: the busy-poll budget before sleeping adapts to how often polling pays off */
  uint64_t dim_up, dim_down;
} ums_stats_t;
UMS_EXPORT void ums_get_stats(ums_stats_t* out);
/* used by the preload shim */
UMS_EXPORT int ums_adopt_listener(int fd);                 /* after a real listen() */
UMS_EXPORT int ums_adopt_accepted(int listen_fd, int fd);  /* after a real accept(): server-side handshake */
UMS_EXPORT int ums_adopt_connected(int fd, const struct sockaddr* peer); /* after a real connect() */
UMS_EXPORT int ums_owns(int fd);
/* Link-layer test of the connection's link: sends TEST LINK on the control ring and waits for the peer's UMS layer to
 * answer (the peer answers from inside its next UMS call on any connection of that link; a peer blocked in recv is
 * woken). 0 = answered, -1 = no answer within timeout_ms or fd is not on a link. */
UMS_EXPORT int ums_link_test(int fd, int timeout_ms);
/* Where a connection lives: link file name (empty for a connection with a file of its own), slot, the link's
 * connection count and the receive side's current moderation level (0 = never busy-poll .. 4). */
typedef struct ums_conn_info {
  char link[64];
  uint32_t slot, link_conns, link_state, dim_level;
} ums_conn_info_t;
UMS_EXPORT int ums_conn_info(int fd, ums_conn_info_t* out);
#ifdef __cplusplus
}
#endif
#endif
