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
} ums_stats_t;
UMS_EXPORT void ums_get_stats(ums_stats_t* out);
/* used by the preload shim */
UMS_EXPORT int ums_adopt_listener(int fd);                 /* after a real listen() */
UMS_EXPORT int ums_adopt_accepted(int listen_fd, int fd);  /* after a real accept(): server-side handshake */
UMS_EXPORT int ums_adopt_connected(int fd, const struct sockaddr* peer); /* after a real connect() */
UMS_EXPORT int ums_owns(int fd);
#ifdef __cplusplus
}
#endif
#endif
