// urpc_admin: asks a running URPC process for its state over the management socket.
//
//   urpc_admin <socket path> <command>      command: version | stats | perf | channels | sessions | funcs
//
// The process serves the socket when URPC_ADMIN_SOCKET names a path at urpc_init time or after urpc_admin_start().
// Counterpart of the reference's urpc_admin, which reads stats, channel / queue / handshaker dumps and the version
// from the framework's unix-domain control socket (src/urpc/tools/urpc_admin/**).
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

int main(int argc, char** argv) {
  if (argc < 3) {
    fprintf(stderr, "usage: urpc_admin <socket path> version|stats|perf|channels|sessions|funcs\n");
    return 2;
  }
  const int fd = socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  snprintf(a.sun_path, sizeof(a.sun_path), "%s", argv[1]);
  if (fd < 0 || connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) != 0) {
    fprintf(stderr, "urpc_admin: cannot connect to %s\n", argv[1]);
    return 1;
  }
  if (write(fd, argv[2], strlen(argv[2])) < 0) return 1;
  shutdown(fd, SHUT_WR);
  char buf[4096];
  ssize_t n;
  while ((n = read(fd, buf, sizeof(buf))) > 0) fwrite(buf, 1, n, stdout);
  close(fd);
  return 0;
}
