// ums_admin: shows the accelerated listeners and connections of the user-space UMS sockets on this host.
//
//   ums_admin show [directory]      default directory: $UMS_SHM_DIR or /dev/shm/ums_<uid>
//
// Every accelerated listener leaves a marker file and every accelerated connection one shared-memory file with two
// byte rings; the tool maps the rings read-only and prints, per direction, the bytes produced and consumed so far, what
// is in flight, and whether the producer has shut down. Counterpart of the reference's ums_admin, which reads the same
// kind of state from the kernel module (src/usock/ums/tools/ums_admin/ums_admin.c).
#include <dirent.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>

#include "ums_shm.h"

int main(int argc, char** argv) {
  if (argc < 2 || strcmp(argv[1], "show") != 0) {
    fprintf(stderr, "usage: ums_admin show [directory]\n");
    return 2;
  }
  std::string dir;
  if (argc >= 3) dir = argv[2];
  else if (const char* e = getenv("UMS_SHM_DIR")) dir = e;
  else dir = "/dev/shm/ums_" + std::to_string(getuid());
  DIR* d = opendir(dir.c_str());
  if (!d) {
    printf("no UMS state in %s\n", dir.c_str());
    return 0;
  }
  int listeners = 0, conns = 0;
  while (dirent* e = readdir(d)) {
    const std::string name = e->d_name;
    if (name == "." || name == "..") continue;
    if (name.rfind("listen_", 0) == 0) {
      printf("listener  port %s\n", name.c_str() + 7);
      ++listeners;
      continue;
    }
    const std::string path = dir + "/" + name;
    struct stat st;
    if (stat(path.c_str(), &st) != 0 || (size_t)st.st_size < sizeof(ums_shm::ConnShm)) continue;
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) continue;
    void* p = mmap(nullptr, sizeof(ums_shm::ConnShm), PROT_READ, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) continue;
    const ums_shm::ConnShm* c = static_cast<const ums_shm::ConnShm*>(p);
    const ums_shm::Ring* rings[2] = {&c->c2s, &c->s2c};
    const char* label[2] = {"client->server", "server->client"};
    printf("connection %s\n", name.c_str());
    for (int i = 0; i < 2; ++i) {
      const unsigned long long prod = rings[i]->prod.load(), cons = rings[i]->cons.load();
      printf("  %s  produced %llu  consumed %llu  in flight %llu  %s\n", label[i], prod, cons, prod - cons,
             rings[i]->closed.load() ? "closed" : "open");
    }
    munmap(p, sizeof(ums_shm::ConnShm));
    ++conns;
  }
  closedir(d);
  printf("%d listener(s), %d connection(s) in %s\n", listeners, conns, dir.c_str());
  return 0;
}
