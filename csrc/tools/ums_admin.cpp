// ums_admin: shows the accelerated listeners and connections of the user-space UMS sockets on this host.
//
//   ums_admin show [directory]      default directory: $UMS_SHM_DIR or /dev/shm/ums_<uid>
//   ums_admin agent [socket]        counters of the token agent (default socket: $UMS_AGENT_SOCK)
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

#include "ums_agent_proto.h"
#include "ums_shm.h"

// Prints the agent's one-line report as one counter per line.
static int show_agent(const char* sock) {
  char text[UMS_AGENT_MAX_VALUE + 1];
  const int rc = ums_agent_stats(sock, text, sizeof(text));
  if (rc != 0) {
    fprintf(stderr, "ums_admin: the agent does not answer (%d)\n", rc);
    return 1;
  }
  static const char* const names[][2] = {
      {"tok", "tokens stored"},          {"put", "tokens published"},       {"del", "tokens removed"},
      {"get", "local lookups"},          {"fwd", "lookups sent to a peer"}, {"srv", "lookups served to peers"},
      {"miss", "unknown token ids"},     {"perr", "peer failures"},         {"tls", "TLS accepted/refused"},
      {"pool", "pool open/dials/reuses"}};
  char* save = nullptr;
  for (char* k = strtok_r(text, " ", &save); k; k = strtok_r(nullptr, " ", &save)) {
    const char* v = strtok_r(nullptr, " ", &save);
    if (!v) break;
    const char* label = k;
    for (auto& n : names)
      if (!strcmp(n[0], k)) label = n[1];
    printf("%-26s %s\n", label, v);
  }
  return 0;
}

int main(int argc, char** argv) {
  if (argc >= 2 && !strcmp(argv[1], "agent")) return show_agent(argc >= 3 ? argv[2] : nullptr);
  if (argc < 2 || strcmp(argv[1], "show") != 0) {
    fprintf(stderr, "usage: ums_admin show [directory] | ums_admin agent [socket]\n");
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
  int listeners = 0, conns = 0, links = 0;
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
    if (name.rfind("lg_", 0) == 0) {   // a link: up to 32 connections in one file plus the control rings
      if (stat(path.c_str(), &st) != 0 || (size_t)st.st_size != sizeof(ums_shm::LinkShm)) continue;
      const int lfd = open(path.c_str(), O_RDONLY);
      if (lfd < 0) continue;
      void* lp = mmap(nullptr, sizeof(ums_shm::LinkShm), PROT_READ, MAP_SHARED, lfd, 0);
      close(lfd);
      if (lp == MAP_FAILED) continue;
      const ums_shm::LinkShm* lk = static_cast<const ums_shm::LinkShm*>(lp);
      static const char* const states[] = {"created", "active", "deleted"};
      const uint32_t used = lk->slot_used.load(), done = lk->closed_c.load() & lk->closed_s.load();
      const uint32_t state = lk->state.load();
      printf("link %s  group %.63s  state %s  client pid %u  server pid %u  connections carried %u\n", name.c_str(),
             lk->group, states[state < 3 ? state : 0], lk->owner_pid, lk->peer_pid.load(), lk->conns_total.load());
      printf("  control ring client->server %llu/%llu  server->client %llu/%llu (produced/consumed)\n",
             (unsigned long long)lk->llc_c2s.prod.load(), (unsigned long long)lk->llc_c2s.cons.load(),
             (unsigned long long)lk->llc_s2c.prod.load(), (unsigned long long)lk->llc_s2c.cons.load());
      for (uint32_t i = 0; i < ums_shm::kLinkSlots; ++i) {
        if (!(used & (1u << i)) || (done & (1u << i))) continue;
        const ums_shm::Ring* rings[2] = {&lk->conn[i].c2s, &lk->conn[i].s2c};
        const char* label[2] = {"client->server", "server->client"};
        printf("connection %s slot %u\n", name.c_str(), i);
        for (int k = 0; k < 2; ++k) {
          const unsigned long long prod = rings[k]->prod.load(), cons = rings[k]->cons.load();
          printf("  %s  produced %llu  consumed %llu  in flight %llu  %s\n", label[k], prod, cons, prod - cons,
                 rings[k]->closed.load() ? "closed" : "open");
        }
        ++conns;
      }
      munmap(lp, sizeof(ums_shm::LinkShm));
      ++links;
      continue;
    }
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
  printf("%d listener(s), %d connection(s), %d link(s) in %s\n", listeners, conns, links, dir.c_str());
  return 0;
}
