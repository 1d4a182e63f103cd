// dlock_example: exercises the distributed lock service end to end inside one process (server + client threads) and
// prints lock-operation latency / throughput (--clients N: N clients in parallel, each on its own lock). With
// --selftest it also checks mutual exclusion, reader/writer semantics, FIFO order of the fair lock, lease expiry, atomic objects and recovery after a server restart.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <thread>
#include <vector>

#include "dlock_api.h"
#include "ub_util.h"

static int fail(const char* w) {
  fprintf(stderr, "dlock_example: FAILED: %s\n", w);
  return 1;
}
#define CHECK(cond, what) \
  do {                    \
    if (!(cond)) return fail(what); \
  } while (0)

static dlock_lock_desc_t desc(const char* name, dlock_type_t t) {
  dlock_lock_desc_t d{};
  snprintf(d.name, sizeof(d.name), "%s", name);
  d.type = t;
  return d;
}

int main(int argc, char** argv) {
  bool selftest = false;
  int iters = 20000, nclients = 0;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--selftest")) selftest = true;
    else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--clients") && i + 1 < argc) nclients = atoi(argv[++i]);
  }
  dlock_server_cfg_t sc{};
  int sid;
  uint16_t port;
  CHECK(dlock_server_start(&sc, &sid, &port) == DLOCK_SUCCESS, "server start");
  int c1, c2, c3;
  CHECK(dlock_client_init(&c1, "127.0.0.1", port) == DLOCK_SUCCESS, "client 1");
  CHECK(dlock_client_init(&c2, "127.0.0.1", port) == DLOCK_SUCCESS, "client 2");
  CHECK(dlock_client_init(&c3, "127.0.0.1", port) == DLOCK_SUCCESS, "client 3");

  // --- latency / throughput of lock + unlock
  dlock_lock_desc_t d = desc("bench", DLOCK_ATOMIC);
  int32_t lb;
  CHECK(dlock_get_lock(c1, &d, &lb) == DLOCK_SUCCESS, "get_lock");
  dlock_lock_req_t rq{lb, DLOCK_LOCK_EXCLUSIVE, 5000};
  uint64_t t0 = ub::now_ns();
  for (int i = 0; i < iters; ++i) {
    CHECK(dlock_trylock(c1, &rq) == DLOCK_SUCCESS, "bench trylock");
    CHECK(dlock_unlock(c1, lb) == DLOCK_SUCCESS, "bench unlock");
  }
  double sec = (ub::now_ns() - t0) * 1e-9;
  printf("lock+unlock: %.1f us per operation, %.0f lock ops/s (one client)\n", sec / (2.0 * iters) * 1e6,
         2.0 * iters / sec);
  int32_t ob;
  CHECK(dlock_umo_atomic64_create(c1, "bench-obj", 0, &ob) == DLOCK_SUCCESS, "object create");
  t0 = ub::now_ns();
  uint64_t old;
  for (int i = 0; i < iters; ++i) CHECK(dlock_umo_atomic64_faa(c1, ob, 1, &old) == DLOCK_SUCCESS, "faa");
  sec = (ub::now_ns() - t0) * 1e-9;
  printf("object fetch-add: %.1f us end to end, %.0f ops/s\n", sec / iters * 1e6, iters / sec);

  if (nclients > 0) {
    // aggregate rate: every client (own connection, own thread) works on a lock of its own, as the clients of a
    // cluster that partition their data do; the server's one command thread serves them all
    std::vector<int> cl(nclients);
    std::vector<int32_t> ids(nclients);
    for (int k = 0; k < nclients; ++k) {
      CHECK(dlock_client_init(&cl[k], "127.0.0.1", port) == DLOCK_SUCCESS, "client init (--clients)");
      char nm[32];
      snprintf(nm, sizeof(nm), "part-%d", k);
      dlock_lock_desc_t dk = desc(nm, DLOCK_ATOMIC);
      CHECK(dlock_get_lock(cl[k], &dk, &ids[k]) == DLOCK_SUCCESS, "get_lock (--clients)");
    }
    std::atomic<int> go{0}, failed{0};
    std::vector<std::thread> th;
    for (int k = 0; k < nclients; ++k)
      th.emplace_back([&, k] {
        dlock_lock_req_t r{ids[k], DLOCK_LOCK_EXCLUSIVE, 5000};
        while (!go.load()) sched_yield();
        for (int i = 0; i < iters; ++i)
          if (dlock_trylock(cl[k], &r) != DLOCK_SUCCESS || dlock_unlock(cl[k], ids[k]) != DLOCK_SUCCESS) {
            ++failed;
            return;
          }
      });
    t0 = ub::now_ns();
    go = 1;
    for (auto& t : th) t.join();
    sec = (ub::now_ns() - t0) * 1e-9;
    CHECK(failed.load() == 0, "lock operations of the parallel clients");
    printf("%d clients: %.0f lock ops/s in total, %.1f us per operation seen by a client\n", nclients,
           2.0 * iters * nclients / sec, sec / (2.0 * iters) * 1e6);
    for (int k = 0; k < nclients; ++k) dlock_client_deinit(cl[k]);
  }

  if (selftest) {
    // mutual exclusion: three clients increment a plain counter under the lock
    dlock_lock_desc_t dm = desc("mutex", DLOCK_ATOMIC);
    int32_t m1, m2, m3;
    CHECK(dlock_get_lock(c1, &dm, &m1) == 0 && dlock_get_lock(c2, &dm, &m2) == 0 && dlock_get_lock(c3, &dm, &m3) == 0,
          "shared lock ids");
    CHECK(m1 == m2 && m2 == m3, "same name must map to the same lock");
    volatile long counter = 0;
    std::atomic<int> inside{0}, violations{0};
    auto worker = [&](int cli, int32_t id) {
      dlock_lock_req_t r{id, DLOCK_LOCK_EXCLUSIVE, 5000};
      for (int i = 0; i < 300; ++i) {
        if (dlock_lock(cli, &r, 10000) != DLOCK_SUCCESS) {
          ++violations;
          return;
        }
        if (inside.fetch_add(1) != 0) ++violations;
        counter = counter + 1;
        inside.fetch_sub(1);
        dlock_unlock(cli, id);
      }
    };
    std::thread ta(worker, c1, m1), tb(worker, c2, m2), tc(worker, c3, m3);
    ta.join();
    tb.join();
    tc.join();
    CHECK(violations.load() == 0 && counter == 900, "mutual exclusion");
    // reader / writer
    dlock_lock_desc_t dr = desc("rw", DLOCK_RW);
    int32_t r1, r2, r3;
    dlock_get_lock(c1, &dr, &r1);
    dlock_get_lock(c2, &dr, &r2);
    dlock_get_lock(c3, &dr, &r3);
    dlock_lock_req_t sh1{r1, DLOCK_LOCK_SHARED, 5000}, sh2{r2, DLOCK_LOCK_SHARED, 5000}, ex3{r3, DLOCK_LOCK_EXCLUSIVE, 5000};
    CHECK(dlock_trylock(c1, &sh1) == DLOCK_SUCCESS && dlock_trylock(c2, &sh2) == DLOCK_SUCCESS, "two readers");
    CHECK(dlock_trylock(c3, &ex3) == DLOCK_EAGAIN, "writer must wait for readers");
    dlock_unlock(c1, r1);
    dlock_unlock(c2, r2);
    CHECK(dlock_trylock(c3, &ex3) == DLOCK_SUCCESS, "writer after readers left");
    CHECK(dlock_trylock(c1, &sh1) == DLOCK_EAGAIN, "reader must wait for the writer");
    CHECK(dlock_unlock(c1, r1) == DLOCK_NOT_OWNER, "unlock by a non-owner");
    dlock_unlock(c3, r3);
    // fair lock: queued clients are served in arrival order
    dlock_lock_desc_t df = desc("fair", DLOCK_FAIR);
    int32_t f1, f2, f3;
    dlock_get_lock(c1, &df, &f1);
    dlock_get_lock(c2, &df, &f2);
    dlock_get_lock(c3, &df, &f3);
    dlock_lock_req_t q1{f1, DLOCK_LOCK_EXCLUSIVE, 5000}, q2{f2, DLOCK_LOCK_EXCLUSIVE, 5000}, q3{f3, DLOCK_LOCK_EXCLUSIVE, 5000};
    CHECK(dlock_trylock(c1, &q1) == DLOCK_SUCCESS, "fair: first");
    CHECK(dlock_trylock(c3, &q3) == DLOCK_EAGAIN, "fair: c3 queues first");
    CHECK(dlock_trylock(c2, &q2) == DLOCK_EAGAIN, "fair: c2 queues second");
    dlock_unlock(c1, f1);
    CHECK(dlock_trylock(c2, &q2) == DLOCK_EAGAIN, "fair: c2 must not overtake c3");
    CHECK(dlock_trylock(c3, &q3) == DLOCK_SUCCESS, "fair: c3 served first");
    dlock_unlock(c3, f3);
    CHECK(dlock_trylock(c2, &q2) == DLOCK_SUCCESS, "fair: c2 served next");
    dlock_unlock(c2, f2);
    // lease expiry: an abandoned lock can be taken over
    dlock_lock_req_t shortl{m1, DLOCK_LOCK_EXCLUSIVE, 100};
    CHECK(dlock_trylock(c1, &shortl) == DLOCK_SUCCESS, "short lease");
    dlock_lock_req_t other{m2, DLOCK_LOCK_EXCLUSIVE, 5000};
    CHECK(dlock_trylock(c2, &other) == DLOCK_EAGAIN, "held before expiry");
    usleep(150000);
    CHECK(dlock_trylock(c2, &other) == DLOCK_SUCCESS, "takeover after expiry");
    CHECK(dlock_lock_extend(c2, m2, 5000) == DLOCK_SUCCESS, "extend");
    dlock_unlock(c2, m2);
    // atomic objects: concurrent fetch-add is exact, compare-and-swap has one winner
    int32_t o1, o2;
    CHECK(dlock_umo_atomic64_create(c1, "cnt", 5, &o1) == DLOCK_SUCCESS, "obj create");
    CHECK(dlock_umo_atomic64_get(c2, "cnt", &o2) == DLOCK_SUCCESS && o1 == o2, "obj get");
    std::thread fa([&] { uint64_t o; for (int i = 0; i < 2000; ++i) dlock_umo_atomic64_faa(c1, o1, 1, &o); });
    std::thread fb([&] { uint64_t o; for (int i = 0; i < 2000; ++i) dlock_umo_atomic64_faa(c2, o2, 2, &o); });
    fa.join();
    fb.join();
    uint64_t v;
    CHECK(dlock_umo_atomic64_get_snapshot(c3, o1, &v) == DLOCK_SUCCESS && v == 5 + 2000 + 4000, "object sum");
    uint64_t oa, obb;
    dlock_umo_atomic64_cas(c1, o1, v, 1, &oa);
    dlock_umo_atomic64_cas(c2, o1, v, 2, &obb);
    CHECK((oa == v) != (obb == v), "exactly one compare-and-swap wins");
    // batch API
    dlock_lock_desc_t bd[3] = {desc("b0", DLOCK_ATOMIC), desc("b1", DLOCK_ATOMIC), desc("b2", DLOCK_RW)};
    int32_t bid[3];
    CHECK(dlock_batch_get_lock(c1, 3, bd, bid) == DLOCK_SUCCESS, "batch get");
    dlock_lock_req_t br[3] = {{bid[0], DLOCK_LOCK_EXCLUSIVE, 5000}, {bid[1], DLOCK_LOCK_EXCLUSIVE, 5000}, {bid[2], DLOCK_LOCK_SHARED, 5000}};
    int res[3];
    CHECK(dlock_batch_trylock(c1, 3, br, res) == DLOCK_SUCCESS, "batch trylock");
    CHECK(dlock_batch_unlock(c1, 3, bid, res) == DLOCK_SUCCESS, "batch unlock");
    CHECK(dlock_batch_get_lock(c1, 32, bd, bid) == DLOCK_EINVAL, "batch limit");
    CHECK(dlock_client_heartbeat(c1, 1000) == DLOCK_SUCCESS, "heartbeat");
    // recovery: c1 holds "mutex"; the server is replaced; clients re-register and push their lock state
    dlock_lock_req_t hold{m1, DLOCK_LOCK_EXCLUSIVE, 60000};
    CHECK(dlock_trylock(c1, &hold) == DLOCK_SUCCESS, "hold before restart");
    dlock_server_stop(sid);
    CHECK(dlock_trylock(c2, &other) == DLOCK_BAD_RESPONSE, "a dead server must be reported");
    dlock_server_cfg_t sc2{};
    sc2.port = port;
    sc2.recovery_client_num = 2;
    sc2.recovery_timeout_ms = 5000;
    CHECK(dlock_server_start(&sc2, &sid, &port) == DLOCK_SUCCESS, "server restart");
    CHECK(dlock_client_reinit(c1, "127.0.0.1", port) == DLOCK_SUCCESS, "reinit c1");
    CHECK(dlock_update_all_locks(c1) == DLOCK_SUCCESS, "update_all_locks c1");
    // only one of the two expected clients is back: lock operations are refused as not ready
    dlock_lock_desc_t dm2 = desc("mutex", DLOCK_ATOMIC);
    CHECK(dlock_client_reinit(c2, "127.0.0.1", port) == DLOCK_SUCCESS, "reinit c2");
    CHECK(dlock_update_all_locks(c2) == DLOCK_SUCCESS, "update_all_locks c2");
    int32_t nm2;
    CHECK(dlock_get_lock(c2, &dm2, &nm2) == DLOCK_SUCCESS, "get_lock after recovery");
    dlock_lock_req_t after{nm2, DLOCK_LOCK_EXCLUSIVE, 5000};
    CHECK(dlock_trylock(c2, &after) == DLOCK_EAGAIN, "lock held before the restart is still held by c1");
    dlock_debug_stats_t ss;
    dlock_get_server_debug_stats(sid, &ss);
    CHECK(ss.recovered_locks >= 1, "server recovered lock state from clients");
    int32_t nm1;
    CHECK(dlock_get_lock(c1, &dm2, &nm1) == DLOCK_SUCCESS && dlock_unlock(c1, nm1) == DLOCK_SUCCESS, "owner unlocks");
    CHECK(dlock_trylock(c2, &after) == DLOCK_SUCCESS, "free after the owner unlocked");
    dlock_client_reinit(c3, "127.0.0.1", port);
  }
  dlock_client_deinit(c1);
  dlock_client_deinit(c2);
  dlock_client_deinit(c3);
  dlock_server_stop(sid);
  printf("dlock_example: OK\n");
  return 0;
}
