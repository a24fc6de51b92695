// Concurrency test of the balancer state (meant for a ThreadSanitizer build): worker threads hand out and take back
// tickets, feed the stream-filter counters and eject peers while a reader samples the counters, for every policy.
// At the end every in-flight counter is back at zero and every request was counted once.  A second part shares the
// state between a parent and forked children through a MAP_SHARED mapping, as the proxy's worker processes do.
#include <sys/mman.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "lb.h"

using namespace omni_proxy;

static int g_checks = 0;
#define CHECK(cond) do { ++g_checks; if (!(cond)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } } while (0)

static int stress(const std::string& policy) {
  const int PEERS = 5, THREADS = 8, ITERS = 1500;
  std::unique_ptr<LbShared> shm(new LbShared());
  memset((void*)shm.get(), 0, sizeof(LbShared));
  LbParams p;
  p.policy = policy;
  p.fail_timeout_s = 0.001;
  p.decode_req_limit = 4;
  LoadBalancer lb(shm.get(), PEERS, p);
  std::atomic<bool> stop{false};
  std::atomic<long> failed_total{0};
  std::vector<std::thread> ts;
  for (int t = 0; t < THREADS; ++t)
    ts.emplace_back([&, t] {
      unsigned seed = 17u * (unsigned)t + 3u;
      auto rnd = [&] { seed = seed * 1664525u + 1013904223u; return seed >> 8; };
      for (int i = 0; i < ITERS; ++i) {
        const int64_t len = 64 + (int64_t)(rnd() % 4000);
        const double now = 1.0 + i * 1e-4;
        lb.prefill_started(len);
        Ticket tk = lb.get_peer(len, now);
        lb.on_decoded_tokens(tk, 1 + (int64_t)(rnd() % 50));
        lb.on_token_counts(tk, len / 4, (int64_t)(rnd() % 30));
        lb.on_decoded_tokens(tk, tk.decoded + 5);
        const bool failed = rnd() % 50 == 0;
        if (failed) ++failed_total;
        if (rnd() % 200 == 0) lb.mark_failed((int)(rnd() % PEERS), now);
        lb.prefill_finished(len);
        lb.free_peer(tk, failed, now);
      }
    });
  std::thread reader([&] {   // what the metrics endpoint does while requests are in flight
    long sink = 0;
    while (!stop.load()) {
      for (int i = 0; i < PEERS; ++i) sink += (lb.is_up(i, 2.0) ? 1 : 0) + lb.peer(i).active_requests;
      std::this_thread::yield();
    }
    if (sink < 0) printf("%ld\n", sink);
  });
  for (auto& t : ts) t.join();
  stop = true;
  reader.join();
  int64_t served = 0;
  for (int i = 0; i < PEERS; ++i) {
    const PeerState ps = lb.peer(i);
    CHECK(ps.active_requests == 0 && ps.total_request_length == 0 && ps.total_decode_num == 0 && ps.total_tokens == 0);
    if (policy == "pd_score_balance_prefill" || policy == "prefill_score_balance") CHECK(ps.total_time_cost < 1e-6);
    served += ps.served;
  }
  CHECK(served == (int64_t)THREADS * ITERS - failed_total.load());
  CHECK(shm->n_active_prefill == 0);
  return 0;
}

static int forked() {
  void* mem = mmap(nullptr, sizeof(LbShared), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
  CHECK(mem != MAP_FAILED);
  memset(mem, 0, sizeof(LbShared));
  LbParams p;
  p.policy = "weighted_least_active";
  const int PEERS = 3, KIDS = 4, ITERS = 2000;
  LoadBalancer lb((LbShared*)mem, PEERS, p);
  std::vector<pid_t> kids;
  for (int k = 0; k < KIDS; ++k) {
    pid_t pid = fork();
    CHECK(pid >= 0);
    if (pid == 0) {
      LoadBalancer mine((LbShared*)mem, PEERS, p);
      for (int i = 0; i < ITERS; ++i) {
        Ticket t = mine.get_peer(100 + i % 7, 1.0);
        mine.on_token_counts(t, 100, i % 5);
        mine.free_peer(t, false, 1.0);
      }
      _exit(0);
    }
    kids.push_back(pid);
  }
  for (pid_t pid : kids) {
    int st = 0;
    CHECK(waitpid(pid, &st, 0) == pid && WIFEXITED(st) && WEXITSTATUS(st) == 0);
  }
  int64_t served = 0;
  for (int i = 0; i < PEERS; ++i) {
    CHECK(lb.peer(i).active_requests == 0 && lb.peer(i).total_tokens == 0);
    served += lb.peer(i).served;
  }
  CHECK(served == (int64_t)KIDS * ITERS);
  munmap(mem, sizeof(LbShared));
  return 0;
}

int main(int argc, char** argv) {
  int rc = 0;
  for (const char* pol : {"pd_score_balance_prefill", "pd_score_balance_decode", "prefill_score_balance", "weighted_least_active",
                          "length_balance", "greedy_timeout", "auto_balance_controller", "least_total_load", "round_robin"})
    rc |= stress(pol);
  if (!(argc > 1 && std::string(argv[1]) == "--no-fork")) rc |= forked();   // TSan does not follow fork()ed children
  printf("%s (%d checks)\n", rc ? "FAILED" : "ALL PASSED", g_checks);
  return rc;
}
