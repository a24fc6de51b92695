// Load-balancing policies of the global proxy and their shared state.
//
// One policy object per upstream pool.  State lives in a block that can be placed in process-shared memory
// (mmap MAP_SHARED), guarded by a spin lock, so several worker processes see the same counters - the role of the
// nginx shared-memory zones in the reference.  Policies (reference modules under
// omni/accelerators/sched/global_proxy/lb_sdk/modules/):
//   pd_score_balance (prefill | decode)   ngx_http_upstream_pd_score_balance_module.c:365-542
//   prefill_score_balance                 ngx_http_upstream_prefill_score_balance_module.c:140-263
//   weighted_least_active                 ngx_http_upstream_weighted_least_active_module.c:293-388
//   length_balance                        ngx_http_upstream_length_balance_module.c:294-406
//   greedy_timeout                        ngx_http_upstream_greedy_timeout_module.c:241-301
//   auto_balance_controller               ngx_http_upstream_auto_balance_controller_module.c:107-297
//   least_total_load                      ngx_http_upstream_least_total_load_module.c:169-
//   round_robin                           (nginx default)
// "Length" is the request body length in bytes, as in the reference; token counters come from the response
// stream filters.
#pragma once
#include <atomic>
#include <cstdint>
#include <string>
#include <vector>

namespace omni_proxy {

constexpr int MAX_PEERS = 512;
constexpr int MAX_ACTIVE_PREFILL = 4096;

struct PeerState {
  int64_t active_requests;
  int64_t total_request_length;   // sum of lengths of in-flight requests
  double total_time_cost;         // pd_score: outstanding prefill cost ; prefill_score: sum of cost*...
  int64_t total_decode_num;       // decoded tokens of in-flight requests (stream filter)
  int64_t total_tokens;           // prompt + output tokens of in-flight requests (weighted_least_active)
  double available_time;          // greedy_timeout: time at which the peer becomes free (seconds)
  double length_score;            // length_balance accumulated score
  int64_t served;                 // completed requests
  int64_t failures;               // consecutive connect failures
  double down_until;              // ejected until this time (monotonic seconds); 0 = healthy
};

struct LbShared {
  std::atomic<int> lock;
  int n_peers;
  int rr_next;
  PeerState peers[MAX_PEERS];
  int n_active_prefill;                       // pd_score decode strategy: lengths of requests currently in prefill
  int64_t active_prefill_len[MAX_ACTIVE_PREFILL];
};

struct LbParams {
  std::string policy = "round_robin";
  int decode_req_limit = 0;        // pd_score decode: max active requests per peer (0 = unlimited)
  int batch_size = 25;             // auto_balance_controller / least_total_load
  double req_len_weight = 1.0;     // length_balance
  double decay_factor = 0.9;       // length_balance
  double warmup = 5.0, exponent = 1.8;  // greedy_timeout: cost = warmup + len^exponent (ms)
  double fail_timeout_s = 10.0;    // peer ejection
  int max_fails = 1;
};

struct Ticket {   // what get_peer hands out and free_peer takes back
  int peer = -1;
  int64_t length = 0;
  double cost = 0;
  int64_t decoded = 0, tokens = 0;
};

class LoadBalancer {
 public:
  // `shm` must point to zero-initialised memory of sizeof(LbShared) (heap or shared mapping)
  LoadBalancer(LbShared* shm, int n_peers, LbParams params);
  static double prefill_time_cost(int64_t len) { return (double)(len / 4) * 0.0345 + 120.0745; }

  Ticket get_peer(int64_t request_length, double now_s);
  void free_peer(const Ticket& t, bool failed, double now_s);
  // stream filters
  void on_decoded_tokens(Ticket& t, int64_t total_decoded);          // pd_score: "total_tokens" in SSE chunks
  void on_token_counts(Ticket& t, int64_t prompt, int64_t output);   // weighted_least_active
  // pd_score decode strategy needs the prefill lengths that are in flight
  void prefill_started(int64_t len);
  void prefill_finished(int64_t len);
  void mark_failed(int peer, double now_s);
  bool is_up(int peer, double now_s) const;       // takes the lock: callable from the metrics thread
  PeerState peer(int i) const;                    // a snapshot taken under the lock
  int n_peers() const { return s_->n_peers; }
  const LbParams& params() const { return p_; }

 private:
  int pick(int64_t len, double now_s, Ticket& t);
  bool up_locked(int i, double now_s) const { return s_->peers[i].down_until <= now_s; }
  void lock() const;
  void unlock() const;
  LbShared* s_;
  LbParams p_;
};

}  // namespace omni_proxy
