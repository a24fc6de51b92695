#include "lb.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <thread>

namespace omni_proxy {

LoadBalancer::LoadBalancer(LbShared* shm, int n_peers, LbParams params) : s_(shm), p_(std::move(params)) {
  if (s_->n_peers == 0) s_->n_peers = std::min(n_peers, MAX_PEERS);
}

void LoadBalancer::lock() const {
  int expected = 0;
  while (!s_->lock.compare_exchange_weak(expected, 1, std::memory_order_acquire)) {
    expected = 0;
    std::this_thread::yield();
  }
}
void LoadBalancer::unlock() const { s_->lock.store(0, std::memory_order_release); }

bool LoadBalancer::is_up(int i, double now) const {
  lock();
  const bool up = up_locked(i, now);
  unlock();
  return up;
}

PeerState LoadBalancer::peer(int i) const {
  lock();
  PeerState copy = s_->peers[i];
  unlock();
  return copy;
}

void LoadBalancer::mark_failed(int peer, double now) {
  lock();
  PeerState& ps = s_->peers[peer];
  if (++ps.failures >= p_.max_fails) ps.down_until = now + p_.fail_timeout_s;   // ejected; re-admitted after the timeout
  unlock();
}

int LoadBalancer::pick(int64_t len, double now, Ticket& t) {
  const int n = s_->n_peers;
  std::vector<int> up;
  for (int i = 0; i < n; ++i) if (up_locked(i, now)) up.push_back(i);
  if (up.empty()) for (int i = 0; i < n; ++i) up.push_back(i);   // everything is down: try anyway
  // ties go to the peer after the one that won the last tie (not always to the first): a lightly loaded pool, where
  // every peer scores the same most of the time, then spreads its requests instead of sending them all to peer 0
  auto argmin = [&](auto score) {
    const int m = (int)up.size();
    const int start = s_->rr_next % m;
    int best = up[start];
    double bs = score(best);
    bool tie = false;
    for (int k = 1; k < m; ++k) {
      const int i = up[(start + k) % m];
      const double v = score(i);
      if (v < bs) { bs = v; best = i; tie = false; }
      else if (v == bs) tie = true;
    }
    if (tie) s_->rr_next = (s_->rr_next + 1) % std::max(1, n);
    return best;
  };
  const std::string& pol = p_.policy;
  PeerState* P = s_->peers;
  if (pol == "pd_score_balance_prefill") {
    // min(outstanding cost + this request's length)
    return argmin([&](int i) { return P[i].total_time_cost + (double)len; });
  }
  if (pol == "pd_score_balance_decode") {
    // LPT simulation: requests still in prefill (plus this one), longest first, each to the least loaded decode
    // peer; the peer that receives *this* request is the answer.
    std::vector<int64_t> lens(s_->active_prefill_len, s_->active_prefill_len + s_->n_active_prefill);
    lens.push_back(len);
    std::sort(lens.begin(), lens.end(), [](int64_t a, int64_t b) { return a > b; });
    std::vector<double> load(n);
    for (int i = 0; i < n; ++i) load[i] = (double)P[i].total_decode_num * 4.0;
    std::vector<int64_t> act(n);
    for (int i = 0; i < n; ++i) act[i] = P[i].active_requests;
    int chosen = up[0];
    for (int64_t l : lens) {
      int best = -1;
      for (int i : up) {
        if (p_.decode_req_limit > 0 && act[i] > p_.decode_req_limit) continue;
        if (best < 0 || load[i] < load[best]) best = i;
      }
      if (best < 0) { best = up[0]; for (int i : up) if (load[i] < load[best]) best = i; }
      load[best] += (double)l;
      act[best] += 1;
      chosen = best;
      if (l == len) break;     // this request's turn
    }
    return chosen;
  }
  if (pol == "prefill_score_balance") {
    // increase of sum(cost * active) when the request joins a peer
    const double c = prefill_time_cost(len);
    t.cost = c;
    return argmin([&](int i) { return (P[i].total_time_cost + c) * (double)(P[i].active_requests + 1) - P[i].total_time_cost * (double)P[i].active_requests; });
  }
  if (pol == "weighted_least_active") {
    int best = up[0];
    for (int i : up)
      if (P[i].active_requests < P[best].active_requests ||
          (P[i].active_requests == P[best].active_requests && P[i].total_tokens < P[best].total_tokens)) best = i;
    return best;
  }
  if (pol == "length_balance") {
    // score = requests + accumulated length score + this request's weighted length; random tie-break
    int best = -1; double bs = 0; int ties = 0;
    for (int i : up) {
      double v = (double)P[i].active_requests + P[i].length_score + (double)len * p_.req_len_weight / 1024.0;
      if (best < 0 || v < bs - 1e-12) { best = i; bs = v; ties = 1; }
      else if (std::fabs(v - bs) <= 1e-12 && (rand() % ++ties) == 0) best = i;
    }
    return best;
  }
  if (pol == "greedy_timeout") {
    t.cost = (p_.warmup + std::pow((double)len, p_.exponent)) / 1000.0;
    return argmin([&](int i) { return std::max(P[i].available_time, now); });
  }
  if (pol == "auto_balance_controller") {
    bool below = true;
    for (int i : up) if (P[i].active_requests >= p_.batch_size) below = false;
    if (below) return argmin([&](int i) { return (double)P[i].total_request_length; });
    return argmin([&](int i) { return (double)P[i].active_requests; });
  }
  if (pol == "least_total_load") {
    const int bsz = std::max(1, p_.batch_size);
    return argmin([&](int i) {
      const double reqs = (double)(P[i].active_requests + 1);
      return (double)(P[i].total_request_length + len) * (std::ceil(reqs / bsz) + 1.0) / 2.0;
    });
  }
  // round robin over healthy peers
  int pick = up[s_->rr_next % (int)up.size()];
  s_->rr_next = (s_->rr_next + 1) % std::max(1, n);
  return pick;
}

Ticket LoadBalancer::get_peer(int64_t len, double now) {
  Ticket t;
  t.length = len;
  lock();
  t.peer = pick(len, now, t);
  PeerState& ps = s_->peers[t.peer];
  ps.active_requests += 1;
  ps.total_request_length += len;
  if (p_.policy == "pd_score_balance_prefill") ps.total_time_cost += (double)len;
  if (p_.policy == "prefill_score_balance") ps.total_time_cost += t.cost;
  if (p_.policy == "greedy_timeout") ps.available_time = std::max(ps.available_time, now) + t.cost;
  if (p_.policy == "length_balance") ps.length_score = ps.length_score * p_.decay_factor + (double)len * p_.req_len_weight / 1024.0;
  unlock();
  return t;
}

void LoadBalancer::free_peer(const Ticket& t, bool failed, double now) {
  if (t.peer < 0) return;
  lock();
  PeerState& ps = s_->peers[t.peer];
  ps.active_requests = std::max<int64_t>(0, ps.active_requests - 1);
  ps.total_request_length = std::max<int64_t>(0, ps.total_request_length - t.length);
  if (p_.policy == "pd_score_balance_prefill") ps.total_time_cost = std::max(0.0, ps.total_time_cost - (double)t.length);
  if (p_.policy == "prefill_score_balance") ps.total_time_cost = std::max(0.0, ps.total_time_cost - t.cost);
  ps.total_decode_num = std::max<int64_t>(0, ps.total_decode_num - t.decoded);
  ps.total_tokens = std::max<int64_t>(0, ps.total_tokens - t.tokens);
  if (failed) {
    if (++ps.failures >= p_.max_fails) ps.down_until = now + p_.fail_timeout_s;
  } else {
    ps.failures = 0;
    ps.served += 1;
  }
  unlock();
}

void LoadBalancer::on_decoded_tokens(Ticket& t, int64_t total) {
  if (t.peer < 0 || total <= t.decoded) return;
  lock();
  s_->peers[t.peer].total_decode_num += total - t.decoded;
  unlock();
  t.decoded = total;
}

void LoadBalancer::on_token_counts(Ticket& t, int64_t prompt, int64_t output) {
  if (t.peer < 0) return;
  const int64_t tot = prompt + output;
  if (tot <= t.tokens) return;
  lock();
  s_->peers[t.peer].total_tokens += tot - t.tokens;
  unlock();
  t.tokens = tot;
}

void LoadBalancer::prefill_started(int64_t len) {
  lock();
  if (s_->n_active_prefill < MAX_ACTIVE_PREFILL) s_->active_prefill_len[s_->n_active_prefill++] = len;
  unlock();
}

void LoadBalancer::prefill_finished(int64_t len) {
  lock();
  for (int i = 0; i < s_->n_active_prefill; ++i)
    if (s_->active_prefill_len[i] == len) {
      s_->active_prefill_len[i] = s_->active_prefill_len[--s_->n_active_prefill];
      break;
    }
  unlock();
}

}  // namespace omni_proxy
