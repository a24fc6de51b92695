// Unit tests of the load-balancing formulas and the JSON surgery (no sockets).
#include <cstdio>
#include <cstring>

#include "json_min.h"
#include <cmath>
#include <cstdlib>

#include "lb.h"

using namespace omni_proxy;
static int g_checks = 0;
#define CHECK(c) do { ++g_checks; if (!(c)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)

#include <memory>
#include <vector>
static std::vector<std::unique_ptr<LbShared>> g_blocks;
static LbShared* fresh() { g_blocks.emplace_back(new LbShared()); memset((void*)g_blocks.back().get(), 0, sizeof(LbShared)); return g_blocks.back().get(); }

static int test_json() {
  std::string b = "{\"model\":\"m\",\"stream\":true,\"stream_options\":{\"include_usage\":true},\"prompt\":\"a \\\"q\\\" {x}\",\"max_tokens\":64}";
  std::string v;
  CHECK(json_get(b, "max_tokens", v) && v == "64");
  CHECK(json_set(b, "max_tokens", "1") && json_set(b, "stream", "false") && json_remove(b, "stream_options"));
  CHECK(json_get(b, "max_tokens", v) && v == "1");
  CHECK(json_get(b, "stream", v) && v == "false");
  CHECK(!json_get(b, "stream_options", v));
  CHECK(json_get(b, "prompt", v) && v == "\"a \\\"q\\\" {x}\"");
  CHECK(json_set(b, "kv_transfer_params", "{\"remote_block_ids\":[1,2],\"x\":\"}\"}"));
  CHECK(json_get(b, "kv_transfer_params", v) && v.find("[1,2]") != std::string::npos);
  std::vector<JsonMember> ms;
  CHECK(json_members(b, ms) && ms.size() == 5);
  std::string e = "{}";
  CHECK(json_set(e, "a", "1") && e == "{\"a\":1}");
  CHECK(!json_members("[1,2]", ms));
  long long n;
  CHECK(find_int_after("data: {\"usage\":{\"total_tokens\": 17}}", "total_tokens", n) && n == 17);
  return 0;
}

static int test_policies() {
  {  // pd_score prefill: min(outstanding + len), accounting undone by free_peer
    LbParams p; p.policy = "pd_score_balance_prefill";
    LoadBalancer lb(fresh(), 3, p);
    Ticket a = lb.get_peer(1000, 0), b = lb.get_peer(10, 0), c = lb.get_peer(10, 0), d = lb.get_peer(10, 0);
    // equal scores go round: a -> 0 (all idle), b -> 1 (1 and 2 tie), c -> 2 (the only idle one), d -> 2 (1 and 2 tie again,
    // the turn has moved on)
    CHECK(a.peer == 0 && b.peer == 1 && c.peer == 2 && d.peer == 2);
    CHECK(lb.peer(0).total_time_cost == 1000 && lb.peer(1).total_time_cost == 10 && lb.peer(2).total_time_cost == 20);
    {  // an idle pool spreads equal requests over all peers instead of sending them to the first
      LoadBalancer idle(fresh(), 4, p);
      int hits[4] = {0, 0, 0, 0};
      for (int i = 0; i < 40; ++i) { Ticket t = idle.get_peer(100, 0); ++hits[t.peer]; idle.free_peer(t, false, 0); }
      CHECK(hits[0] == 10 && hits[1] == 10 && hits[2] == 10 && hits[3] == 10);
    }
    lb.free_peer(a, false, 0);
    CHECK(lb.peer(0).total_time_cost == 0 && lb.peer(0).active_requests == 0 && lb.peer(0).served == 1);
  }
  {  // pd_score decode: LPT over the requests still in prefill
    LbParams p; p.policy = "pd_score_balance_decode"; p.decode_req_limit = 8;
    LoadBalancer lb(fresh(), 2, p);
    Ticket t0 = lb.get_peer(100, 0);
    lb.on_decoded_tokens(t0, 50);                       // peer 0 load = 50 * 4 = 200
    CHECK(lb.peer(0).total_decode_num == 50);
    lb.prefill_started(400);                            // a longer request is still in prefill: it will take peer 1
    Ticket t1 = lb.get_peer(100, 0);                    // lens sorted: 400 -> peer1 (0 < 200), then 100 -> peer0 (200 < 400)
    CHECK(t1.peer == 0);
    lb.prefill_finished(400);
    Ticket t2 = lb.get_peer(100, 0);
    CHECK(t2.peer == 1);
    lb.free_peer(t0, false, 0);
    CHECK(lb.peer(0).total_decode_num == 0);
  }
  {  // prefill_score: cost model and marginal score
    CHECK(LoadBalancer::prefill_time_cost(4000) > 154.57 && LoadBalancer::prefill_time_cost(4000) < 154.58);
    LbParams p; p.policy = "prefill_score_balance";
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(8000, 0), b = lb.get_peer(100, 0), c = lb.get_peer(100, 0);
    CHECK(a.peer == 0 && b.peer == 1 && c.peer == 1);   // adding to the peer with the long request costs more
  }
  {  // weighted_least_active: fewest active, ties by tokens
    LbParams p; p.policy = "weighted_least_active";
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(1, 0), b = lb.get_peer(1, 0);
    CHECK(a.peer == 0 && b.peer == 1);
    lb.on_token_counts(a, 100, 50);
    lb.on_token_counts(b, 10, 5);
    lb.free_peer(a, false, 0);
    lb.free_peer(b, false, 0);
    Ticket c = lb.get_peer(1, 0);
    CHECK(c.peer == 0 && lb.peer(0).total_tokens == 0);
    Ticket d = lb.get_peer(1, 0);
    lb.on_token_counts(d, 10, 10);
    lb.free_peer(c, false, 0);
    Ticket e = lb.get_peer(1, 0);
    CHECK(d.peer == 1 && e.peer == 0);
  }
  {  // greedy_timeout: earliest available peer; cost = warmup + len^1.8 ms
    LbParams p; p.policy = "greedy_timeout";
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(100, 0.0), b = lb.get_peer(10, 0.0), c = lb.get_peer(10, 0.0);
    CHECK(a.peer == 0 && b.peer == 1 && c.peer == 1);
    CHECK(a.cost > b.cost);
  }
  {  // auto_balance_controller: below the batch limit by length, above by active requests
    LbParams p; p.policy = "auto_balance_controller"; p.batch_size = 2;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(1000, 0), b = lb.get_peer(10, 0), c = lb.get_peer(10, 0);
    CHECK(a.peer == 0 && b.peer == 1 && c.peer == 1);
    Ticket d = lb.get_peer(10, 0);                      // peer 1 reached the batch size: fewest active wins
    CHECK(d.peer == 0);
  }
  {  // least_total_load
    LbParams p; p.policy = "least_total_load"; p.batch_size = 2;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(100, 0), b = lb.get_peer(100, 0), c = lb.get_peer(50, 0);
    CHECK(a.peer == 0 && b.peer == 1 && (c.peer == 0 || c.peer == 1));
  }
  {  // length_balance spreads, decays
    LbParams p; p.policy = "length_balance";
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(4096, 0), b = lb.get_peer(10, 0);
    CHECK(a.peer != b.peer);
  }
  {  // ejection and re-admission
    LbParams p; p.policy = "round_robin"; p.fail_timeout_s = 5;
    LoadBalancer lb(fresh(), 2, p);
    lb.mark_failed(0, 100.0);
    CHECK(!lb.is_up(0, 101.0) && lb.is_up(0, 106.0));
    for (int i = 0; i < 4; ++i) { Ticket t = lb.get_peer(1, 101.0); CHECK(t.peer == 1); lb.free_peer(t, false, 101.0); }
    Ticket t = lb.get_peer(1, 106.0);
    Ticket u = lb.get_peer(1, 106.0);
    CHECK(t.peer != u.peer);
  }
  return 0;
}

static int test_policy_edges() {
  {  // accounting never goes below zero, also when a ticket is given back twice or with stale counters
    LbParams p; p.policy = "pd_score_balance_prefill";
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(500, 0);
    lb.free_peer(a, false, 0);
    lb.free_peer(a, false, 0);
    CHECK(lb.peer(a.peer).active_requests == 0 && lb.peer(a.peer).total_request_length == 0 && lb.peer(a.peer).total_time_cost == 0);
    Ticket none;
    lb.free_peer(none, false, 0);                       // a ticket that never got a peer: ignored
    lb.on_decoded_tokens(none, 10);
    lb.on_token_counts(none, 1, 1);
    CHECK(lb.peer(0).total_decode_num == 0 && lb.peer(1).total_tokens == 0);
  }
  {  // stream counters only grow: a chunk that reports less than before changes nothing
    LbParams p; p.policy = "pd_score_balance_decode";
    LoadBalancer lb(fresh(), 1, p);
    Ticket t = lb.get_peer(10, 0);
    lb.on_decoded_tokens(t, 30);
    lb.on_decoded_tokens(t, 20);
    lb.on_decoded_tokens(t, 45);
    CHECK(lb.peer(0).total_decode_num == 45 && t.decoded == 45);
    lb.on_token_counts(t, 100, 5);
    lb.on_token_counts(t, 100, 3);
    CHECK(lb.peer(0).total_tokens == 105);
    lb.free_peer(t, false, 0);
    CHECK(lb.peer(0).total_decode_num == 0 && lb.peer(0).total_tokens == 0 && lb.peer(0).served == 1);
  }
  {  // pd_score decode: a peer over its request limit is passed over; when every peer is over it, the least loaded one serves
    LbParams p; p.policy = "pd_score_balance_decode"; p.decode_req_limit = 1;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(10, 0), b = lb.get_peer(10, 0), c = lb.get_peer(10, 0), d = lb.get_peer(10, 0);
    CHECK(a.peer == 0 && b.peer == 0);                  // up to limit + 1 requests on the first peer with equal load
    CHECK(c.peer == 1 && d.peer == 1);                  // then it is passed over
    lb.on_decoded_tokens(c, 1000);                      // peer 1 is now far heavier
    Ticket e = lb.get_peer(10, 0);                      // both over the limit: the lighter one serves
    CHECK(e.peer == 0);
  }
  {  // the list of requests still in prefill is bounded; finishing an unknown length is harmless
    LbParams p; p.policy = "pd_score_balance_decode";
    LbShared* shm = fresh();
    LoadBalancer lb(shm, 2, p);
    for (int i = 0; i < MAX_ACTIVE_PREFILL + 10; ++i) lb.prefill_started(100 + i);
    CHECK(shm->n_active_prefill == MAX_ACTIVE_PREFILL);
    lb.prefill_finished(99999);
    CHECK(shm->n_active_prefill == MAX_ACTIVE_PREFILL);
    lb.prefill_finished(100);
    CHECK(shm->n_active_prefill == MAX_ACTIVE_PREFILL - 1);
  }
  {  // greedy_timeout: a peer is busy until now + cost; time passing frees it
    LbParams p; p.policy = "greedy_timeout"; p.warmup = 5; p.exponent = 1.0;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(1000, 10.0);                 // busy until 10 + 1.005 s
    CHECK(std::fabs(a.cost - 1.005) < 1e-9 && std::fabs(lb.peer(a.peer).available_time - 11.005) < 1e-9);
    Ticket b = lb.get_peer(1000, 10.0);
    CHECK(b.peer != a.peer);
    Ticket c = lb.get_peer(10, 20.0);                   // both free again by now
    CHECK(std::fabs(lb.peer(c.peer).available_time - 20.015) < 1e-9);
  }
  {  // length_balance: the accumulated score decays with every request a peer takes
    LbParams p; p.policy = "length_balance"; p.decay_factor = 0.5; p.req_len_weight = 1.0;
    LoadBalancer lb(fresh(), 1, p);
    Ticket a = lb.get_peer(2048, 0);
    CHECK(std::fabs(lb.peer(0).length_score - 2.0) < 1e-12);
    lb.free_peer(a, false, 0);
    Ticket b = lb.get_peer(1024, 0);
    CHECK(std::fabs(lb.peer(0).length_score - (2.0 * 0.5 + 1.0)) < 1e-12);
    lb.free_peer(b, false, 0);
  }
  {  // least_total_load: (length sum + this request) * (ceil(requests / batch) + 1) / 2
    LbParams p; p.policy = "least_total_load"; p.batch_size = 2;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(100, 0), b = lb.get_peer(300, 0);        // peer loads 100 / 300, one request each
    Ticket c = lb.get_peer(50, 0);                                   // (100+50)*(1+1)/2 = 150 < (300+50)*(1+1)/2
    CHECK(c.peer == a.peer);
    Ticket d = lb.get_peer(50, 0);                                   // a's peer: (150+50)*(ceil(3/2)+1)/2 = 300; b's: 350*(1+1)/2 = 350
    CHECK(d.peer == a.peer);
    Ticket e = lb.get_peer(50, 0);                                   // a's peer: (200+50)*(2+1)/2 = 375; b's: 350
    CHECK(e.peer == b.peer);
  }
  {  // failures: ejected after max_fails consecutive failures, a success in between resets the count
    LbParams p; p.policy = "round_robin"; p.max_fails = 2; p.fail_timeout_s = 10;
    LoadBalancer lb(fresh(), 2, p);
    Ticket a = lb.get_peer(1, 0);
    lb.free_peer(a, true, 0);
    CHECK(lb.is_up(a.peer, 1.0) && lb.peer(a.peer).failures == 1 && lb.peer(a.peer).served == 0);
    Ticket ok = lb.get_peer(1, 0);
    while (ok.peer != a.peer) { lb.free_peer(ok, false, 0); ok = lb.get_peer(1, 0); }
    lb.free_peer(ok, false, 0);
    CHECK(lb.peer(a.peer).failures == 0);
    lb.mark_failed(a.peer, 5.0);
    lb.mark_failed(a.peer, 5.0);
    CHECK(!lb.is_up(a.peer, 6.0) && lb.is_up(a.peer, 15.1));
    // everything down: requests are still handed out rather than refused
    lb.mark_failed(1 - a.peer, 5.0);
    lb.mark_failed(1 - a.peer, 5.0);
    Ticket t = lb.get_peer(1, 6.0);
    CHECK(t.peer == 0 || t.peer == 1);
  }
  {  // a second balancer object on the same state (another worker process) sees and continues it
    LbParams p; p.policy = "weighted_least_active";
    LbShared* shm = fresh();
    LoadBalancer one(shm, 3, p), two(shm, 99, p);        // the second size is ignored: the state is already sized
    CHECK(two.n_peers() == 3);
    Ticket a = one.get_peer(1, 0), b = two.get_peer(1, 0), c = one.get_peer(1, 0);
    CHECK(a.peer != b.peer && b.peer != c.peer && a.peer != c.peer);
    two.free_peer(a, false, 0);
    CHECK(one.peer(a.peer).active_requests == 0 && one.peer(a.peer).served == 1);
  }
  {  // more peers than the state can hold are cut off, not overrun
    LbParams p;
    LoadBalancer lb(fresh(), MAX_PEERS + 50, p);
    CHECK(lb.n_peers() == MAX_PEERS);
  }
  return 0;
}

int main() {
  int rc = test_json() | test_policies() | test_policy_edges();
  printf("%s (%d checks)\n", rc ? "FAILED" : "ALL PASSED", g_checks);
  return rc;
}
