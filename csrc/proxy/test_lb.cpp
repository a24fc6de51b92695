// Unit tests of the load-balancing formulas and the JSON surgery (no sockets).
#include <cstdio>
#include <cstring>

#include "json_min.h"
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

int main() {
  int rc = test_json() | test_policies();
  printf("%s (%d checks)\n", rc ? "FAILED" : "ALL PASSED", g_checks);
  return rc;
}
