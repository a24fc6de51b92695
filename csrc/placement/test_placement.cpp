// Unit tests of the placement core with host memcpy hooks and the in-process transport (no GPU, no NCCL).
// Scenarios follow the reference's gtest suites (cpp/test/test_placement_mapping.cpp, test_expert_activation.cpp,
// test_placement_optimizer.cpp, test_expert_load_balancer.cpp, test_moe_weights.cpp, test_distribution.cpp).
#include <cassert>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <numeric>
#include <thread>

#include <sys/mman.h>
#include <unistd.h>

#include "placement_core.h"

using namespace omni_placement;

static int g_checks = 0;
#define CHECK(cond) do { ++g_checks; if (!(cond)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } } while (0)

static int test_mapping() {
  const int W = 4, L = 2, E = 8;
  auto pat = PlacementMapping::base_pattern(W, L, E);
  std::vector<int32_t> sel(L * E, -7);
  PlacementMapping m(pat, W, L, E, /*rank*/1, /*redundant*/1, /*ranks_per_host*/2, sel.data());
  CHECK(m.slots_per_rank() == 3 && m.num_positions() == 12);
  CHECK(m.expert_at(0, 0) == 0 && m.expert_at(0, 1) == 1 && m.expert_at(0, 2) == -1);
  CHECK(m.expert_at(1, 3) == 2 && m.expert_at(1, 9) == 6);
  for (int e = 0; e < E; ++e) CHECK(m.redundant_count(0, e) == 1);
  CHECK(m.selector(0, 5) == 2 * 3 + 1);
  CHECK(sel[5] == 7);                                    // pushed to the "device" selector through the hook
  // add a replica of expert 5 on own rank (rank 1 slot 2 = position 5): selector must prefer it
  CHECK(!m.update_position(0, 5, 3, 5));                 // wrong old expert: refused
  CHECK(m.update_position(0, 5, -1, 5));
  m.update_selector();
  CHECK(m.redundant_count(0, 5) == 2 && m.selector(0, 5) == 5 && sel[5] == 5);
  CHECK(m.local_slots_of(0, 5).size() == 1 && m.local_slots_of(0, 5)[0] == 2);
  // last replica cannot be removed
  CHECK(!m.update_position(0, 0, 0, 3));
  CHECK(m.update_position(0, 5, 5, -1));                 // a redundant one can
  // replica on the same host (rank 0, host 0 = ranks 0,1) beats a distant one
  CHECK(m.update_position(0, 2, -1, 6));                 // rank 0 slot 2 <- expert 6 (home: rank 3)
  m.update_selector();
  CHECK(m.selector(0, 6) == 2);
  // batch: swap experts 0 and 7 between rank 0 and rank 3
  CHECK(m.apply_batch({{1, 0}, {1, 10}}, {7, 0}));
  CHECK(m.expert_at(1, 0) == 7 && m.expert_at(1, 10) == 0);
  CHECK(!m.apply_batch({{1, 0}}, {6}));                  // would orphan expert 7: rolled back
  CHECK(m.expert_at(1, 0) == 7);
  // invalid patterns
  bool threw = false;
  try { auto bad = pat; bad[0] = 0; PlacementMapping x(bad, W, L, E, 0, 0, 8, nullptr); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  // text loader
  {
    std::ofstream f("/tmp/omni_pattern_test.txt");
    f << "2 1 4\n1 1 0 0\n0 0 1 1\n";
  }
  int w, l, e;
  auto tp = PlacementMapping::load_text_pattern("/tmp/omni_pattern_test.txt", w, l, e);
  CHECK(w == 2 && l == 1 && e == 4 && tp.size() == 8 && tp[6] == 1);
  return 0;
}

static int test_activation() {
  const int L = 2, S = 3, W = 2;
  std::vector<int64_t> c0(L * S, 0), c1(L * S, 0);
  auto hub = make_fake_hub(W);
  ClusterActivation a0(Tensor(c0.data(), L * S, 8), L, S, W, 0, 2), a1(Tensor(c1.data(), L * S, 8), L, S, W, 1, 2);
  FakeDistribution d0(hub, 0, 16), d1(hub, 1, 16);
  a0.set_allgather([&](const int64_t* s, int64_t* r, size_t n) { d0.allgather_i64(s, r, n); });
  a1.set_allgather([&](const int64_t* s, int64_t* r, size_t n) { d1.allgather_i64(s, r, n); });
  auto both = [&] { std::thread t([&] { a1.collect(); }); a0.collect(); t.join(); };
  c0[0] = 5; c1[4] = 9;
  both();
  CHECK(a0.delta(0, 0) == 5 && a0.delta(1, 3 + 1) == 9 && a1.delta(0, 0) == 5);
  c0[0] = 12;
  both();
  CHECK(a0.delta(0, 0) == 7 && a0.delta(1, 4) == 0 && a0.windowed(0, 0) == 12);
  c0[0] = 3;                                             // wrapped around 1e16
  both();
  CHECK(a0.delta(0, 0) == ClusterActivation::kWrap - 9);
  CHECK(a0.windowed(1, 4) == 0);                         // window of 2 forgot the first round
  a0.dump_txt("/tmp/omni_act_test.txt");
  ClusterActivation r(Tensor(c0.data(), L * S, 8), L, S, W, 0, 4);
  r.collect_from_txt("/tmp/omni_act_test.txt");
  CHECK(r.delta(0, 0) == a0.delta(0, 0));
  return 0;
}

static int test_balancers() {
  // 4 ranks x 3 slots (2 home + 1 redundant), 8 experts, expert 0 is very hot
  const int W = 4, S = 3, E = 8;
  std::vector<int> place = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {900, 50, 0, 60, 40, 0, 50, 50, 0, 45, 55, 0};
  GreedyExpertLoadBalancer g(1, W, E, S, 10);
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty() && (int)ins.size() <= 32);
  // replay the instructions on a copy and check that the simulated ratio improved
  auto rank_ratio = [&](const std::vector<int>& p, const std::vector<double>& l) {
    std::vector<double> rl(W, 0);
    for (int i = 0; i < W * S; ++i) if (p[i] >= 0) rl[i / S] += l[i];
    return GreedyExpertLoadBalancer::imbalance(rl);
  };
  std::vector<double> load(act.begin(), act.end());
  const double before = rank_ratio(place, load);
  bool saw_add_of_hot = false;
  for (auto& i : ins) {
    CHECK(i.layer_idx == 0);
    if (i.type == OperationType::ADD && i.source_expert_id == 0) saw_add_of_hot = true;
  }
  CHECK(saw_add_of_hot);
  CHECK(before > 5.0);
  // a balanced input produces nothing
  GreedyExpertLoadBalancer g2(1, W, E, S, 10);
  std::vector<int64_t> flat = {50, 50, 0, 50, 50, 0, 50, 50, 0, 50, 50, 0};
  CHECK(g2.optimize_and_generate_instructions(place, flat).empty());
  // EMA: second round blends 0.6 old + 0.4 new
  g2.optimize_and_generate_instructions(place, std::vector<int64_t>(12, 100));
  CHECK(std::abs(g2.ema_loads()[0] - (0.6 * 50 + 0.4 * 100)) < 1e-9);
  // REMOVE: a redundant replica on the hottest rank goes away
  std::vector<int> place3 = {0, 1, 2, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act3 = {300, 300, 100, 100, 50, 0, 50, 50, 0, 50, 50, 0};
  GreedyExpertLoadBalancer g3(1, W, E, S, 10);
  auto ins3 = g3.optimize_and_generate_instructions(place3, act3);
  CHECK(!ins3.empty() && ins3[0].type == OperationType::REMOVE && ins3[0].source_global_position == 2);

  // static placement: hot experts get the replicas, every expert placed, no rank holds an expert twice
  ExpertLoadBalancer sb(W, E, S, 2);
  std::vector<double> loads = {900, 50, 60, 40, 50, 50, 45, 55};
  auto sp = sb.generate_constrained_placement(loads, 10);
  CHECK(sb.validate(sp));
  CHECK(std::count(sp.begin(), sp.end(), 0) >= 3);
  std::vector<double> rl(W, 0);
  std::vector<int> reps(E, 0);
  for (int e : sp) if (e >= 0) ++reps[e];
  for (int i = 0; i < W * S; ++i) if (sp[i] >= 0) rl[i / S] += loads[sp[i]] / reps[sp[i]];
  CHECK(GreedyExpertLoadBalancer::imbalance(rl) < 1.6);
  // bucket balance without redundancy
  ExpertLoadBalancer nb(2, 4, 2, 8);
  auto sw = nb.bucket_balance(0, {0, 1, 2, 3}, {10, 9, 1, 2}, 4);
  CHECK(!sw.empty() && sw[0].type == OperationType::SWAP);
  return 0;
}

// Two "ranks" as threads: full round (collect -> greedy -> handshake -> swap through staging -> apply).
static int run_cluster(bool corrupt, int& applied0, int& skipped0, std::vector<float>& w_rank1_slot2, int& sel_e0_rank1,
                       const char* replica_name = nullptr, int* transfers = nullptr) {
  const int W = 2, L = 1, E = 4, RED = 1;   // 3 slots per rank
  const int S = E / W + RED;
  auto hub = make_fake_hub(W);
  std::vector<std::vector<float>> storage(W, std::vector<float>(S * 8));
  std::vector<std::vector<int64_t>> counts(W, std::vector<int64_t>(L * S, 0));
  std::vector<std::vector<int32_t>> sel(W, std::vector<int32_t>(L * E, -1));
  for (int r = 0; r < W; ++r)
    for (int s = 0; s < S; ++s)
      for (int k = 0; k < 8; ++k) storage[r][s * 8 + k] = (s < E / W) ? float(100 * (r * (E / W) + s) + k) : -1.f;
  counts[0] = {1000, 10, 0};   // expert 0 is hot on rank 0
  counts[1] = {10, 10, 0};
  std::vector<std::unique_ptr<PlacementMapping>> maps;
  std::vector<std::unique_ptr<MoEWeights>> ws;
  std::vector<std::unique_ptr<ClusterActivation>> acts;
  std::vector<std::unique_ptr<FakeDistribution>> dists;
  std::vector<std::unique_ptr<Placement>> pls;
  auto pat = PlacementMapping::base_pattern(W, L, E);
  for (int r = 0; r < W; ++r) {
    maps.emplace_back(new PlacementMapping(pat, W, L, E, r, RED, 8, sel[r].data()));
    ws.emplace_back(new MoEWeights(L, S));
    for (int s = 0; s < S; ++s) ws[r]->add_tensor(0, s, storage[r].data() + s * 8, 8 * sizeof(float));
    ws[r]->set_initialized();
    acts.emplace_back(new ClusterActivation(Tensor(counts[r].data(), L * S, 8), L, S, W, r, 4));
    dists.emplace_back(new FakeDistribution(hub, r, ws[r]->expert_bytes()));
    pls.emplace_back(new Placement(maps[r].get(), ws[r].get(), acts[r].get(), dists[r].get(), 10, 3600.0));
  }
  if (replica_name != nullptr) {
    // both ranks live on one host: they share one replica segment and fill it side by side
    std::thread tr([&] {
      if (!ws[1]->init_shared_memory(replica_name, E, W)) return;
      ws[1]->replicate_to_shared_memory(*maps[1]);
    });
    if (!ws[0]->init_shared_memory(replica_name, E, W)) { tr.join(); return 2; }
    ws[0]->replicate_to_shared_memory(*maps[0]);
    tr.join();
    if (!ws[0]->replica_complete() || !ws[1]->replica_complete()) return 3;
    for (int e = 0; e < E; ++e)
      if (!ws[0]->replica_has(0, e) || !ws[1]->replica_has(0, e)) return 4;
  }
  if (corrupt) dists[1]->corrupt_next_handshake();
  int done[2] = {0, 0};
  std::thread t([&] { done[1] = pls[1]->run_round(); });
  done[0] = pls[0]->run_round();
  t.join();
  pls[0]->do_placement_optimizer();
  pls[1]->do_placement_optimizer();
  applied0 = done[0];
  skipped0 = pls[0]->skipped_instructions();
  w_rank1_slot2.assign(storage[1].begin() + 2 * 8, storage[1].begin() + 3 * 8);
  sel_e0_rank1 = maps[1]->selector(0, 0);
  if (transfers != nullptr) *transfers = dists[0]->transfers() + dists[1]->transfers();
  if (replica_name != nullptr) { ws[1]->close_shared_memory(false); ws[0]->close_shared_memory(true); }
  // both ranks hold the same view of the placement
  for (int p = 0; p < W * S; ++p)
    if (maps[0]->expert_at(0, p) != maps[1]->expert_at(0, p)) return 1;
  return 0;
}

static int test_manager() {
  set_ut_memcpy_fun();
  int applied, skipped, sel;
  std::vector<float> w;
  CHECK(run_cluster(false, applied, skipped, w, sel) == 0);
  CHECK(applied >= 1 && skipped == 0);
  // the hot expert 0 was replicated onto rank 1's free slot (position 5) with its weights, and rank 1 now routes
  // expert 0 to its own replica
  CHECK(w[0] == 0.f && w[3] == 3.f);
  CHECK(sel == 5);
  // a corrupted handshake tuple makes every rank skip the instruction; nothing moves
  CHECK(run_cluster(true, applied, skipped, w, sel) == 0);
  CHECK(skipped >= 1 && w[0] == -1.f && sel == 0);
  return 0;
}

static int test_replica() {
  set_ut_memcpy_fun();
  const std::string name = "/omni_test_replica_" + std::to_string((long)getpid());
  shm_unlink(name.c_str());
  // the same round as test_manager, with the host replica: the expert arrives by a host -> device copy on the rank
  // that wants it, and nothing goes through the transport
  int applied, skipped, sel, transfers = -1;
  std::vector<float> w;
  CHECK(run_cluster(false, applied, skipped, w, sel, name.c_str(), &transfers) == 0);
  CHECK(applied >= 1 && skipped == 0 && transfers == 0);
  CHECK(w[0] == 0.f && w[3] == 3.f && sel == 5);
  int t2 = -1;
  CHECK(run_cluster(false, applied, skipped, w, sel, nullptr, &t2) == 0 && t2 >= 2);   // without it: a send and a receive
  // segment bookkeeping
  MoEWeights a(2, 2), b(2, 2), c(2, 2);
  float buf_a[2][2][4], buf_b[2][2][4];
  for (int l = 0; l < 2; ++l)
    for (int s = 0; s < 2; ++s) {
      for (int k = 0; k < 4; ++k) { buf_a[l][s][k] = float(100 * l + 10 * s + k); buf_b[l][s][k] = -1.f; }
      a.add_tensor(l, s, buf_a[l][s], sizeof(buf_a[l][s]));
      b.add_tensor(l, s, buf_b[l][s], sizeof(buf_b[l][s]));
      c.add_tensor(l, s, buf_b[l][s], sizeof(buf_b[l][s]));
    }
  CHECK(!a.replica_enabled() && !a.replica_has(0, 0) && !a.replace_from_shared_memory(0, 0, 0));
  CHECK(a.init_shared_memory(name, 4, 2));
  CHECK(!a.init_shared_memory(name, 4, 2));                     // already attached
  CHECK(a.replica_enabled() && !a.replica_complete() && a.replica_bytes() >= 2 * 4 * 256);
  CHECK(!c.init_shared_memory(name, 8, 2));                     // same name, another shape: refused
  CHECK(b.init_shared_memory(name, 4, 2));                      // second rank of the host attaches
  auto pat = PlacementMapping::base_pattern(2, 2, 4);
  PlacementMapping m0(pat, 2, 2, 4, 0, 0, 8, nullptr), m1(pat, 2, 2, 4, 1, 0, 8, nullptr);
  a.replicate_to_shared_memory(m0);                             // rank 0 holds experts 0, 1
  CHECK(a.replica_has(1, 1) && b.replica_has(0, 0) && !b.replica_has(0, 2) && !b.replica_complete());
  CHECK(!b.replace_from_shared_memory(0, 2, 0));                // not there yet: nothing is copied
  CHECK(buf_b[0][0][0] == -1.f);
  CHECK(b.replace_from_shared_memory(1, 1, 0));                 // expert 1 of layer 1 into rank 1's slot 0
  CHECK(buf_b[1][0][0] == 110.f && buf_b[1][0][3] == 113.f);
  b.replicate_to_shared_memory(m1);                             // its own (overwritten) slot goes in as expert 2
  CHECK(a.replica_complete() && b.replica_complete() && a.replica_has(0, 3));
  CHECK(!a.replica_has(0, 4) && !a.replica_has(2, 0) && !a.replace_from_shared_memory(0, 0, 5));
  b.close_shared_memory(false);
  CHECK(!b.replica_enabled());
  a.close_shared_memory(true);
  MoEWeights d(2, 2);
  for (int l = 0; l < 2; ++l) for (int s = 0; s < 2; ++s) d.add_tensor(l, s, buf_b[l][s], sizeof(buf_b[l][s]));
  CHECK(d.init_shared_memory(name, 4, 1) && !d.replica_has(0, 0));   // unlinked: a fresh, empty segment
  d.close_shared_memory(true);
  return 0;
}

static int test_weights_tensor() {
  set_ut_memcpy_fun();
  MoEWeights w(2, 2);
  CHECK(w.expert_bytes() == 0 && !w.is_initialized());
  char a[16], b[32];
  w.add_tensor(1, 0, a, 16);
  w.add_tensor(1, 0, b, 32);
  CHECK(w.expert_bytes() == 48 && w.tensors(1, 0).size() == 2 && w.tensors(0, 0).empty());
  int64_t dev[4] = {1, 2, 3, 4}, host[4] = {0, 0, 0, 0};
  Tensor t(dev, 4, 8, "x");
  t.to_host(host);
  CHECK(host[2] == 3 && t.bytes() == 32);
  host[1] = 42;
  t.to_device(host);
  CHECK(dev[1] == 42);
  unset_ut_memcpy_fun();
  bool threw = false;
  try { t.to_host(host); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  set_ut_memcpy_fun();
  return 0;
}

int main() {
  set_ut_memcpy_fun();
  int rc = 0;
  rc |= test_mapping();
  rc |= test_activation();
  rc |= test_balancers();
  rc |= test_weights_tensor();
  rc |= test_manager();
  rc |= test_replica();
  printf("%s (%d checks)\n", rc ? "FAILED" : "ALL PASSED", g_checks);
  return rc;
}
