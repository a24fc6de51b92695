// Unit tests of the static ExpertLoadBalancer's snapshot planner (placement_static.cpp): analysis helpers, the
// instruction semantics, the per-layer plan under a communication limit, wave priorities, the multi-layer entry, and
// a randomised property test (every prefix of a plan leaves a valid placement; an accepted plan lowers the ratio).
// Scenarios follow the reference's cpp/test/test_expert_load_balancer.cpp and test_placement_optimizer.cpp.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <random>
#include <stdexcept>

#include "placement_core.h"

using namespace omni_placement;

static int g_checks = 0;
#define CHECK(cond) do { ++g_checks; if (!(cond)) { fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); return 1; } } while (0)
#define THROWS(stmt) do { bool t_ = false; try { stmt; } catch (const std::exception&) { t_ = true; } CHECK(t_); } while (0)

static ChangeInstruction ins_of(OperationType t, int slots, int sp, int se, int tp, int te) {
  ChangeInstruction i;
  i.type = t;
  i.source_rank = sp / slots; i.source_expert_id = se; i.source_global_position = sp;
  i.target_rank = tp / slots; i.target_expert_id = te; i.target_global_position = tp;
  return i;
}

// 4 ranks x 3 slots (2 home + 1 redundant), 8 experts
static const int W = 4, S = 3, E = 8;
static const std::vector<int> kBase = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};

static int test_analysis() {
  ExpertLoadBalancer b(W, E, S, 2);
  CHECK(b.positions() == 12);
  std::vector<int> pl = {0, 1, 2, 2, 3, -1, 4, 5, 0, 6, 7, -1};     // experts 0 and 2 have two replicas
  std::vector<int64_t> act = {30, 10, 5, 15, 40, 0, 10, 10, 50, 20, 20, 0};
  auto loads = b.expert_loads(pl, act);
  CHECK(loads[0] == 80 && loads[2] == 20 && loads[3] == 40 && loads[7] == 20);
  auto cnt = b.replica_counts(pl);
  CHECK(cnt[0] == 2 && cnt[2] == 2 && cnt[1] == 1);
  auto rl = b.simulated_rank_loads(pl, loads);
  CHECK(std::fabs(rl[0] - (40 + 10 + 10)) < 1e-9);    // half of expert 0, expert 1, half of expert 2
  CHECK(std::fabs(rl[1] - (10 + 40)) < 1e-9);
  CHECK(std::fabs(rl[2] - (10 + 10 + 40)) < 1e-9);
  CHECK(std::fabs(rl[3] - 40) < 1e-9);
  CHECK(std::fabs(b.simulated_ratio(pl, loads) - 60.0 / (210.0 / 4)) < 1e-9);
  CHECK(std::fabs(b.measured_ratio(pl, act) - 70.0 / (210.0 / 4)) < 1e-9);   // rank 2 measured 10+10+50
  CHECK(b.find_position(pl, 0, 2) == 2 && b.find_position(pl, 1, 2) == 3 && b.find_position(pl, 3, 2) == -1);
  CHECK(b.find_empty(pl, 0) == -1 && b.find_empty(pl, 1) == 5 && b.find_empty(pl, 3) == 11);
  CHECK(b.validate_counts(pl, 2, 3) && !b.validate_counts(pl, 3, 3) && !b.validate_counts(pl, 1, 2));
  CHECK(!b.validate_counts({0, 1}, 0, 3));
  CHECK(b.diff_count(kBase, kBase) == 0);
  CHECK(b.diff_count(kBase, pl) == 2);                        // rank 0 fetches expert 2, rank 2 fetches expert 0
  std::vector<int> sw = kBase;
  std::swap(sw[0], sw[3]);
  CHECK(b.diff_count(kBase, sw) == 4);                        // two ranks each drop one and fetch one
  // all-zero loads: the ratio is defined as 1
  CHECK(b.simulated_ratio(kBase, std::vector<double>(E, 0.0)) == 1.0);
  CHECK(b.measured_ratio(kBase, std::vector<int64_t>(12, 0)) == 1.0);
  THROWS(b.expert_loads({0, 1}, {1, 2}));
  std::vector<int> bad = kBase;
  bad[0] = 99;
  THROWS(b.expert_loads(bad, act));
  return 0;
}

static int test_apply() {
  ExpertLoadBalancer b(W, E, S, 2);
  std::vector<int> pl = kBase;
  // REMOVE of the only replica is refused, placement untouched
  CHECK(!b.apply(pl, ins_of(OperationType::REMOVE, S, 0, 0, 0, -1)) && pl == kBase);
  // ADD expert 0 (rank 0) onto the empty slot of rank 2
  CHECK(b.apply(pl, ins_of(OperationType::ADD, S, 0, 0, 8, -1)) && pl[8] == 0);
  // again onto the same rank: refused
  CHECK(!b.apply(pl, ins_of(OperationType::ADD, S, 0, 0, 6, 4)));
  // wrong expectation of what the target holds: refused
  CHECK(!b.apply(pl, ins_of(OperationType::ADD, S, 0, 0, 5, 3)));
  // ADD that would evict the only replica of expert 2: refused
  CHECK(!b.apply(pl, ins_of(OperationType::ADD, S, 0, 0, 3, 2)));
  // now a replica can be removed, from either holder
  CHECK(b.apply(pl, ins_of(OperationType::REMOVE, S, 0, 0, 0, -1)) && pl[0] == -1 && pl[8] == 0);
  CHECK(!b.apply(pl, ins_of(OperationType::REMOVE, S, 8, 0, 8, -1)));   // it is the last one again
  // SWAP
  pl = kBase;
  CHECK(b.apply(pl, ins_of(OperationType::SWAP, S, 0, 0, 3, 2)) && pl[0] == 2 && pl[3] == 0);
  CHECK(!b.apply(pl, ins_of(OperationType::SWAP, S, 0, 0, 3, 2)));      // stale expert ids
  CHECK(!b.apply(pl, ins_of(OperationType::SWAP, S, 0, 2, 1, 1)));      // same rank
  CHECK(!b.apply(pl, ins_of(OperationType::SWAP, S, 0, 2, 5, -1)));     // empty target
  // a swap that would double an expert on a rank
  std::vector<int> dup = {0, 1, 2, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  CHECK(!b.apply(dup, ins_of(OperationType::SWAP, S, 0, 0, 3, 2)));      // rank 0 would hold expert 2 twice
  // out-of-range positions
  CHECK(!b.apply(pl, ins_of(OperationType::SWAP, S, 0, 2, 40, 2)));
  CHECK(!b.apply(pl, ins_of(OperationType::REMOVE, S, -1, 2, -1, -1)));
  ChangeInstruction none;
  CHECK(b.apply(pl, none));                                              // EMPTY does nothing
  return 0;
}

static bool prefixes_valid(const ExpertLoadBalancer& b, const std::vector<int>& start, const LayerPlan& plan) {
  std::vector<int> cur = start;
  for (const auto& i : plan.instructions) {
    if (!b.apply(cur, i)) return false;
    if (!b.validate(cur)) return false;
  }
  return cur == plan.placement;
}

static int test_plan_hot_expert() {
  ExpertLoadBalancer b(W, E, S, 2);
  std::vector<int64_t> act = {900, 50, 0, 60, 40, 0, 50, 50, 0, 45, 55, 0};
  StaticBalanceOptions opt;
  auto plan = b.plan_layer(3, kBase, act, opt);
  CHECK(plan.accepted && plan.layer == 3);
  CHECK(plan.ratio_before > 2.5 && plan.ratio_after < plan.ratio_before - 0.1);
  CHECK(!plan.instructions.empty() && (int)plan.instructions.size() <= 2 * W);
  CHECK(plan.instructions[0].type == OperationType::ADD && plan.instructions[0].source_expert_id == 0);
  CHECK(plan.instructions[0].layer_idx == 3);
  CHECK(prefixes_valid(b, kBase, plan));
  CHECK(std::count(plan.placement.begin(), plan.placement.end(), 0) >= 3);   // the hot expert got replicas
  const auto loads = b.expert_loads(kBase, act);
  CHECK(std::fabs(b.simulated_ratio(plan.placement, loads) - plan.ratio_after) < 1e-9);
  // the communication limit cuts the list
  opt.diff_limit = 1;
  auto p1 = b.plan_layer(0, kBase, act, opt);
  CHECK(p1.accepted && p1.instructions.size() == 1 && p1.considered > 1);
  CHECK(p1.ratio_after > plan.ratio_after - 1e-12);      // fewer moves cannot do better than the longer plan's best prefix
  opt.diff_limit = 0;
  auto p0 = b.plan_layer(0, kBase, act, opt);
  CHECK(!p0.accepted && p0.instructions.empty() && p0.placement == kBase && p0.ratio_after == p0.ratio_before);
  // no replica allowed: the plan may only swap
  opt.diff_limit = -1;
  opt.max_redundant_per_expert = 0;
  auto ps = b.plan_layer(0, kBase, act, opt);
  for (const auto& i : ps.instructions) CHECK(i.type == OperationType::SWAP);
  for (int e = 0; e < E; ++e) CHECK(std::count(ps.placement.begin(), ps.placement.end(), e) == 1);
  // a margin that the gain cannot reach: rejected, input returned
  opt.max_redundant_per_expert = 10;
  opt.accept_margin = 100.0;
  auto pr = b.plan_layer(0, kBase, act, opt);
  CHECK(!pr.accepted && pr.instructions.empty() && pr.placement == kBase && pr.considered > 0);
  return 0;
}

static int test_plan_balanced_and_zero() {
  ExpertLoadBalancer b(W, E, S, 2);
  StaticBalanceOptions opt;
  std::vector<int64_t> flat = {50, 50, 0, 50, 50, 0, 50, 50, 0, 50, 50, 0};
  auto p = b.plan_layer(0, kBase, flat, opt);
  CHECK(!p.accepted && p.instructions.empty() && std::fabs(p.ratio_before - 1.0) < 1e-12);
  auto z = b.plan_layer(0, kBase, std::vector<int64_t>(12, 0), opt);
  CHECK(!z.accepted && z.instructions.empty() && z.considered == 0);
  // invalid inputs
  std::vector<int> missing = kBase;
  missing[0] = 1;                                         // expert 0 has no replica (and 1 sits twice on rank 0)
  THROWS(b.plan_layer(0, missing, flat, opt));
  THROWS(b.plan_layer(0, {0, 1, 2}, {1, 1, 1}, opt));
  return 0;
}

static int test_plan_without_redundant_slots() {
  // 4 ranks x 2 slots, no spare slot: swaps only (the reference's bucket-balance mode)
  ExpertLoadBalancer b(4, 8, 2, 8);
  std::vector<int> pl = {0, 1, 2, 3, 4, 5, 6, 7};
  std::vector<int64_t> act = {100, 90, 10, 20, 30, 40, 5, 5};
  StaticBalanceOptions opt;
  auto p = b.plan_layer(0, pl, act, opt);
  CHECK(p.accepted && !p.instructions.empty());
  for (const auto& i : p.instructions) CHECK(i.type == OperationType::SWAP);
  CHECK(prefixes_valid(b, pl, p));
  CHECK(p.ratio_before > 2.4 && p.ratio_after < 1.4 + 1e-9);   // 1.4 is the optimum: {100, 5} on one rank
  auto sorted = p.placement;
  std::sort(sorted.begin(), sorted.end());
  CHECK(sorted == pl);                                    // a permutation of the input
  return 0;
}

static int test_plan_surplus_replica() {
  // the cold expert 7 holds the spare slot of rank 0 while expert 0 is hot: the replica goes, a hot one comes
  ExpertLoadBalancer b(W, E, S, 2);
  std::vector<int> pl = {0, 1, 7, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {800, 40, 1, 40, 40, 0, 40, 40, 0, 40, 1, 0};
  StaticBalanceOptions opt;
  opt.max_redundant_per_expert = 2;
  auto p = b.plan_layer(0, pl, act, opt);
  CHECK(p.accepted && prefixes_valid(b, pl, p));
  bool removed7 = false, added0 = false;
  for (const auto& i : p.instructions) {
    if (i.type == OperationType::REMOVE && i.source_expert_id == 7) removed7 = true;
    if (i.type == OperationType::ADD && i.source_expert_id == 0) added0 = true;
  }
  CHECK(removed7 && added0);
  CHECK(std::count(p.placement.begin(), p.placement.end(), 7) == 1);
  CHECK(std::count(p.placement.begin(), p.placement.end(), 0) == 3);       // 1 + max_redundant_per_expert
  return 0;
}

static int test_same_host_source() {
  // 4 ranks, 2 per host.  Expert 0 lives on rank 0 (host 0) and rank 2 (host 1); the next replica lands on rank 3
  // (the lightest rank with room), so the copy should come from rank 2, the holder on rank 3's host
  ExpertLoadBalancer b(4, 8, 3, 2);
  std::vector<int> pl = {0, 1, 6, 2, 3, 7, 4, 5, 0, 6, 7, -1};
  std::vector<int64_t> act = {600, 30, 30, 60, 60, 30, 30, 30, 600, 10, 10, 0};
  StaticBalanceOptions opt;
  auto p = b.plan_layer(0, pl, act, opt);
  CHECK(p.accepted && !p.instructions.empty());
  const ChangeInstruction* add = nullptr;
  for (const auto& i : p.instructions) if (i.type == OperationType::ADD && i.source_expert_id == 0 && !add) add = &i;
  CHECK(add != nullptr);
  CHECK(add->target_rank == 3 && add->source_rank == 2);
  return 0;
}

static int test_priorities() {
  std::vector<ChangeInstruction> v;
  auto mk = [&](int layer, OperationType t, int sp, int se, int tp, int te) {
    auto i = ins_of(t, S, sp, se, tp, te);
    i.layer_idx = layer;
    v.push_back(i);
  };
  mk(1, OperationType::ADD, 0, 0, 5, -1);      // layer 1: wave 1
  mk(0, OperationType::ADD, 0, 0, 5, -1);      // layer 0: wave 1
  mk(0, OperationType::ADD, 0, 0, 8, -1);      // same expert again: wave 2
  mk(0, OperationType::SWAP, 3, 2, 9, 6);      // independent: wave 1
  mk(0, OperationType::REMOVE, 5, 0, 5, -1);   // same expert and same position as the first: wave 3
  mk(0, OperationType::SWAP, 4, 3, 9, 2);      // position 9 and expert 2 were touched in wave 1: wave 2
  ExpertLoadBalancer::assign_priorities(v);
  CHECK(v.size() == 6);
  for (size_t i = 1; i < v.size(); ++i)
    CHECK(v[i - 1].layer_idx < v[i].layer_idx || (v[i - 1].layer_idx == v[i].layer_idx && v[i - 1].prior <= v[i].prior));
  CHECK(v[0].layer_idx == 0 && v[0].prior == 1 && v[1].prior == 1);
  CHECK(v[2].prior == 2 && v[3].prior == 2 && v[4].prior == 3 && v[4].type == OperationType::REMOVE);
  CHECK(v[5].layer_idx == 1 && v[5].prior == 1);
  // instructions of one wave never share an expert or a position
  for (size_t i = 0; i < v.size(); ++i)
    for (size_t j = i + 1; j < v.size(); ++j) {
      if (v[i].layer_idx != v[j].layer_idx || v[i].prior != v[j].prior) continue;
      CHECK(v[i].source_global_position != v[j].source_global_position);
      CHECK(v[i].target_global_position != v[j].target_global_position);
      CHECK(v[i].source_expert_id != v[j].source_expert_id);
    }
  std::vector<ChangeInstruction> none;
  ExpertLoadBalancer::assign_priorities(none);
  CHECK(none.empty());
  return 0;
}

static int test_multi_layer() {
  ExpertLoadBalancer b(W, E, S, 2);
  StaticBalanceOptions opt;
  std::vector<int> pl;
  std::vector<int64_t> act;
  for (int l = 0; l < 3; ++l) pl.insert(pl.end(), kBase.begin(), kBase.end());
  const std::vector<int64_t> hot = {900, 50, 0, 60, 40, 0, 50, 50, 0, 45, 55, 0};
  const std::vector<int64_t> flat = {50, 50, 0, 50, 50, 0, 50, 50, 0, 50, 50, 0};
  act.insert(act.end(), hot.begin(), hot.end());
  act.insert(act.end(), flat.begin(), flat.end());
  act.insert(act.end(), hot.rbegin(), hot.rend());         // layer 2: the hot expert is 7 (positions reversed)
  std::vector<LayerPlan> plans;
  auto ins = b.optimize_and_generate_instructions(3, pl, act, opt, &plans);
  CHECK(plans.size() == 3 && plans[0].accepted && !plans[1].accepted && plans[2].accepted);
  CHECK(ins.size() == plans[0].instructions.size() + plans[2].instructions.size());
  for (const auto& i : ins) CHECK(i.layer_idx != 1 && i.prior >= 1);
  for (size_t i = 1; i < ins.size(); ++i) CHECK(ins[i - 1].layer_idx <= ins[i].layer_idx);
  bool add7 = false;
  for (const auto& i : plans[2].instructions) if (i.type == OperationType::ADD && i.source_expert_id == 7) add7 = true;
  CHECK(add7);
  // replaying the whole list layer by layer gives the planned placements
  std::vector<std::vector<int>> cur(3, kBase);
  for (const auto& i : ins) CHECK(b.apply(cur[i.layer_idx], i));
  for (int l = 0; l < 3; ++l) CHECK(cur[l] == plans[l].placement);
  // shape errors
  THROWS(b.optimize_and_generate_instructions(2, pl, act, opt));
  THROWS(b.optimize_and_generate_instructions(0, {}, {}, opt));
  act.pop_back();
  THROWS(b.optimize_and_generate_instructions(3, pl, act, opt));
  return 0;
}

static int test_random_properties() {
  std::mt19937 rng(1234);
  int accepted = 0;
  for (int trial = 0; trial < 300; ++trial) {
    const int world = 2 + (int)(rng() % 7);                    // 2..8
    const int per = 1 + (int)(rng() % 4);
    const int red = (int)(rng() % 3);
    const int slots = per + red, experts = world * per;
    ExpertLoadBalancer b(world, experts, slots, 1 + (int)(rng() % 4));
    // a valid start: the base layout, then a few random replicas in the spare slots
    std::vector<int> pl(world * slots, -1);
    for (int r = 0; r < world; ++r)
      for (int k = 0; k < per; ++k) pl[r * slots + k] = r * per + k;
    for (int r = 0; r < world; ++r)
      for (int k = per; k < slots; ++k)
        if (rng() % 2) {
          const int e = (int)(rng() % experts);
          if (b.find_position(pl, r, e) < 0) pl[r * slots + k] = e;
        }
    if (!b.validate(pl)) { fprintf(stderr, "generator made an invalid start\n"); return 1; }
    std::vector<int64_t> act(pl.size(), 0);
    const bool skew = rng() % 2;
    for (size_t p = 0; p < pl.size(); ++p)
      if (pl[p] >= 0) act[p] = skew && pl[p] % 5 == 0 ? 500 + rng() % 500 : rng() % 100;
    StaticBalanceOptions opt;
    opt.max_redundant_per_expert = (int)(rng() % 4);
    opt.diff_limit = rng() % 3 == 0 ? (int)(rng() % 5) : -1;
    opt.accept_margin = (rng() % 3) * 0.05;
    const auto plan = b.plan_layer(trial, pl, act, opt);
    const int limit = opt.diff_limit >= 0 ? opt.diff_limit : 2 * world;
    CHECK((int)plan.instructions.size() <= limit);
    CHECK(prefixes_valid(b, pl, plan));
    CHECK(b.validate_counts(plan.placement, 1, slots));
    if (plan.accepted) {
      ++accepted;
      CHECK(plan.ratio_after < plan.ratio_before - opt.accept_margin);
      const auto loads = b.expert_loads(pl, act);
      CHECK(std::fabs(b.simulated_ratio(plan.placement, loads) - plan.ratio_after) < 1e-9);
      // an ADD never takes an expert past its replica limit (replicas beyond it can only come from the input)
      const auto before = b.replica_counts(pl), after = b.replica_counts(plan.placement);
      for (int e = 0; e < experts; ++e) CHECK(after[e] <= std::max(before[e], 1 + opt.max_redundant_per_expert));
    } else {
      CHECK(plan.instructions.empty() && plan.placement == pl);
    }
    for (const auto& i : plan.instructions) CHECK(i.layer_idx == trial);
  }
  CHECK(accepted > 50);   // the generator does produce cases worth planning for
  return 0;
}

int main() {
  int rc = 0;
  rc |= test_analysis();
  rc |= test_apply();
  rc |= test_plan_hot_expert();
  rc |= test_plan_balanced_and_zero();
  rc |= test_plan_without_redundant_slots();
  rc |= test_plan_surplus_replica();
  rc |= test_same_host_source();
  rc |= test_priorities();
  rc |= test_multi_layer();
  rc |= test_random_properties();
  printf("%s (%d checks)\n", rc ? "FAILED" : "ALL PASSED", g_checks);
  return rc;
}
