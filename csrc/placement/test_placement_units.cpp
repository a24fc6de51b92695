// Small single-purpose cases for every unit of the placement core, one function per behaviour (the reference keeps a
// gtest suite per unit: cpp/test/test_placement_mapping.cpp, test_expert_activation.cpp, test_moe_weights.cpp,
// test_tensor.cpp, test_distribution.cpp, test_placement_optimizer.cpp, test_expert_load_balancer.cpp).  Host memcpy
// hooks and the in-process transport stand in for the device and the fabric.  The scenario tests live in
// test_placement.cpp and test_placement_static.cpp.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <chrono>
#include <thread>
#include <vector>

#include <unistd.h>

#include "placement_core.h"

using namespace omni_placement;

namespace {

struct Case { const char* name; std::function<void()> fn; };
std::vector<Case>& cases() { static std::vector<Case> c; return c; }
struct Reg { Reg(const char* n, std::function<void()> f) { cases().push_back({n, std::move(f)}); } };
std::atomic<int> g_checks{0};   // cases check from several threads

struct Failure : std::runtime_error { using std::runtime_error::runtime_error; };
#define CHECK(cond) do { ++g_checks; if (!(cond)) throw Failure(std::string(__FILE__) + ":" + std::to_string(__LINE__) + ": " #cond); } while (0)
#define TEST(name) void name(); Reg reg_##name(#name, name); void name()

template <class F> bool throws(F f) {
  try { f(); } catch (const Failure&) { throw; } catch (const std::exception&) { return true; }
  return false;
}

std::string tmp_path(const char* stem) { return "/tmp/omni_units_" + std::to_string(getpid()) + "_" + stem; }

// a mapping of W ranks x (E/W + red) slots with the base pattern
PlacementMapping base_mapping(int W, int L, int E, int rank, int red, int rph, int32_t* sel = nullptr) {
  return PlacementMapping(PlacementMapping::base_pattern(W, L, E), W, L, E, rank, red, rph, sel);
}

// ================================================================================================ Tensor
TEST(tensor_reports_its_geometry) {
  std::vector<float> buf(6);
  Tensor t(buf.data(), 6, sizeof(float), "w13");
  CHECK(t.data() == buf.data() && t.length() == 6 && t.element_size() == 4 && t.bytes() == 24 && t.name() == "w13");
  Tensor empty;
  CHECK(empty.data() == nullptr && empty.bytes() == 0 && empty.name().empty());
}

TEST(tensor_copies_through_the_hooks) {
  std::vector<int32_t> dev = {1, 2, 3, 4}, host(4, 0);
  Tensor t(dev.data(), 4, 4);
  t.to_host(host.data());
  CHECK(host == dev);
  std::vector<int32_t> src = {9, 8, 7, 6};
  t.to_device(src.data());
  CHECK(dev == src);
}

TEST(tensor_without_hooks_refuses_to_copy) {
  std::vector<int32_t> dev(2), host(2);
  Tensor t(dev.data(), 2, 4);
  unset_ut_memcpy_fun();
  const bool a = throws([&] { t.to_host(host.data()); });
  const bool b = throws([&] { t.to_device(host.data()); });
  set_ut_memcpy_fun();
  CHECK(a && b);
}

TEST(hooks_count_the_bytes_they_move) {
  size_t moved = 0;
  auto saved = hooks();
  hooks().memcpy_d2h = [&](void* d, const void* s, size_t n) { moved += n; std::memcpy(d, s, n); };
  std::vector<int64_t> dev(5, 3), host(5);
  Tensor(dev.data(), 5, 8).to_host(host.data());
  hooks() = saved;
  CHECK(moved == 40 && host[4] == 3);
}

// ================================================================================================ PlacementMapping
TEST(base_pattern_gives_each_rank_its_block) {
  auto p = PlacementMapping::base_pattern(4, 3, 8);
  CHECK(p.size() == 4u * 3 * 8);
  for (int r = 0; r < 4; ++r)
    for (int l = 0; l < 3; ++l)
      for (int e = 0; e < 8; ++e) CHECK(p[(r * 3 + l) * 8 + e] == (e / 2 == r ? 1 : 0));
}

TEST(mapping_geometry_with_redundant_slots) {
  auto m = base_mapping(4, 2, 16, 2, 2, 8);
  CHECK(m.world() == 4 && m.layers() == 2 && m.experts() == 16 && m.rank() == 2);
  CHECK(m.slots_per_rank() == 6 && m.num_positions() == 24);
  // home experts fill the first slots of each rank, redundant slots start empty
  for (int r = 0; r < 4; ++r) {
    for (int s = 0; s < 4; ++s) CHECK(m.expert_at(1, r * 6 + s) == r * 4 + s);
    CHECK(m.expert_at(1, r * 6 + 4) == -1 && m.expert_at(1, r * 6 + 5) == -1);
  }
}

TEST(mapping_rejects_a_pattern_of_the_wrong_size) {
  auto p = PlacementMapping::base_pattern(2, 1, 4);
  p.pop_back();
  CHECK(throws([&] { PlacementMapping m(p, 2, 1, 4, 0, 0, 8, nullptr); }));
}

TEST(mapping_rejects_experts_that_do_not_divide) {
  std::vector<int> p(3 * 1 * 4, 1);
  CHECK(throws([&] { PlacementMapping m(p, 3, 1, 4, 0, 0, 8, nullptr); }));
}

TEST(mapping_rejects_an_orphaned_expert) {
  auto p = PlacementMapping::base_pattern(2, 2, 4);
  p[(1 * 2 + 1) * 4 + 3] = 0;                       // rank 1, layer 1, expert 3
  CHECK(throws([&] { PlacementMapping m(p, 2, 2, 4, 0, 1, 8, nullptr); }));
}

TEST(mapping_rejects_more_experts_than_slots) {
  auto p = PlacementMapping::base_pattern(2, 1, 4);
  p[0 * 4 + 2] = 1;                                 // a third expert on rank 0, which has two slots
  CHECK(throws([&] { PlacementMapping m(p, 2, 1, 4, 0, 0, 8, nullptr); }));
  PlacementMapping ok(p, 2, 1, 4, 0, 1, 8, nullptr);   // fits with one redundant slot
  CHECK(ok.redundant_count(0, 2) == 2 && ok.expert_at(0, 2) == 2);
}

TEST(mapping_reads_a_redundant_pattern) {
  // expert 0 on both ranks
  std::vector<int> p = {1, 1, 0, 0, /*rank 1*/ 1, 0, 1, 1};
  PlacementMapping m(p, 2, 1, 4, 1, 1, 8, nullptr);
  CHECK(m.redundant_count(0, 0) == 2 && m.redundant_count(0, 1) == 1);
  CHECK((m.positions_of(0, 0) == std::vector<int>{0, 3}));
  CHECK((m.local_slots_of(0, 0) == std::vector<int>{0}) && m.local_slots_of(0, 1).empty());
  CHECK(m.selector(0, 0) == 3);                      // own replica
}

TEST(text_pattern_round_trip) {
  const std::string f = tmp_path("pattern.txt");
  { std::ofstream o(f); o << "2 2 4\n1 1 0 0\n1 1 0 0\n0 0 1 1\n0 1 1 1\n"; }
  int w = 0, l = 0, e = 0;
  auto p = PlacementMapping::load_text_pattern(f, w, l, e);
  CHECK(w == 2 && l == 2 && e == 4 && p.size() == 16);
  PlacementMapping m(p, w, l, e, 0, 1, 8, nullptr);
  CHECK(m.redundant_count(1, 1) == 2 && m.redundant_count(0, 1) == 1);
  unlink(f.c_str());
}

TEST(text_pattern_errors) {
  int w, l, e;
  CHECK(throws([&] { PlacementMapping::load_text_pattern("/nonexistent/omni_pattern", w, l, e); }));
  const std::string f = tmp_path("short.txt");
  { std::ofstream o(f); o << "2 1 4\n1 1 0 0\n0 0 1\n"; }
  CHECK(throws([&] { PlacementMapping::load_text_pattern(f, w, l, e); }));
  unlink(f.c_str());
}

TEST(update_checks_bounds_and_ids) {
  auto m = base_mapping(2, 1, 4, 0, 1, 8);
  CHECK(!m.check_update_is_valid(-1, 0, 0, 1) && !m.check_update_is_valid(1, 0, 0, 1));
  CHECK(!m.check_update_is_valid(0, -1, 0, 1) && !m.check_update_is_valid(0, 6, -1, 1));
  CHECK(!m.check_update_is_valid(0, 2, -1, 4) && !m.check_update_is_valid(0, 2, -1, -2));
  CHECK(m.check_update_is_valid(0, 2, -1, 3));
}

TEST(update_needs_the_agreed_old_expert) {
  auto m = base_mapping(2, 1, 4, 0, 1, 8);
  CHECK(!m.update_position(0, 2, 1, 3));             // the slot is empty, not expert 1
  CHECK(m.expert_at(0, 2) == -1 && m.redundant_count(0, 3) == 1);
  CHECK(m.update_position(0, 2, -1, 3));
  CHECK(m.expert_at(0, 2) == 3 && m.redundant_count(0, 3) == 2);
  CHECK(!m.update_position(0, 2, -1, 1));            // now it holds 3
}

TEST(update_never_drops_a_last_replica) {
  auto m = base_mapping(2, 1, 4, 0, 1, 8);
  CHECK(!m.update_position(0, 0, 0, -1) && !m.update_position(0, 0, 0, 2));
  CHECK(m.update_position(0, 0, 0, 0));              // rewriting the same expert is allowed
  CHECK(m.update_position(0, 5, -1, 0));             // a second replica elsewhere ...
  CHECK(m.update_position(0, 0, 0, 2));              // ... frees the first one
  CHECK(m.redundant_count(0, 0) == 1 && m.redundant_count(0, 2) == 2);
}

TEST(batch_update_is_all_or_nothing) {
  auto m = base_mapping(2, 2, 4, 0, 0, 8);
  // rotate three experts of layer 0 in one batch
  CHECK(m.apply_batch({{0, 0}, {0, 1}, {0, 2}}, {1, 2, 0}));
  CHECK(m.expert_at(0, 0) == 1 && m.expert_at(0, 1) == 2 && m.expert_at(0, 2) == 0);
  for (int e = 0; e < 4; ++e) CHECK(m.redundant_count(0, e) == 1);
  // a batch that would orphan expert 3 changes nothing, in either layer it touches
  CHECK(!m.apply_batch({{1, 0}, {0, 3}}, {1, 0}));
  CHECK(m.expert_at(1, 0) == 0 && m.expert_at(0, 3) == 3 && m.redundant_count(1, 0) == 1 && m.redundant_count(0, 3) == 1);
  CHECK(!m.apply_batch({{0, 9}}, {0}) && !m.apply_batch({{0, 0}}, {7}));
}

TEST(selector_prefers_own_rank_then_host_then_distance) {
  // 8 ranks, two hosts of four; expert 0 lives on rank 0; we are rank 5
  std::vector<int32_t> dev(16, -1);
  auto m = base_mapping(8, 1, 16, 5, 1, 4, dev.data());
  CHECK(m.selector(0, 0) == 0 && dev[0] == 0);
  CHECK(m.update_position(0, 6 * 3 + 2, -1, 0));     // replica on rank 6 (same host as 5)
  m.update_selector();
  CHECK(m.selector(0, 0) == 6 * 3 + 2 && dev[0] == 6 * 3 + 2);
  CHECK(m.update_position(0, 5 * 3 + 2, -1, 0));     // replica on our own rank
  m.update_selector_layer(0);
  CHECK(m.selector(0, 0) == 5 * 3 + 2);
  CHECK(dev[0] == 6 * 3 + 2);                        // the device copy changes only on push
  m.push_selector_to_device();
  CHECK(dev[0] == 5 * 3 + 2);
}

TEST(selector_spreads_ranks_over_distant_replicas) {
  // expert 0 has replicas on ranks 0 and 1 (host 0); ranks 4..7 (host 1) must not all pick the same one
  std::vector<int> picks;
  for (int rank = 4; rank < 8; ++rank) {
    auto m = base_mapping(8, 1, 8, rank, 1, 4);
    CHECK(m.update_position(0, 1 * 2 + 1, -1, 0));
    m.update_selector();
    picks.push_back(m.selector(0, 0));
  }
  CHECK(picks[0] != picks[1] && picks[0] == picks[2] && picks[1] == picks[3]);
  CHECK(std::count(picks.begin(), picks.end(), 0) == 2 && std::count(picks.begin(), picks.end(), 3) == 2);
}

TEST(selector_without_a_device_copy_is_host_only) {
  auto m = base_mapping(2, 2, 4, 1, 0, 8, nullptr);
  m.update_selector();
  CHECK(m.selector_host().size() == 8 && m.selector(1, 3) == 3 && m.selector(1, 0) == 0);
}

// ================================================================================================ ClusterActivation
TEST(activation_single_rank_needs_no_collective) {
  std::vector<int64_t> c(2 * 3, 0);
  ClusterActivation a(Tensor(c.data(), 6, 8), 2, 3, 1, 0);
  c[4] = 11;
  a.collect();
  CHECK(a.positions() == 3 && a.layers() == 2 && a.delta(1, 1) == 11 && a.total(1, 1) == 11 && a.delta(0, 0) == 0);
}

TEST(activation_multi_rank_without_allgather_refuses) {
  std::vector<int64_t> c(2, 0);
  ClusterActivation a(Tensor(c.data(), 2, 8), 1, 2, 2, 0);
  CHECK(throws([&] { a.collect(); }));
}

TEST(activation_first_collect_reports_the_counters_themselves) {
  std::vector<int64_t> c = {100, 200};
  ClusterActivation a(Tensor(c.data(), 2, 8), 1, 2, 1, 0);
  a.collect();
  CHECK(a.delta(0, 0) == 100 && a.delta(0, 1) == 200);
  a.collect();
  CHECK(a.delta(0, 0) == 0 && a.delta(0, 1) == 0 && a.total(0, 1) == 200);
}

TEST(activation_wraps_at_1e16) {
  std::vector<int64_t> c = {ClusterActivation::kWrap - 5};
  ClusterActivation a(Tensor(c.data(), 1, 8), 1, 1, 1, 0);
  a.collect();
  c[0] = 7;                                          // 12 more tokens, counter kept modulo 1e16
  a.collect();
  CHECK(a.delta(0, 0) == 12);
}

TEST(activation_window_forgets_old_rounds) {
  std::vector<int64_t> c = {0};
  ClusterActivation a(Tensor(c.data(), 1, 8), 1, 1, 1, 0, /*window*/ 3);
  int64_t want[] = {1, 3, 6, 9, 12};                 // sums of the last three of 1, 2, 3, 4, 5
  for (int i = 1; i <= 5; ++i) {
    c[0] += i;
    a.collect();
    CHECK(a.windowed(0, 0) == want[i - 1]);
  }
}

TEST(activation_layout_is_layer_major_over_ranks) {
  const int L = 2, S = 2, W = 3;
  auto hub = make_fake_hub(W);
  std::vector<std::vector<int64_t>> c(W, std::vector<int64_t>(L * S, 0));
  std::vector<std::unique_ptr<ClusterActivation>> a;
  std::vector<std::unique_ptr<FakeDistribution>> d;
  for (int r = 0; r < W; ++r) {
    for (int i = 0; i < L * S; ++i) c[r][i] = 100 * r + i;     // rank r, layer i / S, slot i % S
    d.emplace_back(new FakeDistribution(hub, r, 8));
    a.emplace_back(new ClusterActivation(Tensor(c[r].data(), L * S, 8), L, S, W, r));
    FakeDistribution* dp = d.back().get();
    a.back()->set_allgather([dp](const int64_t* s, int64_t* rv, size_t n) { dp->allgather_i64(s, rv, n); });
  }
  std::vector<std::thread> th;
  for (int r = 1; r < W; ++r) th.emplace_back([&, r] { a[r]->collect(); });
  a[0]->collect();
  for (auto& t : th) t.join();
  for (int r = 0; r < W; ++r)
    for (int l = 0; l < L; ++l)
      for (int rr = 0; rr < W; ++rr)
        for (int s = 0; s < S; ++s) CHECK(a[r]->delta(l, rr * S + s) == 100 * rr + l * S + s);
}

TEST(activation_dump_and_replay) {
  std::vector<int64_t> c = {4, 5, 6, 7};
  ClusterActivation a(Tensor(c.data(), 4, 8), 2, 2, 1, 0);
  a.collect();
  const std::string f = tmp_path("act.txt");
  a.dump_txt(f);
  std::vector<int64_t> z(4, 0);
  ClusterActivation b(Tensor(z.data(), 4, 8), 2, 2, 1, 0, 2);
  b.collect_from_txt(f);
  b.collect_from_txt(f);
  CHECK(b.delta(1, 1) == 7 && b.total(1, 1) == 14 && b.windowed(0, 0) == 8);
  b.collect_from_txt(f);
  CHECK(b.windowed(0, 0) == 8);                      // window of two
  CHECK(throws([&] { b.collect_from_txt("/nonexistent/omni_act"); }));
  { std::ofstream o(f); o << "1 2 3\n"; }
  CHECK(throws([&] { b.collect_from_txt(f); }));
  unlink(f.c_str());
}

// ================================================================================================ MoEWeights
struct SlotBufs {            // two tensors per slot, as w13 / w2 would be
  std::vector<std::vector<unsigned char>> a, b;
  SlotBufs(int n, size_t na, size_t nb) : a(n, std::vector<unsigned char>(na)), b(n, std::vector<unsigned char>(nb)) {}
};

void fill_slot(SlotBufs& s, int i, unsigned char v) {
  std::fill(s.a[i].begin(), s.a[i].end(), v);
  std::fill(s.b[i].begin(), s.b[i].end(), (unsigned char)(v + 100));
}

TEST(weights_registry_and_expert_bytes) {
  MoEWeights w(2, 3);
  CHECK(w.layers() == 2 && w.slots() == 3 && w.expert_bytes() == 0 && !w.is_initialized());
  SlotBufs s(6, 48, 16);
  for (int l = 0; l < 2; ++l)
    for (int k = 0; k < 3; ++k) {
      w.add_tensor(l, k, s.a[l * 3 + k].data(), 48);
      w.add_tensor(l, k, s.b[l * 3 + k].data(), 16);
    }
  w.set_initialized();
  CHECK(w.is_initialized() && w.expert_bytes() == 64);
  CHECK(w.tensors(1, 2).size() == 2 && w.tensors(1, 2)[0].ptr == s.a[5].data() && w.tensors(1, 2)[1].bytes == 16);
}

TEST(weights_expert_bytes_skips_unregistered_slots) {
  MoEWeights w(1, 3);
  std::vector<unsigned char> buf(24);
  w.add_tensor(0, 2, buf.data(), 24);               // only the last slot is registered so far
  CHECK(w.expert_bytes() == 24 && w.tensors(0, 0).empty());
}

TEST(replica_needs_registered_tensors) {
  MoEWeights w(1, 2);
  CHECK(!w.init_shared_memory("/" + std::to_string(getpid()) + "_omni_units_none", 4, 1));
  CHECK(!w.replica_enabled() && !w.replica_complete() && !w.replica_has(0, 0) && w.replica_bytes() == 0);
}

TEST(replica_round_trip_on_one_rank) {
  const std::string name = "/" + std::to_string(getpid()) + "_omni_units_one";
  auto m = base_mapping(1, 2, 3, 0, 1, 8);          // 3 experts + 1 redundant slot, two layers
  MoEWeights w(2, 4);
  SlotBufs s(8, 40, 24);
  for (int l = 0; l < 2; ++l)
    for (int k = 0; k < 4; ++k) {
      fill_slot(s, l * 4 + k, (unsigned char)(10 * l + k + 1));
      w.add_tensor(l, k, s.a[l * 4 + k].data(), 40);
      w.add_tensor(l, k, s.b[l * 4 + k].data(), 24);
    }
  CHECK(w.init_shared_memory(name, 3, 1));
  CHECK(w.replica_enabled() && !w.replica_complete() && !w.replica_has(1, 2));
  CHECK(!w.init_shared_memory(name, 3, 1));          // already attached
  w.replicate_to_shared_memory(m);
  CHECK(w.replica_complete() && w.replica_has(0, 0) && w.replica_has(1, 2));
  CHECK(!w.replica_has(2, 0) && !w.replica_has(0, 3) && !w.replica_has(-1, 0));
  // expert 2 of layer 1 into the redundant slot of that layer
  CHECK(w.replace_from_shared_memory(1, 2, 3));
  CHECK(s.a[7] == s.a[6] && s.b[7] == s.b[6] && s.a[7][0] == 13 && s.b[7][0] == 113);
  CHECK(!w.replace_from_shared_memory(1, 2, 4) && !w.replace_from_shared_memory(1, 3, 0));
  CHECK(w.replica_bytes() >= 2u * 3 * 64);
  w.close_shared_memory(true);
  CHECK(!w.replica_enabled());
}

TEST(replica_is_shared_by_the_ranks_of_a_host) {
  const std::string name = "/" + std::to_string(getpid()) + "_omni_units_two";
  const int W = 2, E = 4;
  std::vector<std::unique_ptr<MoEWeights>> w;
  std::vector<std::unique_ptr<SlotBufs>> bufs;
  std::vector<PlacementMapping> maps;
  for (int r = 0; r < W; ++r) {
    maps.push_back(base_mapping(W, 1, E, r, 1, 8));
    w.emplace_back(new MoEWeights(1, 3));
    bufs.emplace_back(new SlotBufs(3, 32, 32));
    for (int k = 0; k < 3; ++k) {
      fill_slot(*bufs[r], k, (unsigned char)(k < 2 ? r * 2 + k + 1 : 0));     // value = logical expert + 1
      w[r]->add_tensor(0, k, bufs[r]->a[k].data(), 32);
      w[r]->add_tensor(0, k, bufs[r]->b[k].data(), 32);
    }
  }
  std::thread t([&] { CHECK(w[1]->init_shared_memory(name, E, W)); w[1]->replicate_to_shared_memory(maps[1]); });
  CHECK(w[0]->init_shared_memory(name, E, W));
  w[0]->replicate_to_shared_memory(maps[0]);
  t.join();
  CHECK(w[0]->replica_complete() && w[1]->replica_complete());
  // rank 0 takes expert 3 (home: rank 1) into its spare slot without rank 1 doing anything
  CHECK(w[0]->replace_from_shared_memory(0, 3, 2));
  CHECK(bufs[0]->a[2][5] == 4 && bufs[0]->b[2][5] == 104);
  w[1]->close_shared_memory(false);
  w[0]->close_shared_memory(true);
}

TEST(replica_of_another_deployment_is_refused) {
  const std::string name = "/" + std::to_string(getpid()) + "_omni_units_other";
  std::vector<unsigned char> b1(512), b2(64);
  MoEWeights a(1, 1), b(1, 1);
  a.add_tensor(0, 0, b1.data(), 512);
  b.add_tensor(0, 0, b2.data(), 64);                // other expert size under the same name
  CHECK(a.init_shared_memory(name, 2, 1));
  CHECK(!b.init_shared_memory(name, 2, 1) && !b.replica_enabled());
  a.close_shared_memory(true);
}

// ================================================================================================ Distribution
TEST(fake_allgather_orders_by_rank) {
  const int W = 4;
  auto hub = make_fake_hub(W);
  std::vector<std::vector<int64_t>> got(W, std::vector<int64_t>(2 * W));
  std::vector<std::thread> th;
  for (int r = 0; r < W; ++r)
    th.emplace_back([&, r] {
      FakeDistribution d(hub, r, 8);
      CHECK(d.rank() == r && d.world() == W);
      for (int round = 0; round < 3; ++round) {      // generations must not mix
        int64_t mine[2] = {10 * r + round, -r};
        d.allgather_i64(mine, got[r].data(), 2);
        for (int q = 0; q < W; ++q) CHECK(got[r][2 * q] == 10 * q + round && got[r][2 * q + 1] == -q);
      }
      d.barrier();
    });
  for (auto& t : th) t.join();
}

TEST(fake_swap_lands_in_the_named_stage) {
  auto hub = make_fake_hub(2);
  std::vector<unsigned char> a0(16, 1), b0(8, 2), a1(16, 7), b1(8, 9);
  FakeDistribution d0(hub, 0, 24), d1(hub, 1, 24);
  std::thread t([&] { d1.swap(0, {{a1.data(), 16}, {b1.data(), 8}}, 3); });
  d0.swap(1, {{a0.data(), 16}, {b0.data(), 8}}, 1);
  t.join();
  auto* s0 = (unsigned char*)d0.staging(1);
  auto* s1 = (unsigned char*)d1.staging(3);
  CHECK(s0[0] == 7 && s0[15] == 7 && s0[16] == 9 && s0[23] == 9);
  CHECK(s1[0] == 1 && s1[16] == 2);
  CHECK(d0.transfers() == 1 && d1.transfers() == 1 && !d0.staging_on_device());
}

TEST(fake_one_way_transfer) {
  auto hub = make_fake_hub(3);
  std::vector<unsigned char> payload(12);
  std::iota(payload.begin(), payload.end(), 40);
  FakeDistribution d0(hub, 0, 12), d2(hub, 2, 12);
  d0.send_only(2, {{payload.data(), 12}});          // mailbox: the sender does not wait for the receiver
  d2.recv_only(0, 4, 12);
  CHECK(std::memcmp(d2.staging(4), payload.data(), 12) == 0);
}

TEST(fake_handshake_can_be_corrupted_once) {
  auto hub = make_fake_hub(2);
  FakeDistribution d0(hub, 0, 8), d1(hub, 1, 8);
  d1.corrupt_next_handshake();
  std::vector<HandshakeTuple> all0, all1;
  for (int round = 0; round < 2; ++round) {
    std::thread t([&] { d1.allgather_handshake({1, 2, 5, 1}, all1); });
    d0.allgather_handshake({1, 2, 5, 1}, all0);
    t.join();
    CHECK(all0.size() == 2 && all0[0].expert_id == 5 && all0[1].t_rank == 1 && all0[1].replica_ok == 1);
    CHECK(all0[1].expert_id == (round == 0 ? 1005 : 5) && all1[1].expert_id == all0[1].expert_id);
  }
}

TEST(callback_transport_packs_and_stages_on_the_host) {
  std::vector<unsigned char> wire;
  DistributionCallbacks cb;
  cb.rank = 1; cb.world = 2;
  cb.allgather_i64 = [](const int64_t* s, int64_t* r, size_t n) { for (size_t i = 0; i < n; ++i) { r[i] = s[i] + 1; r[n + i] = s[i]; } };
  cb.sendrecv = [&](int peer, const void* send, void* recv, size_t bytes) {
    CHECK(peer == 0);
    if (send) wire.assign((const unsigned char*)send, (const unsigned char*)send + bytes);
    if (recv) std::memset(recv, 0x5a, bytes);
  };
  int barriers = 0;
  cb.barrier = [&] { ++barriers; };
  CallbackDistribution d(cb, 10);
  CHECK(d.rank() == 1 && d.world() == 2 && !d.staging_on_device());
  std::vector<unsigned char> a(6, 3), b(4, 8);
  d.swap(0, {{a.data(), 6}, {b.data(), 4}}, 2);
  CHECK(wire.size() == 10 && wire[0] == 3 && wire[5] == 3 && wire[6] == 8);
  CHECK(((unsigned char*)d.staging(2))[9] == 0x5a);
  std::vector<HandshakeTuple> all;
  d.allgather_handshake({3, 1, 7, 1}, all);         // tuples travel as four int64 each
  CHECK(all.size() == 2 && all[0].t_rank == 4 && all[0].expert_id == 8 && all[1].position_offset == 1 && all[1].replica_ok == 1);
  d.barrier();
  CHECK(barriers == 1);
}

TEST(callback_transport_with_device_buffers_never_touches_the_host_ring) {
  std::vector<unsigned char> send_buf(16, 0);
  std::vector<std::vector<unsigned char>> stage(Distribution::QUEUE_SIZE, std::vector<unsigned char>(16, 0));
  void* stages[Distribution::QUEUE_SIZE];
  for (int i = 0; i < Distribution::QUEUE_SIZE; ++i) stages[i] = stage[i].data();
  DistributionCallbacks cb;
  cb.rank = 0; cb.world = 2;
  const void* seen_send = nullptr;
  void* seen_recv = nullptr;
  cb.sendrecv = [&](int, const void* s, void* r, size_t n) { seen_send = s; seen_recv = r; if (s && r) std::memcpy(r, s, n); };
  CallbackDistribution d(cb, 16, send_buf.data(), stages);
  CHECK(d.staging_on_device() && d.staging(4) == stage[4].data());
  std::vector<unsigned char> a(10, 6), b(6, 2);
  d.swap(1, {{a.data(), 10}, {b.data(), 6}}, 4);
  CHECK(seen_send == send_buf.data() && seen_recv == stage[4].data());
  CHECK(send_buf[9] == 6 && send_buf[10] == 2 && stage[4][15] == 2);
}

// ================================================================================================ GreedyExpertLoadBalancer
double ratio_of(const std::vector<int>& place, const std::vector<double>& load, int W, int S) {
  std::vector<double> rl(W, 0.0);
  for (int p = 0; p < W * S; ++p) if (place[p] >= 0) rl[p / S] += load[p];
  return GreedyExpertLoadBalancer::imbalance(rl);
}

// replays instructions on one layer the way the balancer's own simulation does: replicas share an expert's load evenly
void replay(std::vector<int>& place, std::vector<double>& load, const std::vector<ChangeInstruction>& ins, int layer) {
  const int P = (int)place.size();
  auto spread = [&](int e) {
    double tot = 0; int n = 0;
    for (int p = 0; p < P; ++p) if (place[p] == e) { tot += load[p]; ++n; }
    for (int p = 0; p < P; ++p) if (place[p] == e) load[p] = tot / n;
  };
  for (const auto& i : ins) {
    if (i.layer_idx != layer) continue;
    const int sp = i.source_global_position, tp = i.target_global_position;
    if (i.type == OperationType::SWAP) { std::swap(place[sp], place[tp]); std::swap(load[sp], load[tp]); }
    else if (i.type == OperationType::REMOVE) { const int e = place[sp]; const double l = load[sp]; place[sp] = -1; load[sp] = 0; for (int p = 0; p < P; ++p) if (place[p] == e) { load[p] += l; break; } spread(e); }
    else if (i.type == OperationType::ADD) {
      const int old = place[tp];
      if (old >= 0) { const double l = load[tp]; place[tp] = -1; load[tp] = 0; for (int p = 0; p < P; ++p) if (place[p] == old) { load[p] += l; break; } spread(old); }
      place[tp] = i.source_expert_id; load[tp] = 0; spread(i.source_expert_id);
    }
  }
}

TEST(imbalance_is_max_over_min) {
  CHECK(std::fabs(GreedyExpertLoadBalancer::imbalance({10, 20, 40}) - 4.0) < 1e-12);
  CHECK(GreedyExpertLoadBalancer::imbalance({0, 0, 0}) == 1.0);
  CHECK(GreedyExpertLoadBalancer::imbalance({5, 0}) > 1e6);         // an idle rank: finite but huge
  CHECK(std::isfinite(GreedyExpertLoadBalancer::imbalance({5, 0})));
}

TEST(greedy_leaves_a_balanced_layer_alone) {
  GreedyExpertLoadBalancer g(1, 4, 8, 3);
  std::vector<int> place = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {50, 50, 0, 50, 50, 0, 50, 50, 0, 50, 50, 0};
  CHECK(g.optimize_and_generate_instructions(place, act).empty());
  CHECK(g.has_ema() && g.ema_loads()[0] == 50.0);
}

TEST(greedy_below_the_threshold_does_nothing) {
  GreedyExpertLoadBalancer g(1, 2, 4, 3);
  std::vector<int> place = {0, 1, -1, 2, 3, -1};
  std::vector<int64_t> act = {52, 50, 0, 49, 50, 0};                 // 102 : 99 = 1.03 < 1.1
  CHECK(g.optimize_and_generate_instructions(place, act).empty());
}

TEST(greedy_replicates_a_hot_expert) {
  const int W = 4, S = 3;
  GreedyExpertLoadBalancer g(1, W, 8, S);
  std::vector<int> place = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {1000, 40, 0, 50, 50, 0, 50, 50, 0, 50, 50, 0};
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty());
  bool added_hot = false;
  for (const auto& i : ins) added_hot = added_hot || (i.type == OperationType::ADD && i.source_expert_id == 0);
  CHECK(added_hot);
  std::vector<double> load(act.begin(), act.end());
  const double before = ratio_of(place, load, W, S);
  replay(place, load, ins, 0);
  CHECK(ratio_of(place, load, W, S) < 0.5 * before);
  for (int r = 0; r < W; ++r) {                                       // never two replicas of one expert on a rank
    std::vector<int> seen;
    for (int s = 0; s < S; ++s) if (place[r * S + s] >= 0) seen.push_back(place[r * S + s]);
    std::sort(seen.begin(), seen.end());
    CHECK(std::adjacent_find(seen.begin(), seen.end()) == seen.end());
  }
}

TEST(greedy_swaps_when_there_is_no_free_slot) {
  const int W = 2, S = 2;
  GreedyExpertLoadBalancer g(1, W, 4, S);
  std::vector<int> place = {0, 1, 2, 3};
  std::vector<int64_t> act = {100, 90, 10, 20};                       // 190 : 30
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty());
  for (const auto& i : ins) CHECK(i.type == OperationType::SWAP && i.source_rank != i.target_rank);
  std::vector<double> load(act.begin(), act.end());
  replay(place, load, ins, 0);
  CHECK(ratio_of(place, load, W, S) < 1.3);                           // 110 : 110 is reachable ({100,10} | {90,20})
}

TEST(greedy_removes_a_replica_that_hurts) {
  // expert 0 has a replica on rank 1, which is the hot rank because of expert 2
  const int W = 2, S = 3;
  GreedyExpertLoadBalancer g(1, W, 4, S);
  std::vector<int> place = {0, 1, -1, 2, 3, 0};
  std::vector<int64_t> act = {10, 10, 0, 300, 20, 10};
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty() && ins[0].type == OperationType::REMOVE && ins[0].source_global_position == 5 && ins[0].source_expert_id == 0);
}

TEST(greedy_respects_the_replica_limit) {
  const int W = 4, S = 3;
  GreedyExpertLoadBalancer g(1, W, 8, S, /*max redundant per expert*/ 1);
  std::vector<int> place = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {5000, 10, 0, 10, 10, 0, 10, 10, 0, 10, 10, 0};
  auto ins = g.optimize_and_generate_instructions(place, act);
  std::vector<double> load(act.begin(), act.end());
  replay(place, load, ins, 0);
  CHECK(std::count(place.begin(), place.end(), 0) <= 2);
}

TEST(greedy_caps_the_instructions_per_layer) {
  const int W = 8, S = 5, E = 32;
  GreedyExpertLoadBalancer g(1, W, E, S, 10, 0.6, 1.0001, /*max instructions*/ 3);
  std::vector<int> place(W * S, -1);
  std::vector<int64_t> act(W * S, 0);
  for (int e = 0; e < E; ++e) { place[(e / 4) * S + e % 4] = e; act[(e / 4) * S + e % 4] = 10 + 37 * ((e * 7) % 11) * (e % 3 == 0 ? 9 : 1); }
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty() && ins.size() <= 3);
  for (size_t i = 0; i < ins.size(); ++i) CHECK(ins[i].prior == (int)i);
}

TEST(greedy_handles_each_layer_on_its_own) {
  const int W = 2, S = 3;
  GreedyExpertLoadBalancer g(2, W, 4, S);
  std::vector<int> place = {0, 1, -1, 2, 3, -1, /*layer 1*/ 0, 1, -1, 2, 3, -1};
  std::vector<int64_t> act = {50, 50, 0, 50, 50, 0, /*layer 1: expert 3 hot*/ 10, 10, 0, 10, 400, 0};
  auto ins = g.optimize_and_generate_instructions(place, act);
  CHECK(!ins.empty());
  for (const auto& i : ins) CHECK(i.layer_idx == 1);
}

TEST(greedy_average_keeps_six_tenths_of_the_history) {
  GreedyExpertLoadBalancer g(1, 2, 2, 1);
  std::vector<int> place = {0, 1};
  g.optimize_and_generate_instructions(place, {100, 100});
  g.optimize_and_generate_instructions(place, {0, 200});
  CHECK(std::fabs(g.ema_loads()[0] - 60.0) < 1e-9 && std::fabs(g.ema_loads()[1] - 140.0) < 1e-9);
}

TEST(greedy_history_can_be_saved_and_restored) {
  GreedyExpertLoadBalancer a(1, 2, 2, 1), b(1, 2, 2, 1);
  std::vector<int> place = {0, 1};
  a.optimize_and_generate_instructions(place, {100, 300});
  CHECK(!b.has_ema() && !b.set_ema({1.0}) && !b.has_ema());           // wrong shape: refused
  CHECK(b.set_ema(a.ema_loads()) && b.has_ema());
  a.optimize_and_generate_instructions(place, {200, 200});
  b.optimize_and_generate_instructions(place, {200, 200});
  CHECK(a.ema_loads() == b.ema_loads());
}

TEST(greedy_rejects_mismatched_shapes) {
  GreedyExpertLoadBalancer g(1, 2, 4, 3);
  CHECK(throws([&] { g.optimize_and_generate_instructions({0, 1, 2, 3}, {1, 1, 1, 1}); }));
  CHECK(throws([&] { g.optimize_and_generate_instructions({0, 1, -1, 2, 3, -1}, {1, 1}); }));
}

// ================================================================================================ ExpertLoadBalancer
TEST(static_placement_gives_spare_slots_to_hot_experts) {
  ExpertLoadBalancer b(4, 8, 3, 2);
  std::vector<double> loads = {800, 10, 10, 10, 400, 10, 10, 10};
  auto p = b.generate_constrained_placement(loads, 10);
  CHECK(b.validate(p));
  auto c = b.replica_counts(p);
  CHECK(c[0] >= 3 && c[4] >= 2 && c[1] == 1 && std::accumulate(c.begin(), c.end(), 0) == 12);
}

TEST(static_placement_respects_the_replica_limit) {
  ExpertLoadBalancer b(4, 8, 3, 2);
  std::vector<double> loads = {800, 10, 10, 10, 400, 10, 10, 10};
  auto p = b.generate_constrained_placement(loads, 1);
  auto c = b.replica_counts(p);
  CHECK(b.validate(p) && *std::max_element(c.begin(), c.end()) <= 2);
}

TEST(static_placement_spreads_replicas_over_hosts) {
  ExpertLoadBalancer b(4, 4, 2, /*ranks per host*/ 2);
  auto p = b.generate_constrained_placement({1000, 1, 1, 1}, 10);
  CHECK(b.validate(p));
  std::vector<int> hosts;
  for (int q = 0; q < 8; ++q) if (p[q] == 0) hosts.push_back((q / 2) / 2);
  CHECK(hosts.size() >= 2 && std::count(hosts.begin(), hosts.end(), 0) >= 1 && std::count(hosts.begin(), hosts.end(), 1) >= 1);
}

TEST(static_placement_argument_errors) {
  ExpertLoadBalancer b(2, 8, 3);
  CHECK(throws([&] { b.generate_constrained_placement({1, 2, 3}, 1); }));            // one load per expert
  CHECK(throws([&] { b.generate_constrained_placement(std::vector<double>(8, 1.0), 1); }));   // 6 slots for 8 experts
}

TEST(validate_finds_each_kind_of_defect) {
  ExpertLoadBalancer b(2, 4, 3);
  CHECK(b.validate({0, 1, -1, 2, 3, -1}) && b.validate({0, 1, 2, 2, 3, 0}));
  CHECK(!b.validate({0, 1, -1, 2, 3}));                 // size
  CHECK(!b.validate({0, 1, -1, 2, 2, -1}));             // expert 3 missing, expert 2 twice on a rank
  CHECK(!b.validate({0, 1, 0, 2, 3, -1}));              // two replicas on one rank
  CHECK(!b.validate({0, 1, -1, 2, 3, 4}));              // id out of range
  CHECK(!b.validate({0, 1, -2, 2, 3, -1}));
}

TEST(bucket_balance_evens_out_two_ranks) {
  ExpertLoadBalancer b(2, 4, 2);
  std::vector<double> loads = {100, 90, 10, 20};
  std::vector<int> place = {0, 1, 2, 3};
  auto ins = b.bucket_balance(0, place, loads, 8);
  CHECK(!ins.empty());
  for (const auto& i : ins) { CHECK(i.type == OperationType::SWAP); CHECK(b.apply(place, i)); }
  CHECK(b.validate(place));
  CHECK(std::fabs(b.simulated_ratio(place, loads) - 1.0) < 1e-9);      // {100, 10} | {90, 20}
  CHECK(b.bucket_balance(0, place, loads, 8).empty());                 // nothing left to gain
  CHECK(b.bucket_balance(0, {0, 1, 2, 3}, loads, 0).empty());          // no budget
}

TEST(analysis_helpers) {
  ExpertLoadBalancer b(2, 4, 3);
  std::vector<int> place = {0, 1, 3, 2, 3, -1};
  std::vector<int64_t> act = {10, 20, 30, 40, 50, 0};
  auto el = b.expert_loads(place, act);
  CHECK(el[0] == 10 && el[1] == 20 && el[2] == 40 && el[3] == 80);
  CHECK((b.replica_counts(place) == std::vector<int>{1, 1, 1, 2}));
  auto rl = b.simulated_rank_loads(place, el);                         // expert 3 is shared evenly: 40 each
  CHECK(rl[0] == 70 && rl[1] == 80);
  CHECK(std::fabs(b.simulated_ratio(place, el) - 80.0 / 75.0) < 1e-12);
  CHECK(std::fabs(b.measured_ratio(place, act) - 90.0 / 75.0) < 1e-12);
  CHECK(b.find_position(place, 1, 3) == 4 && b.find_position(place, 0, 2) == -1);
  CHECK(b.find_empty(place, 1) == 5 && b.find_empty(place, 0) == -1);
  CHECK(b.validate_counts(place, 2, 3) && !b.validate_counts(place, 3, 3) && !b.validate_counts(place, 1, 2));
  CHECK(b.diff_count(place, place) == 0);
  CHECK(b.diff_count(place, {0, 1, 2, 2, 3, -1}) == 2);                // rank 0 drops 3 and fetches 2
}

TEST(apply_checks_each_instruction) {
  ExpertLoadBalancer b(2, 4, 3);
  std::vector<int> place = {0, 1, -1, 2, 3, -1};
  ChangeInstruction add;
  add.type = OperationType::ADD; add.source_rank = 0; add.source_expert_id = 0; add.source_global_position = 0;
  add.target_rank = 1; add.target_expert_id = -1; add.target_global_position = 5;
  CHECK(b.apply(place, add) && place[5] == 0);
  CHECK(!b.apply(place, add));                                          // the slot is no longer empty
  ChangeInstruction rm;
  rm.type = OperationType::REMOVE; rm.source_rank = rm.target_rank = 1; rm.source_expert_id = 0;
  rm.source_global_position = rm.target_global_position = 5;
  CHECK(b.apply(place, rm) && place[5] == -1);
  rm.source_expert_id = 2; rm.source_global_position = rm.target_global_position = 3;
  auto before = place;
  CHECK(!b.apply(place, rm) && place == before);                        // the last replica stays
  ChangeInstruction sw;
  sw.type = OperationType::SWAP; sw.source_rank = 0; sw.source_expert_id = 1; sw.source_global_position = 1;
  sw.target_rank = 1; sw.target_expert_id = 2; sw.target_global_position = 3;
  CHECK(b.apply(place, sw) && place[1] == 2 && place[3] == 1);
  CHECK(!b.apply(place, sw));                                           // stale: the experts have moved
}

TEST(priorities_order_dependent_instructions) {
  auto mk = [](int layer, int se, int sp, int te, int tp) {
    ChangeInstruction i; i.layer_idx = layer; i.type = OperationType::SWAP;
    i.source_expert_id = se; i.source_global_position = sp; i.target_expert_id = te; i.target_global_position = tp;
    i.source_rank = sp / 2; i.target_rank = tp / 2;
    return i;
  };
  // layer 0: the second swap reuses position 2, the third is independent; layer 1 starts again at zero
  std::vector<ChangeInstruction> v = {mk(0, 0, 0, 2, 2), mk(0, 0, 2, 5, 5), mk(0, 6, 6, 7, 9), mk(1, 0, 0, 2, 2)};
  ExpertLoadBalancer::assign_priorities(v);
  CHECK(v.size() == 4);
  std::vector<std::pair<int, int>> lp;
  for (auto& i : v) lp.push_back({i.layer_idx, i.prior});
  CHECK(std::is_sorted(lp.begin(), lp.end()));
  int waves0 = 0, first_wave0 = 0;
  for (auto& i : v) if (i.layer_idx == 0) { waves0 = std::max(waves0, i.prior); first_wave0 += i.prior == v.front().prior; }
  CHECK(first_wave0 == 2 && waves0 == v.front().prior + 1);             // two independent ones first, the dependent one after
  CHECK(v.back().layer_idx == 1 && v.back().prior == v.front().prior);
}

TEST(plan_layer_cuts_at_the_communication_limit) {
  ExpertLoadBalancer b(4, 8, 3, 2);
  std::vector<int> place = {0, 1, -1, 2, 3, -1, 4, 5, -1, 6, 7, -1};
  std::vector<int64_t> act = {900, 300, 0, 20, 20, 0, 20, 20, 0, 20, 20, 0};
  StaticBalanceOptions opt;
  opt.diff_limit = 1;
  auto one = b.plan_layer(0, place, act, opt);
  CHECK(one.instructions.size() <= 1 && one.considered >= (int)one.instructions.size());
  opt.diff_limit = -1;
  auto many = b.plan_layer(0, place, act, opt);
  CHECK(many.accepted && many.ratio_after < many.ratio_before && many.ratio_after <= one.ratio_after + 1e-12);
  CHECK(b.validate(many.placement));
  auto replayed = place;
  for (const auto& i : many.instructions) CHECK(b.apply(replayed, i));
  CHECK(replayed == many.placement);
}

TEST(plan_layer_keeps_a_good_layer) {
  ExpertLoadBalancer b(2, 4, 3);
  std::vector<int> place = {0, 1, -1, 2, 3, -1};
  auto plan = b.plan_layer(0, place, {50, 50, 0, 50, 52, 0}, StaticBalanceOptions());
  CHECK(!plan.accepted && plan.instructions.empty() && plan.placement == place);
}

// ================================================================================================ PlacementOptimizer
TEST(optimizer_reads_the_mapping_and_the_counters) {
  std::vector<int64_t> c = {7, 9, 0, 11, 13, 0};                      // one rank would see only its own; world 1 here
  auto m = base_mapping(1, 2, 2, 0, 1, 8);
  ClusterActivation a(Tensor(c.data(), 6, 8), 2, 3, 1, 0);
  a.collect();
  PlacementOptimizer o(&m, &a);
  CHECK((o.extract_placement() == std::vector<int>{0, 1, -1, 0, 1, -1}));
  CHECK((o.extract_activations() == std::vector<int64_t>{7, 9, 0, 11, 13, 0}));
  CHECK(o.optimize().empty());                                          // one rank: nothing to balance
  CHECK(o.balancer().has_ema());
}

TEST(optimizer_proposes_a_replica_of_the_hot_expert) {
  const int W = 2, L = 1, E = 4, S = 3;
  std::vector<int64_t> c0 = {900, 10, 0}, c1 = {10, 10, 0};
  auto hub = make_fake_hub(W);
  auto m0 = base_mapping(W, L, E, 0, 1, 8), m1 = base_mapping(W, L, E, 1, 1, 8);
  ClusterActivation a0(Tensor(c0.data(), S, 8), L, S, W, 0), a1(Tensor(c1.data(), S, 8), L, S, W, 1);
  FakeDistribution d0(hub, 0, 8), d1(hub, 1, 8);
  a0.set_allgather([&](const int64_t* s, int64_t* r, size_t n) { d0.allgather_i64(s, r, n); });
  a1.set_allgather([&](const int64_t* s, int64_t* r, size_t n) { d1.allgather_i64(s, r, n); });
  std::thread t([&] { a1.collect(); });
  a0.collect();
  t.join();
  PlacementOptimizer o0(&m0, &a0), o1(&m1, &a1);
  auto i0 = o0.optimize(), i1 = o1.optimize();
  CHECK(!i0.empty() && i0.size() == i1.size());                         // every rank derives the same plan
  for (size_t k = 0; k < i0.size(); ++k)
    CHECK(i0[k].type == i1[k].type && i0[k].source_expert_id == i1[k].source_expert_id &&
          i0[k].target_global_position == i1[k].target_global_position);
  CHECK(i0[0].source_expert_id == 0 && i0[0].target_rank == 1);
}

// ================================================================================================ Placement manager
// W ranks as threads, one layer, E experts, one redundant slot per rank; slot contents identify the expert they hold.
struct Cluster {
  int W, E, S, L;
  std::shared_ptr<FakeHub> hub;
  std::vector<std::vector<float>> storage;
  std::vector<std::vector<int64_t>> counts;
  std::vector<std::vector<int32_t>> sel;
  std::vector<std::unique_ptr<PlacementMapping>> maps;
  std::vector<std::unique_ptr<MoEWeights>> ws;
  std::vector<std::unique_ptr<ClusterActivation>> acts;
  std::vector<std::unique_ptr<FakeDistribution>> dists;
  std::vector<std::unique_ptr<Placement>> pls;

  Cluster(int world, int experts, int layers = 1)
      : W(world), E(experts), S(experts / world + 1), L(layers), hub(make_fake_hub(world)) {
    storage.assign(W, std::vector<float>(L * S * 4));
    counts.assign(W, std::vector<int64_t>(L * S, 0));
    sel.assign(W, std::vector<int32_t>(L * E, -1));
    auto pat = PlacementMapping::base_pattern(W, L, E);
    for (int r = 0; r < W; ++r) {
      for (int l = 0; l < L; ++l)
        for (int s = 0; s < S; ++s)
          for (int k = 0; k < 4; ++k) storage[r][(l * S + s) * 4 + k] = s < E / W ? float(100 * l + r * (E / W) + s) : -1.f;
      maps.emplace_back(new PlacementMapping(pat, W, L, E, r, 1, 8, sel[r].data()));
      ws.emplace_back(new MoEWeights(L, S));
      for (int l = 0; l < L; ++l)
        for (int s = 0; s < S; ++s) ws[r]->add_tensor(l, s, storage[r].data() + (l * S + s) * 4, 4 * sizeof(float));
      ws[r]->set_initialized();
      acts.emplace_back(new ClusterActivation(Tensor(counts[r].data(), L * S, 8), L, S, W, r, 4));
      dists.emplace_back(new FakeDistribution(hub, r, ws[r]->expert_bytes()));
      pls.emplace_back(new Placement(maps[r].get(), ws[r].get(), acts[r].get(), dists[r].get(), 10, 3600.0));
    }
  }
  // one round on every rank, then the apply step of every rank; returns what rank 0 executed
  int round(std::vector<int>* replaced = nullptr) {
    std::vector<int> done(W, 0);
    std::vector<std::thread> th;
    for (int r = 1; r < W; ++r) th.emplace_back([&, r] { done[r] = pls[r]->run_round(); });
    done[0] = pls[0]->run_round();
    for (auto& t : th) t.join();
    for (int r = 0; r < W; ++r) {
      const int n = pls[r]->do_placement_optimizer();
      if (replaced) replaced->push_back(n);
    }
    return done[0];
  }
  float held(int rank, int slot, int layer = 0) const { return storage[rank][(layer * S + slot) * 4]; }
  bool views_agree() const {
    for (int r = 1; r < W; ++r)
      for (int l = 0; l < L; ++l)
        for (int p = 0; p < W * S; ++p)
          if (maps[r]->expert_at(l, p) != maps[0]->expert_at(l, p)) return false;
    return true;
  }
};

TEST(manager_apply_step_without_pending_work_is_free) {
  Cluster c(2, 4);
  CHECK(c.pls[0]->do_placement_optimizer() == 0 && c.pls[0]->rounds() == 0 && c.pls[0]->last_instructions().empty());
}

TEST(manager_quiet_cluster_plans_nothing) {
  Cluster c(2, 4);
  c.counts[0] = {50, 50, 0};
  c.counts[1] = {50, 50, 0};
  std::vector<int> replaced;
  CHECK(c.round(&replaced) == 0 && replaced == std::vector<int>({0, 0}));
  CHECK(c.pls[0]->rounds() == 1 && c.pls[1]->rounds() == 1 && c.pls[0]->skipped_instructions() == 0);
  CHECK(c.dists[0]->transfers() == 0);
}

TEST(manager_copies_the_hot_expert_and_reroutes) {
  Cluster c(3, 6);
  c.counts[0] = {10, 10, 0};
  c.counts[1] = {10, 10, 0};
  c.counts[2] = {10, 1500, 0};                       // expert 5 on rank 2
  std::vector<int> replaced;
  CHECK(c.round(&replaced) >= 1);
  CHECK(c.views_agree());
  // The plan replicates expert 5 onto rank 0 and then, from that new replica, onto rank 1.  The new replica's bytes
  // are still in a staging buffer when the second copy is made, so the manager takes them from the settled replica
  // on rank 2 instead: both new replicas must hold expert 5, and only the receiving ranks copied anything.
  auto plan = c.pls[0]->last_instructions();
  CHECK(plan.size() == 2 && plan[1].type == OperationType::ADD && plan[1].source_global_position == plan[0].target_global_position);
  for (int r = 0; r < 2; ++r) {
    CHECK(c.maps[0]->expert_at(0, r * 3 + 2) == 5 && c.held(r, 2) == 5.f && replaced[r] == 1);
    CHECK(c.maps[r]->selector(0, 5) == r * 3 + 2 && c.sel[r][5] == r * 3 + 2);   // routes expert 5 to itself now
  }
  CHECK(replaced[2] == 0 && c.maps[0]->redundant_count(0, 5) == 3);
  CHECK(c.maps[2]->selector(0, 5) == 2 * 3 + 1);     // the home rank keeps its own
  CHECK(c.dists[2]->transfers() == 2 && c.dists[0]->transfers() == 1 && c.dists[1]->transfers() == 1);
}

TEST(manager_full_staging_ring_defers_the_rest_on_every_rank) {
  // seven layers, in each of them rank 0's first expert is hot: seven replicas for rank 1, whose ring holds five
  const int L = 7;
  Cluster c(2, 4, L);
  for (int l = 0; l < L; ++l) { c.counts[0][l * 3] = 1000; c.counts[0][l * 3 + 1] = 10; c.counts[1][l * 3] = 10; c.counts[1][l * 3 + 1] = 10; }
  std::vector<int> replaced;
  const int done = c.round(&replaced);               // would hang if the ranks left the round at different instructions
  CHECK(done == Distribution::QUEUE_SIZE && replaced[1] == Distribution::QUEUE_SIZE && replaced[0] == 0);
  CHECK(c.pls[0]->last_instructions().size() == (size_t)L && c.views_agree());
  int with_replica = 0;
  for (int l = 0; l < L; ++l)
    if (c.maps[0]->expert_at(l, 5) == 0) { ++with_replica; CHECK(c.held(1, 2, l) == float(100 * l)); }
    else CHECK(c.held(1, 2, l) == -1.f);
  CHECK(with_replica == Distribution::QUEUE_SIZE);
  // the next round serves the layers that had to wait (the served ones are quiet: their traffic now goes to the new
  // replica, in the amount that levels the moving averages: 0.6 * 1000 = 0.4 * 1500)
  for (int l = 0; l < L; ++l) {
    const bool served = c.maps[0]->expert_at(l, 5) == 0;
    c.counts[0][l * 3] += served ? 0 : 1000;
    c.counts[1][l * 3 + 2] += served ? 1500 : 0;
    c.counts[0][l * 3 + 1] += 10; c.counts[1][l * 3] += 10; c.counts[1][l * 3 + 1] += 10;
  }
  CHECK(c.round() == L - Distribution::QUEUE_SIZE);
  for (int l = 0; l < L; ++l) CHECK(c.maps[0]->expert_at(l, 5) == 0 && c.held(1, 2, l) == float(100 * l));
}

TEST(manager_second_round_sees_only_new_traffic) {
  Cluster c(2, 4);
  c.counts[0] = {1000, 10, 0};
  c.counts[1] = {10, 10, 0};
  CHECK(c.round() >= 1);
  const int reps = c.maps[0]->redundant_count(0, 0);
  CHECK(reps == 2);
  // no new tokens: deltas are zero, the moving average decays but stays balanced enough; nothing is undone blindly
  CHECK(c.round() >= 0 && c.views_agree());
  CHECK(c.pls[0]->rounds() == 2 && c.maps[0]->redundant_count(0, 0) >= 1);
  for (int e = 0; e < 4; ++e) CHECK(c.maps[0]->redundant_count(0, e) >= 1);
}

TEST(manager_disagreeing_ranks_skip_the_instruction) {
  Cluster c(2, 4);
  c.counts[0] = {1000, 10, 0};
  c.counts[1] = {10, 10, 0};
  c.dists[0]->corrupt_next_handshake();
  std::vector<int> replaced;
  c.round(&replaced);
  CHECK(c.pls[0]->skipped_instructions() >= 1 && c.pls[1]->skipped_instructions() >= 1);
  CHECK(c.held(1, 2) == -1.f && c.maps[1]->expert_at(0, 5) == -1 && c.views_agree());
  // the next round, with honest tuples, goes through
  c.counts[0][0] += 1000;
  CHECK(c.round() >= 1 && c.held(1, 2) == 0.f && c.maps[0]->expert_at(0, 5) == 0);
}

// a transport whose closing barrier of the round waits for the test's signal
class HeldBarrier : public FakeDistribution {
 public:
  using FakeDistribution::FakeDistribution;
  std::atomic<bool> release{false};
  std::atomic<int> at_barrier{0};
  void barrier() override {
    ++at_barrier;
    while (!release.load()) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    FakeDistribution::barrier();
  }
};

TEST(manager_shows_a_round_to_the_inference_thread_only_when_every_rank_has_staged_it) {
  Cluster c(2, 4);
  c.counts[0] = {1000, 10, 0};
  c.counts[1] = {10, 10, 0};
  // rank 1 gets the held transport (it is the receiver of the replica of expert 0)
  auto* held = new HeldBarrier(c.hub, 1, c.ws[1]->expert_bytes());
  c.dists[1].reset(held);
  c.pls[1].reset(new Placement(c.maps[1].get(), c.ws[1].get(), c.acts[1].get(), held, 10, 3600.0));
  std::thread t0([&] { c.pls[0]->run_round(); });
  std::thread t1([&] { c.pls[1]->run_round(); });
  for (int i = 0; i < 2000 && held->at_barrier.load() == 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(1));
  CHECK(held->at_barrier.load() == 1);               // rank 1 has received the expert and stands before the barrier
  // both inference threads look for work now: there is none yet, although the bytes are already in rank 1's staging
  CHECK(c.pls[0]->ready_rounds() == 0 && c.pls[1]->ready_rounds() == 0);
  CHECK(c.pls[0]->do_placement_optimizer() == 0 && c.pls[1]->do_placement_optimizer() == 0);
  CHECK(c.maps[0]->expert_at(0, 5) == -1 && c.maps[0]->selector(0, 0) == 0 && c.held(1, 2) == -1.f);
  held->release = true;
  t0.join();
  t1.join();
  CHECK(c.pls[0]->ready_rounds() == 1 && c.pls[1]->ready_rounds() == 1);
  CHECK(c.pls[0]->do_placement_optimizer() == 0 && c.pls[1]->do_placement_optimizer() == 1);
  CHECK(c.maps[0]->expert_at(0, 5) == 0 && c.maps[1]->selector(0, 0) == 5 && c.held(1, 2) == 0.f && c.views_agree());
}

TEST(manager_random_traffic_keeps_every_rank_consistent) {
  // random clusters and random load, several rounds each: after every round all ranks hold the same placement, every
  // expert has a replica, a slot's bytes are those of the expert the placement names, and every rank's selector points
  // at a position that holds the expert it is asked for
  std::mt19937 rng(1234);
  for (int trial = 0; trial < 12; ++trial) {
    const int W = 2 + (int)(rng() % 3), per = 1 + (int)(rng() % 3), L = 1 + (int)(rng() % 4), E = W * per;
    Cluster c(W, E, L);
    for (int round = 0; round < 5; ++round) {
      for (int r = 0; r < W; ++r)
        for (int l = 0; l < L; ++l)
          for (int s = 0; s < c.S; ++s) {
            const int e = c.maps[0]->expert_at(l, r * c.S + s);
            const bool hot = e >= 0 && (int)(rng() % 4) == 0;
            c.counts[r][l * c.S + s] += e < 0 ? 0 : (hot ? 500 + (int64_t)(rng() % 2000) : (int64_t)(rng() % 60));
          }
      c.round();
      CHECK(c.views_agree());
      for (int l = 0; l < L; ++l) {
        for (int e = 0; e < E; ++e) CHECK(c.maps[0]->redundant_count(l, e) >= 1);
        for (int r = 0; r < W; ++r) {
          for (int s = 0; s < c.S; ++s) {
            const int e = c.maps[0]->expert_at(l, r * c.S + s);
            if (e >= 0) CHECK(c.held(r, s, l) == float(100 * l + e));
          }
          for (int e = 0; e < E; ++e) CHECK(c.maps[r]->expert_at(l, c.maps[r]->selector(l, e)) == e);
        }
      }
      // instructions may be put off (a source that changed in the same round, a full staging ring), but by all ranks alike
      for (int r = 1; r < W; ++r) CHECK(c.pls[r]->skipped_instructions() == c.pls[0]->skipped_instructions());
    }
  }
}

TEST(manager_history_survives_a_restart) {
  std::vector<double> saved;
  {
    Cluster c(2, 4);
    CHECK(c.pls[0]->ema_snapshot().empty());          // nothing collected yet
    c.counts[0] = {400, 10, 0};
    c.counts[1] = {10, 10, 0};
    c.round();
    saved = c.pls[0]->ema_snapshot();
    CHECK(saved.size() == 6 && saved[0] == 400.0);
  }
  Cluster d(2, 4);
  CHECK(!d.pls[0]->restore_ema({1.0, 2.0}));          // wrong shape
  CHECK(d.pls[0]->restore_ema(saved) && d.pls[1]->restore_ema(saved));
  d.counts[0] = {0, 0, 0};
  d.counts[1] = {0, 0, 0};
  d.round();
  CHECK(std::fabs(d.pls[0]->ema_snapshot()[0] - 240.0) < 1e-9);      // 0.6 of the restored value, not a cold start
}

TEST(manager_background_threads_stop_together) {
  Cluster c(2, 4);
  c.counts[0] = {1000, 10, 0};
  c.counts[1] = {10, 10, 0};
  for (auto& p : c.pls) p->start();
  // wait for the first background round, applying on the "inference threads" as the engine would
  for (int i = 0; i < 400 && (c.pls[0]->rounds() < 1 || c.pls[1]->rounds() < 1); ++i) {
    for (auto& p : c.pls) p->do_placement_optimizer();
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
  CHECK(c.pls[0]->rounds() >= 1 && c.pls[1]->rounds() >= 1);
  for (auto& p : c.pls) p->do_placement_optimizer();
  // both ranks ask to stop, one after the other: neither join may hang
  std::thread t([&] { c.pls[1]->stop(); });
  c.pls[0]->stop();
  t.join();
  CHECK(c.views_agree());
}

}  // namespace

int main(int argc, char** argv) {
  set_ut_memcpy_fun();
  const std::string only = argc > 1 ? argv[1] : "";
  int failed = 0, ran = 0;
  for (const auto& c : cases()) {
    if (!only.empty() && only != c.name) continue;
    ++ran;
    try {
      c.fn();
    } catch (const std::exception& e) {
      ++failed;
      fprintf(stderr, "FAILED %s: %s\n", c.name, e.what());
    }
    set_ut_memcpy_fun();                             // a case may have replaced the hooks
  }
  printf("placement units: %d cases, %d checks, %d failed\n", ran, g_checks.load(), failed);
  if (!failed) printf("ALL PASSED\n");
  return failed ? 1 : 0;
}
