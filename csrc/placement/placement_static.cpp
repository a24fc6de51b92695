// Snapshot planner of the static ExpertLoadBalancer: analysis helpers (loads, ratios, validation), the per-layer plan
// (surplus REMOVE, hot-expert ADD, hot/cold SWAP) under a communication limit, wave priorities, and the multi-layer
// entry.  Counterpart of the reference's omni_planner/cpp/expert_load_balancer.cpp (ratio simulation :288-465,
// constrained placement :1121, bucket balance :1311-1490, optimize_and_generate_instructions :1492, transfer :35);
// the algorithm here is an anchored greedy on the simulated max/mean ratio rather than the reference's recursive
// candidate search.
#include <algorithm>
#include <cmath>
#include <numeric>
#include <queue>
#include <set>
#include <stdexcept>

#include "placement_core.h"

namespace omni_placement {

// ------------------------------------------------------------------------------------------------ analysis
std::vector<double> ExpertLoadBalancer::expert_loads(const std::vector<int>& placement,
                                                     const std::vector<int64_t>& activations) const {
  if ((int)placement.size() != positions() || activations.size() != placement.size())
    throw std::invalid_argument("one layer of world * slots positions expected");
  std::vector<double> loads(experts_, 0.0);
  for (int p = 0; p < positions(); ++p) {
    const int e = placement[p];
    if (e < 0) continue;
    if (e >= experts_) throw std::invalid_argument("expert id out of range");
    loads[e] += (double)activations[p];
  }
  return loads;
}

std::vector<int> ExpertLoadBalancer::replica_counts(const std::vector<int>& placement) const {
  std::vector<int> c(experts_, 0);
  for (int e : placement)
    if (e >= 0 && e < experts_) ++c[e];
  return c;
}

std::vector<double> ExpertLoadBalancer::simulated_rank_loads(const std::vector<int>& placement,
                                                             const std::vector<double>& loads) const {
  const auto cnt = replica_counts(placement);
  std::vector<double> rl(world_, 0.0);
  for (int p = 0; p < (int)placement.size(); ++p) {
    const int e = placement[p];
    if (e >= 0 && e < experts_) rl[p / slots_] += loads[e] / cnt[e];
  }
  return rl;
}

static double max_over_mean(const std::vector<double>& rl) {
  double mx = 0, sum = 0;
  for (double v : rl) { mx = std::max(mx, v); sum += v; }
  return sum > 0 ? mx * (double)rl.size() / sum : 1.0;
}

double ExpertLoadBalancer::simulated_ratio(const std::vector<int>& placement, const std::vector<double>& loads) const {
  return max_over_mean(simulated_rank_loads(placement, loads));
}

double ExpertLoadBalancer::measured_ratio(const std::vector<int>& placement, const std::vector<int64_t>& activations) const {
  std::vector<double> rl(world_, 0.0);
  for (int p = 0; p < (int)placement.size(); ++p)
    if (placement[p] >= 0) rl[p / slots_] += (double)activations[p];
  return max_over_mean(rl);
}

int ExpertLoadBalancer::find_position(const std::vector<int>& placement, int rank, int expert) const {
  for (int s = 0; s < slots_; ++s)
    if (placement[rank * slots_ + s] == expert) return rank * slots_ + s;
  return -1;
}

int ExpertLoadBalancer::find_empty(const std::vector<int>& placement, int rank) const { return find_position(placement, rank, -1); }

bool ExpertLoadBalancer::validate_counts(const std::vector<int>& placement, int min_per_rank, int max_per_rank) const {
  if ((int)placement.size() != positions()) return false;
  for (int r = 0; r < world_; ++r) {
    int n = 0;
    for (int s = 0; s < slots_; ++s) n += placement[r * slots_ + s] >= 0;
    if (n < min_per_rank || n > max_per_rank) return false;
  }
  return true;
}

int ExpertLoadBalancer::diff_count(const std::vector<int>& from, const std::vector<int>& to) const {
  int d = 0;
  for (int r = 0; r < world_; ++r) {
    std::set<int> a, b;
    for (int s = 0; s < slots_; ++s) {
      if (from[r * slots_ + s] >= 0) a.insert(from[r * slots_ + s]);
      if (to[r * slots_ + s] >= 0) b.insert(to[r * slots_ + s]);
    }
    for (int e : a) d += !b.count(e);
    for (int e : b) d += !a.count(e);
  }
  return d;
}

bool ExpertLoadBalancer::apply(std::vector<int>& placement, const ChangeInstruction& ins) const {
  const int sp = ins.source_global_position, tp = ins.target_global_position;
  const int P = positions();
  switch (ins.type) {
    case OperationType::REMOVE: {
      if (sp < 0 || sp >= P || placement[sp] != ins.source_expert_id || ins.source_expert_id < 0) return false;
      if (replica_counts(placement)[ins.source_expert_id] < 2) return false;   // never the last replica
      placement[sp] = -1;
      return true;
    }
    case OperationType::ADD: {
      if (sp < 0 || sp >= P || tp < 0 || tp >= P || placement[sp] != ins.source_expert_id || ins.source_expert_id < 0) return false;
      if (placement[tp] != ins.target_expert_id) return false;
      if (find_position(placement, tp / slots_, ins.source_expert_id) >= 0) return false;   // already on that rank
      if (placement[tp] >= 0 && replica_counts(placement)[placement[tp]] < 2) return false; // would orphan the evicted one
      placement[tp] = ins.source_expert_id;
      return true;
    }
    case OperationType::SWAP: {
      if (sp < 0 || sp >= P || tp < 0 || tp >= P || sp / slots_ == tp / slots_) return false;
      if (placement[sp] != ins.source_expert_id || placement[tp] != ins.target_expert_id) return false;
      if (placement[sp] < 0 || placement[tp] < 0) return false;
      if (find_position(placement, tp / slots_, placement[sp]) >= 0 || find_position(placement, sp / slots_, placement[tp]) >= 0)
        return false;
      std::swap(placement[sp], placement[tp]);
      return true;
    }
    default:
      return true;
  }
}

// ------------------------------------------------------------------------------------------------ one layer
namespace {
ChangeInstruction make_ins(int layer, OperationType t, int slots, int sp, int se, int tp, int te) {
  ChangeInstruction i;
  i.layer_idx = layer; i.type = t;
  i.source_rank = sp / slots; i.source_expert_id = se; i.source_global_position = sp;
  i.target_rank = tp / slots; i.target_expert_id = te; i.target_global_position = tp;
  return i;
}
}  // namespace

LayerPlan ExpertLoadBalancer::plan_layer(int layer, const std::vector<int>& placement, const std::vector<int64_t>& activations,
                                         const StaticBalanceOptions& opt) const {
  LayerPlan plan;
  plan.layer = layer;
  plan.placement = placement;
  if (!validate(placement)) throw std::invalid_argument("invalid input placement (expert missing or doubled on a rank)");
  const auto loads = expert_loads(placement, activations);
  plan.ratio_before = plan.ratio_after = simulated_ratio(placement, loads);
  const int limit = opt.diff_limit >= 0 ? opt.diff_limit : 2 * world_;
  const int P = positions();

  // replica targets: every redundant slot goes to the expert with the largest load per replica
  std::vector<int> want(experts_, 1);
  {
    int extra = P - experts_;
    std::priority_queue<std::pair<double, int>> heap;
    for (int e = 0; e < experts_; ++e) heap.push({loads[e], -e});
    while (extra > 0 && !heap.empty()) {
      auto [v, ne] = heap.top();
      heap.pop();
      const int e = -ne;
      if (v <= 0 || want[e] >= 1 + opt.max_redundant_per_expert || want[e] >= world_) continue;
      ++want[e];
      --extra;
      heap.push({loads[e] / want[e], -e});
    }
  }

  std::vector<int> cur = placement;
  std::vector<ChangeInstruction> all;
  std::vector<double> ratio_after;   // simulated ratio after each instruction
  auto emit = [&](const ChangeInstruction& ins) {
    std::vector<int> nxt = cur;
    if (!apply(nxt, ins)) return false;
    cur.swap(nxt);
    all.push_back(ins);
    ratio_after.push_back(simulated_ratio(cur, loads));
    return true;
  };
  const int budget = std::max(limit, 0) * 2 + 8;   // generate somewhat past the limit: the best prefix is chosen below

  // (1) surplus replicas leave the heaviest rank that holds one
  for (bool moved = true; moved && (int)all.size() < budget;) {
    moved = false;
    const auto cnt = replica_counts(cur);
    const auto rl = simulated_rank_loads(cur, loads);
    int be = -1, bp = -1;
    double bl = -1;
    for (int e = 0; e < experts_; ++e) {
      if (cnt[e] <= want[e]) continue;
      for (int r = 0; r < world_; ++r) {
        const int p = find_position(cur, r, e);
        if (p >= 0 && rl[r] > bl) { bl = rl[r]; be = e; bp = p; }
      }
    }
    if (be >= 0) moved = emit(make_ins(layer, OperationType::REMOVE, slots_, bp, be, bp, -1));
  }

  // (2) missing replicas, hottest first, land on the lightest rank with a free slot that lacks the expert; the copy
  // comes from a holder on the same host when there is one
  for (bool moved = true; moved && (int)all.size() < budget;) {
    moved = false;
    const auto cnt = replica_counts(cur);
    int e = -1;
    double hot = -1;
    for (int k = 0; k < experts_; ++k)
      if (cnt[k] < want[k] && loads[k] / cnt[k] > hot) { hot = loads[k] / cnt[k]; e = k; }
    if (e < 0) break;
    const auto rl = simulated_rank_loads(cur, loads);
    int tr = -1;
    for (int r = 0; r < world_; ++r) {
      if (find_empty(cur, r) < 0 || find_position(cur, r, e) >= 0) continue;
      if (tr < 0 || rl[r] < rl[tr]) tr = r;
    }
    if (tr < 0) { want[e] = cnt[e]; moved = true; continue; }   // nowhere to put it: give the slot up
    int sp = -1;
    for (int r = 0; r < world_; ++r) {
      const int p = find_position(cur, r, e);
      if (p < 0) continue;
      if (sp < 0 || (r / rph_ == tr / rph_ && (sp / slots_) / rph_ != tr / rph_)) sp = p;
    }
    moved = emit(make_ins(layer, OperationType::ADD, slots_, sp, e, find_empty(cur, tr), -1));
  }

  // (3) swaps between the heaviest and the lightest rank: the pair whose exchange lowers the ratio most
  for (int it = 0; it < budget && (int)all.size() < budget; ++it) {
    const auto rl = simulated_rank_loads(cur, loads);
    const auto cnt = replica_counts(cur);
    const int hot = (int)(std::max_element(rl.begin(), rl.end()) - rl.begin());
    const double now = max_over_mean(rl);
    double best = now - 1e-9;
    int bs = -1, bt = -1;
    for (int cold = 0; cold < world_; ++cold) {
      if (cold == hot) continue;
      const double gap = rl[hot] - rl[cold];
      if (gap <= 0) continue;
      for (int a = 0; a < slots_; ++a) {
        const int sp = hot * slots_ + a, ea = cur[sp];
        if (ea < 0 || find_position(cur, cold, ea) >= 0) continue;
        for (int b = 0; b < slots_; ++b) {
          const int tp = cold * slots_ + b, eb = cur[tp];
          if (eb < 0 || find_position(cur, hot, eb) >= 0) continue;
          const double delta = loads[ea] / cnt[ea] - loads[eb] / cnt[eb];
          if (delta <= 0 || delta >= gap) continue;
          // rank loads change only on the pair: the new maximum is the larger of the pair and the rest
          double mx = std::max(rl[hot] - delta, rl[cold] + delta);
          for (int r = 0; r < world_; ++r) if (r != hot && r != cold) mx = std::max(mx, rl[r]);
          const double sum = std::accumulate(rl.begin(), rl.end(), 0.0);
          const double ratio = mx * world_ / sum;
          if (ratio < best) { best = ratio; bs = sp; bt = tp; }
        }
      }
    }
    if (bs < 0) break;
    if (!emit(make_ins(layer, OperationType::SWAP, slots_, bs, cur[bs], bt, cur[bt]))) break;
  }

  // cut at the communication limit, then at the best prefix (later instructions that only make it worse are dropped)
  plan.considered = (int)all.size();
  int keep = std::min((int)all.size(), std::max(limit, 0));
  int best_len = 0;
  double best_ratio = plan.ratio_before;
  for (int i = 0; i < keep; ++i)
    if (ratio_after[i] < best_ratio - 1e-12) { best_ratio = ratio_after[i]; best_len = i + 1; }
  if (best_len == 0 || best_ratio >= plan.ratio_before - opt.accept_margin) return plan;
  all.resize(best_len);
  std::vector<int> out = placement;
  for (const auto& ins : all)
    if (!apply(out, ins)) throw std::logic_error("planned instruction does not apply");
  plan.placement = out;
  plan.instructions = all;
  plan.ratio_after = best_ratio;
  plan.accepted = true;
  return plan;
}

// ------------------------------------------------------------------------------------------------ priorities
void ExpertLoadBalancer::assign_priorities(std::vector<ChangeInstruction>& ins) {
  std::map<std::pair<int, int>, int> by_expert, by_pos;   // (layer, id) -> highest prior so far
  for (auto& i : ins) {
    int dep = 0;
    auto look = [&](std::map<std::pair<int, int>, int>& m, int id) {
      if (id < 0) return;
      auto it = m.find({i.layer_idx, id});
      if (it != m.end()) dep = std::max(dep, it->second);
    };
    look(by_expert, i.source_expert_id); look(by_expert, i.target_expert_id);
    look(by_pos, i.source_global_position); look(by_pos, i.target_global_position);
    i.prior = dep + 1;
    auto mark = [&](std::map<std::pair<int, int>, int>& m, int id) { if (id >= 0) m[{i.layer_idx, id}] = i.prior; };
    mark(by_expert, i.source_expert_id); mark(by_expert, i.target_expert_id);
    mark(by_pos, i.source_global_position); mark(by_pos, i.target_global_position);
  }
  std::stable_sort(ins.begin(), ins.end(), [](const ChangeInstruction& a, const ChangeInstruction& b) {
    return a.layer_idx != b.layer_idx ? a.layer_idx < b.layer_idx : a.prior < b.prior;
  });
}

// ------------------------------------------------------------------------------------------------ all layers
std::vector<ChangeInstruction> ExpertLoadBalancer::optimize_and_generate_instructions(
    int layers, const std::vector<int>& placement, const std::vector<int64_t>& activations, const StaticBalanceOptions& opt,
    std::vector<LayerPlan>* plans) const {
  const size_t P = (size_t)positions();
  if (layers <= 0 || placement.size() != (size_t)layers * P || activations.size() != placement.size())
    throw std::invalid_argument("placement / activations must be [layers][world * slots]");
  std::vector<ChangeInstruction> out;
  if (plans) plans->clear();
  for (int l = 0; l < layers; ++l) {
    std::vector<int> pl(placement.begin() + l * P, placement.begin() + (l + 1) * P);
    std::vector<int64_t> ac(activations.begin() + l * P, activations.begin() + (l + 1) * P);
    LayerPlan plan = plan_layer(l, pl, ac, opt);
    out.insert(out.end(), plan.instructions.begin(), plan.instructions.end());
    if (plans) plans->push_back(std::move(plan));
  }
  assign_priorities(out);
  return out;
}

}  // namespace omni_placement
