// GreedyExpertLoadBalancer (dynamic EPLB), ExpertLoadBalancer (static placement), PlacementOptimizer.
// Behaviour follows the reference's dynamic_eplb_greedy.cpp (EMA keep ratio 0.6, REMOVE pass, then SWAP/ADD while
// max/min rank load >= 1.1, at most 32 instructions per layer, stop after two rounds without improvement) and the
// offline pattern generation (redundancy by load-per-replica max-heap, LPT assignment with host interleave).
#include <algorithm>
#include <cmath>
#include <numeric>
#include <queue>
#include <stdexcept>

#include "placement_core.h"

namespace omni_placement {

GreedyExpertLoadBalancer::GreedyExpertLoadBalancer(int layers, int world, int experts, int slots_per_rank,
                                                   int max_redundant_per_expert, double ema_keep, double threshold,
                                                   int max_instructions_per_layer)
    : layers_(layers), world_(world), experts_(experts), slots_(slots_per_rank), max_red_(max_redundant_per_expert),
      keep_(ema_keep), threshold_(threshold), max_instr_(max_instructions_per_layer) {
  ema_.assign((size_t)layers * world * slots_per_rank, 0.0);
}

double GreedyExpertLoadBalancer::imbalance(const std::vector<double>& rl) {
  double mx = 0, mn = 1e300;
  for (double v : rl) { mx = std::max(mx, v); mn = std::min(mn, v); }
  if (mx <= 0) return 1.0;
  return mx / std::max(mn, 1e-9 * mx + 1e-12);
}

std::vector<double> GreedyExpertLoadBalancer::rank_loads(const std::vector<int>& place,
                                                         const std::vector<double>& load) const {
  std::vector<double> rl(world_, 0.0);
  for (int p = 0; p < world_ * slots_; ++p)
    if (place[p] >= 0) rl[p / slots_] += load[p];
  return rl;
}

void GreedyExpertLoadBalancer::optimize_layer(int layer, std::vector<int>& place, std::vector<double>& load,
                                              std::vector<ChangeInstruction>& out) {
  const int P = world_ * slots_;
  auto replicas = [&](int e) { int c = 0; for (int p = 0; p < P; ++p) c += place[p] == e; return c; };
  auto ratio_of = [&]() { return imbalance(rank_loads(place, load)); };
  double ratio = ratio_of();
  if (!(ratio > 1.0) || !std::isfinite(ratio)) return;
  int emitted = 0;

  // ---- REMOVE pass: drop redundant replicas from the hottest rank when that lowers the ratio
  for (int iter = 0; iter < P && emitted < max_instr_; ++iter) {
    auto rl = rank_loads(place, load);
    const double mean = std::accumulate(rl.begin(), rl.end(), 0.0) / world_;
    const int hot = (int)(std::max_element(rl.begin(), rl.end()) - rl.begin());
    if (rl[hot] <= mean) break;
    int best_p = -1;
    double best_ratio = ratio;
    for (int s = 0; s < slots_; ++s) {
      const int p = hot * slots_ + s, e = place[p];
      if (e < 0 || replicas(e) <= 1) continue;
      auto place2 = place;
      auto load2 = load;
      place2[p] = -1;
      const double give = load2[p] / (replicas(e) - 1);
      load2[p] = 0;
      for (int q = 0; q < P; ++q) if (place2[q] == e) load2[q] += give;
      const double r2 = imbalance(rank_loads(place2, load2));
      if (r2 < best_ratio - 1e-12) { best_ratio = r2; best_p = p; }
    }
    if (best_p < 0) break;
    const int e = place[best_p];
    const double give = load[best_p] / (replicas(e) - 1);
    place[best_p] = -1;
    load[best_p] = 0;
    for (int q = 0; q < P; ++q) if (place[q] == e) load[q] += give;
    ChangeInstruction ins;
    ins.layer_idx = layer; ins.type = OperationType::REMOVE;
    ins.source_rank = best_p / slots_; ins.source_expert_id = e; ins.source_global_position = best_p;
    ins.target_rank = best_p / slots_; ins.target_expert_id = -1; ins.target_global_position = best_p;
    ins.prior = emitted;
    out.push_back(ins);
    ++emitted;
    ratio = best_ratio;
  }

  // ---- SWAP / ADD pass
  int no_improve = 0;
  bool fix_high = true;
  while (emitted < max_instr_ && ratio >= threshold_ && no_improve < 2) {
    auto rl = rank_loads(place, load);
    const int hot = (int)(std::max_element(rl.begin(), rl.end()) - rl.begin());
    const int cold = (int)(std::min_element(rl.begin(), rl.end()) - rl.begin());
    double best_ratio = ratio;
    ChangeInstruction best;
    std::vector<int> best_place;
    std::vector<double> best_load;
    // candidate sources: positions of the hot rank (fix_high) or, when fixing the cold rank, positions anywhere that
    // could move onto it
    for (int sp = 0; sp < P; ++sp) {
      const int se = place[sp];
      if (se < 0) continue;
      if (fix_high && sp / slots_ != hot) continue;
      for (int tp = 0; tp < P; ++tp) {
        if (tp / slots_ == sp / slots_) continue;
        if (!fix_high && tp / slots_ != cold) continue;
        const int te = place[tp];
        // SWAP: exchange the two experts when the source is heavier
        if (te >= 0 && te != se && load[sp] > load[tp]) {
          auto p2 = place; auto l2 = load;
          std::swap(p2[sp], p2[tp]);
          std::swap(l2[sp], l2[tp]);
          // the swap must not put two replicas of one expert on one rank
          bool dup = false;
          for (int s = 0; s < slots_ && !dup; ++s) {
            const int a = (tp / slots_) * slots_ + s, b = (sp / slots_) * slots_ + s;
            if (a != tp && p2[a] == se) dup = true;
            if (b != sp && p2[b] == te) dup = true;
          }
          if (!dup) {
            const double r2 = imbalance(rank_loads(p2, l2));
            if (r2 < best_ratio - 1e-12) {
              best_ratio = r2; best_place = p2; best_load = l2;
              best = ChangeInstruction();
              best.layer_idx = layer; best.type = OperationType::SWAP;
              best.source_rank = sp / slots_; best.source_expert_id = se; best.source_global_position = sp;
              best.target_rank = tp / slots_; best.target_expert_id = te; best.target_global_position = tp;
            }
          }
        }
        // ADD: replicate the source expert onto an empty slot or over a redundant replica of another expert
        const bool target_free = te < 0 || (te != se && replicas(te) > 1);
        if (target_free && replicas(se) < 1 + max_red_) {
          bool dup = false;
          for (int s = 0; s < slots_; ++s) if (place[(tp / slots_) * slots_ + s] == se) dup = true;
          if (!dup) {
            auto p2 = place; auto l2 = load;
            if (te >= 0) {   // the evicted replica's load returns to its siblings
              const double give = l2[tp] / (replicas(te) - 1);
              for (int q = 0; q < P; ++q) if (q != tp && p2[q] == te) l2[q] += give;
            }
            const int n_old = replicas(se);
            double tot = 0;
            for (int q = 0; q < P; ++q) if (p2[q] == se) tot += l2[q];
            p2[tp] = se;
            for (int q = 0; q < P; ++q) if (p2[q] == se) l2[q] = tot / (n_old + 1);
            const double r2 = imbalance(rank_loads(p2, l2));
            if (r2 < best_ratio - 1e-12) {
              best_ratio = r2; best_place = p2; best_load = l2;
              best = ChangeInstruction();
              best.layer_idx = layer; best.type = OperationType::ADD;
              best.source_rank = sp / slots_; best.source_expert_id = se; best.source_global_position = sp;
              best.target_rank = tp / slots_; best.target_expert_id = te; best.target_global_position = tp;
            }
          }
        }
      }
    }
    if (best.type == OperationType::EMPTY) {
      ++no_improve;
    } else {
      no_improve = 0;
      place = best_place;
      load = best_load;
      ratio = best_ratio;
      best.prior = emitted;
      out.push_back(best);
      ++emitted;
    }
    fix_high = !fix_high;
  }
}

std::vector<ChangeInstruction> GreedyExpertLoadBalancer::optimize_and_generate_instructions(
    const std::vector<int>& placement, const std::vector<int64_t>& activations) {
  const int P = world_ * slots_;
  if ((int)placement.size() != layers_ * P || activations.size() != placement.size())
    throw std::invalid_argument("placement / activation shape mismatch");
  for (size_t i = 0; i < ema_.size(); ++i)
    ema_[i] = has_ema_ ? keep_ * ema_[i] + (1.0 - keep_) * (double)activations[i] : (double)activations[i];
  has_ema_ = true;
  std::vector<ChangeInstruction> out;
  for (int l = 0; l < layers_; ++l) {
    std::vector<int> place(placement.begin() + (size_t)l * P, placement.begin() + (size_t)(l + 1) * P);
    std::vector<double> load(ema_.begin() + (size_t)l * P, ema_.begin() + (size_t)(l + 1) * P);
    optimize_layer(l, place, load, out);
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ static placement
std::vector<int> ExpertLoadBalancer::generate_constrained_placement(const std::vector<double>& loads,
                                                                    int max_redundant_per_expert) const {
  if ((int)loads.size() != experts_) throw std::invalid_argument("one load per logical expert expected");
  const int total_slots = world_ * slots_;
  int extra = total_slots - experts_;
  if (extra < 0) throw std::invalid_argument("fewer slots than experts");
  std::vector<int> replicas(experts_, 1);
  using Item = std::pair<double, int>;   // load per replica, expert
  std::priority_queue<Item> heap;
  for (int e = 0; e < experts_; ++e) heap.push({loads[e], e});
  while (extra > 0 && !heap.empty()) {
    auto [v, e] = heap.top();
    heap.pop();
    if (replicas[e] >= 1 + max_redundant_per_expert || replicas[e] >= world_) continue;
    ++replicas[e];
    --extra;
    heap.push({loads[e] / replicas[e], e});
  }
  // LPT: heaviest replica first onto the least loaded rank that has a free slot and no replica of that expert;
  // ties prefer a host that holds fewer replicas of the expert (host interleave)
  std::vector<Item> items;
  for (int e = 0; e < experts_; ++e)
    for (int k = 0; k < replicas[e]; ++k) items.push_back({loads[e] / replicas[e], e});
  std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.first > b.first || (a.first == b.first && a.second < b.second); });
  std::vector<int> place(total_slots, -1), used(world_, 0);
  std::vector<double> rl(world_, 0.0);
  for (auto [v, e] : items) {
    int best = -1;
    double best_key = 1e300;
    for (int r = 0; r < world_; ++r) {
      if (used[r] >= slots_) continue;
      bool has = false;
      int host_has = 0;
      for (int q = 0; q < total_slots; ++q)
        if (place[q] == e) { if (q / slots_ == r) has = true; if ((q / slots_) / rph_ == r / rph_) ++host_has; }
      if (has) continue;
      const double key = rl[r] + 1e-9 * host_has;
      if (key < best_key) { best_key = key; best = r; }
    }
    if (best < 0) {   // only ranks that already hold the expert have room: fall back to any free slot
      for (int r = 0; r < world_; ++r) if (used[r] < slots_) { best = r; break; }
    }
    place[best * slots_ + used[best]++] = e;
    rl[best] += v;
  }
  return place;
}

bool ExpertLoadBalancer::validate(const std::vector<int>& placement) const {
  if ((int)placement.size() != world_ * slots_) return false;
  std::vector<int> seen(experts_, 0);
  for (int p = 0; p < (int)placement.size(); ++p) {
    const int e = placement[p];
    if (e < -1 || e >= experts_) return false;
    if (e >= 0) {
      ++seen[e];
      for (int s = 0; s < p % slots_; ++s)
        if (placement[(p / slots_) * slots_ + s] == e) return false;   // two replicas on one rank
    }
  }
  for (int c : seen) if (c == 0) return false;
  return true;
}

std::vector<ChangeInstruction> ExpertLoadBalancer::bucket_balance(int layer, std::vector<int> place,
                                                                  const std::vector<double>& loads, int max_swaps) const {
  std::vector<ChangeInstruction> out;
  auto rank_load = [&](int r) { double s = 0; for (int k = 0; k < slots_; ++k) { int e = place[r * slots_ + k]; if (e >= 0) s += loads[e]; } return s; };
  for (int it = 0; it < max_swaps; ++it) {
    int hot = 0, cold = 0;
    for (int r = 1; r < world_; ++r) { if (rank_load(r) > rank_load(hot)) hot = r; if (rank_load(r) < rank_load(cold)) cold = r; }
    const double gap = rank_load(hot) - rank_load(cold);
    if (gap <= 0) break;
    // the swap that brings the pair closest to equal: move delta = l_a - l_b with 0 < delta < gap, delta ~ gap/2
    int ba = -1, bb = -1;
    double best = gap;
    for (int a = 0; a < slots_; ++a)
      for (int b = 0; b < slots_; ++b) {
        const int ea = place[hot * slots_ + a], eb = place[cold * slots_ + b];
        if (ea < 0 || eb < 0) continue;
        const double delta = loads[ea] - loads[eb];
        if (delta <= 0) continue;
        const double ng = std::fabs(gap - 2 * delta);
        if (ng < best - 1e-12) { best = ng; ba = a; bb = b; }
      }
    if (ba < 0) break;
    ChangeInstruction ins;
    ins.layer_idx = layer; ins.type = OperationType::SWAP; ins.prior = it;
    ins.source_rank = hot; ins.source_global_position = hot * slots_ + ba; ins.source_expert_id = place[hot * slots_ + ba];
    ins.target_rank = cold; ins.target_global_position = cold * slots_ + bb; ins.target_expert_id = place[cold * slots_ + bb];
    std::swap(place[hot * slots_ + ba], place[cold * slots_ + bb]);
    out.push_back(ins);
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ optimizer
PlacementOptimizer::PlacementOptimizer(PlacementMapping* mapping, ClusterActivation* act, int max_redundant_per_expert)
    : mapping_(mapping), act_(act) {
  greedy_.reset(new GreedyExpertLoadBalancer(mapping->layers(), mapping->world(), mapping->experts(),
                                             mapping->slots_per_rank(), max_redundant_per_expert));
}

std::vector<int> PlacementOptimizer::extract_placement() const {
  const int P = mapping_->num_positions();
  std::vector<int> place((size_t)mapping_->layers() * P);
  for (int l = 0; l < mapping_->layers(); ++l)
    for (int p = 0; p < P; ++p) place[(size_t)l * P + p] = mapping_->expert_at(l, p);
  return place;
}

std::vector<int64_t> PlacementOptimizer::extract_activations() const {
  const int P = mapping_->num_positions();
  std::vector<int64_t> a((size_t)mapping_->layers() * P);
  for (int l = 0; l < mapping_->layers(); ++l)
    for (int p = 0; p < P; ++p) a[(size_t)l * P + p] = act_->delta(l, p);
  return a;
}

std::vector<ChangeInstruction> PlacementOptimizer::optimize() {
  return greedy_->optimize_and_generate_instructions(extract_placement(), extract_activations());
}

}  // namespace omni_placement
