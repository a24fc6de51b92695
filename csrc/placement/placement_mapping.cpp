// PlacementMapping, Tensor, ClusterActivation, MoEWeights (see placement_core.h).
#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "placement_core.h"

namespace omni_placement {

// ------------------------------------------------------------------------------------------------ hooks / Tensor
PlacementHooks& hooks() {
  static PlacementHooks h;
  return h;
}
void set_ut_memcpy_fun() {
  auto f = [](void* d, const void* s, size_t n) { std::memcpy(d, s, n); };
  hooks().memcpy_d2d = f;
  hooks().memcpy_h2d = f;
  hooks().memcpy_d2h = f;
}
void unset_ut_memcpy_fun() { hooks() = PlacementHooks(); }

void Tensor::to_host(void* host) const {
  if (!hooks().memcpy_d2h) throw std::runtime_error("no device->host copy hook installed");
  hooks().memcpy_d2h(host, data_, bytes());
}
void Tensor::to_device(const void* host) const {
  if (!hooks().memcpy_h2d) throw std::runtime_error("no host->device copy hook installed");
  hooks().memcpy_h2d(data_, host, bytes());
}

// ------------------------------------------------------------------------------------------------ PlacementMapping
std::vector<int> PlacementMapping::base_pattern(int world, int layers, int experts) {
  std::vector<int> p((size_t)world * layers * experts, 0);
  const int per = experts / world;
  for (int r = 0; r < world; ++r)
    for (int l = 0; l < layers; ++l)
      for (int e = r * per; e < (r + 1) * per; ++e) p[((size_t)r * layers + l) * experts + e] = 1;
  return p;
}

std::vector<int> PlacementMapping::load_text_pattern(const std::string& path, int& world, int& layers, int& experts) {
  // first line: "world layers experts", then world*layers lines of `experts` 0/1 values
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open pattern file " + path);
  in >> world >> layers >> experts;
  std::vector<int> p((size_t)world * layers * experts);
  for (auto& v : p)
    if (!(in >> v)) throw std::runtime_error("pattern file " + path + " is truncated");
  return p;
}

PlacementMapping::PlacementMapping(const std::vector<int>& pattern, int world, int layers, int experts, int rank,
                                   int redundant_per_rank, int ranks_per_host, int32_t* selector)
    : world_(world), layers_(layers), experts_(experts), rank_(rank), ranks_per_host_(std::max(1, ranks_per_host)),
      selector_dev_(selector) {
  if ((size_t)world * layers * experts != pattern.size()) throw std::invalid_argument("pattern has the wrong size");
  if (experts % world != 0) throw std::invalid_argument("experts must divide evenly over the ranks");
  slots_per_rank_ = experts / world + redundant_per_rank;
  pos_to_expert_.assign((size_t)layers * num_positions(), -1);
  deploy_count_.assign((size_t)layers * experts, 0);
  for (int l = 0; l < layers; ++l) {
    for (int r = 0; r < world; ++r) {
      int slot = 0;
      for (int e = 0; e < experts; ++e) {
        if (!pattern[((size_t)r * layers + l) * experts + e]) continue;
        if (slot >= slots_per_rank_)
          throw std::invalid_argument("pattern places more experts on a rank than it has slots");
        pos_to_expert_[(size_t)l * num_positions() + r * slots_per_rank_ + slot] = e;
        ++deploy_count_[(size_t)l * experts + e];
        ++slot;
      }
    }
    for (int e = 0; e < experts; ++e)
      if (deploy_count_[(size_t)l * experts + e] == 0)
        throw std::invalid_argument("pattern leaves expert " + std::to_string(e) + " of layer " + std::to_string(l) +
                                    " without a replica");
  }
  selector_host_.assign((size_t)layers * experts, 0);
  update_selector();
}

std::vector<int> PlacementMapping::positions_of(int layer, int expert) const {
  std::vector<int> out;
  for (int p = 0; p < num_positions(); ++p)
    if (pos_to_expert_[(size_t)layer * num_positions() + p] == expert) out.push_back(p);
  return out;
}

std::vector<int> PlacementMapping::local_slots_of(int layer, int expert) const {
  std::vector<int> out;
  for (int s = 0; s < slots_per_rank_; ++s)
    if (pos_to_expert_[(size_t)layer * num_positions() + rank_ * slots_per_rank_ + s] == expert) out.push_back(s);
  return out;
}

bool PlacementMapping::check_update_is_valid(int layer, int global_pos, int old_expert, int new_expert) const {
  if (layer < 0 || layer >= layers_ || global_pos < 0 || global_pos >= num_positions()) return false;
  if (new_expert < -1 || new_expert >= experts_) return false;
  const int cur = pos_to_expert_[(size_t)layer * num_positions() + global_pos];
  if (cur != old_expert) return false;                                   // ranks disagree about the current state
  if (cur >= 0 && cur != new_expert && deploy_count_[(size_t)layer * experts_ + cur] <= 1) return false;  // last replica
  return true;
}

bool PlacementMapping::update_position(int layer, int global_pos, int old_expert, int new_expert) {
  if (!check_update_is_valid(layer, global_pos, old_expert, new_expert)) return false;
  int& cur = pos_to_expert_[(size_t)layer * num_positions() + global_pos];
  if (cur >= 0) --deploy_count_[(size_t)layer * experts_ + cur];
  cur = new_expert;
  if (new_expert >= 0) ++deploy_count_[(size_t)layer * experts_ + new_expert];
  return true;
}

bool PlacementMapping::apply_batch(const std::vector<std::pair<int, int>>& layer_pos, const std::vector<int>& news) {
  std::vector<int> old(layer_pos.size());
  for (size_t i = 0; i < layer_pos.size(); ++i) {
    const int l = layer_pos[i].first, p = layer_pos[i].second;
    if (l < 0 || l >= layers_ || p < 0 || p >= num_positions() || news[i] < -1 || news[i] >= experts_) return false;
    old[i] = pos_to_expert_[(size_t)l * num_positions() + p];
  }
  auto recount = [&](int l) {
    bool ok = true;
    for (int e = 0; e < experts_; ++e) deploy_count_[(size_t)l * experts_ + e] = 0;
    for (int p = 0; p < num_positions(); ++p) {
      const int e = pos_to_expert_[(size_t)l * num_positions() + p];
      if (e >= 0) ++deploy_count_[(size_t)l * experts_ + e];
    }
    for (int e = 0; e < experts_; ++e) ok = ok && deploy_count_[(size_t)l * experts_ + e] > 0;
    return ok;
  };
  for (size_t i = 0; i < layer_pos.size(); ++i)
    pos_to_expert_[(size_t)layer_pos[i].first * num_positions() + layer_pos[i].second] = news[i];
  bool ok = true;
  for (size_t i = 0; i < layer_pos.size(); ++i) ok = recount(layer_pos[i].first) && ok;
  if (!ok) {
    for (size_t i = layer_pos.size(); i-- > 0;)
      pos_to_expert_[(size_t)layer_pos[i].first * num_positions() + layer_pos[i].second] = old[i];
    for (size_t i = 0; i < layer_pos.size(); ++i) recount(layer_pos[i].first);
  }
  return ok;
}

void PlacementMapping::update_selector_layer(int layer) {
  const int my_host = rank_ / ranks_per_host_;
  for (int e = 0; e < experts_; ++e) {
    std::vector<int> own, same_host, distant;
    for (int p : positions_of(layer, e)) {
      const int r = p / slots_per_rank_;
      if (r == rank_) own.push_back(p);
      else if (r / ranks_per_host_ == my_host) same_host.push_back(p);
      else distant.push_back(p);
    }
    int choice = 0;
    if (!own.empty()) choice = own[0];
    else if (!same_host.empty()) choice = same_host[rank_ % same_host.size()];
    else if (!distant.empty()) choice = distant[rank_ % distant.size()];
    selector_host_[(size_t)layer * experts_ + e] = choice;
  }
}

void PlacementMapping::update_selector() {
  for (int l = 0; l < layers_; ++l) update_selector_layer(l);
  push_selector_to_device();
}

void PlacementMapping::push_selector_to_device() {
  if (selector_dev_ != nullptr && hooks().memcpy_h2d)
    hooks().memcpy_h2d(selector_dev_, selector_host_.data(), selector_host_.size() * sizeof(int32_t));
}

// ------------------------------------------------------------------------------------------------ ClusterActivation
ClusterActivation::ClusterActivation(Tensor counts, int layers, int slots_per_rank, int world, int rank, int window)
    : counts_(counts), layers_(layers), slots_(slots_per_rank), world_(world), rank_(rank), window_(std::max(1, window)) {
  last_.assign((size_t)layers * positions(), 0);
  delta_.assign((size_t)layers * positions(), 0);
}

void ClusterActivation::collect() {
  const size_t n_local = (size_t)layers_ * slots_;
  std::vector<int64_t> local(n_local), all(n_local * world_);
  counts_.to_host(local.data());
  if (world_ > 1) {
    if (!allgather_) throw std::runtime_error("ClusterActivation: no all-gather installed");
    allgather_(local.data(), all.data(), n_local);
  } else {
    all = local;
  }
  // all is [rank][layer][slot]; bookkeeping is [layer][rank*slots + slot]
  std::vector<int64_t> cur((size_t)layers_ * positions());
  for (int r = 0; r < world_; ++r)
    for (int l = 0; l < layers_; ++l)
      for (int s = 0; s < slots_; ++s)
        cur[(size_t)l * positions() + r * slots_ + s] = all[((size_t)r * layers_ + l) * slots_ + s];
  for (size_t i = 0; i < cur.size(); ++i) {
    int64_t d = cur[i] - last_[i];
    if (d < 0) d += kWrap;               // the device counter wrapped
    delta_[i] = first_ ? cur[i] : d;
  }
  first_ = false;
  last_ = cur;
  history_.push_back(delta_);
  if ((int)history_.size() > window_) history_.erase(history_.begin());
}

int64_t ClusterActivation::windowed(int layer, int global_pos) const {
  int64_t s = 0;
  for (const auto& h : history_) s += h[(size_t)layer * positions() + global_pos];
  return s;
}

void ClusterActivation::dump_txt(const std::string& path) const {
  std::ofstream out(path);
  for (int l = 0; l < layers_; ++l) {
    for (int p = 0; p < positions(); ++p) out << (p ? " " : "") << delta_[(size_t)l * positions() + p];
    out << "\n";
  }
}

void ClusterActivation::collect_from_txt(const std::string& path) {
  std::ifstream in(path);
  if (!in) throw std::runtime_error("cannot open activation file " + path);
  for (auto& v : delta_)
    if (!(in >> v)) throw std::runtime_error("activation file " + path + " is truncated");
  for (size_t i = 0; i < delta_.size(); ++i) last_[i] = (last_[i] + delta_[i]) % kWrap;
  first_ = false;
  history_.push_back(delta_);
  if ((int)history_.size() > window_) history_.erase(history_.begin());
}

// ------------------------------------------------------------------------------------------------ MoEWeights
size_t MoEWeights::expert_bytes() const {
  for (const auto& v : w_) {
    if (v.empty()) continue;
    size_t b = 0;
    for (const auto& t : v) b += t.bytes;
    return b;
  }
  return 0;
}

}  // namespace omni_placement
