// PlacementMapping, Tensor, ClusterActivation, MoEWeights (see placement_core.h).
#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstring>
#include <thread>

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

// Layout of the segment: header {magic, ranks_done, expert_bytes, layers, experts}, one "present" byte per
// (layer, expert), then the experts back to back (each the concatenation of its tensors, 256-byte aligned).
namespace {
struct ReplicaHeader {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> ranks_done;
  uint64_t expert_bytes;
  uint32_t layers, experts;
};
constexpr uint32_t kReplicaMagic = 0x4f4d4e49u;   // set last by the creator: attachers wait for it
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
}  // namespace

MoEWeights::~MoEWeights() { close_shared_memory(false); }

bool MoEWeights::init_shared_memory(const std::string& name, int experts, int ranks_on_host) {
  const size_t eb = align_up(expert_bytes(), 256);
  if (eb == 0 || experts <= 0 || ranks_on_host <= 0 || shm_ != nullptr) return false;
  const size_t flags_off = align_up(sizeof(ReplicaHeader), 64);
  const size_t data_off = align_up(flags_off + (size_t)layers_ * experts, 4096);
  const size_t total = data_off + (size_t)layers_ * experts * eb;
  bool creator = true;
  int fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0 && errno == EEXIST) { creator = false; fd = shm_open(name.c_str(), O_RDWR, 0600); }
  if (fd < 0) return false;
  if (creator && ftruncate(fd, (off_t)total) != 0) { close(fd); shm_unlink(name.c_str()); return false; }
  if (!creator) {   // the creator may not have sized the segment yet
    struct stat st;
    for (int i = 0; i < 2000; ++i) {
      if (fstat(fd, &st) == 0 && (size_t)st.st_size >= total) break;
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    if (fstat(fd, &st) != 0 || (size_t)st.st_size < total) { close(fd); return false; }
  }
  void* p = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return false;
  auto* h = reinterpret_cast<ReplicaHeader*>(p);
  if (creator) {
    h->ranks_done.store(0);
    h->expert_bytes = eb;
    h->layers = (uint32_t)layers_;
    h->experts = (uint32_t)experts;
    std::memset((unsigned char*)p + flags_off, 0, (size_t)layers_ * experts);
    h->magic.store(kReplicaMagic, std::memory_order_release);
  } else {
    for (int i = 0; i < 2000 && h->magic.load(std::memory_order_acquire) != kReplicaMagic; ++i)
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
    if (h->magic.load(std::memory_order_acquire) != kReplicaMagic || h->expert_bytes != eb || h->layers != (uint32_t)layers_ ||
        h->experts != (uint32_t)experts) {
      munmap(p, total);
      return false;      // a segment of another deployment under the same name
    }
  }
  shm_ = (unsigned char*)p;
  shm_bytes_ = total;
  shm_data_off_ = data_off;
  shm_experts_ = experts;
  shm_ranks_ = ranks_on_host;
  shm_name_ = name;
  return true;
}

unsigned char* MoEWeights::replica_ptr(int layer, int expert) const {
  const size_t eb = reinterpret_cast<const ReplicaHeader*>(shm_)->expert_bytes;
  return shm_ + shm_data_off_ + ((size_t)layer * shm_experts_ + expert) * eb;
}

void MoEWeights::replicate_to_shared_memory(const PlacementMapping& mapping) {
  if (shm_ == nullptr) return;
  unsigned char* flags = shm_ + align_up(sizeof(ReplicaHeader), 64);
  const int base = mapping.rank() * slots_;
  for (int l = 0; l < layers_; ++l)
    for (int s = 0; s < slots_; ++s) {
      const int e = mapping.expert_at(l, base + s);
      if (e < 0 || e >= shm_experts_) continue;
      unsigned char* flag = &flags[(size_t)l * shm_experts_ + e];
      unsigned char expected = 0;
      // a replica of it on this host already wrote (or writes) it
      if (!__atomic_compare_exchange_n(flag, &expected, (unsigned char)1, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) continue;
      unsigned char* dst = replica_ptr(l, e);
      size_t off = 0;
      for (const auto& t : tensors(l, s)) { hooks().memcpy_d2h(dst + off, t.ptr, t.bytes); off += t.bytes; }
      __atomic_store_n(flag, (unsigned char)2, __ATOMIC_RELEASE);    // 2 = content complete
    }
  reinterpret_cast<ReplicaHeader*>(shm_)->ranks_done.fetch_add(1, std::memory_order_acq_rel);
}

bool MoEWeights::replica_complete() const {
  return shm_ != nullptr && (int)reinterpret_cast<const ReplicaHeader*>(shm_)->ranks_done.load(std::memory_order_acquire) >= shm_ranks_;
}

bool MoEWeights::replica_has(int layer, int expert) const {
  if (shm_ == nullptr || layer < 0 || layer >= layers_ || expert < 0 || expert >= shm_experts_) return false;
  const unsigned char* flags = shm_ + align_up(sizeof(ReplicaHeader), 64);
  return __atomic_load_n(&flags[(size_t)layer * shm_experts_ + expert], __ATOMIC_ACQUIRE) == 2;
}

bool MoEWeights::replace_from_shared_memory(int layer, int expert, int slot) const {
  if (!replica_has(layer, expert) || slot < 0 || slot >= slots_) return false;
  const unsigned char* src = replica_ptr(layer, expert);
  size_t off = 0;
  for (const auto& t : tensors(layer, slot)) { hooks().memcpy_h2d(t.ptr, src + off, t.bytes); off += t.bytes; }
  return true;
}

void MoEWeights::close_shared_memory(bool unlink) {
  if (shm_ != nullptr) munmap(shm_, shm_bytes_);
  shm_ = nullptr;
  if (unlink && !shm_name_.empty()) shm_unlink(shm_name_.c_str());
  if (unlink) shm_name_.clear();
}

}  // namespace omni_placement
