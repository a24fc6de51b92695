// Distribution transports, the Placement manager and the C API used by the Python binding.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <stdexcept>

#include "placement_core.h"

namespace omni_placement {

// ------------------------------------------------------------------------------------------------ FakeHub
// Shared state of an in-process "cluster": every rank is a thread.  Collectives are generation-counted
// rendezvous; point-to-point messages go through per-(src,dst) mailboxes.
class FakeHub {
 public:
  explicit FakeHub(int world) : world_(world), slots_(world), mail_(world * world) {}
  int world() const { return world_; }

  void allgather(int rank, const void* send, void* recv, size_t bytes) {
    std::unique_lock<std::mutex> lk(mu_);
    const long gen = gen_;
    if (buf_.size() != bytes * world_) buf_.assign(bytes * world_, 0);
    std::memcpy(buf_.data() + bytes * rank, send, bytes);
    if (++arrived_ == world_) {
      result_ = buf_;
      arrived_ = 0;
      ++gen_;
      cv_.notify_all();
    } else {
      cv_.wait(lk, [&] { return gen_ != gen; });
    }
    std::memcpy(recv, result_.data(), bytes * world_);
    // second phase so that nobody overwrites result_ while a slow rank still copies it out
    const long gen2 = gen2_;
    if (++left_ == world_) { left_ = 0; ++gen2_; cv_.notify_all(); } else { cv_.wait(lk, [&] { return gen2_ != gen2; }); }
  }

  void send(int src, int dst, std::vector<unsigned char> data) {
    std::unique_lock<std::mutex> lk(mu_);
    mail_[src * world_ + dst].push_back(std::move(data));
    cv_.notify_all();
  }
  std::vector<unsigned char> recv(int src, int dst) {
    std::unique_lock<std::mutex> lk(mu_);
    auto& q = mail_[src * world_ + dst];
    cv_.wait(lk, [&] { return !q.empty(); });
    auto d = std::move(q.front());
    q.erase(q.begin());
    return d;
  }

 private:
  int world_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<int> slots_;
  std::vector<std::vector<std::vector<unsigned char>>> mail_;
  std::vector<unsigned char> buf_, result_;
  int arrived_ = 0, left_ = 0;
  long gen_ = 0, gen2_ = 0;
};

std::shared_ptr<FakeHub> make_fake_hub(int world) { return std::make_shared<FakeHub>(world); }

static std::vector<unsigned char> pack_expert(const std::vector<ExpertTensor>& ts) {
  size_t tot = 0;
  for (auto& t : ts) tot += t.bytes;
  std::vector<unsigned char> out(tot);
  size_t off = 0;
  for (auto& t : ts) {
    hooks().memcpy_d2h(out.data() + off, t.ptr, t.bytes);
    off += t.bytes;
  }
  return out;
}

FakeDistribution::FakeDistribution(std::shared_ptr<FakeHub> hub, int rank, size_t expert_bytes)
    : hub_(std::move(hub)), rank_(rank), stages_(QUEUE_SIZE, std::vector<unsigned char>(expert_bytes)) {}
FakeDistribution::~FakeDistribution() = default;
int FakeDistribution::world() const { return hub_->world(); }
void FakeDistribution::allgather_i64(const int64_t* send, int64_t* recv, size_t count) {
  hub_->allgather(rank_, send, recv, count * sizeof(int64_t));
}
void FakeDistribution::allgather_handshake(const HandshakeTuple& mine, std::vector<HandshakeTuple>& all) {
  HandshakeTuple m = mine;
  if (corrupt_) { m.expert_id += 1000; corrupt_ = false; }
  all.resize(world());
  hub_->allgather(rank_, &m, all.data(), sizeof(HandshakeTuple));
}
void FakeDistribution::swap(int peer, const std::vector<ExpertTensor>& send, int stage) {
  ++transfers_;
  hub_->send(rank_, peer, pack_expert(send));
  auto d = hub_->recv(peer, rank_);
  std::memcpy(stages_[stage].data(), d.data(), std::min(d.size(), stages_[stage].size()));
}
void FakeDistribution::recv_only(int peer, int stage, size_t) {
  ++transfers_;
  auto d = hub_->recv(peer, rank_);
  std::memcpy(stages_[stage].data(), d.data(), std::min(d.size(), stages_[stage].size()));
}
void FakeDistribution::send_only(int peer, const std::vector<ExpertTensor>& send) {
  ++transfers_;
  hub_->send(rank_, peer, pack_expert(send));
}
void FakeDistribution::barrier() {
  int64_t x = 0;
  std::vector<int64_t> all(world());
  allgather_i64(&x, all.data(), 1);
}

CallbackDistribution::CallbackDistribution(DistributionCallbacks cb, size_t expert_bytes)
    : cb_(std::move(cb)), stages_(QUEUE_SIZE, std::vector<unsigned char>(expert_bytes)) {}
void CallbackDistribution::allgather_handshake(const HandshakeTuple& mine, std::vector<HandshakeTuple>& all) {
  int64_t s[4] = {mine.t_rank, mine.position_offset, mine.expert_id, mine.replica_ok};
  std::vector<int64_t> r(4 * (size_t)cb_.world);
  cb_.allgather_i64(s, r.data(), 4);
  all.resize(cb_.world);
  for (int i = 0; i < cb_.world; ++i) all[i] = {(int)r[4 * i], (int)r[4 * i + 1], (int)r[4 * i + 2], (int)r[4 * i + 3]};
}
CallbackDistribution::CallbackDistribution(DistributionCallbacks cb, size_t expert_bytes, void* device_send_buf,
                                           void* const* device_stages)
    : cb_(std::move(cb)), device_send_(device_send_buf), device_stages_(device_stages, device_stages + QUEUE_SIZE) {
  (void)expert_bytes;
}
size_t CallbackDistribution::pack_device(const std::vector<ExpertTensor>& ts) {
  size_t off = 0;
  for (auto& t : ts) {
    hooks().memcpy_d2d((unsigned char*)device_send_ + off, t.ptr, t.bytes);
    off += t.bytes;
  }
  return off;
}
void CallbackDistribution::swap(int peer, const std::vector<ExpertTensor>& send, int stage) {
  if (device_send_) {
    const size_t n = pack_device(send);
    cb_.sendrecv(peer, device_send_, device_stages_[stage], n);
    return;
  }
  pack_ = pack_expert(send);
  cb_.sendrecv(peer, pack_.data(), stages_[stage].data(), pack_.size());
}
void CallbackDistribution::recv_only(int peer, int stage, size_t bytes) {
  cb_.sendrecv(peer, nullptr, staging(stage), bytes);
}
void CallbackDistribution::send_only(int peer, const std::vector<ExpertTensor>& send) {
  if (device_send_) {
    const size_t n = pack_device(send);
    cb_.sendrecv(peer, device_send_, nullptr, n);
    return;
  }
  pack_ = pack_expert(send);
  cb_.sendrecv(peer, pack_.data(), nullptr, pack_.size());
}

// ------------------------------------------------------------------------------------------------ Placement
Placement::Placement(PlacementMapping* mapping, MoEWeights* weights, ClusterActivation* act, Distribution* dist,
                     int max_redundant_per_expert, double period_s)
    : mapping_(mapping), weights_(weights), act_(act), dist_(dist), period_s_(period_s) {
  optimizer_.reset(new PlacementOptimizer(mapping, act, max_redundant_per_expert));
  if (dist_ != nullptr)
    act_->set_allgather([this](const int64_t* s, int64_t* r, size_t n) { dist_->allgather_i64(s, r, n); });
}

Placement::~Placement() { stop(); }

void Placement::start() {
  should_stop_ = false;
  thread_ = std::thread([this] { loop(); });
}

void Placement::stop() {
  should_stop_ = true;
  cv_.notify_all();
  if (thread_.joinable()) thread_.join();
}

void Placement::loop() {
  // wait until the expert tensors are registered
  while (!should_stop_ && !weights_->is_initialized()) std::this_thread::sleep_for(std::chrono::milliseconds(50));
  while (true) {
    {
      // the previous round must have been applied by the inference thread before new data is staged
      std::unique_lock<std::mutex> lk(mu_);
      cv_.wait(lk, [&] { return should_stop_ || pending_.empty(); });   // (staged_ is empty between rounds)
    }
    // The threads of all ranks leave together: a round is a sequence of collectives, so a thread that simply
    // returned when its own rank asked it to stop would leave the others blocked in the next one (and their stop()
    // blocked in join).  Every round therefore starts by exchanging "do I want to stop"; if anybody does, all do.
    int64_t mine = should_stop_ ? 1 : 0;
    std::vector<int64_t> all((size_t)dist_->world(), 0);
    try {
      dist_->allgather_i64(&mine, all.data(), 1);
    } catch (const std::exception&) {
      break;
    }
    bool stop = false;
    for (int64_t v : all) stop = stop || v != 0;
    if (stop) break;
    try {
      run_round();
    } catch (const std::exception&) {
      ++skipped_;
    }
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait_for(lk, std::chrono::duration<double>(period_s_), [&] { return should_stop_.load(); });
  }
}

std::vector<ChangeInstruction> Placement::last_instructions() const { return last_; }

std::vector<double> Placement::ema_snapshot() {
  std::lock_guard<std::mutex> lk(ema_mu_);
  return optimizer_->balancer().has_ema() ? optimizer_->balancer().ema_loads() : std::vector<double>();
}

bool Placement::restore_ema(const std::vector<double>& ema) {
  std::lock_guard<std::mutex> lk(ema_mu_);
  return optimizer_->balancer().set_ema(ema);
}

int Placement::run_round() {
  act_->collect();
  std::vector<ChangeInstruction> instr;
  {
    std::lock_guard<std::mutex> lk(ema_mu_);
    instr = optimizer_->optimize();
  }
  last_ = instr;
  {
    std::lock_guard<std::mutex> lk(mu_);
    staged_.clear();                                      // leftovers of a round that ended in an exception
  }
  int done = 0;
  stage_used_.assign((size_t)(dist_ != nullptr ? dist_->world() : mapping_->world()), 0);
  round_touched_.clear();
  for (const auto& ins : instr) {
    // Every rank must leave this loop at the same instruction (each one starts with a collective), so the test is on
    // state that is identical everywhere: the staging buffers taken so far on the ranks that would receive.  (The stop
    // flag is not: a rank asked to stop finishes the round; the threads agree on stopping at the start of the next.)
    bool full = false;
    if (ins.type == OperationType::ADD || ins.type == OperationType::SWAP) {
      full = stage_used_[ins.target_rank] >= Distribution::QUEUE_SIZE;
      if (ins.type == OperationType::SWAP) full = full || stage_used_[ins.source_rank] >= Distribution::QUEUE_SIZE;
    }
    if (full) break;                                      // a staging ring is full: the rest waits for the next round
    if (execute(ins)) ++done; else ++skipped_;
  }
  if (dist_ != nullptr) dist_->barrier();                 // every rank has finished staging this round
  {
    // Only now may the inference thread see the round: before the barrier another rank could still be waiting for
    // bytes this round sends it, and a rank that applied (and re-routed tokens to) a replica whose holder has not
    // received it yet would read an empty slot.  The apply step itself is agreed between the ranks by the caller
    // (ready_rounds() of every rank, see do_placement_optimizer).
    std::lock_guard<std::mutex> lk(mu_);
    pending_.insert(pending_.end(), staged_.begin(), staged_.end());
    staged_.clear();
    ++ready_rounds_;
  }
  ++rounds_;
  return done;
}

bool Placement::execute(const ChangeInstruction& ins) {
  const int S = mapping_->slots_per_rank();
  const int me = dist_ != nullptr ? dist_->rank() : mapping_->rank();
  // 1. consistency handshake: every rank reports the instruction it is about to execute
  // the host replica is used for this instruction only if every rank can (same decision everywhere): the receiving
  // rank must find the expert in its host's replica
  const bool need_data = ins.type == OperationType::ADD || ins.type == OperationType::SWAP;
  int replica_ok = 0;
  if (need_data && weights_->replica_enabled() && weights_->replica_complete()) {
    replica_ok = 1;
    if (me == ins.target_rank && !weights_->replica_has(ins.layer_idx, ins.source_expert_id)) replica_ok = 0;
    if (ins.type == OperationType::SWAP && me == ins.source_rank && !weights_->replica_has(ins.layer_idx, ins.target_expert_id)) replica_ok = 0;
  }
  HandshakeTuple mine{ins.target_rank, ins.target_global_position % S, ins.source_expert_id, replica_ok};
  if (dist_ != nullptr) {
    std::vector<HandshakeTuple> all;
    dist_->allgather_handshake(mine, all);
    for (const auto& h : all) {
      if (h.t_rank != mine.t_rank || h.position_offset != mine.position_offset || h.expert_id != mine.expert_id)
        return false;                                     // ranks disagree: skip, nothing was transferred
      if (!h.replica_ok) replica_ok = 0;
    }
  }
  // 2. validity against the current mapping (same answer on every rank)
  const int tp = ins.target_global_position, sp = ins.source_global_position;
  switch (ins.type) {
    case OperationType::REMOVE:
      if (!mapping_->check_update_is_valid(ins.layer_idx, sp, ins.source_expert_id, -1)) return false;
      break;
    case OperationType::ADD:
      if (!mapping_->check_update_is_valid(ins.layer_idx, tp, ins.target_expert_id, ins.source_expert_id)) return false;
      break;
    case OperationType::SWAP:
      if (mapping_->expert_at(ins.layer_idx, sp) != ins.source_expert_id ||
          mapping_->expert_at(ins.layer_idx, tp) != ins.target_expert_id) return false;
      break;
    default:
      return false;
  }
  // 3. data movement into the staging ring (only the ranks involved)
  std::lock_guard<std::mutex> lk(mu_);
  if (ins.type == OperationType::REMOVE) {
    staged_.push_back({ins.layer_idx, sp % S, -1, -1, sp, ins.source_expert_id});
    round_touched_.insert({ins.layer_idx, sp});
    return true;
  }
  // A position changed earlier in this round still holds its old bytes (the new ones wait in a staging buffer until
  // the inference thread applies them), so it cannot be the source of a copy.  A replica of the same expert that is
  // settled serves instead (same choice on every rank: the mappings are identical); without one the instruction
  // waits for a later round.  A swap needs both of its positions settled.
  const auto touched = [&](int pos) { return round_touched_.count({ins.layer_idx, pos}) != 0; };
  if (ins.type == OperationType::SWAP && (touched(sp) || touched(tp))) return false;
  if (touched(tp)) return false;
  int src_pos = sp;
  if (ins.type == OperationType::ADD && (touched(sp) || mapping_->expert_at(ins.layer_idx, sp) != ins.source_expert_id)) {
    src_pos = -1;
    for (int p : mapping_->positions_of(ins.layer_idx, ins.source_expert_id))
      if (!touched(p)) { src_pos = p; break; }
    if (src_pos < 0) return false;
  }
  const int src_rank = ins.type == OperationType::ADD ? src_pos / S : ins.source_rank;
  round_touched_.insert({ins.layer_idx, tp});
  if (ins.type == OperationType::SWAP) round_touched_.insert({ins.layer_idx, sp});
  const bool i_am_src = me == src_rank, i_am_dst = me == ins.target_rank;
  if (replica_ok) {
    // replacement from the host replica: nothing travels between ranks and no staging buffer is taken; the rank
    // that receives an expert copies it host -> device when the change is applied between two steps
    if (ins.type == OperationType::SWAP) {
      staged_.push_back({ins.layer_idx, sp % S, -1, ins.target_expert_id, sp, ins.source_expert_id, i_am_src});
      staged_.push_back({ins.layer_idx, tp % S, -1, ins.source_expert_id, tp, ins.target_expert_id, i_am_dst});
    } else {
      staged_.push_back({ins.layer_idx, tp % S, -1, ins.source_expert_id, tp, ins.target_expert_id, i_am_dst});
    }
    return true;
  }
  int stage = -1;
  if (dist_ != nullptr && (i_am_src || i_am_dst)) {
    stage = stage_used_[me];
    if (ins.type == OperationType::SWAP) {
      const int my_pos = i_am_src ? sp : tp, peer = i_am_src ? ins.target_rank : ins.source_rank;
      dist_->swap(peer, weights_->tensors(ins.layer_idx, my_pos % S), stage);
    } else if (i_am_src && i_am_dst) {
      stage = -1;                                         // cannot happen for a valid plan (one replica per rank)
    } else if (i_am_src) {
      dist_->send_only(ins.target_rank, weights_->tensors(ins.layer_idx, src_pos % S));
      stage = -1;
    } else {
      dist_->recv_only(src_rank, stage, weights_->expert_bytes());
    }
  }
  // staging buffers taken by this instruction, counted for every rank (all ranks keep the same table)
  if (dist_ != nullptr) {
    ++stage_used_[ins.target_rank];
    if (ins.type == OperationType::SWAP) ++stage_used_[ins.source_rank];
  }
  // every rank records the mapping change; only the receivers carry a staging buffer
  if (ins.type == OperationType::SWAP) {
    staged_.push_back({ins.layer_idx, sp % S, i_am_src ? stage : -1, ins.target_expert_id, sp, ins.source_expert_id});
    staged_.push_back({ins.layer_idx, tp % S, i_am_dst ? stage : -1, ins.source_expert_id, tp, ins.target_expert_id});
  } else {
    staged_.push_back({ins.layer_idx, tp % S, i_am_dst ? stage : -1, ins.source_expert_id, tp, ins.target_expert_id});
  }
  return true;
}

int Placement::do_placement_optimizer() {
  std::vector<PendingApply> todo;
  {
    std::lock_guard<std::mutex> lk(mu_);
    todo.swap(pending_);
  }
  if (todo.empty()) return 0;
  int replaced = 0;
  const int S = mapping_->slots_per_rank();
  // SWAP is recorded as two entries whose intermediate state would fail the "last replica" check: apply swaps as
  // a pair by clearing validity through a temporary empty position
  for (const auto& a : todo) {
    const bool local = a.global_pos / S == (dist_ != nullptr ? dist_->rank() : mapping_->rank());
    if (local && a.from_replica) {
      if (weights_->replace_from_shared_memory(a.layer, a.new_expert, a.slot)) ++replaced;
    } else if (local && a.stage >= 0) {
      size_t off = 0;
      const unsigned char* src = (const unsigned char*)dist_->staging(a.stage);
      const bool dev = dist_->staging_on_device();
      for (const auto& t : weights_->tensors(a.layer, a.slot)) {
        if (dev) hooks().memcpy_d2d(t.ptr, src + off, t.bytes);
        else hooks().memcpy_h2d(t.ptr, src + off, t.bytes);
        off += t.bytes;
      }
      ++replaced;
    }
  }
  // mapping: a batch (both halves of a swap, a chain of adds) is applied as a whole and rolled back as a whole if
  // it would leave an expert without a replica - the old selector then stays in force
  std::vector<std::pair<int, int>> changes;   // (layer, global_pos) -> new expert, in order
  std::vector<int> news;
  for (const auto& a : todo) { changes.push_back({a.layer, a.global_pos}); news.push_back(a.new_expert); }
  if (!mapping_->apply_batch(changes, news)) ++skipped_;
  mapping_->update_selector();
  cv_.notify_all();
  return replaced;
}

}  // namespace omni_placement

// ------------------------------------------------------------------------------------------------ C API (ctypes)
using namespace omni_placement;
extern "C" {

typedef void (*omni_copy_fn)(void* dst, const void* src, unsigned long long bytes);
typedef void (*omni_allgather_fn)(const long long* send, long long* recv, unsigned long long count);
typedef void (*omni_sendrecv_fn)(int peer, const void* send, void* recv, unsigned long long bytes);
typedef void (*omni_barrier_fn)();

void omni_pl_set_copy_hooks(omni_copy_fn d2d, omni_copy_fn h2d, omni_copy_fn d2h) {
  hooks().memcpy_d2d = [d2d](void* d, const void* s, size_t n) { d2d(d, s, n); };
  hooks().memcpy_h2d = [h2d](void* d, const void* s, size_t n) { h2d(d, s, n); };
  hooks().memcpy_d2h = [d2h](void* d, const void* s, size_t n) { d2h(d, s, n); };
}
void omni_pl_set_ut_memcpy() { set_ut_memcpy_fun(); }
void omni_pl_unset_ut_memcpy() { unset_ut_memcpy_fun(); }

void* omni_pl_mapping_create(const int* pattern, int world, int layers, int experts, int rank, int redundant_per_rank,
                             int ranks_per_host, int* selector) {
  try {
    std::vector<int> p(pattern, pattern + (size_t)world * layers * experts);
    return new PlacementMapping(p, world, layers, experts, rank, redundant_per_rank, ranks_per_host, selector);
  } catch (const std::exception& e) {
    fprintf(stderr, "omni_placement: %s\n", e.what());
    return nullptr;
  }
}
void omni_pl_mapping_destroy(void* m) { delete (PlacementMapping*)m; }
int omni_pl_mapping_slots_per_rank(void* m) { return ((PlacementMapping*)m)->slots_per_rank(); }
int omni_pl_mapping_expert_at(void* m, int layer, int pos) { return ((PlacementMapping*)m)->expert_at(layer, pos); }
int omni_pl_mapping_redundant_count(void* m, int layer, int e) { return ((PlacementMapping*)m)->redundant_count(layer, e); }
int omni_pl_mapping_selector(void* m, int layer, int e) { return ((PlacementMapping*)m)->selector(layer, e); }
void omni_pl_mapping_copy_selector(void* m, int* out) {
  auto& s = ((PlacementMapping*)m)->selector_host();
  memcpy(out, s.data(), s.size() * sizeof(int));
}
int omni_pl_mapping_update(void* m, int layer, int pos, int old_e, int new_e) {
  auto* mp = (PlacementMapping*)m;
  const bool ok = mp->update_position(layer, pos, old_e, new_e);
  if (ok) mp->update_selector();
  return ok ? 1 : 0;
}

void* omni_pl_weights_create(int layers, int slots) { return new MoEWeights(layers, slots); }
void omni_pl_weights_destroy(void* w) { delete (MoEWeights*)w; }
void omni_pl_weights_add(void* w, int layer, int slot, void* ptr, unsigned long long bytes) {
  ((MoEWeights*)w)->add_tensor(layer, slot, ptr, bytes);
}
void omni_pl_weights_set_initialized(void* w) { ((MoEWeights*)w)->set_initialized(); }
unsigned long long omni_pl_weights_expert_bytes(void* w) { return ((MoEWeights*)w)->expert_bytes(); }

void* omni_pl_activation_create(void* counts, int layers, int slots, int world, int rank, int window) {
  return new ClusterActivation(Tensor(counts, (size_t)layers * slots, 8, "activation"), layers, slots, world, rank, window);
}
void omni_pl_activation_destroy(void* a) { delete (ClusterActivation*)a; }
int omni_pl_activation_collect_from_txt(void* a, const char* path) {
  try { ((ClusterActivation*)a)->collect_from_txt(path); return 0; } catch (const std::exception&) { return -1; }
}
void omni_pl_activation_dump(void* a, const char* path) { ((ClusterActivation*)a)->dump_txt(path); }
long long omni_pl_activation_delta(void* a, int layer, int pos) { return ((ClusterActivation*)a)->delta(layer, pos); }

void* omni_pl_distribution_create(int rank, int world, unsigned long long expert_bytes, omni_allgather_fn ag,
                                  omni_sendrecv_fn sr, omni_barrier_fn bar) {
  DistributionCallbacks cb;
  cb.rank = rank; cb.world = world;
  cb.allgather_i64 = [ag](const int64_t* s, int64_t* r, size_t n) { ag((const long long*)s, (long long*)r, n); };
  cb.sendrecv = [sr](int p, const void* s, void* r, size_t n) { sr(p, s, r, n); };
  cb.barrier = [bar]() { if (bar) bar(); };
  return new CallbackDistribution(cb, expert_bytes);
}
void* omni_pl_distribution_create_device(int rank, int world, unsigned long long expert_bytes, omni_allgather_fn ag,
                                         omni_sendrecv_fn sr, omni_barrier_fn bar, void* device_send_buf,
                                         void* const* device_stages) {
  DistributionCallbacks cb;
  cb.rank = rank; cb.world = world;
  cb.allgather_i64 = [ag](const int64_t* s, int64_t* r, size_t n) { ag((const long long*)s, (long long*)r, n); };
  cb.sendrecv = [sr](int p, const void* s, void* r, size_t n) { sr(p, s, r, n); };
  cb.barrier = [bar]() { if (bar) bar(); };
  return new CallbackDistribution(cb, expert_bytes, device_send_buf, device_stages);
}
void omni_pl_distribution_destroy(void* d) { delete (Distribution*)d; }

void* omni_pl_placement_create(void* mapping, void* weights, void* act, void* dist, int max_red, double period_s) {
  return new Placement((PlacementMapping*)mapping, (MoEWeights*)weights, (ClusterActivation*)act, (Distribution*)dist,
                       max_red, period_s);
}
void omni_pl_placement_destroy(void* p) { delete (Placement*)p; }
void omni_pl_placement_start(void* p) { ((Placement*)p)->start(); }
void omni_pl_placement_stop(void* p) { ((Placement*)p)->stop(); }
int omni_pl_placement_run_round(void* p) {
  try { return ((Placement*)p)->run_round(); } catch (const std::exception& e) { fprintf(stderr, "omni_placement: %s\n", e.what()); return -1; }
}
int omni_pl_do_placement_optimizer(void* p) { return ((Placement*)p)->do_placement_optimizer(); }
int omni_pl_placement_rounds(void* p) { return ((Placement*)p)->rounds(); }
int omni_pl_placement_ready_rounds(void* p) { return ((Placement*)p)->ready_rounds(); }
int omni_pl_placement_skipped(void* p) { return ((Placement*)p)->skipped_instructions(); }
int omni_pl_placement_last_instructions(void* p, int* out, int max_n) {
  auto v = ((Placement*)p)->last_instructions();
  int n = 0;
  for (auto& i : v) {
    if (n >= max_n) break;
    int* o = out + 8 * n++;
    o[0] = i.layer_idx; o[1] = (int)i.type; o[2] = i.source_rank; o[3] = i.source_expert_id;
    o[4] = i.source_global_position; o[5] = i.target_rank; o[6] = i.target_expert_id; o[7] = i.target_global_position;
  }
  return n;
}

// host replica of the expert weights (second replacement variant): 0 on success
int omni_pl_weights_init_shm(void* w, const char* name, int experts, int ranks_on_host) {
  return ((MoEWeights*)w)->init_shared_memory(name, experts, ranks_on_host) ? 0 : -1;
}
void omni_pl_weights_replicate(void* w, void* mapping) { ((MoEWeights*)w)->replicate_to_shared_memory(*(PlacementMapping*)mapping); }
int omni_pl_weights_replica_complete(void* w) { return ((MoEWeights*)w)->replica_complete() ? 1 : 0; }
int omni_pl_weights_replica_has(void* w, int layer, int expert) { return ((MoEWeights*)w)->replica_has(layer, expert) ? 1 : 0; }
unsigned long long omni_pl_weights_replica_bytes(void* w) { return ((MoEWeights*)w)->replica_bytes(); }
void omni_pl_weights_close_shm(void* w, int unlink) { ((MoEWeights*)w)->close_shared_memory(unlink != 0); }

// moving average of the balancer: returns the number of doubles written (0 when no round has run yet), -1 if `max_n`
// is too small
int omni_pl_placement_get_ema(void* p, double* out, int max_n) {
  auto v = ((Placement*)p)->ema_snapshot();
  if ((int)v.size() > max_n) return -1;
  memcpy(out, v.data(), v.size() * sizeof(double));
  return (int)v.size();
}
int omni_pl_placement_set_ema(void* p, const double* in, int n) {
  return ((Placement*)p)->restore_ema(std::vector<double>(in, in + n)) ? 0 : -1;
}

// static placement from per-expert loads: out[world*slots]
int omni_pl_static_placement(const double* loads, int world, int experts, int slots, int ranks_per_host, int max_red,
                             int* out) {
  try {
    ExpertLoadBalancer b(world, experts, slots, ranks_per_host);
    auto p = b.generate_constrained_placement(std::vector<double>(loads, loads + experts), max_red);
    memcpy(out, p.data(), p.size() * sizeof(int));
    return b.validate(p) ? 0 : -2;
  } catch (const std::exception& e) {
    fprintf(stderr, "omni_placement: %s\n", e.what());
    return -1;
  }
}

// greedy EPLB on host arrays: placement/activations [layers*world*slots]; out: up to max_n instructions of 8 ints
int omni_pl_greedy_instructions(const int* placement, const long long* activations, int layers, int world, int experts,
                                int slots, int max_red, int* out, int max_n) {
  GreedyExpertLoadBalancer g(layers, world, experts, slots, max_red);
  const size_t n_el = (size_t)layers * world * slots;
  auto v = g.optimize_and_generate_instructions(std::vector<int>(placement, placement + n_el),
                                                std::vector<int64_t>(activations, activations + n_el));
  int n = 0;
  for (auto& i : v) {
    if (n >= max_n) break;
    int* o = out + 8 * n++;
    o[0] = i.layer_idx; o[1] = (int)i.type; o[2] = i.source_rank; o[3] = i.source_expert_id;
    o[4] = i.source_global_position; o[5] = i.target_rank; o[6] = i.target_expert_id; o[7] = i.target_global_position;
  }
  return n;
}

// static planner on host arrays: placement/activations [layers*world*slots].  out: up to max_n instructions of 9 ints
// (the 8 fields of the greedy call, then the wave priority); ratios: [layers][2] simulated max/mean before and after.
int omni_pl_static_instructions(const int* placement, const long long* activations, int layers, int world, int experts,
                                int slots, int ranks_per_host, int max_red, int diff_limit, double accept_margin, int* out,
                                int max_n, double* ratios) {
  try {
    ExpertLoadBalancer b(world, experts, slots, ranks_per_host);
    StaticBalanceOptions opt;
    opt.max_redundant_per_expert = max_red; opt.diff_limit = diff_limit; opt.accept_margin = accept_margin;
    const size_t n_el = (size_t)layers * world * slots;
    std::vector<LayerPlan> plans;
    auto v = b.optimize_and_generate_instructions(layers, std::vector<int>(placement, placement + n_el),
                                                  std::vector<int64_t>(activations, activations + n_el), opt, &plans);
    if (ratios)
      for (int l = 0; l < layers; ++l) { ratios[2 * l] = plans[l].ratio_before; ratios[2 * l + 1] = plans[l].ratio_after; }
    int n = 0;
    for (auto& i : v) {
      if (n >= max_n) break;
      int* o = out + 9 * n++;
      o[0] = i.layer_idx; o[1] = (int)i.type; o[2] = i.source_rank; o[3] = i.source_expert_id;
      o[4] = i.source_global_position; o[5] = i.target_rank; o[6] = i.target_expert_id; o[7] = i.target_global_position;
      o[8] = i.prior;
    }
    return n;
  } catch (const std::exception& e) {
    fprintf(stderr, "omni_placement: %s\n", e.what());
    return -1;
  }
}

}  // extern "C"
