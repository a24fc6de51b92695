// OmniPlacement core: redundant + dynamic expert placement for expert-parallel MoE serving.
//
// Native counterpart of the reference's omni_planner C++ extension
// (omni/accelerators/placement/omni_planner/cpp/*.cpp, include/*.h):
//   PlacementMapping          pattern [rank][layer][expert] -> deployed positions, redundancy counts and the
//                             per-rank selector (logical expert -> physical position) with validated updates
//   ClusterActivation         per-(layer, position) activation counters, cluster-wide collection, wrap-around
//                             deltas, sliding windows, text dump / replay
//   MoEWeights                registry of the device tensors of every local expert slot and their byte sizes
//   GreedyExpertLoadBalancer  dynamic EPLB: EMA of loads, REMOVE / SWAP / ADD instructions
//   ExpertLoadBalancer        static placement: redundancy allocation + LPT, bucket balance with pairwise swaps
//   PlacementOptimizer        glue between activations, mapping and the balancers
//   Distribution              transport: all-gather of small control tuples, pairwise expert-weight swap into a
//                             ring of staging buffers, copy of completed stages into the live weights
//   Placement                 background thread that runs rounds of collect -> optimise -> handshake -> swap, and
//                             do_placement_optimizer() that the inference thread calls between steps
//
// No CUDA or NCCL symbols appear here.  Device copies and collectives go through function pointers
// (PlacementHooks): the Python side installs callbacks backed by torch / NCCL / peer copies, unit tests install
// host memcpy and an in-process transport (threads + shared queues), as the reference does with its
// set_ut_memcpy_fun hook.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

namespace omni_placement {

// ------------------------------------------------------------------------------------------------ hooks
struct PlacementHooks {
  // dst/src are device (or host, in tests) addresses
  std::function<void(void* dst, const void* src, size_t bytes)> memcpy_d2d;
  std::function<void(void* dst, const void* src, size_t bytes)> memcpy_h2d;
  std::function<void(void* dst, const void* src, size_t bytes)> memcpy_d2h;
};
PlacementHooks& hooks();
void set_ut_memcpy_fun();    // host memcpy for all three directions (unit tests, CPU ranks)
void unset_ut_memcpy_fun();

// ------------------------------------------------------------------------------------------------ Tensor
// Thin handle of a buffer owned by the caller.
class Tensor {
 public:
  Tensor() = default;
  Tensor(void* data, size_t length, size_t element_size, std::string name = "")
      : data_(data), length_(length), element_size_(element_size), name_(std::move(name)) {}
  void* data() const { return data_; }
  size_t length() const { return length_; }
  size_t element_size() const { return element_size_; }
  size_t bytes() const { return length_ * element_size_; }
  const std::string& name() const { return name_; }
  void to_host(void* host) const;
  void to_device(const void* host) const;

 private:
  void* data_ = nullptr;
  size_t length_ = 0, element_size_ = 1;
  std::string name_;
};

// ------------------------------------------------------------------------------------------------ Mapping
class PlacementMapping {
 public:
  // pattern: [world][layers][experts] of 0/1.  redundant_per_rank extra slots exist on every rank;
  // ranks_per_host groups ranks into hosts for the selector preference.
  PlacementMapping(const std::vector<int>& pattern, int world, int layers, int experts, int rank,
                   int redundant_per_rank, int ranks_per_host, int32_t* selector /* [layers*experts] or null */);
  static std::vector<int> base_pattern(int world, int layers, int experts);
  static std::vector<int> load_text_pattern(const std::string& path, int& world, int& layers, int& experts);

  int world() const { return world_; }
  int layers() const { return layers_; }
  int experts() const { return experts_; }
  int rank() const { return rank_; }
  int slots_per_rank() const { return slots_per_rank_; }
  int num_positions() const { return world_ * slots_per_rank_; }

  int expert_at(int layer, int global_pos) const { return pos_to_expert_[layer * num_positions() + global_pos]; }
  int redundant_count(int layer, int expert) const { return deploy_count_[layer * experts_ + expert]; }
  std::vector<int> positions_of(int layer, int expert) const;
  std::vector<int> local_slots_of(int layer, int expert) const;
  int selector(int layer, int expert) const { return selector_host_[layer * experts_ + expert]; }
  const std::vector<int32_t>& selector_host() const { return selector_host_; }

  // Validated update: position must currently hold `old_expert` (or be empty = -1); an expert never loses its
  // last replica.  Returns false (and changes nothing) when a check fails.
  bool update_position(int layer, int global_pos, int old_expert, int new_expert);
  bool check_update_is_valid(int layer, int global_pos, int old_expert, int new_expert) const;
  // set several positions at once; succeeds only if afterwards every expert of the touched layers still has a
  // replica, otherwise nothing changes (rollback)
  bool apply_batch(const std::vector<std::pair<int, int>>& layer_pos, const std::vector<int>& new_experts);
  void update_selector_layer(int layer);
  void update_selector();           // all layers, then pushes to the device selector if one was given
  void push_selector_to_device();

 private:
  int world_, layers_, experts_, rank_, slots_per_rank_, ranks_per_host_;
  std::vector<int> pos_to_expert_;   // [layers][world*slots]
  std::vector<int> deploy_count_;    // [layers][experts]
  std::vector<int32_t> selector_host_;
  int32_t* selector_dev_;
};

// ------------------------------------------------------------------------------------------------ Activation
using AllGatherI64 = std::function<void(const int64_t* send, int64_t* recv, size_t count_per_rank)>;

class ClusterActivation {
 public:
  // local counters [layers][slots_per_rank] live at `counts` (device int64, written by the router kernel)
  ClusterActivation(Tensor counts, int layers, int slots_per_rank, int world, int rank, int window = 8);
  void set_allgather(AllGatherI64 fn) { allgather_ = std::move(fn); }
  // reads the local counters, all-gathers, computes wrap-around-corrected deltas since the previous collect
  void collect();
  void collect_from_txt(const std::string& path);   // replay: one line per layer, world*slots values
  void dump_txt(const std::string& path) const;
  int64_t delta(int layer, int global_pos) const { return delta_[layer * positions() + global_pos]; }
  int64_t windowed(int layer, int global_pos) const;
  int64_t total(int layer, int global_pos) const { return last_[layer * positions() + global_pos]; }
  int positions() const { return world_ * slots_; }
  int layers() const { return layers_; }
  static constexpr int64_t kWrap = 10000000000000000LL;   // counters are kept modulo 1e16

 private:
  Tensor counts_;
  int layers_, slots_, world_, rank_, window_;
  AllGatherI64 allgather_;
  std::vector<int64_t> last_, delta_;
  std::vector<std::vector<int64_t>> history_;
  bool first_ = true;
};

// ------------------------------------------------------------------------------------------------ Weights
struct ExpertTensor { void* ptr; size_t bytes; };

class MoEWeights {
 public:
  MoEWeights(int layers, int slots_per_rank) : layers_(layers), slots_(slots_per_rank), w_(layers * slots_per_rank) {}
  ~MoEWeights();
  void add_tensor(int layer, int slot, void* ptr, size_t bytes) { w_[layer * slots_ + slot].push_back({ptr, bytes}); }
  const std::vector<ExpertTensor>& tensors(int layer, int slot) const { return w_[layer * slots_ + slot]; }
  size_t expert_bytes() const;   // bytes of one expert slot (all its tensors); 0 before init
  bool is_initialized() const { return initialized_; }
  void set_initialized() { initialized_ = true; }
  int layers() const { return layers_; }
  int slots() const { return slots_; }

  // ---- host replica: every logical expert of every layer once in POSIX shared memory, shared by the ranks of a host.
  // With it an expert is replaced by a host-to-device copy on the rank that wants it; no other rank takes part.
  // (The other replacement variant moves the expert between ranks through the Distribution.)
  // Creates the segment (first caller) or attaches to it; every rank of the host calls this with the same arguments.
  bool init_shared_memory(const std::string& name, int experts, int ranks_on_host);
  // Copies the experts this rank holds (as the mapping says) into the replica, then counts itself as done.
  void replicate_to_shared_memory(const PlacementMapping& mapping);
  bool replica_enabled() const { return shm_ != nullptr; }
  bool replica_complete() const;                                  // every rank of the host has replicated
  bool replica_has(int layer, int expert) const;
  // host -> device copy of `expert` of `layer` into the tensors of local slot `slot`; false if the replica lacks it
  bool replace_from_shared_memory(int layer, int expert, int slot) const;
  void close_shared_memory(bool unlink);
  size_t replica_bytes() const { return shm_bytes_; }

 private:
  unsigned char* replica_ptr(int layer, int expert) const;
  int layers_, slots_;
  std::vector<std::vector<ExpertTensor>> w_;
  bool initialized_ = false;
  unsigned char* shm_ = nullptr;
  size_t shm_bytes_ = 0, shm_data_off_ = 0;
  int shm_experts_ = 0, shm_ranks_ = 0;
  std::string shm_name_;
};

// ------------------------------------------------------------------------------------------------ Instructions
enum class OperationType : int { SWAP = 0, ADD = 1, REMOVE = 2, EMPTY = 3 };

struct ChangeInstruction {
  int layer_idx = 0;
  OperationType type = OperationType::EMPTY;
  int source_rank = -1, source_expert_id = -1, source_global_position = -1;
  int target_rank = -1, target_expert_id = -1, target_global_position = -1;
  int prior = 0;
};

// ------------------------------------------------------------------------------------------------ Greedy EPLB
class GreedyExpertLoadBalancer {
 public:
  GreedyExpertLoadBalancer(int layers, int world, int experts, int slots_per_rank, int max_redundant_per_expert = 10,
                           double ema_keep = 0.6, double threshold = 1.1, int max_instructions_per_layer = 32);
  // placement: [layers][world*slots] expert id or -1; activations: same shape (delta counts of this round)
  std::vector<ChangeInstruction> optimize_and_generate_instructions(const std::vector<int>& placement,
                                                                    const std::vector<int64_t>& activations);
  static double imbalance(const std::vector<double>& rank_loads);   // max / min (min clipped to > 0)
  const std::vector<double>& ema_loads() const { return ema_; }
  bool has_ema() const { return has_ema_; }
  // restores the moving average saved by an earlier run (same [layers][positions] shape); false if the size differs
  bool set_ema(const std::vector<double>& ema) {
    if (ema.size() != ema_.size()) return false;
    ema_ = ema;
    has_ema_ = true;
    return true;
  }

 private:
  void optimize_layer(int layer, std::vector<int>& place, std::vector<double>& load, std::vector<ChangeInstruction>& out);
  std::vector<double> rank_loads(const std::vector<int>& place, const std::vector<double>& load) const;
  int layers_, world_, experts_, slots_, max_red_;
  double keep_, threshold_;
  int max_instr_;
  std::vector<double> ema_;   // [layers][positions]
  bool has_ema_ = false;
};

// ------------------------------------------------------------------------------------------------ Static balancer
// Plans placement changes for one snapshot of activation counts (no history, unlike the greedy balancer above): the
// target is derived from the loads, the result is a list of instructions bounded by a communication limit.
struct StaticBalanceOptions {
  int max_redundant_per_expert = 10;   // replicas of one expert: at most 1 + this
  int diff_limit = -1;                 // instructions per layer (communication limit); < 0: 2 * world
  double accept_margin = 0.1;          // a layer's plan is kept only if it lowers max/mean by more than this
};

struct LayerPlan {
  int layer = 0;
  std::vector<int> placement;          // placement after the kept instructions
  std::vector<ChangeInstruction> instructions;
  double ratio_before = 1.0, ratio_after = 1.0;   // max rank load / mean rank load, replicas share an expert's load evenly
  int considered = 0;                  // instructions generated before the limit and the acceptance test cut them
  bool accepted = false;
};

class ExpertLoadBalancer {
 public:
  ExpertLoadBalancer(int world, int experts, int slots_per_rank, int ranks_per_host = 8)
      : world_(world), experts_(experts), slots_(slots_per_rank), rph_(ranks_per_host) {}
  // loads: per logical expert.  Returns [world*slots] expert id or -1.  Redundant slots go to the hottest experts
  // (max-heap on load / replicas), replicas are assigned by LPT with host interleave; every expert appears once.
  std::vector<int> generate_constrained_placement(const std::vector<double>& loads, int max_redundant_per_expert) const;
  // no redundancy: starting from `placement`, pairwise swaps between the heaviest and lightest ranks
  std::vector<ChangeInstruction> bucket_balance(int layer, std::vector<int> placement, const std::vector<double>& loads,
                                                int max_swaps) const;
  bool validate(const std::vector<int>& placement) const;

  // ---- analysis of one layer ([world*slots] expert id or -1; activations are per position)
  int positions() const { return world_ * slots_; }
  std::vector<double> expert_loads(const std::vector<int>& placement, const std::vector<int64_t>& activations) const;
  std::vector<int> replica_counts(const std::vector<int>& placement) const;
  std::vector<double> simulated_rank_loads(const std::vector<int>& placement, const std::vector<double>& loads) const;
  double simulated_ratio(const std::vector<int>& placement, const std::vector<double>& loads) const;
  double measured_ratio(const std::vector<int>& placement, const std::vector<int64_t>& activations) const;
  int find_position(const std::vector<int>& placement, int rank, int expert) const;   // -1 if absent
  int find_empty(const std::vector<int>& placement, int rank) const;                  // -1 if full
  bool validate_counts(const std::vector<int>& placement, int min_per_rank, int max_per_rank) const;
  // how many per-rank set differences separate two placements (experts to drop + experts to fetch)
  int diff_count(const std::vector<int>& from, const std::vector<int>& to) const;

  // ---- planning
  // One layer: REMOVE of surplus replicas, ADD of replicas of the hottest experts onto the coldest ranks, then SWAPs
  // between the heaviest and the lightest rank; every prefix of the list leaves a valid placement.  The list is cut at
  // the communication limit and at its best prefix, and dropped entirely if the gain is within the margin.
  LayerPlan plan_layer(int layer, const std::vector<int>& placement, const std::vector<int64_t>& activations,
                       const StaticBalanceOptions& opt) const;
  // All layers: placement / activations are [layers][world*slots].  Returns the kept instructions with priorities.
  std::vector<ChangeInstruction> optimize_and_generate_instructions(int layers, const std::vector<int>& placement,
                                                                    const std::vector<int64_t>& activations,
                                                                    const StaticBalanceOptions& opt,
                                                                    std::vector<LayerPlan>* plans = nullptr) const;
  // prior = 1 + the highest prior of an earlier instruction of the same layer that touches the same expert or the same
  // position: instructions of equal prior are independent and may run in one exchange wave.  Sorts by (layer, prior).
  static void assign_priorities(std::vector<ChangeInstruction>& instructions);
  // applies one instruction to a layer's placement; false (placement untouched) if it does not fit
  bool apply(std::vector<int>& placement, const ChangeInstruction& ins) const;

 private:
  int world_, experts_, slots_, rph_;
};

// ------------------------------------------------------------------------------------------------ Optimizer
class PlacementOptimizer {
 public:
  PlacementOptimizer(PlacementMapping* mapping, ClusterActivation* act, int max_redundant_per_expert = 10);
  std::vector<ChangeInstruction> optimize();
  std::vector<int> extract_placement() const;
  std::vector<int64_t> extract_activations() const;
  GreedyExpertLoadBalancer& balancer() { return *greedy_; }

 private:
  PlacementMapping* mapping_;
  ClusterActivation* act_;
  std::unique_ptr<GreedyExpertLoadBalancer> greedy_;
};

// ------------------------------------------------------------------------------------------------ Distribution
struct HandshakeTuple { int t_rank; int position_offset; int expert_id; int replica_ok = 0; };

class Distribution {
 public:
  static constexpr int QUEUE_SIZE = 5;
  virtual ~Distribution() = default;
  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual void allgather_i64(const int64_t* send, int64_t* recv, size_t count) = 0;
  virtual void allgather_handshake(const HandshakeTuple& mine, std::vector<HandshakeTuple>& all) = 0;
  // exchange one expert (all tensors, packed) with `peer`; the received bytes land in staging buffer `stage`
  virtual void swap(int peer, const std::vector<ExpertTensor>& send, int stage) = 0;
  virtual void recv_only(int peer, int stage, size_t bytes) = 0;
  virtual void send_only(int peer, const std::vector<ExpertTensor>& send) = 0;
  virtual void* staging(int stage) = 0;
  virtual bool staging_on_device() const { return false; }   // staging buffers are device memory (device-fabric transport)
  virtual void barrier() = 0;
};

// In-process transport for tests and CPU ranks: every "rank" is a thread sharing one hub.
class FakeHub;
class FakeDistribution : public Distribution {
 public:
  FakeDistribution(std::shared_ptr<FakeHub> hub, int rank, size_t expert_bytes);
  ~FakeDistribution() override;
  int rank() const override { return rank_; }
  int world() const override;
  void allgather_i64(const int64_t* send, int64_t* recv, size_t count) override;
  void allgather_handshake(const HandshakeTuple& mine, std::vector<HandshakeTuple>& all) override;
  void swap(int peer, const std::vector<ExpertTensor>& send, int stage) override;
  void recv_only(int peer, int stage, size_t bytes) override;
  void send_only(int peer, const std::vector<ExpertTensor>& send) override;
  void* staging(int stage) override { return stages_[stage].data(); }
  int transfers() const { return transfers_; }   // swap / send / receive calls made (tests)
  void barrier() override;
  // fault injection (host side): corrupt the next handshake tuple this rank sends
  void corrupt_next_handshake() { corrupt_ = true; }

 private:
  std::shared_ptr<FakeHub> hub_;
  int rank_;
  std::vector<std::vector<unsigned char>> stages_;
  bool corrupt_ = false;
  int transfers_ = 0;
};
std::shared_ptr<FakeHub> make_fake_hub(int world);

// Callback transport: the embedding process supplies the collectives (torch.distributed / NCCL / peer copies).
struct DistributionCallbacks {
  int rank = 0, world = 1;
  std::function<void(const int64_t*, int64_t*, size_t)> allgather_i64;
  std::function<void(int peer, const void* send, void* recv, size_t bytes)> sendrecv;   // either pointer may be null
  std::function<void()> barrier;
};
class CallbackDistribution : public Distribution {
 public:
  CallbackDistribution(DistributionCallbacks cb, size_t expert_bytes);
  // Device-fabric form: the embedding process owns a device send buffer (one packed expert, visible to the peers)
  // and QUEUE_SIZE device staging buffers.  An expert is packed with device-to-device copies, the callback moves
  // it over the fabric (peer copy or NCCL) straight into the receiver's staging buffer, and the apply step copies
  // from staging into the live weights on the device.  No byte goes through host memory.
  CallbackDistribution(DistributionCallbacks cb, size_t expert_bytes, void* device_send_buf, void* const* device_stages);
  bool staging_on_device() const override { return device_send_ != nullptr; }
  int rank() const override { return cb_.rank; }
  int world() const override { return cb_.world; }
  void allgather_i64(const int64_t* send, int64_t* recv, size_t count) override { cb_.allgather_i64(send, recv, count); }
  void allgather_handshake(const HandshakeTuple& mine, std::vector<HandshakeTuple>& all) override;
  void swap(int peer, const std::vector<ExpertTensor>& send, int stage) override;
  void recv_only(int peer, int stage, size_t bytes) override;
  void send_only(int peer, const std::vector<ExpertTensor>& send) override;
  void* staging(int stage) override { return device_send_ ? device_stages_[stage] : (void*)stages_[stage].data(); }
  void barrier() override { if (cb_.barrier) cb_.barrier(); }

 private:
  size_t pack_device(const std::vector<ExpertTensor>& ts);
  DistributionCallbacks cb_;
  std::vector<std::vector<unsigned char>> stages_;   // host staging; the apply step copies into device weights
  std::vector<unsigned char> pack_;
  void* device_send_ = nullptr;
  std::vector<void*> device_stages_;
};

// ------------------------------------------------------------------------------------------------ Manager
struct PendingApply { int layer, slot, stage, new_expert, global_pos, old_expert; bool from_replica = false; };

class Placement {
 public:
  Placement(PlacementMapping* mapping, MoEWeights* weights, ClusterActivation* act, Distribution* dist,
            int max_redundant_per_expert = 10, double period_s = 60.0);
  ~Placement();
  void start();   // background thread
  void stop();
  // one round on the calling thread (what the background thread repeats); returns number of applied instructions
  int run_round();
  // inference thread, between steps: copies completed staging buffers into the live expert weights and refreshes
  // the selector.  Returns the number of experts replaced.
  int do_placement_optimizer();
  int rounds() const { return rounds_; }
  // Rounds whose changes are complete on every rank (published after the round's closing barrier) and wait to be, or
  // have been, applied.  Ranks apply a round in the same inference step: the embedding process exchanges this counter
  // (minimum over the ranks) and calls do_placement_optimizer() when the minimum has moved past what it has applied.
  int ready_rounds() const { return ready_rounds_; }
  int skipped_instructions() const { return skipped_; }
  std::vector<ChangeInstruction> last_instructions() const;
  // the balancer's moving average of position loads: saved at shutdown and restored at start so that a restart does
  // not begin from a cold history.  Both take the manager's lock (the background thread updates the average).
  std::vector<double> ema_snapshot();
  bool restore_ema(const std::vector<double>& ema);

 private:
  void loop();
  bool execute(const ChangeInstruction& ins);
  PlacementMapping* mapping_;
  MoEWeights* weights_;
  ClusterActivation* act_;
  Distribution* dist_;
  std::unique_ptr<PlacementOptimizer> optimizer_;
  double period_s_;
  std::thread thread_;
  std::atomic<bool> should_stop_{false};
  std::mutex mu_;
  std::mutex ema_mu_;   // the optimizer's history: a round updates it, snapshot / restore read and write it
  std::condition_variable cv_;
  std::vector<PendingApply> pending_;   // complete rounds, visible to the inference thread
  std::vector<PendingApply> staged_;    // the round in progress
  std::vector<ChangeInstruction> last_;
  std::vector<int> stage_used_;                   // staging buffers taken in the current round, per rank (same on all)
  std::set<std::pair<int, int>> round_touched_;   // (layer, position) changed by an instruction of the current round
  std::atomic<int> rounds_{0}, skipped_{0}, ready_rounds_{0};
};

}  // namespace omni_placement
