// Replica state machine, per-replica metrics, planner (autoscaling policy) and steersman (placement).
//
// States and transitions follow router_v2/src/replica/metrics.rs:17-58 and the triggers collected
// in the controller; the legality table below is what the event loops of
// router_v2/src/replica/disaggregation.rs:741-1931 and cybernetics/mod.rs:32-747 can actually do.
// The planner is the three-equation policy of cybernetics/planner.rs:331-449 (decode memory, KV
// bandwidth, prefill throughput; hysteresis bands; scale up to the band midpoint, down by one).
// One deliberate fix: the prefill KV-bandwidth upper count uses the low bound of the band (the
// reference uses the high bound twice, planner.rs:386-391, which makes the band empty).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <optional>
#include <set>
#include <string>
#include <utility>
#include <vector>

namespace blitz {

enum class RState : int {
  Inactive = 0, Prefill, NewPrefill, OldPrefill, RefractoryPrefill, Decode, ShuttingPrefill, ShuttingDecode,
  ShuttingNull, MutatingToDecode, AusPrefill, AusDecode, LoadingPrefill, LoadingDecode,
  // planner-side markers (kept beside the worker state, never replace it)
  RdmaSending, RdmaLoading, NvlinkSending, NvlCasting, RdmaCasting, TanzCasting,
};

inline const char* rstate_name(RState s) {
  static const char* n[] = {"Inactive", "Prefill", "NewPrefill", "OldPrefill", "RefractoryPrefill", "Decode",
                            "ShuttingPrefill", "ShuttingDecode", "ShuttingNull", "MutatingToDecode", "AusPrefill",
                            "AusDecode", "LoadingPrefill", "LoadingDecode", "RdmaSending", "RdmaLoading",
                            "NvlinkSending", "NvlCasting", "RdmaCasting", "TanzCasting"};
  return n[static_cast<int>(s)];
}
inline std::optional<RState> rstate_from_name(const std::string& s) {
  for (int i = 0; i <= static_cast<int>(RState::TanzCasting); ++i)
    if (s == rstate_name(static_cast<RState>(i))) return static_cast<RState>(i);
  if (s == "Normal") return RState::Prefill;  // cluster JSON also accepts "Normal" (colocated) ranks
  return std::nullopt;
}

inline bool transition_allowed(RState a, RState b) {
  using S = RState;
  static const std::set<std::pair<int, int>> ok = [] {
    std::set<std::pair<int, int>> t;
    auto add = [&t](S x, S y) { t.insert({static_cast<int>(x), static_cast<int>(y)}); };
    add(S::Inactive, S::LoadingPrefill); add(S::Inactive, S::LoadingDecode); add(S::Inactive, S::NewPrefill);
    add(S::LoadingPrefill, S::Prefill); add(S::LoadingPrefill, S::AusPrefill); add(S::AusPrefill, S::Prefill);
    add(S::LoadingDecode, S::AusDecode); add(S::LoadingDecode, S::Decode); add(S::AusDecode, S::Decode);
    add(S::LoadingPrefill, S::Inactive); add(S::LoadingDecode, S::Inactive); add(S::NewPrefill, S::Inactive);
    add(S::NewPrefill, S::RefractoryPrefill); add(S::RefractoryPrefill, S::Prefill);
    add(S::Prefill, S::OldPrefill); add(S::OldPrefill, S::Prefill);
    add(S::Prefill, S::MutatingToDecode); add(S::MutatingToDecode, S::Decode);
    add(S::Prefill, S::ShuttingPrefill); add(S::ShuttingPrefill, S::ShuttingNull); add(S::ShuttingPrefill, S::Prefill);
    add(S::Decode, S::ShuttingDecode); add(S::ShuttingDecode, S::ShuttingNull); add(S::ShuttingDecode, S::Decode);
    add(S::Decode, S::ShuttingNull);
    add(S::ShuttingNull, S::Prefill); add(S::ShuttingNull, S::AusDecode); add(S::ShuttingNull, S::Decode);
    add(S::ShuttingNull, S::Inactive);
    // a replica whose workers failed can be dropped from any state
    for (int i = 1; i <= static_cast<int>(S::LoadingDecode); ++i) t.insert({i, static_cast<int>(S::Inactive)});
    return t;
  }();
  return ok.count({static_cast<int>(a), static_cast<int>(b)}) > 0;
}

struct ReplicaMetric {
  RState state = RState::Inactive;
  std::optional<RState> marker;       // planner marker (sending / casting ...)
  uint32_t used_blocks = 0;
  bool model_loaded = false;
  bool dst_busy = false;              // "dst_mutex": held whenever the replica is not a free decode target
  uint32_t flying_partial = 0;
  uint64_t loop_cnt = 0;
  double shutting_since = -1;
  double flow_in_mb = 0, flow_out_mb = 0;
};

// ---------------------------------------------------------------------------------------------------
struct PlannerConfig {
  float prefill_lower = 0.5f, prefill_upper = 0.7f;
  float decode_lower = 0.75f, decode_upper = 0.95f;
  float migration_lower = 0.4f, migration_upper = 0.8f;
  uint32_t min_prefill = 1, max_prefill = 8, min_decode = 1, max_decode = 8;
  uint32_t tokens_prefilled_per_sec = 15000;
  uint32_t tokens_transferred_per_sec = 96000;
  uint32_t max_blocks_per_replica = 30000;
  uint32_t block_size = 64;
  double scale_down_threshold_ms = 333;
  // Arrival-rate signal (feature `planner_arrival_rate`): prompt tokens that arrived during the last
  // `arrival_window_ms`, as a rate, against what one prefill replica takes per second.  The queue-based rule above
  // reacts once a backlog has built up; this one reacts to the rate that builds it.  0 = not configured.
  double prefill_rate_per_sec = 0;
  double arrival_window_ms = 50;
};

struct PlannerView {
  uint32_t num_prefill = 0, num_decode = 0;
  uint64_t decode_used_blocks = 0;        // blocks held by decode-side replicas
  uint64_t prefill_used_blocks = 0;       // blocks held by prefill replicas (their KV awaits migration)
  uint64_t waiting_prefill_tokens = 0;
  double arrival_tokens_per_sec = 0;      // 0 unless the arrival-rate signal is on
};

struct ScaleBands {
  uint32_t prefill_thpt_min = 0, prefill_thpt_max = 0, prefill_kv_min = 0, prefill_kv_max = 0;
  uint32_t decode_mem_min = 0, decode_mem_max = 0, decode_kv_min = 0, decode_kv_max = 0;
  uint32_t prefill_rate_min = 0, prefill_rate_max = 0;
};

struct ScaleTarget {
  int d_prefill = 0, d_decode = 0;
  ScaleBands bands;
};

inline uint32_t ceil_div_f(double x, double a, double b) {
  if (a <= 0 || b <= 0) return 0;
  return static_cast<uint32_t>(std::ceil(x / a / b));
}

inline ScaleTarget plan_scale(const PlannerConfig& c, const PlannerView& v) {
  ScaleTarget t;
  ScaleBands& b = t.bands;
  // Eq.1 decode memory
  b.decode_mem_min = ceil_div_f(static_cast<double>(v.decode_used_blocks), c.decode_upper, c.max_blocks_per_replica);
  b.decode_mem_max = ceil_div_f(static_cast<double>(v.decode_used_blocks), c.decode_lower, c.max_blocks_per_replica);
  // Eq.2 KV bandwidth: tokens sitting on prefill replicas must be absorbed by decode replicas
  const double prefill_tokens = static_cast<double>(v.prefill_used_blocks) * c.block_size;
  b.decode_kv_min = ceil_div_f(prefill_tokens, c.migration_upper, c.tokens_transferred_per_sec);
  b.decode_kv_max = ceil_div_f(prefill_tokens, c.migration_lower, c.tokens_transferred_per_sec);
  b.prefill_kv_min = b.decode_kv_min;
  b.prefill_kv_max = b.decode_kv_max;
  // Eq.3 prefill throughput
  b.prefill_thpt_min = ceil_div_f(static_cast<double>(v.waiting_prefill_tokens), c.prefill_upper, c.tokens_prefilled_per_sec);
  b.prefill_thpt_max = ceil_div_f(static_cast<double>(v.waiting_prefill_tokens), c.prefill_lower, c.tokens_prefilled_per_sec);

  auto decide = [](uint32_t lo, uint32_t hi, uint32_t cur) -> int {
    int d = 0;
    if (lo > cur) d = static_cast<int>((lo + hi + 1) / 2) - static_cast<int>(cur);       // up: to the band midpoint
    else if (hi < cur) d = static_cast<int>(hi) - static_cast<int>(cur);                 // down
    d = std::max(d, -1);                                                                // at most one per tick
    d = std::max(d, -static_cast<int>(cur) + 1);                                        // never below one
    return d;
  };
  const uint32_t dmin = std::max(b.decode_mem_min, b.decode_kv_min);
  const uint32_t dmax = std::max({b.decode_mem_max, b.decode_kv_max, dmin});
  uint32_t pmin = std::max(b.prefill_thpt_min, b.prefill_kv_min);
  uint32_t pmax = std::max({b.prefill_thpt_max, b.prefill_kv_max, pmin});
  if (c.prefill_rate_per_sec > 0 && v.arrival_tokens_per_sec > 0) {
    // utilisation band on the arrival rate: enough replicas to take what arrives at no more than `prefill_upper`
    b.prefill_rate_min = ceil_div_f(v.arrival_tokens_per_sec, c.prefill_upper, c.prefill_rate_per_sec);
    b.prefill_rate_max = ceil_div_f(v.arrival_tokens_per_sec, c.prefill_lower, c.prefill_rate_per_sec);
    pmin = std::max(pmin, b.prefill_rate_min);
    pmax = std::max({pmax, b.prefill_rate_max, pmin});
  }
  t.d_prefill = decide(pmin, pmax, v.num_prefill);
  t.d_decode = decide(dmin, dmax, v.num_decode);
  // clamp to the configured replica counts (planner.rs:110-126)
  const int np = static_cast<int>(v.num_prefill) + t.d_prefill, nd = static_cast<int>(v.num_decode) + t.d_decode;
  t.d_prefill = std::clamp(np, static_cast<int>(c.min_prefill), static_cast<int>(c.max_prefill)) - static_cast<int>(v.num_prefill);
  t.d_decode = std::clamp(nd, static_cast<int>(c.min_decode), static_cast<int>(c.max_decode)) - static_cast<int>(v.num_decode);
  return t;
}

// ---------------------------------------------------------------------------------------------------
// Steersman: which rank lives on which machine, which ranks hold which model (with a host-cache TTL
// for the ServerlessLLM baseline), which ranks' NVLink egress is busy, and who should feed whom
// (router_v2/src/replica/steersman/mod.rs:46-357).
class Steersman {
 public:
  Steersman(std::vector<int> machine_of_rank, int tp, double host_cache_ttl_s = 30.0)
      : machine_(std::move(machine_of_rank)), tp_(tp), ttl_(host_cache_ttl_s), nvl_busy_(machine_.size(), 0) {}

  int num_ranks() const { return static_cast<int>(machine_.size()); }
  int machine_of(int rank) const { return machine_[rank]; }
  int replica_of_rank(int rank) const { return rank / tp_; }  // tp is a power of two; replica id = first rank / tp
  std::vector<int> ranks_of_replica(int r) const {
    std::vector<int> v;
    for (int i = 0; i < tp_; ++i) v.push_back(r * tp_ + i);
    return v;
  }

  void register_model(const std::string& name, const std::string& path, double size_gb) { models_[name] = {path, size_gb}; }
  std::optional<std::pair<std::string, double>> model_info(const std::string& name) const {
    auto it = models_.find(name);
    if (it == models_.end()) return std::nullopt;
    return it->second;
  }

  // GPU-resident copies
  void record_model_loaded(int replica) { loaded_.insert(replica); }
  void record_model_unloaded(int replica, double now) {
    loaded_.erase(replica);
    for (int r : ranks_of_replica(replica)) host_cache_[machine_[r]] = now;  // weights stay in host memory for a while
  }
  bool model_on_gpu(int replica) const { return loaded_.count(replica) > 0; }
  // Host cache (ServerlessLLM baseline): a machine keeps the model in pinned host memory for `ttl` seconds
  // after last use; `touch` refreshes.
  bool host_cache_hit(int machine, double now) const {
    auto it = host_cache_.find(machine);
    return it != host_cache_.end() && now - it->second <= ttl_;
  }
  void touch_host_cache(int machine, double now) { host_cache_[machine] = now; }

  bool nvlink_busy(int replica) const { return nvl_busy_[replica * tp_] != 0; }
  void set_nvlink_busy(int replica, bool b) {
    for (int r : ranks_of_replica(replica)) nvl_busy_[r] = b ? 1 : 0;
  }

  // For every inactive replica pick a same-machine source among `sources` (replicas holding the model whose
  // egress is idle), at most `fanout` destinations per source.  Returns (source replica -> destinations).
  std::map<int, std::vector<int>> assign_nvlink_chains(const std::vector<int>& sources, const std::vector<int>& targets,
                                                       int fanout = 7) const {
    std::map<int, std::vector<int>> plan;
    for (int t : targets) {
      int best = -1;
      size_t best_load = SIZE_MAX;
      for (int s : sources) {
        if (machine_[s * tp_] != machine_[t * tp_] || nvlink_busy(s) || !model_on_gpu(s)) continue;
        const size_t load = plan.count(s) ? plan[s].size() : 0;
        if (static_cast<int>(load) >= fanout) continue;
        if (load < best_load) { best = s; best_load = load; }
      }
      if (best >= 0) plan[best].push_back(t);
    }
    return plan;
  }
  // Multi-source ("Tanz") plan: per machine, all idle sources jointly feed all targets, each source one stripe.
  struct TanzPlan { std::vector<int> sources, targets; };
  std::vector<TanzPlan> assign_tanz_chains(const std::vector<int>& sources, const std::vector<int>& targets) const {
    std::map<int, TanzPlan> by_machine;
    for (int s : sources)
      if (!nvlink_busy(s) && model_on_gpu(s)) by_machine[machine_[s * tp_]].sources.push_back(s);
    for (int t : targets) by_machine[machine_[t * tp_]].targets.push_back(t);
    std::vector<TanzPlan> out;
    for (auto& kv : by_machine)
      if (!kv.second.sources.empty() && !kv.second.targets.empty()) out.push_back(kv.second);
    return out;
  }

 private:
  std::vector<int> machine_;
  int tp_;
  double ttl_;
  std::vector<uint8_t> nvl_busy_;
  std::map<std::string, std::pair<std::string, double>> models_;
  std::set<int> loaded_;
  std::map<int, double> host_cache_;
};

}  // namespace blitz
