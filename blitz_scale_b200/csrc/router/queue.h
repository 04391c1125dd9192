// Router-side request queue, validation and the feature-flag set.
//
// Batching semantics follow router_v2/src/queue.rs:207-363: FIFO only; a request costs
// ceil((input + max_new) / block) * block tokens of KV budget; packing stops (the entry goes back to
// the front) when the padded total would exceed `block_budget` blocks, when the cumulative prompt
// tokens exceed `prefill_token_budget`, or when a single request (+ speculation) exceeds
// `token_budget`; entries whose client went away are dropped; batch ids count up from 0;
// `waiting_prefill_tokens` (the autoscaler's prefill-demand signal) is maintained incrementally.
// Unlike the reference, an entry restored by a failed `min_size` check also restores its waiting
// tokens (the reference leaks them, queue.rs:325-336).
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <optional>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace blitz {

struct RequestEntry {
  uint64_t id = 0;
  uint32_t input_len = 0;
  uint32_t max_new_tokens = 0;
  bool client_alive = true;
  double t_arrival = 0;
  // filled in by the controller
  double t_batched = -1, t_first_token = -1, t_last_token = -1, t_first_decode_token = -1;
  uint32_t generated = 0;
  std::vector<double> tbt;  // time between tokens, first interval excluded (router_v2/src/infer.rs:324-325)
};

struct RouterBatch {
  uint64_t id = 0;
  std::vector<uint64_t> request_ids;
  uint32_t max_tokens = 0;     // sum of page-padded per-request maxima
  uint32_t prompt_tokens = 0;
  uint32_t size() const { return static_cast<uint32_t>(request_ids.size()); }
};

class BatchQueue {
 public:
  explicit BatchQueue(uint32_t block_size = 64, uint32_t speculate = 0, std::optional<uint32_t> window = std::nullopt)
      : block_(block_size), speculate_(speculate), window_(window) {}

  void append(const RequestEntry& e) {
    waiting_prefill_tokens_ += e.input_len;
    entries_.push_back(e);
  }
  size_t size() const { return entries_.size(); }
  bool empty() const { return entries_.empty(); }
  uint64_t waiting_prefill_tokens() const { return waiting_prefill_tokens_; }
  uint32_t block_size() const { return block_; }
  void mark_client_gone(uint64_t id) {
    for (auto& e : entries_)
      if (e.id == id) e.client_alive = false;
  }

  struct Next {
    RouterBatch batch;
    std::vector<RequestEntry> entries;
  };

  // `max_size` (0 = no limit) caps the number of requests in the batch: a worker's step handles a bounded number of
  // sequences whatever their lengths.
  std::optional<Next> next_batch(std::optional<size_t> min_size, uint32_t prefill_token_budget, uint32_t token_budget,
                                 std::optional<uint32_t> block_budget, size_t max_size = 0) {
    if (entries_.empty()) return std::nullopt;
    if (min_size && entries_.size() < *min_size) return std::nullopt;
    Next out;
    uint32_t prefill_tokens = 0, max_tokens = 0;
    while (!entries_.empty()) {
      RequestEntry e = entries_.front();
      entries_.pop_front();
      if (!e.client_alive) {
        waiting_prefill_tokens_ -= e.input_len;
        dropped_ += 1;
        continue;
      }
      uint32_t max_new = e.max_new_tokens;
      if (window_) max_new = std::min(max_new, *window_ > e.input_len ? *window_ - e.input_len : 0u);
      const uint32_t max_req = (e.input_len + max_new + block_ - 1) / block_ * block_;
      const bool over_blocks = block_budget && (max_req + max_tokens > *block_budget * block_);
      // with `split_long_prompts` a prompt that alone exceeds the prefill budget gets a batch of its own, which the
      // worker prefills in chunks; without it (the reference's rule) such a prompt is never admitted, and validation
      // has to keep it out of the queue
      const bool over_prefill = prefill_tokens + e.input_len > prefill_token_budget &&
                                !(split_long_prompts_ && out.entries.empty());
      const bool over_total = max_req + speculate_ > token_budget;
      const bool over_size = max_size > 0 && out.entries.size() >= max_size;
      if (over_blocks || over_prefill || over_total || over_size) {
        entries_.push_front(e);
        break;
      }
      prefill_tokens += e.input_len;
      waiting_prefill_tokens_ -= e.input_len;
      max_tokens += max_req;
      out.batch.request_ids.push_back(e.id);
      out.entries.push_back(e);
    }
    if (out.entries.empty()) return std::nullopt;
    if (min_size && out.entries.size() < *min_size) {
      for (auto it = out.entries.rbegin(); it != out.entries.rend(); ++it) {
        waiting_prefill_tokens_ += it->input_len;
        entries_.push_front(*it);
      }
      return std::nullopt;
    }
    out.batch.id = next_batch_id_++;
    out.batch.max_tokens = max_tokens;
    out.batch.prompt_tokens = prefill_tokens;
    return out;
  }
  // Put the requests of a batch that could not be served back at the front (replica lost).
  void requeue_front(const std::vector<RequestEntry>& es) {
    for (auto it = es.rbegin(); it != es.rend(); ++it) {
      waiting_prefill_tokens_ += it->input_len;
      entries_.push_front(*it);
    }
  }
  uint64_t dropped() const { return dropped_; }
  void set_split_long_prompts(bool on) { split_long_prompts_ = on; }
  // Prompt length of the entry at the head of the queue (0 when empty).
  uint32_t front_input_len() const { return entries_.empty() ? 0u : entries_.front().input_len; }

 private:
  uint32_t block_, speculate_;
  std::optional<uint32_t> window_;
  bool split_long_prompts_ = false;
  std::deque<RequestEntry> entries_;
  uint64_t waiting_prefill_tokens_ = 0;
  uint64_t next_batch_id_ = 0;
  uint64_t dropped_ = 0;
};

// ---------------------------------------------------------------------------------------------------
// Request validation (router_v2/src/validation.rs:152-305): the checks that do not need a tokenizer.
struct GenerateParams {
  uint32_t input_len = 0;
  uint32_t max_new_tokens = 20;
  uint32_t best_of = 1;
  bool do_sample = false;
  float temperature = 1.f, repetition_penalty = 1.f, top_p = 1.f, typical_p = 1.f;
  int32_t top_k = 0;
  uint32_t top_n_tokens = 0;
  uint32_t num_stop_sequences = 0;
  std::optional<uint32_t> truncate;
  bool has_seed = false;
};
struct ValidationLimits {
  uint32_t max_best_of = 2, max_stop_sequences = 4, max_top_n_tokens = 5, max_input_length = 4095,
           max_total_tokens = 4096;
};
// Returns an empty string when valid, else the error message.
inline std::string validate_request(const GenerateParams& p, const ValidationLimits& lim) {
  std::ostringstream e;
  if (p.best_of == 0 || p.best_of > lim.max_best_of) { e << "`best_of` must be > 0 and <= " << lim.max_best_of; return e.str(); }
  const bool sampling = p.do_sample || p.temperature != 1.f || p.top_k != 0 || p.top_p != 1.f || p.typical_p != 1.f;
  if (p.best_of > 1 && !sampling) return "you must use sampling when `best_of` is > 1";
  if (p.best_of > 1 && p.has_seed) return "`seed` must not be set when `best_of` > 1";
  if (!(p.temperature > 0.f)) return "`temperature` must be strictly positive";
  if (!(p.repetition_penalty > 0.f)) return "`repetition_penalty` must be strictly positive";
  if (!(p.top_p > 0.f && p.top_p <= 1.f)) return "`top_p` must be > 0.0 and <= 1.0";
  if (!(p.typical_p > 0.f && p.typical_p <= 1.f)) return "`typical_p` must be > 0.0 and <= 1.0";
  if (p.top_k < 0) return "`top_k` must be positive";
  if (p.max_new_tokens == 0) return "`max_new_tokens` must be strictly positive";
  if (p.num_stop_sequences > lim.max_stop_sequences) { e << "`stop` supports up to " << lim.max_stop_sequences << " stop sequences"; return e.str(); }
  if (p.top_n_tokens > lim.max_top_n_tokens) { e << "`top_n_tokens` must be >= 0 and <= " << lim.max_top_n_tokens; return e.str(); }
  if (p.truncate && (*p.truncate == 0 || *p.truncate > lim.max_input_length)) { e << "`truncate` must be strictly positive and less than " << lim.max_input_length; return e.str(); }
  const uint32_t in_len = p.truncate ? std::min(p.input_len, *p.truncate) : p.input_len;
  if (in_len == 0) return "`inputs` cannot be empty";
  if (in_len > lim.max_input_length) { e << "`inputs` must have less than " << lim.max_input_length << " tokens. Given: " << in_len; return e.str(); }
  if (in_len + p.max_new_tokens > lim.max_total_tokens) {
    e << "`inputs` tokens + `max_new_tokens` must be <= " << lim.max_total_tokens << ". Given: " << in_len
      << " `inputs` tokens and " << p.max_new_tokens << " `max_new_tokens`";
    return e.str();
  }
  return "";
}

// ---------------------------------------------------------------------------------------------------
// Feature flags (names and implications of router_v2/Cargo.toml:64-118; satisfiability rules of
// router_v2/src/lib.rs:10-64).  Chosen at run time (`--features a,b,c`) instead of at compile time.
class FeatureSet {
 public:
  static const std::map<std::string, std::vector<std::string>>& implications() {
    static const std::map<std::string, std::vector<std::string>> m = {
        {"impl_blitz", {"impl_rdma", "mutate"}},
        {"impl_fast", {"fast", "impl_rdma"}},
        {"impl_fast_pro", {"fast", "impl_tanz"}},
        {"impl_tanz", {"fast", "impl_rdma", "impl_nvl"}},
        {"impl_live", {"live"}},
        {"impl_live_pro", {"live", "impl_tanz"}},
        {"impl_sllm", {}}, {"impl_nvl", {}}, {"impl_rdma", {}}, {"unidirect", {}}, {"mutate", {}},
        {"fast", {}}, {"live", {}},
        {"cache_replace", {}}, {"cache_all_hit", {}}, {"cache_all_miss", {}},
        {"manually_scale", {}}, {"motiv", {}}, {"mock_transfer", {}}, {"optimize_op_loading", {}},
        {"optimize_network_interference", {}}, {"decode_load_balance", {}}, {"decode_first_fit", {}}, {"prefill_share_idle", {}}, {"migrate_progressive", {}}, {"planner_arrival_rate", {}}, {"statistic", {}}, {"ngrok", {}},
        {"eval_all", {"impl_blitz", "impl_fast_pro", "impl_live_pro"}},
        {"eval_net", {"impl_blitz", "impl_fast_pro", "impl_live_pro", "optimize_network_interference"}},
        {"eval_fast", {"impl_blitz", "impl_fast_pro"}},
        {"eval_sllm", {"impl_sllm", "cache_replace"}},
        {"eval_sllm_pro", {"impl_sllm", "cache_all_hit", "mutate"}},
        {"eval_fast_wo_nvl", {"impl_blitz", "impl_fast"}},
        {"eval_fast_live_wo_nvl", {"impl_blitz", "impl_fast", "impl_live"}},
        {"test_live", {"impl_blitz", "impl_live", "manually_scale"}},
        {"test_nvl", {"impl_blitz", "impl_nvl", "manually_scale"}},
        {"test_tanz", {"impl_blitz", "impl_tanz", "manually_scale"}},
    };
    return m;
  }
  static FeatureSet parse(const std::string& csv) {
    FeatureSet f;
    std::stringstream ss(csv);
    std::string tok;
    while (std::getline(ss, tok, ',')) {
      size_t a = tok.find_first_not_of(" \t"), b = tok.find_last_not_of(" \t");
      if (a == std::string::npos) continue;
      f.enable(tok.substr(a, b - a + 1));
    }
    f.validate();
    return f;
  }
  void enable(const std::string& name) {
    auto it = implications().find(name);
    if (it == implications().end()) throw std::invalid_argument("unknown feature: " + name);
    if (!on_.insert(name).second) return;
    for (auto& d : it->second) enable(d);
  }
  bool has(const std::string& name) const { return on_.count(name) > 0; }
  std::vector<std::string> list() const { return {on_.begin(), on_.end()}; }
  // The combinations the reference rejects at compile time.
  void validate() const {
    const bool blitz = has("impl_blitz"), sllm = has("impl_sllm");
    if (blitz == sllm) throw std::invalid_argument("exactly one of impl_blitz / impl_sllm must be enabled");
    const int caches = has("cache_replace") + has("cache_all_hit") + has("cache_all_miss");
    if (sllm && caches != 1) throw std::invalid_argument("impl_sllm needs exactly one of cache_replace / cache_all_hit / cache_all_miss");
    if (!sllm && caches != 0) throw std::invalid_argument("host-cache policies only apply to impl_sllm");
    if (sllm && (has("fast") || has("live") || has("impl_nvl") || has("impl_rdma")))
      throw std::invalid_argument("impl_sllm cannot be combined with network scaling features");
    if (has("live") && !(has("impl_rdma") || has("impl_nvl"))) throw std::invalid_argument("live needs a parameter transport");
  }

 private:
  std::set<std::string> on_;
};

}  // namespace blitz
