// Sans-IO orchestrator core: request queue -> prefill replicas -> KV migration -> decode replicas, plus
// the autoscaler (planner, executors for the multicast-based system and for the ServerlessLLM-style
// baseline), live scaling (ZigZag) pairing and the relay queue.
//
// The core never performs IO and never reads a clock: the shell (asyncio + gRPC, or the virtual-time
// simulator) calls `step(now)` to obtain `Action`s, carries them out, and reports completions with the
// `on_*` methods.  The behaviour condenses the per-replica event loops, migration watchers and
// executors of the reference router (router_v2/src/replica/disaggregation.rs:741-2543,
// cybernetics/{planner,exec_blitz,exec_serverless,mod}.rs, relay_queue.rs:10-54) into one
// deterministic state machine; busy-wait loops become explicit "nothing to do" returns.
#pragma once
#include <algorithm>
#include <deque>
#include <map>
#include <optional>
#include <sstream>
#include <string>
#include <tuple>
#include <vector>

#include "queue.h"
#include "replica.h"

namespace blitz {

enum class ActionType : int {
  Prefill = 0, ZagPrefill, PrefillPP, Decode, Migrate, MigratePartial, Relay,
  NvlBroadcast, TanzBroadcast, RdmaBroadcast, LoadParams, ResetStatus, SetStatusReady, ClearCache,
  Deliver, Fail,
  FilterBatch,   // drop requests whose client went away from a resident batch (request_ids = the ones to keep)
};

struct Action {
  ActionType type = ActionType::Deliver;
  uint64_t op_id = 0;              // completion handle (0: fire and forget)
  int replica = -1;                // replica that executes
  int peer = -1;                   // migrate: destination replica; relay / PrefillPP: partner replica
  uint64_t batch_id = 0;
  std::vector<uint64_t> batch_ids; // decode: resident batches to run (first id survives the merge)
  std::vector<uint64_t> request_ids;
  uint32_t max_tokens = 0;
  std::vector<int> src_ranks, dst_ranks;
  int load_case = 1;               // 0 host memory, 1 disk
  int partial = 0;                 // 1 first half, 2 second half
  int num_layer = 0;               // dividing layer of a partial migration / start layer of PrefillPP
  uint32_t zag_seq = 0;
  bool live = false;               // broadcast feeds a NewPrefill (per-layer readiness matters)
  bool mock = false;
  // Deliver / Fail
  uint64_t request_id = 0;
  int32_t token = -1;
  bool final = false;
  int finish_reason = 0;           // with `final`: 0 length, 1 EOS token, 2 stop sequence (proto FinishReason)
};

struct ControllerConfig {
  int num_ranks = 2, tp = 1;
  std::vector<int> machines;               // machine id per rank (default all 0)
  std::vector<std::string> init_states;    // per rank: Prefill | Decode | Normal | Inactive
  uint32_t block_size = 64;
  uint32_t max_prefill_tokens = 8192, max_total_tokens = 16000;
  uint32_t max_blocks_per_replica = 30000;
  uint32_t zigzag_req_limit = 4, zigzag_req_floor = 2;
  double zigzag_decay_ms = 200;
  double planner_interval_ms = 10;
  uint32_t model_layers = 32;
  std::string model_name = "llama3_8b";
  PlannerConfig planner;
  std::string features = "impl_blitz,impl_fast_pro,impl_live_pro";
  bool autoscale = true;
  double mock_load_ms = 0;
  double param_gb = 0;   // parameter bytes per replica in GB (0: unknown); only used for the transfer-rate metric
  double kv_mb_per_token = 0;  // KV bytes of one token over all layers of a replica, in MB (0: unknown); flow report only
  // Migrations that may be in flight towards one decode replica at a time.  1 is the reference's behaviour (a mutex
  // per destination, router_v2/src/replica/disaggregation.rs try_lock scan); more lets the RPC latency of one
  // migration overlap the transfer of another.  Concurrent migrations never share a transfer slot of the worker
  // (slot = batch id mod `kv_transfer_slots`).
  // Sequences one worker step can carry (the workers' --max-batch-size).  No prefill batch is larger, and a decode
  // replica is not given a batch that would take its resident sequences beyond it (the batch waits for room, like one
  // that waits for free KV blocks).  0 = no limit.
  uint32_t max_batch_seqs = 256;
  bool chunked_prefill = true;  // workers prefill a prompt longer than max_prefill_tokens in chunks: admit it alone
  int max_incoming_migrations = 1;
  int kv_transfer_slots = 8;
  double quarantine_ms = 5000;  // a lost replica is not chosen for scale-up again before this much time has passed
};

class Controller {
 public:
  explicit Controller(const ControllerConfig& cfg)
      : cfg_(cfg), features_(FeatureSet::parse(cfg.features)), queue_(cfg.block_size),
        steer_(cfg.machines.empty() ? std::vector<int>(cfg.num_ranks, 0) : cfg.machines, cfg.tp) {
    if (cfg.num_ranks % cfg.tp) throw std::invalid_argument("num_ranks not divisible by tp");
    queue_.set_split_long_prompts(cfg.chunked_prefill);
    const int R = cfg.num_ranks / cfg.tp;
    reps_.resize(R);
    for (int r = 0; r < R; ++r) {
      std::string s = cfg.init_states.empty() ? (r == 0 ? "Prefill" : (r == 1 ? "Decode" : "Inactive"))
                                              : cfg.init_states[r * cfg.tp];
      auto st = rstate_from_name(s);
      if (!st) throw std::invalid_argument("bad init state " + s);
      reps_[r].m.state = *st;
      reps_[r].colocated = (s == "Normal");
      reps_[r].m.model_loaded = (*st != RState::Inactive);
      reps_[r].m.dst_busy = (*st != RState::Decode);
      if (reps_[r].m.model_loaded) steer_.record_model_loaded(r);
      log_transition(r, RState::Inactive, *st, true);
    }
    arrival_signal_ = features_.has("planner_arrival_rate") && cfg.planner.prefill_rate_per_sec > 0;
    cfg_.planner.block_size = cfg.block_size;
    cfg_.planner.max_blocks_per_replica = cfg.max_blocks_per_replica;
  }

  // ------------------------------------------------------------------------------------ inputs
  void submit(const RequestEntry& e) {
    requests_[e.id] = e;
    queue_.append(e);
    counters_["blitz_request_count"] += 1;
    if (arrival_signal_) arrivals_.push_back({e.t_arrival, e.input_len});
  }
  // The client of `id` went away.  A request that still waits in the queue is forgotten at once (returns true; the
  // queue drops its entry when it reaches it); one that is being served ends with its next token and, if the
  // worker would go on with it, is filtered out of its batch.
  bool client_gone(uint64_t id) {
    queue_.mark_client_gone(id);
    auto it = requests_.find(id);
    if (it == requests_.end()) return false;
    if (it->second.t_batched < 0) {
      requests_.erase(it);
      return true;
    }
    it->second.client_alive = false;
    return false;
  }

  // `reason`: why the worker finished the request (proto FinishReason: 0 length, 1 EOS token, 2 stop sequence)
  struct TokenOut { uint64_t request_id; int32_t token; bool finished; int8_t reason = 0; };

  void on_prefill_done(uint64_t op_id, const std::vector<TokenOut>& toks, double now) {
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    Rep& rep = reps_[op.replica];
    rep.busy = false;
    ResidentBatch rb = std::move(op.batch);
    stats_prefill_tokens_ += rb.prompt_tokens;
    const size_t before = rb.request_ids.size();
    deliver_tokens(rb, toks, now, true);
    if (op.kind == ActionType::ZagPrefill) {
      erase_inflight_zag(rep, rb.id);
      maybe_finish_refractory(op.replica, now);
    }
    if (op.kind == ActionType::PrefillPP) {
      // second half of a relayed batch: its KV for layers [k, L) lives here, first half on the new instance
      auto it = relayed_.find(rb.id);
      if (it != relayed_.end()) {
        it->second.batch = rb;
        it->second.pp_done = true;
        if (rb.request_ids.empty()) {  // everything finished at the first token: nothing to migrate
          release_blocks(op.replica, it->second.blocks);
          release_blocks(it->second.new_replica, it->second.blocks);
          finish_relayed_target(it->second);
          relayed_.erase(it);
        }
      }
      reps_[op.replica].relay_wait = false;
      return;
    }
    if (op.kind == ActionType::Prefill && op.peer >= 0) {
      // pushed layer by layer while it ran: the KV is on the decode replica already and the prefill replica has let
      // go of its copy
      release_blocks(op.replica, rb.blocks);
      counters_["blitz_kv_cache_times"] += 1;
      counters_["blitz_progressive_kv_cache_times"] += 1;
      const double kv_mb = cfg_.kv_mb_per_token * rb.prompt_tokens;
      rep.m.flow_out_mb += kv_mb;
      reps_[op.peer].m.flow_in_mb += kv_mb;
      if (rb.request_ids.empty()) {
        release_blocks(op.peer, rb.blocks);
        unlock_target(op.peer, rb.id);
        out_.push_back(make_simple(ActionType::ClearCache, op.peer, rb.id));
        return;
      }
      shrink_blocks(op.peer, rb);
      if (rb.request_ids.size() == before) {
        unlock_target(op.peer, rb.id);
        reps_[op.peer].decode_batches.push_back(std::move(rb));
        return;
      }
      // some requests ended at their first token: the decode replica drops them from the batch it received before
      // it decodes it (the batch stays locked to the replica, and out of its steps, until that is done)
      Action f = make_simple(ActionType::FilterBatch, op.peer, rb.id);
      f.request_ids = rb.request_ids;
      f.op_id = new_op(ActionType::FilterBatch, op.peer, -1, rb);
      ops_[f.op_id].partial = kAdoptAfterFilter;
      out_.push_back(f);
      counters_["blitz_filtered_batches"] += 1;
      return;
    }
    if (rb.request_ids.empty()) {
      release_blocks(op.replica, rb.blocks);
      out_.push_back(make_simple(ActionType::ClearCache, op.replica, rb.id));
      return;
    }
    shrink_blocks(op.replica, rb);
    if (rep.colocated || no_decode_side()) {
      rep.decode_batches.push_back(std::move(rb));  // no decode side: decode where the KV already is
    } else {
      rb.ready_at = now;
      rep.pending_migration.push_back(std::move(rb));
    }
  }

  void on_decode_done(uint64_t op_id, const std::vector<TokenOut>& toks, double now) {
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    Rep& rep = reps_[op.replica];
    rep.busy = false;
    // the worker merged all resident batches into the first one
    ResidentBatch merged = std::move(rep.decode_batches.front());
    for (size_t i = 1; i < rep.decode_batches.size(); ++i) {
      if (!rep.decode_batches[i].in_step) break;
      merge_into(merged, rep.decode_batches[i]);
    }
    size_t consumed = 0;
    while (consumed < rep.decode_batches.size() && rep.decode_batches[consumed].in_step) ++consumed;
    rep.decode_batches.erase(rep.decode_batches.begin(), rep.decode_batches.begin() + consumed);
    merged.in_step = false;
    stats_decode_tokens_ += toks.size();
    const bool dropped_alive = deliver_tokens(merged, toks, now, false);
    if (merged.request_ids.empty()) {
      release_blocks(op.replica, merged.blocks);
      out_.push_back(make_simple(ActionType::ClearCache, op.replica, merged.id));
    } else {
      shrink_blocks(op.replica, merged);
      if (dropped_alive) {
        // the worker would go on decoding for a client that is gone: take those requests out of its batch before
        // the next step (router_v2/src/replica/mod.rs:37-100 filters after every step)
        Action a = make_simple(ActionType::FilterBatch, op.replica, merged.id);
        a.request_ids = merged.request_ids;
        a.op_id = new_op(ActionType::FilterBatch, op.replica, -1, merged);
        out_.push_back(a);
        rep.busy = true;
        counters_["blitz_filtered_batches"] += 1;
      }
      rep.decode_batches.insert(rep.decode_batches.begin(), std::move(merged));
    }
  }

  void on_filter_done(uint64_t op_id, double now) {
    (void)now;
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    if (op.partial == kAdoptAfterFilter) {   // a progressively migrated batch: now it may join the replica's steps
      unlock_target(op.replica, op.batch.id);
      reps_[op.replica].decode_batches.push_back(std::move(op.batch));
      return;
    }
    reps_[op.replica].busy = false;
  }

  void on_migrate_done(uint64_t op_id, double now) {
    (void)now;
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    Rep& src = reps_[op.replica];
    Rep& dst = reps_[op.peer];
    counters_[op.kind == ActionType::Migrate ? "blitz_kv_cache_times" : "blitz_partial_kv_cache_times"] += 1;
    auto count_flow = [&](double fraction) {
      const double kv_mb = cfg_.kv_mb_per_token * op.batch.prompt_tokens * fraction;
      src.m.flow_out_mb += kv_mb;
      dst.m.flow_in_mb += kv_mb;
    };
    if (op.kind == ActionType::Migrate) {
      count_flow(1.0);
      src.migrating = false;
      release_blocks(op.replica, op.batch.blocks);
      unlock_target(op.peer, op.batch.id);
      dst.decode_batches.push_back(std::move(op.batch));
      return;
    }
    auto it = relayed_.find(op.batch.id);
    if (it == relayed_.end()) return;
    Relayed& r = it->second;
    const double first = static_cast<double>(r.next_layer) / std::max<uint32_t>(1, cfg_.model_layers);
    count_flow(op.partial == 1 ? first : 1.0 - first);   // layers [0, k) from the new instance, [k, L) from the old one
    release_blocks(op.replica, r.blocks);
    if (op.partial == 1) { r.fst_done = true; reps_[r.new_replica].m.flying_partial -= 1; }
    if (op.partial == 2) r.snd_done = true;
    if (r.fst_done && r.snd_done) {
      unlock_target(op.peer, r.batch.id);
      dst.decode_batches.push_back(r.batch);
      relayed_.erase(it);
    }
  }

  // A parameter transfer / load finished on `replica` (its op may cover several destinations).
  void on_params_done(uint64_t op_id, double now) {
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    if (op.started >= 0 && !op.targets.empty()) {
      // first-class scale-out metrics: how long the parameter transfer took and what each destination received
      const double dt = std::max(1e-9, now - op.started);
      counters_["blitz_scale_out_total"] += static_cast<double>(op.targets.size());
      counters_["blitz_scale_out_seconds_sum"] += dt;
      gauges_["blitz_last_scale_out_seconds"] = dt;
      gauges_["blitz_last_scale_out_fanout"] = static_cast<double>(op.targets.size());
      if (cfg_.param_gb > 0) gauges_["blitz_last_param_transfer_gbs_per_replica"] = cfg_.param_gb / dt;
    }
    for (int s : op.sources) {
      steer_.set_nvlink_busy(s, false);
      reps_[s].m.marker.reset();
      // every source streams its stripe of the parameters to all targets
      reps_[s].m.flow_out_mb += cfg_.param_gb * 1e3 * static_cast<double>(op.targets.size()) / static_cast<double>(op.sources.size());
    }
    for (int d : op.targets) {
      Rep& rep = reps_[d];
      if (!op.sources.empty()) rep.m.flow_in_mb += cfg_.param_gb * 1e3;
      rep.m.model_loaded = true;
      steer_.record_model_loaded(d);
      steer_.touch_host_cache(steer_.machine_of(d * cfg_.tp), now);
      switch (rep.m.state) {
        case RState::LoadingPrefill: set_state(d, RState::Prefill); break;
        case RState::LoadingDecode: set_state(d, RState::AusDecode); set_state(d, RState::Decode); break;
        case RState::NewPrefill:
          set_state(d, RState::RefractoryPrefill);
          maybe_finish_refractory(d, now);
          break;
        default: break;
      }
    }
  }

  // Relay RPC answered: the new instance handed over `batch_id` at transformer layer `next_layer`
  // (has_batch = false: nothing was left to hand over).
  void on_relay_done(uint64_t op_id, bool has_batch, uint64_t batch_id, int next_layer, double now) {
    if (late_answer(op_id)) return;
    Op op = take_op(op_id);
    const int neu = op.replica, old = op.peer;
    Rep& nrep = reps_[neu];
    if (!has_batch) {
      reps_[old].busy = false;
      reps_[old].relay_wait = false;
      maybe_finish_refractory(neu, now);
      return;
    }
    ResidentBatch rb;
    bool found = false;
    for (auto it = nrep.inflight_zag.begin(); it != nrep.inflight_zag.end(); ++it) {
      if (it->id == batch_id) { rb = *it; nrep.inflight_zag.erase(it); found = true; break; }
    }
    if (!found) { reps_[old].busy = false; reps_[old].relay_wait = false; return; }
    // the pending ZagPrefill op of this batch is answered by the hand-over, not by tokens
    for (auto it = ops_.begin(); it != ops_.end(); ++it)
      if (it->second.kind == ActionType::ZagPrefill && it->second.batch.id == batch_id) { ops_.erase(it); break; }
    nrep.busy = !nrep.inflight_zag.empty();
    Relayed r;
    r.batch = rb; r.new_replica = neu; r.old_replica = old; r.next_layer = std::max(0, next_layer); r.blocks = rb.blocks;
    r.target = pick_decode_target(rb.blocks, rb.id, rb.request_ids.size());
    // both replicas hold KV pages of this batch until their half has migrated
    reps_[old].m.used_blocks += rb.blocks;
    if (r.target >= 0) acquire_target(r.target, rb.blocks, rb.id, rb.request_ids.size());
    Action a = make_simple(ActionType::PrefillPP, old, rb.id);
    a.op_id = new_op(ActionType::PrefillPP, old, neu, rb);
    a.peer = neu; a.num_layer = r.next_layer; a.request_ids = rb.request_ids; a.max_tokens = rb.max_tokens;
    a.dst_ranks = steer_.ranks_of_replica(neu);
    out_.push_back(a);
    r.fst_done = (r.next_layer == 0);  // nothing on the new instance if it had not run a layer yet
    relayed_[rb.id] = r;
    maybe_finish_refractory(neu, now);
  }

  // An RPC of `op_id` failed: a replica is lost (fail-stop workers, src/util/cuda_utils.h:15-22).  `failed_replica`
  // names the participant whose call failed when the caller knows it (a migration or a broadcast has several);
  // without it the replica the operation was issued to is taken.
  void on_failure(uint64_t op_id, double now, int failed_replica = -1) {
    if (late_answer(op_id)) return;
    auto it = ops_.find(op_id);
    if (it == ops_.end()) return;
    counters_["blitz_request_failure"] += 1;
    const int issued_to = it->second.replica;
    lose_replica(failed_replica >= 0 && failed_replica < num_replicas() ? failed_replica : issued_to, now);
    if (ops_.count(op_id)) lose_replica(issued_to, now);  // the named replica was no participant after all
  }

  // The workers' answer to Warmup (how many KV tokens a rank can hold) bounds what the router lets a replica hold.
  void limit_blocks_per_replica(uint32_t blocks) {
    if (blocks > 0 && blocks < cfg_.max_blocks_per_replica) {
      cfg_.max_blocks_per_replica = blocks;
      cfg_.planner.max_blocks_per_replica = blocks;
    }
  }
  uint32_t max_blocks_per_replica() const { return cfg_.max_blocks_per_replica; }

  // A shell with a failure detector reports whether a replica that is out of service answers again; the planner
  // loads into a lost replica only once it does (and its quarantine has passed).
  void set_reachable(int replica, bool ok) {
    if (replica >= 0 && replica < num_replicas()) reps_[replica].reachable = ok;
  }
  bool reachable(int replica) const { return replica >= 0 && replica < num_replicas() && reps_[replica].reachable; }

  // Failure detector verdict (missed heartbeats): the replica is gone even if no operation was in flight on it.
  bool on_replica_unhealthy(int replica, double now) {
    if (replica < 0 || replica >= num_replicas() || reps_[replica].m.state == RState::Inactive) return false;
    counters_["blitz_replica_lost"] += 1;
    lose_replica(replica, now);
    return true;
  }

  // ------------------------------------------------------------------------------------ step
  std::vector<Action> step(double now) {
    if (cfg_.autoscale && !features_.has("manually_scale") && now - last_plan_ >= cfg_.planner_interval_ms * 1e-3) {
      last_plan_ = now;
      run_planner(now);
    }
    if (!pending_scale_.empty()) {
      std::vector<std::pair<int, bool>> group;
      for (auto& pr : pending_scale_) if (reps_[pr.first].m.state == RState::Inactive) group.push_back(pr);
      if (group.empty() || scale_up_group(group, now)) pending_scale_.clear();  // else: no idle source yet, retry
    }
    expire_parked(now);
    for (int r = 0; r < num_replicas(); ++r) drive_replica(r, now);
    {
      // Batches leave for the decode side oldest first, whichever replica prefilled them.  (Scanning the replicas in
      // index order would hand a free destination to replica 0 whenever it has something waiting and starve the
      // others under load; the reference's per-replica watchers race for the destination's lock instead.)
      std::vector<std::pair<double, int>> order;
      for (int r = 0; r < num_replicas(); ++r)
        if (!reps_[r].pending_migration.empty() && !reps_[r].migrating)
          order.emplace_back(reps_[r].pending_migration.front().ready_at, r);
      std::sort(order.begin(), order.end());
      for (auto& o : order) drive_migration(o.second, now);
    }
    drive_relayed(now);
    std::vector<Action> o;
    o.swap(out_);
    return o;
  }

  // Manual scaling (HTTP /modify_cluster_state under `manually_scale`, router_v2/src/server.rs:388-483).
  bool manual_scale(int replica, const std::string& target, double now) {
    auto st = rstate_from_name(target);
    if (!st || replica < 0 || replica >= num_replicas()) return false;
    if (*st == RState::Prefill || *st == RState::Decode) {
      if (reps_[replica].m.state != RState::Inactive && reps_[replica].m.state != RState::ShuttingNull) return false;
      if (reps_[replica].m.state == RState::ShuttingNull) { scale_up_one(replica, *st == RState::Prefill, now); return true; }
      // requests made before the next step() are served by ONE parameter multicast (1 -> N through the switch)
      for (auto& pr : pending_scale_) if (pr.first == replica) return true;
      pending_scale_.emplace_back(replica, *st == RState::Prefill);
      return true;
    }
    if (*st == RState::Inactive) { begin_shutdown(replica, now); return true; }
    return false;
  }

  // ------------------------------------------------------------------------------------ views
  int num_replicas() const { return static_cast<int>(reps_.size()); }
  const ReplicaMetric& metric(int r) const { return reps_[r].m; }
  std::string state_name(int r) const { return rstate_name(reps_[r].m.state); }
  size_t queue_size() const { return queue_.size(); }
  uint64_t waiting_prefill_tokens() const { return queue_.waiting_prefill_tokens(); }
  const std::map<std::string, double>& counters() const { return counters_; }
  const FeatureSet& features() const { return features_; }
  const RequestEntry* request(uint64_t id) const {
    auto it = requests_.find(id);
    return it == requests_.end() ? nullptr : &it->second;
  }
  std::vector<std::string> drain_log() { std::vector<std::string> l; l.swap(log_); return l; }
  // Token deliveries are by far the most frequent output.  A shell that serves many tokens per second switches them
  // from one `Action` each to a compact list that it drains after every completion it reports.
  struct Delivery { uint64_t request_id; int32_t token; bool final; int8_t reason = 0; };
  void set_compact_deliveries(bool on) { compact_deliveries_ = on; }
  std::vector<Delivery> take_deliveries() { std::vector<Delivery> d; d.swap(deliveries_); return d; }
  // Network flow since the last call, per replica that moved anything: (replica, MB in, MB out).  Parameters count
  // with `param_gb`, migrated KV with `kv_mb_per_token` x the batch's prompt tokens (the periodic report of
  // router_v2/src/replica/disaggregation.rs:244-298).
  std::vector<std::tuple<int, double, double>> take_flows() {
    std::vector<std::tuple<int, double, double>> out;
    for (int r = 0; r < num_replicas(); ++r) {
      ReplicaMetric& m = reps_[r].m;
      if (m.flow_in_mb + m.flow_out_mb > 0) out.emplace_back(r, m.flow_in_mb, m.flow_out_mb);
      m.flow_in_mb = m.flow_out_mb = 0;
    }
    return out;
  }
  // Prompt tokens of batches that have been prefilled and wait for their migration to a decode replica.
  uint64_t waiting_migration_tokens() const {
    uint64_t t = 0;
    for (auto& r : reps_)
      for (auto& b : r.pending_migration) t += b.prompt_tokens;
    return t;
  }
  std::string system_metrics_line() const {
    std::ostringstream s;
    s << "System Metrics: prefill_tokens: " << stats_prefill_tokens_ << ", decode_tokens: " << stats_decode_tokens_;
    return s.str();
  }
  std::pair<uint64_t, uint64_t> token_counts() const { return {stats_prefill_tokens_, stats_decode_tokens_}; }
  size_t inflight_ops() const { return ops_.size(); }
  bool idle() const {
    if (!queue_.empty() || !ops_.empty() || !relayed_.empty()) return false;
    for (auto& r : reps_)
      if (!r.decode_batches.empty() || !r.pending_migration.empty() || !r.inflight_zag.empty()) return false;
    return true;
  }
  uint64_t total_used_blocks() const {
    uint64_t t = 0;
    for (auto& r : reps_) t += r.m.used_blocks;
    return t;
  }
  ScaleTarget last_target() const { return last_target_; }

 private:
  struct ResidentBatch {
    uint64_t id = 0;
    std::vector<uint64_t> request_ids;
    uint32_t max_tokens = 0, prompt_tokens = 0, blocks = 0;
    bool in_step = false;
    double ready_at = 0;   // when its prefill finished (order of service in the migration queue)
  };
  struct Rep {
    ReplicaMetric m;
    bool colocated = false;
    double lost_at = -1e18;   // when the replica was last declared lost
    bool reachable = true;    // failure detector's view (a shell without a detector leaves it true)
    bool busy = false;        // an inference RPC is in flight
    bool migrating = false;   // this source has a migration in flight
    bool relay_wait = false;  // OldPrefill parked in the relay queue
    bool last_was_decode = false;
    std::deque<ResidentBatch> pending_migration;
    std::vector<ResidentBatch> decode_batches;
    std::vector<ResidentBatch> inflight_zag;
    uint32_t zag_seq = 0;
    double zag_started = 0;
    int partner = -1;         // OldPrefill <-> NewPrefill pairing
    int incoming = 0;         // migrations in flight towards this replica
    std::vector<uint64_t> incoming_batches;  // their batch ids (for the transfer-slot rule)
    uint32_t incoming_seqs = 0;              // sequences of those batches
  };
  static constexpr int kAdoptAfterFilter = 3;   // Op::partial of a FilterBatch that precedes a batch's first decode step
  struct Op {
    ActionType kind;
    int replica = -1, peer = -1, partial = 0;
    ResidentBatch batch;
    std::vector<int> sources, targets;
    double started = -1;   // parameter transfers: when the operation was issued
  };
  struct Cancelled {
    uint64_t batch_id = 0;
    std::vector<int> clear_on;   // surviving replicas that may still build state for the batch
  };
  struct Relayed {
    ResidentBatch batch;
    int new_replica = -1, old_replica = -1, target = -1, next_layer = 0;
    uint32_t blocks = 0;
    bool pp_done = false, fst_started = false, snd_started = false, fst_done = false, snd_done = false;
  };

  // ---------------- helpers
  uint64_t new_op(ActionType k, int replica, int peer, const ResidentBatch& b) {
    Op op;
    op.kind = k; op.replica = replica; op.peer = peer; op.batch = b;
    ops_[++next_op_] = op;
    return next_op_;
  }
  Op take_op(uint64_t id) {
    auto it = ops_.find(id);
    if (it == ops_.end()) throw std::invalid_argument("unknown op id");
    Op op = std::move(it->second);
    ops_.erase(it);
    return op;
  }
  Action make_simple(ActionType t, int replica, uint64_t batch_id) {
    Action a;
    a.type = t; a.replica = replica; a.batch_id = batch_id;
    return a;
  }
  void log_transition(int r, RState a, RState b, bool boot = false) {
    std::ostringstream s;
    s << "Replica<" << r << "> " << (boot ? "boot" : rstate_name(a)) << " => " << rstate_name(b);
    log_.push_back(s.str());
  }
  void set_state(int r, RState s) {
    RState old = reps_[r].m.state;
    if (old == s) return;
    if (!transition_allowed(old, s))
      throw std::logic_error(std::string("illegal transition ") + rstate_name(old) + " => " + rstate_name(s));
    reps_[r].m.state = s;
    // dst_mutex invariant: a replica holds its own mutex whenever it is not a decode target
    if (s == RState::Decode) reps_[r].m.dst_busy = target_full(reps_[r]);
    else if (old == RState::Decode) reps_[r].m.dst_busy = true;
    log_transition(r, old, s);
  }
  int num_in_state(RState s) const {
    int n = 0;
    for (auto& r : reps_) n += r.m.state == s;
    return n;
  }
  void release_blocks(int r, uint32_t blocks) {
    reps_[r].m.used_blocks = reps_[r].m.used_blocks >= blocks ? reps_[r].m.used_blocks - blocks : 0;
  }
  uint32_t blocks_of(const ResidentBatch& b) const {
    uint64_t t = 0;
    for (uint64_t id : b.request_ids) {
      const RequestEntry& e = requests_.at(id);
      t += (e.input_len + e.max_new_tokens + cfg_.block_size - 1) / cfg_.block_size;
    }
    return static_cast<uint32_t>(t);
  }
  // FilterBatch accounting: finished requests give their blocks back (router_v2/src/replica/mod.rs:251-269)
  void shrink_blocks(int r, ResidentBatch& b) {
    const uint32_t nb = blocks_of(b);
    if (nb < b.blocks) release_blocks(r, b.blocks - nb);
    b.blocks = nb;
    b.max_tokens = nb * cfg_.block_size;
  }
  void merge_into(ResidentBatch& a, const ResidentBatch& b) {
    a.request_ids.insert(a.request_ids.end(), b.request_ids.begin(), b.request_ids.end());
    a.blocks += b.blocks;
    a.max_tokens += b.max_tokens;
  }
  // Returns true when a request was finished here although the worker still runs it (its client went away).
  bool deliver_tokens(ResidentBatch& b, const std::vector<TokenOut>& toks, double now, bool prefill) {
    bool dropped_alive = false;
    for (const TokenOut& t : toks) {
      auto it = requests_.find(t.request_id);
      if (it == requests_.end()) continue;
      RequestEntry& e = it->second;
      if (prefill) {
        e.t_first_token = now;  // "PrefillDone" precedes the first token (router_v2/src/infer.rs:330-333)
      } else {
        if (e.generated == 1) e.t_first_decode_token = now;
        if (e.generated >= 1 && e.t_last_token >= 0 && e.generated >= 2) e.tbt.push_back(now - e.t_last_token);
      }
      e.generated += 1;
      e.t_last_token = now;
      // a client that left ends its request at a decode step, where the worker's batch can be filtered before the
      // next step; ending it at the prefill token would leave the batch that is about to migrate out of step with
      // the worker's copy of it
      const bool fin = t.finished || e.generated >= e.max_new_tokens || (!prefill && !e.client_alive);
      if (fin && !t.finished && e.generated < e.max_new_tokens) dropped_alive = true;
      // a request the router ends itself (token budget reached, client gone) is a length stop
      const int8_t reason = t.finished ? t.reason : int8_t{0};
      if (compact_deliveries_) {
        deliveries_.push_back({t.request_id, t.token, fin, reason});
      } else {
        Action a;
        a.type = ActionType::Deliver; a.request_id = t.request_id; a.token = t.token; a.final = fin;
        a.finish_reason = reason;
        out_.push_back(a);
      }
      if (fin) {
        b.request_ids.erase(std::remove(b.request_ids.begin(), b.request_ids.end(), t.request_id), b.request_ids.end());
        counters_["blitz_request_success"] += 1;
        finished_[t.request_id] = e;
        requests_.erase(it);
      }
    }
    return dropped_alive;
  }
  void erase_inflight_zag(Rep& rep, uint64_t batch_id) {
    for (auto it = rep.inflight_zag.begin(); it != rep.inflight_zag.end(); ++it)
      if (it->id == batch_id) { rep.inflight_zag.erase(it); break; }
    rep.busy = !rep.inflight_zag.empty();
  }
  static uint32_t resident_seqs(const Rep& r) {
    size_t n = r.incoming_seqs;
    for (auto& b : r.decode_batches) n += b.request_ids.size();
    return static_cast<uint32_t>(n);
  }
  int pick_decode_target(uint32_t need_blocks, uint64_t batch_id, size_t nseqs = 0) const {
    int best = -1;
    uint32_t best_used = UINT32_MAX;
    const uint64_t slots = static_cast<uint64_t>(std::max(1, cfg_.kv_transfer_slots));
    for (int d = 0; d < num_replicas(); ++d) {
      const Rep& r = reps_[d];
      if (r.m.state != RState::Decode || r.m.dst_busy) continue;
      if (cfg_.max_batch_seqs > 0 && resident_seqs(r) > 0 && resident_seqs(r) + nseqs > cfg_.max_batch_seqs) continue;
      bool slot_taken = false;
      for (uint64_t other : r.incoming_batches) slot_taken = slot_taken || (other % slots == batch_id % slots);
      if (slot_taken) continue;
      if (r.m.used_blocks + need_blocks > cfg_.max_blocks_per_replica) continue;
      // The reference takes the first decode replica whose lock is free (a try_lock scan from index 0; its
      // `decode_load_balance` feature is declared but unimplemented), which piles every request on the first one
      // while the others idle.  Here the least loaded one is taken; `decode_first_fit` restores the scan.
      if (features_.has("decode_first_fit")) return d;
      if (r.m.used_blocks < best_used) { best = d; best_used = r.m.used_blocks; }
    }
    return best;
  }
  bool target_full(const Rep& r) const { return r.incoming >= std::max(1, cfg_.max_incoming_migrations); }
  void acquire_target(int d, uint32_t blocks, uint64_t batch_id, size_t nseqs = 0) {
    reps_[d].incoming += 1;
    reps_[d].incoming_batches.push_back(batch_id);
    reps_[d].incoming_seqs += static_cast<uint32_t>(nseqs);
    incoming_seqs_of_[batch_id] = static_cast<uint32_t>(nseqs);
    reps_[d].m.dst_busy = reps_[d].m.state != RState::Decode || target_full(reps_[d]);
    reps_[d].m.used_blocks += blocks;
  }
  void unlock_target(int d, uint64_t batch_id) {
    Rep& r = reps_[d];
    r.incoming = std::max(0, r.incoming - 1);
    auto it = std::find(r.incoming_batches.begin(), r.incoming_batches.end(), batch_id);
    if (it != r.incoming_batches.end()) r.incoming_batches.erase(it);
    auto sq = incoming_seqs_of_.find(batch_id);
    if (sq != incoming_seqs_of_.end()) {
      r.incoming_seqs = r.incoming_seqs >= sq->second ? r.incoming_seqs - sq->second : 0;
      incoming_seqs_of_.erase(sq);
    }
    r.m.dst_busy = r.m.state != RState::Decode || target_full(r);
  }
  void finish_relayed_target(Relayed& r) {
    if (r.target >= 0) {
      release_blocks(r.target, r.blocks);
      unlock_target(r.target, r.batch.id);
    }
  }

  // ---------------- per-replica driving
  void drive_replica(int r, double now) {
    Rep& rep = reps_[r];
    rep.m.loop_cnt += 1;
    switch (rep.m.state) {
      case RState::Prefill:
      case RState::ShuttingPrefill:
      case RState::MutatingToDecode:
        // A replica that also holds decode batches (colocated deployment, or no decode side exists)
        // alternates: a waiting prompt goes first after a decode step, otherwise it keeps decoding.
        if (!rep.busy && !rep.decode_batches.empty()) {
          const bool prefill_first = rep.m.state == RState::Prefill && rep.last_was_decode && !queue_.empty();
          if (prefill_first && try_prefill(r, now)) { rep.last_was_decode = false; return; }
          if (try_decode(r)) { rep.last_was_decode = true; return; }
        }
        if (rep.m.state == RState::Prefill && try_prefill(r, now)) rep.last_was_decode = false;
        if (rep.m.state == RState::ShuttingPrefill && !rep.busy && rep.pending_migration.empty() && !rep.migrating &&
            rep.decode_batches.empty())
          park(r, now);
        if (rep.m.state == RState::MutatingToDecode && !rep.busy && !rep.migrating) {
          // flush the batches awaiting migration into itself, then serve as a decode replica
          while (!rep.pending_migration.empty()) {
            rep.decode_batches.push_back(rep.pending_migration.front());
            rep.pending_migration.pop_front();
          }
          set_state(r, RState::Decode);
        }
        break;
      case RState::OldPrefill:
        if (!rep.busy) {
          if (!try_relay(r, now)) try_prefill(r, now);
        }
        break;
      case RState::NewPrefill:
        try_zag_prefill(r, now);
        break;
      case RState::RefractoryPrefill:
        maybe_finish_refractory(r, now);
        break;
      case RState::Decode:
      case RState::ShuttingDecode:
        try_decode(r);
        if (rep.m.state == RState::ShuttingDecode && !rep.busy && rep.decode_batches.empty() && rep.incoming == 0)
          park(r, now);
        break;
      default: break;
    }
  }

  bool try_prefill(int r, double now) {
    Rep& rep = reps_[r];
    if (rep.busy || queue_.empty()) return false;
    if (rep.m.used_blocks > cfg_.max_blocks_per_replica) return false;
    const uint32_t free_blocks = cfg_.max_blocks_per_replica - rep.m.used_blocks;
    size_t max_size = cfg_.max_batch_seqs;
    if (max_size > 0 && (rep.colocated || no_decode_side())) {
      // what it prefills stays here for decoding: leave room for it in this replica's decode step
      const uint32_t held = resident_seqs(rep);
      if (held >= max_size) return false;
      max_size -= held;
    }
    auto nb = queue_.next_batch(std::nullopt, prefill_share(), cfg_.max_total_tokens, free_blocks, max_size);
    if (!nb) return false;
    ResidentBatch rb;
    rb.id = nb->batch.id; rb.request_ids = nb->batch.request_ids; rb.max_tokens = nb->batch.max_tokens;
    rb.prompt_tokens = nb->batch.prompt_tokens; rb.blocks = nb->batch.max_tokens / cfg_.block_size;
    rep.m.used_blocks += rb.blocks;
    for (auto& e : nb->entries) requests_[e.id].t_batched = now;
    rep.busy = true;
    // Layer-progressive migration (`PREFILL_CASE_MIGRATE_PROGRESSIVE`, proto/generate.proto:315-326; the reference
    // declares the case and never issues it): the decode replica is chosen now and reserves its pages while the prefill
    // runs, and the prefill replica pushes every layer's KV as soon as that layer has run.  Without a free decode
    // replica at this moment the batch takes the ordinary path (prefill, then a migration of all layers).
    int dst = -1;
    if (features_.has("migrate_progressive") && !rep.colocated && !no_decode_side())
      dst = pick_decode_target(rb.blocks, rb.id, rb.request_ids.size());
    Action a = make_simple(ActionType::Prefill, r, rb.id);
    if (dst >= 0) {
      acquire_target(dst, rb.blocks, rb.id, rb.request_ids.size());
      a.peer = dst;
      a.src_ranks = steer_.ranks_of_replica(r); a.dst_ranks = steer_.ranks_of_replica(dst);
    }
    a.op_id = new_op(ActionType::Prefill, r, dst, rb);
    a.request_ids = rb.request_ids; a.max_tokens = rb.max_tokens;
    out_.push_back(a);
    return true;
  }

  // Prefill token budget of the batch an idle prefill replica takes now.  By default, as in the reference, whichever
  // replica asks first takes everything that fits its budget.  With the feature `prefill_share_idle` the waiting
  // prompt tokens are shared among the prefill replicas that are idle at this moment (a lone idle replica still takes
  // a full batch).  In the simulator this lowers the median TTFT at low load (106 -> 77 ms) but leaves no idle
  // replica for the arrivals that follow a burst (p99 170 -> 192 ms) and is neutral under load, so it is opt-in.
  uint32_t prefill_share() const {
    if (!features_.has("prefill_share_idle")) return cfg_.max_prefill_tokens;
    uint32_t idle = 0;
    for (auto& r : reps_)
      if (r.m.state == RState::Prefill && !r.busy && r.decode_batches.empty()) ++idle;
    if (idle <= 1) return cfg_.max_prefill_tokens;
    const uint64_t waiting = queue_.waiting_prefill_tokens();
    const uint32_t share = static_cast<uint32_t>((waiting + idle - 1) / idle);
    return std::min(cfg_.max_prefill_tokens, std::max(share, queue_.front_input_len()));
  }

  void try_zag_prefill(int r, double now) {
    Rep& rep = reps_[r];
    // in-flight limit decays from `zigzag_req_limit` by one every `zigzag_decay_ms`, floor `zigzag_req_floor`
    uint32_t limit = cfg_.zigzag_req_limit;
    const uint32_t decay = static_cast<uint32_t>((now - rep.zag_started) * 1e3 / std::max(1.0, cfg_.zigzag_decay_ms));
    limit = limit > decay ? limit - decay : 0;
    limit = std::max(limit, cfg_.zigzag_req_floor);
    if (rep.inflight_zag.size() >= limit || queue_.empty()) return;
    if (rep.m.used_blocks > cfg_.max_blocks_per_replica) return;
    auto nb = queue_.next_batch(std::nullopt, cfg_.max_prefill_tokens, cfg_.max_total_tokens,
                                cfg_.max_blocks_per_replica - rep.m.used_blocks, cfg_.max_batch_seqs);
    if (!nb) return;
    ResidentBatch rb;
    rb.id = nb->batch.id; rb.request_ids = nb->batch.request_ids; rb.max_tokens = nb->batch.max_tokens;
    rb.prompt_tokens = nb->batch.prompt_tokens; rb.blocks = nb->batch.max_tokens / cfg_.block_size;
    rep.m.used_blocks += rb.blocks;
    for (auto& e : nb->entries) requests_[e.id].t_batched = now;
    rep.inflight_zag.push_back(rb);
    rep.busy = true;
    Action a = make_simple(ActionType::ZagPrefill, r, rb.id);
    a.op_id = new_op(ActionType::ZagPrefill, r, -1, rb);
    a.request_ids = rb.request_ids; a.max_tokens = rb.max_tokens; a.zag_seq = rep.zag_seq++;
    out_.push_back(a);
  }

  bool try_relay(int old, double now) {
    (void)now;
    Rep& orep = reps_[old];
    if (orep.relay_wait) return true;
    int neu = orep.partner;
    if (neu < 0) return false;
    Rep& nrep = reps_[neu];
    const bool live = nrep.m.state == RState::NewPrefill || nrep.m.state == RState::RefractoryPrefill;
    if (!live) {  // partner finished loading: leave the pairing
      orep.partner = -1;
      set_state(old, RState::Prefill);
      return false;
    }
    if (nrep.inflight_zag.empty()) return false;
    if (pick_decode_target(nrep.inflight_zag.front().blocks, nrep.inflight_zag.front().id) < 0 && num_in_state(RState::Decode) > 0)
      return false;
    orep.busy = true;
    orep.relay_wait = true;
    Action a = make_simple(ActionType::Relay, neu, 0);
    a.peer = old;
    a.op_id = new_op(ActionType::Relay, neu, old, ResidentBatch{});
    a.src_ranks = steer_.ranks_of_replica(old);
    // while draining, the head task is about to finish locally: take the second one
    a.final = nrep.m.state == RState::RefractoryPrefill;
    out_.push_back(a);
    return true;
  }

  void maybe_finish_refractory(int r, double now) {
    (void)now;
    Rep& rep = reps_[r];
    if (rep.m.state != RState::RefractoryPrefill || !rep.inflight_zag.empty()) return;
    for (auto& op : ops_)
      if (op.second.kind == ActionType::Relay && op.second.replica == r) return;  // a relay is still being answered
    set_state(r, RState::Prefill);
    rep.busy = false;
    if (rep.partner >= 0) {
      Rep& old = reps_[rep.partner];
      if (old.m.state == RState::OldPrefill && !old.relay_wait) {
        old.partner = -1;
        set_state(rep.partner, RState::Prefill);
      }
      rep.partner = -1;
    }
  }

  bool try_decode(int r) {
    Rep& rep = reps_[r];
    if (rep.busy || rep.decode_batches.empty()) return false;
    Action a = make_simple(ActionType::Decode, r, rep.decode_batches.front().id);
    ResidentBatch all;
    all.id = rep.decode_batches.front().id;
    for (auto& b : rep.decode_batches) {
      b.in_step = true;
      a.batch_ids.push_back(b.id);
      all.request_ids.insert(all.request_ids.end(), b.request_ids.begin(), b.request_ids.end());
    }
    a.request_ids = all.request_ids;
    a.op_id = new_op(ActionType::Decode, r, -1, all);
    rep.busy = true;
    out_.push_back(a);
    return true;
  }

  void drive_migration(int src, double now) {
    (void)now;
    Rep& rep = reps_[src];
    if (rep.migrating || rep.pending_migration.empty()) return;
    ResidentBatch& b = rep.pending_migration.front();
    const int dst = pick_decode_target(b.blocks, b.id, b.request_ids.size());
    if (dst < 0) {
      // no decode side is left (it was lost after this batch was queued for it): decode where the KV already is,
      // as a prefill that completes in that situation does
      if (no_decode_side() && (rep.m.state == RState::Prefill || rep.m.state == RState::ShuttingPrefill)) {
        rep.decode_batches.push_back(std::move(b));
        rep.pending_migration.pop_front();
      }
      return;
    }
    acquire_target(dst, b.blocks, b.id, b.request_ids.size());
    rep.migrating = true;
    Action a = make_simple(ActionType::Migrate, src, b.id);
    a.peer = dst; a.request_ids = b.request_ids; a.max_tokens = b.max_tokens;
    a.src_ranks = steer_.ranks_of_replica(src); a.dst_ranks = steer_.ranks_of_replica(dst);
    a.op_id = new_op(ActionType::Migrate, src, dst, b);
    out_.push_back(a);
    rep.pending_migration.pop_front();
  }

  void drive_relayed(double now) {
    (void)now;
    for (auto& kv : relayed_) {
      Relayed& r = kv.second;
      if (r.target < 0) {
        r.target = pick_decode_target(r.blocks, r.batch.id, r.batch.request_ids.size());
        if (r.target < 0) continue;
        acquire_target(r.target, r.blocks, r.batch.id, r.batch.request_ids.size());
      }
      auto emit = [&](int part, int from) {
        Action a = make_simple(ActionType::MigratePartial, from, r.batch.id);
        a.peer = r.target; a.partial = part; a.num_layer = r.next_layer; a.request_ids = r.batch.request_ids;
        a.max_tokens = r.batch.max_tokens;
        a.src_ranks = steer_.ranks_of_replica(from); a.dst_ranks = steer_.ranks_of_replica(r.target);
        Op op;
        op.kind = ActionType::MigratePartial; op.replica = from; op.peer = r.target; op.partial = part; op.batch = r.batch;
        ops_[++next_op_] = op;
        a.op_id = next_op_;
        out_.push_back(a);
      };
      if (!r.fst_started && !r.fst_done) {
        r.fst_started = true;
        reps_[r.new_replica].m.flying_partial += 1;
        emit(1, r.new_replica);
      }
      if (r.pp_done && !r.snd_started) {
        r.snd_started = true;
        if (r.fst_done && r.next_layer == 0) release_blocks(r.new_replica, r.blocks);
        emit(2, r.old_replica);
      }
    }
  }

  // ---------------- autoscaling
  static bool is_prefill_side(RState s) {
    return s == RState::Prefill || s == RState::NewPrefill || s == RState::OldPrefill || s == RState::RefractoryPrefill ||
           s == RState::LoadingPrefill || s == RState::AusPrefill;
  }
  static bool is_decode_side(RState s) {
    return s == RState::Decode || s == RState::AusDecode || s == RState::LoadingDecode || s == RState::MutatingToDecode;
  }
  void run_planner(double now) {
    PlannerView v;
    for (auto& r : reps_) {
      if (is_prefill_side(r.m.state)) { v.num_prefill += 1; v.prefill_used_blocks += r.m.used_blocks; }
      if (is_decode_side(r.m.state)) { v.num_decode += 1; v.decode_used_blocks += r.m.used_blocks; }
    }
    if (v.num_prefill == 0 || v.num_decode == 0) {
      bool any_colocated = false;
      for (auto& r : reps_) any_colocated = any_colocated || r.colocated;
      if (any_colocated) return;  // colocated deployments do not autoscale roles
      // a disaggregated deployment lost every replica of one role (failures): restore it before anything else
      if (v.num_decode == 0 && !scale_up(false, now)) {
        // nothing to load into: turn the least loaded of two or more prefill replicas into the decode side
        int pick = -1, n_prefill = 0;
        for (int r = 0; r < num_replicas(); ++r) {
          if (reps_[r].m.state != RState::Prefill || reps_[r].partner >= 0) continue;
          ++n_prefill;
          if (pick < 0 || reps_[r].m.used_blocks < reps_[pick].m.used_blocks) pick = r;
        }
        if (n_prefill >= 2) set_state(pick, RState::MutatingToDecode);
      }
      if (v.num_prefill == 0 && !scale_up(true, now)) {
        // nothing to load into either: the least loaded decode replica takes the prefill role; if it was the only
        // one it keeps its resident batches and serves both phases until a replica can be added
        int pick = -1;
        for (int r = 0; r < num_replicas(); ++r) {
          if (reps_[r].m.state != RState::Decode) continue;
          if (pick < 0 || reps_[r].m.used_blocks < reps_[pick].m.used_blocks) pick = r;
        }
        if (pick >= 0) {
          set_state(pick, RState::ShuttingNull);
          reps_[pick].m.shutting_since = -1;
          set_state(pick, RState::Prefill);
        }
      }
      return;
    }
    v.waiting_prefill_tokens = queue_.waiting_prefill_tokens();
    if (arrival_signal_) {
      const double w = std::max(1.0, cfg_.planner.arrival_window_ms) * 1e-3;
      while (!arrivals_.empty() && arrivals_.front().first < now - w) arrivals_.pop_front();
      uint64_t tokens = 0;
      for (auto& a : arrivals_) tokens += a.second;
      v.arrival_tokens_per_sec = static_cast<double>(tokens) / w;
    }
    ScaleTarget t = plan_scale(cfg_.planner, v);
    // The reference sizes the decode side by KV memory only.  A decode replica is also full when it holds as many
    // sequences as a worker step carries: when the decode side is nearly full in that sense (or prefilled batches
    // already wait for room), ask for one more decode replica, and never shrink it then.
    if (cfg_.max_batch_seqs > 0 && v.num_decode > 0) {
      uint64_t seqs = 0, waiting = 0;
      for (auto& r : reps_) {
        if (is_decode_side(r.m.state)) seqs += resident_seqs(r);
        for (auto& b : r.pending_migration) waiting += b.request_ids.size();
      }
      const double util = static_cast<double>(seqs + waiting) / (static_cast<double>(v.num_decode) * cfg_.max_batch_seqs);
      if (util > cfg_.planner.decode_upper && v.num_decode < cfg_.planner.max_decode) t.d_decode = std::max(t.d_decode, 1);
      else if (util > cfg_.planner.decode_lower) t.d_decode = std::max(t.d_decode, 0);
    }
    last_target_ = t;
    gauges_["blitz_prefill_replica"] = v.num_prefill;
    gauges_["blitz_decode_replica"] = v.num_decode;
    if (t.d_prefill == 0 && t.d_decode == 0) { last_logged_ = {0, 0}; return; }
    const bool changed = std::make_pair(t.d_prefill, t.d_decode) != last_logged_;
    last_logged_ = {t.d_prefill, t.d_decode};
    std::ostringstream s;
    s << "Control signal: P" << std::showpos << t.d_prefill << " D" << t.d_decode << std::noshowpos << " | Prefill thpt : ["
      << t.bands.prefill_thpt_min << "," << t.bands.prefill_thpt_max << "]; KV$ : [" << t.bands.prefill_kv_min << ","
      << t.bands.prefill_kv_max << "] | Decode Mem : [" << t.bands.decode_mem_min << "," << t.bands.decode_mem_max
      << "]; KV$ : [" << t.bands.decode_kv_min << "," << t.bands.decode_kv_max << "]";
    if (changed) log_.push_back(s.str());  // a standing signal is logged once, not every tick
    int dp = t.d_prefill, dd = t.d_decode;
    // decode shortage with prefill surplus: mutate a prefill replica in place, no reload
    if (dd > 0 && dp < 0 && features_.has("mutate")) {
      for (int r = 0; r < num_replicas() && dd > 0 && dp < 0; ++r) {
        if (reps_[r].m.state == RState::Prefill && !reps_[r].colocated && reps_[r].partner < 0) {
          set_state(r, RState::MutatingToDecode);
          dd -= 1; dp += 1;
        }
      }
    }
    std::vector<std::pair<int, bool>> group;
    for (; dp > 0; --dp) if (!scale_up(true, now, &group)) break;
    for (; dd > 0; --dd) if (!scale_up(false, now, &group)) break;
    if (!group.empty()) scale_up_group(group, now);
    // scale down only on a signal that has persisted for the scale-down threshold: with short planner horizons the
    // raw signal flips within milliseconds and replicas would bounce between serving and draining
    const double patience = cfg_.planner.scale_down_threshold_ms * 1e-3;
    if (dp < 0) { if (down_since_p_ < 0) down_since_p_ = now; } else down_since_p_ = -1;
    if (dd < 0) { if (down_since_d_ < 0) down_since_d_ = now; } else down_since_d_ = -1;
    if (dp < 0 && now - down_since_p_ >= patience) scale_down(true, now);
    if (dd < 0 && now - down_since_d_ >= patience) scale_down(false, now);
  }

  bool quarantined(int r, double now) const {
    return !reps_[r].reachable || (now - reps_[r].lost_at) * 1e3 < cfg_.quarantine_ms;
  }
  bool no_decode_side() const {
    return num_in_state(RState::Decode) + num_in_state(RState::AusDecode) + num_in_state(RState::MutatingToDecode) +
               num_in_state(RState::LoadingDecode) == 0;
  }

  // `group`: inactive replicas chosen so far in this planner turn; they start together (one multicast).
  bool scale_up(bool prefill, double now, std::vector<std::pair<int, bool>>* group = nullptr) {
    // 1. revive a replica that is shutting down
    const RState shutting = prefill ? RState::ShuttingPrefill : RState::ShuttingDecode;
    for (int r = 0; r < num_replicas(); ++r)
      if (reps_[r].m.state == shutting) { set_state(r, prefill ? RState::Prefill : RState::Decode); return true; }
    // 2. reuse a parked replica whose weights are still resident
    for (int r = 0; r < num_replicas(); ++r)
      if (reps_[r].m.state == RState::ShuttingNull) { scale_up_one(r, prefill, now); return true; }
    // 3. bring up an inactive replica
    for (int r = 0; r < num_replicas(); ++r) {
      if (reps_[r].m.state != RState::Inactive || quarantined(r, now)) continue;
      if (!group) return scale_up_one(r, prefill, now);
      bool taken = false;
      for (auto& pr : *group) taken = taken || pr.first == r;
      if (taken) continue;
      group->emplace_back(r, prefill);
      return true;
    }
    return false;
  }

  // Bring several inactive replicas up with one parameter transfer: every idle loaded source (at most two) streams
  // a stripe of every unit to ALL destinations at once (the worker uses one multimem store per 16 bytes when there
  // is more than one destination), so the time is that of one transfer whatever the fan-out.  The reference builds
  // chains and per-destination sends instead (router_v2/src/replica/cybernetics/exec_blitz.rs:21-1198).
  bool scale_up_group(const std::vector<std::pair<int, bool>>& targets, double now) {
    if (targets.size() == 1 || features_.has("impl_sllm")) {
      bool any = false;
      for (auto& t : targets) any = scale_up_one(t.first, t.second, now) || any;
      return any;
    }
    std::vector<int> sources;
    auto is_target = [&](int s) { for (auto& t : targets) if (t.first == s) return true; return false; };
    for (int pass = 0; pass < 2 && sources.empty(); ++pass)
      for (int s = 0; s < num_replicas(); ++s) {
        const RState st = reps_[s].m.state;
        const bool preferred = st == RState::Decode || st == RState::ShuttingDecode || st == RState::ShuttingNull ||
                               (features_.has("unidirect") && st == RState::Prefill) || reps_[s].colocated;
        if ((pass == 1 || preferred) && reps_[s].m.model_loaded && !steer_.nvlink_busy(s) && !is_target(s)) sources.push_back(s);
      }
    if (sources.empty()) return false;
    if (sources.size() < 2)  // a second source doubles what each destination can receive
      for (int s = 0; s < num_replicas() && sources.size() < 2; ++s)
        if (reps_[s].m.model_loaded && !steer_.nvlink_busy(s) && !is_target(s) && s != sources[0]) sources.push_back(s);
    if (sources.size() > 2) sources.resize(2);
    const bool multi = sources.size() > 1;
    const bool nvl = features_.has("impl_nvl");
    Action a;
    a.replica = targets.front().first;
    a.mock = features_.has("mock_transfer") || features_.has("motiv");
    a.type = multi ? ActionType::TanzBroadcast : (nvl ? ActionType::NvlBroadcast : ActionType::RdmaBroadcast);
    if (a.type != ActionType::RdmaBroadcast) counters_["blitz_nvbroadcast_times"] += 1;
    counters_["blitz_scale_up_times"] += static_cast<double>(targets.size());
    Op op;
    op.replica = a.replica;
    for (int s2 : sources) {
      steer_.set_nvlink_busy(s2, true);
      reps_[s2].m.marker = multi ? RState::TanzCasting : (nvl ? RState::NvlCasting : RState::RdmaCasting);
      for (int rk : steer_.ranks_of_replica(s2)) a.src_ranks.push_back(rk);
    }
    op.sources = sources;
    bool any_live = false;
    for (auto& t : targets) {
      const int r = t.first;
      Rep& rep = reps_[r];
      for (int rk : steer_.ranks_of_replica(r)) a.dst_ranks.push_back(rk);
      op.targets.push_back(r);
      const bool live = t.second && features_.has("live");
      if (live) {
        any_live = true;
        set_state(r, RState::NewPrefill);
        rep.zag_started = now;
        rep.zag_seq = 0;
        for (int o = 0; o < num_replicas(); ++o) {
          if (reps_[o].m.state == RState::Prefill && reps_[o].partner < 0 && !reps_[o].colocated) {
            set_state(o, RState::OldPrefill);
            reps_[o].partner = r;
            rep.partner = o;
            break;
          }
        }
      } else {
        set_state(r, t.second ? RState::LoadingPrefill : RState::LoadingDecode);
      }
    }
    a.live = any_live;
    op.kind = a.type;
    op.started = now;
    ops_[++next_op_] = op;
    a.op_id = next_op_;
    out_.push_back(a);
    return true;
  }

  bool scale_up_one(int r, bool prefill, double now) {
    Rep& rep = reps_[r];
    if (rep.m.state == RState::ShuttingNull) {
      rep.m.shutting_since = -1;
      if (prefill) set_state(r, RState::Prefill);
      else { set_state(r, RState::AusDecode); set_state(r, RState::Decode); }
      return true;
    }
    if (rep.m.state != RState::Inactive) return false;
    Action a;
    a.replica = r;
    a.dst_ranks = steer_.ranks_of_replica(r);
    a.mock = features_.has("mock_transfer") || features_.has("motiv");
    Op op;
    op.replica = r; op.targets = {r};
    if (features_.has("impl_sllm")) {
      a.type = ActionType::LoadParams;
      const int machine = steer_.machine_of(r * cfg_.tp);
      bool hit = features_.has("cache_all_hit") || (features_.has("cache_replace") && steer_.host_cache_hit(machine, now));
      if (features_.has("cache_all_miss")) hit = false;
      a.load_case = hit ? 0 : 1;
      set_state(r, prefill ? RState::LoadingPrefill : RState::LoadingDecode);
    } else {
      // sources: decode-side replicas (their NVLink egress is idle: KV flows into them), parked replicas,
      // and prefill replicas when `unidirect` is on (router_v2/src/replica/cybernetics/exec_blitz.rs:1200-1243)
      std::vector<int> sources;
      for (int s = 0; s < num_replicas(); ++s) {
        const RState st = reps_[s].m.state;
        const bool ok = st == RState::Decode || st == RState::ShuttingDecode || st == RState::ShuttingNull ||
                        (features_.has("unidirect") && st == RState::Prefill) || reps_[s].colocated;
        if (ok && reps_[s].m.model_loaded && !steer_.nvlink_busy(s)) sources.push_back(s);
      }
      if (sources.empty())
        for (int s = 0; s < num_replicas(); ++s)  // last resort: any loaded replica
          if (reps_[s].m.model_loaded && !steer_.nvlink_busy(s) && s != r) sources.push_back(s);
      if (sources.empty()) return false;
      const bool multi = features_.has("impl_tanz") && sources.size() > 1;
      const bool nvl = features_.has("impl_nvl");
      a.type = multi ? ActionType::TanzBroadcast : (nvl ? ActionType::NvlBroadcast : ActionType::RdmaBroadcast);
      if (a.type != ActionType::RdmaBroadcast) counters_["blitz_nvbroadcast_times"] += 1;
      counters_["blitz_scale_up_times"] += 1;
      if (!multi) sources.resize(1);
      for (int s : sources) {
        steer_.set_nvlink_busy(s, true);
        reps_[s].m.marker = multi ? RState::TanzCasting : (nvl ? RState::NvlCasting : RState::RdmaCasting);
        for (int rk : steer_.ranks_of_replica(s)) a.src_ranks.push_back(rk);
      }
      op.sources = sources;
      const bool live = prefill && features_.has("live");
      a.live = live;
      if (live) {
        set_state(r, RState::NewPrefill);
        rep.zag_started = now;
        rep.zag_seq = 0;
        // pair one normal prefill replica as the helper that finishes relayed batches
        for (int o = 0; o < num_replicas(); ++o) {
          if (reps_[o].m.state == RState::Prefill && reps_[o].partner < 0 && !reps_[o].colocated) {
            set_state(o, RState::OldPrefill);
            reps_[o].partner = r;
            rep.partner = o;
            break;
          }
        }
      } else {
        set_state(r, prefill ? RState::LoadingPrefill : RState::LoadingDecode);
      }
    }
    op.kind = a.type;
    op.started = now;
    ops_[++next_op_] = op;
    a.op_id = next_op_;
    out_.push_back(a);
    return true;
  }

  void scale_down(bool prefill, double now) {
    // one per planner turn, never the last one, never a replica in a live pairing
    const RState want = prefill ? RState::Prefill : RState::Decode;
    if (num_in_state(want) <= 1) return;
    int pick = -1;
    uint32_t least = UINT32_MAX;
    for (int r = num_replicas() - 1; r >= 0; --r) {
      if (reps_[r].m.state != want || reps_[r].partner >= 0 || reps_[r].colocated) continue;
      if (reps_[r].m.used_blocks < least) { least = reps_[r].m.used_blocks; pick = r; }
    }
    if (pick >= 0) begin_shutdown(pick, now);
  }
  void begin_shutdown(int r, double now) {
    if (reps_[r].m.state == RState::Prefill) set_state(r, RState::ShuttingPrefill);
    else if (reps_[r].m.state == RState::Decode) set_state(r, RState::ShuttingDecode);
    else if (reps_[r].m.state == RState::ShuttingNull) { reps_[r].m.shutting_since = now - 1e9; }
  }
  void park(int r, double now) {
    set_state(r, RState::ShuttingNull);
    reps_[r].m.shutting_since = now;
  }
  void expire_parked(double now) {
    for (int r = 0; r < num_replicas(); ++r) {
      Rep& rep = reps_[r];
      if (rep.m.state != RState::ShuttingNull || rep.m.shutting_since < 0) continue;
      if ((now - rep.m.shutting_since) * 1e3 < cfg_.planner.scale_down_threshold_ms) continue;
      if (steer_.nvlink_busy(r)) continue;  // still feeding someone
      set_state(r, RState::Inactive);
      rep.m.model_loaded = false;
      rep.m.shutting_since = -1;
      steer_.record_model_unloaded(r, now);
      log_.push_back("Replica<" + std::to_string(r) + "> >>= unload");
      Action a = make_simple(ActionType::ResetStatus, r, 0);
      a.dst_ranks = steer_.ranks_of_replica(r);
      out_.push_back(a);
    }
  }

  // Replica `r` is gone.  Everything that involved it is settled here, at once: operations in flight on it or
  // towards it are cancelled (their answers, if they still come, are ignored), prompts it had not answered go back
  // to the head of the queue, requests whose KV lived on it or was on its way to or from it fail, and the surviving
  // side of every such operation gets its pages and locks back.  `quarantine` = false resets a healthy replica whose
  // parameter transfer was aborted because another participant was lost.
  void lose_replica(int r, double now, bool quarantine = true) {
    Rep& rep = reps_[r];
    if (quarantine) rep.lost_at = now;
    auto fail_ids = [&](const std::vector<uint64_t>& ids) {
      for (uint64_t id : ids) {
        if (!requests_.count(id)) continue;
        Action a;
        a.type = ActionType::Fail; a.request_id = id; a.final = true;
        out_.push_back(a);
        requests_.erase(id);
      }
    };
    std::vector<uint64_t> requeued;  // a live-prefill batch is known both by its operation and by its replica
    auto requeue_ids = [&](const std::vector<uint64_t>& ids) {
      std::vector<RequestEntry> es;
      for (uint64_t id : ids) {
        if (!requests_.count(id) || std::find(requeued.begin(), requeued.end(), id) != requeued.end()) continue;
        if (!requests_[id].client_alive) {   // nobody waits for it any more: end it here instead of queueing it again
          fail_ids({id});
          continue;
        }
        requests_[id].t_batched = -1;   // waiting again: a client that leaves now is forgotten at once
        es.push_back(requests_[id]);
        requeued.push_back(id);
      }
      if (!es.empty()) queue_.requeue_front(es);
    };
    auto cancel = [&](uint64_t id, uint64_t batch_id, std::vector<int> survivors) {
      Cancelled c;
      c.batch_id = batch_id;
      for (int s : survivors)
        if (s >= 0 && s != r) c.clear_on.push_back(s);
      cancelled_[id] = c;
    };
    auto involves = [&](const Op& o) {
      return o.replica == r || o.peer == r || std::find(o.sources.begin(), o.sources.end(), r) != o.sources.end() ||
             std::find(o.targets.begin(), o.targets.end(), r) != o.targets.end();
    };

    // relayed batches with the lost replica as first half, second half or destination
    for (auto it = relayed_.begin(); it != relayed_.end();) {
      Relayed& x = it->second;
      if (x.new_replica != r && x.old_replica != r && x.target != r) { ++it; continue; }
      fail_ids(x.batch.request_ids);
      for (auto oi = ops_.begin(); oi != ops_.end();) {
        Op& o = oi->second;
        const bool mine = (o.kind == ActionType::PrefillPP || o.kind == ActionType::MigratePartial) && o.batch.id == x.batch.id;
        if (!mine) { ++oi; continue; }
        if (o.kind == ActionType::PrefillPP) reps_[o.replica].busy = reps_[o.replica].relay_wait = false;
        cancel(oi->first, x.batch.id, {o.replica, o.peer});
        oi = ops_.erase(oi);
      }
      const bool new_holds = !((x.fst_started && x.fst_done) || (x.next_layer == 0 && x.fst_done && x.snd_started));
      if (x.fst_started && !x.fst_done && reps_[x.new_replica].m.flying_partial > 0) reps_[x.new_replica].m.flying_partial -= 1;
      if (new_holds && x.new_replica != r) {
        release_blocks(x.new_replica, x.blocks);
        out_.push_back(make_simple(ActionType::ClearCache, x.new_replica, x.batch.id));
      }
      if (!x.snd_done && x.old_replica != r) {
        release_blocks(x.old_replica, x.blocks);
        out_.push_back(make_simple(ActionType::ClearCache, x.old_replica, x.batch.id));
      }
      if (x.target == r) incoming_seqs_of_.erase(x.batch.id);
      if (x.target >= 0 && x.target != r) {
        finish_relayed_target(x);
        out_.push_back(make_simple(ActionType::ClearCache, x.target, x.batch.id));
      }
      it = relayed_.erase(it);
    }

    // every other operation in flight that involves the lost replica
    std::vector<uint64_t> ids;
    for (auto& kv : ops_)
      if (involves(kv.second)) ids.push_back(kv.first);
    std::vector<int> aborted_loads;
    for (uint64_t id : ids) {
      auto it = ops_.find(id);
      if (it == ops_.end()) continue;
      Op o = std::move(it->second);
      ops_.erase(it);
      const int other = o.replica == r ? o.peer : o.replica;
      switch (o.kind) {
        case ActionType::Prefill:
        case ActionType::ZagPrefill:
          requeue_ids(o.batch.request_ids);  // nothing was delivered yet
          if (o.kind == ActionType::Prefill && o.peer >= 0) {
            // a progressive migration: the surviving side gives back what it holds for the batch
            release_blocks(other, o.batch.blocks);
            if (o.replica == r) unlock_target(other, o.batch.id);
            else reps_[other].busy = false;
            incoming_seqs_of_.erase(o.batch.id);
            out_.push_back(make_simple(ActionType::ClearCache, other, o.batch.id));
            cancel(id, o.batch.id, {other});
            break;
          }
          cancel(id, o.batch.id, {});
          break;
        case ActionType::Decode:
        case ActionType::FilterBatch:
          // its batches are resident on the lost replica: failed below (a batch that waits for its filter before it
          // joins the replica's steps is known by the operation only)
          if (o.partial == kAdoptAfterFilter) {
            fail_ids(o.batch.request_ids);
            incoming_seqs_of_.erase(o.batch.id);
          }
          cancel(id, o.batch.id, {});
          break;
        case ActionType::Migrate:
          fail_ids(o.batch.request_ids);
          release_blocks(other, o.batch.blocks);
          if (o.replica == r) unlock_target(other, o.batch.id);
          else reps_[other].migrating = false;
          incoming_seqs_of_.erase(o.batch.id);
          out_.push_back(make_simple(ActionType::ClearCache, other, o.batch.id));
          cancel(id, o.batch.id, {other});
          break;
        case ActionType::Relay:
          if (o.peer != r) reps_[o.peer].busy = reps_[o.peer].relay_wait = false;
          cancel(id, 0, {});
          break;
        case ActionType::PrefillPP:
        case ActionType::MigratePartial:  // a relayed batch that is no longer tracked: nothing left to settle
          if (o.kind == ActionType::PrefillPP && o.replica != r) reps_[o.replica].busy = reps_[o.replica].relay_wait = false;
          cancel(id, o.batch.id, {o.replica, o.peer});
          break;
        default:  // a parameter transfer: without one of its participants nobody's copy completes
          for (int s : o.sources) {
            steer_.set_nvlink_busy(s, false);
            reps_[s].m.marker.reset();
          }
          for (int d : o.targets)
            if (d != r) aborted_loads.push_back(d);
          cancel(id, 0, {});
          break;
      }
    }

    for (auto& b : rep.pending_migration) fail_ids(b.request_ids);
    for (auto& b : rep.decode_batches) fail_ids(b.request_ids);
    for (auto& b : rep.inflight_zag) requeue_ids(b.request_ids);
    rep.pending_migration.clear();
    rep.decode_batches.clear();
    rep.inflight_zag.clear();
    rep.busy = rep.migrating = rep.relay_wait = false;
    rep.incoming = 0;
    rep.incoming_batches.clear();
    rep.incoming_seqs = 0;
    rep.m.used_blocks = 0;
    rep.m.flying_partial = 0;
    rep.m.model_loaded = false;
    rep.m.shutting_since = -1;
    rep.m.marker.reset();
    if (rep.partner >= 0) {
      Rep& other = reps_[rep.partner];
      if (other.partner == r) {
        other.partner = -1;
        other.relay_wait = false;
        if (other.m.state == RState::OldPrefill) {
          other.busy = false;
          for (auto& kv : ops_) other.busy = other.busy || (kv.second.replica == rep.partner &&
                                                              (kv.second.kind == ActionType::Prefill || kv.second.kind == ActionType::Decode));
          set_state(rep.partner, RState::Prefill);
        }
      }
      rep.partner = -1;
    }
    steer_.record_model_unloaded(r, now);
    steer_.set_nvlink_busy(r, false);
    if (rep.m.state != RState::Inactive) {
      RState old = rep.m.state;
      rep.m.state = RState::Inactive;
      rep.m.dst_busy = true;
      log_transition(r, old, RState::Inactive);
    }
    if (quarantine && cfg_.tp > 1) {
      // the replica is lost as a whole, but some of its shards may still run: they drop what they hold, so that
      // nothing stale is left if the replica is brought back (calls to the shard that is gone simply fail)
      Action c = make_simple(ActionType::ClearCache, r, 0);
      c.final = true;   // every batch
      out_.push_back(c);
      Action z = make_simple(ActionType::ResetStatus, r, 0);
      z.dst_ranks = steer_.ranks_of_replica(r);
      out_.push_back(z);
    }
    for (int d : aborted_loads) {
      lose_replica(d, now, false);
      Action a = make_simple(ActionType::ResetStatus, d, 0);
      a.dst_ranks = steer_.ranks_of_replica(d);
      out_.push_back(a);
    }
  }

  // Answer (or failure) of an operation that was cancelled when a replica was lost: what the surviving workers
  // built for it in the meantime is dropped.
  bool late_answer(uint64_t op_id) {
    auto it = cancelled_.find(op_id);
    if (it == cancelled_.end()) return false;
    for (int s : it->second.clear_on)
      if (reps_[s].m.state != RState::Inactive) out_.push_back(make_simple(ActionType::ClearCache, s, it->second.batch_id));
    cancelled_.erase(it);
    return true;
  }

  ControllerConfig cfg_;
  FeatureSet features_;
  bool arrival_signal_ = false;                            // feature planner_arrival_rate with a configured rate
  std::deque<std::pair<double, uint32_t>> arrivals_;       // (arrival time, prompt tokens) inside the rate window
  BatchQueue queue_;
  Steersman steer_;
  std::vector<Rep> reps_;
  std::map<uint64_t, RequestEntry> requests_, finished_;
  std::map<uint64_t, Op> ops_;
  std::map<uint64_t, Relayed> relayed_;
  std::map<uint64_t, Cancelled> cancelled_;
  std::map<uint64_t, uint32_t> incoming_seqs_of_;   // batch on its way to a decode replica -> its sequences
  std::vector<Action> out_;
  std::vector<Delivery> deliveries_;
  bool compact_deliveries_ = false;
  std::vector<std::string> log_;
  std::map<std::string, double> counters_, gauges_;
  uint64_t next_op_ = 0;
  double down_since_p_ = -1, down_since_d_ = -1;      // since when the planner has been asking for fewer replicas
  std::vector<std::pair<int, bool>> pending_scale_;  // (replica, as prefill) requested since the last step
  uint64_t stats_prefill_tokens_ = 0, stats_decode_tokens_ = 0;
  double last_plan_ = -1e9;
  ScaleTarget last_target_;
  std::pair<int, int> last_logged_{0, 0};

 public:
  const std::map<uint64_t, RequestEntry>& finished() const { return finished_; }
  // Take the record of a finished request out of the core (a long-running shell must, or the map grows for ever).
  std::optional<RequestEntry> pop_finished(uint64_t id) {
    auto it = finished_.find(id);
    if (it == finished_.end()) return std::nullopt;
    RequestEntry e = std::move(it->second);
    finished_.erase(it);
    return e;
  }
  // Gauges of the planner's last turn plus the queue and replica gauges of the reference's metric list
  // (router_v2/src/server.rs:1084-1134, declared there and mostly never updated), taken from the state as it is now.
  const std::map<std::string, double>& gauges() {
    uint64_t waiting_full = 0, waiting_partial = 0, shutting = 0, n_prefill = 0, n_decode = 0;
    for (auto& r : reps_) {
      waiting_full += r.pending_migration.size();
      const RState st = r.m.state;
      n_prefill += is_prefill_side(st) ? 1 : 0;
      n_decode += is_decode_side(st) ? 1 : 0;
      if (st == RState::ShuttingPrefill || st == RState::ShuttingDecode || st == RState::ShuttingNull) ++shutting;
    }
    for (auto& kv : relayed_) waiting_partial += (kv.second.fst_done ? 0 : 1) + (kv.second.snd_done ? 0 : 1);
    gauges_["blitz_migration_queue_size"] = static_cast<double>(waiting_full);
    gauges_["blitz_waiting_full_batches"] = static_cast<double>(waiting_full);
    gauges_["blitz_relay_queue_size"] = static_cast<double>(relayed_.size());
    gauges_["blitz_waiting_partial_batches"] = static_cast<double>(waiting_partial);
    gauges_["blitz_used_blocks"] = static_cast<double>(total_used_blocks());
    gauges_["blitz_shutting_replica"] = static_cast<double>(shutting);
    gauges_["blitz_prefill_replica"] = static_cast<double>(n_prefill);
    gauges_["blitz_decode_replica"] = static_cast<double>(n_decode);
    gauges_["blitz_queue_size"] = static_cast<double>(queue_.size());
    return gauges_;
  }
  Steersman& steersman() { return steer_; }
};

}  // namespace blitz
