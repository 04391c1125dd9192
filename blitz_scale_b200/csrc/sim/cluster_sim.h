// Virtual-time cluster simulator: the real Controller driven by simulated workers whose service times
// come from a small cost model.  Used to test scaling policies and request conservation without GPUs
// (the reference has no such harness: its only system test is the batch runner on real machines,
// scripts/batch/main.py:62-188) and to replay the benchmark traces deterministically.
#pragma once
#include <cmath>
#include <map>
#include <queue>
#include <string>
#include <vector>

#include "../router/controller.h"
#include "trace.h"

namespace blitz {

struct CostModel {
  double prefill_tokens_per_s = 60000;   // per replica
  double prefill_overhead_s = 0.004;
  double decode_step_base_s = 0.006;     // weights streaming floor per step
  double decode_step_per_seq_s = 0.00002;
  double kv_tokens_per_s = 3.0e6;        // KV migration rate
  double migrate_overhead_s = 0.0005;
  double param_gb = 16.0;
  double nvlink_gbs = 600.0;             // per-destination ingress on the multicast path
  double host_gbs = 50.0, disk_gbs = 4.0;
  double rpc_overhead_s = 0.0003;
  int layers = 32;
};

struct SimRequestResult {
  uint64_t id;
  double t_arrival, ttft, max_tbt, avg_tbt, t_done;
  uint32_t input_len, output_len;
};

struct SimReport {
  std::vector<SimRequestResult> requests;
  std::vector<std::string> log;
  uint64_t submitted = 0, completed = 0, failed = 0, delivered_tokens = 0;
  uint64_t gone_in_queue = 0, gone_in_service = 0;  // clients that left before / after their request was batched
  double end_time = 0;
  uint64_t leftover_blocks = 0;
  std::vector<std::pair<double, int>> prefill_replicas, decode_replicas;  // (time, count) samples
  std::map<int, double> scale_up_latency;  // replica -> seconds from trigger to serving state
};

struct SimEv {
  double t = 0; uint64_t seq = 0; uint64_t op_id = 0; ActionType type = ActionType::Deliver; int replica = -1;
  std::vector<uint64_t> request_ids;
  bool has_batch = false; uint64_t batch_id = 0; int next_layer = 0;
  uint64_t batch_key = 0;  // batch the action was about
  bool operator<(const SimEv& o) const { return t > o.t || (t == o.t && seq > o.seq); }
};

class ClusterSim {
 public:
  ClusterSim(const ControllerConfig& cc, const CostModel& cm) : ctl_(cc), cm_(cm), cc_(cc) {}

  // `gone_every` = n > 0: the client of every n-th request leaves a little after it arrived (in the queue, during
  // prefill or in the middle of decoding, depending on the load).
  SimReport run(const std::vector<TraceItem>& trace, double tick_s = 0.001, double drain_s = 120.0,
                int kill_replica = -1, double kill_at = -1, int gone_every = 0) {
    SimReport rep;
    size_t next = 0;
    double now = 0;
    std::multimap<double, uint64_t> leaving;
    const double t_last = trace.empty() ? 0 : trace.back().t;
    std::map<int, double> load_started;
    while (true) {
      // arrivals up to `now`
      while (next < trace.size() && trace[next].t <= now) {
        RequestEntry e;
        e.id = next;
        e.input_len = static_cast<uint32_t>(trace[next].input_len);
        e.max_new_tokens = static_cast<uint32_t>(trace[next].output_len);
        e.t_arrival = trace[next].t;
        ctl_.submit(e);
        rep.submitted += 1;
        if (gone_every > 0 && next % static_cast<size_t>(gone_every) == 0)
          leaving.emplace(trace[next].t + 0.02 + 0.045 * static_cast<double>(next % 11), next);
        ++next;
      }
      while (!leaving.empty() && leaving.begin()->first <= now) {
        const uint64_t id = leaving.begin()->second;
        leaving.erase(leaving.begin());
        if (ctl_.client_gone(id)) rep.gone_in_queue += 1;
        else if (ctl_.request(id)) rep.gone_in_service += 1;
      }
      // completions due
      while (!events_.empty() && events_.top().t <= now) {
        SimEv ev = events_.top();
        events_.pop();
        if (kill_replica >= 0 && ev.replica == kill_replica && kill_at >= 0 && ev.t >= kill_at && !killed_) {
          killed_ = true;
          ctl_.on_failure(ev.op_id, ev.t);
          continue;
        }
        if (killed_ && ev.replica == kill_replica) { ctl_.on_failure(ev.op_id, ev.t); continue; }
        complete(ev);
      }
      for (const Action& a : ctl_.step(now)) handle(a, now, rep, load_started);
      for (auto& l : ctl_.drain_log()) {
        rep.log.push_back("[" + std::to_string(now) + "] " + l);
        note_transition(l, now, load_started, rep);
      }
      if (next >= trace.size() && events_.empty() && ctl_.idle() && leaving.empty()) break;
      if (now > t_last + drain_s) break;
      // advance: next tick, or jump to the next arrival / completion when idle
      double tn = now + tick_s;
      if (ctl_.idle() && events_.empty() && next < trace.size()) tn = std::max(tn, trace[next].t);
      now = tn;
    }
    rep.end_time = now;
    rep.leftover_blocks = ctl_.total_used_blocks();
    for (auto& kv : ctl_.finished()) {
      const RequestEntry& e = kv.second;
      SimRequestResult r;
      r.id = e.id; r.t_arrival = e.t_arrival; r.ttft = e.t_first_token - e.t_arrival; r.t_done = e.t_last_token;
      r.input_len = e.input_len; r.output_len = e.generated;
      r.max_tbt = 0; r.avg_tbt = 0;
      for (double d : e.tbt) { r.max_tbt = std::max(r.max_tbt, d); r.avg_tbt += d; }
      if (!e.tbt.empty()) r.avg_tbt /= e.tbt.size();
      rep.requests.push_back(r);
    }
    rep.completed = rep.requests.size();
    return rep;
  }
  Controller& controller() { return ctl_; }

 private:
  void push(double t, const Action& a, SimEv ev = SimEv{}) {
    ev.t = t; ev.seq = ++seq_; ev.op_id = a.op_id; ev.type = a.type; ev.replica = a.replica; ev.batch_key = a.batch_id;
    if (ev.request_ids.empty()) ev.request_ids = a.request_ids;
    events_.push(ev);
  }
  uint32_t tokens_of(const std::vector<uint64_t>& ids) const {
    uint32_t t = 0;
    for (uint64_t id : ids) { const RequestEntry* e = ctl_.request(id); if (e) t += e->input_len; }
    return t;
  }
  int32_t fake_token(uint64_t req, uint32_t k) const { return static_cast<int32_t>((req * 2654435761u + k * 40503u) % 32000u); }

  void handle(const Action& a, double now, SimReport& rep, std::map<int, double>& load_started) {
    switch (a.type) {
      case ActionType::Prefill: {
        double d = cm_.rpc_overhead_s + cm_.prefill_overhead_s + tokens_of(a.request_ids) / cm_.prefill_tokens_per_s;
        // layer-progressive migration: every layer's KV leaves while the next layers run; only the last layer's
        // push comes after the pass
        if (a.peer >= 0) d += tokens_of(a.request_ids) / cm_.kv_tokens_per_s / std::max(1, cm_.layers);
        push(now + d, a);
        break;
      }
      case ActionType::ZagPrefill: {
        // serving while loading: the batch cannot finish before the parameters it needs have arrived
        double d = cm_.rpc_overhead_s + cm_.prefill_overhead_s + tokens_of(a.request_ids) / cm_.prefill_tokens_per_s;
        auto it = load_done_at_.find(a.replica);
        double fin = std::max(now + d, it == load_done_at_.end() ? now : it->second);
        zag_inflight_[a.replica].push_back({a.batch_id, now});
        push(fin, a);
        break;
      }
      case ActionType::PrefillPP: {
        const double frac = 1.0 - static_cast<double>(a.num_layer) / std::max(1, cm_.layers);
        const double d = cm_.rpc_overhead_s + cm_.prefill_overhead_s + frac * tokens_of(a.request_ids) / cm_.prefill_tokens_per_s;
        push(now + d, a);
        break;
      }
      case ActionType::Decode: {
        const double d = cm_.rpc_overhead_s + cm_.decode_step_base_s + cm_.decode_step_per_seq_s * a.request_ids.size();
        push(now + d, a);
        break;
      }
      case ActionType::Migrate:
      case ActionType::MigratePartial: {
        double frac = 1.0;
        if (a.type == ActionType::MigratePartial)
          frac = a.partial == 1 ? static_cast<double>(a.num_layer) / cm_.layers : 1.0 - static_cast<double>(a.num_layer) / cm_.layers;
        push(now + cm_.migrate_overhead_s + frac * tokens_of(a.request_ids) / cm_.kv_tokens_per_s, a);
        break;
      }
      case ActionType::Relay: {
        SimEv ev;
        auto& fl = zag_inflight_[a.replica];
        // drop entries of batches that already completed
        size_t idx = a.final ? 1 : 0;
        if (fl.size() > idx) {
          ev.has_batch = true;
          ev.batch_id = fl[idx].first;
          auto it = load_done_at_.find(a.replica);
          auto st = load_started.find(a.replica);
          double frac = 1.0;
          if (it != load_done_at_.end() && st != load_started.end() && it->second > st->second)
            frac = std::clamp((now - st->second) / (it->second - st->second), 0.0, 1.0);
          ev.next_layer = static_cast<int>(frac * cm_.layers);
          cancelled_zag_.insert(ev.batch_id);
          fl.erase(fl.begin() + idx);
        }
        push(now + cm_.rpc_overhead_s, a, ev);
        break;
      }
      case ActionType::NvlBroadcast:
      case ActionType::TanzBroadcast:
      case ActionType::RdmaBroadcast: {
        double d = cc_.mock_load_ms > 0 || a.mock ? cc_.mock_load_ms * 1e-3 : cm_.param_gb / cm_.nvlink_gbs;
        load_done_at_[a.replica] = now + d;
        load_started[a.replica] = now;
        push(now + d + cm_.rpc_overhead_s, a);
        break;
      }
      case ActionType::LoadParams: {
        double d = a.mock ? cc_.mock_load_ms * 1e-3 : cm_.param_gb / (a.load_case == 0 ? cm_.host_gbs : cm_.disk_gbs);
        load_done_at_[a.replica] = now + d;
        load_started[a.replica] = now;
        push(now + d + cm_.rpc_overhead_s, a);
        break;
      }
      case ActionType::FilterBatch: push(now + cm_.rpc_overhead_s, a); break;
      case ActionType::Deliver: rep.delivered_tokens += 1; break;
      case ActionType::Fail: rep.failed += 1; break;
      default: break;
    }
  }

  void complete(const SimEv& ev) {
    std::vector<Controller::TokenOut> toks;
    switch (ev.type) {
      case ActionType::ZagPrefill:
        if (cancelled_zag_.count(ev.batch_key)) return;
        [[fallthrough]];
      case ActionType::Prefill:
      case ActionType::PrefillPP:
      case ActionType::Decode: {
        if (ev.type == ActionType::ZagPrefill) {
          auto& fl = zag_inflight_[ev.replica];
          for (auto it = fl.begin(); it != fl.end(); ++it)
            if (it->first == ev.batch_key) { fl.erase(it); break; }
        }
        for (uint64_t id : ev.request_ids) {
          const RequestEntry* e = ctl_.request(id);
          if (!e) continue;
          toks.push_back({id, fake_token(id, e->generated), e->generated + 1 >= e->max_new_tokens});
        }
        if (ev.type == ActionType::Decode) ctl_.on_decode_done(ev.op_id, toks, ev.t);
        else ctl_.on_prefill_done(ev.op_id, toks, ev.t);
        break;
      }
      case ActionType::Migrate:
      case ActionType::MigratePartial: ctl_.on_migrate_done(ev.op_id, ev.t); break;
      case ActionType::Relay: ctl_.on_relay_done(ev.op_id, ev.has_batch, ev.batch_id, ev.next_layer, ev.t); break;
      case ActionType::NvlBroadcast:
      case ActionType::TanzBroadcast:
      case ActionType::RdmaBroadcast:
      case ActionType::LoadParams: ctl_.on_params_done(ev.op_id, ev.t); break;
      case ActionType::FilterBatch: ctl_.on_filter_done(ev.op_id, ev.t); break;
      default: break;
    }
  }

  void note_transition(const std::string& l, double now, std::map<int, double>& load_started, SimReport& rep) {
    // "Replica<i> A => B"
    auto p = l.find("Replica<");
    auto arrow = l.find(" => ");
    if (p == std::string::npos || arrow == std::string::npos) return;
    const int r = std::stoi(l.substr(p + 8));
    const std::string to = l.substr(arrow + 4);
    if ((to == "Prefill" || to == "Decode") && load_started.count(r) && !rep.scale_up_latency.count(r))
      rep.scale_up_latency[r] = now - load_started[r];
    int np = 0, nd = 0;
    for (int i = 0; i < ctl_.num_replicas(); ++i) {
      const std::string s = ctl_.state_name(i);
      np += (s == "Prefill" || s == "NewPrefill" || s == "OldPrefill" || s == "RefractoryPrefill");
      nd += (s == "Decode");
    }
    rep.prefill_replicas.push_back({now, np});
    rep.decode_replicas.push_back({now, nd});
  }

  Controller ctl_;
  CostModel cm_;
  ControllerConfig cc_;
  std::priority_queue<SimEv> events_;
  uint64_t seq_ = 0;
  bool killed_ = false;
  std::map<int, double> load_done_at_;
  std::map<int, std::vector<std::pair<uint64_t, double>>> zag_inflight_;
  std::set<uint64_t> cancelled_zag_;
};

}  // namespace blitz
