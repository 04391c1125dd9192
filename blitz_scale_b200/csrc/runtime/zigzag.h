// Live-execution ("ZigZag") layer scheduler: decides which in-flight prefill batch runs which
// piece (embedding, attention block, FFN block, LM head) next while parameters are still arriving.
//
// Sans-IO: the engine asks `next()`, runs the kernels, reports `complete()`.  Behaviour follows
// src/blitz/zigzag_manager.h:439-637: tasks execute strictly in arrival (sequence-number) order
// of admission, one block at a time; the head task is preferred whenever the layer it needs has
// arrived (preemption), otherwise the first other task that can advance runs (yield), otherwise
// the scheduler reports Blocked.  A relay request (src/blitz/zigzag_manager.h:123-234) removes the
// head task (or the second one in refractory mode) and reports the layer the old instance must
// resume from; a task interrupted between its attention and FFN blocks resumes from the start of
// that layer (:409-430), which is safe because the residual is only updated by whole blocks here
// (the engine snapshots nothing: attention writes the residual only through the o_proj epilogue,
// so the engine defers that GEMM's residual add until the FFN is certain to run; see engine).
//
// Layer availability is a single monotonic counter written by the parameter receiver, so every
// tensor-parallel shard of a replica sees the same value by construction; the reference needs an
// MPI barrier + allgather per layer for the same agreement (src/include/step_locker.hpp:19-97).
#pragma once
#include <pybind11/pybind11.h>
#include <cstdint>
#include <deque>
#include <optional>
#include <stdexcept>

namespace blitz {

enum class ZagStep : int { Idle = 0, Blocked = 1, Embed = 2, Layer = 3, Head = 4 };

struct ZagTask {
  uint64_t batch_id = 0;
  uint32_t seq_num = 0;
  int num_tokens = 0;
  int slot = -1;        // activation slot holding the residual stream
  bool embedded = false;
  int next_layer = 0;   // first layer not yet executed
};

struct ZagDecision {
  ZagStep step = ZagStep::Idle;
  uint64_t batch_id = 0;
  int layer = -1;
  int slot = -1;
};

struct ZagRelay {
  uint64_t batch_id = 0;
  uint32_t seq_num = 0;
  int next_layer = 0;  // old instance continues from this transformer layer
  int slot = -1;
  int num_tokens = 0;
};

class ZigzagScheduler {
 public:
  explicit ZigzagScheduler(int total_layers, int num_slots = 16) : total_layers_(total_layers) {
    for (int i = num_slots - 1; i >= 0; --i) free_slots_.push_back(i);
  }

  void set_loaded(bool embed_ready, int layers_ready, bool head_ready) {
    if (layers_ready < layers_ready_) throw std::logic_error("layer counter went backwards");
    embed_ready_ = embed_ready;
    layers_ready_ = layers_ready;
    head_ready_ = head_ready;
  }
  void reset() {
    embed_ready_ = head_ready_ = false;
    layers_ready_ = 0;
  }
  int pending() const { return static_cast<int>(tasks_.size()); }
  int free_slots() const { return static_cast<int>(free_slots_.size()); }

  // Tasks must be added in sequence-number order (the service serialises ZagPrefill RPCs by
  // sequence number, src/service/service.cc:798-818).  Returns the activation slot, -1 if none is free.
  int add_task(uint64_t batch_id, uint32_t seq_num, int num_tokens) {
    if (!tasks_.empty() && seq_num <= tasks_.back().seq_num) throw std::invalid_argument("zag tasks out of order");
    if (free_slots_.empty()) return -1;
    ZagTask t;
    t.batch_id = batch_id; t.seq_num = seq_num; t.num_tokens = num_tokens;
    t.slot = free_slots_.back();
    free_slots_.pop_back();
    tasks_.push_back(t);
    return t.slot;
  }

  ZagDecision next() const {
    if (tasks_.empty()) return {};
    for (const ZagTask& t : tasks_) {  // head first: preemption; then the others: yield
      ZagDecision d;
      d.batch_id = t.batch_id; d.slot = t.slot;
      if (!t.embedded) {
        if (embed_ready_) { d.step = ZagStep::Embed; return d; }
        continue;
      }
      if (t.next_layer < total_layers_) {
        if (t.next_layer < layers_ready_) { d.step = ZagStep::Layer; d.layer = t.next_layer; return d; }
        continue;
      }
      if (head_ready_) { d.step = ZagStep::Head; return d; }
    }
    ZagDecision b;
    b.step = ZagStep::Blocked;
    return b;
  }

  // Report that the step returned by next() finished.  Returns true when the task is done (Head ran).
  bool complete(const ZagDecision& d) {
    for (auto it = tasks_.begin(); it != tasks_.end(); ++it) {
      if (it->batch_id != d.batch_id) continue;
      switch (d.step) {
        case ZagStep::Embed: it->embedded = true; return false;
        case ZagStep::Layer:
          if (d.layer != it->next_layer) throw std::logic_error("layer completed out of order");
          it->next_layer += 1;
          return false;
        case ZagStep::Head:
          free_slots_.push_back(it->slot);
          tasks_.erase(it);
          return true;
        default: throw std::logic_error("complete(): not a runnable step");
      }
    }
    throw std::logic_error("complete(): unknown task");
  }

  // Hand the head task (second task when `relax_not_head`, used while the instance drains) to the old
  // instance.  The task leaves the queue; its slot is released by `release_slot` once the activations
  // have been shipped.
  std::optional<ZagRelay> relay(bool relax_not_head) {
    size_t idx = relax_not_head ? 1 : 0;
    if (tasks_.size() <= idx) return std::nullopt;
    // a task that has not been embedded yet restarts from the embedding on the old instance
    ZagTask t = tasks_[idx];
    tasks_.erase(tasks_.begin() + idx);
    ZagRelay r;
    r.batch_id = t.batch_id; r.seq_num = t.seq_num; r.slot = t.slot; r.num_tokens = t.num_tokens;
    r.next_layer = t.embedded ? t.next_layer : -1;
    return r;
  }
  // The same hand-over for a task named by its sequence number: what the other tensor-parallel shards of a replica
  // do once the leading shard has chosen (their queues may momentarily hold a different set of tasks, so "head" or
  // "second" would not name the same task everywhere).
  std::optional<ZagRelay> relay_task(uint32_t seq_num) {
    for (auto it = tasks_.begin(); it != tasks_.end(); ++it) {
      if (it->seq_num != seq_num) continue;
      ZagRelay r;
      r.batch_id = it->batch_id; r.seq_num = it->seq_num; r.slot = it->slot; r.num_tokens = it->num_tokens;
      r.next_layer = it->embedded ? it->next_layer : -1;
      tasks_.erase(it);
      return r;
    }
    return std::nullopt;
  }
  void release_slot(int slot) { free_slots_.push_back(slot); }
  // batch id of the queued task with this sequence number (nullopt while its request has not arrived here)
  std::optional<uint64_t> batch_of(uint32_t seq_num) const {
    for (const ZagTask& t : tasks_)
      if (t.seq_num == seq_num) return t.batch_id;
    return std::nullopt;
  }
  std::optional<uint32_t> seq_of(uint64_t batch_id) const {
    for (const ZagTask& t : tasks_)
      if (t.batch_id == batch_id) return t.seq_num;
    return std::nullopt;
  }

  bool embed_ready() const { return embed_ready_; }
  int layers_ready() const { return layers_ready_; }
  bool head_ready() const { return head_ready_; }

 private:
  int total_layers_;
  bool embed_ready_ = false, head_ready_ = false;
  int layers_ready_ = 0;
  std::deque<ZagTask> tasks_;
  std::deque<int> free_slots_;
};

inline void bind_zigzag(pybind11::module_& m) {
  namespace py = pybind11;
  py::enum_<ZagStep>(m, "ZagStep").value("Idle", ZagStep::Idle).value("Blocked", ZagStep::Blocked)
      .value("Embed", ZagStep::Embed).value("Layer", ZagStep::Layer).value("Head", ZagStep::Head);
  py::class_<ZagDecision>(m, "ZagDecision").def(py::init<>()).def_readwrite("step", &ZagDecision::step)
      .def_readwrite("batch_id", &ZagDecision::batch_id).def_readwrite("layer", &ZagDecision::layer)
      .def_readwrite("slot", &ZagDecision::slot);
  py::class_<ZagRelay>(m, "ZagRelay").def_readonly("batch_id", &ZagRelay::batch_id)
      .def_readonly("seq_num", &ZagRelay::seq_num).def_readonly("next_layer", &ZagRelay::next_layer)
      .def_readonly("slot", &ZagRelay::slot).def_readonly("num_tokens", &ZagRelay::num_tokens);
  py::class_<ZigzagScheduler>(m, "ZigzagScheduler").def(py::init<int, int>(), py::arg("total_layers"), py::arg("num_slots") = 16)
      .def("set_loaded", &ZigzagScheduler::set_loaded).def("reset", &ZigzagScheduler::reset)
      .def("pending", &ZigzagScheduler::pending).def("free_slots", &ZigzagScheduler::free_slots)
      .def("add_task", &ZigzagScheduler::add_task).def("next", &ZigzagScheduler::next)
      .def("complete", &ZigzagScheduler::complete).def("relay", &ZigzagScheduler::relay)
      .def("relay_task", &ZigzagScheduler::relay_task).def("batch_of", &ZigzagScheduler::batch_of)
      .def("seq_of", &ZigzagScheduler::seq_of)
      .def("release_slot", &ZigzagScheduler::release_slot)
      .def_property_readonly("layers_ready", &ZigzagScheduler::layers_ready);
}

}  // namespace blitz
using blitz::bind_zigzag;
