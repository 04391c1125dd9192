// Model shape registry and weight-segment layout (native twin of models/config.py; a test
// checks that both agree byte for byte).  Shapes follow the table the reference keeps in
// src/model/common_hyper.h:11-177; the parallelism descriptor follows
// src/model/hyper.h:156-232 (tensor-parallel degree and rank, layer range).
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace blitz {

struct ModelShape {
  std::string name;
  int vocab = 0, hidden = 0, layers = 0, q_heads = 0, kv_heads = 0, head_dim = 0, inter = 0;
  double rope_theta = 10000.0;
  double rms_eps = 1e-5;
  int max_positions = 16384;
  double param_gb = 0.0;
  // architecture flags (every served model is a pre-norm, RoPE, gated-FFN, bias-free decoder)
  bool pre_norm = true, rope = true, gated_ffn = true, rms_norm = true, qkv_bias = false;
  int64_t kv_bytes_per_token(int tp, int elem_bytes) const {
    return 2ll * (kv_heads / tp) * head_dim * elem_bytes * layers;
  }
};

struct ParallelSpec {
  int tp_size = 1, tp_rank = 0;
  int layer_begin = 0, layer_end = 0;  // [begin, end): all layers unless a live pipeline splits them
};

inline ModelShape mk(const char* n, int vocab, int hidden, int layers, int qh, int kvh, int inter, double theta = 1e4,
                     int hd = 0, double gb = 0, double eps = 1e-5) {
  ModelShape s;
  s.name = n; s.vocab = vocab; s.hidden = hidden; s.layers = layers; s.q_heads = qh; s.kv_heads = kvh;
  s.head_dim = hd ? hd : hidden / qh; s.inter = inter; s.rope_theta = theta; s.param_gb = gb; s.rms_eps = eps;
  return s;
}

inline const std::map<std::string, ModelShape>& model_registry() {
  static const std::map<std::string, ModelShape> reg = [] {
    std::map<std::string, ModelShape> r;
    for (const ModelShape& s : {
             mk("tiny", 32000, 256, 2, 4, 2, 688),
             mk("tiny_gpu", 4096, 512, 2, 4, 2, 1408, 5e5),
             mk("tiny_gpu_deep", 4096, 512, 8, 4, 2, 1408, 5e5),
             mk("tiny_gpu_wide", 4096, 1024, 2, 8, 4, 2816, 5e5),
             mk("opt_125m", 50272, 768, 12, 12, 12, 3072),
             mk("opt_1.3b", 50272, 2048, 24, 32, 32, 8192),
             mk("opt_6.7b", 50272, 4096, 32, 32, 32, 16384),
             mk("opt_13b", 50272, 5120, 40, 40, 40, 20480),
             mk("opt_30b", 50272, 7168, 48, 56, 56, 28672),
             mk("llama2_7b", 32000, 4096, 32, 32, 32, 11008, 1e4, 0, 14),
             mk("llama2_13b", 32000, 5120, 40, 40, 40, 13824, 1e4, 0, 26),
             mk("llama2_70b", 32000, 8192, 80, 64, 8, 28672, 1e4, 0, 140),
             mk("llama3_8b", 128256, 4096, 32, 32, 8, 14336, 5e5, 0, 16),
             mk("mistral_13b", 32000, 5120, 40, 40, 8, 14336, 1e6, 0, 26),
             mk("mistral_24b", 131072, 5120, 40, 32, 8, 32768, 1e8, 128, 48),
             mk("qwen_72b", 152064, 8192, 80, 64, 8, 29568, 1e6, 0, 145, 1e-6),
         })
      r[s.name] = s;
    return r;
  }();
  return reg;
}

inline const ModelShape& get_model(const std::string& name) {
  auto it = model_registry().find(name);
  if (it == model_registry().end()) throw std::invalid_argument("unknown model: " + name);
  return it->second;
}

struct TensorSlot {
  std::string name;
  std::vector<int64_t> shape;
  int64_t offset = 0, nbytes = 0;
};
struct UnitSlot {
  std::string name;
  int64_t offset = 0, nbytes = 0;
};
struct SegmentLayout {
  std::vector<TensorSlot> tensors;
  std::vector<UnitSlot> units;  // embed | layer.0 .. layer.L-1 | head : the transfer granularity
  int64_t total_bytes = 0;
};

constexpr int64_t kSegAlign = 256;

inline SegmentLayout build_segment_layout(const ModelShape& m, int tp, int elem_bytes) {
  if (m.q_heads % tp || m.kv_heads % tp || m.inter % tp || m.vocab % tp)
    throw std::invalid_argument(m.name + ": heads/inter/vocab not divisible by tp");
  SegmentLayout L;
  int64_t cur = 0;
  auto add = [&](const std::string& name, std::vector<int64_t> shape) {
    int64_t n = 1;
    for (auto s : shape) n *= s;
    TensorSlot t{name, shape, cur, n * elem_bytes};
    L.tensors.push_back(t);
    cur = (cur + t.nbytes + kSegAlign - 1) / kSegAlign * kSegAlign;
  };
  const int64_t qh = m.q_heads / tp, kvh = m.kv_heads / tp, hd = m.head_dim, it = m.inter / tp, H = m.hidden;
  int64_t start = cur;
  add("embed", {m.vocab / tp, H});
  L.units.push_back({"embed", start, cur - start});
  for (int l = 0; l < m.layers; ++l) {
    start = cur;
    const std::string p = "layers." + std::to_string(l) + ".";
    add(p + "input_ln", {H});
    add(p + "qkv", {H, (qh + 2 * kvh) * hd});
    add(p + "o", {qh * hd, H});
    add(p + "post_ln", {H});
    add(p + "gate_up", {H, 2 * it});
    add(p + "down", {it, H});
    L.units.push_back({"layer." + std::to_string(l), start, cur - start});
  }
  start = cur;
  add("final_norm", {H});
  add("lm_head", {H, m.vocab / tp});
  L.units.push_back({"head", start, cur - start});
  L.total_bytes = cur;
  return L;
}

// Loaded-parameter markers of one worker: what the live scheduler and the forward path consult
// before touching a unit (src/blitz/stub.h:118-119, :356-384, invariant :1194-1210).
struct ModelStatus {
  bool embed_ready = false;
  int layers_ready = 0;
  bool head_ready = false;
  int total_layers = 0;
  bool fully_loaded() const { return embed_ready && head_ready && layers_ready == total_layers; }
  bool empty() const { return !embed_ready && !head_ready && layers_ready == 0; }
  void set_ready() { embed_ready = head_ready = true; layers_ready = total_layers; }
  void reset() { embed_ready = head_ready = false; layers_ready = 0; }
  // unit index: 0 = embed, 1..L = layers, L + 1 = head; units arrive in order
  void unit_arrived(int unit) {
    if (unit == 0) embed_ready = true;
    else if (unit == total_layers + 1) head_ready = true;
    else if (unit == layers_ready + 1) layers_ready = unit;
    else throw std::logic_error("unit arrived out of order");
  }
};

}  // namespace blitz
