// Seeded synthetic request traces: Poisson and Gamma (chosen coefficient of variation) arrivals with a
// piecewise-constant rate, uniform / lognormal / fixed length distributions, and CSV replay
// (`timestamp_ms,prefill,decode`, the dataset format of the reference's trace client: scripts/batch/runner.py:471-492,
// scripts/figure/process_dataset_v2.py:40-55).  All sampling is implemented here (no <random> distributions), so a
// seed gives the same trace on every platform.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <fstream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace blitz {

class Rng {
 public:
  explicit Rng(uint64_t seed) : s_(seed + 0x9e3779b97f4a7c15ull) {}
  uint64_t next_u64() {
    uint64_t z = (s_ += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
  }
  double uniform() { return static_cast<double>(next_u64() >> 11) * (1.0 / 9007199254740992.0); }  // [0,1)
  double exponential(double rate) { return -std::log(1.0 - uniform()) / rate; }
  double normal() {
    const double u1 = 1.0 - uniform(), u2 = uniform();
    return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
  }
  // Marsaglia-Tsang
  double gamma(double shape, double scale) {
    if (shape < 1.0) return gamma(shape + 1.0, scale) * std::pow(uniform() + 1e-300, 1.0 / shape);
    const double d = shape - 1.0 / 3.0, c = 1.0 / std::sqrt(9.0 * d);
    while (true) {
      double x = normal(), v = 1.0 + c * x;
      if (v <= 0) continue;
      v = v * v * v;
      const double u = uniform();
      if (u < 1.0 - 0.0331 * x * x * x * x || std::log(u + 1e-300) < 0.5 * x * x + d * (1.0 - v + std::log(v))) return d * v * scale;
    }
  }
  int64_t uniform_int(int64_t lo, int64_t hi) { return lo + static_cast<int64_t>(uniform() * static_cast<double>(hi - lo + 1)); }

 private:
  uint64_t s_;
};

struct LengthDist {
  enum Kind { Fixed, Uniform, LogNormal } kind = Fixed;
  double a = 128, b = 128;   // Fixed: a; Uniform: [a, b]; LogNormal: median a, sigma b
  int64_t max_len = 1 << 30, min_len = 1;
  int64_t sample(Rng& r) const {
    double v = a;
    if (kind == Uniform) v = static_cast<double>(r.uniform_int(static_cast<int64_t>(a), static_cast<int64_t>(b)));
    if (kind == LogNormal) v = a * std::exp(b * r.normal());
    return std::clamp<int64_t>(static_cast<int64_t>(std::llround(v)), min_len, max_len);
  }
};

struct RatePhase { double t_start; double rate; };  // requests / s from t_start on

struct TraceItem { double t; int64_t input_len, output_len; uint64_t seed; };

struct TraceSpec {
  std::vector<RatePhase> phases{{0.0, 4.0}};
  double cv = 1.0;            // 1 = Poisson; > 1 burstier (Gamma interarrivals with shape 1/cv^2)
  double duration = 60.0;
  int64_t max_requests = 1 << 30;
  LengthDist input, output;
  uint64_t seed = 0;
};

inline double rate_at(const std::vector<RatePhase>& ph, double t) {
  double r = ph.front().rate;
  for (auto& p : ph) if (t >= p.t_start) r = p.rate;
  return r;
}

inline std::vector<TraceItem> generate_trace(const TraceSpec& spec) {
  Rng rng(spec.seed);
  std::vector<TraceItem> out;
  double t = 0;
  const double shape = 1.0 / (spec.cv * spec.cv);
  while (static_cast<int64_t>(out.size()) < spec.max_requests) {
    const double rate = std::max(1e-9, rate_at(spec.phases, t));
    t += (spec.cv == 1.0) ? rng.exponential(rate) : rng.gamma(shape, 1.0 / (rate * shape));
    if (t >= spec.duration) break;
    TraceItem it;
    it.t = t;
    it.input_len = spec.input.sample(rng);
    it.output_len = spec.output.sample(rng);
    it.seed = rng.next_u64();
    out.push_back(it);
  }
  return out;
}

inline std::vector<TraceItem> load_trace_csv(const std::string& path, double scale_factor = 1.0, int64_t truncate = 4095) {
  std::ifstream f(path);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::vector<TraceItem> out;
  std::string line;
  uint64_t n = 0;
  while (std::getline(f, line)) {
    if (line.empty() || !(std::isdigit(static_cast<unsigned char>(line[0])))) continue;  // header
    std::stringstream ss(line);
    std::string a, b, c;
    if (!std::getline(ss, a, ',') || !std::getline(ss, b, ',') || !std::getline(ss, c, ',')) continue;
    TraceItem it;
    try {
      it.t = std::stod(a) * 1e-3 / scale_factor;
      it.input_len = std::min<int64_t>(std::stoll(b), truncate);
      it.output_len = std::max<int64_t>(1, std::stoll(c));
    } catch (const std::exception&) {
      continue;   // a row whose fields are not numbers of a sane size is skipped like a header
    }
    if (!(it.t >= 0) || !std::isfinite(it.t) || it.input_len < 1) continue;
    it.seed = n++;
    out.push_back(it);
  }
  std::sort(out.begin(), out.end(), [](const TraceItem& x, const TraceItem& y) { return x.t < y.t; });
  return out;
}

}  // namespace blitz
