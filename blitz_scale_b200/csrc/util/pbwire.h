// Minimal protobuf wire-format reader for the one message the router reads at token rate: the `generations` field
// (number 1, repeated `Generation`) of the generate.v2 prefill / decode responses.  Per generation the router needs
// the request id (field 1), the first token id (field 3 `tokens`, sub-field 1 `ids`, unpacked or packed) and whether
// `generated_text` (field 4) is present, which marks the request as finished.  Everything else is skipped by wire
// type.  Malformed input raises; nothing is read past the end of the buffer.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string_view>
#include <vector>

namespace blitz {
namespace pbwire {

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool done() const { return p >= end; }
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (p >= end) throw std::invalid_argument("protobuf: truncated varint");
      const uint8_t b = *p++;
      v |= static_cast<uint64_t>(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
    }
    throw std::invalid_argument("protobuf: varint too long");
  }
  Reader sub() {
    const uint64_t n = varint();
    if (n > static_cast<uint64_t>(end - p)) throw std::invalid_argument("protobuf: length runs past the buffer");
    Reader r{p, p + n};
    p += n;
    return r;
  }
  void skip(uint32_t wire_type) {
    switch (wire_type) {
      case 0: varint(); break;
      case 1: advance(8); break;
      case 2: sub(); break;
      case 5: advance(4); break;
      default: throw std::invalid_argument("protobuf: unsupported wire type");
    }
  }
  void advance(size_t n) {
    if (n > static_cast<size_t>(end - p)) throw std::invalid_argument("protobuf: field runs past the buffer");
    p += n;
  }
};

struct Generations {
  std::vector<uint64_t> request_ids;
  std::vector<int32_t> tokens;   // -1 when a generation carries no token
  std::vector<bool> finished;
  std::vector<int8_t> reasons;   // FinishReason of a finished generation (0 length, 1 EOS token, 2 stop sequence), else -1
};

inline Generations parse_generations(std::string_view response) {
  Generations out;
  Reader top{reinterpret_cast<const uint8_t*>(response.data()), reinterpret_cast<const uint8_t*>(response.data()) + response.size()};
  while (!top.done()) {
    const uint64_t tag = top.varint();
    if (tag != ((1u << 3) | 2u)) { top.skip(static_cast<uint32_t>(tag & 7)); continue; }
    Reader g = top.sub();
    uint64_t rid = 0;
    int32_t tok = -1;
    bool fin = false;
    int8_t reason = -1;
    while (!g.done()) {
      const uint64_t t = g.varint();
      const uint32_t field = static_cast<uint32_t>(t >> 3), wt = static_cast<uint32_t>(t & 7);
      if (field == 1 && wt == 0) {
        rid = g.varint();
      } else if (field == 3 && wt == 2) {
        Reader tk = g.sub();
        while (!tk.done()) {
          const uint64_t tt = tk.varint();
          const uint32_t f2 = static_cast<uint32_t>(tt >> 3), w2 = static_cast<uint32_t>(tt & 7);
          if (f2 == 1 && w2 == 0) {
            const uint64_t v = tk.varint();
            if (tok < 0) tok = static_cast<int32_t>(v);
          } else if (f2 == 1 && w2 == 2) {
            Reader packed = tk.sub();
            while (!packed.done()) {
              const uint64_t v = packed.varint();
              if (tok < 0) tok = static_cast<int32_t>(v);
            }
          } else {
            tk.skip(w2);
          }
        }
      } else if (field == 4 && wt == 2) {
        Reader gt = g.sub();   // GeneratedText: text = 1, generated_tokens = 2, finish_reason = 3
        fin = true;
        reason = 0;
        while (!gt.done()) {
          const uint64_t tt = gt.varint();
          const uint32_t f2 = static_cast<uint32_t>(tt >> 3), w2 = static_cast<uint32_t>(tt & 7);
          if (f2 == 3 && w2 == 0) reason = static_cast<int8_t>(gt.varint());
          else gt.skip(w2);
        }
      } else {
        g.skip(wt);
      }
    }
    out.request_ids.push_back(rid);
    out.tokens.push_back(tok);
    out.finished.push_back(fin);
    out.reasons.push_back(reason);
  }
  return out;
}

}  // namespace pbwire
}  // namespace blitz
