// Native BPE tokenizer reading the Hugging Face `tokenizer.json` format.
//
// Two families are covered, which is what the served model zoo needs:
//   * byte-level BPE (GPT-2 / Llama-3 / Qwen / Mistral-v3 style): text is cut into words by a scanner that follows the
//     GPT-2 pattern (contractions, letter runs, digit runs of at most `max_digits`, punctuation runs, white space),
//     every byte is mapped to a printable code point, and merges are applied by rank;
//   * SentencePiece-style BPE (Llama-2 / Mistral-v1): spaces become U+2581, the text is merged as one piece, unknown
//     characters fall back to <0xNN> byte tokens.
// Added (special) tokens are matched literally before anything else.  Counterpart of the reference's tokenizer
// binding (Rust `tokenizers` behind a C ABI: create_tokenizer_from_file / encode / decode / num_ids / get_id,
// src/tokenizer/): the same five operations are exported with C linkage by the core module.
//
// The scanner classifies characters with Unicode tables (letters L*, numbers N*, White_Space; generated into
// unicode_tables.h) and evaluates the word pattern as a first-match alternation, so token boundaries are those of
// the regular-expression engine the format's own library uses; two patterns are known: GPT-2's (ByteLevel) and the
// cl100k family's (Llama-3, Qwen-2).  decode(encode(s)) == s always holds for byte-level models.
#pragma once
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <limits>
#include <memory>
#include <mutex>
#include <queue>
#include <sstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../util/minijson.h"
#include "unicode_tables.h"

namespace blitz {

class Tokenizer {
 public:
  static Tokenizer from_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("tokenizer: cannot open " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return from_json(ss.str());
  }

  static Tokenizer from_json(const std::string& text) {
    const json::Value root = json::parse(text);
    Tokenizer t;
    const json::Value& model = root.at("model");
    if (const json::Value* ty = model.find("type"))
      if (ty->type == json::Value::String && ty->str != "BPE") throw std::runtime_error("tokenizer: only BPE models");
    for (const auto& kv : model.at("vocab").obj) t.add_token(kv.first, kv.second.as_int());
    int rank = 0;
    for (const json::Value& m : model.at("merges").arr) {
      std::string a, b;
      if (m.type == json::Value::String) {
        const size_t sp = m.str.find(' ');
        if (sp == std::string::npos) continue;
        a = m.str.substr(0, sp);
        b = m.str.substr(sp + 1);
      } else if (m.type == json::Value::Array && m.arr.size() == 2) {
        a = m.arr[0].str;
        b = m.arr[1].str;
      } else {
        continue;
      }
      t.merges_.emplace(a + '\x01' + b, rank++);
    }
    if (const json::Value* bf = model.find("byte_fallback")) t.byte_fallback_ = bf->type == json::Value::Bool && bf->b;
    if (const json::Value* unk = model.find("unk_token"))
      if (unk->type == json::Value::String) {
        auto it = t.vocab_.find(unk->str);
        if (it != t.vocab_.end()) t.unk_id_ = it->second;
      }
    // byte-level if the pre-tokenizer or decoder says so; otherwise SentencePiece conventions
    t.byte_level_ = mentions(root.find("pre_tokenizer"), "ByteLevel") || mentions(root.find("decoder"), "ByteLevel");
    // the word pattern: ByteLevel's own (GPT-2) unless a Split pre-tokenizer carries the cl100k-family expression
    auto has = [&](const char* needle) { return text.find(needle) != std::string::npos; };
    t.cl100k_ = has("?\\\\p{L}+|\\\\p{N}") || has("?\\p{L}+|\\p{N}");
    if (has("\\\\p{N}{1,3}") || has("\\p{N}{1,3}")) t.max_digits_ = 3;
    else if (t.cl100k_ && (has("|\\\\p{N}|") || has("|\\p{N}|"))) t.max_digits_ = 1;
    else t.max_digits_ = std::numeric_limits<int>::max();
    if (const json::Value* add = root.find("added_tokens"))
      for (const json::Value& a : add->arr) {
        const std::string& content = a.at("content").str;
        const int64_t id64 = a.at("id").as_int();
        t.add_token(content, id64);
        const int32_t id = static_cast<int32_t>(id64);
        bool special = false;
        if (const json::Value* sp = a.find("special")) special = sp->type == json::Value::Bool && sp->b;
        t.added_.push_back({content, id, special});
        if (id >= 0) {
          if (static_cast<size_t>(id) >= t.added_flag_.size()) t.added_flag_.resize(static_cast<size_t>(id) + 1, 0);
          t.added_flag_[static_cast<size_t>(id)] = special ? 2 : 1;
        }
      }
    t.init_byte_maps();
    return t;
  }

  int32_t num_ids() const { return static_cast<int32_t>(id_to_token_.size()); }
  // An added token that the tokenizer file marks as special (end-of-text and the like).
  bool is_special(int32_t id) const {
    return id >= 0 && static_cast<size_t>(id) < added_flag_.size() && added_flag_[static_cast<size_t>(id)] == 2;
  }
  // -1 when the token string is unknown.
  int32_t get_id(const std::string& token) const {
    auto it = vocab_.find(token);
    return it == vocab_.end() ? -1 : it->second;
  }
  const std::string& token(int32_t id) const {
    static const std::string empty;
    return id >= 0 && id < num_ids() ? id_to_token_[id] : empty;
  }

  std::vector<int32_t> encode(std::string_view text) const {
    std::vector<int32_t> out;
    size_t pos = 0;
    // next occurrence of every added token at or after `pos`, searched again only once `pos` has passed it: every
    // added token scans the text once in total, however many of them the text contains
    constexpr size_t kUnknown = std::string_view::npos - 1;
    std::vector<size_t> next_at(added_.size(), kUnknown);
    while (pos < text.size()) {
      // earliest added token at or after pos (longest on ties)
      size_t best = std::string_view::npos, best_len = 0;
      int32_t best_id = -1;
      for (size_t ai = 0; ai < added_.size(); ++ai) {
        const Added& a = added_[ai];
        if (a.content.empty()) continue;
        if (next_at[ai] == kUnknown || (next_at[ai] != std::string_view::npos && next_at[ai] < pos))
          next_at[ai] = text.find(a.content, pos);
        const size_t f = next_at[ai];
        if (f != std::string_view::npos && (f < best || (f == best && a.content.size() > best_len))) {
          best = f;
          best_len = a.content.size();
          best_id = a.id;
        }
      }
      const size_t end = best == std::string_view::npos ? text.size() : best;
      if (end > pos) encode_plain(text.substr(pos, end - pos), out);
      if (best == std::string_view::npos) break;
      out.push_back(best_id);
      pos = best + best_len;
    }
    return out;
  }

  std::string decode(const std::vector<int32_t>& ids, bool skip_special = true) const {
    std::string out, pending;
    auto flush = [&]() {
      if (pending.empty()) return;
      if (byte_level_) {
        size_t i = 0;
        while (i < pending.size()) {
          uint32_t cp;
          const size_t n = utf8_decode(pending, i, cp);
          i += n;
          auto it = cp_to_byte_.find(cp);
          if (it != cp_to_byte_.end()) out.push_back(static_cast<char>(it->second));
          else json_put(out, cp);
        }
      } else {
        // U+2581 -> space
        size_t i = 0;
        while (i < pending.size()) {
          if (pending.compare(i, 3, "\xE2\x96\x81") == 0) { out.push_back(' '); i += 3; }
          else out.push_back(pending[i++]);
        }
      }
      pending.clear();
    };
    for (int32_t id : ids) {
      if (id < 0 || id >= num_ids()) continue;
      if (is_added(id)) {
        flush();
        if (!(skip_special && is_special(id))) out += id_to_token_[id];
        continue;
      }
      const std::string& tk = id_to_token_[id];
      if (!byte_level_ && tk.size() == 6 && tk.compare(0, 3, "<0x") == 0 && tk[5] == '>') {
        flush();
        out.push_back(static_cast<char>(std::stoi(tk.substr(3, 2), nullptr, 16)));
        continue;
      }
      pending += tk;
    }
    flush();
    if (!byte_level_ && !out.empty() && out[0] == ' ') out.erase(0, 1);  // the prepended word boundary
    return out;
  }

 private:
  struct Added { std::string content; int32_t id; bool special; };
  std::unordered_map<std::string, int32_t> vocab_;
  std::vector<std::string> id_to_token_;
  std::unordered_map<std::string, int> merges_;
  std::vector<Added> added_;
  bool byte_level_ = true, byte_fallback_ = false;
  int32_t unk_id_ = -1;
  int max_digits_ = std::numeric_limits<int>::max();
  bool cl100k_ = false;   // word pattern of the cl100k family instead of GPT-2's
  std::string byte_to_str_[256];
  std::unordered_map<uint32_t, uint8_t> cp_to_byte_;
  mutable std::unique_ptr<std::mutex> cache_mu_ = std::make_unique<std::mutex>();
  mutable std::unordered_map<std::string, std::vector<int32_t>> cache_;

  void add_token(const std::string& s, int64_t id) {
    if (id < 0) return;
    // the id table is dense: an id far beyond any real vocabulary (a damaged file) must not size it
    if (id >= (int64_t{1} << 24)) throw std::runtime_error("tokenizer: token id " + std::to_string(id) + " is out of range");
    vocab_[s] = static_cast<int32_t>(id);
    if (static_cast<size_t>(id) >= id_to_token_.size()) id_to_token_.resize(static_cast<size_t>(id) + 1);
    id_to_token_[static_cast<size_t>(id)] = s;
  }
  // per id: 0 ordinary, 1 added token, 2 added and special (looked up for every token of a decode)
  std::vector<uint8_t> added_flag_;
  bool is_added(int32_t id) const {
    return id >= 0 && static_cast<size_t>(id) < added_flag_.size() && added_flag_[static_cast<size_t>(id)] != 0;
  }
  static bool mentions(const json::Value* v, const char* what) {
    if (!v) return false;
    if (v->type == json::Value::String) return v->str == what;
    for (const auto& kv : v->obj) if (mentions(&kv.second, what)) return true;
    for (const auto& e : v->arr) if (mentions(&e, what)) return true;
    return false;
  }
  static void json_put(std::string& o, uint32_t cp) {
    if (cp < 0x80) o.push_back(static_cast<char>(cp));
    else if (cp < 0x800) { o.push_back(static_cast<char>(0xC0 | (cp >> 6))); o.push_back(static_cast<char>(0x80 | (cp & 0x3F))); }
    else if (cp < 0x10000) {
      o.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      o.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      o.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  static size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1; }
  static size_t utf8_decode(const std::string& s, size_t i, uint32_t& cp) {
    const unsigned char c = s[i];
    size_t n = utf8_len(c);
    if (i + n > s.size()) n = 1;
    if (n == 1) { cp = c; return 1; }
    cp = c & (0xFF >> (n + 1));
    for (size_t k = 1; k < n; ++k) cp = (cp << 6) | (static_cast<unsigned char>(s[i + k]) & 0x3F);
    return n;
  }
  // GPT-2 byte <-> printable code point table: printable Latin-1 bytes map to themselves, the rest to U+0100...
  void init_byte_maps() {
    int extra = 0;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      const uint32_t cp = keep ? static_cast<uint32_t>(b) : 256u + static_cast<uint32_t>(extra++);
      std::string s;
      json_put(s, cp);
      byte_to_str_[b] = s;
      cp_to_byte_[cp] = static_cast<uint8_t>(b);
    }
  }

  // ---- word scanner -------------------------------------------------------------------------------------------
  // One decoded character of the text: code point and byte length (malformed bytes count as one-byte characters of
  // class "other", so nothing is ever lost).
  struct Ch { uint32_t cp; uint32_t len; };
  static Ch char_at(std::string_view s, size_t i) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    size_t n = utf8_len(c);
    if (n == 1 || i + n > s.size()) return {c < 0x80 ? c : 0xFFFDu, 1};
    uint32_t cp = c & (0xFFu >> (n + 1));
    for (size_t k = 1; k < n; ++k) {
      const unsigned char cc = static_cast<unsigned char>(s[i + k]);
      if ((cc & 0xC0) != 0x80) return {0xFFFDu, 1};
      cp = (cp << 6) | (cc & 0x3F);
    }
    return {cp, static_cast<uint32_t>(n)};
  }
  enum Cls { kL, kN, kS, kO };   // letter, number, white space, anything else
  static Cls cls(uint32_t cp) {
    if (cp < 0x80) {   // the common case without the range tables
      if ((cp | 0x20) >= 'a' && (cp | 0x20) <= 'z') return kL;
      if (cp >= '0' && cp <= '9') return kN;
      return (cp == ' ' || (cp >= 0x09 && cp <= 0x0D)) ? kS : kO;
    }
    if (unicode::is_letter(cp)) return kL;
    if (unicode::is_number(cp)) return kN;
    if (unicode::is_space(cp)) return kS;
    return kO;
  }
  static bool is_crlf(uint32_t cp) { return cp == '\r' || cp == '\n'; }

  // End of the contraction that starts at i ('s 't 're 've 'm 'll 'd, tried in this order), or i if there is none.
  static size_t contraction_end(std::string_view s, size_t i, bool ignore_case) {
    if (s[i] != '\'' || i + 1 >= s.size()) return i;
    static const char* kContr[] = {"s", "t", "re", "ve", "m", "ll", "d"};
    for (const char* c : kContr) {
      const size_t l = std::char_traits<char>::length(c);
      if (i + 1 + l > s.size()) continue;
      bool ok = true;
      for (size_t k = 0; k < l && ok; ++k) {
        char x = s[i + 1 + k];
        if (ignore_case && x >= 'A' && x <= 'Z') x = static_cast<char>(x - 'A' + 'a');
        ok = x == c[k];
      }
      if (ok) return i + 1 + l;
    }
    return i;
  }
  // End of the maximal run of characters of class `want` starting at i (at most `limit` characters).
  static size_t run_end(std::string_view s, size_t i, Cls want, int limit = std::numeric_limits<int>::max()) {
    int k = 0;
    while (i < s.size() && k < limit) {
      const Ch c = char_at(s, i);
      if (cls(c.cp) != want) break;
      i += c.len;
      ++k;
    }
    return i;
  }
  // White space starting at i, as the tail of both patterns matches it: `\s+(?!\S)` (the run without its last
  // character when something follows it, so that the last blank can prefix the next word), else `\s+`.
  static size_t space_end(std::string_view s, size_t i) {
    size_t j = i, last = i, count = 0;
    while (j < s.size()) {
      const Ch c = char_at(s, j);
      if (cls(c.cp) != kS) break;
      last = j;
      j += c.len;
      ++count;
    }
    if (j < s.size() && count > 1) return last;
    return j;
  }

  // End of the word that starts at i.  Two patterns are implemented as first-match alternations, exactly as a
  // regular-expression engine evaluates them:
  //   GPT-2 (ByteLevel's own):  's|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+
  //   cl100k family (Llama-3, Qwen-2; a Split pre-tokenizer in tokenizer.json):
  //     (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,k}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
  size_t next_word(std::string_view s, size_t i) const {
    const size_t n = s.size();
    const size_t ce = contraction_end(s, i, cl100k_);
    if (ce != i) return ce;
    const Ch c0 = char_at(s, i);
    const Cls k0 = cls(c0.cp);
    const size_t i1 = i + c0.len;
    const bool has1 = i1 < n;
    const Ch c1 = has1 ? char_at(s, i1) : Ch{0, 0};
    const Cls k1 = has1 ? cls(c1.cp) : kO;
    if (cl100k_) {
      // [^\r\n\p{L}\p{N}]?\p{L}+
      if (k0 != kL && k0 != kN && !is_crlf(c0.cp) && has1 && k1 == kL) return run_end(s, i1, kL);
      if (k0 == kL) return run_end(s, i, kL);
      // \p{N}{1,k}
      if (k0 == kN) return run_end(s, i, kN, max_digits_);
      // ` ?[^\s\p{L}\p{N}]+[\r\n]*`
      size_t j = i;
      if (c0.cp == ' ' && has1 && k1 == kO) j = i1;
      if (j < n && cls(char_at(s, j).cp) == kO) {
        j = run_end(s, j, kO);
        while (j < n && is_crlf(static_cast<unsigned char>(s[j]))) ++j;
        return j;
      }
      // \s*[\r\n]+ : through the last line break of the white-space run, if it has one
      size_t e = i, last_break_end = i;
      while (e < n) {
        const Ch c = char_at(s, e);
        if (cls(c.cp) != kS) break;
        e += c.len;
        if (is_crlf(c.cp)) last_break_end = e;
      }
      if (last_break_end != i) return last_break_end;
      return space_end(s, i);
    }
    // GPT-2: an optional blank, then a run of one class
    size_t j = i;
    Cls k = k0;
    if (c0.cp == ' ' && has1 && k1 != kS) { j = i1; k = k1; }
    if (k == kL) return run_end(s, j, kL);
    if (k == kN) return run_end(s, j, kN, max_digits_);
    if (k == kO) return run_end(s, j, kO);
    return space_end(s, i);
  }

  // Apply the merges to the symbols of one piece: always the adjacent pair of lowest rank, the leftmost one among
  // equals.  The symbols form a linked list and the candidate pairs a heap keyed by (rank, position), so a piece of
  // n symbols costs O(n log n) whatever it contains (a long run of one letter, or a whole prompt for the
  // SentencePiece-style models, which merge the text as one piece).  A heap entry remembers the byte lengths of its
  // two symbols; symbols only ever grow, so an entry whose lengths no longer match is stale and skipped.
  void bpe(std::vector<std::string>& sym) const {
    const int n = static_cast<int>(sym.size());
    if (n < 2) return;
    struct Node { int prev, next; bool alive; };
    std::vector<Node> nd(static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) nd[i] = {i - 1, i + 1 < n ? i + 1 : -1, true};
    struct Ent { int rank, left; uint32_t len_l, len_r; };
    auto later = [](const Ent& a, const Ent& b) { return a.rank != b.rank ? a.rank > b.rank : a.left > b.left; };
    std::priority_queue<Ent, std::vector<Ent>, decltype(later)> heap(later);
    std::string key;
    auto consider = [&](int l) {
      const int r = nd[l].next;
      if (r < 0) return;
      key.assign(sym[l]);
      key.push_back('\x01');
      key += sym[r];
      auto it = merges_.find(key);
      if (it != merges_.end())
        heap.push({it->second, l, static_cast<uint32_t>(sym[l].size()), static_cast<uint32_t>(sym[r].size())});
    };
    for (int i = 0; i + 1 < n; ++i) consider(i);
    while (!heap.empty()) {
      const Ent e = heap.top();
      heap.pop();
      const int l = e.left;
      if (!nd[l].alive) continue;
      const int r = nd[l].next;
      if (r < 0 || sym[l].size() != e.len_l || sym[r].size() != e.len_r) continue;
      sym[l] += sym[r];
      sym[r].clear();
      nd[r].alive = false;
      nd[l].next = nd[r].next;
      if (nd[r].next >= 0) nd[nd[r].next].prev = l;
      if (nd[l].prev >= 0) consider(nd[l].prev);
      consider(l);
    }
    size_t w = 0;
    for (int i = 0; i < n; ++i) {
      if (!nd[i].alive) continue;
      if (w != static_cast<size_t>(i)) sym[w] = std::move(sym[i]);
      ++w;
    }
    sym.resize(w);
  }

  void emit(const std::vector<std::string>& sym, std::vector<int32_t>& out) const {
    for (const std::string& s : sym) {
      auto it = vocab_.find(s);
      if (it != vocab_.end()) { out.push_back(it->second); continue; }
      if (byte_fallback_) {
        bool ok = true;
        std::vector<int32_t> tmp;
        for (unsigned char c : s) {
          char buf[8];
          std::snprintf(buf, sizeof buf, "<0x%02X>", c);
          auto bt = vocab_.find(buf);
          if (bt == vocab_.end()) { ok = false; break; }
          tmp.push_back(bt->second);
        }
        if (ok) { out.insert(out.end(), tmp.begin(), tmp.end()); continue; }
      }
      if (unk_id_ >= 0) out.push_back(unk_id_);
    }
  }

  void encode_plain(std::string_view text, std::vector<int32_t>& out) const {
    if (byte_level_) {
      size_t i = 0;
      while (i < text.size()) {
        const size_t j = next_word(text, i);
        const std::string word(text.substr(i, j - i));
        i = j;
        {
          std::lock_guard<std::mutex> g(*cache_mu_);
          auto it = cache_.find(word);
          if (it != cache_.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); continue; }
        }
        std::vector<std::string> sym;
        sym.reserve(word.size());
        for (unsigned char c : word) sym.push_back(byte_to_str_[c]);
        bpe(sym);
        std::vector<int32_t> ids;
        emit(sym, ids);
        out.insert(out.end(), ids.begin(), ids.end());
        std::lock_guard<std::mutex> g(*cache_mu_);
        if (cache_.size() < 200000 && word.size() <= 256) cache_.emplace(word, std::move(ids));   // words, not blobs
      }
    } else {
      std::string norm = "\xE2\x96\x81";
      for (char c : text) {
        if (c == ' ') norm += "\xE2\x96\x81";
        else norm.push_back(c);
      }
      std::vector<std::string> sym;
      for (size_t i = 0; i < norm.size();) {
        const size_t n = utf8_len(static_cast<unsigned char>(norm[i]));
        sym.push_back(norm.substr(i, n));
        i += n;
      }
      bpe(sym);
      emit(sym, out);
    }
  }
};

}  // namespace blitz
