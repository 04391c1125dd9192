// Paged KV-cache bookkeeping: an O(1) page allocator and the server-side batch
// state (token lists, page tables, stop criteria, page-table staging).
//
// The device memory itself is one tensor [layers][pages][K|V][page][kv_heads][head_dim]
// owned by the engine; a page id addresses the same page in every layer, as in
// the reference (src/blitz/cache_manager.h:123-143).  The reference finds free
// pages by scanning a byte mask (cache_manager.h:163-196); here a free-list
// stack makes allocate/free O(pages touched).  Batch mirrors the behaviour of
// src/blitz/batch.h: a request reserves ceil((prompt + 1) / page) pages at
// prefill (:246-250), grows by one page when its last page fills (:280-296),
// `filter` drops finished requests and returns their pages (:298-418),
// `extend` concatenates cached batches for one decode step (:483-576).
#pragma once
#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <tuple>
#include <vector>

namespace blitz {

class PagePool {
 public:
  explicit PagePool(int num_pages, int page_size) : page_size_(page_size), in_use_(num_pages, 0) {
    free_.reserve(num_pages);
    for (int i = num_pages - 1; i >= 0; --i) free_.push_back(i);
  }
  int page_size() const { return page_size_; }
  int total_pages() const { return static_cast<int>(in_use_.size()); }
  int free_pages() const { return static_cast<int>(free_.size()); }
  int used_pages() const { return total_pages() - free_pages(); }

  // All-or-nothing: returns false (and allocates nothing) when fewer than n pages are free.
  bool allocate(int n, std::vector<int32_t>& out) {
    if (n < 0 || n > free_pages()) return false;
    for (int i = 0; i < n; ++i) {
      int p = free_.back();
      free_.pop_back();
      in_use_[p] = 1;
      out.push_back(p);
    }
    return true;
  }
  void release(const std::vector<int32_t>& pages) {
    for (int p : pages) {
      if (p < 0 || p >= total_pages() || !in_use_[p]) throw std::logic_error("PagePool: double free or bad page id");
      in_use_[p] = 0;
      free_.push_back(p);
    }
  }
  bool is_used(int p) const { return p >= 0 && p < total_pages() && in_use_[p]; }

 private:
  int page_size_;
  std::vector<int32_t> free_;
  std::vector<uint8_t> in_use_;
};

enum FinishReason : int { kFinishNone = -1, kFinishLength = 0, kFinishEos = 1, kFinishStop = 2 };

struct SeqSpec {
  uint64_t id = 0;
  std::vector<int32_t> prompt;
  int max_new_tokens = 16;
  bool ignore_eos = true;
  int eos_token = -1;
  // sampling (greedy when do_sample is false)
  bool do_sample = false;
  float temperature = 1.f, top_p = 1.f;
  int top_k = 0;
  uint64_t seed = 0;
};

struct SeqState {
  SeqSpec spec;
  std::vector<int32_t> generated;
  std::vector<int32_t> pages;
  int cached_tokens = 0;  // tokens whose K/V are in the cache
  FinishReason finish = kFinishNone;
  int total_len() const { return static_cast<int>(spec.prompt.size() + generated.size()); }
};

// Offsets (in int32 elements) of the fields of the pinned staging array one step copies to the device.
struct MetaLayout {
  int ids = 0, pos = 0, slot = 0, tok_indptr = 0, page_indptr = 0, last_page_len = 0, page_indices = 0, total = 0;
  static MetaLayout make(int max_tokens, int max_batch, int max_pages) {
    MetaLayout m;
    m.ids = 0;
    m.pos = m.ids + max_tokens;
    m.slot = m.pos + max_tokens;
    m.tok_indptr = m.slot + max_tokens;
    m.page_indptr = m.tok_indptr + max_batch + 1;
    m.last_page_len = m.page_indptr + max_batch + 1;
    m.page_indices = m.last_page_len + max_batch;
    m.total = m.page_indices + max_pages;
    return m;
  }
};

class Batch {
 public:
  Batch(uint64_t id, PagePool* pool) : id_(id), pool_(pool) {}
  ~Batch() { clear(); }
  Batch(const Batch&) = delete;
  Batch& operator=(const Batch&) = delete;

  uint64_t id() const { return id_; }
  int size() const { return static_cast<int>(seqs_.size()); }
  const std::vector<SeqState>& seqs() const { return seqs_; }
  bool is_decode() const { return decode_; }
  void set_decode(bool d) { decode_ = d; }

  // Sum over requests of page-padded (prompt + max_new_tokens): the router's `max_tokens`.
  uint32_t max_tokens() const {
    const int ps = pool_->page_size();
    uint64_t t = 0;
    for (auto& s : seqs_) t += (static_cast<uint64_t>(s.spec.prompt.size() + s.spec.max_new_tokens) + ps - 1) / ps * ps;
    return static_cast<uint32_t>(t);
  }
  int num_pages() const {
    int n = 0;
    for (auto& s : seqs_) n += static_cast<int>(s.pages.size());
    return n;
  }
  int num_prompt_tokens() const {
    int n = 0;
    for (auto& s : seqs_) n += static_cast<int>(s.spec.prompt.size());
    return n;
  }

  // Admit prompts: each reserves ceil((len + 1) / page) pages.  All-or-nothing.
  bool add_prompts(const std::vector<SeqSpec>& specs) {
    const int ps = pool_->page_size();
    int need = 0;
    for (auto& sp : specs) need += (static_cast<int>(sp.prompt.size()) + 1 + ps - 1) / ps;
    if (need > pool_->free_pages()) return false;
    for (auto& sp : specs) {
      SeqState st;
      st.spec = sp;
      pool_->allocate((static_cast<int>(sp.prompt.size()) + 1 + ps - 1) / ps, st.pages);
      seqs_.push_back(std::move(st));
    }
    return true;
  }

  // After a prefill forward: all prompt tokens are cached.
  void mark_prefilled() {
    for (auto& s : seqs_) s.cached_tokens = static_cast<int>(s.spec.prompt.size());
  }

  // Append one sampled token per live request (order = seqs()), evaluate stop criteria and
  // make sure the page that will hold the token's K/V on the next step exists.
  // Returns false if the pool ran out of pages (the token is still recorded and the request is finished).
  bool append_tokens(const std::vector<int32_t>& tokens, bool count_cached) {
    if (tokens.size() != seqs_.size()) throw std::invalid_argument("append_tokens: size mismatch");
    const int ps = pool_->page_size();
    bool ok = true;
    for (size_t i = 0; i < seqs_.size(); ++i) {
      auto& s = seqs_[i];
      if (s.finish != kFinishNone) continue;
      if (count_cached) s.cached_tokens += 1;  // the previous step wrote the fed token's K/V
      s.generated.push_back(tokens[i]);
      if (!s.spec.ignore_eos && s.spec.eos_token >= 0 && tokens[i] == s.spec.eos_token)
        s.finish = kFinishEos;
      else if (static_cast<int>(s.generated.size()) >= s.spec.max_new_tokens)
        s.finish = kFinishLength;
      if (s.finish == kFinishNone) {
        // the next step writes position total_len() - 1
        const int need = (s.total_len() + ps - 1) / ps;
        while (static_cast<int>(s.pages.size()) < need) {
          if (!pool_->allocate(1, s.pages)) {
            // no page for the next position: the request ends here (reported as a length stop) instead of writing its
            // next K/V outside its pages; callers that budget blocks up front (the router does) never get here
            s.finish = kFinishLength;
            ok = false;
            break;
          }
        }
      }
    }
    return ok;
  }

  // Keep only `keep` ids (finished or dropped requests release their pages).
  void filter(const std::vector<uint64_t>& keep) {
    // the common call of a decode step keeps everybody, in order: nothing to do
    if (keep.size() == seqs_.size()) {
      bool same = true;
      for (size_t i = 0; i < keep.size() && same; ++i) same = keep[i] == seqs_[i].spec.id;
      if (same) return;
    }
    std::vector<SeqState> kept;
    for (auto& s : seqs_) {
      if (std::find(keep.begin(), keep.end(), s.spec.id) != keep.end()) {
        kept.push_back(std::move(s));
      } else {
        pool_->release(s.pages);
      }
    }
    seqs_ = std::move(kept);
  }
  std::vector<uint64_t> unfinished_ids() const {
    std::vector<uint64_t> ids;
    for (auto& s : seqs_)
      if (s.finish == kFinishNone) ids.push_back(s.spec.id);
    return ids;
  }
  // Compact per-request views for the serving loop (the per-step paths must not copy prompts or token histories).
  // The last `k` generated tokens of request `id` (fewer if it has not generated that many; empty if unknown).
  std::vector<int32_t> generated_tail(uint64_t id, int k) const {
    for (auto& s : seqs_) {
      if (s.spec.id != id) continue;
      const size_t n = s.generated.size(), take = std::min<size_t>(n, static_cast<size_t>(std::max(0, k)));
      return std::vector<int32_t>(s.generated.end() - static_cast<long>(take), s.generated.end());
    }
    return {};
  }
  // End request `id` for a reason the caller found (a stop sequence in its text).  False if it is unknown or has
  // finished already, in which case its recorded reason stays.
  bool finish_request(uint64_t id, int reason) {
    for (auto& s : seqs_) {
      if (s.spec.id != id) continue;
      if (s.finish != kFinishNone) return false;
      s.finish = static_cast<FinishReason>(reason);
      return true;
    }
    return false;
  }
  std::vector<uint64_t> request_ids() const {
    std::vector<uint64_t> ids;
    ids.reserve(seqs_.size());
    for (auto& s : seqs_) ids.push_back(s.spec.id);
    return ids;
  }
  std::vector<int> prompt_lens() const {
    std::vector<int> n;
    n.reserve(seqs_.size());
    for (auto& s : seqs_) n.push_back(static_cast<int>(s.spec.prompt.size()));
    return n;
  }
  // (request id, finish code or -1, tokens generated so far) of every request, in batch order.
  std::vector<std::tuple<uint64_t, int, int>> emit_info() const {
    std::vector<std::tuple<uint64_t, int, int>> out;
    out.reserve(seqs_.size());
    for (auto& s : seqs_) out.emplace_back(s.spec.id, static_cast<int>(s.finish), static_cast<int>(s.generated.size()));
    return out;
  }
  // Wire bytes of one `Generation` message per request (field 1 of the prefill / decode responses of the
  // generate.v2 contract), carrying this step's token: request_id, tokens{ids, logprobs = 0, texts = "<id>",
  // is_special = false} and, for requests that finished with this token, generated_text{text, generated_tokens,
  // finish_reason}.  Building these messages one by one in the scripting layer costs more than the decode step's
  // launch overhead at large batch; the service parses the bytes back in one call.
  std::string encode_generations(const std::vector<int32_t>& tokens) const {
    if (tokens.size() != seqs_.size()) throw std::invalid_argument("encode_generations: one token per request");
    auto put_varint = [](std::string& o, uint64_t v) {
      while (v >= 0x80) { o.push_back(static_cast<char>((v & 0x7f) | 0x80)); v >>= 7; }
      o.push_back(static_cast<char>(v));
    };
    std::string out, gen, sub;
    out.reserve(seqs_.size() * 32);
    for (size_t i = 0; i < seqs_.size(); ++i) {
      const SeqState& s = seqs_[i];
      const std::string text = "<" + std::to_string(tokens[i]) + ">";
      gen.clear();
      gen.push_back(0x08); put_varint(gen, s.spec.id);
      sub.clear();
      sub.push_back(0x08); put_varint(sub, static_cast<uint32_t>(tokens[i]));
      sub.push_back(0x15); sub.append(4, '\0');
      sub.push_back(0x1a); put_varint(sub, text.size()); sub += text;
      sub.push_back(0x20); sub.push_back(0);
      gen.push_back(0x1a); put_varint(gen, sub.size()); gen += sub;
      if (s.finish != kFinishNone) {
        sub.clear();
        sub.push_back(0x0a); put_varint(sub, text.size()); sub += text;
        sub.push_back(0x10); put_varint(sub, s.generated.size());
        sub.push_back(0x18); put_varint(sub, static_cast<uint64_t>(s.finish));
        gen.push_back(0x22); put_varint(gen, sub.size()); gen += sub;
      }
      out.push_back(0x0a); put_varint(out, gen.size()); out += gen;
    }
    return out;
  }
  // Rows of the batch that sample their next token instead of taking the arg-max, with their parameters; the seed
  // of a row is mixed with the number of tokens it has generated so that every step draws a fresh, reproducible
  // number.  Empty when the whole batch is greedy (the common case: one pass over the batch, no allocation).
  struct SamplingRows {
    std::vector<int64_t> rows;
    std::vector<float> temperature, top_p;
    std::vector<int32_t> top_k;
    std::vector<int64_t> seeds;
  };
  SamplingRows sampling_rows() const {
    SamplingRows out;
    for (size_t i = 0; i < seqs_.size(); ++i) {
      const SeqSpec& sp = seqs_[i].spec;
      if (!sp.do_sample) continue;
      out.rows.push_back(static_cast<int64_t>(i));
      out.temperature.push_back(sp.temperature > 0.f ? sp.temperature : 1.f);
      out.top_p.push_back(sp.top_p > 0.f && sp.top_p <= 1.f ? sp.top_p : 1.f);
      out.top_k.push_back(sp.top_k > 0 ? sp.top_k : 0);
      const uint64_t mixed = sp.seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(seqs_[i].generated.size()) + 1ull;
      out.seeds.push_back(static_cast<int64_t>(mixed));
    }
    return out;
  }
  bool none_generated() const {
    for (auto& s : seqs_)
      if (!s.generated.empty()) return false;
    return true;
  }
  // Pages that hold the prompts' KV, request after request (what a migration ships).
  std::vector<int32_t> prompt_page_ids() const {
    const int ps = pool_->page_size();
    std::vector<int32_t> out;
    for (auto& s : seqs_) {
      const size_t used = (s.spec.prompt.size() + ps - 1) / ps;
      out.insert(out.end(), s.pages.begin(), s.pages.begin() + static_cast<long>(std::min(used, s.pages.size())));
    }
    return out;
  }
  // The same for the requests `ids` with prompt lengths `lens`, in that order: both ends of a migration build
  // their page lists from the requests named in the RPC, so that entry i of one side always faces entry i of the
  // other.  A request that is not (or no longer) in this batch still takes its ceil(len / page) entries, filled
  // with -1, which the push kernel skips: the two lists have the same length whatever each side has filtered.
  std::vector<int32_t> prompt_page_ids_for(const std::vector<uint64_t>& ids, const std::vector<int>& lens) const {
    if (ids.size() != lens.size()) throw std::invalid_argument("prompt_page_ids_for: one length per request");
    const int ps = pool_->page_size();
    std::vector<int32_t> out;
    for (size_t i = 0; i < ids.size(); ++i) {
      const SeqState* found = nullptr;
      for (auto& s : seqs_)
        if (s.spec.id == ids[i]) { found = &s; break; }
      const size_t used = (static_cast<size_t>(std::max(0, lens[i])) + ps - 1) / ps;
      for (size_t k = 0; k < used; ++k)
        out.push_back(found && k < found->pages.size() ? found->pages[k] : -1);
    }
    return out;
  }
  // Move the requests of `other` to the end of this batch (page ownership moves too).
  void extend(Batch& other) {
    if (other.pool_ != pool_) throw std::invalid_argument("extend: different pools");
    for (auto& s : other.seqs_) seqs_.push_back(std::move(s));
    other.seqs_.clear();
  }
  void clear() {
    for (auto& s : seqs_) pool_->release(s.pages);
    seqs_.clear();
  }

  // ---- staging for the device (int32 array laid out per MetaLayout)
  // Prefill: every prompt token, positions from 0.  Returns {num_tokens, num_page_entries}.
  std::pair<int, int> fill_prefill(int32_t* h, const MetaLayout& L) const {
    const int ps = pool_->page_size();
    int t = 0, np = 0;
    h[L.tok_indptr] = 0;
    h[L.page_indptr] = 0;
    for (size_t b = 0; b < seqs_.size(); ++b) {
      const auto& s = seqs_[b];
      const int n = static_cast<int>(s.spec.prompt.size());
      for (int i = 0; i < n; ++i) {
        h[L.ids + t + i] = s.spec.prompt[i];
        h[L.pos + t + i] = i;
        h[L.slot + t + i] = s.pages[i / ps] * ps + i % ps;
      }
      t += n;
      const int used = (n + ps - 1) / ps;
      for (int i = 0; i < used; ++i) h[L.page_indices + np + i] = s.pages[i];
      np += used;
      h[L.tok_indptr + b + 1] = t;
      h[L.page_indptr + b + 1] = np;
      h[L.last_page_len + b] = n ? n - (used - 1) * ps : 0;
    }
    return {t, np};
  }
  // Prefill in chunks, for prompts that together exceed what one forward pass takes: the window [tok0, tok0 +
  // max_tokens) over the prompts laid end to end.  Only the sequences the window touches get a row; a row's tokens
  // are the part of its prompt inside the window (positions continue where the previous chunk stopped) while its
  // page list covers everything up to the end of that part, i.e. the keys and values of earlier chunks too.
  struct PrefillChunk {
    int tokens = 0, pages = 0, rows = 0, first_seq = -1;
    std::vector<int> q_lens, kv_lens;  // per row: tokens in this chunk, tokens cached after it
    std::vector<int> ended;            // per row: 1 if the prompt ends in this chunk (its last row yields the first token)
  };
  PrefillChunk fill_prefill_chunk(int32_t* h, const MetaLayout& L, int64_t tok0, int max_tokens) const {
    const int ps = pool_->page_size();
    PrefillChunk c;
    int64_t base = 0;
    h[L.tok_indptr] = 0;
    h[L.page_indptr] = 0;
    for (size_t b = 0; b < seqs_.size(); ++b) {
      const auto& s = seqs_[b];
      const int64_t n = static_cast<int64_t>(s.spec.prompt.size());
      const int64_t lo = std::max<int64_t>(tok0, base) - base, hi = std::min<int64_t>(tok0 + max_tokens, base + n) - base;
      base += n;
      if (hi <= lo) continue;
      if (c.first_seq < 0) c.first_seq = static_cast<int>(b);
      for (int64_t i = lo; i < hi; ++i) {
        const int t = c.tokens + static_cast<int>(i - lo);
        h[L.ids + t] = s.spec.prompt[i];
        h[L.pos + t] = static_cast<int32_t>(i);
        h[L.slot + t] = s.pages[i / ps] * ps + static_cast<int32_t>(i % ps);
      }
      c.tokens += static_cast<int>(hi - lo);
      const int used = static_cast<int>((hi + ps - 1) / ps);
      for (int i = 0; i < used; ++i) h[L.page_indices + c.pages + i] = s.pages[i];
      c.pages += used;
      h[L.tok_indptr + c.rows + 1] = c.tokens;
      h[L.page_indptr + c.rows + 1] = c.pages;
      h[L.last_page_len + c.rows] = static_cast<int32_t>(hi - static_cast<int64_t>(used - 1) * ps);
      c.q_lens.push_back(static_cast<int>(hi - lo));
      c.kv_lens.push_back(static_cast<int>(hi));
      c.ended.push_back(hi == n ? 1 : 0);
      c.rows += 1;
    }
    return c;
  }
  // Decode: feed each request's last token at position total_len - 1; padded rows (b >= size) are
  // empty sequences whose cache write is skipped.  Returns the number of page entries.
  int fill_decode(int32_t* h, const MetaLayout& L, int pad_to) const {
    const int ps = pool_->page_size();
    const int B = size();
    int np = 0;
    h[L.page_indptr] = 0;
    for (int b = 0; b < B; ++b) {
      const auto& s = seqs_[b];
      const int n = s.total_len() - 1;  // position of the fed token
      if (s.finish != kFinishNone || n < 0 || n / ps >= static_cast<int>(s.pages.size())) {
        // a finished request, an empty one, or one without a page for the next position: the row is carried as
        // padding (no page, no cache write) instead of indexing past its page list; its token is meaningless
        h[L.ids + b] = 0;
        h[L.pos + b] = 0;
        h[L.slot + b] = -1;
        h[L.page_indptr + b + 1] = np;
        h[L.last_page_len + b] = 0;
        continue;
      }
      h[L.ids + b] = s.generated.empty() ? s.spec.prompt.back() : s.generated.back();
      h[L.pos + b] = n;
      h[L.slot + b] = s.pages[n / ps] * ps + n % ps;
      const int used = n / ps + 1;
      for (int i = 0; i < used; ++i) h[L.page_indices + np + i] = s.pages[i];
      np += used;
      h[L.page_indptr + b + 1] = np;
      h[L.last_page_len + b] = n + 1 - (used - 1) * ps;
    }
    for (int b = B; b < pad_to; ++b) {
      h[L.ids + b] = 0;
      h[L.pos + b] = 0;
      h[L.slot + b] = -1;
      h[L.page_indptr + b + 1] = np;
      h[L.last_page_len + b] = 0;
    }
    return np;
  }
  int max_seq_len() const {
    int m = 0;
    for (auto& s : seqs_) m = std::max(m, s.total_len());
    return m;
  }

  std::vector<SeqState>& mutable_seqs() { return seqs_; }

 private:
  uint64_t id_;
  PagePool* pool_;
  std::vector<SeqState> seqs_;
  bool decode_ = false;
};

}  // namespace blitz
