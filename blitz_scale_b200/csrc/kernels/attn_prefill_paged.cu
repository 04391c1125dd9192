// Causal prefill attention over the paged KV cache on tcgen05 for sm_100a: GQA, head_dim 64 or 128, queries of
// the current chunk against everything the cache holds for the sequence (earlier chunks and the chunk itself).
//
// Q comes from the fused QKV activation of the chunk (2-D TMA boxes); K and V come from the paged pool, where
// rope_kv_store has already put the chunk's own keys and values, as 3-D TMA boxes of one page (or 64 tokens of
// one) each, looked up through the page table.  A prompt that does not fit one batch is therefore prefetched in
// chunks with no other kernel: the first chunk has an empty prefix, later ones a prefix of whole earlier chunks.
//
// A work item is 256 query rows of one sequence and one q head, as two tiles of 128 rows that walk the KV blocks
// of 128 tokens up to the diagonal once for both:
//
//   S_t = Q_t K^T      tcgen05.mma, A = Q_t (smem), B = K block (smem), S_t in TMEM                      t = 0, 1
//   P_t = softmax      warpgroup t (4 warps, thread = row): one tcgen05.ld pass over S_t, running max and sum in
//                      fp32, P_t written back over S_t's first 64 columns (two 16-bit values per column)
//   O_t += P_t V       tcgen05.mma with A = P_t from tensor memory, accumulating in TMEM over all blocks
//
// A ninth warp issues the MMAs (one thread), a tenth the TMA loads.  While warpgroup 0 turns S_0 into P_0 the
// tensor core works on S_1 and on O_1, and the other way round: the two tiles ping-pong, and every K and V block
// feeds two tiles from one load.  O stays in TMEM for the whole walk: the maximum a row's probabilities refer to
// only moves when the true maximum has grown by more than 2^8 (the probabilities then stay below 256, harmless in
// 16 bits and fp32), and only then the warp rescales its O rows in place (tcgen05.ld, multiply, tcgen05.st); with
// ordinary inputs that happens in the first block or two of a row and never again.
//
// The grid is persistent: one CTA per SM takes work items in a fixed order (heaviest first, dealt back and forth
// over the CTAs so that every CTA gets a similar sum).  The three roles walk the same list on their own, all
// barrier phases come from running counts, and nothing is drained between items: the next item's Q, K and V are
// loaded and its first S products issued while the warpgroups still write the previous item's output, so the
// latency of starting an item (its page ids, its first loads, the first MMA) is paid once per CTA, not per item.
//
// Replaces FlashInfer's BatchPrefillWithRaggedKVCacheWrapper / paged wrapper calls and their host Plan()
// (src/kernel/attention_prefill.cu:11-45, src/kernel/flashinfer_types.cu:24-49).
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include "common.cuh"

namespace blitz {

constexpr int kPpThreads = 320;  // warpgroup 0, warpgroup 1, MMA warp, load warp
constexpr int kPpTile = 128;     // q rows per tile and kv tokens per block
constexpr float kPpRescaleAt = 8.f;  // log2 units
constexpr int kPpWorkInts = 8;   // per (sequence, pair of tiles): first row, rows, first page entry, pages, cached tokens, pair

struct PagedPrefillParams {
  void* out;  // [tokens, q_heads * HD]
  int64_t out_stride;
  const int32_t* page_indices;  // page ids of every sequence, back to back
  const int32_t* work;          // [entries][kPpWorkInts], heaviest first
  int entries, q_heads, kv_heads, page_size, box_tokens, oob_row;
  float scale_log2;
  int* status;
  long long* trace;  // profiling aid (null in production): clock stamps of CTA 0's first item, see the set_trace call
};

constexpr int kPpTraceIters = 32, kPpTraceSlots = 8;
// role 0 / 1: first lane of warpgroup 0 / 1; role 2: the MMA thread
__device__ __forceinline__ void pp_trace(const PagedPrefillParams& p, bool on, int role, int j, int slot) {
  if (on && p.trace != nullptr && j < kPpTraceIters) p.trace[(role * kPpTraceIters + j) * kPpTraceSlots + slot] = clock64();
}

template <int HD>
struct PpCfg {
  static constexpr int kTileBytes = kPpTile * HD * 2;  // one Q, K or V tile
  static constexpr int kSlabs = HD / 64;               // 64-column slabs of 128 rows x 128 bytes
  static constexpr int kSmemBytes = 6 * kTileBytes + 1024 + 256;  // Q x 2 tiles, K x 2 stages, V x 2 stages
};

struct PpItem {
  int seq_start, q_len, pg0, npages, kv_len, prefix, q0, nt, nblk, head, kv_head;
  int nblk_t[2];
};
// Work item `idx` of the flattened list (entry x q head; the heads of one entry are neighbours, so CTAs that run
// at the same time share its K and V in L2).
__device__ __forceinline__ PpItem pp_item(const PagedPrefillParams& p, int idx) {
  PpItem it;
  const int entry = idx / p.q_heads;
  it.head = idx - entry * p.q_heads;
  it.kv_head = it.head / (p.q_heads / p.kv_heads);
  const int4 a = __ldg(reinterpret_cast<const int4*>(p.work + entry * kPpWorkInts));
  const int4 b = __ldg(reinterpret_cast<const int4*>(p.work + entry * kPpWorkInts + 4));
  it.seq_start = a.x; it.q_len = a.y; it.pg0 = a.z; it.npages = a.w; it.kv_len = b.x;
  it.prefix = it.kv_len - it.q_len;  // tokens of earlier chunks
  it.q0 = b.y * 2 * kPpTile;
  it.nt = (it.q0 + kPpTile < it.q_len) ? 2 : 1;
#pragma unroll
  for (int t = 0; t < 2; ++t) {  // blocks tile t needs: keys up to its last row's position
    const int last = min(it.kv_len, it.prefix + min(it.q_len, it.q0 + kPpTile * (t + 1)));
    it.nblk_t[t] = t < it.nt ? (last + kPpTile - 1) / kPpTile : 0;
  }
  it.nblk = max(it.nblk_t[0], it.nblk_t[1]);
  return it;
}
// The r-th item of this CTA: rounds alternate direction over the CTAs.  -1: this CTA has none in round r.
__device__ __forceinline__ int pp_index(int r, int total) {
  const int G = gridDim.x;
  const int idx = r * G + ((r & 1) ? G - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x));
  return idx < total ? idx : -1;
}

template <typename T, int HD, bool POLY>
__global__ void __launch_bounds__(kPpThreads, 1)
attn_prefill_paged_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                          const PagedPrefillParams p) {
  using C = PpCfg<HD>;
  constexpr int TB = C::kTileBytes;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdescS = ptx::make_idesc_f16(kFmt, 0u, 0u, 128, 128);
  constexpr uint32_t kIdescPV = ptx::make_idesc_f16(kFmt, 0u, 1u, 128, HD);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem;            // [2 tiles]
  uint8_t* sK = sQ + 2 * TB;     // [2 stages]
  uint8_t* sV = sK + 2 * TB;     // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * TB);
  uint64_t* q_full = bars;        // once per item
  uint64_t* q_empty = bars + 1;   // once per item: its last S products are done
  uint64_t* k_full = bars + 2;    // [2] per block
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_full = bars + 6;    // [2]
  uint64_t* v_empty = bars + 8;   // [2]
  uint64_t* s_full = bars + 10;   // [2] per tile and block
  uint64_t* p_ready = bars + 12;  // [2]
  uint64_t* o_full = bars + 14;   // [2]
  uint64_t* o_free = bars + 16;   // [2] per tile and item: the warpgroup has read its output rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.entries * p.q_heads;

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&k_empty[i], 1);
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&v_empty[i], 1);
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&p_ready[i], 128);
      ptx::mbar_init(&o_full[i], 1);
      ptx::mbar_init(&o_free[i], 128);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_q);
    ptx::tma_prefetch_desc(&tmap_kv);
  }
  if (warp == 8) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;        // S_t (and P_t over its first 64 columns) at + 128 t
  const uint32_t tmem_O = tmem_base + 256;  // O_t at + HD t

  if (warp == 9) {
    // ------------------------------------------------------------ load warp: Q, then K and V block by block
    // K or V block j -> one tile of 128 token rows: every lane fetches one box (a page, or 64 tokens of one)
    const int bt = p.box_tokens;
    const bool mine = lane < kPpTile / bt;
    auto box_row = [&](const PpItem& it, int j) {  // this lane's first K row of block j (V: + page_size)
      const int tok = j * kPpTile + lane * bt;
      const int slot = tok / p.page_size;
      if (!mine || slot >= it.npages) return p.oob_row;  // past the pool: the box arrives as zeros
      return p.page_indices[it.pg0 + slot] * 2 * p.page_size + (tok & (p.page_size - 1));
    };
    auto load_kv = [&](uint8_t* dst, uint64_t* bar, int kv_head, int row) {
      if (lane == 0) ptx::mbar_expect_tx(bar, TB);
      __syncwarp();
      if (mine) {
#pragma unroll
        for (int s = 0; s < C::kSlabs; ++s)
          ptx::tma_load_3d(dst + s * (TB / C::kSlabs) + lane * bt * 128, &tmap_kv, bar, s * 64, kv_head, row);
      }
    };
    auto wait = [&](uint64_t* bar, uint32_t parity) {
      int ok = 1;
      if (lane == 0) ok = ptx::bounded_mbar_wait(bar, parity, abort_flag) ? 1 : 0;
      return __shfl_sync(0xffffffffu, ok, 0) != 0;
    };
    bool ok = true;
    uint32_t g = 0, n_items = 0;  // blocks and items loaded so far
    for (int r = 0; r * static_cast<int>(gridDim.x) < total && ok; ++r) {
      const int idx = pp_index(r, total);
      if (idx < 0) continue;
      const PpItem it = pp_item(p, idx);
      if (n_items > 0) ok = wait(q_empty, (n_items - 1) & 1);  // the previous item's S products have read Q
      if (!ok) break;
      if (lane == 0) {
        ptx::mbar_expect_tx(q_full, it.nt * TB);
        for (int t = 0; t < it.nt; ++t)
#pragma unroll
          for (int s = 0; s < C::kSlabs; ++s)
            ptx::tma_load_2d(sQ + t * TB + s * (TB / C::kSlabs), &tmap_q, q_full, it.head * HD + s * 64,
                             it.seq_start + it.q0 + t * kPpTile);
      }
      int row = box_row(it, 0);
      for (int j = 0; j < it.nblk && ok; ++j, ++g) {
        const int row_next = j + 1 < it.nblk ? box_row(it, j + 1) : p.oob_row;  // looked up a block ahead of its use
        // a block's K goes where the K of two blocks ago was, once the S products of that block are done; V likewise
        if (g >= 2) ok = wait(&k_empty[g & 1], ((g - 2) >> 1) & 1);
        if (!ok) break;
        load_kv(sK + (g & 1) * TB, &k_full[g & 1], it.kv_head, row);
        if (g >= 2) ok = wait(&v_empty[g & 1], ((g - 2) >> 1) & 1);
        if (!ok) break;
        load_kv(sV + (g & 1) * TB, &v_full[g & 1], it.kv_head, row == p.oob_row ? row : row + p.page_size);
        row = row_next;
      }
      ++n_items;
    }
    if (!ok && lane == 0 && p.status) atomicCAS(p.status, 0, kStatusTimeoutProducer);
  } else if (warp == 8) {
    // ------------------------------------------------------------ MMA warp: one thread issues
    if (lane == 0) {
      auto issue_S = [&](int t, int stage) {
        const uint32_t a = ptx::smem_u32(sQ + t * TB), bb = ptx::smem_u32(sK + stage * TB);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * (TB / C::kSlabs) + (k & 3) * 32;
          ptx::umma_f16_ss(tmem_S + t * 128, ptx::make_smem_desc(a + off, 16, 1024, ptx::kLayoutSw128),
                           ptx::make_smem_desc(bb + off, 16, 1024, ptx::kLayoutSw128), kIdescS, k != 0 ? 1u : 0u);
        }
        ptx::umma_commit(&s_full[t]);
      };
      auto issue_PV = [&](int t, int stage, bool accumulate) {
        const uint32_t bb = ptx::smem_u32(sV + stage * TB);
#pragma unroll
        for (int k = 0; k < kPpTile / 16; ++k) {
          // A = P in tensor memory: row = lane, 16 tokens = 8 columns.  B = V: N-major, slabs of 64 head-dim
          // columns; 16 tokens (K) advance 2 KB.
          ptx::umma_f16_ts(tmem_O + t * HD, tmem_S + t * 128 + k * 8,
                           ptx::make_smem_desc(bb + k * 2048, TB / C::kSlabs, 1024, ptx::kLayoutSw128), kIdescPV,
                           (accumulate || k != 0) ? 1u : 0u);
        }
        ptx::umma_commit(&o_full[t]);
      };
      auto wait = [&](uint64_t* bar, uint32_t parity) { return ptx::bounded_mbar_wait(bar, parity, abort_flag); };
      // Everything this thread touches between two MMAs stays in registers (no arrays indexed by the tile number):
      // it is the one thread the tensor pipe waits for.
      bool ok = true;
      uint32_t g = 0, n_items = 0;   // blocks and items started so far
      uint32_t cnt0 = 0, cnt1 = 0;   // blocks tile t has been through
      uint32_t outs0 = 0, outs1 = 0; // items tile t has produced output for
      for (int r = 0; r * static_cast<int>(gridDim.x) < total && ok; ++r) {
        const int idx = pp_index(r, total);
        if (idx < 0) continue;
        const PpItem it = pp_item(p, idx);
        const int nb0 = it.nblk_t[0], nb1 = it.nblk_t[1], nblk = it.nblk;
        const bool tr = n_items == 0 && blockIdx.x == 0;
        ok = wait(q_full, n_items & 1) && wait(&k_full[g & 1], (g >> 1) & 1);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        // S of the first block: the tiles' score columns are free (their last P of the previous item was waited for)
        issue_S(0, g & 1);
        if (nb1 > 0) issue_S(1, g & 1);
        ptx::umma_commit(&k_empty[g & 1]);
        if (nblk == 1) ptx::umma_commit(q_empty);
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t gj = g + j;
          pp_trace(p, tr, 2, j, 0);
          bool v_here = false, k_next = false;
          // one tile's turn: wait for its P, then its P V and its next S
          auto turn = [&](const int t, const int nbt, const uint32_t cnt_t, const uint32_t outs_t) {
            if (j >= nbt || !ok) return;
            ok = wait(&p_ready[t], (cnt_t + j) & 1);  // P_t of block j is written; S_t and (after a rescale) O_t are settled
            pp_trace(p, tr, 2, j, 2 + 2 * t);
            if (ok && !v_here) {
              ok = wait(&v_full[gj & 1], (gj >> 1) & 1);
              v_here = true;
            }
            if (ok && j + 1 < nbt && !k_next) {
              ok = wait(&k_full[(gj + 1) & 1], ((gj + 1) >> 1) & 1);
              k_next = true;
            }
            // the first product of an item overwrites O_t: the warpgroup must have read the previous item's rows
            if (ok && j == 0 && outs_t > 0) ok = wait(&o_free[t], (outs_t - 1) & 1);
            if (!ok) return;
            ptx::tc_fence_after_sync();
            issue_PV(t, gj & 1, j > 0);
            if (j + 1 < nbt) issue_S(t, (gj + 1) & 1);
            pp_trace(p, tr, 2, j, 3 + 2 * t);
          };
          turn(0, nb0, cnt0, outs0);
          turn(1, nb1, cnt1, outs1);
          if (!ok) break;
          if (k_next) ptx::umma_commit(&k_empty[(gj + 1) & 1]);
          ptx::umma_commit(&v_empty[gj & 1]);
          if (j + 2 == nblk) ptx::umma_commit(q_empty);  // the S products of the last block have just been issued
        }
        cnt0 += nb0;
        cnt1 += nb1;
        outs0 += 1;
        outs1 += nb1 > 0 ? 1 : 0;
        g += nblk;
        ++n_items;
      }
      if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups (thread = query row)
    const int t = warp >> 2;
    const int r_ = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_S + t * 128 + lane_addr;
    const uint32_t tO = tmem_O + t * HD + lane_addr;
    bool ok = true;
    uint32_t cnt = 0;  // blocks this tile has been through
    bool first = true;
    for (int r = 0; r * static_cast<int>(gridDim.x) < total && ok; ++r) {
      const int idx = pp_index(r, total);
      if (idx < 0) continue;
      const PpItem it = pp_item(p, idx);
      const int my_blocks = it.nblk_t[t];
      if (my_blocks == 0) continue;  // a short last pair has no second tile
      const bool tracer = first && blockIdx.x == 0 && (warp & 3) == 0 && lane == 0;
      first = false;
      const int q_idx = it.q0 + t * kPpTile + r_;  // row within the chunk
      const int limit = it.prefix + q_idx;         // last key position this row may see
      float m_ref = 0.f, l = 0.f;
      for (int j = 0; j < my_blocks; ++j) {
        pp_trace(p, tracer, t, j, 0);
        if (!ptx::bounded_mbar_wait(&s_full[t], (cnt + j) & 1, abort_flag)) {
          ok = false;
          break;
        }
        pp_trace(p, tracer, t, j, 1);
        ptx::tc_fence_after_sync();
        uint32_t v0[32], v1[32], v2[32], v3[32];  // the row's 128 scores (fp32 bits)
        ptx::tmem_ld_32x32(tS, v0);
        ptx::tmem_ld_32x32(tS + 32, v1);
        ptx::tmem_ld_32x32(tS + 64, v2);
        ptx::tmem_ld_32x32(tS + 96, v3);
        ptx::tmem_ld_wait();
        pp_trace(p, tracer, t, j, 2);
        auto score = [&](int i) -> uint32_t& { return i < 32 ? v0[i] : i < 64 ? v1[i - 32] : i < 96 ? v2[i - 64] : v3[i - 96]; };
        const int kv0 = j * kPpTile;
        if (kv0 + kPpTile - 1 > it.prefix + it.q0 + t * kPpTile) {  // the block reaches past the tile's first row: mask
#pragma unroll
          for (int i = 0; i < kPpTile; ++i)
            if (kv0 + i > limit) score(i) = 0xff800000u;  // -inf
        }
        // eight independent chains of three-input maxima: with two softmax warps per scheduler nothing else hides a
        // serial one
        float mxs[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mxs[i] = __uint_as_float(score(i));
#pragma unroll
        for (int i = 8; i < kPpTile - 8; i += 16)
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mxs[k] = ptx::fmax3(mxs[k], __uint_as_float(score(i + 2 * k)), __uint_as_float(score(i + 2 * k + 1)));
#pragma unroll
        for (int i = kPpTile - 8; i < kPpTile; ++i) mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(score(i)));
        float mx = fmaxf(ptx::fmax3(mxs[0], mxs[1], mxs[2]), ptx::fmax3(mxs[3], mxs[4], mxs[5]));
        mx = ptx::fmax3(mx, mxs[6], mxs[7]);
        mx *= p.scale_log2;
        // (S of this block was issued after P V of the previous one, so that product is complete: O_t is stable and
        // the columns P is about to overwrite have been read)
        if (j == 0) {
          m_ref = (mx == -INFINITY) ? 0.f : mx;
        } else {
          const bool grow = mx > m_ref + kPpRescaleAt;
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = grow ? ptx::ex2_approx(m_ref - mx) : 1.f;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
              uint32_t o[32];
              ptx::tmem_ld_32x32(tO + c, o);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              ptx::tmem_st_32x32(tO + c, o);
            }
            ptx::tmem_st_wait();
            l *= alpha;
            if (grow) m_ref = mx;
          }
        }
        pp_trace(p, tracer, t, j, 3);
        // probabilities (16 bit) -> tensor memory over the scores; row sum
        float rs[4] = {0.f, 0.f, 0.f, 0.f};
        const float neg_m = -m_ref;
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // 64 scores -> 32 columns of pairs
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c = h * 64 + 2 * i;
            const float x0 = fmaf(__uint_as_float(score(c)), p.scale_log2, neg_m);
            const float x1 = fmaf(__uint_as_float(score(c + 1)), p.scale_log2, neg_m);
            const float e0 = ptx::ex2_approx(x0);
            const float e1 = (POLY && (i & 1)) ? ptx::ex2_poly(x1) : ptx::ex2_approx(x1);
            rs[i & 3] += e0 + e1;
            pk[i] = pk2<T>(e0, e1);
          }
          ptx::tmem_st_32x32(tS + h * 32, pk);
        }
        pp_trace(p, tracer, t, j, 4);
        ptx::tmem_st_wait();
        l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(&p_ready[t]);
        pp_trace(p, tracer, t, j, 5);
      }
      if (ok) ok = ptx::bounded_mbar_wait(&o_full[t], (cnt + my_blocks - 1) & 1, abort_flag);
      if (!ok) break;
      cnt += my_blocks;
      ptx::tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(it.seq_start + q_idx) * p.out_stride + it.head * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t o[32];
        ptx::tmem_ld_32x32(tO + c, o);
        ptx::tmem_ld_wait();
        if (c + 32 >= HD) {  // all of this item's output rows are in registers: the next item may overwrite them
          ptx::tc_fence_before_sync();
          ptx::mbar_arrive(&o_free[t]);
        }
        if (q_idx < it.q_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            *reinterpret_cast<uint4*>(dst + c + i) = make_uint4(
                pk2<T>(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv),
                pk2<T>(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv),
                pk2<T>(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv),
                pk2<T>(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv));
          }
        }
      }
    }
    if (!ok && p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int HD, bool POLY>
static int launch_paged_prefill(const CUtensorMap& tq, const CUtensorMap& tkv, const PagedPrefillParams& p, int grid,
                                cudaStream_t stream) {
  static PerDeviceOnce once;
  cudaError_t e = once.run([] {
    return cudaFuncSetAttribute(attn_prefill_paged_kernel<T, HD, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                PpCfg<HD>::kSmemBytes);
  });
  if (e != cudaSuccess) return (int)e;
  attn_prefill_paged_kernel<T, HD, POLY><<<grid, kPpThreads, PpCfg<HD>::kSmemBytes, stream>>>(tq, tkv, p);
  return (int)cudaGetLastError();
}

static long long* g_pp_trace = nullptr;

}  // namespace blitz

extern "C" {
using namespace blitz;

// Profiling aid: while `buf` (3 roles x 32 iterations x 8 int64 clock stamps, device memory) is set, CTA 0 of every
// following launch records when its warpgroups and its MMA thread pass each phase of its first work item.
void blitz_attn_prefill_paged_set_trace(long long* buf) { blitz::g_pp_trace = buf; }

// qkv: [num_tokens, (q_heads + 2 kv_heads) * head_dim] of the current chunk, rotated in place; kv_layer: the
// layer's pool [max_pages][2][page_size][kv_heads][head_dim], which already holds the chunk's keys and values;
// out: [num_tokens, q_heads * head_dim].  page_indices: device array of the sequences' page ids, back to back (the
// lists cover prefix + chunk).  work: device array (16-byte aligned) of `entries` records of 8 int32, one per
// (sequence, 256 rows of it), heaviest first: first row of the sequence in qkv, rows of the sequence in this chunk,
// index of its first page id, number of its pages, tokens cached for it (chunk included), which 256-row pair, 0, 0.
// page_size: a power of two >= 8.  flags bit 0: compute a quarter of the exponentials on the FMA pipe.
int blitz_attn_prefill_paged(const void* qkv, const void* kv_layer, void* out, int64_t out_stride,
                             const int32_t* page_indices, const int32_t* work, int entries, int num_tokens,
                             int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, float sm_scale,
                             int flags, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || entries <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || (q_heads % kv_heads) != 0 || (out_stride & 7)) return -1;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0 || work == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(work) & 15) != 0) return -1;
  const uint64_t row = (uint64_t)(q_heads + 2 * kv_heads) * head_dim;
  const int bt = page_size < 64 ? page_size : 64;
  CUtensorMap tq, tkv;
  if (!get_tmap_2d(&tq, qkv, row, (uint64_t)num_tokens, row * 2, 64, kPpTile)) return -2;
  if (!get_tmap_3d(&tkv, kv_layer, (uint64_t)head_dim, (uint64_t)kv_heads, (uint64_t)max_pages * 2 * page_size,
                   (uint64_t)head_dim * 2, (uint64_t)kv_heads * head_dim * 2, 64, 1, (uint32_t)bt))
    return -2;
  PagedPrefillParams p;
  p.out = out; p.out_stride = out_stride; p.page_indices = page_indices; p.work = work; p.entries = entries;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.page_size = page_size; p.box_tokens = bt;
  p.oob_row = max_pages * 2 * page_size;
  p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status; p.trace = g_pp_trace;
  const long long total = (long long)entries * q_heads;
  const int sms = device_sm_count();
  const int grid = (int)(total < sms ? total : sms);
  const bool poly = (flags & 1) != 0;
  if (dtype == 1) {
    if (head_dim == 128)
      return poly ? launch_paged_prefill<__nv_bfloat16, 128, true>(tq, tkv, p, grid, stream)
                  : launch_paged_prefill<__nv_bfloat16, 128, false>(tq, tkv, p, grid, stream);
    return poly ? launch_paged_prefill<__nv_bfloat16, 64, true>(tq, tkv, p, grid, stream)
                : launch_paged_prefill<__nv_bfloat16, 64, false>(tq, tkv, p, grid, stream);
  }
  if (head_dim == 128)
    return poly ? launch_paged_prefill<__half, 128, true>(tq, tkv, p, grid, stream)
                : launch_paged_prefill<__half, 128, false>(tq, tkv, p, grid, stream);
  return poly ? launch_paged_prefill<__half, 64, true>(tq, tkv, p, grid, stream)
              : launch_paged_prefill<__half, 64, false>(tq, tkv, p, grid, stream);
}

}  // extern "C"
