// Causal prefill attention over the paged KV cache on tcgen05 for sm_100a: GQA, head_dim 64 or 128, queries of
// the current chunk against everything the cache holds for the sequence (earlier chunks and the chunk itself).
//
// Q comes from the fused QKV activation of the chunk (2-D TMA boxes); K and V come from the paged pool, where
// rope_kv_store has already put the chunk's own keys and values, as 3-D TMA boxes of one page (or 64 tokens of
// one) each, looked up through the page table.  A prompt that does not fit one batch is therefore prefetched in
// chunks with no other kernel: the first chunk has an empty prefix, later ones a prefix of whole earlier chunks.
//
// One CTA owns 256 query rows of one sequence and one q head, as two tiles of 128 rows, and walks the KV blocks
// of 128 tokens up to the diagonal once for both tiles:
//
//   S_t = Q_t K^T      tcgen05.mma, A = Q_t (smem), B = K block (smem), S_t in TMEM                      t = 0, 1
//   P_t = softmax      warpgroup t (4 warps, thread = row): one tcgen05.ld pass over S_t, running max and sum in
//                      fp32, P_t -> smem (16 bit, 128-byte swizzle)
//   O_t += P_t V       tcgen05.mma accumulating in TMEM over all blocks
//
// A ninth warp issues the MMAs (one thread), a tenth the TMA loads.
// While warpgroup 0 turns S_0 into P_0 the tensor core works on S_1 and on O_1, and the other way round: the
// two tiles ping-pong, and every K and V block feeds two tiles from one load.  O stays in TMEM for the whole
// walk: the running maximum a row's probabilities refer to only moves when the true maximum has grown by more
// than 2^8 (the probabilities then stay below 256, harmless in 16 bits and fp32), and only then the warp
// rescales its O rows in place (tcgen05.ld, multiply, tcgen05.st); with ordinary inputs that happens in the
// first block or two of a row and never again.  Part of the exponentials is computed on the FMA pipe by a
// cubic (ex2_poly): one exponential per score is what bounds the softmax of a 128-wide tile on the
// special-function unit, not the tensor core.
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
constexpr int kPpPBytes = kPpTile * kPpTile * 2;
constexpr float kPpRescaleAt = 8.f;  // log2 units

struct PagedPrefillParams {
  void* out;  // [tokens, q_heads * HD]
  int64_t out_stride;
  const int32_t* tok_indptr;     // [batch + 1] offsets of the chunk's rows in the activation
  const int32_t* page_indices;   // page ids of every sequence, back to back
  const int32_t* page_indptr;    // [batch + 1]
  const int32_t* last_page_len;  // [batch] tokens in the last page, the chunk included
  const int32_t* work;           // [gridDim.y] (sequence << 12 | pair of tiles), heaviest first; null: in order
  int batch, q_heads, kv_heads, page_size, box_tokens, oob_row;
  float scale_log2;
  int* status;
  long long* trace;  // profiling aid (null in production): clock stamps of CTA (0, 0), see blitz_attn_prefill_paged_set_trace
};

constexpr int kPpTraceIters = 32, kPpTraceSlots = 8;
// role 0 / 1: first lane of warpgroup 0 / 1; role 2: the control warp's first lane
__device__ __forceinline__ void pp_trace(const PagedPrefillParams& p, int role, int j, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && j < kPpTraceIters)
    p.trace[(role * kPpTraceIters + j) * kPpTraceSlots + slot] = clock64();
}

// PTMEM: the probabilities stay in tensor memory (written over the first 64 columns of the scores they came from,
// two 16-bit values per column) and the P V product takes its A operand from there; the 64 KB of shared memory the
// two P tiles would need go to a second V stage.  Without it (head_dim 128) V is single-buffered and every block
// waits for its V behind the previous block's products.
template <int HD, bool PTMEM>
struct PpCfg {
  static constexpr int kTileBytes = kPpTile * HD * 2;        // one Q, K or V tile
  static constexpr int kSlabs = HD / 64;                     // 64-column slabs of 128 rows x 128 bytes
  static constexpr int kVStages = (HD == 128 && !PTMEM) ? 1 : 2;
  static constexpr int kPBytes = PTMEM ? 0 : 2 * kPpPBytes;
  static constexpr int kSmemBytes = 2 * kTileBytes + kPBytes + 2 * kTileBytes + kVStages * kTileBytes + 1024 + 256;
};

template <typename T, int HD, bool POLY, bool PTMEM>
__global__ void __launch_bounds__(kPpThreads, 1)
attn_prefill_paged_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                          const PagedPrefillParams p) {
  using C = PpCfg<HD, PTMEM>;
  constexpr int TB = C::kTileBytes;
  constexpr int NV = C::kVStages;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdescS = ptx::make_idesc_f16(kFmt, 0u, 0u, 128, 128);
  constexpr uint32_t kIdescPV = ptx::make_idesc_f16(kFmt, 0u, 1u, 128, HD);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem;                      // [2 tiles]
  uint8_t* sP = sQ + 2 * TB;               // [2 tiles]
  uint8_t* sK = sP + C::kPBytes;           // [2 stages]
  uint8_t* sV = sK + 2 * TB;               // [NV stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NV * TB);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* v_full = bars + 5;      // [2]
  uint64_t* v_empty = bars + 7;     // [2]
  uint64_t* s_full = bars + 9;      // [2] per tile
  uint64_t* p_ready = bars + 11;    // [2] per tile
  uint64_t* o_full = bars + 13;     // [2] per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- this CTA's (sequence, pair of q tiles)
  int b = -1, pair = 0;
  if (p.work != nullptr) {
    const int w = p.work[blockIdx.y];
    b = w >> 12;
    pair = w & 4095;
  } else {
    int idx = blockIdx.y;
    for (int i = 0; i < p.batch; ++i) {
      const int np = (p.tok_indptr[i + 1] - p.tok_indptr[i] + 2 * kPpTile - 1) / (2 * kPpTile);
      if (idx < np) {
        b = i;
        pair = idx;
        break;
      }
      idx -= np;
    }
  }
  if (b < 0 || b >= p.batch) return;  // uniform across the CTA
  const int seq_start = p.tok_indptr[b];
  const int q_len = p.tok_indptr[b + 1] - seq_start;
  const int pg0 = p.page_indptr[b];
  const int npages = p.page_indptr[b + 1] - pg0;
  const int kv_len = npages > 0 ? (npages - 1) * p.page_size + p.last_page_len[b] : 0;
  const int prefix = kv_len - q_len;  // tokens of earlier chunks
  const int q0 = pair * 2 * kPpTile;
  if (q0 >= q_len || prefix < 0) return;
  const int nt = (q0 + kPpTile < q_len) ? 2 : 1;
  // blocks tile t needs: keys up to its last row's position
  int nblk_t[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int last = min(kv_len, prefix + min(q_len, q0 + kPpTile * (t + 1)));
    nblk_t[t] = t < nt ? (last + kPpTile - 1) / kPpTile : 0;
  }
  const int nblk = max(nblk_t[0], nblk_t[1]);
  const int head = blockIdx.x;
  const int kv_head = head / (p.q_heads / p.kv_heads);

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&k_empty[i], 1);
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&v_empty[i], 1);
      ptx::mbar_init(&s_full[i], 1);
      ptx::mbar_init(&p_ready[i], 128);
      ptx::mbar_init(&o_full[i], 1);
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
  const uint32_t tmem_S = tmem_base;         // S_t at + 128 t
  const uint32_t tmem_O = tmem_base + 256;   // O_t at + HD t

  if (warp == 9) {
    // ------------------------------------------------------------ load warp: Q, then K and V block by block
    // K or V block j -> one tile of 128 token rows: every lane fetches one box (a page, or 64 tokens of one)
    const int bt = p.box_tokens;
    const bool mine = lane < kPpTile / bt;
    auto box_row = [&](int j) {  // this lane's first K row of block j (V: + page_size); past the pool = zeros
      const int tok = j * kPpTile + lane * bt;
      const int slot = tok / p.page_size;
      if (!mine || slot >= npages) return p.oob_row;
      return p.page_indices[pg0 + slot] * 2 * p.page_size + (tok & (p.page_size - 1));
    };
    auto load_kv = [&](uint8_t* dst, uint64_t* bar, int row) {
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
    if (lane == 0) {
      ptx::mbar_expect_tx(q_full, nt * TB);
      for (int t = 0; t < nt; ++t)
#pragma unroll
        for (int s = 0; s < C::kSlabs; ++s)
          ptx::tma_load_2d(sQ + t * TB + s * (TB / C::kSlabs), &tmap_q, q_full, head * HD + s * 64,
                           seq_start + q0 + t * kPpTile);
    }
    bool ok = true;
    int row = box_row(0);
    for (int j = 0; j < nblk && ok; ++j) {
      const int row_next = j + 1 < nblk ? box_row(j + 1) : p.oob_row;  // looked up a block ahead of its use
      // K of block j goes where block j - 2's was, once the S products of that block are done; V likewise
      if (j >= 2) ok = wait(&k_empty[j & 1], ((j - 2) >> 1) & 1);
      if (!ok) break;
      load_kv(sK + (j & 1) * TB, &k_full[j & 1], row);
      if (j >= NV) ok = wait(&v_empty[j % NV], ((j - NV) / NV) & 1);
      if (!ok) break;
      load_kv(sV + (j % NV) * TB, &v_full[j % NV], row == p.oob_row ? row : row + p.page_size);
      row = row_next;
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
        const uint32_t a = ptx::smem_u32(sP + t * kPpPBytes), bb = ptx::smem_u32(sV + stage * TB);
#pragma unroll
        for (int k = 0; k < kPpTile / 16; ++k) {
          // B = V: N-major, slabs of 64 head-dim columns; 16 tokens (K) advance 2 KB.
          const uint64_t bdesc = ptx::make_smem_desc(bb + k * 2048, TB / C::kSlabs, 1024, ptx::kLayoutSw128);
          if (PTMEM) {
            // A = P in tensor memory: row = lane, 16 tokens = 8 columns
            ptx::umma_f16_ts(tmem_O + t * HD, tmem_S + t * 128 + k * 8, bdesc, kIdescPV,
                             (accumulate || k != 0) ? 1u : 0u);
          } else {
            // A = P in shared memory: K-major, two slabs of 64 tokens
            const uint32_t aoff = (k >> 2) * (kPpPBytes / 2) + (k & 3) * 32;
            ptx::umma_f16_ss(tmem_O + t * HD, ptx::make_smem_desc(a + aoff, 16, 1024, ptx::kLayoutSw128), bdesc,
                             kIdescPV, (accumulate || k != 0) ? 1u : 0u);
          }
        }
        ptx::umma_commit(&o_full[t]);
      };
      auto wait = [&](uint64_t* bar, uint32_t parity) { return ptx::bounded_mbar_wait(bar, parity, abort_flag); };
      bool ok = wait(q_full, 0) && wait(&k_full[0], 0);
      if (ok) {
        ptx::tc_fence_after_sync();
        for (int t = 0; t < nt; ++t)
          if (nblk_t[t] > 0) issue_S(t, 0);
        ptx::umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int vs = j % NV;
        pp_trace(p, 2, j, 0);
        bool v_here = false, k_next = false;
        for (int t = 0; t < nt && ok; ++t) {
          if (j >= nblk_t[t]) continue;
          ok = wait(&p_ready[t], j & 1);  // P_t of block j is written; S_t and (after a rescale) O_t are settled
          pp_trace(p, 2, j, 2 + 2 * t);
          if (ok && !v_here) {
            ok = wait(&v_full[vs], (j / NV) & 1);
            v_here = true;
          }
          if (!ok) break;
          if (j + 1 < nblk_t[t] && !k_next) {
            ok = wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
            k_next = true;
            if (!ok) break;
          }
          ptx::tc_fence_after_sync();
          issue_PV(t, vs, j > 0);
          if (j + 1 < nblk_t[t]) issue_S(t, (j + 1) & 1);
          pp_trace(p, 2, j, 3 + 2 * t);
        }
        if (!ok) break;
        if (k_next) ptx::umma_commit(&k_empty[(j + 1) & 1]);
        ptx::umma_commit(&v_empty[vs]);
      }
      if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups (thread = query row)
    const int t = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int q_idx = q0 + t * kPpTile + r;    // row within the chunk
    const int limit = prefix + q_idx;          // last key position this row may see
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_S + t * 128 + lane_addr;
    const uint32_t tO = tmem_O + t * HD + lane_addr;
    uint8_t* sPt = sP + t * kPpPBytes;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    const int my_blocks = nblk_t[t];
    const bool tracer = (warp & 3) == 0 && lane == 0;
    for (int j = 0; j < my_blocks; ++j) {
      if (tracer) pp_trace(p, t, j, 0);
      if (!ptx::bounded_mbar_wait(&s_full[t], j & 1, abort_flag)) {
        ok = false;
        break;
      }
      if (tracer) pp_trace(p, t, j, 1);
      ptx::tc_fence_after_sync();
      uint32_t v0[32], v1[32], v2[32], v3[32];  // the row's 128 scores (fp32 bits)
      ptx::tmem_ld_32x32(tS, v0);
      ptx::tmem_ld_32x32(tS + 32, v1);
      ptx::tmem_ld_32x32(tS + 64, v2);
      ptx::tmem_ld_32x32(tS + 96, v3);
      ptx::tmem_ld_wait();
      if (tracer) pp_trace(p, t, j, 2);
      auto score = [&](int i) -> uint32_t& { return i < 32 ? v0[i] : i < 64 ? v1[i - 32] : i < 96 ? v2[i - 64] : v3[i - 96]; };
      const int kv0 = j * kPpTile;
      if (kv0 + kPpTile - 1 > prefix + q0 + t * kPpTile) {  // the block reaches past the tile's first row: mask
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
      // the previous block's P V must have been read out of P's buffer (and into O) before either is touched
      if (j > 0 && !ptx::bounded_mbar_wait(&o_full[t], (j - 1) & 1, abort_flag)) {
        ok = false;
        break;
      }
      if (j == 0) {
        m_ref = (mx == -INFINITY) ? 0.f : mx;
      } else {
        const bool grow = mx > m_ref + kPpRescaleAt;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? ptx::ex2_approx(m_ref - mx) : 1.f;
          ptx::tc_fence_after_sync();
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
      if (tracer) pp_trace(p, t, j, 3);
      // probabilities (16 bit) -> tensor memory over the scores, or shared memory in 128-byte swizzled rows; row sum
      float rs[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_m = -m_ref;
      if (PTMEM) {
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
        if (tracer) pp_trace(p, t, j, 4);
        ptx::tmem_st_wait();
      } else {
#pragma unroll
        for (int c = 0; c < kPpTile; c += 8) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x = fmaf(__uint_as_float(score(c + i)), p.scale_log2, neg_m);
            e[i] = (POLY && (i & 3) == 3) ? ptx::ex2_poly(x) : ptx::ex2_approx(x);
            rs[i & 3] += e[i];
          }
          const int chunk = c >> 3;  // 16-byte chunk along the token axis: 0..15
          const uint32_t off = (chunk >> 3) * (kPpPBytes / 2) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(sPt + off) =
              make_uint4(pk2<T>(e[0], e[1]), pk2<T>(e[2], e[3]), pk2<T>(e[4], e[5]), pk2<T>(e[6], e[7]));
        }
        ptx::fence_proxy_async_smem();
      }
      l += (rs[0] + rs[1]) + (rs[2] + rs[3]);
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&p_ready[t]);
      if (tracer) pp_trace(p, t, j, 5);
    }
    if (ok && my_blocks > 0) ok = ptx::bounded_mbar_wait(&o_full[t], (my_blocks - 1) & 1, abort_flag);
    if (!ok) {
      if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
    } else if (my_blocks > 0) {
      ptx::tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(seq_start + q_idx) * p.out_stride + head * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t o[32];
        ptx::tmem_ld_32x32(tO + c, o);
        ptx::tmem_ld_wait();
        if (q_idx < q_len) {
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
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

template <typename T, int HD, bool POLY, bool PTMEM>
static int launch_paged_prefill(const CUtensorMap& tq, const CUtensorMap& tkv, const PagedPrefillParams& p, dim3 grid,
                                cudaStream_t stream) {
  static PerDeviceOnce once;
  cudaError_t e = once.run([] {
    return cudaFuncSetAttribute(attn_prefill_paged_kernel<T, HD, POLY, PTMEM>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, PpCfg<HD, PTMEM>::kSmemBytes);
  });
  if (e != cudaSuccess) return (int)e;
  attn_prefill_paged_kernel<T, HD, POLY, PTMEM>
      <<<grid, kPpThreads, PpCfg<HD, PTMEM>::kSmemBytes, stream>>>(tq, tkv, p);
  return (int)cudaGetLastError();
}

}  // namespace blitz

namespace blitz {
static long long* g_pp_trace = nullptr;
}

extern "C" {
using namespace blitz;

// Profiling aid: while `buf` (3 roles x 32 iterations x 8 int64 clock stamps, device memory) is set, the CTA at grid
// position (0, 0) of every following launch records when its warpgroups and its control warp pass each phase.
void blitz_attn_prefill_paged_set_trace(long long* buf) { blitz::g_pp_trace = buf; }

// qkv: [num_tokens, (q_heads + 2 kv_heads) * head_dim] of the current chunk, rotated in place; kv_layer: the
// layer's pool [max_pages][2][page_size][kv_heads][head_dim], which already holds the chunk's keys and values;
// out: [num_tokens, q_heads * head_dim].  tok_indptr / page_indices / page_indptr / last_page_len: device arrays as
// for the decode kernel (the page table covers prefix + chunk).  total_pairs = sum over sequences of
// ceil(chunk rows / 256); work: optional device list of total_pairs entries (sequence << 12 | pair), heaviest first.
// page_size: a power of two >= 8.  flags bit 0: compute a quarter of the exponentials on the FMA pipe; bit 1: keep
// the probabilities in tensor memory (see PpCfg).
int blitz_attn_prefill_paged(const void* qkv, const void* kv_layer, void* out, int64_t out_stride,
                             const int32_t* tok_indptr, const int32_t* page_indices, const int32_t* page_indptr,
                             const int32_t* last_page_len, const int32_t* work, int batch, int num_tokens,
                             int total_pairs, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages,
                             float sm_scale, int flags, int* status, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || total_pairs <= 0) return 0;
  if ((head_dim != 64 && head_dim != 128) || (q_heads % kv_heads) != 0 || (out_stride & 7)) return -1;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0 || batch >= (1 << 19)) return -1;
  const uint64_t row = (uint64_t)(q_heads + 2 * kv_heads) * head_dim;
  const int bt = page_size < 64 ? page_size : 64;
  CUtensorMap tq, tkv;
  if (!get_tmap_2d(&tq, qkv, row, (uint64_t)num_tokens, row * 2, 64, kPpTile)) return -2;
  if (!get_tmap_3d(&tkv, kv_layer, (uint64_t)head_dim, (uint64_t)kv_heads, (uint64_t)max_pages * 2 * page_size,
                   (uint64_t)head_dim * 2, (uint64_t)kv_heads * head_dim * 2, 64, 1, (uint32_t)bt))
    return -2;
  PagedPrefillParams p;
  p.out = out; p.out_stride = out_stride; p.tok_indptr = tok_indptr; p.page_indices = page_indices;
  p.page_indptr = page_indptr; p.last_page_len = last_page_len; p.work = work; p.batch = batch;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.page_size = page_size; p.box_tokens = bt;
  p.oob_row = max_pages * 2 * page_size;
  p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status; p.trace = g_pp_trace;
  dim3 grid(q_heads, total_pairs);
  const bool poly = (flags & 1) != 0, ptmem = (flags & 2) != 0;
#define BLITZ_PP_LAUNCH(T, HD)                                                                            \
  (ptmem ? (poly ? launch_paged_prefill<T, HD, true, true>(tq, tkv, p, grid, stream)                      \
                 : launch_paged_prefill<T, HD, false, true>(tq, tkv, p, grid, stream))                    \
         : (poly ? launch_paged_prefill<T, HD, true, false>(tq, tkv, p, grid, stream)                     \
                 : launch_paged_prefill<T, HD, false, false>(tq, tkv, p, grid, stream)))
  if (dtype == 1) return head_dim == 128 ? BLITZ_PP_LAUNCH(__nv_bfloat16, 128) : BLITZ_PP_LAUNCH(__nv_bfloat16, 64);
  return head_dim == 128 ? BLITZ_PP_LAUNCH(__half, 128) : BLITZ_PP_LAUNCH(__half, 64);
#undef BLITZ_PP_LAUNCH
}

}  // extern "C"
