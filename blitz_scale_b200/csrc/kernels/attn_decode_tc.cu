// Paged-KV decode attention, tensor-core version (the serving path).
//
// Decode attention is a stream over the K and V pages of every sequence; with
// GQA the 4-8 query heads that share a KV head turn the per-token work into a
// small matrix product, so the FLOPs go to mma.sync (m16n8k16, query heads
// padded to 16 rows) and the instruction stream per token drops ~10x against a
// CUDA-core dot product; the kernel is then bound by HBM as it should be.
// tcgen05 is not used here on purpose: its minimum M of 64 rows would waste
// 94 % of each instruction on padding for one query token per sequence.
//
// Data movement: a producer warp walks the page table and issues TMA
// (cp.async.bulk.tensor.3d, plain per-CTA loads) boxes of [tokens x 64 dims]
// straight from the paged layout [page][K|V][token][kv_head][head_dim] into
// 128-byte-swizzled shared memory, 4 stages of 64 tokens (128 KB in flight
// per SM for head_dim 128).  Four consumer warps each own 16 of the 64 tokens
// of a stage: S = Q K^T via ldmatrix + mma, online softmax in registers
// (exp2, fp32), O += P V via ldmatrix.trans + mma.  Warps merge their partial
// (m, l, O) through shared memory; with num_splits > 1 each item writes an fp32
// partial and a merge kernel combines the splits (flash-decoding).
//
// The kernel is persistent: one CTA per SM walks the work items (sequence,
// KV head, split) in a grid-stride loop and the TMA pipeline runs across item
// boundaries, so it never drains between sequences (5.6 TB/s at batch 256,
// context 1024).  It is launched with programmatic dependent launch: shared
// memory is cleared and the barriers are set up while the previous kernel is
// still running; the first load waits for it.
//
// The cache must hold finite values in every slot of an allocated page (the
// pool is zero-filled at creation): masked positions get probability 0, and
// 0 x NaN would still poison the accumulator.
//
// Replaces src/kernel/attention_decode.cu:13-40 and the host-side plan of
// src/kernel/flashinfer_types.cu:52-80.
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include "common.cuh"

namespace blitz {

constexpr int kTcThreads = 160;
constexpr int kTcChunk = 64;
constexpr int kTcStages = 6;
constexpr int kTcSlabBytes = kTcChunk * 128;

struct DecodeTcParams {
  const void* q;
  int64_t q_stride;
  const int32_t* indices;
  const int32_t* indptr;
  const int32_t* last_page_len;
  void* out;
  int64_t out_stride;
  float* part_o;
  float* part_lse;
  int batch, q_heads, kv_heads, group, page_size, max_pages, num_splits, box_tokens;
  int tail_box_tokens;  // box height of the second tensor map, used for the last (partly filled) chunk of a sequence
  float scale_log2;
  int* status;
  long long* trace;  // profiling aid (null in production): clock stamps of CTA 0's first items, see blitz_attn_decode_set_trace
};

constexpr int kTcTraceItems = 16, kTcTraceSlots = 8;
__device__ __forceinline__ void tc_trace(const DecodeTcParams& p, int n, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && n < kTcTraceItems) p.trace[n * kTcTraceSlots + slot] = clock64();
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int HD>
struct TcCfg {
  static constexpr int kSlabs = HD / 64;
  static constexpr int kStageBytes = 2 * kSlabs * kTcSlabBytes;
  static constexpr int kMergeFloats = 4 * 8 * HD + 2 * 4 * 8;
  static constexpr int kSmemBytes = kTcStages * kStageBytes + kMergeFloats * 4 + 1024 + 128;
};

// Work item = (sequence, kv head, split).  The kernel is persistent: each CTA walks items
// blockIdx.x, blockIdx.x + gridDim.x, ... and the producer keeps streaming the next item's pages while
// the consumers finish the current one, so the 4-stage pipeline never drains between items.
struct DecItem {
  int b, h, split, pg_beg, seq_len, c_beg, c_end;
};
__device__ __forceinline__ DecItem dec_item(const DecodeTcParams& p, int item) {
  DecItem it;
  it.split = item % p.num_splits;
  it.h = (item / p.num_splits) % p.kv_heads;
  it.b = item / (p.num_splits * p.kv_heads);
  it.pg_beg = p.indptr[it.b];
  const int npages = p.indptr[it.b + 1] - it.pg_beg;
  it.seq_len = npages > 0 ? (npages - 1) * p.page_size + p.last_page_len[it.b] : 0;
  const int nchunks = (it.seq_len + kTcChunk - 1) / kTcChunk;
  const int cps = (nchunks + p.num_splits - 1) / p.num_splits;
  it.c_beg = min(nchunks, it.split * cps);
  it.c_end = min(nchunks, (it.split + 1) * cps);
  return it;
}

template <typename T, int HD>
__global__ void __launch_bounds__(kTcThreads)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_tail,
                      const DecodeTcParams p) {
  using Cfg = TcCfg<HD>;
  constexpr int SL = Cfg::kSlabs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  float* mrg_o = reinterpret_cast<float*>(smem + kTcStages * Cfg::kStageBytes);  // [4][8][HD]
  float* mrg_m = mrg_o + 4 * 8 * HD;                                              // [4][8]
  float* mrg_l = mrg_m + 32;                                                      // [4][8]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(mrg_l + 32);
  uint64_t* empty_bar = full_bar + kTcStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kTcStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  const int num_items = p.batch * p.kv_heads * p.num_splits;

  // zero the stages once: rows a short last chunk never fills must stay finite
  for (int i = threadIdx.x; i < kTcStages * Cfg::kStageBytes / 16; i += kTcThreads)
    reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < kTcStages; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap);
    ptx::tma_prefetch_desc(&tmap_tail);
  }
  ptx::fence_proxy_async_smem();
  __syncthreads();
  // programmatic dependent launch: the set-up above may overlap the previous kernel; q and the KV pages
  // are its outputs, so wait before the first load
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();

  if (warp == 4) {
    // ------------------------------------------------------------ producer (whole warp; lane 0 issues)
    // A TMA box can only be issued once its page id is known, and a page id read from global memory right before
    // the issue costs one memory latency per chunk, which by itself caps the stream near 50 GB/s per SM.  So the
    // warp reads page ids 32 at a time (one coalesced load, lane l keeps entry l of the window), hands them out by
    // shuffle, and requests the next item's page-table window and lengths while the current item streams.
    const int ps = p.page_size;
    auto load_window = [&](const DecItem& it, int first_page) -> int {
      const int npages = p.indptr[it.b + 1] - it.pg_beg;
      return (first_page + lane < npages) ? p.indices[it.pg_beg + first_page + lane] : 0;
    };
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int item = blockIdx.x;
    DecItem it = item < num_items ? dec_item(p, item) : DecItem{};
    int win_base = item < num_items ? (it.c_beg * kTcChunk) / ps : 0;
    int win = item < num_items ? load_window(it, win_base) : 0;
    int n_done = 0;
    while (item < num_items && ok) {
      if (lane == 0) tc_trace(p, n_done, 4);
      // next item's metadata and first window: in flight while this item streams
      const int next = item + gridDim.x;
      DecItem nit = next < num_items ? dec_item(p, next) : DecItem{};
      const int nwin_base = next < num_items ? (nit.c_beg * kTcChunk) / ps : 0;
      const int nwin = next < num_items ? load_window(nit, nwin_base) : 0;
      for (int c = it.c_beg; c < it.c_end && ok; ++c) {
        const int tok0 = c * kTcChunk;
        const int ntok = min(kTcChunk, it.seq_len - tok0);
        // a full chunk comes in boxes of box_tokens rows; the last chunk of a sequence only as far as it is
        // filled, in the smaller boxes of the second map (a 64-token page with 18 live tokens costs 32 rows)
        const bool tail = ntok < kTcChunk;
        const int bt = tail ? p.tail_box_tokens : p.box_tokens;
        const CUtensorMap* tm = tail ? &tmap_tail : &tmap;
        const uint32_t box_bytes = static_cast<uint32_t>(bt) * 128u;
        const int pieces = (ntok + bt - 1) / bt;
        const int last_page = (tok0 + ntok - 1) / ps;
        if (last_page >= win_base + 32) {  // sequences of more than 32 pages: move the window
          win_base = tok0 / ps;
          win = load_window(it, win_base);
        }
        int good = 1;
        if (lane == 0) {
          if (!ptx::bounded_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutProducer);
            good = 0;
          } else {
            ptx::mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(pieces) * 2u * SL * box_bytes);
          }
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + stage * Cfg::kStageBytes;
        for (int i = 0; i < pieces; ++i) {
          const int t = tok0 + i * bt;
          int page = __shfl_sync(0xffffffffu, win, (t / ps - win_base) & 31);
          if (lane == 0) {
            if (page < 0 || page >= p.max_pages) {
              if (p.status) atomicCAS(p.status, 0, kStatusBadIndex);
              page = 0;
            }
            const int z = page * 2 * ps + (t % ps);
#pragma unroll
            for (int s = 0; s < SL; ++s) {
              ptx::tma_load_3d(sb + s * kTcSlabBytes + i * box_bytes, tm, &full_bar[stage], s * 64, it.h, z);
              ptx::tma_load_3d(sb + (SL + s) * kTcSlabBytes + i * box_bytes, tm, &full_bar[stage], s * 64, it.h, z + ps);
            }
          }
        }
        if (++stage == kTcStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (lane == 0) tc_trace(p, n_done, 5);
      ++n_done;
      item = next;
      it = nit;
      win_base = nwin_base;
      win = nwin;
    }
  } else {
    // ------------------------------------------------------------ consumers (128 threads, named barrier 1)
    const int g = lane >> 2, t4 = lane & 3;
    const int tokw = warp * 16;
    const int mi = lane >> 3, mr = lane & 7;  // ldmatrix: matrix index and row within it
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;  // after a timeout this warp stops waiting but keeps meeting the others at the barriers
    // The consumers stop consuming between two items (merge, then the next item's lengths and query rows), and a
    // pause longer than the pipeline can absorb empties the memory pipe, which then costs a full latency to refill.
    // So the next item's descriptor and Q fragments are requested while the current item is being processed.
    auto load_q = [&](const DecItem& d, uint32_t (&a0)[HD / 16], uint32_t (&a2)[HD / 16]) {
      // Q as A fragments (rows >= G are zero padding; rows 8..15 are never populated since G <= 8)
      const T* qrow = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(d.b) * p.q_stride +
                      static_cast<int64_t>(d.h * G + g) * HD;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        a0[ks] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4) : 0u;
        a2[ks] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4 + 8) : 0u;
      }
    };
    DecItem it = blockIdx.x < num_items ? dec_item(p, blockIdx.x) : DecItem{};
    uint32_t qa0[HD / 16], qa2[HD / 16];
    if (blockIdx.x < num_items) load_q(it, qa0, qa2);
    int n_done = 0;
    const bool tracer = warp == 0 && lane == 0;
    for (int item = blockIdx.x; item < num_items; item += gridDim.x, ++n_done) {
      if (tracer) tc_trace(p, n_done, 0);
      const int next = item + gridDim.x;
      DecItem nit = DecItem{};
      uint32_t nqa0[HD / 16], nqa2[HD / 16];
      if (next < num_items) {
        nit = dec_item(p, next);
        load_q(nit, nqa0, nqa2);
      }
      float o[HD / 8][4];
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      float m = -INFINITY, l = 0.f;
      for (int c = it.c_beg; c < it.c_end; ++c) {
        if (ok && !ptx::bounded_mbar_wait(&full_bar[stage], phase, abort_flag)) {
          if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          ok = false;
        }
        if (tracer && c == it.c_beg) tc_trace(p, n_done, 1);
        const int nvalid = min(kTcChunk, it.seq_len - c * kTcChunk);
        if (ok && tokw < nvalid) {
          const uint32_t kbase = ptx::smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t vbase = kbase + SL * kTcSlabBytes;
          float s_lo[4] = {0.f, 0.f, 0.f, 0.f}, s_hi[4] = {0.f, 0.f, 0.f, 0.f};
          {
            const int tok = tokw + (mi >> 1) * 8 + mr;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
              const int ch = ks * 2 + (mi & 1);
              const uint32_t addr = kbase + (ch >> 3) * kTcSlabBytes + tok * 128 + (((ch & 7) ^ (tok & 7)) << 4);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4(addr, b0, b1, b2, b3);
              mma16816<T>(s_lo, qa0[ks], 0u, qa2[ks], 0u, b0, b1);
              mma16816<T>(s_hi, qa0[ks], 0u, qa2[ks], 0u, b2, b3);
            }
          }
          const int col = tokw + 2 * t4;
          const bool v0 = col < nvalid, v1 = col + 1 < nvalid, v2 = col + 8 < nvalid, v3 = col + 9 < nvalid;
          float mx = -INFINITY;
          if (v0) mx = fmaxf(mx, s_lo[0]);
          if (v1) mx = fmaxf(mx, s_lo[1]);
          if (v2) mx = fmaxf(mx, s_hi[0]);
          if (v3) mx = fmaxf(mx, s_hi[1]);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          const float m_new = fmaxf(m, mx * p.scale_log2);
          const float alpha = exp2f(m - m_new);  // m = -inf -> 0
          const float p0 = v0 ? exp2f(s_lo[0] * p.scale_log2 - m_new) : 0.f;
          const float p1 = v1 ? exp2f(s_lo[1] * p.scale_log2 - m_new) : 0.f;
          const float p2 = v2 ? exp2f(s_hi[0] * p.scale_log2 - m_new) : 0.f;
          const float p3 = v3 ? exp2f(s_hi[1] * p.scale_log2 - m_new) : 0.f;
          l = l * alpha + (p0 + p1 + p2 + p3);
          m = m_new;
          const uint32_t pa0 = pk2<T>(p0, p1), pa2 = pk2<T>(p2, p3);
#pragma unroll
          for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= alpha;
            o[i][1] *= alpha;
          }
          {
            const int tok = tokw + (mi & 1) * 8 + mr;
#pragma unroll
            for (int np = 0; np < HD / 16; ++np) {
              const int ch = np * 2 + (mi >> 1);
              const uint32_t addr = vbase + (ch >> 3) * kTcSlabBytes + tok * 128 + (((ch & 7) ^ (tok & 7)) << 4);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4_trans(addr, b0, b1, b2, b3);
              mma16816<T>(o[2 * np], pa0, 0u, pa2, 0u, b0, b1);
              mma16816<T>(o[2 * np + 1], pa0, 0u, pa2, 0u, b2, b3);
            }
          }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty_bar[stage]);
        if (++stage == kTcStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (tracer) tc_trace(p, n_done, 2);
      // per-warp partials -> shared memory (rows < 8 only), then the 4 warps combine them
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t4 == 0) {
        mrg_m[warp * 8 + g] = m;
        mrg_l[warp * 8 + g] = l;
      }
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        float2 v = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(&mrg_o[(warp * 8 + g) * HD + i * 8 + 2 * t4]) = v;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int e = threadIdx.x; e < G * HD; e += 128) {
        const int gg = e / HD, d = e % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mrg_m[w * 8 + gg]);
        float L = 0.f, O = 0.f;
        if (M > -INFINITY) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float sc = exp2f(mrg_m[w * 8 + gg] - M);
            L += mrg_l[w * 8 + gg] * sc;
            O += mrg_o[(w * 8 + gg) * HD + d] * sc;
          }
        }
        const float val = L > 0.f ? O / L : 0.f;
        const int head = it.h * G + gg;
        if (p.num_splits == 1) {
          T* op = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(it.b) * p.out_stride +
                  static_cast<int64_t>(head) * HD;
          if (std::is_same<T, __nv_bfloat16>::value)
            reinterpret_cast<__nv_bfloat16*>(op)[d] = __float2bfloat16(val);
          else
            reinterpret_cast<__half*>(op)[d] = __float2half(val);
        } else {
          const int64_t base = (static_cast<int64_t>(it.b) * p.q_heads + head) * p.num_splits + it.split;
          p.part_o[base * HD + d] = val;
          if (d == 0) p.part_lse[base] = L > 0.f ? M + log2f(L) : -INFINITY;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // merge buffers are reused by the next item
      if (tracer) tc_trace(p, n_done, 3);
      it = nit;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        qa0[ks] = nqa0[ks];
        qa2[ks] = nqa2[ks];
      }
    }
  }
}

// Combine split partials: out = sum_s w_s o_s / sum_s w_s, w_s = 2^(lse_s - max lse).
template <typename T>
__global__ void attn_merge_tc_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                     T* __restrict__ out, int64_t out_stride, int q_heads, int hd, int num_splits) {
  const int b = blockIdx.x, head = blockIdx.y;
  const int64_t base = (static_cast<int64_t>(b) * q_heads + head) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_lse[base + s]);
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float acc = 0.f, wsum = 0.f;
    if (M > -INFINITY) {
      for (int s = 0; s < num_splits; ++s) {
        const float w = exp2f(part_lse[base + s] - M);
        wsum += w;
        acc += w * part_o[(base + s) * hd + d];
      }
    }
    const float val = wsum > 0.f ? acc / wsum : 0.f;
    T* op = out + static_cast<int64_t>(b) * out_stride + static_cast<int64_t>(head) * hd;
    if (std::is_same<T, __nv_bfloat16>::value)
      reinterpret_cast<__nv_bfloat16*>(op)[d] = __float2bfloat16(val);
    else
      reinterpret_cast<__half*>(op)[d] = __float2half(val);
  }
}

template <typename T, int HD>
static int launch_tc(const CUtensorMap& tm, const CUtensorMap& tm_tail, const DecodeTcParams& p, int batch,
                     cudaStream_t stream) {
  auto kern = attn_decode_tc_kernel<T, HD>;
  static PerDeviceOnce once;
  cudaError_t e = once.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<HD>::kSmemBytes); });
  if (e != cudaSuccess) return (int)e;
  const int items = batch * p.kv_heads * p.num_splits;
  const int sms = device_sm_count();
  return (int)launch_pdl(kern, dim3(items < sms ? items : sms), dim3(kTcThreads), TcCfg<HD>::kSmemBytes, stream, tm,
                         tm_tail, p);
}

}  // namespace blitz

namespace blitz {
static long long* g_tc_trace = nullptr;
}

extern "C" {
// Profiling aid: while `buf` (16 items x 8 int64 clock stamps, device memory) is set, CTA 0 of every following
// blitz_attn_decode launch records, per work item, when its first consumer warp starts the item, gets its first chunk,
// finishes its last chunk and finishes the merge (slots 0-3), and when the producer starts and ends issuing the item's
// loads (slots 4-5).
void blitz_attn_decode_set_trace(long long* buf) { blitz::g_tc_trace = buf; }
using namespace blitz;

// Bytes of fp32 scratch the split path needs: part_o then part_lse.
int64_t blitz_attn_decode_workspace_bytes(int batch, int q_heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return (int64_t)batch * q_heads * num_splits * (head_dim + 1) * (int64_t)sizeof(float);
}

// kv_layer: [max_pages][2][page_size][kv_heads][head_dim].  workspace: scratch of
// blitz_attn_decode_workspace_bytes() bytes (may be null when num_splits == 1).
// page_size must be a power of two >= 8 (pages smaller than 64 tokens are fetched as
// several boxes per stage).  q_heads / kv_heads <= 8; head_dim 64 or 128.
int blitz_attn_decode(const void* q, int64_t q_stride, const void* kv_layer, const int32_t* indices,
                      const int32_t* indptr, const int32_t* last_page_len, void* out, int64_t out_stride,
                      void* workspace, int batch, int q_heads, int kv_heads, int head_dim, int page_size,
                      int max_pages, int num_splits, float sm_scale, int* status, int dtype, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (num_splits < 1 || (q_heads % kv_heads) != 0 || (q_stride & 1) || (out_stride & 1)) return -1;
  const int G = q_heads / kv_heads;
  if (G > 8 || (head_dim != 64 && head_dim != 128)) return -1;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0) return -1;
  if (num_splits > 1 && workspace == nullptr) return -1;
  const int bt = page_size < kTcChunk ? page_size : kTcChunk;
  const int bt_tail = bt < 16 ? bt : 16;
  CUtensorMap tm, tm_tail;
  if (!get_tmap_3d(&tm, kv_layer, (uint64_t)head_dim, (uint64_t)kv_heads, (uint64_t)max_pages * 2 * page_size,
                   (uint64_t)head_dim * 2, (uint64_t)kv_heads * head_dim * 2, 64, 1, (uint32_t)bt))
    return -2;
  if (!get_tmap_3d(&tm_tail, kv_layer, (uint64_t)head_dim, (uint64_t)kv_heads, (uint64_t)max_pages * 2 * page_size,
                   (uint64_t)head_dim * 2, (uint64_t)kv_heads * head_dim * 2, 64, 1, (uint32_t)bt_tail))
    return -2;
  DecodeTcParams p;
  p.q = q; p.q_stride = q_stride; p.indices = indices; p.indptr = indptr; p.last_page_len = last_page_len;
  p.out = out; p.out_stride = out_stride;
  p.part_o = reinterpret_cast<float*>(workspace);
  p.part_lse = p.part_o ? p.part_o + (int64_t)batch * q_heads * num_splits * head_dim : nullptr;
  p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = G; p.page_size = page_size; p.max_pages = max_pages;
  p.num_splits = num_splits; p.box_tokens = bt; p.tail_box_tokens = bt_tail;
  p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status; p.trace = g_tc_trace;
  int rc;
  if (dtype == 1)
    rc = head_dim == 128 ? launch_tc<__nv_bfloat16, 128>(tm, tm_tail, p, batch, stream)
                         : launch_tc<__nv_bfloat16, 64>(tm, tm_tail, p, batch, stream);
  else
    rc = head_dim == 128 ? launch_tc<__half, 128>(tm, tm_tail, p, batch, stream)
                         : launch_tc<__half, 64>(tm, tm_tail, p, batch, stream);
  if (rc != 0) return rc;
  if (num_splits > 1) {
    dim3 grid(batch, q_heads);
    if (dtype == 1)
      attn_merge_tc_kernel<__nv_bfloat16><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__nv_bfloat16*)out,
                                                                         out_stride, q_heads, head_dim, num_splits);
    else
      attn_merge_tc_kernel<__half><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__half*)out, out_stride,
                                                                  q_heads, head_dim, num_splits);
    rc = (int)cudaGetLastError();
  }
  return rc;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant (declared and documented in attn_decode_noalloc.h).  The split-KV partials go to
// an array that is part of the library image instead of a caller-provided workspace.
#include "attn_decode_noalloc.h"

namespace blitz {

// Device global memory, present on every GPU that loads the library.  In host code this name is only a
// handle for the runtime: its device address is looked up once per device below and that address, not the
// name, is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[BLITZ_ATTN_NOALLOC_SCRATCH_BYTES];

constexpr int kNoallocMaxDevices = kMaxDevicesPerProcess;
// Device address of the scratch on each device: written once under the set-up lock and published with release
// order, so a host thread that sees a non-null value also sees a fully set-up device.
static std::atomic<void*> g_noalloc_ptr[kNoallocMaxDevices];
static PerDeviceOnce g_noalloc_once;

// Per-device set-up with that device current: resolve the scratch address, raise the shared-memory limits.
static cudaError_t noalloc_setup(int dev) {
  void* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
  if (e != cudaSuccess) return e;
  if (ptr == nullptr) return cudaErrorInvalidSymbol;
  e = cudaFuncSetAttribute(attn_decode_tc_kernel<__nv_bfloat16, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<128>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(attn_decode_tc_kernel<__nv_bfloat16, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<64>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(attn_decode_tc_kernel<__half, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<128>::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(attn_decode_tc_kernel<__half, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<64>::kSmemBytes);
  if (e != cudaSuccess) return e;
  g_noalloc_ptr[dev].store(ptr, std::memory_order_release);
  return cudaSuccess;
}

// Tensor map of one KV layer built on the stack (the cached builder keeps a host-side table; this path keeps nothing).
static bool noalloc_tmap(CUtensorMap* out, const void* kv_layer, int head_dim, int kv_heads, int max_pages, int page_size,
                         int box_tokens) {
  PFN_encodeTiled enc = get_encode_fn();
  if (!enc || (reinterpret_cast<uintptr_t>(kv_layer) & 15) != 0) return false;
  cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)kv_heads, (cuuint64_t)max_pages * 2 * page_size};
  cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)kv_heads * head_dim * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(kv_layer), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int HD>
static int noalloc_launch(const CUtensorMap& tm, const CUtensorMap& tm_tail, const DecodeTcParams& p, int sms,
                          cudaStream_t stream) {
  const int items = p.batch * p.kv_heads * p.num_splits;
  attn_decode_tc_kernel<T, HD><<<items < sms ? items : sms, kTcThreads, TcCfg<HD>::kSmemBytes, stream>>>(tm, tm_tail, p);
  return (int)cudaGetLastError();
}

}  // namespace blitz

extern "C" int blitz_attn_decode_noalloc(const void* q, int64_t q_stride, const void* kv_layer, const int32_t* indices,
                                         const int32_t* indptr, const int32_t* last_page_len, void* out,
                                         int64_t out_stride, int batch, int q_heads, int kv_heads, int head_dim,
                                         int page_size, int max_pages, int num_splits, float sm_scale, int* status,
                                         int dtype, cudaStream_t stream) {
  using namespace blitz;
  if (batch <= 0) return 0;
  if (num_splits < 1 || kv_heads <= 0 || (q_heads % kv_heads) != 0 || (q_stride & 1) || (out_stride & 1)) return -1;
  const int G = q_heads / kv_heads;
  if (G > 8 || (head_dim != 64 && head_dim != 128)) return -1;
  if (page_size < 8 || (page_size & (page_size - 1)) != 0) return -1;
  const int64_t need = num_splits > 1 ? (int64_t)batch * q_heads * num_splits * (head_dim + 1) * (int64_t)sizeof(float) : 0;
  if (need > (int64_t)BLITZ_ATTN_NOALLOC_SCRATCH_BYTES) return BLITZ_ATTN_NOALLOC_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return -1;
  e = g_noalloc_once.run([&] { return noalloc_setup(dev); });
  if (e != cudaSuccess) return (int)e;
  void* const scratch = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) return (int)cudaErrorInvalidSymbol;
  const int bt = page_size < kTcChunk ? page_size : kTcChunk;
  const int bt_tail = bt < 16 ? bt : 16;
  CUtensorMap tm, tm_tail;
  if (!noalloc_tmap(&tm, kv_layer, head_dim, kv_heads, max_pages, page_size, bt)) return -2;
  if (!noalloc_tmap(&tm_tail, kv_layer, head_dim, kv_heads, max_pages, page_size, bt_tail)) return -2;
  DecodeTcParams p;
  p.q = q; p.q_stride = q_stride; p.indices = indices; p.indptr = indptr; p.last_page_len = last_page_len;
  p.out = out; p.out_stride = out_stride;
  p.part_o = reinterpret_cast<float*>(scratch);
  p.part_lse = p.part_o + (int64_t)batch * q_heads * num_splits * head_dim;
  p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.group = G; p.page_size = page_size;
  p.max_pages = max_pages; p.num_splits = num_splits; p.box_tokens = bt; p.tail_box_tokens = bt_tail;
  p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status; p.trace = nullptr;
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  int rc;
  if (dtype == 1)
    rc = head_dim == 128 ? noalloc_launch<__nv_bfloat16, 128>(tm, tm_tail, p, sms, stream)
                         : noalloc_launch<__nv_bfloat16, 64>(tm, tm_tail, p, sms, stream);
  else
    rc = head_dim == 128 ? noalloc_launch<__half, 128>(tm, tm_tail, p, sms, stream)
                         : noalloc_launch<__half, 64>(tm, tm_tail, p, sms, stream);
  if (rc != 0 || num_splits == 1) return rc;
  dim3 grid(batch, q_heads);
  if (dtype == 1)
    attn_merge_tc_kernel<__nv_bfloat16><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__nv_bfloat16*)out, out_stride,
                                                                       q_heads, head_dim, num_splits);
  else
    attn_merge_tc_kernel<__half><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__half*)out, out_stride, q_heads,
                                                                head_dim, num_splits);
  return (int)cudaGetLastError();
}
