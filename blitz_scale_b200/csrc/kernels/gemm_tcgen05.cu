// Persistent, warp-specialised tcgen05 GEMM for sm_100a with fused epilogues and in-kernel split-K.
//
//   C[M,N] = A[M,K] * B          (16-bit inputs, fp32 accumulation in TMEM)
//
// A is row-major (K contiguous).  B is either the serving weight layout [K,N] row-major ("in,out":
// N contiguous, an MN-major UMMA operand) or [N,K] row-major (K-major operand).  Operands are staged
// by TMA into 128-byte-swizzled shared memory; one elected thread issues tcgen05.mma with the
// accumulator in TMEM (double buffered: the epilogue of one work item overlaps the main loop of the
// next); four epilogue warps read TMEM with tcgen05.ld and apply the fused epilogue:
//   store      C = acc
//   add        C = acc + R                  (residual add of o_proj / down_proj)
//   silu_mul   C = silu(acc_gate) * acc_up  (gate||up projection; B holds N gate columns, then N up columns)
//
// Measured on B200: a 128-row tcgen05.mma of K = 16 occupies the tensor pipe for ~95 / 105 / 150 cycles at
// N = 64 / 128 / 256, so (1) wide tiles are the most efficient per FLOP and (2) the time of a skinny GEMM
// is (K / 16) x that cost per CTA unless K is split.  Skinny GEMMs that do not qualify for the
// weight-streaming decode kernel (gemm_decode.cu: M <= 256, [K,N] weights) split K across CTAs until
// every SM has work: each CTA stores its fp32
// partial tile to a scratch buffer, takes a ticket, and the CTA that arrives last sums the partials
// in split order (deterministic), applies the epilogue and resets the ticket.  No second kernel.
//
// Replaces the cuBLAS wrapper of the reference (src/util/cublas_wrapper.h:31-141, call sites
// src/layer/attn.h:137-215, src/layer/glu.h:109-136, src/layer/lm_head.h:89-98); the silu_mul and add
// epilogues absorb src/kernel/activation.cu:9-23 and src/kernel/add.cu:13-55.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = UMMA issuer + TMEM owner, warps 2..5 =
// epilogue (TMEM lane quarter = warp_idx % 4).
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include <type_traits>

namespace blitz {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;
constexpr int kMaxSplitK = 16;

enum GemmEpilogue : int { kEpiStore = 0, kEpiAdd = 1, kEpiSiluMul = 2, kEpiPushRS = 3 };

struct GemmParams {
  void* C;
  const void* R;
  int64_t ldc;
  int M, N, K;        // N = output columns
  int a_box_rows;     // rows actually fetched per A tile (<= 128, multiple of 8)
  int up_col_off;     // silu_mul: column of B where the "up" half starts
  int tiles_m, tiles_n;
  int split_k;        // CTAs sharing one output tile along K
  int kb_per_split;   // 64-wide K blocks per split
  float* ws;          // split-K partials: [tile][split][128][BN] fp32
  unsigned* tickets;  // one per output tile, zero between launches
  int* status;
  // Tensor-parallel fusion.  push epilogue (GEMM -> reduce-scatter): row r of the partial result belongs to
  // rank r / rows_per_rank and is stored into that rank's staging area [src rank][N/8][local row][8] over NVLink;
  // one counter per (owner, source) is bumped per finished tile.  wait_flags (all-gather -> GEMM): the TMA
  // producer waits until each of n_wait counters reaches wait_value before its first load of A, whose rows
  // other ranks have stored into local memory.
  uint8_t* push_base[8];
  uint32_t* push_flags[8];
  int tp, tp_rank, rows_per_rank;
  const uint32_t* wait_flags;
  int n_wait;
  uint32_t wait_value;
  int n_fast;  // tensor-parallel fusion: N runs fastest over the tiles, M blocks start at m_rot (see gemm_tile_blocks)
  int m_rot;
};

// Tile number -> (M block, N block).  Normally M runs fastest.  When the rows of A arrive from other ranks
// (n_wait > 0: counter s = rows that source s has delivered, wait_value rows each) N runs fastest and the M blocks
// start at this rank's own rows and go on through the other sources' in rank order: every CTA first works on rows
// that are here already, and waits (see the producer) only for the source whose rows it is about to load, so the
// GEMM overlaps the arrival of the later sources' rows instead of starting after the last one.
// (The push epilogue, GEMM -> reduce-scatter, keeps M fastest: an owner's block of rows is complete only when the
// last source has produced it, and the kernel that reduces it is a later launch of the same stream, so a different
// order buys no overlap and costs weight-tile reuse in L2: measured 252 against 233 us at M = 4096, K = 4096 per rank.)
__device__ __forceinline__ void gemm_tile_blocks(const GemmParams& p, int tile, int& mb, int& nb) {
  if (p.n_fast) {
    const int lin = tile / p.tiles_n;
    nb = tile - lin * p.tiles_n;
    mb = lin + p.m_rot;
    if (mb >= p.tiles_m) mb -= p.tiles_m;
  } else {
    mb = tile % p.tiles_m;
    nb = tile / p.tiles_m;
  }
}

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  // Shared memory is carved at run time: A stages are only as tall as the rows TMA actually fetches
  // (small-M decode GEMMs then keep more weight bytes in flight); all A stages come first so that the
  // 128-row UMMA view of a short A stage still lies inside the allocation (the extra rows are garbage
  // and their output rows are never stored).
  static constexpr int kMaxStages = 24;
  static constexpr int kBarrierBytes = (2 * kMaxStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 227 * 1024;
  static constexpr int kUsableBytes = kSmemBytes - 1024 /*align slack*/ - kBarrierBytes;
  __host__ __device__ static int a_stage_bytes(int a_rows) { return ((a_rows * kBK * 2) + 1023) & ~1023; }
  __host__ __device__ static int num_stages(int a_rows) {
    int s = (kUsableBytes - kABytes) / (a_stage_bytes(a_rows) + kBBytes);
    return s > kMaxStages ? kMaxStages : s;
  }
  static constexpr int kTmemCols = 2 * BN;
};

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Epilogue of 32 consecutive output columns of one row: acc (and up for silu_mul) -> C.
template <typename T, int EPI>
__device__ __forceinline__ void store_chunk(const GemmParams& p, const float (&acc)[32], const float (&up)[32], int row,
                                            int col0, bool row_ok) {
  uint32_t out[16];
  if (EPI == kEpiSiluMul) {
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = pack2<T>(silu_f(acc[2 * i]) * up[2 * i], silu_f(acc[2 * i + 1]) * up[2 * i + 1]);
  } else if (EPI == kEpiAdd) {
    const T* Rp = reinterpret_cast<const T*>(p.R);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = col0 + j * 8;
      uint4 r = make_uint4(0, 0, 0, 0);
      if (row_ok && col < p.N) r = *reinterpret_cast<const uint4*>(Rp + static_cast<int64_t>(row) * p.ldc + col);
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<T>(rr[i]);
        out[j * 4 + i] = pack2<T>(acc[j * 8 + 2 * i] + f.x, acc[j * 8 + 2 * i + 1] + f.y);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = pack2<T>(acc[2 * i], acc[2 * i + 1]);
  }
  if (row_ok) {
    if (EPI == kEpiPushRS) {
      // staging layout of the owner: [source rank][8-column vector][local row][8 elements].  The 32 lanes of a warp
      // hold 32 consecutive rows, so each of these stores is 512 contiguous bytes on the wire (a row-major
      // staging area would make it 32 separate 16-byte pieces)
      const int owner = row / p.rows_per_rank, lrow = row - owner * p.rows_per_rank;
      const int64_t nvec = p.N >> 3;
      T* base = reinterpret_cast<T*>(p.push_base[owner]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t vc = (col0 >> 3) + j;
        if (col0 + j * 8 < p.N)
          ptx::st_na_v4(base + ((static_cast<int64_t>(p.tp_rank) * nvec + vc) * p.rows_per_rank + lrow) * 8,
                        make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]));
      }
    } else {
      T* dst = reinterpret_cast<T*>(p.C) + static_cast<int64_t>(row) * p.ldc + col0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (col0 + j * 8 < p.N)
          *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
      }
    }
  }
}

// After every epilogue thread has stored its rows of a tile: make them visible system-wide and tell each
// owner rank that one more tile from this source has landed in the 128-row block(s) of its rows the tile covers.
__device__ __forceinline__ void push_signal(const GemmParams& p, int m0, int epi_tid) {
  __threadfence_system();
  asm volatile("bar.sync 2, 128;" ::: "memory");
  if (epi_tid == 0) {
    // counters of an owner: [block of 128 of its rows][source]
    const int last_row = min(p.M, m0 + kBM) - 1;
    ptx::fence_acq_rel_sys();
    for (int o = m0 / p.rows_per_rank; o <= last_row / p.rows_per_rank; ++o) {
      const int base = o * p.rows_per_rank;
      const int lo = max(m0, base) - base, hi = min(last_row, base + p.rows_per_rank - 1) - base;
      for (int lb = lo >> 7; lb <= (hi >> 7); ++lb) ptx::red_add_release_sys(p.push_flags[o] + lb * 8 + p.tp_rank, 1u);
    }
  }
}

template <typename T, int BN, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kOutCols = (EPI == kEpiSiluMul) ? BN / 2 : BN;  // output columns per tile
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdesc = ptx::make_idesc_f16(kFmt, 0u, B_KMAJOR ? 0u : 1u, kBM, BN);
  const int S = Cfg::num_stages(p.a_box_rows);
  const int a_stage = Cfg::a_stage_bytes(p.a_box_rows);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + S * a_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kUsableBytes);
  uint64_t* full_bar = bars;                               // [S]
  uint64_t* empty_bar = bars + Cfg::kMaxStages;            // [S]
  uint64_t* tfull_bar = bars + 2 * Cfg::kMaxStages;        // [2]
  uint64_t* tempty_bar = bars + 2 * Cfg::kMaxStages + 2;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_items = num_tiles * p.split_k;  // item = tile * split_k + split

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], 128);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_a);
    ptx::tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // programmatic dependent launch: set-up above overlapped the previous kernel's tail; from here on we
  // touch memory that earlier kernels may have written
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = static_cast<uint32_t>(p.a_box_rows) * kBK * 2 + Cfg::kBBytes;
      bool ok = true;
      uint32_t arrived = 0;  // sources whose rows are known to be here
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        const int tile = w / p.split_k, split = w % p.split_k;
        int mb, nb;
        gemm_tile_blocks(p, tile, mb, nb);
        const int m0 = mb * kBM;
        const int n0 = nb * kOutCols;
        if (p.n_wait > 0) {
          // rows of A arrive by peer stores (generic proxy); TMA reads them through the async proxy: wait for the
          // sources this M block takes rows from, then fence
          const int s_lo = m0 / static_cast<int>(p.wait_value);
          const int s_hi = min(p.n_wait - 1, (min(p.M, m0 + kBM) - 1) / static_cast<int>(p.wait_value));
          bool fresh = false;
          for (int sidx = s_lo; sidx <= s_hi && ok; ++sidx) {
            if ((arrived >> sidx) & 1u) continue;
            if (!ptx::bounded_flag_wait_ge(p.wait_flags + sidx, p.wait_value, ptx::kDefaultWaitNs)) ok = false;
            arrived |= 1u << sidx;
            fresh = true;
          }
          if (!ok) {
            *abort_flag = 1;
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
            break;
          }
          if (fresh) ptx::fence_proxy_async_all();
        }
        const int kb_beg = split * p.kb_per_split;
        const int kb_end = min(num_kb, kb_beg + p.kb_per_split);
        for (int kb = kb_beg; kb < kb_end; ++kb) {
          if (!ptx::bounded_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          ptx::mbar_expect_tx(&full_bar[stage], tx_bytes);
          ptx::tma_load_2d(smem_a + stage * a_stage, &tmap_a, &full_bar[stage], kb * kBK, m0);
          uint8_t* sb = smem_b + stage * Cfg::kBBytes;
          if (B_KMAJOR) {
            // B is [N,K]: one box of BN rows x 64 K-elements per half (silu: gate rows then up rows).
            if (EPI == kEpiSiluMul) {
              ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, n0);
              ptx::tma_load_2d(sb + (BN / 2) * 128, &tmap_b, &full_bar[stage], kb * kBK, p.up_col_off + n0);
            } else {
              ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, n0);
            }
          } else {
            // B is [K,N]: slabs of 64 columns x 64 K-rows (8 KB each, 128-byte rows).
            constexpr int kSlabs = BN / 64;
#pragma unroll
            for (int s = 0; s < kSlabs; ++s) {
              int col;
              if (EPI == kEpiSiluMul) {
                constexpr int kHalfSlabs = kSlabs / 2;
                col = (s < kHalfSlabs) ? (n0 + s * 64) : (p.up_col_off + n0 + (s - kHalfSlabs) * 64);
              } else {
                col = n0 + s * 64;
              }
              ptx::tma_load_2d(sb + s * 8192, &tmap_b, &full_bar[stage], col, kb * kBK);
            }
          }
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        const int split = w % p.split_k;
        const int kb_beg = split * p.kb_per_split;
        const int kb_end = min(num_kb, kb_beg + p.kb_per_split);
        if (!ptx::bounded_mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb_beg; kb < kb_end; ++kb) {
          if (!ptx::bounded_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t a_base = ptx::smem_u32(smem_a + stage * a_stage);
          const uint32_t b_base = ptx::smem_u32(smem_b + stage * Cfg::kBBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // A: K-major, 128-byte rows, 8-row groups 1024 B apart; 16 K-elements = 32 B.
            const uint64_t adesc = ptx::make_smem_desc(a_base + k * 32, 16, 1024, ptx::kLayoutSw128);
            uint64_t bdesc;
            if (B_KMAJOR) {
              bdesc = ptx::make_smem_desc(b_base + k * 32, 16, 1024, ptx::kLayoutSw128);
            } else {
              // B: N-major slabs; 64-column chunks 8192 B apart (leading offset),
              // 8-K-row groups 1024 B apart (stride offset); 16 K-rows = 2048 B.
              bdesc = ptx::make_smem_desc(b_base + k * 2048, 8192, 1024, ptx::kLayoutSw128);
            }
            ptx::umma_f16_ss(d_tmem, adesc, bdesc, kIdesc, (kb != kb_beg || k != 0) ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[stage]);
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (128 threads, named barrier 2)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
      const int tile = w / p.split_k;
      int mb, nb;
      gemm_tile_blocks(p, tile, mb, nb);
      const int m0 = mb * kBM;
      const int n0 = nb * kOutCols;
      if (!ptx::bounded_mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const int row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
      if (p.split_k == 1) {
#pragma unroll 1
        for (int c = 0; c < kOutCols; c += 32) {
          uint32_t v[32];
          float a[32], u[32];
          ptx::tmem_ld_32x32(taddr + c, v);
          if (EPI == kEpiSiluMul) {
            uint32_t t[32];
            ptx::tmem_ld_32x32(taddr + BN / 2 + c, t);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) u[i] = __uint_as_float(t[i]);
          } else {
            ptx::tmem_ld_wait();
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = __uint_as_float(v[i]);
          store_chunk<T, EPI>(p, a, u, row, n0 + c, row_ok);
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(&tempty_bar[acc]);
        if (EPI == kEpiPushRS) push_signal(p, m0, epi_tid);
      } else {
        // split-K: park the fp32 partial, the last CTA of the tile reduces and finishes it
        // partial layout [BN/4][128 rows][4 floats]: the 32 lanes (= 32 rows) of a store write 512 contiguous bytes
        float* part = p.ws + static_cast<size_t>(w) * (kBM * BN) + static_cast<size_t>(row_in_tile) * 4;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(taddr + c, v);
          ptx::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              __stcg(reinterpret_cast<uint4*>(part + static_cast<size_t>(c / 4 + j) * (kBM * 4)),
                     make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
          }
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(&tempty_bar[acc]);
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (epi_tid == 0) {
          const unsigned old = atomicAdd(&p.tickets[tile], 1u);
          const int last = (old == static_cast<unsigned>(p.split_k - 1)) ? 1 : 0;
          if (last) p.tickets[tile] = 0;  // ready for the next launch
          *last_flag = last;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          const float* base = p.ws + static_cast<size_t>(tile) * p.split_k * (kBM * BN) + static_cast<size_t>(row_in_tile) * 4;
#pragma unroll 1
          for (int c = 0; c < kOutCols; c += 32) {
            float a[32], u[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = u[i] = 0.f;
            if (row_ok) {
              for (int s = 0; s < p.split_k; ++s) {
                const float* ps = base + static_cast<size_t>(s) * (kBM * BN);
                float4 f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  f[j] = __ldcg(reinterpret_cast<const float4*>(ps + static_cast<size_t>(c / 4 + j) * (kBM * 4)));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  a[4 * j] += f[j].x; a[4 * j + 1] += f[j].y; a[4 * j + 2] += f[j].z; a[4 * j + 3] += f[j].w;
                }
                if (EPI == kEpiSiluMul) {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    f[j] = __ldcg(reinterpret_cast<const float4*>(ps + static_cast<size_t>((BN / 2 + c) / 4 + j) * (kBM * 4)));
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    u[4 * j] += f[j].x; u[4 * j + 1] += f[j].y; u[4 * j + 2] += f[j].z; u[4 * j + 3] += f[j].w;
                  }
                }
              }
            }
            store_chunk<T, EPI>(p, a, u, row, n0 + c, row_ok);
          }
          if (EPI == kEpiPushRS) push_signal(p, m0, epi_tid);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");  // last_flag is rewritten by the next item
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
template <typename T, int BN, bool B_KMAJOR, int EPI>
static cudaError_t launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                               cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tcgen05_kernel<T, BN, B_KMAJOR, EPI>;
  static PerDeviceOnce once;
  cudaError_t e = once.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes); });
  if (e != cudaSuccess) return e;
  return launch_pdl(kern, dim3(grid), dim3(kGemmThreads), Cfg::kSmemBytes, stream, ta, tb, p);
}

template <typename T, bool B_KMAJOR, int EPI>
static cudaError_t dispatch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                               cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_gemm<T, 256, B_KMAJOR, EPI>(ta, tb, p, grid, stream);
    case 128: return launch_gemm<T, 128, B_KMAJOR, EPI>(ta, tb, p, grid, stream);
    default:
      if (EPI == kEpiSiluMul) return launch_gemm<T, 128, B_KMAJOR, EPI>(ta, tb, p, grid, stream);
      return launch_gemm<T, 64, B_KMAJOR, (EPI == kEpiSiluMul ? kEpiStore : EPI)>(ta, tb, p, grid, stream);
  }
}

template <typename T, bool B_KMAJOR>
static cudaError_t dispatch_epi(int epi, int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                                int grid, cudaStream_t stream) {
  switch (epi) {
    case kEpiAdd: return dispatch_bn<T, B_KMAJOR, kEpiAdd>(bn, ta, tb, p, grid, stream);
    case kEpiSiluMul: return dispatch_bn<T, B_KMAJOR, kEpiSiluMul>(bn, ta, tb, p, grid, stream);
    case kEpiPushRS: return dispatch_bn<T, B_KMAJOR, kEpiPushRS>(bn, ta, tb, p, grid, stream);
    default: return dispatch_bn<T, B_KMAJOR, kEpiStore>(bn, ta, tb, p, grid, stream);
  }
}

}  // namespace blitz

extern "C" {

// Scratch the split-K path needs for a problem: bytes of fp32 partials (tickets are separate: one
// uint32 per output tile, zero-initialised once by the caller; the kernel leaves them zero).
int64_t blitz_gemm_workspace_bytes(int sms) { return (int64_t)(sms + 16) * blitz::kBM * 256 * 4; }

// dtype: 0 = fp16, 1 = bf16.  b_layout: 0 = B is [K, ldb>=Ncols] row-major (weights stored in,out),
// 1 = B is [Ncols, ldb>=K] row-major.  epilogue: 0 store, 1 add residual R (same pitch as C),
// 2 silu(gate)*up where B carries N gate columns followed (at column `up_col_off`) by N up columns.
// bn_hint: 0 = 256-wide tiles, else 64/128/256.  split_hint: 0 = choose, 1 = never split, else the
// number of K splits.  ws / ws_bytes: fp32 scratch for split-K partials, tickets / num_tickets:
// zeroed uint32 array (both may be null: the GEMM then never splits).
// Returns a cudaError_t value, or -1 for an argument the kernel cannot take, -2 when the TMA
// encoder is missing.
// Tile width the launcher uses for a problem (callers of the push epilogue need it to know how many tiles
// each owner rank will receive: ceil(N / tile_n) per 128-row block that overlaps the owner's rows).
int blitz_gemm_tile_n(int M, int N, int epilogue, int bn_hint) {
  using namespace blitz;
  const int sms = device_sm_count();
  int bn = bn_hint;
  if (!bn) {
    const int oc256 = epilogue == kEpiSiluMul ? 128 : 256;
    const int tiles256 = ((M + kBM - 1) / kBM) * ((N + oc256 - 1) / oc256);
    bn = tiles256 >= sms ? 256 : 128;
  }
  if (epilogue == kEpiSiluMul && bn < 128) bn = 128;
  return bn;
}

struct BlitzGemmTp {
  void* push_base[8];      // kEpiPushRS: staging base of every rank (peer pointers), [tp][rows_per_rank][N] each
  uint32_t* push_flags[8];  // flag array of every rank; entry [tp_rank] is bumped per tile
  int tp, tp_rank, rows_per_rank;
  const uint32_t* wait_flags;  // local counters to wait for before loading A (null: none)
  int n_wait;
  uint32_t wait_value;
};

static int gemm_impl(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int M,
                     int N, int K, int b_layout, int epilogue, int up_col_off, int dtype, int bn_hint, int split_hint,
                     void* ws, int64_t ws_bytes, unsigned* tickets, int num_tickets, int* status,
                     const BlitzGemmTp* tpa, cudaStream_t stream) {
  using namespace blitz;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -1;
  if (epilogue == kEpiSiluMul && (up_col_off & 7)) return -1;
  const int sms = device_sm_count();
  // 256-wide tiles are the most efficient per FLOP (a 128xNx16 instruction costs ~95 cycles at N = 64,
  // ~105 at N = 128, ~150 at N = 256); when they would leave SMs idle, 128-wide tiles plus split-K win.
  const int bn = blitz_gemm_tile_n(M, N, epilogue, bn_hint);
  const int out_cols = epilogue == kEpiSiluMul ? bn / 2 : bn;
  const int b_cols_total = epilogue == kEpiSiluMul ? up_col_off + N : N;

  GemmParams p;
  p.C = C;
  p.R = R;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.a_box_rows = M >= kBM ? kBM : ((M + 7) & ~7);
  p.up_col_off = up_col_off;
  p.tiles_m = (M + kBM - 1) / kBM;
  p.tiles_n = (N + out_cols - 1) / out_cols;
  p.status = status;
  p.tp = 1; p.tp_rank = 0; p.rows_per_rank = M; p.wait_flags = nullptr; p.n_wait = 0; p.wait_value = 0; p.m_rot = 0; p.n_fast = 0;
  for (int i = 0; i < 8; ++i) { p.push_base[i] = nullptr; p.push_flags[i] = nullptr; }
  if (tpa) {
    p.tp = tpa->tp; p.tp_rank = tpa->tp_rank; p.rows_per_rank = tpa->rows_per_rank > 0 ? tpa->rows_per_rank : M;
    p.wait_flags = tpa->wait_flags; p.n_wait = tpa->wait_flags ? tpa->n_wait : 0; p.wait_value = tpa->wait_value;
    if (p.n_wait > 0) {
      if (p.wait_value == 0 || p.n_wait > 32) return -1;
      p.n_fast = 1;
      p.m_rot = (int)(((int64_t)tpa->tp_rank * p.wait_value) / kBM) % ((M + kBM - 1) / kBM);
    }

    for (int i = 0; i < 8 && i < tpa->tp; ++i) {
      p.push_base[i] = reinterpret_cast<uint8_t*>(tpa->push_base[i]);
      p.push_flags[i] = tpa->push_flags[i];
    }
  }
  if (epilogue == kEpiPushRS && (!tpa || tpa->tp < 1 || tpa->tp > 8 || p.rows_per_rank * tpa->tp < M)) return -1;
  const int tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (K + kBK - 1) / kBK;

  // split K until every SM has a work item (skinny decode GEMMs), bounded by the scratch we were given
  int split = 1;
  if (split_hint != 1 && ws && tickets && tiles <= num_tickets && tiles * 4 < sms * 3) {
    // measured sweet spot: enough splits to fill the SMs but at most 4 (the reduction grows with the split count)
    split = split_hint > 1 ? split_hint : (sms / tiles > 4 ? 4 : sms / tiles);
    if (split > kMaxSplitK) split = kMaxSplitK;
    if (split > num_kb) split = num_kb;
    const int64_t per_item = (int64_t)kBM * bn * 4;
    if ((int64_t)tiles * split * per_item > ws_bytes) split = (int)(ws_bytes / (tiles * per_item));
    if (split < 1) split = 1;
  }
  p.kb_per_split = (num_kb + split - 1) / split;
  p.split_k = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
  p.ws = reinterpret_cast<float*>(ws);
  p.tickets = tickets;

  CUtensorMap ta, tb;
  if (!get_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kBK, (uint32_t)p.a_box_rows)) return -2;
  bool okb;
  if (b_layout == 0) {
    okb = get_tmap_2d(&tb, B, (uint64_t)b_cols_total, (uint64_t)K, (uint64_t)ldb * 2, 64, kBK);
  } else {
    const uint32_t box_rows = epilogue == kEpiSiluMul ? bn / 2 : bn;
    okb = get_tmap_2d(&tb, B, (uint64_t)K, (uint64_t)b_cols_total, (uint64_t)ldb * 2, kBK, box_rows);
  }
  if (!okb) return -2;

  const int items = tiles * p.split_k;
  const int grid = items < sms ? items : sms;
  cudaError_t e;
  if (dtype == 1) {
    e = b_layout == 0 ? dispatch_epi<__nv_bfloat16, false>(epilogue, bn, ta, tb, p, grid, stream)
                      : dispatch_epi<__nv_bfloat16, true>(epilogue, bn, ta, tb, p, grid, stream);
  } else {
    e = b_layout == 0 ? dispatch_epi<__half, false>(epilogue, bn, ta, tb, p, grid, stream)
                      : dispatch_epi<__half, true>(epilogue, bn, ta, tb, p, grid, stream);
  }
  return static_cast<int>(e);
}

int blitz_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int M,
               int N, int K, int b_layout, int epilogue, int up_col_off, int dtype, int bn_hint, int split_hint,
               void* ws, int64_t ws_bytes, unsigned* tickets, int num_tickets, int* status, cudaStream_t stream) {
  return gemm_impl(A, lda, B, ldb, C, ldc, R, M, N, K, b_layout, epilogue, up_col_off, dtype, bn_hint, split_hint, ws,
                   ws_bytes, tickets, num_tickets, status, nullptr, stream);
}

// Tensor-parallel variant: epilogue 3 pushes the partial result to the owner ranks' staging areas
// (GEMM -> reduce-scatter); a non-null tp->wait_flags makes the kernel wait for rows of A that other
// ranks are storing into local memory (all-gather -> GEMM).  See BlitzGemmTp.
int blitz_gemm_tp(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int M,
                  int N, int K, int b_layout, int epilogue, int up_col_off, int dtype, int bn_hint, int split_hint,
                  void* ws, int64_t ws_bytes, unsigned* tickets, int num_tickets, int* status, const BlitzGemmTp* tp,
                  cudaStream_t stream) {
  return gemm_impl(A, lda, B, ldb, C, ldc, R, M, N, K, b_layout, epilogue, up_col_off, dtype, bn_hint, split_hint, ws,
                   ws_bytes, tickets, num_tickets, status, tp, stream);
}

}  // extern "C"
