// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] = A[M,K] * B          (16-bit inputs, fp32 accumulation in TMEM)
//
// A is row-major (K contiguous).  B is either the serving weight layout
// [K,N] row-major ("in,out": N contiguous, an MN-major UMMA operand) or
// [N,K] row-major (K-major operand).  Operands are staged by TMA into
// 128-byte-swizzled shared memory; one elected thread issues tcgen05.mma with
// the accumulator in TMEM (double buffered so the epilogue of tile i overlaps
// the main loop of tile i+1); four epilogue warps read TMEM with tcgen05.ld
// and apply the fused epilogue:
//   store            C = acc
//   add              C = acc + R                (residual add of o_proj / down_proj)
//   silu_mul         C = silu(acc_gate) * acc_up  (gate||up projection; B holds
//                    N gate columns followed by N up columns)
//
// Replaces the cuBLAS wrapper of the reference (src/util/cublas_wrapper.h:31-141,
// call sites src/layer/attn.h:137-215, src/layer/glu.h:109-136,
// src/layer/lm_head.h:89-98); the silu_mul and add epilogues absorb
// src/kernel/activation.cu:9-23 and src/kernel/add.cu:13-55.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = UMMA issuer + TMEM
// owner, warps 2..5 = epilogue (TMEM lane quarter = warp_idx % 4).
#include "ptx.cuh"
#include "tmap.cuh"
#include <type_traits>

namespace blitz {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kGemmThreads = 192;

enum GemmEpilogue : int { kEpiStore = 0, kEpiAdd = 1, kEpiSiluMul = 2 };

struct GemmParams {
  void* C;
  const void* R;
  int64_t ldc;
  int M, N, K;      // N = output columns
  int a_box_rows;   // rows actually fetched per A tile (<= 128, multiple of 8)
  int up_col_off;   // silu_mul: column of B where the "up" half starts
  int tiles_m, tiles_n;
  int* status;
};

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // Shared memory is carved at run time: A stages are only as tall as the rows TMA actually fetches
  // (small-M decode GEMMs then keep 2-3x more weight bytes in flight); all A stages come first so that
  // the 128-row UMMA view of a short A stage still lies inside the allocation (the extra rows are
  // garbage and their output rows are never stored).
  static constexpr int kMaxStages = 24;
  static constexpr int kBarrierBytes = (2 * kMaxStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 227 * 1024;
  static constexpr int kUsableBytes = kSmemBytes - 1024 /*align slack*/ - kBarrierBytes;
  __host__ __device__ static int a_stage_bytes(int a_rows) { return ((a_rows * kBK * 2) + 1023) & ~1023; }
  __host__ __device__ static int num_stages(int a_rows) {
    int s = (kUsableBytes - kABytes) / (a_stage_bytes(a_rows) + kBBytes);
    return s > kMaxStages ? kMaxStages : s;
  }
  // A tcgen05.mma that accumulates into the accumulator of the previous one waits for it (~140 cycles
  // measured), which is longer than a 128xNx16 instruction runs when N < 256.  Narrow tiles therefore
  // rotate their K steps over kSplit independent TMEM accumulators (summed in the epilogue) so the
  // tensor pipe always has independent work: 4 accumulators for N = 64, 2 for N = 128.
  static constexpr int kSplit = 256 / BN;
  static constexpr int kAccCols = kSplit * BN;   // columns of one (double-buffered) accumulator set = 256
  static constexpr int kTmemCols = 2 * kAccCols; // 512: the whole TMEM of the SM
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

template <typename T, int BN, bool B_KMAJOR, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  const int S = Cfg::num_stages(p.a_box_rows);
  const int a_stage = Cfg::a_stage_bytes(p.a_box_rows);
  constexpr int kOutCols = (EPI == kEpiSiluMul) ? BN / 2 : BN;  // output columns per tile
  constexpr uint32_t kFmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdesc = ptx::make_idesc_f16(kFmt, 0u, B_KMAJOR ? 0u : 1u, kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + S * a_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kUsableBytes);
  uint64_t* full_bar = bars;             // [S]
  uint64_t* empty_bar = bars + Cfg::kMaxStages;        // [S]
  uint64_t* tfull_bar = bars + 2 * Cfg::kMaxStages;    // [2]
  uint64_t* tempty_bar = bars + 2 * Cfg::kMaxStages + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBK - 1) / kBK;
  const int num_tiles = p.tiles_m * p.tiles_n;

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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = static_cast<uint32_t>(p.a_box_rows) * kBK * 2 + Cfg::kBBytes;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % p.tiles_m) * kBM;
        const int n0 = (t / p.tiles_m) * kOutCols;
        for (int kb = 0; kb < num_kb; ++kb) {
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!ptx::bounded_mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
        for (int kb = 0; kb < num_kb; ++kb) {
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
            // K step k goes to sub-accumulator k % kSplit; its first use in a tile overwrites
            ptx::umma_f16_ss(d_tmem + static_cast<uint32_t>((k % Cfg::kSplit) * BN), adesc, bdesc, kIdesc,
                             (kb != 0 || k >= Cfg::kSplit) ? 1u : 0u);
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
    // ------------------------------------------------------------ epilogue warps
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    T* Cp = reinterpret_cast<T*>(p.C);
    const T* Rp = reinterpret_cast<const T*>(p.R);
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int m0 = (t % p.tiles_m) * kBM;
      const int n0 = (t / p.tiles_m) * kOutCols;
      if (!ptx::bounded_mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
        if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * Cfg::kAccCols);
      const int row = m0 + row_in_tile;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < kOutCols; c += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(taddr + c, v);
        if (Cfg::kSplit > 1) {  // sum the sub-accumulators
#pragma unroll
          for (int j = 1; j < Cfg::kSplit; ++j) {
            uint32_t w[32];
            ptx::tmem_ld_32x32(taddr + j * BN + c, w);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(w[i]));
          }
        }
        uint32_t out[16];
        if (EPI == kEpiSiluMul) {
          uint32_t u[32];
          ptx::tmem_ld_32x32(taddr + BN / 2 + c, u);
          ptx::tmem_ld_wait();
          if (Cfg::kSplit > 1) {
#pragma unroll
            for (int j = 1; j < Cfg::kSplit; ++j) {
              uint32_t w[32];
              ptx::tmem_ld_32x32(taddr + j * BN + BN / 2 + c, w);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) u[i] = __float_as_uint(__uint_as_float(u[i]) + __uint_as_float(w[i]));
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float g0 = __uint_as_float(v[2 * i]), g1 = __uint_as_float(v[2 * i + 1]);
            float u0 = __uint_as_float(u[2 * i]), u1 = __uint_as_float(u[2 * i + 1]);
            out[i] = pack2<T>(silu_f(g0) * u0, silu_f(g1) * u1);
          }
        } else {
          ptx::tmem_ld_wait();
          if (EPI == kEpiAdd) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + c + j * 8;
              uint4 r = make_uint4(0, 0, 0, 0);
              if (row_ok && col < p.N) r = *reinterpret_cast<const uint4*>(Rp + static_cast<int64_t>(row) * p.ldc + col);
              const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float2 f = unpack2<T>(rr[i]);
                out[j * 4 + i] = pack2<T>(__uint_as_float(v[j * 8 + 2 * i]) + f.x,
                                          __uint_as_float(v[j * 8 + 2 * i + 1]) + f.y);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) out[i] = pack2<T>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
          }
        }
        if (row_ok) {
          T* dst = Cp + static_cast<int64_t>(row) * p.ldc + n0 + c;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (n0 + c + j * 8 < p.N)
              *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
          }
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&tempty_bar[acc]);
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
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
    default: return dispatch_bn<T, B_KMAJOR, kEpiStore>(bn, ta, tb, p, grid, stream);
  }
}

// Tile width.  Measured on B200 at decode sizes: 128-wide tiles win once they give at least ~0.45 tiles per
// SM; below that 64-wide tiles (more CTAs streaming weights) are better; 256-wide only when it still
// fills the machine (large M) or for the gate||up GEMM, where a 256-wide tile yields 128 outputs.
static int choose_bn(int M, int N, int epi, int sms) {
  const int tiles_m = (M + kBM - 1) / kBM;
  auto tiles = [&](int bn) {
    const int out_cols = epi == kEpiSiluMul ? bn / 2 : bn;
    return tiles_m * ((N + out_cols - 1) / out_cols);
  };
  if (tiles(256) >= sms) return 256;
  if (epi == kEpiSiluMul) return 128;
  if (tiles(128) * 100 >= sms * 45) return 128;
  return 64;
}

}  // namespace blitz

extern "C" {

// dtype: 0 = fp16, 1 = bf16.  b_layout: 0 = B is [K, ldb>=Ncols] row-major
// (weights stored in,out), 1 = B is [Ncols, ldb>=K] row-major.  epilogue: 0
// store, 1 add residual R (same pitch as C), 2 silu(gate)*up where B carries N
// gate columns followed (at column `up_col_off`) by N up columns.
// bn_hint: 0 = choose, else 64/128/256.  Returns a cudaError_t value, or -1
// for an argument the kernel cannot take, -2 when the TMA encoder is missing.
int blitz_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, const void* R, int M,
               int N, int K, int b_layout, int epilogue, int up_col_off, int dtype, int bn_hint, int* status,
               cudaStream_t stream) {
  using namespace blitz;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 7)) return -1;
  if (epilogue == kEpiSiluMul && (up_col_off & 7)) return -1;
  const int sms = device_sm_count();
  int bn = bn_hint ? bn_hint : choose_bn(M, N, epilogue, sms);
  if (epilogue == kEpiSiluMul && bn < 128) bn = 128;
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

  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sms ? tiles : sms;
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

}  // extern "C"
