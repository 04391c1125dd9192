// Weight-streaming tcgen05 GEMM for decode batches (M <= 256 tokens) on sm_100a.
//
//   C[M,N] = X[M,K] * W[K,N]      W in the serving layout ("in,out", N contiguous), 16-bit, fp32 accumulation
//
// A decode step multiplies a few activation rows with every weight matrix of the model, so the work is
// a stream of weight bytes and the kernel is built around that:
//
//  * Operands are swapped on the tensor core.  The weight tile is the 128-row operand of tcgen05.mma
//    (128 output features per instruction, MN-major because N is contiguous in memory) and the batch is
//    the instruction's N (16..256, M rounded up to 16).  One instruction covers the whole batch, and a
//    small batch costs a small instruction instead of a 128-row tile that is mostly padding.  The
//    accumulator in TMEM holds C transposed: lane = output feature, column = token.
//  * A single SM cannot pull more than ~50 GB/s through TMA (measured), so HBM is only saturated when
//    ~128 or more SMs stream.  Matrices with fewer than that many 128-feature tiles therefore split K
//    over a thread-block cluster: the `split` CTAs of a cluster work on the same tile, each on 1/split
//    of K.  The reduction never touches global memory: after a cluster barrier every CTA stores its fp32
//    accumulator, slice by slice, straight into the shared memory of the CTA that owns that slice of
//    tokens (st.shared::cluster), a second cluster barrier publishes the stores, and every CTA adds the
//    slices for its own tokens in rank order (deterministic) and runs the epilogue for them.  The
//    reduction and the epilogue are thus spread over all CTAs of the cluster.
//  * Programmatic dependent launch: the kernel lets its successor start early and waits for its own
//    predecessor only when it first needs activations.  When the caller declares the weights static, the
//    producer fills the whole TMA pipeline with weight tiles before that wait, so the HBM stream of this
//    GEMM starts while the previous kernel is still draining.
//
// Epilogues: store, residual add, silu(gate)*up (two accumulators per tile: gate features and up features).
// Replaces the cuBLAS calls of the reference at decode sizes (src/util/cublas_wrapper.h:31-141; call
// sites src/layer/attn.h:137-215, src/layer/glu.h:109-136).
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = UMMA issuer + TMEM owner, warps 2..5 = epilogue.
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include <cstdlib>
#include <type_traits>

namespace blitz {

constexpr int kDecThreads = 192;
constexpr int kDecBK = 64;
constexpr int kDecTile = 128;  // output features per tile = UMMA M
constexpr int kDecMaxSplit = 8;

struct DecGemmParams {
  void* C;
  const void* R;
  int64_t ldc;
  int M, N, K;
  int npad;          // UMMA N: M rounded up to 16
  int x_box_rows;    // rows of X that TMA fetches per stage (M rounded up to 8)
  int up_col_off;    // silu_mul: column of W where the "up" half starts
  int num_kb;        // 64-wide K blocks
  int tiles;         // 128-feature tiles
  int split;         // CTAs per tile = cluster size
  int kb_per_split;  // K blocks per CTA of a cluster
  int slice;         // tokens each cluster rank reduces and stores (multiple of 32: TMEM is read 32 columns at a time)
  int static_w;      // weights do not depend on earlier kernels of the stream
  int smem_bytes;    // dynamic shared memory of this launch (227 KB, or about half of it for two CTAs per SM)
  int* status;
};

struct DecCfg {
  static constexpr int kMaxStages = 12;
  static constexpr int kBarrierBytes = (2 * kMaxStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 227 * 1024;       // one CTA per SM
  static constexpr int kSmemBytesHalf = 113 * 1024;   // two CTAs per SM
  __host__ __device__ static int usable_bytes(int smem_bytes) { return smem_bytes - 1024 - kBarrierBytes; }
  __host__ __device__ static int x_stage_bytes(int npad) { return (npad * kDecBK * 2 + 1023) & ~1023; }
  __host__ __device__ static int num_stages(int npad, int w_bytes, int smem_bytes) {
    const int s = usable_bytes(smem_bytes) / (x_stage_bytes(npad) + w_bytes);
    return s > kMaxStages ? kMaxStages : s;
  }
  // The epilogue reads TMEM 32 columns at a time, so an accumulator is read up to `extent` columns from its
  // start: (halves - 1) * npad + M rounded up to 32.
  __host__ __device__ static int extent(int M, int npad, int halves) { return (halves - 1) * npad + ((M + 31) & ~31); }
  __host__ __device__ static int num_acc(int M, int npad, int halves, int split) {
    return (split == 1 && halves * npad + extent(M, npad, halves) <= 512) ? 2 : 1;
  }
  __host__ __device__ static int tmem_cols(int M, int npad, int halves, int split) {
    const int need = (num_acc(M, npad, halves, split) - 1) * halves * npad + extent(M, npad, halves);
    int c = 32;
    while (c < need) c <<= 1;
    return c;
  }
};

template <typename T>
__device__ __forceinline__ T dec_cvt(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 dec_cvt<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half dec_cvt<__half>(float v) { return __float2half_rn(v); }
template <typename T>
__device__ __forceinline__ float dec_f32(T v);
template <>
__device__ __forceinline__ float dec_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float dec_f32<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ float dec_silu(float x) { return x / (1.0f + __expf(-x)); }

// EPI: 0 store, 1 add residual, 2 silu(gate)*up.  Thread = output feature n; tokens b0 .. min(b0 + 32, b_end).
// A warp writes 64 contiguous bytes per token.
template <typename T, int EPI>
__device__ __forceinline__ void dec_store32(const DecGemmParams& p, const float (&g)[32], const float (&u)[32], int n,
                                            int b0, int b_end) {
  if (n >= p.N) return;
  T* c = reinterpret_cast<T*>(p.C) + n;
  float res[32];
  if (EPI == 1) {
    // C may alias R (in-place residual update): read all residual values before the first store, otherwise
    // every load would have to wait for the store before it
    const T* r = reinterpret_cast<const T*>(p.R) + n;
#pragma unroll
    for (int i = 0; i < 32; ++i) res[i] = (b0 + i < b_end) ? dec_f32<T>(r[static_cast<int64_t>(b0 + i) * p.ldc]) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int b = b0 + i;
    if (b < b_end) {
      float v = g[i];
      if (EPI == 2) v = dec_silu(v) * u[i];
      if (EPI == 1) v += res[i];
      c[static_cast<int64_t>(b) * p.ldc] = dec_cvt<T>(v);
    }
  }
}

template <typename T, int EPI>
__global__ void __launch_bounds__(kDecThreads, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const DecGemmParams p) {
  using Cfg = DecCfg;
  constexpr int kHalves = (EPI == 2) ? 2 : 1;
  constexpr int kWBytes = kHalves * kDecTile * kDecBK * 2;  // weight bytes per stage
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  const int cols = kHalves * p.npad;  // TMEM columns per accumulator
  const int num_acc = Cfg::num_acc(p.M, p.npad, kHalves, p.split);
  const int tmem_cols = Cfg::tmem_cols(p.M, p.npad, kHalves, p.split);
  const int S = Cfg::num_stages(p.npad, kWBytes, p.smem_bytes);
  const int x_stage = Cfg::x_stage_bytes(p.npad);
  const uint32_t idesc = ptx::make_idesc_f16(kFmt, 1u, 0u, kDecTile, static_cast<uint32_t>(p.npad));

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* smem_x = smem;
  uint8_t* smem_w = smem + S * x_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::usable_bytes(p.smem_bytes));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + Cfg::kMaxStages;
  uint64_t* tfull_bar = bars + 2 * Cfg::kMaxStages;
  uint64_t* tempty_bar = bars + 2 * Cfg::kMaxStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * Cfg::kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_items = p.tiles * p.split;  // item = tile * split + K part; with split > 1 the grid has one CTA per item
  const int crank = (p.split > 1) ? static_cast<int>(ptx::cluster_ctarank()) : 0;

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
    ptx::tma_prefetch_desc(&tmap_x);
    ptx::tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::griddep_launch_dependents();  // the next kernel may begin its own set-up; it waits for us before reading

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint32_t tx_bytes = static_cast<uint32_t>(p.x_box_rows) * kDecBK * 2 + kWBytes;
      auto load_w = [&](int stage, int tile, int kb) {
        uint8_t* sw = smem_w + stage * kWBytes;
        const int n0 = tile * kDecTile;
        ptx::tma_load_2d(sw, &tmap_w, &full_bar[stage], n0, kb * kDecBK);
        ptx::tma_load_2d(sw + 8192, &tmap_w, &full_bar[stage], n0 + 64, kb * kDecBK);
        if (EPI == 2) {
          ptx::tma_load_2d(sw + 16384, &tmap_w, &full_bar[stage], p.up_col_off + n0, kb * kDecBK);
          ptx::tma_load_2d(sw + 24576, &tmap_w, &full_bar[stage], p.up_col_off + n0 + 64, kb * kDecBK);
        }
      };
      auto load_x = [&](int stage, int kb) {
        ptx::tma_load_2d(smem_x + stage * x_stage, &tmap_x, &full_bar[stage], kb * kDecBK, 0);
      };
      // first item: with static weights its first S weight tiles are requested before the dependency wait
      int npre = 0;
      {
        const int w = blockIdx.x;
        if (p.static_w && w < num_items) {
          const int tile = w / p.split, part = w - tile * p.split;
          const int kb_beg = part * p.kb_per_split, kb_end = min(p.num_kb, kb_beg + p.kb_per_split);
          npre = min(S, kb_end - kb_beg);
          for (int i = 0; i < npre; ++i) {
            ptx::mbar_expect_tx(&full_bar[i], tx_bytes);
            load_w(i, tile, kb_beg + i);
          }
        }
      }
      ptx::griddep_wait();  // activations (and, unless static, weights) come from earlier kernels
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        const int tile = w / p.split, part = w - tile * p.split;
        const int kb_beg = part * p.kb_per_split, kb_end = min(p.num_kb, kb_beg + p.kb_per_split);
        for (int kb = kb_beg; kb < kb_end; ++kb) {
          if (npre > 0) {
            // weight tile already in flight for this stage
            load_x(stage, kb);
            --npre;
          } else {
            if (!ptx::bounded_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
              if (p.status) atomicCAS(p.status, 0, kStatusTimeoutProducer);
              ok = false;
              break;
            }
            ptx::mbar_expect_tx(&full_bar[stage], tx_bytes);
            load_x(stage, kb);
            load_w(stage, tile, kb);
          }
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else {
      ptx::griddep_wait();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    ptx::griddep_wait();
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
        const int part = w % p.split;
        const int kb_beg = part * p.kb_per_split, kb_end = min(p.num_kb, kb_beg + p.kb_per_split);
        if (!ptx::bounded_mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * cols);
        for (int kb = kb_beg; kb < kb_end; ++kb) {
          if (!ptx::bounded_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          const uint32_t w_base = ptx::smem_u32(smem_w + stage * kWBytes);
          const uint32_t x_base = ptx::smem_u32(smem_x + stage * x_stage);
#pragma unroll
          for (int k = 0; k < kDecBK / 16; ++k) {
            // W: MN-major, two 64-feature slabs 8192 B apart, 8-K-row groups 1024 B apart; 16 K rows = 2048 B.
            // X: K-major, 128-byte rows, 8-row groups 1024 B apart; 16 K elements = 32 B.
            const uint64_t wdesc = ptx::make_smem_desc(w_base + k * 2048, 8192, 1024, ptx::kLayoutSw128);
            const uint64_t xdesc = ptx::make_smem_desc(x_base + k * 32, 16, 1024, ptx::kLayoutSw128);
            const uint32_t accum = (kb != kb_beg || k != 0) ? 1u : 0u;
            ptx::umma_f16_ss(d_tmem, wdesc, xdesc, idesc, accum);
            if (EPI == 2) {
              const uint64_t udesc = ptx::make_smem_desc(w_base + 16384 + k * 2048, 8192, 1024, ptx::kLayoutSw128);
              ptx::umma_f16_ss(d_tmem + static_cast<uint32_t>(p.npad), udesc, xdesc, idesc, accum);
            }
          }
          ptx::umma_commit(&empty_bar[stage]);
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        ptx::umma_commit(&tfull_bar[acc]);
        if (num_acc == 2) {
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        } else {
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (128 threads)
    ptx::griddep_wait();
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int feat = q * 32 + lane;
    if (p.split == 1) {
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int w = blockIdx.x; w < num_items; w += gridDim.x) {
        const int n = w * kDecTile + feat;
        if (!ptx::bounded_mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) {
          if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          break;
        }
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * cols);
#pragma unroll 1
        for (int c = 0; c < p.M; c += 32) {
          uint32_t v[32];
          float g[32], up[32];
          ptx::tmem_ld_32x32(taddr + c, v);
          if (EPI == 2) {
            uint32_t t[32];
            ptx::tmem_ld_32x32(taddr + p.npad + c, t);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) up[i] = __uint_as_float(t[i]);
          } else {
            ptx::tmem_ld_wait();
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = __uint_as_float(v[i]);
          dec_store32<T, EPI>(p, g, up, n, c, p.M);
        }
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive(&tempty_bar[acc]);
        if (num_acc == 2) {
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        } else {
          acc_phase ^= 1u;
        }
      }
    }
  }

  __syncwarp();  // lanes of the producer / issuer warps rejoin their lane 0 before the warp-aligned barriers
  if (p.split > 1) {
    // ------------------------------------------------------------ cluster reduction (one item per CTA)
    // Landing zone in every CTA, over its (by then dead) pipeline stages:
    //   [source rank][half][token group of 4 within the slice][128 features][4 tokens] fp32
    // Every thread of the cluster executes both barriers, whatever happened in its role loop.
    const int tile = blockIdx.x / p.split;
    const bool epi = warp >= 2;
    const int q = warp & 3, feat = q * 32 + lane;
    const int groups = p.slice >> 2;                             // float4 groups per slice
    const uint32_t src_stride = kHalves * groups * (kDecTile * 16);  // bytes per source rank
    bool acc_ready = false;
    if (epi) {
      acc_ready = ptx::bounded_mbar_wait(&tfull_bar[0], 0, abort_flag);
      if (!acc_ready && p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
      ptx::tc_fence_after_sync();
    }
    // barrier 1: every CTA of the cluster has finished its MMAs, so nobody's stages are read or written any more
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t zone = ptx::smem_u32(smem);
    if (epi && acc_ready) {
      // send every foreign slice of the accumulator to its owner
      for (int h = 0; h < kHalves; ++h) {
#pragma unroll 1
        for (int c = 0; c < p.M; c += 32) {
          uint32_t v[32];
          ptx::tmem_ld_32x32(taddr + h * p.npad + c, v);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t0 = c + 4 * j;
            if (t0 < p.M) {
              const int owner = t0 / p.slice;
              if (owner != crank) {
                const int grp = (t0 - owner * p.slice) >> 2;
                const uint32_t local = zone + static_cast<uint32_t>(crank) * src_stride +
                                       static_cast<uint32_t>((h * groups + grp) * kDecTile + feat) * 16u;
                ptx::st_shared_cluster_v4(ptx::mapa_shared(local, static_cast<uint32_t>(owner)), v[4 * j], v[4 * j + 1],
                                          v[4 * j + 2], v[4 * j + 3]);
              }
            }
          }
        }
      }
    }
    // barrier 2: the slices are in place
    ptx::cluster_arrive_release();
    ptx::cluster_wait_acquire();
    if (epi && acc_ready) {
      const int t_beg = crank * p.slice;
      const int t_end = min(p.M, t_beg + p.slice);
      const int n = tile * kDecTile + feat;
#pragma unroll 1
      for (int c = t_beg; c < t_end; c += 32) {
        float g[32], up[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) g[i] = up[i] = 0.f;
        for (int h = 0; h < kHalves; ++h) {
          uint32_t own[32];
          ptx::tmem_ld_32x32(taddr + h * p.npad + c, own);
          ptx::tmem_ld_wait();
          for (int s = 0; s < p.split; ++s) {  // rank order: the sum does not depend on timing
            if (s == crank) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (h == 0) g[i] += __uint_as_float(own[i]);
                else up[i] += __uint_as_float(own[i]);
              }
            } else {
              const uint8_t* zs = smem + static_cast<size_t>(s) * src_stride;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (c + 4 * j < t_end) {
                  const int grp = (c + 4 * j - t_beg) >> 2;
                  const float4 f = *reinterpret_cast<const float4*>(
                      zs + static_cast<size_t>((h * groups + grp) * kDecTile + feat) * 16);
                  if (h == 0) {
                    g[4 * j] += f.x; g[4 * j + 1] += f.y; g[4 * j + 2] += f.z; g[4 * j + 3] += f.w;
                  } else {
                    up[4 * j] += f.x; up[4 * j + 1] += f.y; up[4 * j + 2] += f.z; up[4 * j + 3] += f.w;
                  }
                }
              }
            }
          }
        }
        dec_store32<T, EPI>(p, g, up, n, c, t_end);
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, tmem_cols);
  }
}

template <typename T, int EPI>
static cudaError_t launch_dec(const CUtensorMap& tx, const CUtensorMap& tw, DecGemmParams& p, int split_hint, int sms,
                              cudaStream_t stream) {
  auto kern = gemm_decode_kernel<T, EPI>;
  // per device: the shared-memory attribute; the cluster occupancy is the same on every GPU of a box (the first
  // device to get here fills the table under the set-up lock)
  static PerDeviceOnce once;
  static int max_clusters[2][kDecMaxSplit + 1];
  static int occ_env = -1;
  cudaError_t e0 = once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DecCfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    if (occ_env < 0) {
      for (int s = 2; s <= kDecMaxSplit; ++s) {
        max_clusters[0][s] = max_active_clusters(kern, dim3(kDecThreads), DecCfg::kSmemBytes, s);
        max_clusters[1][s] = max_active_clusters(kern, dim3(kDecThreads), DecCfg::kSmemBytesHalf, s);
      }
      const char* env = std::getenv("BLITZ_DECODE_OCC");
      occ_env = env ? std::atoi(env) : 0;
    }
    return cudaSuccess;
  });
  if (e0 != cudaSuccess) return e0;
  const int halves = EPI == 2 ? 2 : 1;
  const int stage_bytes = DecCfg::x_stage_bytes(p.npad) + halves * kDecTile * kDecBK * 2;
  // One CTA per SM.  BLITZ_DECODE_OCC=2 runs two CTAs per SM on half the shared memory each (so that one CTA's
  // set-up or reduction overlaps the other's weight stream); measured on B200 it changes nothing (15.2 vs 15.3 us
  // at M=16, N=6144, K=4096), so it stays an experiment switch.
  int occ = 1;
  if (occ_env == 1 || occ_env == 2) occ = occ_env;
  if (DecCfg::num_stages(p.npad, halves * kDecTile * kDecBK * 2, DecCfg::kSmemBytesHalf) < 2) occ = 1;
  p.smem_bytes = occ == 2 ? DecCfg::kSmemBytesHalf : DecCfg::kSmemBytes;
  // K split = cluster size: as many CTAs per tile as it takes to put (nearly) every SM to work, provided all
  // clusters are resident at once and the landing zone of the reduction fits over the pipeline stages
  int split = split_hint > 0 ? split_hint : (sms * occ) / p.tiles;
  if (split > kDecMaxSplit) split = kDecMaxSplit;
  if (split > p.num_kb) split = p.num_kb;
  const int stage_area = DecCfg::num_stages(p.npad, halves * kDecTile * kDecBK * 2, p.smem_bytes) * stage_bytes;
  while (split > 1) {
    const int slice = (((p.M + split - 1) / split) + 31) & ~31;
    const int64_t zone = (int64_t)split * halves * (slice / 4) * kDecTile * 16;
    const int kbs = (p.num_kb + split - 1) / split;
    const bool every_rank_has_work = (int64_t)kbs * (split - 1) < p.num_kb;
    if (p.tiles <= max_clusters[occ - 1][split] && zone <= stage_area && every_rank_has_work) break;
    --split;
  }
  if (split < 1) split = 1;
  p.split = split;
  p.kb_per_split = (p.num_kb + split - 1) / split;
  p.slice = (((p.M + split - 1) / split) + 31) & ~31;
  int grid;
  if (split > 1) {
    grid = p.tiles * split;
  } else {
    grid = p.tiles < sms * occ ? p.tiles : sms * occ;
  }
  return launch_pdl_cluster(kern, dim3(grid), dim3(kDecThreads), (size_t)p.smem_bytes, (unsigned)split, stream, tx, tw, p);
}

}  // namespace blitz

extern "C" {

// Programmatic dependent launch for every kernel of the library: 1 = on (default; BLITZ_PDL=0 in the
// environment turns it off at start-up), 0 = plain stream order.  Takes effect for launches (and graph
// captures) made afterwards.
void blitz_set_pdl(int on) { blitz::pdl_flag() = on ? 1 : 0; }
int blitz_get_pdl() { return blitz::pdl_flag(); }

// Whether blitz_gemm_decode takes this problem (the general GEMM handles everything else).
int blitz_gemm_decode_supported(int M, int N, int K, int b_layout, int epilogue) {
  return M >= 1 && M <= 256 && b_layout == 0 && epilogue >= 0 && epilogue <= 2 && (N & 7) == 0 && (K & 7) == 0;
}

// C = X W (+R | silu-mul).  X [M, lda>=K], W [K, ldb>=columns] row-major, C/R [M, ldc>=N].  dtype 0 fp16, 1 bf16.
// epilogue 0 store, 1 add R (C may be R), 2 silu(gate)*up with the up columns starting at up_col_off.
// static_w != 0 promises that W was not written by kernels still running in this stream (weights), which lets
// the kernel start streaming it before its predecessor has finished.  split_hint: 0 = choose, 1 = no K split,
// n = at most n CTAs (a cluster) per 128-feature tile.
// Returns a cudaError_t value, -1 for arguments it cannot take, -2 when the TMA encoder is missing.
int blitz_gemm_decode(const void* X, int64_t lda, const void* W, int64_t ldb, void* C, int64_t ldc, const void* R,
                      int M, int N, int K, int epilogue, int up_col_off, int dtype, int static_w, int split_hint,
                      int* status, cudaStream_t stream) {
  using namespace blitz;
  if (!blitz_gemm_decode_supported(M, N, K, 0, epilogue)) return -1;
  if ((lda & 7) || (ldb & 7) || (epilogue == 2 && (up_col_off & 7))) return -1;
  const int sms = device_sm_count();
  DecGemmParams p;
  p.C = C;
  p.R = R;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.npad = (M + 15) & ~15;
  p.x_box_rows = (M + 7) & ~7;
  p.up_col_off = up_col_off;
  p.num_kb = (K + kDecBK - 1) / kDecBK;
  p.tiles = (N + kDecTile - 1) / kDecTile;
  p.static_w = static_w;
  p.status = status;

  CUtensorMap tx, tw;
  if (!get_tmap_2d(&tx, X, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kDecBK, (uint32_t)p.x_box_rows)) return -2;
  const int w_cols = epilogue == 2 ? up_col_off + N : N;
  if (!get_tmap_2d(&tw, W, (uint64_t)w_cols, (uint64_t)K, (uint64_t)ldb * 2, 64, kDecBK)) return -2;

  cudaError_t e;
  if (dtype == 1) {
    e = epilogue == 2   ? launch_dec<__nv_bfloat16, 2>(tx, tw, p, split_hint, sms, stream)
        : epilogue == 1 ? launch_dec<__nv_bfloat16, 1>(tx, tw, p, split_hint, sms, stream)
                        : launch_dec<__nv_bfloat16, 0>(tx, tw, p, split_hint, sms, stream);
  } else {
    e = epilogue == 2   ? launch_dec<__half, 2>(tx, tw, p, split_hint, sms, stream)
        : epilogue == 1 ? launch_dec<__half, 1>(tx, tw, p, split_hint, sms, stream)
                        : launch_dec<__half, 0>(tx, tw, p, split_hint, sms, stream);
  }
  return static_cast<int>(e);
}

}  // extern "C"
