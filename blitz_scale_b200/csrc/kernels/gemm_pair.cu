// Paired-SM tcgen05 GEMM with stream-K scheduling, for activation blocks of up to 256 rows against a
// weight matrix in the serving layout (and, 256 rows at a time, for taller A as well).
//
//   C[M,N] = A[M,K] * W[K,N]      W "in,out" (N contiguous), 16-bit, fp32 accumulation in TMEM
//
// Why a pair.  At 129..256 rows a decode GEMM sits on the ridge of the roofline: the weight stream and the
// tensor pipe take the same time, and every weight tile drags an activation tile of its own size out of L2.
// Measured on B200, the sum of those two streams is what bounds such a GEMM (the L2 -> SM fabric delivers about
// 10 TB/s to all SMs together, the weight stream alone could run at 6.5), and a single CTA is additionally bound
// by shared-memory operand reads of a 128-row tcgen05.mma.  Two CTAs of a 2-wide cluster issue ONE
// `tcgen05.mma.cta_group::2` of 256 rows: each CTA keeps 128 rows of A and half of the N columns of the weight
// tile, so per SM the operand reads and the activation re-read are halved.  With two accumulators per pair
// (a "super tile" of 2 x 256 columns that shares every activation tile) the re-read halves again.
// Each CTA loads only its own halves with plain per-CTA TMA (no cluster multicast anywhere); the bytes of both
// are counted on the even CTA's barrier, whose elected thread issues the instructions for the pair.
//
// Scheduling.  Work is cut into units of (super tile, 64-wide K block); pair p takes the units
// [p*upp, (p+1)*upp) in order, so all pairs finish together whatever the tile count (stream-K).  A pair whose
// range starts inside a super tile contributes fp32 partials for it (its FIRST piece of work: written to
// scratch, one counter per tile bumped); the pair that holds the first K block owns the tile and finishes it as
// its LAST piece of work: it waits (bounded) for the counter, pulls the partials into the by then idle pipeline
// stages with the copy engine (in rounds of columns when they do not fit at once), sums in ascending pair order
// (deterministic) and runs the epilogue.  Owners therefore rarely wait: their contributors started with the
// shared tile.
//
// Epilogue.  What follows the last UMMA of a pair is exposed time.  Eight warps (two per TMEM lane quarter) read
// the accumulator, apply store / residual add (C may alias R) / silu(gate)*up (the even CTA loads gate columns,
// the odd CTA up columns, so a thread finds gate and up of one output element in its own TMEM lane), write
// 128-byte-swizzled 32 x 64 boxes to a staging area and hand them to TMA stores: a thread-per-row epilogue would
// issue one 16-byte store per lane into 32 different rows, which the load/store unit serialises.  Residual values
// are requested before the wait for the accumulator.
// Replaces cuBLAS at these sizes (src/util/cublas_wrapper.h:31-141 of the reference; call sites
// src/layer/attn.h:137-215, src/layer/glu.h:109-136, src/layer/lm_head.h:89-98).
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner (+ UMMA issuer in the even CTA),
// warps 2..9 = epilogue (TMEM lane quarter = warp % 4, two warps per quarter).
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include <cstdlib>
#include <type_traits>

namespace blitz {

constexpr int kPairEpiWarps = 8;
constexpr int kPairThreads = 64 + 32 * kPairEpiWarps;
constexpr int kPairSlabsMax = 4;     // 64-column slabs of one tile's output (256 columns)
constexpr int kPairBK = 64;
constexpr int kPairRows = 128;       // rows of A per CTA; the pair covers 256
constexpr int kPairMaxStages = 12;
constexpr int kPairMaxContrib = 6;   // partial contributions one tile may receive
constexpr int kPairStagingBytes = 2 * 4 * 4096;  // two buffers of four 32-row x 128-byte boxes (one per lane quarter)
constexpr int kPairFinalStagingBytes = kPairSlabsMax * 4 * 4096;  // a pair's last tile: one box per slab and quarter, in the idle stages

struct PairParams {
  const void* R;
  int64_t ldc;
  int M, N, K;
  int bnf;         // UMMA N = accumulator columns of a tile (128 or 256)
  int nacc;        // accumulators (adjacent tiles sharing the activation tiles) per pair: 1 or 2
  int out_cols;    // output columns of a tile: bnf, or bnf / 2 with silu_mul
  int up_col_off;  // silu_mul: column of W where the "up" half starts
  int num_kb, tiles_m, tiles_n, supers_n;  // tiles_n = column tiles, supers_n = ceil(tiles_n / nacc)
  int upp;         // units (super tile x K block) per CTA pair
  int split;       // 0 = stream-K; 2..4 = every tile is cut into that many equal K parts, one pair each (nacc = 1)
  int total_units;
  int static_b;    // W is not written by kernels still running in this stream
  float* ws;       // partials: [pair][cta rank][accumulator][bnf / 4][128 rows][4] fp32
  uint32_t* flags; // [tile][cta rank][4]: contributions landed (stream-K: word 0; split mode: one word per part); zero between launches
  int* status;
  unsigned long long* trace;  // profiling aid (null in production): 16 globaltimer stamps per CTA, see blitz_gemm_pair_set_trace
};

// Stamp slots of the optional per-CTA timeline.
enum PairTrace : int { kTrStart = 0, kTrSetupDone = 1, kTrFirstFull = 2, kTrLastCommit = 3, kTrLastTfull = 4,
                       kTrEpilogueDone = 5, kTrDepWaitDone = 6, kTrEnd = 7, kTrParked = 8, kTrFlagsSeen = 9,
                       kTrLanded = 10, kTrStoresIssued = 11, kTrSlots = 16 };
__device__ __forceinline__ void pair_stamp(const PairParams& p, int slot) {
  if (p.trace) p.trace[static_cast<size_t>(blockIdx.x) * kTrSlots + slot] = ptx::globaltimer_ns();
}

struct PairCfg {
  static constexpr int kSmemBytes = 227 * 1024;
  static constexpr int kBarrierBytes = (2 * kPairMaxStages + 9) * 8 + 32;
  // stages | staging (1 KB aligned) | barriers
  static constexpr int kStageArea = (kSmemBytes - 1024 - kBarrierBytes - kPairStagingBytes) & ~1023;
  __host__ __device__ static int stage_bytes(int bnf, int nacc) { return kPairRows * kPairBK * 2 + nacc * bnf * kPairBK; }
  __host__ __device__ static int num_stages(int bnf, int nacc) {
    const int s = kStageArea / stage_bytes(bnf, nacc);
    return s > kPairMaxStages ? kPairMaxStages : s;
  }
  // accumulator buffers in TMEM: two sets (epilogue of one piece of work overlaps the UMMAs of the next) when they fit
  __host__ __device__ static int acc_bufs(int bnf, int nacc) { return 2 * nacc * bnf <= 512 ? 2 : 1; }
};

template <typename T>
__device__ __forceinline__ uint32_t pair_pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pair_pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pair_pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float2 pair_unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 pair_unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <>
__device__ __forceinline__ float2 pair_unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
// fast-math sigmoid: the epilogue after the last UMMA is exposed time, and an IEEE division per element is a long
// dependent chain on a handful of warps
__device__ __forceinline__ float pair_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// 32 consecutive output columns of one row -> four 16-byte chunks.  EPI: 0 store, 1 add residual (its 32 values
// come in `res`, read before the accumulator was waited for), 2 silu(g) * u.
template <typename T, int EPI>
__device__ __forceinline__ void pair_convert32(const float (&g)[32], const float (&u)[32], const uint4 (&res)[4],
                                               uint4 (&out4)[4]) {
  uint32_t out[16];
  if (EPI == 2) {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      out[i] = pair_pack2<T>(pair_silu(g[2 * i]) * u[2 * i], pair_silu(g[2 * i + 1]) * u[2 * i + 1]);
  } else if (EPI == 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t rr[4] = {res[j].x, res[j].y, res[j].z, res[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = pair_unpack2<T>(rr[i]);
        out[j * 4 + i] = pair_pack2<T>(g[j * 8 + 2 * i] + f.x, g[j * 8 + 2 * i + 1] + f.y);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = pair_pack2<T>(g[2 * i], g[2 * i + 1]);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) out4[j] = make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
}

template <typename T, int EPI>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const PairParams p) {
  using Cfg = PairCfg;
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  const int bnf = p.bnf, half = bnf >> 1, nacc = p.nacc;
  const int S = Cfg::num_stages(bnf, nacc);
  const int stage_bytes = Cfg::stage_bytes(bnf, nacc);
  const int acc_bufs = Cfg::acc_bufs(bnf, nacc);
  const uint32_t idesc = ptx::make_idesc_f16(kFmt, 0u, 1u, 2 * kPairRows, static_cast<uint32_t>(bnf));
  const uint32_t tmem_cols = static_cast<uint32_t>(acc_bufs * nacc * bnf);  // 256 or 512

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* staging = smem + Cfg::kStageArea;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kPairStagingBytes);
  uint64_t* full_bar = bars;                                   // [S]  used in the even CTA: bytes of both CTAs
  uint64_t* empty_bar = bars + kPairMaxStages;                 // [S]  per CTA: stage released by the pair's UMMAs
  uint64_t* tfull_bar = bars + 2 * kPairMaxStages;             // [4]  per CTA: accumulator (buffer, index) complete
  uint64_t* tempty_bar = bars + 2 * kPairMaxStages + 4;        // [4]  used in the even CTA: the 16 epilogue warps of the pair drained it
  uint64_t* fix_bar = bars + 2 * kPairMaxStages + 8;           // partials of other pairs have landed in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPairMaxStages + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();  // 0 = even CTA (issues the UMMAs), 1 = odd CTA
  const int pair = blockIdx.x >> 1;
  const int u_beg = pair * p.upp;
  const int u_end = min(p.total_units, u_beg + p.upp);
  if (threadIdx.x == 0) pair_stamp(p, kTrStart);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) {
      ptx::mbar_init(&full_bar[i], 1);
      ptx::mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 4; ++i) {
      ptx::mbar_init(&tfull_bar[i], 1);
      ptx::mbar_init(&tempty_bar[i], 2 * kPairEpiWarps);
    }
    ptx::mbar_init(fix_bar, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap_a);
    ptx::tma_prefetch_desc(&tmap_b);
    ptx::tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, tmem_cols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  // both CTAs have initialised their barriers before either signals the other's
  ptx::cluster_arrive_release();
  ptx::cluster_wait_acquire();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  ptx::griddep_launch_dependents();
  if (threadIdx.x == 0) pair_stamp(p, kTrSetupDone);

  const int a_bytes = kPairRows * kPairBK * 2;
  const int b_bytes = bnf * kPairBK;  // this CTA's half of one weight tile: (bnf / 2) columns x 64 K rows x 2 bytes

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs, own halves)
    if (lane == 0) {
      const uint32_t full0 = ptx::mapa_shared(ptx::smem_u32(full_bar), 0u);  // the even CTA's full barriers
      const uint32_t tx_bytes = 2u * static_cast<uint32_t>(stage_bytes);
      auto load_b = [&](int stage, int st, int kb) {
        const int n_super = st / p.tiles_m;
        for (int a = 0; a < nacc; ++a) {
          const int nt = n_super * nacc + a;
          uint8_t* sb = smem + stage * stage_bytes + a_bytes + a * b_bytes;
          int col;
          if (EPI == 2) col = (rank == 0 ? 0 : p.up_col_off) + nt * half;
          else col = nt * bnf + static_cast<int>(rank) * half;
          for (int s = 0; s < half / 64; ++s)
            ptx::tma_load_2d_pair(sb + s * 8192, &tmap_b, full0 + 8u * stage, col + s * 64, kb * kPairBK);
        }
      };
      auto load_a = [&](int stage, int st, int kb) {
        const int m0 = (st % p.tiles_m) * (2 * kPairRows) + static_cast<int>(rank) * kPairRows;
        ptx::tma_load_2d_pair(smem + stage * stage_bytes, &tmap_a, full0 + 8u * stage, kb * kPairBK, m0);
      };
      int st = u_beg / p.num_kb, kb = u_beg - st * p.num_kb;
      // with static weights the first stages' weight tiles are requested before the dependency wait
      int npre = 0;
      if (p.static_b) {
        npre = min(S, u_end - u_beg);
        int t2 = st, k2 = kb;
        for (int i = 0; i < npre; ++i) {
          if (rank == 0) ptx::mbar_expect_tx(&full_bar[i], tx_bytes);
          load_b(i, t2, k2);
          if (++k2 == p.num_kb) { k2 = 0; ++t2; }
        }
      }
      ptx::griddep_wait();
      pair_stamp(p, kTrDepWaitDone);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = u_beg; u < u_end; ++u) {
        if (npre > 0) {
          load_a(stage, st, kb);
          --npre;
        } else {
          if (!ptx::bounded_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          if (rank == 0) ptx::mbar_expect_tx(&full_bar[stage], tx_bytes);
          load_a(stage, st, kb);
          load_b(stage, st, kb);
        }
        if (++stage == S) { stage = 0; phase ^= 1u; }
        if (++kb == p.num_kb) { kb = 0; ++st; }
      }
      // drain: the releases of the last stages are remote barrier signals; take them before this CTA may exit
      if (ok) {
        const int tail = min(S, u_end - u_beg);
        for (int i = 0; i < tail; ++i) {
          if (!ptx::bounded_mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) break;
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
      }
    } else {
      ptx::griddep_wait();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer (even CTA only)
    ptx::griddep_wait();
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      int u = u_beg;
      while (u < u_end && ok) {
        const int st = u / p.num_kb, kb_beg = u - st * p.num_kb;
        const int len = min(p.num_kb - kb_beg, u_end - u);
        for (int i = 0; i < len && ok; ++i) {
          if (!ptx::bounded_mbar_wait(&full_bar[stage], phase, abort_flag)) {
            if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
            ok = false;
            break;
          }
          ptx::tc_fence_after_sync();
          if (u == u_beg && i == 0) pair_stamp(p, kTrFirstFull);
          const uint32_t a_base = ptx::smem_u32(smem + stage * stage_bytes);
          for (int a = 0; a < nacc; ++a) {
            const int slot = buf * nacc + a;
            if (i == 0) {
              // the epilogue drains accumulator 0 first, so its UMMAs start while accumulator 1 is still being read
              if (!ptx::bounded_mbar_wait(&tempty_bar[slot], buf_phase ^ 1u, abort_flag)) {
                if (p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
                ok = false;
                break;
              }
              ptx::tc_fence_after_sync();
            }
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(slot * bnf);
            const uint32_t b_base = a_base + a_bytes + a * b_bytes;
#pragma unroll
            for (int k = 0; k < kPairBK / 16; ++k) {
              // A: K-major, 128-byte rows, 8-row groups 1024 B apart; 16 K elements = 32 B.
              // W: N-major slabs of 64 columns 8192 B apart, 8-K-row groups 1024 B apart; 16 K rows = 2048 B.
              const uint64_t adesc = ptx::make_smem_desc(a_base + k * 32, 16, 1024, ptx::kLayoutSw128);
              const uint64_t bdesc = ptx::make_smem_desc(b_base + k * 2048, 8192, 1024, ptx::kLayoutSw128);
              ptx::umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (i != 0 || k != 0) ? 1u : 0u);
            }
          }
          if (!ok) break;
          ptx::umma_commit_pair(&empty_bar[stage], 3);
          if (++stage == S) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        for (int a = 0; a < nacc; ++a) ptx::umma_commit_pair(&tfull_bar[buf * nacc + a], 3);
        if (acc_bufs == 2) {
          buf ^= 1;
          if (buf == 0) buf_phase ^= 1u;
        } else {
          buf_phase ^= 1u;
        }
        u += len;
      }
      pair_stamp(p, kTrLastCommit);
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (256 threads, named barrier 2;
    // the two warps of lane quarter q also meet on named barrier 3 + q)
    ptx::griddep_wait();
    const int q = warp & 3;
    const int ch = (warp - 2) >> 2;  // 0 or 1: which 32-column half of every 64-column slab this warp takes
    const int row_in = q * 32 + lane;
    const int epi_tid = threadIdx.x - 64;
    const bool issuer = (ch == 0 && lane == 0);  // issues this quarter's TMA stores
    const uint32_t tempty0 = ptx::mapa_shared(ptx::smem_u32(tempty_bar), 0u);
    const size_t slot_floats = static_cast<size_t>(kPairRows) * bnf;
    const uint32_t slot_bytes = static_cast<uint32_t>(slot_floats) * 4u;
    const int area = S * stage_bytes;
    const int land_area = area - kPairFinalStagingBytes;  // partials land below the final tile's staging boxes
    const int nslab = p.out_cols / 64;                    // 1, 2 or 4 slabs of 64 output columns per tile
    const int split = p.split;                            // 0: stream-K; 2..4: K parts per tile, one per pair
    int buf = 0;
    uint32_t buf_phase = 0, fix_phase = 0;
    int u = u_beg;
    bool alive = true;
    while (u < u_end && alive) {
      const int st = u / p.num_kb, kb_beg = u - st * p.num_kb;
      const int len = min(p.num_kb - kb_beg, u_end - u);
      const int row0 = (st % p.tiles_m) * (2 * kPairRows) + static_cast<int>(rank) * kPairRows;
      const int row = row0 + row_in;
      const bool row_ok = row < p.M;
      const bool quarter_ok = row0 + q * 32 < p.M;  // the same for both warps of a quarter
      const bool last_piece = (u + len >= u_end);
      for (int a = 0; a < nacc && alive; ++a) {
        const int slot = buf * nacc + a;
        const int nt = (st / p.tiles_m) * nacc + a;  // column tile of this accumulator
        const int tile = nt * p.tiles_m + (st % p.tiles_m);
        const int n0 = nt * p.out_cols;
        const bool tile_valid = nt < p.tiles_n;
        uint32_t* tile_flags = p.flags + (static_cast<size_t>(tile) * 2 + rank) * 4;
        // Slabs of this tile that this pair finalises.  Stream-K: all of them if it holds the tile's first K block,
        // none otherwise.  Split mode: the pairs of a tile finish together, so each finalises its share of the
        // slabs (slab i belongs to part i mod split) and sends the others' columns to them.
        const int part = split ? kb_beg / p.upp : 0;
        uint32_t own_mask = 0;
        if (tile_valid) {
          if (split) {
            for (int i = 0; i < nslab; ++i)
              if (i % split == part) own_mask |= 1u << i;
          } else if (kb_beg == 0) {
            own_mask = (1u << nslab) - 1u;
          }
        }
        const int n_own = __popc(own_mask);
        uint4 rpre[kPairSlabsMax][4];
        if (EPI == 1) {
          const T* Rp = reinterpret_cast<const T*>(p.R) + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
          for (int i = 0; i < kPairSlabsMax; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + i * 64 + ch * 32 + j * 8;
              rpre[i][j] = make_uint4(0, 0, 0, 0);
              if (((own_mask >> i) & 1u) && row_ok && col < p.N) rpre[i][j] = *reinterpret_cast<const uint4*>(Rp + col);
            }
          }
        }
        if (!ptx::bounded_mbar_wait(&tfull_bar[slot], buf_phase, abort_flag)) {
          if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          alive = false;
          break;
        }
        ptx::tc_fence_after_sync();
        if (epi_tid == 0 && last_piece && a == nacc - 1) pair_stamp(p, kTrLastTfull);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(slot * bnf);

        // ---- 1. park the fp32 partials of the columns other pairs finalise
        if (tile_valid && (split != 0 || kb_beg != 0)) {
          float* pslot = p.ws + ((static_cast<size_t>(pair) * 2 + rank) * nacc + a) * slot_floats +
                         static_cast<size_t>(row_in) * 4;
#pragma unroll 1
          for (int c = ch * 32; c < bnf; c += 64) {
            if (split != 0 && ((own_mask >> (c >> 6)) & 1u)) continue;  // split mode: own slabs stay in TMEM
            uint32_t v[32];
            ptx::tmem_ld_32x32(taddr + c, v);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              __stcg(reinterpret_cast<uint4*>(pslot + static_cast<size_t>(c / 4 + j) * (kPairRows * 4)),
                     make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
          }
          __threadfence();
          asm volatile("bar.sync 2, 256;" ::: "memory");
          if (epi_tid == 0) {
            if (split == 0) {
              ptx::red_add_release_gpu(tile_flags, 1u);
            } else {
              for (int g = 0; g < split; ++g)
                if (g != part) ptx::red_add_release_gpu(tile_flags + g, 1u);
            }
            if (last_piece) pair_stamp(p, kTrParked);
          }
        }
        if (own_mask == 0) {
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(tempty0 + 8u * slot);
          continue;
        }

        // ---- 2. partials this pair receives.  Stream-K: from the pairs that hold the tile's later K blocks, for all
        // columns, in `rounds` groups of slabs when they do not fit the landing area at once.  Split mode: from the
        // other parts' pairs, for the own slabs only.  Either way this is the pair's last piece of work and its
        // UMMAs have completed, so the pipeline stages are free to receive them.
        int n_contrib;
        if (split) {
          n_contrib = split - 1;
        } else {
          const int last_pair = (st * p.num_kb + p.num_kb - 1) / p.upp;
          n_contrib = (len == p.num_kb) ? 0 : last_pair - pair;
        }
        int rounds = 1;
        if (!split)
          while (rounds < nslab && static_cast<int64_t>(n_contrib) * (slot_bytes / rounds) > land_area) rounds <<= 1;
        const uint32_t round_bytes = slot_bytes / rounds;  // stream-K: per contributor and round
        const int slabs_per_round = nslab / rounds;
        const uint32_t slab_bytes = 64u * kPairRows * 4u;  // split mode: one slab of one contributor
        bool fix_ok = true;
        if (n_contrib > 0) {
          if (epi_tid == 0) {
            const int64_t need = split ? static_cast<int64_t>(n_contrib) * n_own * slab_bytes
                                       : static_cast<int64_t>(n_contrib) * round_bytes;
            if (need > land_area || !last_piece) {
              if (p.status) atomicCAS(p.status, 0, kStatusTooLarge);
              *abort_flag = 1;
            } else if (!ptx::bounded_flag_wait_ge_gpu(tile_flags + part, static_cast<uint32_t>(n_contrib),
                                                      ptx::kDefaultWaitNs)) {
              if (p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
              *abort_flag = 1;
            } else {
              tile_flags[part] = 0u;  // ready for the next launch
            }
            pair_stamp(p, kTrFlagsSeen);
          }
          asm volatile("bar.sync 2, 256;" ::: "memory");
          fix_ok = (*abort_flag == 0);
        }

        // ---- 3. finalise the own slabs: accumulate, convert, stage 32 x 64 boxes, TMA-store them
        if (fix_ok) {
          // staging boxes: the last piece of work has a box per slab in the idle pipeline stages (no waiting);
          // earlier pieces share the two dedicated buffers and flush after two slabs
          uint8_t* boxes = last_piece ? smem + land_area : staging;
          const int nbuf = last_piece ? kPairSlabsMax : 2;
          if (quarter_ok) {
            if (issuer) ptx::tma_store_wait_read<0>();  // boxes of the previous tile have been read out
            asm volatile("bar.sync %0, 64;" ::"r"(3 + q) : "memory");
          }
          uint32_t staged = 0;  // slabs staged and not yet handed to TMA
          int own_idx = 0;      // index of the current slab among the own ones
#pragma unroll
          for (int i = 0; i < kPairSlabsMax; ++i) {
            if (((own_mask >> i) & 1u) && n0 + i * 64 < p.N) {
              if (n_contrib > 0 && (split ? own_idx == 0 : (i % slabs_per_round) == 0)) {
                const int r = split ? 0 : i / slabs_per_round;
                if (r > 0) asm volatile("bar.sync 2, 256;" ::: "memory");  // everyone has read the previous round
                if (epi_tid == 0) {
                  ptx::fence_proxy_async_all();  // partials were written with ordinary stores; the copy engine reads them
                  if (split) {
                    ptx::mbar_expect_tx(fix_bar, static_cast<uint32_t>(n_contrib * n_own) * slab_bytes);
                    int j = 0;
                    for (int g = 0; g < split; ++g) {
                      if (g == part) continue;
                      const float* src = p.ws + (static_cast<size_t>(pair - part + g) * 2 + rank) * slot_floats;
                      int k = 0;
                      for (int i2 = 0; i2 < nslab; ++i2) {
                        if (!((own_mask >> i2) & 1u)) continue;
                        ptx::bulk_load_1d(smem + static_cast<size_t>(j * n_own + k) * slab_bytes,
                                          src + static_cast<size_t>(i2) * 64 * kPairRows, slab_bytes, fix_bar);
                        ++k;
                      }
                      ++j;
                    }
                  } else {
                    ptx::mbar_expect_tx(fix_bar, static_cast<uint32_t>(n_contrib) * round_bytes);
                    for (int j = 0; j < n_contrib; ++j) {
                      const float* src = p.ws + ((static_cast<size_t>(pair + 1 + j) * 2 + rank) * nacc + a) * slot_floats;
                      uint8_t* dst = smem + static_cast<size_t>(j) * round_bytes;
                      if (EPI == 2) {
                        // gate columns [r * w, (r + 1) * w) and up columns half + the same, w = out_cols / rounds
                        const uint32_t w = static_cast<uint32_t>(p.out_cols / rounds);
                        ptx::bulk_load_1d(dst, src + static_cast<size_t>(r * w) * kPairRows, w * kPairRows * 4, fix_bar);
                        ptx::bulk_load_1d(dst + round_bytes / 2, src + static_cast<size_t>(half + r * w) * kPairRows,
                                          w * kPairRows * 4, fix_bar);
                      } else {
                        ptx::bulk_load_1d(dst, src + static_cast<size_t>(r) * (round_bytes / 4), round_bytes, fix_bar);
                      }
                    }
                  }
                }
                if (!ptx::bounded_mbar_wait(fix_bar, fix_phase, abort_flag)) {
                  if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
                }
                fix_phase ^= 1u;
                if (epi_tid == 0) pair_stamp(p, kTrLanded);
              }
              if (quarter_ok) {
                if (!last_piece && i == 2 && staged != 0) {
                  // the two dedicated buffers are full: hand them over and wait until they have been read out
                  ptx::fence_proxy_async_smem();
                  asm volatile("bar.sync %0, 64;" ::"r"(3 + q) : "memory");
                  if (issuer) {
                    for (int i2 = 0; i2 < 2; ++i2)
                      if ((staged >> i2) & 1u)
                        ptx::tma_store_2d(&tmap_c, boxes + ((i2 & (nbuf - 1)) * 4 + q) * 4096, n0 + i2 * 64, row0 + q * 32);
                    ptx::tma_store_commit();
                    ptx::tma_store_wait_read<0>();
                  }
                  staged = 0;
                  asm volatile("bar.sync %0, 64;" ::"r"(3 + q) : "memory");
                }
                const int c = i * 64 + ch * 32;  // first of this thread's 32 output columns within the tile
                uint32_t v[32];
                float gt[32], up[32];
                ptx::tmem_ld_32x32(taddr + c, v);
                if (EPI == 2) {
                  uint32_t t[32];
                  ptx::tmem_ld_32x32(taddr + half + c, t);
                  ptx::tmem_ld_wait();
#pragma unroll
                  for (int k = 0; k < 32; ++k) up[k] = __uint_as_float(t[k]);
                } else {
                  ptx::tmem_ld_wait();
                }
#pragma unroll
                for (int k = 0; k < 32; ++k) gt[k] = __uint_as_float(v[k]);
                if (n_contrib > 0) {
                  // ascending pair order: the sum does not depend on timing
                  const int c_in = split ? ch * 32 : c - (i / slabs_per_round) * (p.out_cols / rounds);
                  for (int j = 0; j < n_contrib; ++j) {
                    const uint8_t* base = smem + (split ? static_cast<size_t>(j * n_own + own_idx) * slab_bytes
                                                        : static_cast<size_t>(j) * round_bytes) +
                                          static_cast<size_t>(row_in) * 16;
#pragma unroll
                    for (int jj = 0; jj < 8; ++jj) {
                      const float4 f =
                          *reinterpret_cast<const float4*>(base + static_cast<size_t>(c_in / 4 + jj) * (kPairRows * 16));
                      gt[4 * jj] += f.x; gt[4 * jj + 1] += f.y; gt[4 * jj + 2] += f.z; gt[4 * jj + 3] += f.w;
                    }
                    if (EPI == 2) {
                      const uint8_t* ub = base + round_bytes / 2;
#pragma unroll
                      for (int jj = 0; jj < 8; ++jj) {
                        const float4 f =
                            *reinterpret_cast<const float4*>(ub + static_cast<size_t>(c_in / 4 + jj) * (kPairRows * 16));
                        up[4 * jj] += f.x; up[4 * jj + 1] += f.y; up[4 * jj + 2] += f.z; up[4 * jj + 3] += f.w;
                      }
                    }
                  }
                }
                uint4 o4[4];
                pair_convert32<T, EPI>(gt, up, rpre[i], o4);
                // 128-byte rows, 16-byte chunks XOR-swizzled by row: the layout the TMA store expects
                uint8_t* rowp = boxes + ((i & (nbuf - 1)) * 4 + q) * 4096 + lane * 128;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  *reinterpret_cast<uint4*>(rowp + (((ch * 4 + j) ^ (lane & 7)) << 4)) = o4[j];
                staged |= 1u << i;
              }
              ++own_idx;
            }
          }
          if (quarter_ok && staged != 0) {
            ptx::fence_proxy_async_smem();
            asm volatile("bar.sync %0, 64;" ::"r"(3 + q) : "memory");
            if (issuer) {
#pragma unroll
              for (int i2 = 0; i2 < kPairSlabsMax; ++i2)
                if ((staged >> i2) & 1u)
                  ptx::tma_store_2d(&tmap_c, boxes + ((i2 & (nbuf - 1)) * 4 + q) * 4096, n0 + i2 * 64, row0 + q * 32);
              ptx::tma_store_commit();
              if (epi_tid == 0 && last_piece) pair_stamp(p, kTrStoresIssued);
            }
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(tempty0 + 8u * slot);
      }
      if (acc_bufs == 2) {
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1u;
      } else {
        buf_phase ^= 1u;
      }
      u += len;
    }
    if (issuer) ptx::tma_store_wait<0>();  // the staged boxes have been written out before the CTA may exit
    if (epi_tid == 0) pair_stamp(p, kTrEpilogueDone);
  }

  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  // neither CTA leaves (or frees TMEM) while its partner may still signal its barriers or read its tiles
  ptx::cluster_arrive_release();
  ptx::cluster_wait_acquire();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc_pair(tmem_base, tmem_cols);
  }
  if (threadIdx.x == 0) pair_stamp(p, kTrEnd);
}

static unsigned long long* g_pair_trace = nullptr;

// Pairs that can be resident at once, per device (also raises the kernel's shared-memory limit there).
template <typename T, int EPI>
static cudaError_t pair_prepare(int* max_pairs) {
  static PerDeviceOnce once;
  static std::atomic<int> pairs[kMaxDevicesPerProcess];
  auto kern = gemm_pair_kernel<T, EPI>;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaError_t e = once.run([&] {
    cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes);
    if (e2 != cudaSuccess) return e2;
    pairs[dev].store(max_active_clusters(kern, dim3(kPairThreads), PairCfg::kSmemBytes, 2), std::memory_order_relaxed);
    return cudaSuccess;
  });
  if (e != cudaSuccess) return e;
  *max_pairs = pairs[dev].load(std::memory_order_relaxed);
  return cudaSuccess;
}

template <typename T, int EPI>
static int pair_launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, PairParams& p, int upp_hint,
                       int64_t ws_bytes, int num_flags, cudaStream_t stream) {
  int resident = 0;
  cudaError_t e = pair_prepare<T, EPI>(&resident);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int sms = device_sm_count();
  int max_pairs = resident < sms / 2 ? resident : sms / 2;
  const int64_t slot_bytes = (int64_t)kPairRows * p.bnf * 4;  // one accumulator of one CTA
  const int64_t pair_bytes = 2 * p.nacc * slot_bytes;
  if (ws_bytes / pair_bytes < max_pairs) max_pairs = (int)(ws_bytes / pair_bytes);
  if (max_pairs < 1) return -1;
  const int tiles = p.tiles_m * p.tiles_n;
  if (tiles * 8 > num_flags) return -1;
  const int nslab = p.out_cols / 64;
  const int area = PairCfg::num_stages(p.bnf, p.nacc) * PairCfg::stage_bytes(p.bnf, p.nacc);
  const int land = area - kPairFinalStagingBytes;
  // Split mode: with fewer tiles than pairs, every tile is cut into `split` equal K parts (K padded with blocks
  // beyond the matrix, which TMA reads as zeros), one pair each; the pairs of a tile finish together, exchange
  // partials and each finalises its share of the slabs.  upp_hint = -n asks for n parts.
  p.split = 0;
  int upp = 0;
  if (EPI != 2 && p.nacc == 1 && upp_hint <= 0) {
    int parts = upp_hint < 0 ? -upp_hint : max_pairs / tiles;
    if (parts > nslab) parts = nslab;
    if (parts > 4) parts = 4;
    if (parts > p.num_kb) parts = p.num_kb;
    if (parts >= 2 && tiles * parts <= max_pairs) {
      const int own_max = (nslab + parts - 1) / parts;
      if ((int64_t)(parts - 1) * own_max * 64 * kPairRows * 4 <= land) {
        p.split = parts;
        upp = (p.num_kb + parts - 1) / parts;
        p.num_kb = upp * parts;
      }
    }
  }
  p.total_units = p.tiles_m * p.supers_n * p.num_kb;
  if (!p.split) {
    upp = upp_hint > 0 ? upp_hint : (p.total_units + max_pairs - 1) / max_pairs;
    // a tile may not be cut into more pieces than its owner can merge: the partials of all contributors of one
    // round (a quarter of the tile's columns at the least) land in the owner's pipeline stages at once
    int max_contrib = (int)((int64_t)land * nslab / slot_bytes);
    if (max_contrib > kPairMaxContrib) max_contrib = kPairMaxContrib;
    const int min_upp = max_contrib >= 1 ? (p.num_kb + max_contrib - 1) / max_contrib : p.num_kb;
    if (upp < min_upp) upp = min_upp;
    if (upp_hint <= 0) {
      // Pairs whose whole range lies inside one tile finish when its owner does and make it wait for their
      // partials; with at least a tile's worth of units per pair every contribution is the FIRST thing its pair
      // does.  Prefer that, and a cut on tile boundaries when it costs at most a fifth more units per pair.
      if (upp < p.num_kb) upp = p.num_kb;
      for (int e2 = upp; e2 * 5 <= upp * 6; ++e2) {
        if (e2 % p.num_kb == 0) {
          upp = e2;
          break;
        }
      }
    }
    if ((p.total_units + upp - 1) / upp > max_pairs) upp = (p.total_units + max_pairs - 1) / max_pairs;
  }
  p.upp = upp;
  const int pairs = (p.total_units + upp - 1) / upp;
  return static_cast<int>(launch_pdl_cluster(gemm_pair_kernel<T, EPI>, dim3(2 * pairs), dim3(kPairThreads),
                                             (size_t)PairCfg::kSmemBytes, 2u, stream, ta, tb, tc, p));
}

}  // namespace blitz

extern "C" {

// Scratch of the paired GEMM: bytes of fp32 partials for `sms / 2` pairs at the widest super tile.
int64_t blitz_gemm_pair_workspace_bytes(int sms) { return (int64_t)(sms / 2 + 1) * 2 * 2 * blitz::kPairRows * 256 * 4; }

// Profiling aid: with a non-null device buffer of (grid size) x 16 uint64, every CTA of later launches records
// globaltimer stamps (start, set-up done, first operands landed, last UMMA committed, last accumulator seen,
// epilogue done, dependency wait passed, end, partials parked, counters seen, partials landed, stores issued).
// Null (the default) turns it off.
void blitz_gemm_pair_set_trace(unsigned long long* buf) { blitz::g_pair_trace = buf; }

// Whether blitz_gemm_pair takes this problem.
int blitz_gemm_pair_supported(int M, int N, int K, int b_layout, int epilogue) {
  return M >= 1 && b_layout == 0 && epilogue >= 0 && epilogue <= 2 && (N & 7) == 0 && (K & 7) == 0 && N >= 64;
}

// C = A W (+R | silu-mul).  A [M, lda>=K], W [K, ldb>=columns] row-major, C/R [M, ldc>=N].  dtype 0 fp16, 1 bf16.
// epilogue 0 store, 1 add R (C may be R), 2 silu(gate)*up with the up columns starting at up_col_off.
// bnf_hint: accumulator columns per tile (0 = choose, 128 or 256); nacc_hint: tiles per pair that share the
// activation tiles (0 = choose, 1 or 2); upp_hint: units per CTA pair (0 = choose; -n = cut every tile into n
// equal K parts, one pair each).
// ws / ws_bytes: scratch for partials (blitz_gemm_pair_workspace_bytes); flags / num_flags: uint32 counters,
// eight per output tile, zeroed once by the caller (the kernel leaves them zero).
// Returns a cudaError_t value, -1 for arguments it cannot take, -2 when the TMA encoder is missing.
int blitz_gemm_pair(const void* A, int64_t lda, const void* W, int64_t ldb, void* C, int64_t ldc, const void* R, int M,
                    int N, int K, int epilogue, int up_col_off, int dtype, int static_b, int bnf_hint, int nacc_hint,
                    int upp_hint, void* ws, int64_t ws_bytes, unsigned* flags, int num_flags, int* status,
                    cudaStream_t stream) {
  using namespace blitz;
  if (!blitz_gemm_pair_supported(M, N, K, 0, epilogue) || !ws || !flags) return -1;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (epilogue == 2 && (up_col_off & 7))) return -1;
  if (bnf_hint != 0 && bnf_hint != 128 && bnf_hint != 256) return -1;
  if (nacc_hint < 0 || nacc_hint > 2) return -1;
  const int sms = device_sm_count();
  PairParams p;
  p.R = R;
  p.ldc = ldc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.up_col_off = up_col_off;
  p.num_kb = (K + kPairBK - 1) / kPairBK;
  p.tiles_m = (M + 2 * kPairRows - 1) / (2 * kPairRows);
  // Wide tiles cut the activation re-read per weight byte (256 accumulator columns: as many activation bytes as
  // weight bytes; two such accumulators per pair: half as many) but leave fewer tiles to spread over the pairs, and
  // every cut through a tile costs a partial exchange.  256 columns once no tile is cut into more than about six
  // pieces; two accumulators once there are about one and a half tiles per pair (measured: the gate-up projection of
  // Llama-3-8B, 112 tiles, takes 59.5 us on 56 pairs with two accumulators against 62.5 us on 74 pairs with one).
  const int oc256 = epilogue == 2 ? 128 : 256;
  const int tiles256 = p.tiles_m * ((N + oc256 - 1) / oc256);
  int bnf = bnf_hint ? bnf_hint : (tiles256 * 6 >= sms / 2 ? 256 : 128);
  int nacc = nacc_hint ? nacc_hint : ((bnf == 256 && tiles256 * 4 >= sms * 3) ? 2 : 1);
  p.bnf = bnf;
  p.nacc = nacc;
  p.out_cols = epilogue == 2 ? bnf / 2 : bnf;
  p.tiles_n = (N + p.out_cols - 1) / p.out_cols;
  p.supers_n = (p.tiles_n + nacc - 1) / nacc;
  p.static_b = static_b;
  p.ws = reinterpret_cast<float*>(ws);
  p.flags = flags;
  p.status = status;
  p.upp = 0;
  p.total_units = 0;
  p.trace = g_pair_trace;

  CUtensorMap ta, tb, tc;
  if (!get_tmap_2d(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, kPairBK, kPairRows)) return -2;
  const int w_cols = epilogue == 2 ? up_col_off + N : N;
  if (!get_tmap_2d(&tb, W, (uint64_t)w_cols, (uint64_t)K, (uint64_t)ldb * 2, 64, kPairBK)) return -2;
  if (!get_tmap_2d(&tc, C, (uint64_t)N, (uint64_t)M, (uint64_t)ldc * 2, 64, 32)) return -2;

  if (dtype == 1) {
    return epilogue == 2   ? pair_launch<__nv_bfloat16, 2>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream)
           : epilogue == 1 ? pair_launch<__nv_bfloat16, 1>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream)
                           : pair_launch<__nv_bfloat16, 0>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream);
  }
  return epilogue == 2   ? pair_launch<__half, 2>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream)
         : epilogue == 1 ? pair_launch<__half, 1>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream)
                         : pair_launch<__half, 0>(ta, tb, tc, p, upp_hint, ws_bytes, num_flags, stream);
}

}  // extern "C"
