// Causal ragged (varlen) prefill attention on tcgen05 for sm_100a, GQA, head_dim 128.
//
// Input is the fused QKV activation [tokens, (q_heads + 2 kv_heads) * 128] after
// RoPE (rope_kv_store rotates q and k in place and writes the cache), so Q, K
// and V tiles are plain 2-D TMA boxes of the same tensor.  One CTA owns a tile
// of 128 query rows of one sequence and one q head, and walks the KV blocks of
// 128 tokens up to the diagonal:
//
//   S = Q K^T          tcgen05.mma, A = Q (smem, K-major), B = K block (smem, K-major), S in TMEM cols [0,128)
//   P = softmax tile   4 warps, thread = row: tcgen05.ld S, online max/sum in fp32, P -> smem (bf16, 128B swizzle)
//   PV = P V           tcgen05.mma, A = P (smem), B = V block (smem, N-major), PV in TMEM cols [128,256)
//   O  = O * alpha + PV in registers (thread = row), normalised and stored at the end.
//
// A fifth warp drives TMA and issues the MMAs; K/V blocks are double buffered
// and S of block j+1 is issued as soon as PV of block j is in flight, so the
// tensor core works while the softmax warps rescale O.
//
// Replaces FlashInfer's BatchPrefillWithRaggedKVCacheWrapper call and its host
// Plan() (src/kernel/attention_prefill.cu:11-45, src/kernel/flashinfer_types.cu:24-49).
#include "launch.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include "common.cuh"

namespace blitz {

constexpr int kPfThreads = 160;
constexpr int kPfTile = 128;   // q rows per CTA and kv tokens per block
constexpr int kPfHD = 128;
constexpr int kTileBytes = kPfTile * kPfHD * 2;  // 32 KB: two 16 KB slabs of 64 columns

struct PrefillParams {
  void* out;            // [tokens, q_heads * 128]
  int64_t out_stride;
  const int32_t* indptr;  // [batch + 1] token offsets
  int batch;
  int q_heads, kv_heads;
  float scale_log2;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(kPfThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap, const PrefillParams p) {
  constexpr uint32_t kFmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t kIdescS = ptx::make_idesc_f16(kFmt, 0u, 0u, 128, 128);
  constexpr uint32_t kIdescPV = ptx::make_idesc_f16(kFmt, 0u, 1u, 128, 128);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* sQ = smem;
  uint8_t* sP = smem + kTileBytes;
  uint8_t* sK = smem + 2 * kTileBytes;  // [2 stages]
  uint8_t* sV = smem + 4 * kTileBytes;  // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* v_full = bars + 3;    // [2]
  uint64_t* kv_empty = bars + 5;  // [2]
  uint64_t* s_full = bars + 7;
  uint64_t* p_ready = bars + 8;
  uint64_t* o_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- locate this CTA's (sequence, q tile)
  int seq_start = 0, seq_len = 0, q0 = -1;
  {
    int tile = blockIdx.x;
    for (int b = 0; b < p.batch; ++b) {
      const int s = p.indptr[b], e = p.indptr[b + 1];
      const int nt = (e - s + kPfTile - 1) / kPfTile;
      if (tile < nt) {
        seq_start = s;
        seq_len = e - s;
        q0 = tile * kPfTile;
        break;
      }
      tile -= nt;
    }
  }
  if (q0 < 0) return;  // uniform across the CTA
  const int head = blockIdx.y;
  const int kv_head = head / (p.q_heads / p.kv_heads);
  const int q_col = head * kPfHD;
  const int k_col = (p.q_heads + kv_head) * kPfHD;
  const int v_col = (p.q_heads + p.kv_heads + kv_head) * kPfHD;
  const int nblk = q0 / kPfTile + 1;

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&kv_empty[i], 1);
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(p_ready, 128);
    ptx::mbar_init(o_full, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
    ptx::tma_prefetch_desc(&tmap);
  }
  if (warp == 4) {
    ptx::tmem_alloc(tmem_slot, 256);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + 128;

  if (warp == 4) {
    // ------------------------------------------------------------ control: TMA + MMA issue
    if (lane == 0) {
      auto load_tile = [&](uint8_t* dst, uint64_t* bar, int col, int row) {
        ptx::mbar_expect_tx(bar, kTileBytes);
        ptx::tma_load_2d(dst, &tmap, bar, col, row);
        ptx::tma_load_2d(dst + kTileBytes / 2, &tmap, bar, col + 64, row);
      };
      auto issue_S = [&](int stage) {
        const uint32_t a = ptx::smem_u32(sQ), b = ptx::smem_u32(sK + stage * kTileBytes);
#pragma unroll
        for (int k = 0; k < kPfHD / 16; ++k) {
          const uint32_t off = (k >> 2) * (kTileBytes / 2) + (k & 3) * 32;
          ptx::umma_f16_ss(tmem_S, ptx::make_smem_desc(a + off, 16, 1024, ptx::kLayoutSw128),
                           ptx::make_smem_desc(b + off, 16, 1024, ptx::kLayoutSw128), kIdescS, k != 0 ? 1u : 0u);
        }
        ptx::umma_commit(s_full);
      };
      bool ok = true;
      load_tile(sQ, q_full, q_col, seq_start + q0);
      load_tile(sK, &k_full[0], k_col, seq_start);
      load_tile(sV, &v_full[0], v_col, seq_start);
      ok = ptx::bounded_mbar_wait(q_full, 0, abort_flag) && ptx::bounded_mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        ptx::tc_fence_after_sync();
        issue_S(0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1, ns = s ^ 1;
        if (j + 1 < nblk) {
          if (j >= 1) ok = ptx::bounded_mbar_wait(&kv_empty[ns], ((j - 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          load_tile(sK + ns * kTileBytes, &k_full[ns], k_col, seq_start + (j + 1) * kPfTile);
          load_tile(sV + ns * kTileBytes, &v_full[ns], v_col, seq_start + (j + 1) * kPfTile);
        }
        ok = ptx::bounded_mbar_wait(p_ready, j & 1, abort_flag) &&
             ptx::bounded_mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        {
          const uint32_t a = ptx::smem_u32(sP), b = ptx::smem_u32(sV + s * kTileBytes);
#pragma unroll
          for (int k = 0; k < kPfTile / 16; ++k) {
            // A = P: K-major, two slabs of 64 tokens.  B = V: N-major, two slabs of 64
            // head-dim columns 16 KB apart; 16 tokens (K) advance 2 KB.
            const uint32_t aoff = (k >> 2) * (kTileBytes / 2) + (k & 3) * 32;
            ptx::umma_f16_ss(tmem_O, ptx::make_smem_desc(a + aoff, 16, 1024, ptx::kLayoutSw128),
                             ptx::make_smem_desc(b + k * 2048, kTileBytes / 2, 1024, ptx::kLayoutSw128), kIdescPV,
                             k != 0 ? 1u : 0u);
          }
          ptx::umma_commit(o_full);
          ptx::umma_commit(&kv_empty[s]);
        }
        if (j + 1 < nblk) {
          ok = ptx::bounded_mbar_wait(&k_full[ns], ((j + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          issue_S(ns);
        }
      }
      if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------ softmax warps (thread = query row)
    const int r = warp * 32 + lane;
    const int q_idx = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float o[kPfHD];
#pragma unroll
    for (int i = 0; i < kPfHD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (!ptx::bounded_mbar_wait(s_full, j & 1, abort_flag)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after_sync();
      const bool diag = (j == nblk - 1);
      const int kv0 = j * kPfTile;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kPfTile; c += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_S + lane_addr + c, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(v[i]);
          if (!diag || (kv0 + c + i <= q_idx)) mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx * p.scale_log2);
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // pass 2: probabilities -> shared memory (bf16/fp16, 128-byte swizzled rows), row sum
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < kPfTile; c += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_S + lane_addr + c, v);
        ptx::tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = exp2f(__uint_as_float(v[2 * i]) * p.scale_log2 - m_use);
          float p1 = exp2f(__uint_as_float(v[2 * i + 1]) * p.scale_log2 - m_use);
          if (diag) {
            if (kv0 + c + 2 * i > q_idx) p0 = 0.f;
            if (kv0 + c + 2 * i + 1 > q_idx) p1 = 0.f;
          }
          rowsum += p0 + p1;
          pk[i] = pk2<T>(p0, p1);
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = (c >> 3) + g;  // 16-byte chunk index along the token axis: 0..15
          const uint32_t off = (chunk >> 3) * (kTileBytes / 2) + r * 128 + (((chunk & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(sP + off) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
        }
      }
      l = l * alpha + rowsum;
      m = m_new;
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(p_ready);
      // O = O * alpha + P V
      if (!ptx::bounded_mbar_wait(o_full, j & 1, abort_flag)) {
        ok = false;
        break;
      }
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < kPfHD; c += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32(tmem_O + lane_addr + c, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(v[i]);
      }
    }
    if (!ok) {
      if (p.status && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
    } else if (q_idx < seq_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* dst = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(seq_start + q_idx) * p.out_stride + q_col;
#pragma unroll
      for (int c = 0; c < kPfHD; c += 8) {
        *reinterpret_cast<uint4*>(dst + c) =
            make_uint4(pk2<T>(o[c] * inv, o[c + 1] * inv), pk2<T>(o[c + 2] * inv, o[c + 3] * inv),
                       pk2<T>(o[c + 4] * inv, o[c + 5] * inv), pk2<T>(o[c + 6] * inv, o[c + 7] * inv));
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, 256);
  }
}

constexpr int kPfSmemBytes = 6 * kTileBytes + 1024 + 256;

}  // namespace blitz

extern "C" {
using namespace blitz;

// qkv: [num_tokens, (q_heads + 2 kv_heads) * 128] rotated in place; out: [num_tokens, q_heads * 128].
// indptr_dev: device copy of the token offsets; total_q_tiles = sum over sequences of ceil(len / 128)
// (the caller knows the lengths on the host).  Only head_dim 128 is built.
int blitz_attn_prefill(const void* qkv, void* out, int64_t out_stride, const int32_t* indptr_dev, int batch,
                       int num_tokens, int total_q_tiles, int q_heads, int kv_heads, int head_dim, float sm_scale,
                       int* status, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0 || total_q_tiles <= 0) return 0;
  if (head_dim != kPfHD || (q_heads % kv_heads) != 0 || (out_stride & 7)) return -1;
  const uint64_t row = (uint64_t)(q_heads + 2 * kv_heads) * kPfHD;
  CUtensorMap tm;
  if (!get_tmap_2d(&tm, qkv, row, (uint64_t)num_tokens, row * 2, 64, kPfTile)) return -2;
  PrefillParams p;
  p.out = out; p.out_stride = out_stride; p.indptr = indptr_dev; p.batch = batch;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status;
  dim3 grid(total_q_tiles, q_heads);
  static PerDeviceOnce once_bf16, once_f16;
  if (dtype == 1) {
    cudaError_t e = once_bf16.run([] {
      return cudaFuncSetAttribute(attn_prefill_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kPfSmemBytes);
    });
    if (e != cudaSuccess) return (int)e;
    attn_prefill_kernel<__nv_bfloat16><<<grid, kPfThreads, kPfSmemBytes, stream>>>(tm, p);
  } else {
    cudaError_t e = once_f16.run([] {
      return cudaFuncSetAttribute(attn_prefill_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  kPfSmemBytes);
    });
    if (e != cudaSuccess) return (int)e;
    attn_prefill_kernel<__half><<<grid, kPfThreads, kPfSmemBytes, stream>>>(tm, p);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
