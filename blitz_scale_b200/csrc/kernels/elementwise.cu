// Memory-bound serving kernels for sm_100a: embedding lookup (plain and
// vocab-sharded), RMSNorm, fused residual-add + RMSNorm, SiLU*mul, residual
// add, last-token gather, greedy argmax and temperature/top-k/top-p sampling,
// RoPE fused with the paged KV-cache write.
//
// Counterparts in the reference: src/kernel/embedding.cu:7-90,
// src/kernel/norm.cu:7-39, src/kernel/activation.cu:9-23, src/kernel/add.cu:13-55,
// src/kernel/sampler.cu:7-141, src/kernel/page.cu:21-115.  All kernels move
// 16 bytes per thread access and keep reductions in fp32.
#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace blitz {

// ------------------------------------------------------------------ embedding
// out[t,:] = table[ids[t] - vocab_start,:] when the id is owned by this shard
// ([vocab_start, vocab_start + vocab_rows)); otherwise zeros (zero_missing) or
// the row is left untouched.  dst_rows optionally redirects row t to another
// output row.
template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int hidden, int vocab_start, int vocab_rows, int zero_missing,
                                 const int32_t* __restrict__ dst_rows) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const int t = blockIdx.x;
  const int id = ids[t] - vocab_start;
  const int row = dst_rows ? dst_rows[t] : t;
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<int64_t>(row) * hidden);
  const int nvec = hidden >> 3;
  if (id >= 0 && id < vocab_rows) {
    const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<int64_t>(id) * hidden);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = __ldg(src + i);
  } else if (zero_missing) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
  }
}

// ------------------------------------------------------------------ RMSNorm
// ADD = false: out = x * rsqrt(mean(x^2) + eps) * w
// ADD = true : residual += x; out = RMSNorm(residual) * w     (out may alias x)
template <typename T, bool ADD>
__global__ void rms_norm_kernel(const T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ w,
                                T* __restrict__ out, int hidden, float eps) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  __shared__ float red[33];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * hidden;
  const int nvec = hidden >> 3;
  const uint4* xv = reinterpret_cast<const uint4*>(x + base);
  uint4* rv = ADD ? reinterpret_cast<uint4*>(residual + base) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8<T>(xv[i], f);
    if (ADD) {
      float r[8];
      unpack8<T>(rv[i], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += r[j];
      uint4 packed = pack8<T>(f);
      rv[i] = packed;
      unpack8<T>(packed, f);  // normalise the rounded residual, as a separate add kernel would
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float scale = rsqrtf(ss / static_cast<float>(hidden) + eps);
  const uint4* src = ADD ? reinterpret_cast<const uint4*>(residual + base) : xv;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* ov = reinterpret_cast<uint4*>(out + base);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8], g[8];
    unpack8<T>(src[i], f);
    unpack8<T>(__ldg(wv + i), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * scale * g[j];
    ov[i] = pack8<T>(f);
  }
}

// ------------------------------------------------------------------ SiLU * mul, residual add
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int64_t in_stride) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const int64_t t = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(in + t * in_stride);
  const uint4* u = reinterpret_cast<const uint4*>(in + t * in_stride + inter);
  uint4* o = reinterpret_cast<uint4*>(out + t * inter);
  for (int i = threadIdx.x; i < (inter >> 3); i += blockDim.x) {
    float a[8], b[8];
    unpack8<T>(g[i], a);
    unpack8<T>(u[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    o[i] = pack8<T>(a);
  }
}

template <typename T>
__global__ void add_kernel(T* __restrict__ residual, const T* __restrict__ x, int64_t nvec) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float a[8], b[8];
    unpack8<T>(reinterpret_cast<uint4*>(residual)[i], a);
    unpack8<T>(reinterpret_cast<const uint4*>(x)[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j];
    reinterpret_cast<uint4*>(residual)[i] = pack8<T>(a);
  }
}

// ------------------------------------------------------------------ gather last token of each sequence
template <typename T>
__global__ void gather_last_kernel(const T* __restrict__ x, const int32_t* __restrict__ indptr, T* __restrict__ out,
                                   int hidden) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const int b = blockIdx.x;
  const int64_t row = static_cast<int64_t>(indptr[b + 1]) - 1;
  const uint4* src = reinterpret_cast<const uint4*>(x + row * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<int64_t>(b) * hidden);
  for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------ greedy argmax
// One block per row.  Ties resolve to the smallest index (torch.argmax order).
// Also emits the maximum value so vocab-sharded ranks can exchange (value, index).
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int vocab, int64_t stride, int32_t* __restrict__ out_idx,
                              float* __restrict__ out_val, int idx_offset) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  __shared__ float sval[32];
  __shared__ int sidx[32];
  const T* row = logits + static_cast<int64_t>(blockIdx.x) * stride;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  const int nvec = vocab >> 3;
  const uint4* rv = reinterpret_cast<const uint4*>(row);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8<T>(rv[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (f[j] > best) {
        best = f[j];
        besti = i * 8 + j;
      }
    }
  }
  for (int i = (nvec << 3) + threadIdx.x; i < vocab; i += blockDim.x) {
    float v = to_f<T>(row[i]);
    if (v > best) {
      best = v;
      besti = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) {
      best = ov;
      besti = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sval[warp] = best;
    sidx[warp] = besti;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sval[lane] : -INFINITY;
    besti = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, besti, o);
      if (ov > best || (ov == best && oi < besti)) {
        best = ov;
        besti = oi;
      }
    }
    if (lane == 0) {
      out_idx[blockIdx.x] = besti + idx_offset;
      if (out_val) out_val[blockIdx.x] = best;
    }
  }
}

// ------------------------------------------------------------------ temperature / top-k / top-p sampling
// One block per row.  Keeps the k most likely tokens, then the smallest
// prefix of them (by probability) whose mass reaches top_p, and draws from the
// renormalised rest with a counter-based hash of (seed, step, row).  Both
// thresholds are found by bisection on the value axis, so no sort is needed.
__device__ __forceinline__ float hash_uniform(uint64_t seed, uint64_t a, uint64_t b) {
  uint64_t z = seed + 0x9e3779b97f4a7c15ull * (a + 1) + 0xbf58476d1ce4e5b9ull * (b + 1);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

template <typename T>
__global__ void sample_kernel(const T* __restrict__ logits, int vocab, int64_t stride, const float* __restrict__ temp,
                              const int32_t* __restrict__ top_k, const float* __restrict__ top_p,
                              const uint64_t* __restrict__ seeds, uint64_t step, int32_t* __restrict__ out_idx) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  __shared__ float red[33];
  __shared__ float scan[1025];
  __shared__ int chosen;
  const int b = blockIdx.x;
  const T* row = logits + static_cast<int64_t>(b) * stride;
  const float inv_t = 1.f / fmaxf(temp[b], 1e-6f);
  const int k = top_k[b] > 0 ? min(top_k[b], vocab) : vocab;
  const float pcut = top_p[b] > 0.f ? fminf(top_p[b], 1.f) : 1.f;

  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, to_f<T>(row[i]) * inv_t);
  mx = block_max(mx, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) z += __expf(to_f<T>(row[i]) * inv_t - mx);
  z = block_sum(z, red);

  // threshold in "weight" space w = exp(l/T - mx) in (0, 1]
  float lo = 0.f, hi = 1.f;  // keep tokens with w >= thr; thr in [lo, hi]
  if (k < vocab) {
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) cnt += (__expf(to_f<T>(row[i]) * inv_t - mx) >= mid) ? 1.f : 0.f;
      cnt = block_sum(cnt, red);
      if (cnt >= static_cast<float>(k)) lo = mid; else hi = mid;
    }
  }
  float thr_k = lo;  // at least k tokens have w >= thr_k
  if (pcut < 1.f) {
    float lo2 = thr_k, hi2 = 1.f;
    for (int it = 0; it < 30; ++it) {
      const float mid = 0.5f * (lo2 + hi2);
      float mass = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float w = __expf(to_f<T>(row[i]) * inv_t - mx);
        mass += w >= mid ? w : 0.f;
      }
      mass = block_sum(mass, red);
      if (mass >= pcut * z) lo2 = mid; else hi2 = mid;
    }
    thr_k = lo2;
  }
  // inverse-CDF draw over kept tokens in index order; contiguous chunk per thread
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int beg = threadIdx.x * chunk, end = min(vocab, beg + chunk);
  float local = 0.f;
  for (int i = beg; i < end; ++i) {
    float w = __expf(to_f<T>(row[i]) * inv_t - mx);
    local += w >= thr_k ? w : 0.f;
  }
  scan[threadIdx.x + 1] = local;
  if (threadIdx.x == 0) {
    scan[0] = 0.f;
    chosen = -1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i <= static_cast<int>(blockDim.x); ++i) scan[i] += scan[i - 1];
  }
  __syncthreads();
  const float total = scan[blockDim.x];
  const float u = hash_uniform(seeds[b], step, static_cast<uint64_t>(b)) * total;
  if (u >= scan[threadIdx.x] && (u < scan[threadIdx.x + 1] || (threadIdx.x == blockDim.x - 1)) && local > 0.f) {
    float acc = scan[threadIdx.x];
    int pick = -1;
    for (int i = beg; i < end; ++i) {
      float w = __expf(to_f<T>(row[i]) * inv_t - mx);
      if (w >= thr_k) {
        acc += w;
        pick = i;
        if (acc > u) break;
      }
    }
    if (pick >= 0) atomicMax(&chosen, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = chosen;
    if (c < 0) {  // numerical corner: fall back to the arg-max token
      float best = -INFINITY;
      for (int i = 0; i < vocab; ++i) {
        float v = to_f<T>(row[i]);
        if (v > best) { best = v; c = i; }
      }
    }
    out_idx[b] = c;
  }
}

// ------------------------------------------------------------------ RoPE + paged KV write
// qkv row t = [q heads | k heads | v heads].  Rotates q and k in place with the
// Llama (rotate-half) convention at position pos[t], then writes the rotated
// k row and the v row to the paged cache at slot[t] = page_id * page_size +
// offset.  Cache layout of one layer: [page][K|V][token][kv_head][head_dim].
// A negative slot skips the cache write (bounds: slot < max_pages * page_size
// is checked; a bad slot sets *status and skips).
constexpr int kRopeMaxHalf = 128;  // head_dim <= 256
template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, const int32_t* __restrict__ pos,
                                     const int32_t* __restrict__ slot, T* __restrict__ kv_layer, int q_heads,
                                     int kv_heads, int head_dim, int page_size, int max_pages, float log2_theta,
                                     int* __restrict__ status) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const int t = blockIdx.x;
  const int half = head_dim >> 1;
  const int vec_per_half = half >> 3;
  const int64_t row_stride = static_cast<int64_t>(q_heads + 2 * kv_heads) * head_dim;
  T* row = qkv + t * row_stride;
  const float p = static_cast<float>(pos[t]);
  int s = slot[t];
  if (s >= max_pages * page_size) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, kStatusBadIndex);
    s = -1;
  }
  const int page = s >= 0 ? s / page_size : 0;
  const int off = s >= 0 ? s % page_size : 0;
  const int64_t plane = static_cast<int64_t>(page_size) * kv_heads * head_dim;
  T* kdst = kv_layer + (static_cast<int64_t>(page) * 2) * plane + static_cast<int64_t>(off) * kv_heads * head_dim;
  T* vdst = kdst + plane;

  // the angle of pair i depends on the token's position only: computed once per token (accurate sincosf: positions
  // of thousands of radians) and shared by all heads through shared memory
  __shared__ float s_cs[kRopeMaxHalf], s_sn[kRopeMaxHalf];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float inv_freq = exp2f(-(2.0f * static_cast<float>(i) / static_cast<float>(head_dim)) * log2_theta);
    sincosf(p * inv_freq, &s_sn[i], &s_cs[i]);
  }
  __syncthreads();
  const int rot_items = (q_heads + kv_heads) * vec_per_half;
  for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
    const int head = it / vec_per_half;
    const int v = it % vec_per_half;
    T* hp = row + static_cast<int64_t>(head) * head_dim;
    float a[8], b[8];
    unpack8<T>(*reinterpret_cast<uint4*>(hp + v * 8), a);
    unpack8<T>(*reinterpret_cast<uint4*>(hp + half + v * 8), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cs = s_cs[v * 8 + j], sn = s_sn[v * 8 + j];
      const float x0 = a[j], x1 = b[j];
      a[j] = x0 * cs - x1 * sn;
      b[j] = x1 * cs + x0 * sn;
    }
    const uint4 pa = pack8<T>(a), pb = pack8<T>(b);
    *reinterpret_cast<uint4*>(hp + v * 8) = pa;
    *reinterpret_cast<uint4*>(hp + half + v * 8) = pb;
    if (head >= q_heads && s >= 0) {
      T* kd = kdst + static_cast<int64_t>(head - q_heads) * head_dim;
      *reinterpret_cast<uint4*>(kd + v * 8) = pa;
      *reinterpret_cast<uint4*>(kd + half + v * 8) = pb;
    }
  }
  if (s >= 0) {
    const uint4* vsrc = reinterpret_cast<const uint4*>(row + static_cast<int64_t>(q_heads + kv_heads) * head_dim);
    uint4* vd = reinterpret_cast<uint4*>(vdst);
    for (int i = threadIdx.x; i < ((kv_heads * head_dim) >> 3); i += blockDim.x) vd[i] = vsrc[i];
  }
}

static inline int pick_threads(int nvec) {
  int t = 32;
  while (t < nvec && t < 1024) t <<= 1;
  return t;
}

}  // namespace blitz

extern "C" {
using namespace blitz;

int blitz_embedding(const int32_t* ids, const void* table, void* out, int num_tokens, int hidden, int vocab_start,
                    int vocab_rows, int zero_missing, const int32_t* dst_rows, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden & 7) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(embedding_kernel<T>, dim3(num_tokens), dim3(pick_threads(hidden >> 3)), 0, stream,
                                  ids, (const T*)table, (T*)out, hidden, vocab_start, vocab_rows, zero_missing,
                                  dst_rows)));
  return (int)blitz_last;
}

int blitz_rms_norm(const void* x, const void* w, void* out, int num_tokens, int hidden, float eps, int dtype,
                   cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden & 7) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(rms_norm_kernel<T, false>, dim3(num_tokens), dim3(pick_threads(hidden >> 3)), 0, stream,
                                  (const T*)x, nullptr, (const T*)w, (T*)out, hidden, eps)));
  return (int)blitz_last;
}

// residual += x ; out = RMSNorm(residual) * w.  `out` may alias `x`.
int blitz_add_rms_norm(const void* x, void* residual, const void* w, void* out, int num_tokens, int hidden, float eps,
                       int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (hidden & 7) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(rms_norm_kernel<T, true>, dim3(num_tokens), dim3(pick_threads(hidden >> 3)), 0, stream,
                                  (const T*)x, (T*)residual, (const T*)w, (T*)out, hidden, eps)));
  return (int)blitz_last;
}

int blitz_silu_mul(const void* in, void* out, int num_tokens, int inter, int64_t in_stride, int dtype,
                   cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if ((inter & 7) || (in_stride & 7)) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(silu_mul_kernel<T>, dim3(num_tokens), dim3(pick_threads(inter >> 3)), 0, stream,
                                  (const T*)in, (T*)out, inter, in_stride)));
  return (int)blitz_last;
}

int blitz_add_residual(void* residual, const void* x, int64_t numel, int dtype, cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (numel & 7) return -1;
  const int64_t nvec = numel >> 3;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(add_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)residual, (const T*)x, nvec)));
  return (int)blitz_last;
}

int blitz_gather_last(const void* x, const int32_t* indptr, void* out, int batch, int hidden, int dtype,
                      cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (hidden & 7) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(gather_last_kernel<T>, dim3(batch), dim3(pick_threads(hidden >> 3)), 0, stream,
                                  (const T*)x, indptr, (T*)out, hidden)));
  return (int)blitz_last;
}

int blitz_argmax(const void* logits, int batch, int vocab, int64_t stride, int32_t* out_idx, float* out_val,
                 int idx_offset, int dtype, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (stride & 7) return -1;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(argmax_kernel<T>, dim3(batch), dim3(1024), 0, stream, (const T*)logits, vocab, stride, out_idx,
                                                                            out_val, idx_offset)));
  return (int)blitz_last;
}

int blitz_sample(const void* logits, int batch, int vocab, int64_t stride, const float* temperature,
                 const int32_t* top_k, const float* top_p, const uint64_t* seeds, uint64_t step, int32_t* out_idx,
                 int dtype, cudaStream_t stream) {
  if (batch <= 0) return 0;
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(sample_kernel<T>, dim3(batch), dim3(1024), 0, stream, (const T*)logits, vocab, stride,
                                                                            temperature, top_k, top_p, seeds, step,
                                                                            out_idx)));
  return (int)blitz_last;
}

int blitz_rope_kv_store(void* qkv, const int32_t* pos, const int32_t* slot, void* kv_layer, int num_tokens,
                        int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, float rope_theta,
                        int* status, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if ((head_dim & 15) || head_dim > 2 * kRopeMaxHalf) return -1;
  const float log2_theta = log2f(rope_theta);
  cudaError_t blitz_last = cudaSuccess;
  BLITZ_DISPATCH_DTYPE(dtype, (blitz_last = launch_pdl(rope_kv_store_kernel<T>, dim3(num_tokens), dim3(256), 0, stream,
                                  (T*)qkv, pos, slot, (T*)kv_layer, q_heads, kv_heads, head_dim, page_size, max_pages,
                                  log2_theta, status)));
  return (int)blitz_last;
}

}  // extern "C"
