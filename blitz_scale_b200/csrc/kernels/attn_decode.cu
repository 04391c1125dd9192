// Paged-KV decode attention, CUDA-core version (cross-check and fallback for shapes the tensor-core kernel
// does not take): one query token per sequence, GQA,
// split-KV (flash-decoding) with an fp32 merge.  The cache holds rotated K, so
// the kernel is a pure streaming reduction over K and V pages and is bound by
// HBM bandwidth; the work is laid out to keep >= 64 KB of 16-byte loads in
// flight per SM.
//
// Cache layout of one layer: [page][K|V][token_in_page][kv_head][head_dim].
// Page table: CSR (indices, indptr[batch+1]) + last_page_len[batch], the same
// triple the reference stages per step (src/blitz/cache_manager.h:198-253).
// Replaces the FlashInfer decode wrapper (src/kernel/attention_decode.cu:13-40)
// and its host-side planning (src/kernel/flashinfer_types.cu:52-80): no plan
// step, the split count is a launch parameter.
//
// Thread layout: a "group" of HD/8 lanes owns one token at a time (each lane 8
// head-dim elements, i.e. one 16-byte load of K and of V); all q heads that
// share the kv head are evaluated against the same K/V registers.
#include "common.cuh"

namespace blitz {

constexpr int kDecThreads = 128;
constexpr int kDecUnroll = 4;

struct DecodeParams {
  const void* q;         // [batch, q_heads, hd], row pitch q_stride elements
  int64_t q_stride;
  const void* kv;        // layer base
  const int32_t* indices;
  const int32_t* indptr;
  const int32_t* last_page_len;
  void* out;             // [batch, q_heads, hd], row pitch out_stride
  int64_t out_stride;
  float* part_o;         // [batch, q_heads, splits, hd]   (splits > 1)
  float* part_lse;       // [batch, q_heads, splits]
  int q_heads, kv_heads, page_size, max_pages, num_splits;
  float scale_log2;      // softmax scale * log2(e)
  int* status;
};

template <typename T, int HD, int G>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_kernel(const DecodeParams p) {
  constexpr int LPT = HD / 8;            // lanes per token
  constexpr int GPW = 32 / LPT;          // groups per warp
  constexpr int NG = (kDecThreads / 32) * GPW;  // groups per CTA
  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gl = lane % LPT;             // lane within group
  const int grp = warp * GPW + lane / LPT;

  const int pg_beg = p.indptr[b], pg_end = p.indptr[b + 1];
  const int npages = pg_end - pg_beg;
  const int seq_len = npages > 0 ? (npages - 1) * p.page_size + p.last_page_len[b] : 0;
  const int pages_per_split = (npages + p.num_splits - 1) / p.num_splits;
  const int tok_beg = min(seq_len, split * pages_per_split * p.page_size);
  const int tok_end = min(seq_len, (split + 1) * pages_per_split * p.page_size);

  // q for the G heads of this kv head, pre-scaled
  float q[G][8];
  const T* qrow = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(b) * p.q_stride +
                  static_cast<int64_t>(h) * G * HD;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    unpack8<T>(*reinterpret_cast<const uint4*>(qrow + g * HD + gl * 8), q[g]);
#pragma unroll
    for (int j = 0; j < 8; ++j) q[g][j] *= p.scale_log2;
  }
  float o[G][8];
  float m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) o[g][j] = 0.f;
  }

  const int64_t plane = static_cast<int64_t>(p.page_size) * p.kv_heads * HD;
  const T* kv = reinterpret_cast<const T*>(p.kv);
  const int64_t head_off = static_cast<int64_t>(h) * HD + gl * 8;

  // The trip count is uniform across the CTA (the shuffles below need whole warps).
  for (int base = tok_beg; base < tok_end; base += NG * kDecUnroll) {
    const int t0 = base + grp;
    uint4 kreg[kDecUnroll], vreg[kDecUnroll];
    bool valid[kDecUnroll];
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
      const int t = t0 + u * NG;
      valid[u] = t < tok_end;
      kreg[u] = make_uint4(0, 0, 0, 0);
      vreg[u] = make_uint4(0, 0, 0, 0);
      if (valid[u]) {
        const int page = p.indices[pg_beg + t / p.page_size];
        if (page < 0 || page >= p.max_pages) {
          if (p.status) atomicCAS(p.status, 0, kStatusBadIndex);
          valid[u] = false;
        } else {
          const T* kp = kv + static_cast<int64_t>(page) * 2 * plane +
                        static_cast<int64_t>(t % p.page_size) * p.kv_heads * HD + head_off;
          kreg[u] = ld_nc16(kp);
          vreg[u] = ld_nc16(kp + plane);
        }
      }
    }
    float s[kDecUnroll][G];
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
      float kf[8];
      unpack8<T>(kreg[u], kf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += q[g][j] * kf[j];
        s[u][g] = acc;
      }
    }
#pragma unroll
    for (int off = LPT / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int u = 0; u < kDecUnroll; ++u)
#pragma unroll
        for (int g = 0; g < G; ++g) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], off);
    }
    float pr[kDecUnroll][G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int u = 0; u < kDecUnroll; ++u)
        if (valid[u]) mx = fmaxf(mx, s[u][g]);
      const float corr = (mx == -INFINITY) ? 1.f : exp2f(m[g] - mx);
      float lsum = 0.f;
#pragma unroll
      for (int u = 0; u < kDecUnroll; ++u) {
        pr[u][g] = valid[u] ? exp2f(s[u][g] - mx) : 0.f;
        lsum += pr[u][g];
      }
      l[g] = l[g] * corr + lsum;
      m[g] = mx;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[g][j] *= corr;
    }
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
      float vf[8];
      unpack8<T>(vreg[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 8; ++j) o[g][j] += pr[u][g] * vf[j];
    }
  }

  // ---- merge the NG groups of this CTA through shared memory
  __shared__ float sm_o[NG][G][HD];
  __shared__ float sm_m[NG][G];
  __shared__ float sm_l[NG][G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int j = 0; j < 8; ++j) sm_o[grp][g][gl * 8 + j] = o[g][j];
    if (gl == 0) {
      sm_m[grp][g] = m[g];
      sm_l[grp][g] = l[g];
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * HD; e += kDecThreads) {
    const int g = e / HD, d = e % HD;
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < NG; ++i) M = fmaxf(M, sm_m[i][g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
#pragma unroll
      for (int i = 0; i < NG; ++i) {
        const float w = exp2f(sm_m[i][g] - M);
        L += sm_l[i][g] * w;
        O += sm_o[i][g][d] * w;
      }
    }
    const float val = L > 0.f ? O / L : 0.f;
    const int head = h * G + g;
    if (p.num_splits == 1) {
      T* op = reinterpret_cast<T*>(p.out) + static_cast<int64_t>(b) * p.out_stride + static_cast<int64_t>(head) * HD;
      if (std::is_same<T, __nv_bfloat16>::value)
        reinterpret_cast<__nv_bfloat16*>(op)[d] = __float2bfloat16(val);
      else
        reinterpret_cast<__half*>(op)[d] = __float2half(val);
    } else {
      const int64_t base = (static_cast<int64_t>(b) * p.q_heads + head) * p.num_splits + split;
      p.part_o[base * HD + d] = val;
      if (d == 0) p.part_lse[base] = L > 0.f ? M + log2f(L) : -INFINITY;
    }
  }
}

// Combine split partials: out = sum_s w_s o_s / sum_s w_s, w_s = 2^(lse_s - max lse).
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
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
static int launch_decode(const DecodeParams& p, int batch, cudaStream_t stream) {
  const int G = p.q_heads / p.kv_heads;
  dim3 grid(batch, p.kv_heads, p.num_splits);
  switch (G) {
    case 1: attn_decode_kernel<T, HD, 1><<<grid, kDecThreads, 0, stream>>>(p); break;
    case 2: attn_decode_kernel<T, HD, 2><<<grid, kDecThreads, 0, stream>>>(p); break;
    case 4: attn_decode_kernel<T, HD, 4><<<grid, kDecThreads, 0, stream>>>(p); break;
    case 8: attn_decode_kernel<T, HD, 8><<<grid, kDecThreads, 0, stream>>>(p); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

}  // namespace blitz

extern "C" {
using namespace blitz;

// Bytes of fp32 scratch the split path needs: part_o then part_lse.
int64_t blitz_attn_decode_simt_workspace_bytes(int batch, int q_heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return (int64_t)batch * q_heads * num_splits * (head_dim + 1) * (int64_t)sizeof(float);
}

// workspace: caller-provided scratch of blitz_attn_decode_workspace_bytes() bytes (may be null when num_splits == 1).
int blitz_attn_decode_simt(const void* q, int64_t q_stride, const void* kv_layer, const int32_t* indices,
                      const int32_t* indptr, const int32_t* last_page_len, void* out, int64_t out_stride,
                      void* workspace, int batch, int q_heads, int kv_heads, int head_dim, int page_size,
                      int max_pages, int num_splits, float sm_scale, int* status, int dtype, cudaStream_t stream) {
  if (batch <= 0) return 0;
  if (num_splits < 1 || (q_heads % kv_heads) != 0 || (q_stride & 7) || (out_stride & 7)) return -1;
  if (num_splits > 1 && workspace == nullptr) return -1;
  DecodeParams p;
  p.q = q; p.q_stride = q_stride; p.kv = kv_layer; p.indices = indices; p.indptr = indptr;
  p.last_page_len = last_page_len; p.out = out; p.out_stride = out_stride;
  p.part_o = reinterpret_cast<float*>(workspace);
  p.part_lse = p.part_o ? p.part_o + (int64_t)batch * q_heads * num_splits * head_dim : nullptr;
  p.q_heads = q_heads; p.kv_heads = kv_heads; p.page_size = page_size; p.max_pages = max_pages;
  p.num_splits = num_splits; p.scale_log2 = sm_scale * 1.4426950408889634f; p.status = status;
  int rc;
  if (dtype == 1) {
    rc = head_dim == 128 ? launch_decode<__nv_bfloat16, 128>(p, batch, stream)
         : head_dim == 64 ? launch_decode<__nv_bfloat16, 64>(p, batch, stream) : -1;
  } else {
    rc = head_dim == 128 ? launch_decode<__half, 128>(p, batch, stream)
         : head_dim == 64 ? launch_decode<__half, 64>(p, batch, stream) : -1;
  }
  if (rc != 0) return rc;
  if (num_splits > 1) {
    dim3 grid(batch, q_heads);
    if (dtype == 1)
      attn_merge_kernel<__nv_bfloat16><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__nv_bfloat16*)out,
                                                                      out_stride, q_heads, head_dim, num_splits);
    else
      attn_merge_kernel<__half><<<grid, head_dim, 0, stream>>>(p.part_o, p.part_lse, (__half*)out, out_stride,
                                                               q_heads, head_dim, num_splits);
    rc = (int)cudaGetLastError();
  }
  return rc;
}

}  // extern "C"
