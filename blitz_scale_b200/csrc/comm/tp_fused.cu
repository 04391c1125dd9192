// Tensor-parallel glue kernels for the fused GEMM->reduce-scatter / all-gather->GEMM pair.
//
// Data flow of one row-parallel + column-parallel pair on `tp` GPUs (push model, no collective library):
//
//   GEMM (push epilogue)   every rank stores its bf16 partial rows straight into the staging slot
//                          stage[owner][src_rank][column / 8][local_row][8] of the rank that owns those rows
//                          (sequence-sharded residual), then bumps flag_rs[owner][src] once per tile.
//   rs_reduce_norm (here)  the owner waits (bounded) for all tiles of all sources, sums the partials in
//                          rank order in fp32 (deterministic), adds its residual shard, writes the new
//                          residual, applies RMSNorm and stores the normalised rows into the gathered
//                          activation buffer xg[M][H] of EVERY rank (all-gather by push), bumping
//                          flag_ag[dst][src] once per row.
//   next GEMM (wait flags) its TMA producer waits for flag_ag from all sources, fences the async proxy
//                          and then reads xg from local memory only.
//
// This is the AllReduce of src/layer/attn.h:217-233 and src/layer/glu.h:138-154 split into its
// reduce-scatter and all-gather halves with the add+RMSNorm (src/kernel/norm.cu:24-39) in between.
// Flags are counters that their single consumer resets after use, so a captured CUDA graph can be
// replayed without changing any launch parameter.
#include "../kernels/common.cuh"
#include "../kernels/ptx.cuh"

namespace blitz {

constexpr int kMaxTp = 8;
constexpr int kRsBlocks = 64;  // 128-row blocks of one owner's rows: rows_per_rank <= 8192

struct RsReduceParams {
  const void* stage;        // local staging: [tp][H/8][rows_per_rank][8] partials from every source rank
  uint32_t* flag_rs;        // local: [kRsBlocks][kMaxTp] tiles landed per (block of 128 local rows, source), then a
                            // ticket word (all reset here)
  uint32_t tiles_n;         // tiles per block of 128 GEMM rows that every source pushes
  int total_rows;           // rows of the GEMM whose partials arrive (all owners together)
  void* residual;           // local residual shard [rows_per_rank][H] (in/out); may be null (no residual)
  const void* norm_w;       // [H]
  void* xg[kMaxTp];         // gathered activations [M][H] on every rank (peer pointers, self included)
  uint32_t* flag_ag[kMaxTp];  // flag_ag[dst] + my_rank : rows this rank has delivered to dst
  int tp, my_rank, rows_per_rank, rows_valid, hidden;
  float eps;
  uint64_t budget_ns;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) rs_reduce_norm_kernel(const RsReduceParams p) {
  __shared__ float red[33];
  __shared__ int s_ok;
  const int row = blockIdx.x;  // local row
  if (threadIdx.x == 0) {
    // only the tiles that cover this row's block of 128 local rows are waited for: rows whose partials have all
    // arrived are reduced, normalised and sent on while the sources still compute the later blocks.  A block's global
    // rows may lie in more than one 128-row tile of the GEMM when rows_per_rank is not a multiple of 128.
    const int lb = row >> 7;
    const int g0 = p.my_rank * p.rows_per_rank + lb * 128;
    const int g1 = min(p.total_rows, p.my_rank * p.rows_per_rank + min(p.rows_per_rank, (lb + 1) * 128)) - 1;
    const uint32_t expect = p.tiles_n * static_cast<uint32_t>((g1 >> 7) - (g0 >> 7) + 1);
    int ok = 1;
    for (int s = 0; s < p.tp; ++s)
      if (!ptx::bounded_flag_wait_ge(p.flag_rs + lb * kMaxTp + s, expect, p.budget_ns)) ok = 0;
    if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const int H = p.hidden, nvec = H >> 3;
  const T* stage = reinterpret_cast<const T*>(p.stage);
  T* res = reinterpret_cast<T*>(p.residual);
  const int64_t roff = static_cast<int64_t>(row) * H;
  // pass 1: sum partials (+ residual), write residual, accumulate sum of squares
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.tp; ++s) {
      float f[8];
      // staging is written by peers while this kernel runs: coherent L2 loads after the acquire, never the read-only path
      unpack8<T>(__ldcg(reinterpret_cast<const uint4*>(stage + ((static_cast<int64_t>(s) * nvec + i) * p.rows_per_rank + row) * 8)), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    if (res) {
      float f[8];
      unpack8<T>(*reinterpret_cast<const uint4*>(res + roff + i * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
      const uint4 packed = pack8<T>(acc);
      *reinterpret_cast<uint4*>(res + roff + i * 8) = packed;
      unpack8<T>(packed, acc);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += acc[j] * acc[j];
    if (!res) {  // keep the summed row for pass 2 where source 0's vector (consumed just above) was
      *reinterpret_cast<uint4*>(const_cast<T*>(stage) + (static_cast<int64_t>(i) * p.rows_per_rank + row) * 8) = pack8<T>(acc);
    }
  }
  ss = block_sum(ss, red);
  const float scale = rsqrtf(ss / static_cast<float>(H) + p.eps);
  const bool from_stage = res == nullptr;
  const T* w = reinterpret_cast<const T*>(p.norm_w);
  const int64_t grow = static_cast<int64_t>(p.my_rank) * p.rows_per_rank + row;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8], g[8];
    const T* src = from_stage ? stage + (static_cast<int64_t>(i) * p.rows_per_rank + row) * 8 : res + roff + i * 8;
    unpack8<T>(*reinterpret_cast<const uint4*>(src), f);
    unpack8<T>(__ldg(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * scale * g[j];
    const uint4 v = pack8<T>(f);
    for (int d = 0; d < p.tp; ++d)
      ptx::st_na_v4(reinterpret_cast<T*>(p.xg[d]) + grow * H + i * 8, v);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.tp) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.flag_ag[threadIdx.x] + p.my_rank, 1u);
  }
  // the last block to finish re-arms the reduce-scatter flags for the next call
  if (threadIdx.x == 0) {
    const uint32_t t = ptx::atom_add_acq_rel_gpu(p.flag_rs + kRsBlocks * kMaxTp, 1u);
    if (t == gridDim.x - 1) {
      const int nb = (p.rows_per_rank + 127) >> 7;
      for (int i = 0; i < nb * kMaxTp; ++i) p.flag_rs[i] = 0;
      p.flag_rs[kRsBlocks * kMaxTp] = 0;
      __threadfence_system();
    }
  }
}

__global__ void flags_zero_kernel(uint32_t* flags, int n) {
  if (threadIdx.x < n) flags[threadIdx.x] = 0;
  __threadfence_system();
}

// One-shot all-reduce for small tensors over peer memory: every rank pushes its contribution to all
// peers' slot [src], then sums the tp slots in rank order.  Used for the vocab-sharded embedding and as
// the low-latency all-reduce at tiny M.
struct OneShotParams {
  const void* x;            // local contribution [n] elements
  void* slots[kMaxTp];      // slots[d]: base of rank d's receive area [tp][n]
  uint32_t* flags[kMaxTp];  // flags[d] + src
  void* out;                // local result [n]
  int tp, my_rank;
  int64_t n;
  uint32_t want;            // flag value after this call (counter, caller tracks it; 0 = reset mode)
  uint64_t budget_ns;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) oneshot_push_kernel(const OneShotParams p) {
  const int64_t nvec = p.n >> 3;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = ld_nc16(reinterpret_cast<const T*>(p.x) + i * 8);
    for (int d = 0; d < p.tp; ++d)
      ptx::st_na_v4(reinterpret_cast<T*>(p.slots[d]) + static_cast<int64_t>(p.my_rank) * p.n + i * 8, v);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.tp) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.flags[threadIdx.x] + p.my_rank, 1u);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) oneshot_reduce_kernel(const OneShotParams p, uint32_t expect_blocks) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < p.tp; ++s)
      if (!ptx::bounded_flag_wait_ge(p.flags[p.my_rank] + s, expect_blocks, p.budget_ns)) ok = 0;
    if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const int64_t nvec = p.n >> 3;
  const T* mine = reinterpret_cast<const T*>(p.slots[p.my_rank]);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.tp; ++s) {
      float f[8];
      unpack8<T>(__ldcg(reinterpret_cast<const uint4*>(mine + static_cast<int64_t>(s) * p.n + i * 8)), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + i * 8) = pack8<T>(acc);
  }
  // consumer-side reset: the block that finishes last re-arms this rank's arrival counters (nobody reads them any
  // more for this call; the peers' next pushes into this parity come only after they have seen our next push)
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* ticket = p.flags[p.my_rank] + kMaxTp;
    const uint32_t t = ptx::atom_add_acq_rel_gpu(ticket, 1u);
    if (t == gridDim.x - 1) {
      for (int s2 = 0; s2 < p.tp; ++s2) p.flags[p.my_rank][s2] = 0;
      *ticket = 0;
      __threadfence_system();
    }
  }
}

// One-kernel form of the one-shot all-reduce.  Block b owns one contiguous chunk of the vector: it pushes its chunk
// of the local contribution into every rank's slot, bumps counter [src = me][b] on every rank, waits (bounded) until
// counter [s][b] of every source s has arrived here, sums the tp slots of its chunk in rank order, and re-arms the
// counters it consumed.  Blocks with the same index on the tp GPUs thus rendezvous pairwise: there is no grid-wide
// wait and no second launch, and a chunk is summed as soon as its tp pieces are in.  (The blocks wait on blocks
// of OTHER GPUs' kernels only, never on blocks of their own grid.)
constexpr int kArBlocks = 64;

template <typename T>
__global__ void __launch_bounds__(256) allreduce_fused_kernel(const OneShotParams p) {
  __shared__ int s_ok;
  const int64_t nvec = p.n >> 3;
  const int64_t chunk = (nvec + gridDim.x - 1) / gridDim.x;
  const int64_t v0 = static_cast<int64_t>(blockIdx.x) * chunk;
  const int64_t v1 = min(nvec, v0 + chunk);
  const T* x = reinterpret_cast<const T*>(p.x);
  for (int64_t i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    const uint4 v = ld_nc16(x + i * 8);
    for (int d = 0; d < p.tp; ++d)
      ptx::st_na_v4(reinterpret_cast<T*>(p.slots[d]) + static_cast<int64_t>(p.my_rank) * p.n + i * 8, v);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.tp) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.flags[threadIdx.x] + p.my_rank * kArBlocks + blockIdx.x, 1u);
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < p.tp; ++s)
      if (!ptx::bounded_flag_wait_ge(p.flags[p.my_rank] + s * kArBlocks + blockIdx.x, 1u, p.budget_ns)) ok = 0;
    if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const T* mine = reinterpret_cast<const T*>(p.slots[p.my_rank]);
  for (int64_t i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.tp; ++s) {
      float f[8];
      unpack8<T>(__ldcg(reinterpret_cast<const uint4*>(mine + static_cast<int64_t>(s) * p.n + i * 8)), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + i * 8) = pack8<T>(acc);
  }
  __syncthreads();
  if (threadIdx.x < p.tp) p.flags[p.my_rank][threadIdx.x * kArBlocks + blockIdx.x] = 0;  // consumed: re-arm
}


// ---------------------------------------------------------------------------------------------------------------
// All-reduce + residual add + RMSNorm in one kernel through the switch (NVLS), for steps of a few hundred rows.
//
// Every rank's partial result x[M][H] lies in its own copy of a symmetric buffer.  Rows are dealt out evenly: rank r
// finalises rows [r * rpr, (r + 1) * rpr).  For each of its rows a block
//   1. pulls the sum over all ranks with multimem.ld_reduce (the switch adds the tp copies, fp32 accumulation),
//   2. adds its own copy of the residual row, computes the row's RMS statistic,
//   3. writes the new residual row and the normalised row into EVERY rank's copies with multimem.st.
// Per GPU that is one partial out and two rows in per element, whatever tp is (a push-to-everyone all-reduce moves
// tp - 1 copies), and the add + norm launches disappear.  Rendezvous: a "partial is ready" counter per (rank,
// source) before step 1 and an "I have written my rows" counter per (rank, source) after step 3, which the last
// block of the kernel waits for, so that whatever runs next in the stream sees all rows; the waits are bounded.
// Calls alternate between two counter sets (parity): a rank cannot run two calls ahead of a peer because every
// call ends with the all-ranks wait, so a counter is always consumed and re-armed before its next use.
// This is the AllReduce of src/layer/attn.h:217-233 / src/layer/glu.h:138-154 fused with src/kernel/add.cu and
// src/kernel/norm.cu:24-39.
struct ArNormParams {
  const void* x_mc;        // multicast address of the partial-result buffer (all ranks' copies)
  const void* res_local;   // this rank's copy of the residual stream [M][H] (null: no residual, e.g. after the embedding)
  void* res_mc;            // multicast address of the residual stream (written)
  void* xn_mc;             // multicast address of the normalised activations (written)
  const void* norm_w;      // [H]
  uint32_t* flags[kMaxTp]; // flags[d]: rank d's counters of this parity: ready[kMaxTp] | done[kMaxTp] | ticket
  int tp, my_rank, rows, rows_per_rank, hidden;
  float eps;
  uint64_t budget_ns;
  int* status;
};

template <typename T>
__device__ __forceinline__ uint4 mm_ld_reduce8(const void* p);
template <>
__device__ __forceinline__ uint4 mm_ld_reduce8<__nv_bfloat16>(const void* p) { return ptx::multimem_ld_reduce_bf16x8(p); }
template <>
__device__ __forceinline__ uint4 mm_ld_reduce8<__half>(const void* p) { return ptx::multimem_ld_reduce_f16x8(p); }

constexpr int kArNormVecs = 4;  // 16-byte vectors per thread: hidden <= 256 threads x 4 x 8 = 8192

template <typename T>
__global__ void __launch_bounds__(256) ar_add_norm_mm_kernel(const ArNormParams p) {
  __shared__ float red[33];
  __shared__ int s_ok;
  uint32_t* mine = p.flags[p.my_rank];
  // tell every rank that this rank's partial is complete (it was written by earlier kernels of this stream)
  if (blockIdx.x == 0 && threadIdx.x < p.tp) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.flags[threadIdx.x] + p.my_rank, 1u);
  }
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int s = 0; s < p.tp; ++s)
      if (!ptx::bounded_flag_wait_ge(mine + s, 1u, p.budget_ns)) ok = 0;
    if (!ok && p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
    s_ok = ok;
  }
  __syncthreads();
  const int row = p.my_rank * p.rows_per_rank + blockIdx.x;
  if (s_ok && blockIdx.x < p.rows_per_rank && row < p.rows) {
    const int H = p.hidden, nvec = H >> 3;
    const int64_t roff = static_cast<int64_t>(row) * H;
    const T* xm = reinterpret_cast<const T*>(p.x_mc) + roff;
    const T* rl = p.res_local ? reinterpret_cast<const T*>(p.res_local) + roff : nullptr;
    float v[kArNormVecs][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kArNormVecs; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        unpack8<T>(mm_ld_reduce8<T>(xm + i * 8), v[k]);
        if (rl) {
          float f[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(rl + i * 8), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[k][j] += f[j];
        }
        // the residual stream is kept in 16 bits: normalise what is stored
        const uint4 packed = pack8<T>(v[k]);
        ptx::multimem_st_v4(reinterpret_cast<T*>(p.res_mc) + roff + i * 8, packed);
        unpack8<T>(packed, v[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[k][j] * v[k][j];
      }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / static_cast<float>(H) + p.eps);
    const T* w = reinterpret_cast<const T*>(p.norm_w);
#pragma unroll
    for (int k = 0; k < kArNormVecs; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        float g[8];
        unpack8<T>(__ldg(reinterpret_cast<const uint4*>(w) + i), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[k][j] = v[k][j] * scale * g[j];
        ptx::multimem_st_v4(reinterpret_cast<T*>(p.xn_mc) + roff + i * 8, pack8<T>(v[k]));
      }
    }
  }
  // the last block of this rank: tell every rank that this rank's rows are written, wait for everybody's, re-arm
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t t = ptx::atom_add_acq_rel_gpu(mine + 2 * kMaxTp, 1u);
    s_ok = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_ok) {
    if (threadIdx.x < p.tp) {
      ptx::fence_acq_rel_sys();
      ptx::red_add_release_sys(p.flags[threadIdx.x] + kMaxTp + p.my_rank, 1u);
      if (!ptx::bounded_flag_wait_ge(mine + kMaxTp + threadIdx.x, 1u, p.budget_ns)) {
        if (p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
      }
    }
    __syncthreads();
    if (threadIdx.x < p.tp) {
      mine[threadIdx.x] = 0;
      mine[kMaxTp + threadIdx.x] = 0;
    }
    if (threadIdx.x == 0) mine[2 * kMaxTp] = 0;
    __threadfence_system();
  }
}

// Small all-gather over peer memory: every rank stores its n bytes into slot [my_rank] of every rank's receive
// area and bumps a counter there; after the (bounded) wait for all tp counters the area holds everybody's piece.
// One block; for (value, index) pairs of a sharded arg-max and the logit rows of sampled requests.
struct PeerGatherParams {
  const void* x;
  void* slots[kMaxTp];      // slots[d]: rank d's receive area [tp][n bytes]
  uint32_t* flags[kMaxTp];  // flags[d] + src, zero between calls of one parity
  int tp, my_rank;
  int64_t nbytes;           // multiple of 16
  uint64_t budget_ns;
  int* status;
};
__global__ void __launch_bounds__(256) peer_allgather_kernel(const PeerGatherParams p) {
  const int64_t nvec = p.nbytes >> 4;
  const uint4* x = reinterpret_cast<const uint4*>(p.x);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = x[i];
    for (int d = 0; d < p.tp; ++d)
      ptx::st_na_v4(reinterpret_cast<uint8_t*>(p.slots[d]) + static_cast<int64_t>(p.my_rank) * p.nbytes + (i << 4), v);
  }
  __threadfence_system();
  __syncthreads();
  uint32_t* mine = p.flags[p.my_rank];
  if (threadIdx.x < p.tp) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.flags[threadIdx.x] + p.my_rank, 1u);
  }
  // the last block waits for every source's blocks and re-arms the counters
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const uint32_t t = ptx::atom_add_acq_rel_gpu(mine + kMaxTp, 1u);
    s_last = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.tp) {
      if (!ptx::bounded_flag_wait_ge(mine + threadIdx.x, gridDim.x, p.budget_ns)) {
        if (p.status) atomicCAS(p.status, 0, kStatusTimeoutFlag);
      }
    }
    __syncthreads();
    if (threadIdx.x < p.tp) mine[threadIdx.x] = 0;
    if (threadIdx.x == 0) mine[kMaxTp] = 0;
    __threadfence_system();
  }
}

}  // namespace blitz

extern "C" {

// One-kernel one-shot all-reduce (see allreduce_fused_kernel).  flags[d]: peer pointer to rank d's uint32[tp][64]
// per-block arrival counters, zero at start.  Same slots / parity rules as blitz_allreduce_oneshot.
int blitz_allreduce_fused(const void* x, void* const* slots, uint32_t* const* flags, void* out, int tp, int my_rank,
                          int64_t n, uint64_t budget_ns, int* status, int dtype, cudaStream_t stream) {
  using namespace blitz;
  if (n <= 0) return 0;
  if (tp < 1 || tp > kMaxTp || (n & 7)) return -1;
  OneShotParams p;
  p.x = x; p.out = out; p.tp = tp; p.my_rank = my_rank; p.n = n; p.want = 0; p.budget_ns = budget_ns; p.status = status;
  for (int d = 0; d < kMaxTp; ++d) {
    p.slots[d] = d < tp ? slots[d] : nullptr;
    p.flags[d] = d < tp ? flags[d] : nullptr;
  }
  const int64_t nvec = n >> 3;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > kArBlocks) blocks = kArBlocks;
  if (dtype == 1) allreduce_fused_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(p);
  else allreduce_fused_kernel<__half><<<blocks, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}


// All-reduce + residual add + RMSNorm through the switch (see ar_add_norm_mm_kernel).  x_mc / res_mc / xn_mc:
// multicast addresses of the symmetric buffers; res_local: this rank's residual copy or null; flags[d]: rank d's
// counter block of this call's parity (2 * kMaxTp + 1 words, zero at start).  rows_per_rank = ceil(rows / tp).
int blitz_ar_add_norm_mm(const void* x_mc, const void* res_local, void* res_mc, void* xn_mc, const void* norm_w,
                         uint32_t* const* flags, int tp, int my_rank, int rows, int hidden, float eps,
                         uint64_t budget_ns, int* status, int dtype, cudaStream_t stream) {
  using namespace blitz;
  if (rows <= 0) return 0;
  if (tp < 1 || tp > kMaxTp || (hidden & 7) || hidden > 256 * kArNormVecs * 8 || !x_mc || !res_mc || !xn_mc) return -1;
  ArNormParams p;
  p.x_mc = x_mc; p.res_local = res_local; p.res_mc = res_mc; p.xn_mc = xn_mc; p.norm_w = norm_w;
  for (int d = 0; d < kMaxTp; ++d) p.flags[d] = d < tp ? flags[d] : nullptr;
  p.tp = tp; p.my_rank = my_rank; p.rows = rows; p.rows_per_rank = (rows + tp - 1) / tp; p.hidden = hidden;
  p.eps = eps; p.budget_ns = budget_ns; p.status = status;
  // every rank launches the same grid (the counters count ranks, not blocks), even where its last rows are padding
  if (dtype == 1) ar_add_norm_mm_kernel<__nv_bfloat16><<<p.rows_per_rank, 256, 0, stream>>>(p);
  else ar_add_norm_mm_kernel<__half><<<p.rows_per_rank, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

// All-gather of nbytes (multiple of 16) per rank into every rank's receive area (see peer_allgather_kernel).
// flags[d]: rank d's kMaxTp + 1 counters of this call's parity, zero at start.
int blitz_peer_allgather(const void* x, void* const* slots, uint32_t* const* flags, int tp, int my_rank, int64_t nbytes,
                         uint64_t budget_ns, int* status, cudaStream_t stream) {
  using namespace blitz;
  if (nbytes <= 0) return 0;
  if (tp < 1 || tp > kMaxTp || (nbytes & 15)) return -1;
  PeerGatherParams p;
  p.x = x; p.tp = tp; p.my_rank = my_rank; p.nbytes = nbytes; p.budget_ns = budget_ns; p.status = status;
  for (int d = 0; d < kMaxTp; ++d) {
    p.slots[d] = d < tp ? slots[d] : nullptr;
    p.flags[d] = d < tp ? flags[d] : nullptr;
  }
  int blocks = (int)(((nbytes >> 4) + 255) / 256);
  if (blocks > 32) blocks = 32;
  peer_allgather_kernel<<<blocks, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

using namespace blitz;

// stage: local [tp][hidden / 8][rows_per_rank][8] (the layout the GEMM push epilogue writes); flag_rs: local
// uint32[64 blocks][8 sources] + a ticket word (zero at start); tiles_n: tiles per 128 GEMM rows each source pushes;
// xg / flag_ag: tp peer pointers each.  rows_valid <= rows_per_rank local rows are processed.
int blitz_rs_reduce_norm(const void* stage, uint32_t* flag_rs, uint32_t tiles_n, void* residual,
                         const void* norm_w, void* const* xg, uint32_t* const* flag_ag, int tp, int my_rank,
                         int rows_per_rank, int rows_valid, int total_rows, int hidden, float eps, uint64_t budget_ns,
                         int* status, int dtype, cudaStream_t stream) {
  if (rows_valid <= 0) return 0;
  if (tp < 1 || tp > kMaxTp || (hidden & 7) || rows_per_rank > kRsBlocks * 128) return -1;
  RsReduceParams p;
  p.stage = stage; p.flag_rs = flag_rs; p.tiles_n = tiles_n; p.total_rows = total_rows; p.residual = residual;
  p.norm_w = norm_w;
  for (int d = 0; d < kMaxTp; ++d) {
    p.xg[d] = d < tp ? xg[d] : nullptr;
    p.flag_ag[d] = d < tp ? flag_ag[d] : nullptr;
  }
  p.tp = tp; p.my_rank = my_rank; p.rows_per_rank = rows_per_rank; p.rows_valid = rows_valid; p.hidden = hidden;
  p.eps = eps; p.budget_ns = budget_ns; p.status = status;
  if (dtype == 1) rs_reduce_norm_kernel<__nv_bfloat16><<<rows_valid, 256, 0, stream>>>(p);
  else rs_reduce_norm_kernel<__half><<<rows_valid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

int blitz_flags_zero(uint32_t* flags, int n, cudaStream_t stream) {
  if (n <= 0 || n > 1024) return -1;
  flags_zero_kernel<<<1, 1024, 0, stream>>>(flags, n);
  return (int)cudaGetLastError();
}

// One-shot all-reduce of n elements (multiple of 8).  slots[d]: peer pointer to rank d's receive area of tp * n
// elements; flags[d]: peer pointer to rank d's uint32[kMaxTp + 1] arrival counters (+ a ticket word), zero at start.  `expect` = number of push blocks per
// rank (returned through *blocks_out on the first call with expect = 0 is not needed: it equals the grid used here).
int blitz_allreduce_oneshot(const void* x, void* const* slots, uint32_t* const* flags, void* out, int tp, int my_rank,
                            int64_t n, uint64_t budget_ns, int* status, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (tp < 1 || tp > kMaxTp || (n & 7)) return -1;
  OneShotParams p;
  p.x = x; p.out = out; p.tp = tp; p.my_rank = my_rank; p.n = n; p.want = 0; p.budget_ns = budget_ns; p.status = status;
  for (int d = 0; d < kMaxTp; ++d) {
    p.slots[d] = d < tp ? slots[d] : nullptr;
    p.flags[d] = d < tp ? flags[d] : nullptr;
  }
  const int64_t nvec = n >> 3;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > 64) blocks = 64;
  if (dtype == 1) {
    oneshot_push_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(p);
    oneshot_reduce_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(p, (uint32_t)blocks);
  } else {
    oneshot_push_kernel<__half><<<blocks, 256, 0, stream>>>(p);
    oneshot_reduce_kernel<__half><<<blocks, 256, 0, stream>>>(p, (uint32_t)blocks);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
