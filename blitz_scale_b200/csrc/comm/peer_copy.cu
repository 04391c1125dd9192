// In-kernel NVLink data paths over peer-mapped (symmetric) memory:
//
//  * peer_copy_units : stream a list of byte ranges ("units": embed | layer i | head for parameters,
//    one unit for an activation slot) from this GPU to the same offsets of up to 8 destination GPUs,
//    either with one NVLS `multimem.st` per 16 bytes (the switch replicates the store to every GPU
//    bound to the multicast address) or with one plain peer store per destination; when a unit is
//    complete the last CTA bumps that unit's readiness flag in every destination with a
//    system-scope release.  Several sources can share the work: source s of k copies byte stripe s
//    of every unit and the unit is ready when its flag has been bumped k times.
//    Replaces the NCCL send/recv chain and ring of the reference's NVLink broadcaster
//    (src/blitz/nccl_bcastor.h:105-373), its per-layer RDMA parameter sends
//    (src/blitz/stub.h:534-825) and the activation hand-off of live execution
//    (src/blitz/activation_manager.h:111-168): destinations run nothing, they only read flags.
//
//  * kv_push : the prefill GPU stores a batch's prompt pages straight into the decode GPU's paged
//    pool, translating source page ids to the destination's page ids, for a layer range
//    (all / first k / remaining layers), with one readiness flag per layer.  Replaces the
//    per-(page, layer) RDMA operations of src/blitz/migration_manager.h:436-536.
//
//  * flag_wait / flag_set : bounded device-side wait on a readiness flag (a timeout writes a status
//    code and returns, it never traps) and a release store, for stream-ordered hand-offs.
//
// All loads are local; all remote traffic is stores (push model), so consumers only ever read their
// own memory and TMA-fed kernels never touch peer memory.
#include "../kernels/ptx.cuh"

namespace blitz {

constexpr int kMaxDst = 8;
constexpr int kMaxUnits = 96;

struct CopyUnits {
  int64_t offset[kMaxUnits];
  int64_t nbytes[kMaxUnits];
};
struct PeerPtrs {
  uint8_t* base[kMaxDst];
  uint32_t* flags[kMaxDst];
};

template <bool MULTIMEM>
__global__ void __launch_bounds__(256)
peer_copy_units_kernel(const uint8_t* __restrict__ src_base, PeerPtrs dst, int n_dst, uint8_t* mc_base,
                       CopyUnits units, int n_units, int flag_index0, int stripe, int n_stripes,
                       uint32_t* __restrict__ tickets) {
  constexpr int kUnroll = 8;
  __shared__ uint32_t s_last;
  for (int u = 0; u < n_units; ++u) {
    // this source's stripe of the unit, in 16-byte vectors
    const int64_t nvec_total = units.nbytes[u] >> 4;
    const int64_t per = (nvec_total + n_stripes - 1) / n_stripes;
    const int64_t v_beg = min(nvec_total, per * stripe), v_end = min(nvec_total, per * (stripe + 1));
    const uint4* src = reinterpret_cast<const uint4*>(src_base + units.offset[u]);
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x * kUnroll;
    for (int64_t base = v_beg + static_cast<int64_t>(blockIdx.x) * blockDim.x * kUnroll; base < v_end; base += step) {
      uint4 v[kUnroll];
      // multimem: every warp owns one contiguous 4 KB run (the switch replicates larger contiguous bursts better);
      // peer stores: the CTA's threads interleave 512-byte rows
      const int64_t t0 = MULTIMEM ? base + (threadIdx.x >> 5) * (32 * kUnroll) + (threadIdx.x & 31) : base + threadIdx.x;
      const int64_t tstep = MULTIMEM ? 32 : blockDim.x;
#pragma unroll
      for (int k = 0; k < kUnroll; ++k) {
        const int64_t i = t0 + k * tstep;
        if (i < v_end) v[k] = ptx::ld_nc_na_v4(src + i);
      }
#pragma unroll
      for (int k = 0; k < kUnroll; ++k) {
        const int64_t i = t0 + k * tstep;
        if (i < v_end) {
          if (MULTIMEM) {
            ptx::multimem_st_v4(mc_base + units.offset[u] + (i << 4), v[k]);
          } else {
            for (int d = 0; d < n_dst; ++d) ptx::st_na_v4(dst.base[d] + units.offset[u] + (i << 4), v[k]);
          }
        }
      }
    }
    // unit done for this CTA: publish, and let the last CTA bump the destinations' flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t t = ptx::atom_add_acq_rel_gpu(&tickets[u], 1u);
      s_last = (t == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x < n_dst) {
      ptx::fence_acq_rel_sys();
      ptx::red_add_release_sys(dst.flags[threadIdx.x] + flag_index0 + u, 1u);
    }
  }
}

struct KvPushParams {
  const uint8_t* src_base;
  uint8_t* dst_base;
  const int32_t* src_pages;
  const int32_t* dst_pages;
  int n_pages, layer_begin, layer_end;
  int64_t page_bytes, src_layer_stride, dst_layer_stride;
  int src_max_pages, dst_max_pages;
  uint32_t* dst_flags;   // one per layer (indexed by absolute layer), bumped by 1 per push
  uint32_t* tickets;     // one per layer in [layer_begin, layer_end), zero on entry
  int ctas_per_layer;
  const int32_t* dst_count;  // optional: number of page ids the destination published; must equal n_pages
  int* status;
};

// grid = (ctas_per_layer, layers in range): the CTAs of one layer split its pages' vectors evenly.
__global__ void __launch_bounds__(256) kv_push_kernel(const KvPushParams p) {
  __shared__ uint32_t s_last;
  const int layer = p.layer_begin + blockIdx.y;
  const int64_t vec_per_page = p.page_bytes >> 4;
  // the two ends built their page lists independently: if they disagree on the count, page i of one side does not
  // face page i of the other, so nothing is copied and the layer is not flagged (the receiver's wait reports it)
  if (p.dst_count != nullptr && *reinterpret_cast<const volatile int32_t*>(p.dst_count) != p.n_pages) {
    if (p.status && threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadIndex);
    return;
  }
  const int64_t total = vec_per_page * p.n_pages;
  constexpr int kUnroll = 4;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x * kUnroll;
  for (int64_t base = static_cast<int64_t>(blockIdx.x) * blockDim.x * kUnroll; base < total; base += step) {
    uint4 v[kUnroll];
    uint4* dptr[kUnroll];
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      const int64_t i = base + k * blockDim.x + threadIdx.x;
      dptr[k] = nullptr;
      if (i < total) {
        const int pg = static_cast<int>(i / vec_per_page);
        const int64_t within = i % vec_per_page;
        const int sp = p.src_pages[pg], dp = p.dst_pages[pg];
        if (sp == -1 || dp == -1) {
          // a request one side no longer holds: its entries stay in both lists so that the others keep their places
        } else if (sp < 0 || sp >= p.src_max_pages || dp < 0 || dp >= p.dst_max_pages) {
          if (p.status) atomicCAS(p.status, 0, kStatusBadIndex);
        } else {
          v[k] = ptx::ld_nc_na_v4(p.src_base + layer * p.src_layer_stride + sp * p.page_bytes + (within << 4));
          dptr[k] = reinterpret_cast<uint4*>(p.dst_base + layer * p.dst_layer_stride + dp * p.page_bytes + (within << 4));
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kUnroll; ++k)
      if (dptr[k]) ptx::st_na_v4(dptr[k], v[k]);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t t = ptx::atom_add_acq_rel_gpu(&p.tickets[blockIdx.y], 1u);
    s_last = (t == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0 && p.dst_flags) {
    ptx::fence_acq_rel_sys();
    ptx::red_add_release_sys(p.dst_flags + layer, 1u);
  }
}

__global__ void flag_wait_kernel(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status) {
  if (!ptx::bounded_flag_wait_ge(flag, want, budget_ns)) {
    if (status) atomicCAS(status, 0, kStatusTimeoutFlag);
  }
}
// Wait for an exact value: a transfer tag that a stale, larger tag of an earlier transfer must not satisfy.
__global__ void flag_wait_eq_kernel(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status) {
  if (ptx::ld_acquire_sys(flag) == want) return;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t it = 0;
  while (ptx::ld_acquire_sys(flag) != want) {
    if ((++it & 15u) == 0) {
      if (ptx::globaltimer_ns() - t0 > budget_ns) {
        if (status) atomicCAS(status, 0, kStatusTimeoutFlag);
        return;
      }
      __nanosleep(64);
    }
  }
}
__global__ void flag_set_kernel(uint32_t* flag, uint32_t value, int add) {
  ptx::fence_acq_rel_sys();
  if (add) ptx::red_add_release_sys(flag, value);
  else ptx::st_release_sys(flag, value);
}

}  // namespace blitz

extern "C" {
using namespace blitz;

// Copy `n_units` byte ranges (offset, nbytes; multiples of 16) of the local region at src_base to the
// same offsets of every destination region.  dst_bases / dst_flags: n_dst peer pointers (region base,
// flag array).  mc_base: multicast address of the region or null (null = plain peer stores).
// Flags flag_index0 + u are incremented by 1 per call and stripe.  tickets: n_units uint32 of local
// scratch that must be zero on entry (the caller memsets it on the same stream).
int blitz_peer_copy_units(const void* src_base, void* const* dst_bases, uint32_t* const* dst_flags, int n_dst,
                          void* mc_base, const int64_t* unit_offsets, const int64_t* unit_nbytes, int n_units,
                          int flag_index0, int stripe, int n_stripes, uint32_t* tickets, int num_ctas,
                          cudaStream_t stream) {
  if (n_units <= 0) return 0;
  if (n_dst < 1 || n_dst > kMaxDst || n_units > kMaxUnits || n_stripes < 1 || stripe < 0 || stripe >= n_stripes)
    return -1;
  CopyUnits cu;
  for (int u = 0; u < n_units; ++u) {
    if ((unit_offsets[u] & 15) || (unit_nbytes[u] & 15)) return -1;
    cu.offset[u] = unit_offsets[u];
    cu.nbytes[u] = unit_nbytes[u];
  }
  PeerPtrs pp;
  for (int d = 0; d < kMaxDst; ++d) {
    pp.base[d] = d < n_dst ? reinterpret_cast<uint8_t*>(dst_bases[d]) : nullptr;
    pp.flags[d] = d < n_dst ? dst_flags[d] : nullptr;
  }
  if (num_ctas <= 0) num_ctas = 64;
  if (mc_base)
    peer_copy_units_kernel<true><<<num_ctas, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src_base), pp, n_dst,
                                                              reinterpret_cast<uint8_t*>(mc_base), cu, n_units,
                                                              flag_index0, stripe, n_stripes, tickets);
  else
    peer_copy_units_kernel<false><<<num_ctas, 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(src_base), pp, n_dst,
                                                               nullptr, cu, n_units, flag_index0, stripe, n_stripes,
                                                               tickets);
  return (int)cudaGetLastError();
}

// Push pages src_pages[i] -> dst_pages[i] (device int32 arrays) of layers [layer_begin, layer_end) from the
// local pool at src_base into the peer pool at dst_base.  page_bytes = K plane + V plane of one page of one
// layer.  dst_flags (peer pointer, may be null): one counter per layer, +1 when the layer's pages landed.
// tickets: (layer_end - layer_begin) zeroed uint32 of local scratch.  dst_count (may be null): address of the
// number of ids the destination published; when it differs from n_pages the push copies nothing and reports
// kStatusBadIndex.
int blitz_kv_push(const void* src_base, void* dst_base, const int32_t* src_pages, const int32_t* dst_pages,
                  int n_pages, int layer_begin, int layer_end, int64_t page_bytes, int64_t src_layer_stride,
                  int64_t dst_layer_stride, int src_max_pages, int dst_max_pages, uint32_t* dst_flags,
                  uint32_t* tickets, int ctas_per_layer, const int32_t* dst_count, int* status, cudaStream_t stream) {
  if (n_pages <= 0 || layer_end <= layer_begin) return 0;
  if (page_bytes & 15) return -1;
  KvPushParams p;
  p.src_base = reinterpret_cast<const uint8_t*>(src_base);
  p.dst_base = reinterpret_cast<uint8_t*>(dst_base);
  p.src_pages = src_pages; p.dst_pages = dst_pages; p.n_pages = n_pages;
  p.layer_begin = layer_begin; p.layer_end = layer_end; p.page_bytes = page_bytes;
  p.src_layer_stride = src_layer_stride; p.dst_layer_stride = dst_layer_stride;
  p.src_max_pages = src_max_pages; p.dst_max_pages = dst_max_pages;
  p.dst_flags = dst_flags; p.tickets = tickets; p.status = status; p.dst_count = dst_count;
  if (ctas_per_layer <= 0) {
    const int64_t work = (page_bytes >> 4) * n_pages;  // vectors per layer
    int64_t c = (work + 256 * 4 * 4 - 1) / (256 * 4 * 4);
    ctas_per_layer = (int)(c < 1 ? 1 : (c > 16 ? 16 : c));
  }
  p.ctas_per_layer = ctas_per_layer;
  dim3 grid(ctas_per_layer, layer_end - layer_begin);
  kv_push_kernel<<<grid, 256, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

int blitz_flag_wait(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status, cudaStream_t stream) {
  flag_wait_kernel<<<1, 1, 0, stream>>>(flag, want, budget_ns, status);
  return (int)cudaGetLastError();
}
int blitz_flag_wait_eq(const uint32_t* flag, uint32_t want, uint64_t budget_ns, int* status, cudaStream_t stream) {
  flag_wait_eq_kernel<<<1, 1, 0, stream>>>(flag, want, budget_ns, status);
  return (int)cudaGetLastError();
}
int blitz_flag_set(uint32_t* flag, uint32_t value, int add, cudaStream_t stream) {
  flag_set_kernel<<<1, 1, 0, stream>>>(flag, value, add);
  return (int)cudaGetLastError();
}

}  // extern "C"
