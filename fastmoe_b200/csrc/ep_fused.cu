// Dispatch permute fused with the expert-parallel exchange: every routed copy of a token
// row is stored directly into the receive buffer of the GPU that owns its expert, at the
// row where that GPU's grouped GEMM expects it. Plain 16-byte peer stores over NVLink
// (no multicast, no TMA): the copy IS the all-to-all. Replaces, for several GPUs,
// x_flat[reverse_map] + dist.all_to_all_single + the receive-side split of
// polkadot21/fastmoe (src/fastmoe/models/tiny_model.py:133, :210-216, :282-294).
#include "common.cuh"

namespace fmoe {

// fmoe_tune "peer_ctas_per_sm": CTAs per SM of the dispatch kernel when it sends ONE group of
// experts (a pass that is meant to run beside the persistent grouped GEMM): few, so that the
// GEMM's CTA, which needs an SM's whole shared memory and a third of its registers, always
// finds room beside them. A pass over all experts runs alone and uses one CTA per work item.
int g_peer_ctas_per_sm = 2;

struct PeerPermuteArgs {
  const void* x;
  int64_t x_row_stride;
  const int64_t* topk_idx;
  const int32_t* slot_of;
  const int64_t* local_offsets;
  const int64_t* dst_row0;
  const int64_t* peer_bases;
  void* ret_local;  // optional: this GPU's return buffer, [T*K, D], one row per sorted slot
  int64_t T, D, dvec, cap_rows;
  int K, E, experts_per_rank, tiles;
  int local_lo, local_hi;  // only copies for experts whose index on their owner lies in [lo, hi) travel
  int32_t* status;
};

template <int DT, int V>
__global__ void __launch_bounds__(256) permute_peer_kernel(const PeerPermuteArgs a) {
  using El = Elem<DT>;
  using Ty = typename El::type;
  const int64_t items = a.T * a.tiles;
  int flags = 0;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t t = item / a.tiles;
    const int tile = static_cast<int>(item - t * a.tiles);
    const uint4* xrow = reinterpret_cast<const uint4*>(reinterpret_cast<const Ty*>(a.x) + t * a.x_row_stride);
    const bool filtered = a.local_lo > 0 || a.local_hi < a.experts_per_rank;
    if (filtered) {  // a pass over one group of experts: skip the tokens it has nothing for
      bool any = false;
      for (int k = 0; k < a.K; ++k) {
        const int64_t e = a.topk_idx[t * a.K + k];
        const int le = (e >= 0 && e < a.E) ? static_cast<int>(e % a.experts_per_rank) : -1;
        any |= le >= a.local_lo && le < a.local_hi;
      }
      if (!any) continue;
    }
    uint4 val[V];
    int64_t col[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      col[v] = (static_cast<int64_t>(tile) * V + v) * blockDim.x + threadIdx.x;
      if (col[v] < a.dvec) val[v] = filtered ? xrow[col[v]] : ld_stream16(xrow + col[v]);  // a later pass reads it again
    }
    for (int k0 = 0; k0 < a.K; k0 += 8) {
      uint4* drow[8];  // resolve the destinations together: one round of lookups, not eight
      bool dropped[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        drow[u] = nullptr;
        dropped[u] = false;
        if (k0 + u < a.K) {
          const int64_t e = a.topk_idx[t * a.K + k0 + u];
          const int32_t slot = a.slot_of[t * a.K + k0 + u];
          const int le = (e >= 0 && e < a.E) ? static_cast<int>(e % a.experts_per_rank) : -1;
          if (le >= a.local_lo && le < a.local_hi && slot >= 0) {
            const int64_t row = a.dst_row0[e] + (slot - a.local_offsets[e]);
            if (row >= 0 && row < a.cap_rows) {
              char* base = reinterpret_cast<char*>(a.peer_bases[e / a.experts_per_rank]);
              drow[u] = reinterpret_cast<uint4*>(base + row * a.D * El::kBytes);
            } else {
              // The receive buffer is full: the copy is dropped. Nobody will send a result for
              // it, so its row of this GPU's return buffer is cleared here: the dropped copy
              // then adds zero to its token instead of whatever an earlier call left there.
              flags |= FMOE_STATUS_BAD_INDEX;
              if (a.ret_local != nullptr && slot < a.T * a.K) {
                drow[u] = reinterpret_cast<uint4*>(static_cast<char*>(a.ret_local) +
                                                   static_cast<int64_t>(slot) * a.D * El::kBytes);
                dropped[u] = true;
              }
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (drow[u] == nullptr) continue;
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (col[v] < a.dvec) drow[u][col[v]] = dropped[u] ? make_uint4(0, 0, 0, 0) : val[v];
      }
    }
  }
  if (flags != 0 && a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, flags);
}

// ---- placement arithmetic of the exchange ---------------------------------------------------
// From everybody's per-expert counts C[s, g] (rows that rank s routes to global expert g;
// experts sharded contiguously, el per rank) every rank derives, without a host round trip,
// where its rows go, what its experts receive and where every received row came from. A
// rank's receive buffer is expert-major with the sources in rank order inside an expert:
// segment j = e * world + s holds the rows rank s sends to local expert e. Rows past
// cap_rows do not exist: senders drop them, and the counts handed to the GEMMs stop there.

constexpr int kLayoutThreads = 1024;

// Exclusive prefix sum over the block's threads (int64); `total` receives the block sum.
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t* warp_sums, int64_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int64_t n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  __syncthreads();  // warp_sums may still be read from an earlier scan
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int64_t w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
    int64_t wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int64_t n = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d) wi += n;
    }
    warp_sums[lane] = wi - w;  // exclusive over warps
    if (lane == 31) warp_sums[32] = wi;
  }
  __syncthreads();
  if (total != nullptr) *total = warp_sums[32];
  return warp_sums[warp] + incl - v;
}

struct LayoutArgs {
  const int64_t* C;  // [world, E]
  int64_t* dst_row0;       // [E]
  int64_t* counts_local;   // [el]
  int64_t* offsets_local;  // [el]
  int64_t* rows_used;      // [1]
  int64_t* seg_end;        // [E] scratch: end row of segment j in this rank's receive buffer
  int64_t* seg_delta;      // [E] scratch: (slot in the source's sorted rows) - (receive row) for segment j
  int64_t cap_rows;
  int world, E, el, rank;
  int32_t* status;
};

__global__ void __launch_bounds__(kLayoutThreads) ep_layout_tables_kernel(const LayoutArgs a) {
  __shared__ int64_t warp_sums[33];
  __shared__ int64_t col_excl[1024];  // exclusive prefix over global experts of the column sums
  const int g = threadIdx.x;          // one thread per global expert, and later per segment
  auto count = [&](int s, int e) -> int64_t {
    const int64_t c = a.C[static_cast<int64_t>(s) * a.E + e];
    return c > 0 ? c : 0;
  };
  // column sums (what expert g receives in all) and the part of them that precedes this rank
  int64_t col = 0, before_me = 0;
  if (g < a.E) {
    for (int s = 0; s < a.world; ++s) {
      const int64_t c = count(s, g);
      col += c;
      if (s < a.rank) before_me += c;
    }
  }
  const int64_t excl = block_exclusive_scan(col, warp_sums, nullptr);
  if (g < a.E) col_excl[g] = excl;
  __syncthreads();
  if (g < a.E) {
    const int d = g / a.el;
    const int64_t in_dest = excl - col_excl[d * a.el];  // first row of expert g on its owner
    a.dst_row0[g] = in_dest + before_me;
    if (d == a.rank) {
      const int e = g - d * a.el;
      const int64_t room = a.cap_rows - in_dest;
      a.offsets_local[e] = in_dest < a.cap_rows ? in_dest : a.cap_rows;
      a.counts_local[e] = room <= 0 ? 0 : (col < room ? col : room);
      if (e == a.el - 1) {
        const int64_t total = in_dest + col;
        *a.rows_used = total < a.cap_rows ? total : a.cap_rows;
        if (total > a.cap_rows && a.status != nullptr) atomicOr(a.status, FMOE_STATUS_BAD_INDEX);
      }
    }
  }
  // segments of this rank's receive buffer: j = e * world + s
  const int j = threadIdx.x;
  const int e = j / a.world, s = j - e * a.world;
  const int64_t size = j < a.E ? count(s, a.rank * a.el + e) : 0;
  const int64_t start = block_exclusive_scan(size, warp_sums, nullptr);
  if (j < a.E) a.seg_end[j] = start + size;
  // where segment j begins in its source's sorted rows: prefix of C[s, :] up to my expert
  for (int src = 0; src < a.world; ++src) {
    const int64_t c = g < a.E ? count(src, g) : 0;
    const int64_t origin = block_exclusive_scan(c, warp_sums, nullptr);
    __syncthreads();
    if (g < a.E) col_excl[g] = origin;  // reused as a staging row
    __syncthreads();
    if (j < a.E && s == src) a.seg_delta[j] = col_excl[a.rank * a.el + e] - start;
  }
}

// row_ptrs[i] = address, in the return buffer of the rank that sent receive row i, of the
// slot that row came from; 0 for rows the buffer does not hold. Up to two address tables
// (forward results, gradients) are filled from two sets of base addresses.
__global__ void __launch_bounds__(256)
    ep_layout_rows_kernel(const int64_t* __restrict__ seg_end, const int64_t* __restrict__ seg_delta,
                          const int64_t* __restrict__ rows_used, const int64_t* __restrict__ bases0,
                          const int64_t* __restrict__ bases1, int64_t* __restrict__ ptrs0,
                          int64_t* __restrict__ ptrs1, int64_t cap_rows, int64_t row_bytes, int world, int nseg) {
  extern __shared__ int64_t ends[];
  for (int j = threadIdx.x; j < nseg; j += blockDim.x) ends[j] = seg_end[j];
  __syncthreads();
  const int64_t used = *rows_used;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < cap_rows;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t p0 = 0, p1 = 0;
    if (i < used) {
      int lo = 0, hi = nseg;  // first segment whose end lies beyond row i
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (ends[mid] > i) hi = mid; else lo = mid + 1;
      }
      if (lo < nseg) {
        const int64_t byte = (i + seg_delta[lo]) * row_bytes;
        const int src = lo % world;
        p0 = bases0[src] + byte;
        if (bases1 != nullptr) p1 = bases1[src] + byte;
      }
    }
    ptrs0[i] = p0;
    if (ptrs1 != nullptr) ptrs1[i] = p1;
  }
}

// ---- barrier between the GPUs of the exchange -------------------------------------------------
// Thread p tells rank p that this rank's earlier work on the stream is complete (a release
// store of the call's sequence number into slot `rank` of p's flag array, over NVLink) and
// waits until rank p has said the same (its number appears in slot p of this rank's own
// array). Flags only grow, so nothing is ever reset. The wait is bounded by a clock: a peer
// that never arrives costs `timeout_ns`, sets FMOE_STATUS_WAIT_TIMEOUT and the kernel returns.
__global__ void __launch_bounds__(32)
    peer_barrier_kernel(const int64_t* __restrict__ flag_bases, int world, int rank, int32_t seq,
                        unsigned long long timeout_ns, int32_t* status) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();  // everything this stream did before the barrier, peer stores included
  int32_t* theirs = reinterpret_cast<int32_t*>(flag_bases[p]) + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
  const int32_t* mine = reinterpret_cast<const int32_t*>(flag_bases[rank]) + p;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (uint32_t spin = 0;; ++spin) {
    int32_t seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    // the peer is at this barrier or already past it (sequence numbers may wrap)
    if (static_cast<int32_t>(static_cast<uint32_t>(seen) - static_cast<uint32_t>(seq)) >= 0) break;
    if ((spin & 255u) == 255u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > timeout_ns) {
        if (status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __threadfence_system();
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_peer_barrier(const int64_t* flag_bases, int64_t world, int64_t rank, int32_t seq,
                                 int64_t timeout_ms, int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_peer_barrier");
  FMOE_REQUIRE(world > 0 && world <= 32 && rank >= 0 && rank < world && timeout_ms > 0, FMOE_ERR_ARG,
               "fmoe_peer_barrier: bad sizes (world %lld, rank %lld, timeout %lld ms)", (long long)world,
               (long long)rank, (long long)timeout_ms);
  FMOE_REQUIRE(flag_bases != nullptr, FMOE_ERR_ARG, "fmoe_peer_barrier: null pointer argument");
  cudaFuncSetAttribute(peer_barrier_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       cudaSharedmemCarveoutMaxShared);  // see fmoe_permute_peer_fwd
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flag_bases, static_cast<int>(world), static_cast<int>(rank), seq,
      static_cast<unsigned long long>(timeout_ms) * 1000000ull, status);
  return check_launch("peer_barrier_kernel");
}

extern "C" int fmoe_ep_layout(const int64_t* counts_all, int64_t world, int64_t E, int64_t rank, int64_t cap_rows,
                              int64_t row_bytes, const int64_t* ret_bases, const int64_t* grad_ret_bases,
                              int64_t* dst_row0, int64_t* counts_local, int64_t* offsets_local, int64_t* rows_used,
                              int64_t* row_ptrs, int64_t* grad_row_ptrs, int64_t* scratch, int32_t* status,
                              void* stream) {
  FMOE_RANGE("fmoe_ep_layout");
  FMOE_REQUIRE(world > 0 && E > 0 && rank >= 0 && rank < world && cap_rows >= 0 && row_bytes > 0, FMOE_ERR_ARG,
               "fmoe_ep_layout: bad sizes");
  FMOE_REQUIRE(E % world == 0, FMOE_ERR_ARG, "fmoe_ep_layout: E=%lld is not a multiple of world=%lld", (long long)E,
               (long long)world);
  FMOE_REQUIRE(E <= kLayoutThreads, FMOE_ERR_UNSUPPORTED, "fmoe_ep_layout: supports E <= %d", kLayoutThreads);
  FMOE_REQUIRE(counts_all && ret_bases && dst_row0 && counts_local && offsets_local && rows_used && row_ptrs && scratch,
               FMOE_ERR_ARG, "fmoe_ep_layout: null pointer argument");
  FMOE_REQUIRE((grad_ret_bases == nullptr) == (grad_row_ptrs == nullptr), FMOE_ERR_ARG,
               "fmoe_ep_layout: grad_ret_bases and grad_row_ptrs go together");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  LayoutArgs a;
  a.C = counts_all;
  a.dst_row0 = dst_row0;
  a.counts_local = counts_local;
  a.offsets_local = offsets_local;
  a.rows_used = rows_used;
  a.seg_end = scratch;
  a.seg_delta = scratch + E;
  a.cap_rows = cap_rows;
  a.world = static_cast<int>(world);
  a.E = static_cast<int>(E);
  a.el = static_cast<int>(E / world);
  a.rank = static_cast<int>(rank);
  a.status = status;
  ep_layout_tables_kernel<<<1, kLayoutThreads, 0, s>>>(a);
  int rc = check_launch("ep_layout_tables_kernel");
  if (rc != 0 || cap_rows == 0) return rc;
  const int64_t blocks = (cap_rows + 255) / 256;
  const int grid = static_cast<int>(blocks < kNumSMs * 4 ? blocks : kNumSMs * 4);
  ep_layout_rows_kernel<<<grid, 256, static_cast<size_t>(E) * sizeof(int64_t), s>>>(
      a.seg_end, a.seg_delta, rows_used, ret_bases, grad_ret_bases, row_ptrs, grad_row_ptrs, cap_rows, row_bytes,
      a.world, a.E);
  return check_launch("ep_layout_rows_kernel");
}

extern "C" int fmoe_permute_peer_fwd(const void* x, int64_t x_row_stride, const int64_t* topk_idx,
                                     const int32_t* slot_of, const int64_t* local_offsets,
                                     const int64_t* dst_row0, const int64_t* peer_bases, int64_t T,
                                     int64_t K, int64_t D, int64_t E, int64_t experts_per_rank,
                                     int64_t cap_rows, void* ret_local, int64_t local_lo, int64_t local_hi,
                                     int dtype, int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_permute_peer_fwd");
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_permute_peer_fwd: bad dtype %d", dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0 && E > 0 && experts_per_rank > 0 && cap_rows >= 0, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: bad sizes");
  FMOE_REQUIRE(E % experts_per_rank == 0, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: E=%lld is not a multiple of experts_per_rank=%lld", (long long)E,
               (long long)experts_per_rank);
  FMOE_REQUIRE(T * K < (1ll << 31) && E < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_permute_peer_fwd: T*K and E must fit in int32");
  FMOE_REQUIRE(local_lo >= 0 && local_lo <= local_hi && local_hi <= experts_per_rank, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: expert group [%lld, %lld) is not inside [0, %lld)", (long long)local_lo,
               (long long)local_hi, (long long)experts_per_rank);
  if (local_lo == local_hi) return FMOE_OK;
  if (T == 0 || K == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(x && topk_idx && slot_of && local_offsets && dst_row0 && peer_bases, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: null pointer argument");
  FMOE_REQUIRE(x_row_stride >= D, FMOE_ERR_ARG, "fmoe_permute_peer_fwd: x_row_stride < D");
  const int eb = dtype_size(dtype);
  const int kvec = 16 / eb;
  FMOE_REQUIRE(D % kvec == 0 && aligned_to(x, 16) && (x_row_stride * eb) % 16 == 0 && aligned_to(ret_local, 16),
               FMOE_ERR_UNSUPPORTED, "fmoe_permute_peer_fwd: D must be a multiple of %d and x 16-byte aligned", kvec);
  PeerPermuteArgs a;
  a.x = x;
  a.x_row_stride = x_row_stride;
  a.topk_idx = topk_idx;
  a.slot_of = slot_of;
  a.local_offsets = local_offsets;
  a.dst_row0 = dst_row0;
  a.peer_bases = peer_bases;
  a.ret_local = ret_local;
  a.T = T;
  a.D = D;
  a.dvec = D / kvec;
  a.cap_rows = cap_rows;
  a.K = static_cast<int>(K);
  a.E = static_cast<int>(E);
  a.experts_per_rank = static_cast<int>(experts_per_rank);
  a.local_lo = static_cast<int>(local_lo);
  a.local_hi = static_cast<int>(local_hi);
  a.status = status;
  // same tile shapes as the local permute: threads x vectors that divide a row evenly
  int threads = 256, v = 2;
  int64_t best_tiles = -1;
  double best_eff = -1.0;
  for (int th = 32; th <= 256; th += 32)
    for (int vv = 1; vv <= 2; vv *= 2) {
      const int64_t span = static_cast<int64_t>(th) * vv;
      const int64_t tiles = (a.dvec + span - 1) / span;
      const double eff = static_cast<double>(a.dvec) / static_cast<double>(tiles * span) + vv * 1e-3 + th * 1e-6;
      if (eff > best_eff) best_eff = eff, threads = th, v = vv, best_tiles = tiles;
    }
  a.tiles = static_cast<int>(best_tiles);
  const int64_t items = T * a.tiles;
  int64_t blocks = items < 0x7fffffffll ? items : 0x7fffffffll;
  const bool one_group = local_lo > 0 || local_hi < experts_per_rank;
  if (one_group && g_peer_ctas_per_sm > 0 && blocks > static_cast<int64_t>(kNumSMs) * g_peer_ctas_per_sm)
    blocks = static_cast<int64_t>(kNumSMs) * g_peer_ctas_per_sm;  // the kernel strides over the items
  const int grid = static_cast<int>(blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  // The kernel uses no shared memory, but it asks for the SM to be set up with the largest
  // shared-memory share all the same: an SM cannot change that split while a CTA runs on it,
  // so a grouped GEMM CTA (which needs nearly all of it) launched while this kernel is still
  // running would otherwise wait for it to drain (measured: 200 us per step on 2 GPUs).
  FMOE_DISPATCH_DTYPE(dtype, DT, {
    if (v == 1) {
      cudaFuncSetAttribute(permute_peer_kernel<DT, 1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared);
      permute_peer_kernel<DT, 1><<<grid, threads, 0, s>>>(a);
    } else {
      cudaFuncSetAttribute(permute_peer_kernel<DT, 2>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared);
      permute_peer_kernel<DT, 2><<<grid, threads, 0, s>>>(a);
    }
    rc = check_launch("permute_peer_kernel");
  });
  return rc;
}
