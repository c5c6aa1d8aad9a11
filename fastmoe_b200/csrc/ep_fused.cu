// Dispatch permute fused with the expert-parallel exchange: every routed copy of a token
// row is stored directly into the receive buffer of the GPU that owns its expert, at the
// row where that GPU's grouped GEMM expects it. Plain 16-byte peer stores over NVLink
// (no multicast, no TMA): the copy IS the all-to-all. Replaces, for several GPUs,
// x_flat[reverse_map] + dist.all_to_all_single + the receive-side split of
// polkadot21/fastmoe (src/fastmoe/models/tiny_model.py:133, :210-216, :282-294).
#include "common.cuh"

namespace fmoe {

struct PeerPermuteArgs {
  const void* x;
  int64_t x_row_stride;
  const int64_t* topk_idx;
  const int32_t* slot_of;
  const int64_t* local_offsets;
  const int64_t* dst_row0;
  const int64_t* peer_bases;
  int64_t T, D, dvec, cap_rows;
  int K, E, experts_per_rank, tiles;
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
    uint4 val[V];
    int64_t col[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      col[v] = (static_cast<int64_t>(tile) * V + v) * blockDim.x + threadIdx.x;
      if (col[v] < a.dvec) val[v] = ld_stream16(xrow + col[v]);
    }
    for (int k0 = 0; k0 < a.K; k0 += 8) {
      uint4* drow[8];  // resolve the destinations together: one round of lookups, not eight
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        drow[u] = nullptr;
        if (k0 + u < a.K) {
          const int64_t e = a.topk_idx[t * a.K + k0 + u];
          const int32_t slot = a.slot_of[t * a.K + k0 + u];
          if (e >= 0 && e < a.E && slot >= 0) {
            const int64_t row = a.dst_row0[e] + (slot - a.local_offsets[e]);
            if (row >= 0 && row < a.cap_rows) {
              char* base = reinterpret_cast<char*>(a.peer_bases[e / a.experts_per_rank]);
              drow[u] = reinterpret_cast<uint4*>(base + row * a.D * El::kBytes);
            } else {
              flags |= FMOE_STATUS_BAD_INDEX;  // the receive buffer is full: the row is dropped
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (drow[u] == nullptr) continue;
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (col[v] < a.dvec) drow[u][col[v]] = val[v];
      }
    }
  }
  if (flags != 0 && a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, flags);
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_permute_peer_fwd(const void* x, int64_t x_row_stride, const int64_t* topk_idx,
                                     const int32_t* slot_of, const int64_t* local_offsets,
                                     const int64_t* dst_row0, const int64_t* peer_bases, int64_t T,
                                     int64_t K, int64_t D, int64_t E, int64_t experts_per_rank,
                                     int64_t cap_rows, int dtype, int32_t* status, void* stream) {
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_permute_peer_fwd: bad dtype %d", dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0 && E > 0 && experts_per_rank > 0 && cap_rows >= 0, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: bad sizes");
  FMOE_REQUIRE(E % experts_per_rank == 0, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: E=%lld is not a multiple of experts_per_rank=%lld", (long long)E,
               (long long)experts_per_rank);
  FMOE_REQUIRE(T * K < (1ll << 31) && E < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_permute_peer_fwd: T*K and E must fit in int32");
  if (T == 0 || K == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(x && topk_idx && slot_of && local_offsets && dst_row0 && peer_bases, FMOE_ERR_ARG,
               "fmoe_permute_peer_fwd: null pointer argument");
  FMOE_REQUIRE(x_row_stride >= D, FMOE_ERR_ARG, "fmoe_permute_peer_fwd: x_row_stride < D");
  const int eb = dtype_size(dtype);
  const int kvec = 16 / eb;
  FMOE_REQUIRE(D % kvec == 0 && aligned_to(x, 16) && (x_row_stride * eb) % 16 == 0, FMOE_ERR_UNSUPPORTED,
               "fmoe_permute_peer_fwd: D must be a multiple of %d and x 16-byte aligned", kvec);
  PeerPermuteArgs a;
  a.x = x;
  a.x_row_stride = x_row_stride;
  a.topk_idx = topk_idx;
  a.slot_of = slot_of;
  a.local_offsets = local_offsets;
  a.dst_row0 = dst_row0;
  a.peer_bases = peer_bases;
  a.T = T;
  a.D = D;
  a.dvec = D / kvec;
  a.cap_rows = cap_rows;
  a.K = static_cast<int>(K);
  a.E = static_cast<int>(E);
  a.experts_per_rank = static_cast<int>(experts_per_rank);
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
  const int grid = static_cast<int>(items < 0x7fffffffll ? items : 0x7fffffffll);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT, {
    if (v == 1)
      permute_peer_kernel<DT, 1><<<grid, threads, 0, s>>>(a);
    else
      permute_peer_kernel<DT, 2><<<grid, threads, 0, s>>>(a);
    rc = check_launch("permute_peer_kernel");
  });
  return rc;
}
