// Scatter form of the grouped pointer-table combine:
//   out[idx[g], :] += src_e[r, :] * w[g]
// One launch over the flattened (expert,row) space, so skewed expert loads
// balance themselves and empty experts cost nothing. Replaces the Triton kernel
// of polkadot21/fastmoe (src/fastmoe/kernels/ops.py:57-194, launch :277-310),
// whose (max_rows, E) grid spends most of its programs on early exits when the
// load is skewed.
#include "common.cuh"

namespace fmoe {

constexpr int kScatterThreads = 256;
constexpr int kScatterRows = 4;  // consecutive global rows per work item

struct ScatterArgs {
  const int64_t* ptr_table;
  const int32_t* chunk_sizes;
  const int64_t* expert_offsets;
  const void* idx;
  const void* w;
  void* out;
  int64_t out_row_stride;  // elements
  int64_t N, T, D;
  int E;
  int idx_type, w_dtype;
  int tiles;  // column tiles per row
  int32_t* status;
};

// Resolves global row g to its source row pointer (nullptr = skip), walking the
// expert cursor `e` forward. Uniform across the CTA.
__device__ __forceinline__ const char* resolve_row(const ScatterArgs& a, int& e, int64_t g,
                                                   int elem_bytes, int& flags) {
  while (e + 1 < a.E && a.expert_offsets[e + 1] <= g) ++e;
  const int64_t local = g - a.expert_offsets[e];
  if (local < 0 || local >= a.chunk_sizes[e]) {
    flags |= FMOE_STATUS_BAD_EXPERT;
    return nullptr;
  }
  const int64_t base = a.ptr_table[e];
  if (base == 0) {
    flags |= FMOE_STATUS_NULL_PTR;
    return nullptr;
  }
  return reinterpret_cast<const char*>(base) + local * a.D * elem_bytes;
}

template <int DT, int V>
__global__ void __launch_bounds__(kScatterThreads)
    combine_scatter_kernel(const ScatterArgs a) {
  using El = Elem<DT>;
  constexpr int R = kScatterRows;
  const int64_t dvec = a.D / El::kVec;
  const int64_t row_blocks = (a.N + R - 1) / R;
  const int64_t items = row_blocks * a.tiles;
  int flags = 0;

  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t rb = item / a.tiles;
    const int tile = static_cast<int>(item - rb * a.tiles);
    const int64_t g0 = rb * R;
    const int nr = static_cast<int>(min(static_cast<int64_t>(R), a.N - g0));

    const char* src[R];
    float wr[R];
    int64_t tgt[R];
    int e = find_expert(a.expert_offsets, a.E, g0);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      src[r] = nullptr;
      wr[r] = 0.f;
      tgt[r] = -1;
      if (r < nr) {
        const int64_t g = g0 + r;
        const int64_t t = load_index(a.idx, g, a.idx_type);
        if (t < 0 || t >= a.T) {
          flags |= FMOE_STATUS_BAD_INDEX;
        } else {
          src[r] = resolve_row(a, e, g, El::kBytes, flags);
          tgt[r] = t;
          wr[r] = load_scalar_as_float(a.w, g, a.w_dtype);
        }
      }
    }

    // Issue every load of the item before the first use.
    uint4 x[R][V];
    int64_t col[V];
#pragma unroll
    for (int v = 0; v < V; ++v)
      col[v] = (static_cast<int64_t>(tile) * V + v) * kScatterThreads + threadIdx.x;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool aligned = (reinterpret_cast<uintptr_t>(src[r]) & 15) == 0;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        x[r][v] = make_uint4(0, 0, 0, 0);
        if (src[r] != nullptr && col[v] < dvec) {
          if (aligned) {
            x[r][v] = ld_stream16(reinterpret_cast<const uint4*>(src[r]) + col[v]);
          } else {  // odd base address: element loads, same arithmetic
            const typename El::type* s =
                reinterpret_cast<const typename El::type*>(src[r]) + col[v] * El::kVec;
            typename El::type* d = reinterpret_cast<typename El::type*>(&x[r][v]);
#pragma unroll
            for (int i = 0; i < El::kVec; ++i) d[i] = s[i];
          }
        }
      }
    }

    // Segmented reduction along the rows of the item: rows that share a target
    // are summed in fp32 registers and leave as one reduction.
    float acc[V][El::kVec];
    int64_t cur = -1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (src[r] == nullptr) continue;
      if (tgt[r] != cur) {
        if (cur >= 0) {
#pragma unroll
          for (int v = 0; v < V; ++v)
            if (col[v] < dvec)
              red_add16<DT>(reinterpret_cast<typename El::type*>(a.out) +
                                cur * a.out_row_stride + col[v] * El::kVec,
                            acc[v]);
        }
        cur = tgt[r];
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
          for (int i = 0; i < El::kVec; ++i) acc[v][i] = 0.f;
      }
#pragma unroll
      for (int v = 0; v < V; ++v) {
        float f[El::kVec];
        unpack16<DT>(x[r][v], f);
#pragma unroll
        for (int i = 0; i < El::kVec; ++i) acc[v][i] = __fadd_rn(acc[v][i], __fmul_rn(f[i], wr[r]));
      }
    }
    if (cur >= 0) {
#pragma unroll
      for (int v = 0; v < V; ++v)
        if (col[v] < dvec)
          red_add16<DT>(reinterpret_cast<typename El::type*>(a.out) + cur * a.out_row_stride +
                            col[v] * El::kVec,
                        acc[v]);
    }
  }
  if (flags != 0 && a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, flags);
}

// Element-wise fallback for widths or output layouts that rule out 16-byte
// accesses (D not a multiple of the vector width, odd out stride or base).
template <int DT>
__global__ void __launch_bounds__(256) combine_scatter_scalar_kernel(const ScatterArgs a) {
  using El = Elem<DT>;
  using T = typename El::type;
  const int64_t total = a.N * a.D;
  int flags = 0;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t g = i / a.D;
    const int64_t c = i - g * a.D;
    const int64_t t = load_index(a.idx, g, a.idx_type);
    if (t < 0 || t >= a.T) {
      flags |= FMOE_STATUS_BAD_INDEX;
      continue;
    }
    int e = find_expert(a.expert_offsets, a.E, g);
    const char* row = resolve_row(a, e, g, El::kBytes, flags);
    if (row == nullptr) continue;
    const float v = to_float<DT>(reinterpret_cast<const T*>(row)[c]);
    const float wv = load_scalar_as_float(a.w, g, a.w_dtype);
    red_add1<DT>(reinterpret_cast<T*>(a.out) + t * a.out_row_stride + c, __fmul_rn(v, wv));
  }
  if (flags != 0 && a.status != nullptr) atomicOr(a.status, flags);
}

template <int DT>
static int launch_scatter(const ScatterArgs& a0, cudaStream_t stream) {
  using El = Elem<DT>;
  ScatterArgs a = a0;
  const bool vec_ok = (a.D % El::kVec == 0) && aligned_to(a.out, 16) &&
                      ((a.out_row_stride * El::kBytes) % 16 == 0);
  if (!vec_ok) {
    const int64_t total = a.N * a.D;
    const int64_t blocks = (total + 255) / 256;
    const int grid = static_cast<int>(blocks < kNumSMs * 16 ? blocks : kNumSMs * 16);
    combine_scatter_scalar_kernel<DT><<<grid, 256, 0, stream>>>(a);
    return check_launch("combine_scatter_scalar_kernel");
  }
  const int64_t dvec = a.D / El::kVec;
  const int v = dvec > kScatterThreads ? 2 : 1;
  a.tiles = static_cast<int>((dvec + static_cast<int64_t>(kScatterThreads) * v - 1) /
                             (static_cast<int64_t>(kScatterThreads) * v));
  const int64_t items = (a.N + kScatterRows - 1) / kScatterRows * a.tiles;
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
  const int grid = static_cast<int>(items < cap ? items : cap);
  if (v == 2)
    combine_scatter_kernel<DT, 2><<<grid, kScatterThreads, 0, stream>>>(a);
  else
    combine_scatter_kernel<DT, 1><<<grid, kScatterThreads, 0, stream>>>(a);
  return check_launch("combine_scatter_kernel");
}

}  // namespace fmoe

extern "C" int fmoe_combine_scatter(const int64_t* ptr_table, const int32_t* chunk_sizes,
                                    const int64_t* expert_offsets, const void* idx, int idx_type,
                                    const void* w, int w_dtype, void* out, int64_t out_row_stride,
                                    int64_t E, int64_t N, int64_t T, int64_t D, int dtype,
                                    int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_combine_scatter");
  using namespace fmoe;
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype), FMOE_ERR_ARG,
               "fmoe_combine_scatter: bad dtype %d / w_dtype %d", dtype, w_dtype);
  FMOE_REQUIRE(valid_itype(idx_type), FMOE_ERR_ARG, "fmoe_combine_scatter: bad idx_type %d",
               idx_type);
  FMOE_REQUIRE(E >= 0 && N >= 0 && T >= 0 && D >= 0, FMOE_ERR_ARG,
               "fmoe_combine_scatter: negative size (E=%lld N=%lld T=%lld D=%lld)", (long long)E,
               (long long)N, (long long)T, (long long)D);
  FMOE_REQUIRE(E < (1ll << 31) && N < (1ll << 31) && T < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_scatter: E, N and T must fit in int32");
  if (N == 0 || D == 0 || E == 0) return FMOE_OK;  // nothing to add (ops.py:286)
  FMOE_REQUIRE(T > 0, FMOE_ERR_ARG, "fmoe_combine_scatter: N > 0 rows but T == 0 output rows");
  FMOE_REQUIRE(ptr_table && chunk_sizes && expert_offsets && idx && w && out, FMOE_ERR_ARG,
               "fmoe_combine_scatter: null pointer argument");
  FMOE_REQUIRE(out_row_stride >= D, FMOE_ERR_ARG,
               "fmoe_combine_scatter: out_row_stride %lld < D %lld", (long long)out_row_stride,
               (long long)D);
  ScatterArgs a;
  a.ptr_table = ptr_table;
  a.chunk_sizes = chunk_sizes;
  a.expert_offsets = expert_offsets;
  a.idx = idx;
  a.w = w;
  a.out = out;
  a.out_row_stride = out_row_stride;
  a.N = N;
  a.T = T;
  a.D = D;
  a.E = static_cast<int>(E);
  a.idx_type = idx_type;
  a.w_dtype = w_dtype;
  a.tiles = 1;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT, rc = launch_scatter<DT>(a, s));
  return rc;
}
