// Token-major data movers of the MoE hot path. Each work item owns a tile of
// one token row and walks the routed rows that belong to it, so every byte of
// payload crosses HBM once and every output element is written once:
//   combine forward   out[t]       = sum_j src_j * w_j            (plan order)
//   combine backward  grad_rows[g] = grad_out[t] * w_g ; grad_w[g] = <grad_out[t], src_g>
//   dispatch permute  permuted[slot_of[t,k]] = x[t]
//   permute backward  grad_x[t]    = sum_k grad_permuted[slot_of[t,k]]
// They replace, in polkadot21/fastmoe: the Triton scatter-add kernel
// (src/fastmoe/kernels/ops.py:57-194), GroupedWeightedScatterAdd.backward
// (ops.py:334-359), the row gather x_flat[reverse_map]
// (src/fastmoe/models/tiny_model.py:133) and its autograd backward.
#include <string_view>

#include "plan.cuh"

namespace fmoe {

// ---- tuning knobs (fmoe_tune) -------------------------------------------------
static int g_gather_v = 0;         // vectors per thread, 0 = choose from D
static int g_gather_threads = 0;   // threads per CTA, 0 = choose from D
static int g_gather_ctas_per_sm = -1;  // persistent grid = 148 * this; 0 = one CTA per item; -1 = auto
static int g_bwd_ctas_per_sm = 3;
static int g_gather_pdl = 1;  // launch the gather kernels as programmatic dependents of their predecessor
int g_host_chunks = 1;  // column slices of fmoe_combine_host (host_api.cu); 0 = choose from the sizes
extern int g_gemm_sms, g_gemm_skip_loads, g_gemm_spin_limit, g_gemm_prefetch, g_gemm_tokens_as_n;  // grouped_gemm.cu
extern int g_peer_ctas_per_sm;  // ep_fused.cu
extern int g_plan_rows_per_thread;  // combine_plan.cu

struct TileCfg {
  int threads;
  int v;
  int tiles;
};

// Picks threads-per-CTA (a multiple of 32) and vectors-per-thread so that a row
// of `dvec` 16-byte vectors splits into whole tiles with the fewest idle lanes.
static TileCfg pick_tile(int64_t dvec, int pref_v, int force_threads, int max_v = 4) {
  TileCfg best{32, 1, static_cast<int>(dvec)};
  double best_score = -1.0;
  for (int threads = 32; threads <= 256; threads += 32) {
    if (force_threads > 0 && threads != force_threads) continue;
    for (int v = 1; v <= max_v; v *= 2) {
      const int64_t span = static_cast<int64_t>(threads) * v;
      const int64_t tiles = (dvec + span - 1) / span;
      const double eff = static_cast<double>(dvec) / static_cast<double>(tiles * span);
      // prefer full lanes, then the preferred vector count, then wide CTAs
      const double score = eff * 1000.0 + (v == pref_v ? 1.0 : 0.0) + threads / 1024.0;
      if (score > best_score) {
        best_score = score;
        best = TileCfg{threads, v, static_cast<int>(tiles)};
      }
    }
  }
  return best;
}

// Grid for `items` work items: one CTA per item, or a persistent grid of
// 148 x ctas_per_sm CTAs that stride over the items.
static int64_t clamp_grid(int64_t items, int ctas_per_sm) {
  int64_t grid = items;
  if (ctas_per_sm > 0 && items > static_cast<int64_t>(kNumSMs) * ctas_per_sm)
    grid = static_cast<int64_t>(kNumSMs) * ctas_per_sm;
  if (grid > 0x7fffffffll) grid = 0x7fffffffll;
  return grid;
}

// ---- row sources ----------------------------------------------------------------
// A source tells, for output row t, which slots feed it, and for a slot, where
// its row lives and what it is scaled by.
struct PlanSource {
  const int32_t* seg_off;
  const int64_t* src_sorted;
  const float* w_sorted;
  __device__ __forceinline__ void segment(int64_t t, int& beg, int& end) const {
    beg = seg_off[t];
    end = seg_off[t + 1];
  }
  __device__ __forceinline__ void row(int j, const char*& p, float& w) const {
    p = reinterpret_cast<const char*>(src_sorted[j]);
    w = w_sorted[j];
  }
};

struct PlanWindowSource {  // the plan's rows, read from a byte offset inside every row
  const int32_t* seg_off;
  const int64_t* src_sorted;
  const float* w_sorted;
  int64_t col_bytes;
  __device__ __forceinline__ void segment(int64_t t, int& beg, int& end) const {
    beg = seg_off[t];
    end = seg_off[t + 1];
  }
  __device__ __forceinline__ void row(int j, const char*& p, float& w) const {
    const int64_t a = src_sorted[j];
    p = a != 0 ? reinterpret_cast<const char*>(a + col_bytes) : nullptr;
    w = w_sorted[j];
  }
};

struct SlotSource {  // K rows of one matrix per token, unit weights
  const int32_t* slot_of;
  const char* base;
  int64_t row_bytes;
  int64_t rows;  // rows of the matrix (bounds check)
  int K;
  __device__ __forceinline__ void segment(int64_t t, int& beg, int& end) const {
    beg = static_cast<int>(t * K);
    end = beg + K;
  }
  __device__ __forceinline__ void row(int j, const char*& p, float& w) const {
    const int32_t s = slot_of[j];
    p = (s >= 0 && s < rows) ? base + s * row_bytes : nullptr;
    w = 1.f;
  }
};

struct WeightedSlotSource {  // K rows of one matrix per token, each scaled by the gate weight of its slot
  const int32_t* slot_of;
  const char* base;
  const void* w;  // [rows] gate weight per sorted slot
  int64_t row_bytes;
  int64_t rows;
  int K;
  int w_dtype;
  __device__ __forceinline__ void segment(int64_t t, int& beg, int& end) const {
    beg = static_cast<int>(t * K);
    end = beg + K;
  }
  __device__ __forceinline__ void row(int j, const char*& p, float& wt) const {
    const int32_t s = slot_of[j];
    const bool ok = s >= 0 && s < rows;
    p = ok ? base + s * row_bytes : nullptr;
    wt = ok ? load_scalar_as_float(w, s, w_dtype) : 0.f;
  }
};

template <int DT>
__device__ __forceinline__ uint4 load_row_vec(const char* p, int64_t col) {
  using El = Elem<DT>;
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0)
    return ld_stream16(reinterpret_cast<const uint4*>(p) + col);
  uint4 x;  // odd base address: element loads
  const typename El::type* s = reinterpret_cast<const typename El::type*>(p) + col * El::kVec;
  typename El::type* d = reinterpret_cast<typename El::type*>(&x);
#pragma unroll
  for (int i = 0; i < El::kVec; ++i) d[i] = s[i];
  return x;
}

// ---- gather-sum: combine forward and permute backward --------------------------------
template <int DT, int V, bool WEIGHTED, class Source>
__global__ void __launch_bounds__(256)
    gather_sum_kernel(const Source src, void* __restrict__ out, int64_t out_row_stride, int64_t T,
                      int64_t dvec, int tiles, int accumulate) {
  using El = Elem<DT>;
  using Ty = typename El::type;
  constexpr int U = 4;  // rows in flight
  const int64_t items = T * tiles;
  // Launched as a programmatic dependent of the kernel that writes what `src` reads (the plan
  // build), this kernel's CTAs may already be resident while that kernel finishes: wait for
  // it here. Without such a launch the instruction returns at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t t = item / tiles;
    const int tile = static_cast<int>(item - t * tiles);
    int64_t col[V];
#pragma unroll
    for (int v = 0; v < V; ++v) col[v] = (static_cast<int64_t>(tile) * V + v) * blockDim.x + threadIdx.x;

    int beg, end;
    src.segment(t, beg, end);

    float acc[V][El::kVec];
    uint4* orow = reinterpret_cast<uint4*>(reinterpret_cast<Ty*>(out) + t * out_row_stride);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      if (accumulate && col[v] < dvec) {
        unpack16<DT>(orow[col[v]], acc[v]);
      } else {
#pragma unroll
        for (int i = 0; i < El::kVec; ++i) acc[v][i] = 0.f;
      }
    }

    int j = beg;
    for (; j + U <= end; j += U) {
      const char* p[U];
      float w[U];
#pragma unroll
      for (int u = 0; u < U; ++u) src.row(j + u, p[u], w[u]);
      uint4 x[U][V];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < V; ++v)
          x[u][v] = (p[u] != nullptr && col[v] < dvec) ? load_row_vec<DT>(p[u], col[v])
                                                       : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int v = 0; v < V; ++v) {
          float f[El::kVec];
          unpack16<DT>(x[u][v], f);
#pragma unroll
          for (int i = 0; i < El::kVec; ++i)
            acc[v][i] = WEIGHTED ? __fadd_rn(acc[v][i], __fmul_rn(f[i], w[u]))
                                 : __fadd_rn(acc[v][i], f[i]);
        }
    }
    for (; j < end; ++j) {
      const char* p;
      float w;
      src.row(j, p, w);
      uint4 x[V];
#pragma unroll
      for (int v = 0; v < V; ++v)
        x[v] = (p != nullptr && col[v] < dvec) ? load_row_vec<DT>(p, col[v]) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        float f[El::kVec];
        unpack16<DT>(x[v], f);
#pragma unroll
        for (int i = 0; i < El::kVec; ++i)
          acc[v][i] = WEIGHTED ? __fadd_rn(acc[v][i], __fmul_rn(f[i], w)) : __fadd_rn(acc[v][i], f[i]);
      }
    }
#pragma unroll
    for (int v = 0; v < V; ++v)
      if (col[v] < dvec) st_stream16(orow + col[v], pack16<DT>(acc[v]));
  }
}

// Element-wise variant for widths or layouts that rule out 16-byte accesses.
template <int DT, bool WEIGHTED, class Source>
__global__ void __launch_bounds__(256)
    gather_sum_scalar_kernel(const Source src, void* __restrict__ out, int64_t out_row_stride,
                             int64_t T, int64_t D, int accumulate) {
  using Ty = typename Elem<DT>::type;
  const int64_t total = T * D;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / D, c = i - t * D;
    Ty* o = reinterpret_cast<Ty*>(out) + t * out_row_stride + c;
    float acc = accumulate ? to_float<DT>(*o) : 0.f;
    int beg, end;
    src.segment(t, beg, end);
    for (int j = beg; j < end; ++j) {
      const char* p;
      float w;
      src.row(j, p, w);
      if (p == nullptr) continue;
      const float f = to_float<DT>(reinterpret_cast<const Ty*>(p)[c]);
      acc = WEIGHTED ? __fadd_rn(acc, __fmul_rn(f, w)) : __fadd_rn(acc, f);
    }
    *o = from_float<DT>(acc);
  }
}

template <int DT, bool WEIGHTED, class Source>
static int launch_gather_sum(const Source& src, void* out, int64_t out_row_stride, int64_t T,
                             int64_t D, int accumulate, cudaStream_t s) {
  using El = Elem<DT>;
  if (T == 0 || D == 0) return FMOE_OK;
  const bool vec_ok =
      (D % El::kVec == 0) && aligned_to(out, 16) && ((out_row_stride * El::kBytes) % 16 == 0);
  if (!vec_ok) {
    const int64_t blocks = (T * D + 255) / 256;
    const int grid = static_cast<int>(blocks < kNumSMs * 16 ? blocks : kNumSMs * 16);
    gather_sum_scalar_kernel<DT, WEIGHTED, Source><<<grid, 256, 0, s>>>(src, out, out_row_stride, T, D, accumulate);
    return check_launch("gather_sum_scalar_kernel");
  }
  const int64_t dvec = D / El::kVec;
  const TileCfg cfg = pick_tile(dvec, g_gather_v > 0 ? g_gather_v : 2, g_gather_threads);
  auto launch = [&](auto kernel) {
    int ctas = g_gather_ctas_per_sm;
    if (ctas < 0) {  // auto: exactly as many CTAs as stay resident (asked once per kernel and CTA size)
      static int resident[9] = {};  // indexed by threads / 32; one array per kernel instantiation
      int& slot = resident[cfg.threads / 32];
      if (slot == 0 &&
          (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&slot, kernel, cfg.threads, 0) != cudaSuccess || slot < 1))
        slot = 1;
      ctas = slot;
    }
    const int g = static_cast<int>(clamp_grid(T * cfg.tiles, ctas));
    // programmatic dependent launch: the CTAs may be placed while the previous kernel of the
    // stream drains (they wait inside, see the kernel); saves the launch gap after the plan build
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(g);
    lc.blockDim = dim3(cfg.threads);
    lc.dynamicSmemBytes = 0;
    lc.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_gather_pdl ? 1 : 0;
    lc.attrs = attr;
    lc.numAttrs = 1;
    int acc = accumulate;
    cudaLaunchKernelEx(&lc, kernel, src, out, out_row_stride, T, dvec, cfg.tiles, acc);
  };
  switch (cfg.v) {
    case 1: launch(gather_sum_kernel<DT, 1, WEIGHTED, Source>); break;
    case 2: launch(gather_sum_kernel<DT, 2, WEIGHTED, Source>); break;
    default: launch(gather_sum_kernel<DT, 4, WEIGHTED, Source>); break;
  }
  return check_launch("gather_sum_kernel");
}

// ---- combine backward ---------------------------------------------------------------
// One warp per routed row: it streams grad_out[t] (shared through L1/L2 with the
// other warps working on the same token) and, for the gate gradient, the forward
// source row; writes the scaled copy; and reduces the row dot with shuffles in a
// fixed order. Warps never wait for each other. A CTA takes `group` consecutive
// tokens per step so that its 8 warps stay busy when tokens have fewer than 8 rows.
constexpr int kBwdWarps = 8;

// What the backward walks: per token a run of entries, per entry the routed row it stands
// for (g: its row in grad_rows and grad_w), the forward source row and the gate weight.
struct PlanBwdSource {  // the combine plan: entries are the plan's slots
  const int32_t* seg_off;
  const int32_t* row_of_slot;
  const int64_t* src_sorted;
  const float* w_sorted;
  __device__ __forceinline__ int first(int64_t t) const { return seg_off[t]; }
  __device__ __forceinline__ bool entry(int j, int64_t& g, const char*& p, float& w) const {
    g = row_of_slot[j];
    w = w_sorted[j];
    p = reinterpret_cast<const char*>(src_sorted[j]);
    return true;
  }
};
struct SlotBwdSource {  // the routing index: entry t*K+k is routed copy k of token t, at sorted slot slot_of[t*K+k]
  const int32_t* slot_of;
  const char* base;  // the forward's rows, one per sorted slot
  const void* w;
  int64_t row_bytes, rows;
  int K, w_dtype;
  __device__ __forceinline__ int first(int64_t t) const { return static_cast<int>(t * K); }
  __device__ __forceinline__ bool entry(int j, int64_t& g, const char*& p, float& wt) const {
    const int32_t s = slot_of[j];
    if (s < 0 || s >= rows) return false;
    g = s;
    p = base + s * row_bytes;
    wt = load_scalar_as_float(w, s, w_dtype);
    return true;
  }
};

template <int DT, bool WITH_GW, class Source>
__global__ void __launch_bounds__(kBwdWarps * 32)
    combine_bwd_kernel(const Source src, const void* __restrict__ grad_out, int64_t go_row_stride,
                       void* __restrict__ grad_rows, float* __restrict__ grad_w, int64_t T,
                       int64_t D, int64_t dvec, int group) {
  using El = Elem<DT>;
  using Ty = typename El::type;
  constexpr int U = 4;  // vectors in flight per lane and stream
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t items = (T + group - 1) / group;

  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t t0 = item * group;
    const int64_t t1 = min(T, t0 + group);
    const int beg = src.first(t0), end = src.first(t1);
    int64_t t = t0;
    for (int j = beg + warp; j < end; j += kBwdWarps) {
      while (t + 1 < t1 && src.first(t + 1) <= j) ++t;  // token that owns entry j
      int64_t g;
      float w;
      const char* p;
      if (!src.entry(j, g, p, w)) continue;
      const uint4* gorow =
          reinterpret_cast<const uint4*>(reinterpret_cast<const Ty*>(grad_out) + t * go_row_stride);
      uint4* drow = reinterpret_cast<uint4*>(reinterpret_cast<Ty*>(grad_rows) + g * D);
      float dot = 0.f;
      for (int64_t c0 = lane; c0 < dvec; c0 += 32 * U) {
        uint4 gv[U], xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t c = c0 + 32 * u;
          if (c < dvec) {
            gv[u] = ld_cached16(gorow + c);
            if (WITH_GW) xv[u] = p != nullptr ? load_row_vec<DT>(p, c) : make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t c = c0 + 32 * u;
          if (c < dvec) {
            float go[El::kVec], f[El::kVec];
            unpack16<DT>(gv[u], go);
#pragma unroll
            for (int i = 0; i < El::kVec; ++i) f[i] = __fmul_rn(go[i], w);
            st_stream16(drow + c, pack16<DT>(f));
            if (WITH_GW) {
              float xf[El::kVec];
              unpack16<DT>(xv[u], xf);
#pragma unroll
              for (int i = 0; i < El::kVec; ++i) dot = fmaf(go[i], xf[i], dot);
            }
          }
        }
      }
      if (WITH_GW) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (lane == 0) grad_w[g] = dot;
      }
    }
  }
}

// ---- dispatch permute forward ----------------------------------------------------
template <int DT, int V>
__global__ void __launch_bounds__(256)
    permute_fwd_kernel(const void* __restrict__ x, int64_t x_row_stride,
                       const int32_t* __restrict__ slot_of, void* __restrict__ permuted, int64_t T,
                       int K, int64_t D, int64_t dvec, int tiles) {
  using El = Elem<DT>;
  using Ty = typename El::type;
  const int64_t items = T * tiles;
  const int64_t rows = T * K;
  for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
    const int64_t t = item / tiles;
    const int tile = static_cast<int>(item - t * tiles);
    const uint4* xrow = reinterpret_cast<const uint4*>(reinterpret_cast<const Ty*>(x) + t * x_row_stride);
    uint4 val[V];
    int64_t col[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
      col[v] = (static_cast<int64_t>(tile) * V + v) * blockDim.x + threadIdx.x;
      if (col[v] < dvec) val[v] = ld_stream16(xrow + col[v]);
    }
    for (int k0 = 0; k0 < K; k0 += 8) {
      int32_t slot[8];  // fetch the destinations together: one latency, not eight
#pragma unroll
      for (int u = 0; u < 8; ++u) slot[u] = k0 + u < K ? slot_of[t * K + k0 + u] : -1;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (slot[u] < 0 || slot[u] >= rows) continue;
        uint4* drow =
            reinterpret_cast<uint4*>(reinterpret_cast<Ty*>(permuted) + static_cast<int64_t>(slot[u]) * D);
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (col[v] < dvec) st_stream16(drow + col[v], val[v]);
      }
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(256)
    permute_fwd_scalar_kernel(const void* __restrict__ x, int64_t x_row_stride,
                              const int32_t* __restrict__ slot_of, void* __restrict__ permuted,
                              int64_t T, int K, int64_t D) {
  using Ty = typename Elem<DT>::type;
  const int64_t rows = T * K;
  const int64_t total = rows * D;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t tk = i / D, c = i - tk * D;
    const int32_t s = slot_of[tk];
    if (s < 0 || s >= rows) continue;
    reinterpret_cast<Ty*>(permuted)[static_cast<int64_t>(s) * D + c] =
        reinterpret_cast<const Ty*>(x)[(tk / K) * x_row_stride + c];
  }
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_tune(const char* key, int value) {
  if (key == nullptr) return FMOE_ERR_ARG;
  const std::string_view k(key);
  if (k == "gather_v") {
    FMOE_REQUIRE(value == 0 || value == 1 || value == 2 || value == 4, FMOE_ERR_ARG,
                 "fmoe_tune: gather_v must be 0, 1, 2 or 4");
    g_gather_v = value;
  } else if (k == "gather_threads") {
    FMOE_REQUIRE(value >= 0 && value <= 256 && value % 32 == 0, FMOE_ERR_ARG,
                 "fmoe_tune: gather_threads must be a multiple of 32 in [0, 256]");
    g_gather_threads = value;
  } else if (k == "gather_ctas_per_sm") {
    FMOE_REQUIRE(value >= -1 && value <= 64, FMOE_ERR_ARG, "fmoe_tune: gather_ctas_per_sm in [-1, 64]");
    g_gather_ctas_per_sm = value;
  } else if (k == "bwd_ctas_per_sm") {
    FMOE_REQUIRE(value >= 1 && value <= 64, FMOE_ERR_ARG, "fmoe_tune: bwd_ctas_per_sm in [1, 64]");
    g_bwd_ctas_per_sm = value;
  } else if (k == "host_chunks") {
    FMOE_REQUIRE(value >= 0 && value <= 64, FMOE_ERR_ARG, "fmoe_tune: host_chunks in [0, 64]");
    g_host_chunks = value;
  } else if (k == "gemm_sms") {
    FMOE_REQUIRE(value >= 1 && value <= kNumSMs, FMOE_ERR_ARG, "fmoe_tune: gemm_sms in [1, %d]", kNumSMs);
    g_gemm_sms = value;
  } else if (k == "gemm_prefetch") {
    FMOE_REQUIRE(value >= 0 && value <= 64, FMOE_ERR_ARG, "fmoe_tune: gemm_prefetch in [0, 64]");
    g_gemm_prefetch = value;
  } else if (k == "gemm_tokens_as_n") {
    FMOE_REQUIRE(value >= -1 && value <= 1, FMOE_ERR_ARG, "fmoe_tune: gemm_tokens_as_n is -1 (auto), 0 or 1");
    g_gemm_tokens_as_n = value;
  } else if (k == "gather_pdl") {
    g_gather_pdl = value != 0;
  } else if (k == "plan_rows_per_thread") {
    FMOE_REQUIRE(value >= 1 && value <= 64, FMOE_ERR_ARG, "fmoe_tune: plan_rows_per_thread in [1, 64]");
    g_plan_rows_per_thread = value;
  } else if (k == "peer_ctas_per_sm") {
    FMOE_REQUIRE(value >= 0 && value <= 16, FMOE_ERR_ARG, "fmoe_tune: peer_ctas_per_sm in [0, 16]");
    g_peer_ctas_per_sm = value;
  } else if (k == "gemm_skip_loads") {
    g_gemm_skip_loads = value != 0;
  } else if (k == "gemm_spin_limit") {
    FMOE_REQUIRE(value >= 1, FMOE_ERR_ARG, "fmoe_tune: gemm_spin_limit must be positive");
    g_gemm_spin_limit = value;
  } else {
    return fail(FMOE_ERR_ARG, "fmoe_tune: unknown key '%s'", key);
  }
  return FMOE_OK;
}

extern "C" int fmoe_combine_gather(const void* plan, void* out, int64_t out_row_stride, int64_t N,
                                   int64_t T, int64_t D, int dtype, int accumulate, void* stream) {
  FMOE_RANGE("fmoe_combine_gather");
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_combine_gather: bad dtype %d", dtype);
  FMOE_REQUIRE(N >= 0 && T >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_combine_gather: negative size");
  FMOE_REQUIRE(N < (1ll << 31) && T < (1ll << 31) - 1, FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_gather: N and T must fit in int32");
  if (T == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(plan != nullptr && aligned_to(plan, 256), FMOE_ERR_WORKSPACE,
               "fmoe_combine_gather: plan is null or not 256-byte aligned");
  FMOE_REQUIRE(out != nullptr, FMOE_ERR_ARG, "fmoe_combine_gather: out is null");
  FMOE_REQUIRE(out_row_stride >= D, FMOE_ERR_ARG, "fmoe_combine_gather: out_row_stride %lld < D %lld",
               (long long)out_row_stride, (long long)D);
  const PlanView pv = plan_view(const_cast<void*>(plan), N, T);
  const PlanSource src{pv.seg_off, pv.src_sorted, pv.w_sorted};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT,
                      rc = (launch_gather_sum<DT, true, PlanSource>(src, out, out_row_stride, T, D,
                                                                    accumulate != 0, s)));
  return rc;
}

namespace fmoe {
// Columns [col0, col0 + cols) of the combine: sources are read `col0` elements into every planned
// row, `out` points at column col0 of the output's first row. Used by the host-buffer entry
// point to finish one slice of columns while the next one is still arriving.
int combine_gather_window(const void* plan, void* out, int64_t out_row_stride, int64_t N, int64_t T,
                          int64_t col0, int64_t cols, int dtype, cudaStream_t s) {
  const PlanView pv = plan_view(const_cast<void*>(plan), N, T);
  const PlanWindowSource src{pv.seg_off, pv.src_sorted, pv.w_sorted,
                             col0 * static_cast<int64_t>(dtype_size(dtype))};
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT,
                      rc = (launch_gather_sum<DT, true, PlanWindowSource>(src, out, out_row_stride, T,
                                                                          cols, 0, s)));
  return rc;
}
}  // namespace fmoe

extern "C" int fmoe_combine_bwd(const void* plan, const void* grad_out, int64_t grad_out_row_stride,
                                void* grad_rows, float* grad_w, int64_t N, int64_t T, int64_t D,
                                int dtype, void* stream) {
  FMOE_RANGE("fmoe_combine_bwd");
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_combine_bwd: bad dtype %d", dtype);
  FMOE_REQUIRE(N >= 0 && T >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_combine_bwd: negative size");
  FMOE_REQUIRE(N < (1ll << 31) && T < (1ll << 31) - 1, FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_bwd: N and T must fit in int32");
  if (N == 0 || T == 0) return FMOE_OK;
  FMOE_REQUIRE(plan != nullptr && aligned_to(plan, 256), FMOE_ERR_WORKSPACE,
               "fmoe_combine_bwd: plan is null or not 256-byte aligned");
  FMOE_REQUIRE(grad_out != nullptr && grad_rows != nullptr, FMOE_ERR_ARG,
               "fmoe_combine_bwd: null pointer argument");
  FMOE_REQUIRE(grad_out_row_stride >= D, FMOE_ERR_ARG, "fmoe_combine_bwd: grad_out_row_stride < D");
  const int eb = dtype_size(dtype);
  const int kvec = 16 / eb;
  FMOE_REQUIRE(D % kvec == 0 && aligned_to(grad_out, 16) && aligned_to(grad_rows, 16) &&
                   (grad_out_row_stride * eb) % 16 == 0,
               FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_bwd: D must be a multiple of %d and buffers 16-byte aligned", kvec);
  const PlanView pv = plan_view(const_cast<void*>(plan), N, T);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 0) {
    if (grad_w != nullptr) FMOE_CUDA(cudaMemsetAsync(grad_w, 0, sizeof(float) * N, s));
    return FMOE_OK;
  }
  // rows that were skipped when the plan was built (bad index) get no slot:
  // their gate gradient must still be defined
  if (grad_w != nullptr) FMOE_CUDA(cudaMemsetAsync(grad_w, 0, sizeof(float) * N, s));
  const int64_t dvec = D / kvec;
  // tokens per CTA step: enough that the CTA's 8 warps each find a routed row
  const int64_t avg_rows = T > 0 ? (N + T - 1) / T : 1;
  int group = static_cast<int>(avg_rows >= kBwdWarps ? 1 : (kBwdWarps + avg_rows - 1) / (avg_rows > 0 ? avg_rows : 1));
  if (group > kBwdWarps) group = kBwdWarps;
  const int grid = static_cast<int>(clamp_grid((T + group - 1) / group, g_bwd_ctas_per_sm));
  int rc = 0;
  const PlanBwdSource src{pv.seg_off, pv.row_of_slot, pv.src_sorted, pv.w_sorted};
#define FMOE_BWD_LAUNCH(DT, GW)                                                    \
  combine_bwd_kernel<DT, GW, PlanBwdSource><<<grid, kBwdWarps * 32, 0, s>>>(       \
      src, grad_out, grad_out_row_stride, grad_rows, grad_w, T, D, dvec, group)
  FMOE_DISPATCH_DTYPE(dtype, DT, {
    if (grad_w) FMOE_BWD_LAUNCH(DT, true); else FMOE_BWD_LAUNCH(DT, false);
    rc = check_launch("combine_bwd_kernel");
  });
#undef FMOE_BWD_LAUNCH
  return rc;
}

extern "C" int fmoe_permute_fwd(const void* x, int64_t x_row_stride, const int32_t* slot_of,
                                void* permuted, int64_t T, int64_t K, int64_t D, int dtype,
                                void* stream) {
  FMOE_RANGE("fmoe_permute_fwd");
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_permute_fwd: bad dtype %d", dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_permute_fwd: negative size");
  FMOE_REQUIRE(T * K < (1ll << 31), FMOE_ERR_UNSUPPORTED, "fmoe_permute_fwd: T*K must fit in int32");
  if (T == 0 || K == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(x && slot_of && permuted, FMOE_ERR_ARG, "fmoe_permute_fwd: null pointer argument");
  FMOE_REQUIRE(x_row_stride >= D, FMOE_ERR_ARG, "fmoe_permute_fwd: x_row_stride < D");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int eb = dtype_size(dtype);
  const int kvec = 16 / eb;
  const bool vec_ok = D % kvec == 0 && aligned_to(x, 16) && aligned_to(permuted, 16) &&
                      (x_row_stride * eb) % 16 == 0;
  int rc = 0;
  if (!vec_ok) {
    const int64_t blocks = (T * K * D + 255) / 256;
    const int grid = static_cast<int>(blocks < kNumSMs * 16 ? blocks : kNumSMs * 16);
    FMOE_DISPATCH_DTYPE(dtype, DT, {
      permute_fwd_scalar_kernel<DT><<<grid, 256, 0, s>>>(x, x_row_stride, slot_of, permuted, T,
                                                         static_cast<int>(K), D);
      rc = check_launch("permute_fwd_scalar_kernel");
    });
    return rc;
  }
  const int64_t dvec = D / kvec;
  const TileCfg cfg = pick_tile(dvec, g_gather_v > 0 ? g_gather_v : 2, g_gather_threads);
  // one short-lived CTA per item measured 15% faster than a persistent grid for this write-heavy copy
  const int grid = static_cast<int>(clamp_grid(T * cfg.tiles, g_gather_ctas_per_sm < 0 ? 0 : g_gather_ctas_per_sm));
#define FMOE_PERM_LAUNCH(DT, V)                                                            \
  permute_fwd_kernel<DT, V><<<grid, cfg.threads, 0, s>>>(x, x_row_stride, slot_of, permuted, T, \
                                                         static_cast<int>(K), D, dvec, cfg.tiles)
  FMOE_DISPATCH_DTYPE(dtype, DT, {
    if (cfg.v == 1) FMOE_PERM_LAUNCH(DT, 1);
    else if (cfg.v == 2) FMOE_PERM_LAUNCH(DT, 2);
    else FMOE_PERM_LAUNCH(DT, 4);
    rc = check_launch("permute_fwd_kernel");
  });
#undef FMOE_PERM_LAUNCH
  return rc;
}

extern "C" int fmoe_permute_bwd(const void* grad_permuted, const int32_t* slot_of, void* grad_x,
                                int64_t grad_x_row_stride, int64_t T, int64_t K, int64_t D,
                                int dtype, void* stream) {
  FMOE_RANGE("fmoe_permute_bwd");
  FMOE_REQUIRE(valid_dtype(dtype), FMOE_ERR_ARG, "fmoe_permute_bwd: bad dtype %d", dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_permute_bwd: negative size");
  FMOE_REQUIRE(T * K < (1ll << 31), FMOE_ERR_UNSUPPORTED, "fmoe_permute_bwd: T*K must fit in int32");
  if (T == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(grad_x != nullptr, FMOE_ERR_ARG, "fmoe_permute_bwd: grad_x is null");
  FMOE_REQUIRE(K == 0 || (grad_permuted && slot_of), FMOE_ERR_ARG,
               "fmoe_permute_bwd: null pointer argument");
  FMOE_REQUIRE(grad_x_row_stride >= D, FMOE_ERR_ARG, "fmoe_permute_bwd: grad_x_row_stride < D");
  const SlotSource src{slot_of, static_cast<const char*>(grad_permuted),
                       D * static_cast<int64_t>(dtype_size(dtype)), T * K, static_cast<int>(K)};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT,
                      rc = (launch_gather_sum<DT, false, SlotSource>(src, grad_x, grad_x_row_stride,
                                                                     T, D, 0, s)));
  return rc;
}

// ---- combine straight from the routing index (no plan) -----------------------------------------
extern "C" int fmoe_combine_routed(const void* rows, const int32_t* slot_of, const void* w_sorted, int w_dtype,
                                   void* out, int64_t out_row_stride, int64_t T, int64_t K, int64_t D, int dtype,
                                   int accumulate, void* stream) {
  FMOE_RANGE("fmoe_combine_routed");
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype), FMOE_ERR_ARG, "fmoe_combine_routed: bad dtype %d / %d",
               dtype, w_dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_combine_routed: negative size");
  FMOE_REQUIRE(T * K < (1ll << 31), FMOE_ERR_UNSUPPORTED, "fmoe_combine_routed: T*K must fit in int32");
  if (T == 0 || D == 0) return FMOE_OK;
  FMOE_REQUIRE(out != nullptr, FMOE_ERR_ARG, "fmoe_combine_routed: out is null");
  FMOE_REQUIRE(K == 0 || (rows && slot_of && w_sorted), FMOE_ERR_ARG, "fmoe_combine_routed: null pointer argument");
  FMOE_REQUIRE(out_row_stride >= D, FMOE_ERR_ARG, "fmoe_combine_routed: out_row_stride < D");
  const WeightedSlotSource src{slot_of, static_cast<const char*>(rows), w_sorted,
                               D * static_cast<int64_t>(dtype_size(dtype)), T * K, static_cast<int>(K), w_dtype};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = 0;
  FMOE_DISPATCH_DTYPE(dtype, DT,
                      rc = (launch_gather_sum<DT, true, WeightedSlotSource>(src, out, out_row_stride, T, D,
                                                                            accumulate != 0, s)));
  return rc;
}

extern "C" int fmoe_combine_routed_bwd(const void* rows, const int32_t* slot_of, const void* w_sorted, int w_dtype,
                                       const void* grad_out, int64_t grad_out_row_stride, void* grad_rows,
                                       float* grad_w, int64_t T, int64_t K, int64_t D, int dtype, void* stream) {
  FMOE_RANGE("fmoe_combine_routed_bwd");
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype), FMOE_ERR_ARG,
               "fmoe_combine_routed_bwd: bad dtype %d / %d", dtype, w_dtype);
  FMOE_REQUIRE(T >= 0 && K >= 0 && D >= 0, FMOE_ERR_ARG, "fmoe_combine_routed_bwd: negative size");
  FMOE_REQUIRE(T * K < (1ll << 31), FMOE_ERR_UNSUPPORTED, "fmoe_combine_routed_bwd: T*K must fit in int32");
  const int64_t N = T * K;
  if (N == 0) return FMOE_OK;
  FMOE_REQUIRE(slot_of && w_sorted && grad_out && grad_rows && (grad_w == nullptr || rows != nullptr), FMOE_ERR_ARG,
               "fmoe_combine_routed_bwd: null pointer argument");
  FMOE_REQUIRE(grad_out_row_stride >= D, FMOE_ERR_ARG, "fmoe_combine_routed_bwd: grad_out_row_stride < D");
  const int eb = dtype_size(dtype);
  const int kvec = 16 / eb;
  FMOE_REQUIRE(D % kvec == 0 && aligned_to(grad_out, 16) && aligned_to(grad_rows, 16) && aligned_to(rows, 16) &&
                   (grad_out_row_stride * eb) % 16 == 0,
               FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_routed_bwd: D must be a multiple of %d and buffers 16-byte aligned", kvec);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (grad_w != nullptr) FMOE_CUDA(cudaMemsetAsync(grad_w, 0, sizeof(float) * N, s));  // slots no token names
  if (D == 0) return FMOE_OK;
  const int64_t dvec = D / kvec;
  int group = static_cast<int>(K >= kBwdWarps ? 1 : (kBwdWarps + K - 1) / K);
  if (group > kBwdWarps) group = kBwdWarps;
  const int grid = static_cast<int>(clamp_grid((T + group - 1) / group, g_bwd_ctas_per_sm));
  const SlotBwdSource src{slot_of, static_cast<const char*>(rows), w_sorted, D * static_cast<int64_t>(eb), N,
                          static_cast<int>(K), w_dtype};
  int rc = 0;
#define FMOE_BWD_LAUNCH(DT, GW)                                                  \
  combine_bwd_kernel<DT, GW, SlotBwdSource><<<grid, kBwdWarps * 32, 0, s>>>(     \
      src, grad_out, grad_out_row_stride, grad_rows, grad_w, T, D, dvec, group)
  FMOE_DISPATCH_DTYPE(dtype, DT, {
    if (grad_w) FMOE_BWD_LAUNCH(DT, true); else FMOE_BWD_LAUNCH(DT, false);
    rc = check_launch("combine_bwd_kernel (routed)");
  });
#undef FMOE_BWD_LAUNCH
  return rc;
}

// ---- SwiGLU derivative ------------------------------------------------------------------------
// h = [gate | up] (pre-activations, [R, 2*ff]), g = gradient of silu(gate) * up ([R, ff]):
//   d_gate = g * up * s * (1 + gate * (1 - s)),  d_up = g * gate * s,  s = sigmoid(gate)
// written as [d_gate | d_up] in the layout of h. One pass: 2*ff + ff elements read and 2*ff
// written per row, 16-byte accesses, fp32 arithmetic, one rounding to bf16.
namespace fmoe {
__global__ void __launch_bounds__(256)
    swiglu_bwd_kernel(const uint4* __restrict__ h, const uint4* __restrict__ g, uint4* __restrict__ dh,
                      int64_t rows, int64_t ffvec, const int64_t* __restrict__ rows_used) {
  if (rows_used != nullptr) {  // a capacity-sized buffer: only its first *rows_used rows hold data
    const int64_t used = *rows_used;
    rows = used < 0 ? 0 : (used < rows ? used : rows);
  }
  const int64_t total = rows * ffvec;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / ffvec, c = i - r * ffvec;
    float gate[8], up[8], gr[8], dg[8], du[8];
    unpack16<FMOE_BF16>(ld_stream16(h + r * 2 * ffvec + c), gate);
    unpack16<FMOE_BF16>(ld_stream16(h + r * 2 * ffvec + ffvec + c), up);
    unpack16<FMOE_BF16>(ld_stream16(g + r * ffvec + c), gr);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-gate[k]));
      dg[k] = gr[k] * up[k] * s * (1.f + gate[k] * (1.f - s));
      du[k] = gr[k] * gate[k] * s;
    }
    st_stream16(dh + r * 2 * ffvec + c, pack16<FMOE_BF16>(dg));
    st_stream16(dh + r * 2 * ffvec + ffvec + c, pack16<FMOE_BF16>(du));
  }
}
// Derivative of the exact GELU epilogue: grad_h = grad_act * (Phi(h) + h * phi(h)), Phi and phi
// the standard normal distribution and density; streaming, fp32 arithmetic.
__global__ void __launch_bounds__(256)
    gelu_bwd_kernel(const uint4* __restrict__ h, const uint4* __restrict__ g, uint4* __restrict__ dh, int64_t total) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float x[8], gr[8], d[8];
    unpack16<FMOE_BF16>(ld_stream16(h + i), x);
    unpack16<FMOE_BF16>(ld_stream16(g + i), gr);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float cdf = 0.5f * (1.f + erff(x[k] * 0.70710678118654752f));
      const float pdf = 0.39894228040143268f * __expf(-0.5f * x[k] * x[k]);
      d[k] = gr[k] * (cdf + x[k] * pdf);
    }
    st_stream16(dh + i, pack16<FMOE_BF16>(d));
  }
}
}  // namespace fmoe

extern "C" int fmoe_gelu_bwd(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t n,
                             void* stream) {
  FMOE_RANGE("fmoe_gelu_bwd");
  FMOE_REQUIRE(rows >= 0 && n >= 0, FMOE_ERR_ARG, "fmoe_gelu_bwd: negative size");
  FMOE_REQUIRE(n % 8 == 0, FMOE_ERR_UNSUPPORTED, "fmoe_gelu_bwd: n=%lld must be a multiple of 8", (long long)n);
  if (rows == 0 || n == 0) return FMOE_OK;
  FMOE_REQUIRE(h && grad_act && grad_h, FMOE_ERR_ARG, "fmoe_gelu_bwd: null pointer argument");
  FMOE_REQUIRE(aligned_to(h, 16) && aligned_to(grad_act, 16) && aligned_to(grad_h, 16), FMOE_ERR_ARG,
               "fmoe_gelu_bwd: buffers must be 16-byte aligned");
  const int64_t total = rows * (n / 8);
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < kNumSMs * 8 ? blocks : kNumSMs * 8);
  gelu_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(h), static_cast<const uint4*>(grad_act), static_cast<uint4*>(grad_h), total);
  return check_launch("gelu_bwd_kernel");
}

extern "C" int fmoe_swiglu_bwd(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t ff,
                               void* stream) {
  FMOE_RANGE("fmoe_swiglu_bwd");
  return fmoe_swiglu_bwd_ragged(h, grad_act, grad_h, rows, ff, nullptr, stream);
}

extern "C" int fmoe_swiglu_bwd_ragged(const void* h, const void* grad_act, void* grad_h, int64_t rows, int64_t ff,
                                      const int64_t* rows_used, void* stream) {
  FMOE_RANGE("fmoe_swiglu_bwd_ragged");
  FMOE_REQUIRE(rows >= 0 && ff >= 0, FMOE_ERR_ARG, "fmoe_swiglu_bwd: negative size");
  FMOE_REQUIRE(ff % 8 == 0, FMOE_ERR_UNSUPPORTED, "fmoe_swiglu_bwd: ff=%lld must be a multiple of 8", (long long)ff);
  if (rows == 0 || ff == 0) return FMOE_OK;
  FMOE_REQUIRE(h && grad_act && grad_h, FMOE_ERR_ARG, "fmoe_swiglu_bwd: null pointer argument");
  FMOE_REQUIRE(aligned_to(h, 16) && aligned_to(grad_act, 16) && aligned_to(grad_h, 16), FMOE_ERR_ARG,
               "fmoe_swiglu_bwd: buffers must be 16-byte aligned");
  const int64_t total = rows * (ff / 8);
  const int64_t blocks = (total + 255) / 256;
  const int grid = static_cast<int>(blocks < kNumSMs * 8 ? blocks : kNumSMs * 8);
  swiglu_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(h), static_cast<const uint4*>(grad_act), static_cast<uint4*>(grad_h), rows, ff / 8,
      rows_used);
  return check_launch("swiglu_bwd_kernel");
}
