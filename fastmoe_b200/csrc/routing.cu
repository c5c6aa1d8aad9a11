// Router top-k / gate softmax and the index-offset builder (histogram +
// prefix sum + stable placement). Replaces the torch.topk, softmax, argsort,
// gathers and bincount of MoEFeedForward.gate_and_sort in polkadot21/fastmoe
// (src/fastmoe/models/tiny_model.py:97-153) with three small launches and no
// comparison sort. The order produced is the stable one: by expert id, then by
// flat routed position t*K+k.
#include "common.cuh"

namespace fmoe {

// ---- top-k + softmax -----------------------------------------------------------
// Monotone map float -> uint32 (larger float = larger key); NaN sorts above
// +inf, as torch.topk treats it.
__device__ __forceinline__ uint32_t order_key(float f) {
  if (f != f) return 0xffffffffu;
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  if (k == 0xffffffffu) return __uint_as_float(0x7fc00000u);
  const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(b);
}

// One warp per token; lane l holds experts l, l+32, ... (ITEMS of them).
template <int ITEMS>
__global__ void __launch_bounds__(256)
    route_topk_kernel(const void* __restrict__ logits, int dtype, int64_t T, int E, int K,
                      int64_t* __restrict__ topk_idx, void* __restrict__ topk_w, int w_dtype) {
  const int lane = threadIdx.x & 31;
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;

  // (key << 32) | (0xffffffff - expert): max picks the larger value, then the lower expert id
  uint64_t item[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    const int e = lane + 32 * i;
    item[i] = 0;  // below every real entry (real ones have a non-zero low word)
    if (e < E) {
      const float f = load_scalar_as_float(logits, t * E + e, dtype);
      item[i] = (static_cast<uint64_t>(order_key(f)) << 32) | (0xffffffffu - static_cast<uint32_t>(e));
    }
  }

  float my_val = 0.f;  // lane k keeps the k-th selected logit
  int my_idx = 0;
  for (int k = 0; k < K; ++k) {
    uint64_t best = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) best = item[i] > best ? item[i] : best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const uint64_t other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    // retire the winner (its lane is the only one holding this exact item)
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      if (item[i] == best) item[i] = 0;
    if (lane == k) {
      my_val = key_to_float(static_cast<uint32_t>(best >> 32));
      my_idx = static_cast<int>(0xffffffffu - static_cast<uint32_t>(best & 0xffffffffu));
    }
  }

  // softmax over the K selected logits in fp32 (tiny_model.py:100)
  const float m = __shfl_sync(0xffffffffu, my_val, 0);
  float ex = lane < K ? expf(my_val - m) : 0.f;
  float sum = ex;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane < K) {
    topk_idx[t * K + lane] = my_idx;
    store_scalar_from_float(topk_w, t * K + lane, w_dtype, ex / sum);
  }
}

// ---- index builder ----------------------------------------------------------------
constexpr int kChunkTokens = 32;  // tokens per warp-chunk

// Per chunk histogram of expert ids.
__global__ void __launch_bounds__(256)
    index_hist_kernel(const int64_t* __restrict__ topk_idx, int64_t T, int E, int K,
                      int32_t* __restrict__ chunk_hist, int32_t* status) {
  extern __shared__ int32_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int64_t chunk = blockIdx.x * static_cast<int64_t>(nwarps) + warp;
  const int64_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  if (chunk >= nchunks) return;  // whole warp leaves; no block-level barrier below
  int32_t* cnt = smem + warp * E;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t first = chunk * kChunkTokens * K;
  const int64_t last = min(T * K, first + static_cast<int64_t>(kChunkTokens) * K);
  int flags = 0;
  for (int64_t i = first + lane; i < last; i += 32) {
    const int64_t e = topk_idx[i];
    if (e < 0 || e >= E)
      flags |= FMOE_STATUS_BAD_EXPERT;
    else
      atomicAdd(&cnt[e], 1);
  }
  __syncwarp();
  for (int e = lane; e < E; e += 32) chunk_hist[chunk * E + e] = cnt[e];
  if (flags && status != nullptr) atomicOr(status, flags);
}

// One warp per expert: turns that expert's per-chunk counts into an exclusive prefix over
// the chunks (in place) and leaves the expert's total. Up to 16 x 32 chunks are loaded
// before the first store, so the strided loads overlap instead of queueing behind stores.
__global__ void __launch_bounds__(256)
    index_chunk_scan_kernel(int32_t* __restrict__ chunk_hist, int64_t nchunks, int E,
                            int32_t* __restrict__ totals) {
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= E) return;
  constexpr int kBatch = 16;
  int32_t carry = 0;
  for (int64_t base = 0; base < nchunks; base += 32 * kBatch) {
    int32_t v[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int64_t c = base + 32 * i + lane;
      v[i] = c < nchunks ? chunk_hist[c * E + e] : 0;
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int64_t c = base + 32 * i + lane;
      int32_t incl = v[i];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (c < nchunks) chunk_hist[c * E + e] = carry + incl - v[i];
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  if (lane == 0) totals[e] = carry;
}

// Stable placement: slot = offsets[e] + rows of e in earlier chunks + rows of e earlier in
// this chunk. Every CTA first rebuilds the exclusive prefix over the experts' totals in
// shared memory (E values: cheaper than another launch); CTA 0 also publishes counts,
// offsets and the per-rank sums. A warp then walks its chunk in flat order, 32 entries at
// a time; __match_any_sync ranks equal experts inside a step.
__global__ void __launch_bounds__(256)
    index_place_kernel(const int64_t* __restrict__ topk_idx, const void* __restrict__ topk_w,
                       int w_dtype, int64_t T, int E, int K, int world,
                       const int32_t* __restrict__ chunk_hist, const int32_t* __restrict__ totals,
                       int64_t* __restrict__ counts, int64_t* __restrict__ offsets,
                       int64_t* __restrict__ rank_counts, int64_t* __restrict__ reverse_map,
                       void* __restrict__ sorted_w, int32_t* __restrict__ slot_of) {
  extern __shared__ int32_t smem[];
  int32_t* off_s = smem;          // [E + 1] exclusive prefix of the totals
  int32_t* cnt_all = smem + E + 1;  // [warps][E] running counts inside each warp's chunk
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;

  if (warp == 0) {
    int32_t carry = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      const int32_t v = e < E ? totals[e] : 0;
      int32_t incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t n = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += n;
      }
      if (e < E) off_s[e] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) off_s[E] = carry;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      counts[e] = off_s[e + 1] - off_s[e];
      offsets[e] = off_s[e];
    }
    const int e_local = E / world;
    for (int r = threadIdx.x; r < world; r += blockDim.x)
      rank_counts[r] = off_s[(r + 1) * e_local] - off_s[r * e_local];
  }

  const int64_t chunk = blockIdx.x * static_cast<int64_t>(nwarps) + warp;
  const int64_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  if (chunk >= nchunks) return;
  int32_t* cnt = cnt_all + warp * E;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t first = chunk * kChunkTokens * K;
  const int64_t last = min(T * K, first + static_cast<int64_t>(kChunkTokens) * K);
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int64_t base = first; base < last; base += 32) {
    const int64_t i = base + lane;
    const bool in = i < last;
    int64_t e = in ? topk_idx[i] : -1;
    const bool ok = in && e >= 0 && e < E;
    // lanes without a valid expert get distinct keys so they never group
    const int key = ok ? static_cast<int>(e) : -1 - lane;
    const uint32_t peers = __match_any_sync(0xffffffffu, key);
    int32_t before = 0;
    if (ok) before = cnt[e];
    __syncwarp();
    if (ok && (peers & lt_mask) == 0) cnt[e] = before + __popc(peers);  // group leader
    __syncwarp();
    if (ok) {
      const int64_t slot = static_cast<int64_t>(off_s[e]) + chunk_hist[chunk * E + e] + before +
                           __popc(peers & lt_mask);
      reverse_map[slot] = i / K;
      store_scalar_from_float(sorted_w, slot, w_dtype, load_scalar_as_float(topk_w, i, w_dtype));
      slot_of[i] = static_cast<int32_t>(slot);
    } else if (in) {
      slot_of[i] = -1;
    }
  }
}

// Single CTA that publishes all-zero counts, offsets and rank sums when there is nothing to place.
__global__ void index_empty_kernel(int E, int world, int64_t* counts, int64_t* offsets, int64_t* rank_counts) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = offsets[e] = 0;
  for (int r = threadIdx.x; r < world; r += blockDim.x) rank_counts[r] = 0;
}

// Warps per CTA of the histogram / placement kernels: per-warp counters of E ints each, plus
// the E+1 offsets of the placement kernel, inside the default 48 KB of shared memory.
static int warps_for(int E) {
  int w = static_cast<int>((48 * 1024 - sizeof(int32_t) * (static_cast<size_t>(E) + 1)) /
                           (sizeof(int32_t) * static_cast<size_t>(E)));
  if (w > 8) w = 8;
  return w;
}

}  // namespace fmoe

using namespace fmoe;

extern "C" int fmoe_route_topk(const void* logits, int dtype, int64_t T, int64_t E, int64_t K,
                               int64_t* topk_idx, void* topk_w, int w_dtype, void* stream) {
  FMOE_RANGE("fmoe_route_topk");
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype), FMOE_ERR_ARG,
               "fmoe_route_topk: bad dtype %d / w_dtype %d", dtype, w_dtype);
  FMOE_REQUIRE(T >= 0 && E >= 0 && K >= 0, FMOE_ERR_ARG, "fmoe_route_topk: negative size");
  FMOE_REQUIRE(K <= E, FMOE_ERR_ARG, "fmoe_route_topk: K=%lld exceeds E=%lld", (long long)K,
               (long long)E);
  FMOE_REQUIRE(K <= 32 && E <= 2048, FMOE_ERR_UNSUPPORTED,
               "fmoe_route_topk: supports K <= 32 and E <= 2048 (got K=%lld E=%lld)", (long long)K,
               (long long)E);
  if (T == 0 || K == 0) return FMOE_OK;
  FMOE_REQUIRE(logits && topk_idx && topk_w, FMOE_ERR_ARG, "fmoe_route_topk: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int warps = 8;
  const int grid = static_cast<int>((T + warps - 1) / warps);
  const int items = static_cast<int>((E + 31) / 32);
#define FMOE_TOPK(I)                                                                          \
  route_topk_kernel<I><<<grid, warps * 32, 0, s>>>(logits, dtype, T, static_cast<int>(E),     \
                                                   static_cast<int>(K), topk_idx, topk_w, w_dtype)
  if (items <= 1) FMOE_TOPK(1);
  else if (items <= 2) FMOE_TOPK(2);
  else if (items <= 4) FMOE_TOPK(4);
  else if (items <= 8) FMOE_TOPK(8);
  else if (items <= 16) FMOE_TOPK(16);
  else if (items <= 32) FMOE_TOPK(32);
  else FMOE_TOPK(64);
#undef FMOE_TOPK
  return check_launch("route_topk_kernel");
}

extern "C" size_t fmoe_build_index_bytes(int64_t T, int64_t E, int64_t K) {
  (void)K;
  if (T < 0 || E < 0) return 0;
  const int64_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  // per-chunk histograms [nchunks][E] followed by the per-expert totals [E]
  return round_up(sizeof(int32_t) * static_cast<size_t>(nchunks > 0 ? nchunks : 1) *
                      static_cast<size_t>(E > 0 ? E : 1),
                  256) +
         round_up(sizeof(int32_t) * static_cast<size_t>(E > 0 ? E : 1), 256);
}

extern "C" int fmoe_build_index(const int64_t* topk_idx, const void* topk_w, int w_dtype, int64_t T,
                                int64_t E, int64_t K, int64_t world, int64_t* reverse_map,
                                void* sorted_w, int64_t* counts, int64_t* offsets,
                                int64_t* rank_counts, int32_t* slot_of, void* scratch,
                                size_t scratch_bytes, int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_build_index");
  FMOE_REQUIRE(valid_dtype(w_dtype), FMOE_ERR_ARG, "fmoe_build_index: bad w_dtype %d", w_dtype);
  FMOE_REQUIRE(T >= 0 && E > 0 && K >= 0 && world > 0, FMOE_ERR_ARG,
               "fmoe_build_index: sizes must be T >= 0, E > 0, K >= 0, world > 0");
  FMOE_REQUIRE(E % world == 0, FMOE_ERR_ARG, "fmoe_build_index: E=%lld not divisible by world=%lld",
               (long long)E, (long long)world);
  FMOE_REQUIRE(E <= 4096, FMOE_ERR_UNSUPPORTED, "fmoe_build_index: supports E <= 4096");
  FMOE_REQUIRE(T * K < (1ll << 31), FMOE_ERR_UNSUPPORTED, "fmoe_build_index: T*K must fit in int32");
  FMOE_REQUIRE(counts && offsets && rank_counts, FMOE_ERR_ARG,
               "fmoe_build_index: counts/offsets/rank_counts must not be null");
  FMOE_REQUIRE(scratch != nullptr && aligned_to(scratch, 256) &&
                   scratch_bytes >= fmoe_build_index_bytes(T, E, K),
               FMOE_ERR_WORKSPACE, "fmoe_build_index: scratch null, misaligned or smaller than %zu",
               fmoe_build_index_bytes(T, E, K));
  const int64_t N = T * K;
  FMOE_REQUIRE(N == 0 || (topk_idx && topk_w && reverse_map && sorted_w && slot_of), FMOE_ERR_ARG,
               "fmoe_build_index: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int e = static_cast<int>(E);
  if (N == 0) {
    index_empty_kernel<<<1, 256, 0, s>>>(e, static_cast<int>(world), counts, offsets, rank_counts);
    return check_launch("index_empty_kernel");
  }
  const int64_t nchunks = (T + kChunkTokens - 1) / kChunkTokens;
  int32_t* chunk_hist = static_cast<int32_t*>(scratch);
  int32_t* totals = reinterpret_cast<int32_t*>(
      static_cast<char*>(scratch) + round_up(sizeof(int32_t) * static_cast<size_t>(nchunks) * E, 256));
  const int warps = warps_for(e);
  const int grid = static_cast<int>((nchunks + warps - 1) / warps);
  index_hist_kernel<<<grid, warps * 32, sizeof(int32_t) * static_cast<size_t>(E) * warps, s>>>(
      topk_idx, T, e, static_cast<int>(K), chunk_hist, status);
  FMOE_CUDA(cudaGetLastError());
  index_chunk_scan_kernel<<<(e + 7) / 8, 256, 0, s>>>(chunk_hist, nchunks, e, totals);
  FMOE_CUDA(cudaGetLastError());
  index_place_kernel<<<grid, warps * 32, sizeof(int32_t) * (static_cast<size_t>(E) * warps + E + 1), s>>>(
      topk_idx, topk_w, w_dtype, T, e, static_cast<int>(K), static_cast<int>(world), chunk_hist, totals,
      counts, offsets, rank_counts, reverse_map, sorted_w, slot_of);
  return check_launch("index_place_kernel");
}
