// Builds the combine plan: a counting sort of the N routed rows by target row,
// stable in the global row id, with every row resolved through the pointer
// table. Stands in for the per-row lookups of the reference kernel
// (src/fastmoe/kernels/ops.py:129-163) so that the data kernels stream rows
// without touching idx, w, offsets or the pointer table.
#include <cooperative_groups.h>

#include "plan.cuh"

namespace fmoe {

struct PlanArgs {
  const int64_t* ptr_table;
  const int32_t* chunk_sizes;
  const int64_t* expert_offsets;
  const void* idx;
  const void* w;
  int64_t N, T, D;
  int E;
  int idx_type, w_dtype, elem_bytes;
  PlanView p;
  int32_t* status;
};

// 1. histogram of targets; the atomic's return value is the row's arrival rank
__global__ void __launch_bounds__(256) plan_hist_kernel(const PlanArgs a) {
  const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= a.N) return;
  const int64_t t = load_index(a.idx, g, a.idx_type);
  if (t < 0 || t >= a.T) {
    a.p.rank[g] = -1;
    if (a.status != nullptr) atomicOr(a.status, FMOE_STATUS_BAD_INDEX);
    return;
  }
  a.p.rank[g] = atomicAdd(&a.p.cnt[t], 1);
}

// 2. exclusive prefix sum of the histogram -> seg_off[0..T]; one CTA walks the
//    array in 1024-wide steps carrying the running total
__global__ void __launch_bounds__(1024) plan_scan_kernel(const int32_t* __restrict__ cnt,
                                                         int32_t* __restrict__ seg_off, int64_t T) {
  __shared__ int32_t warp_sums[32];
  __shared__ int32_t carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int64_t base = 0; base < T; base += 1024) {
    const int64_t i = base + threadIdx.x;
    const int32_t v = i < T ? cnt[i] : 0;
    int32_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t n = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int32_t s = warp_sums[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int32_t n = __shfl_up_sync(0xffffffffu, s, d);
        if (lane >= d) s += n;
      }
      warp_sums[lane] = s;  // inclusive over warps
    }
    __syncthreads();
    const int32_t carry = carry_s;
    const int32_t warp_excl = warp == 0 ? 0 : warp_sums[warp - 1];
    if (i < T) seg_off[i] = carry + warp_excl + incl - v;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) seg_off[T] = carry_s;
}

// 3. place every row at seg_off[target] + arrival rank
__global__ void __launch_bounds__(256) plan_place_kernel(const PlanArgs a) {
  const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= a.N) return;
  const int32_t r = a.p.rank[g];
  if (r < 0) return;
  const int64_t t = load_index(a.idx, g, a.idx_type);
  a.p.seg_rows[a.p.seg_off[t] + r] = static_cast<int32_t>(g);
}

// 4. stable rank inside the segment (rows smaller than mine), then resolve the
//    row through the pointer table and store address + fp32 weight by slot
__global__ void __launch_bounds__(256) plan_finalize_kernel(const PlanArgs a) {
  const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (g >= a.N) return;
  int32_t r = a.p.rank[g];
  if (r < 0) return;
  const int64_t t = load_index(a.idx, g, a.idx_type);
  const int32_t beg = a.p.seg_off[t], end = a.p.seg_off[t + 1];
  if (end - beg <= kPlanStableCap) {
    r = 0;
    for (int32_t j = beg; j < end; ++j) r += (a.p.seg_rows[j] < g) ? 1 : 0;
  }
  const int32_t slot = beg + r;

  int64_t addr = 0;
  int flags = 0;
  const int e = find_expert(a.expert_offsets, a.E, g);
  const int64_t local = g - a.expert_offsets[e];
  if (local < 0 || local >= a.chunk_sizes[e]) {
    flags = FMOE_STATUS_BAD_EXPERT;
  } else {
    const int64_t base = a.ptr_table[e];
    if (base == 0)
      flags = FMOE_STATUS_NULL_PTR;
    else
      addr = base + local * a.D * a.elem_bytes;
  }
  if (flags != 0 && a.status != nullptr) atomicOr(a.status, flags);
  a.p.row_of_slot[slot] = static_cast<int32_t>(g);
  a.p.src_sorted[slot] = addr;
  a.p.w_sorted[slot] = load_scalar_as_float(a.w, g, a.w_dtype);
}

// ---- all four steps in one cooperative launch -----------------------------------------
// The separate kernels above are launch-latency bound (a few microseconds each for 64k
// rows). This kernel runs the same steps with grid-wide barriers in between: zero the
// histogram, count, scan inside 512-wide pieces (the piece-local offsets overwrite the
// histogram), place, finalize. The prefix over the piece totals is not a step of its own:
// every CTA works it out in shared memory at the start of the place step, which then adds
// it on the fly and also writes the final offsets of the pieces the CTA owns. Every step
// is a round trip of dependent global accesses plus a grid barrier, so one step fewer is
// what counts. The piece totals borrow the row_of_slot section, which is not written before
// the last step.
constexpr int kFusedThreads = 512;
constexpr int kFusedMaxPieces = 2048;  // pieces of 512 targets: T up to 1M (their prefix sits in shared memory)

__device__ __forceinline__ int32_t block_exclusive_scan(int32_t v, int32_t* warp_sums, int32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int32_t n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  __syncthreads();  // warp_sums may still be read from the previous call
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t s = lane < (kFusedThreads >> 5) ? warp_sums[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t n = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += n;
    }
    warp_sums[lane] = s;
  }
  __syncthreads();
  total = warp_sums[(kFusedThreads >> 5) - 1];
  return (warp == 0 ? 0 : warp_sums[warp - 1]) + incl - v;
}

__global__ void __launch_bounds__(kFusedThreads) plan_fused_kernel(const PlanArgs a) {
  namespace cg = cooperative_groups;
  cg::grid_group grid = cg::this_grid();
  __shared__ int32_t warp_sums[32];
  __shared__ int32_t piece_base[kFusedMaxPieces];
  const int64_t tid = blockIdx.x * static_cast<int64_t>(kFusedThreads) + threadIdx.x;
  const int64_t nthreads = static_cast<int64_t>(gridDim.x) * kFusedThreads;
  int32_t* piece_total = a.p.row_of_slot;
  const int64_t pieces = (a.T + kFusedThreads - 1) / kFusedThreads;

  for (int64_t t = tid; t < a.T; t += nthreads) a.p.cnt[t] = 0;
  grid.sync();

  int flags = 0;
  for (int64_t g = tid; g < a.N; g += nthreads) {
    const int64_t t = load_index(a.idx, g, a.idx_type);
    if (t < 0 || t >= a.T) {
      a.p.rank[g] = -1;
      flags |= FMOE_STATUS_BAD_INDEX;
    } else {
      a.p.rank[g] = atomicAdd(&a.p.cnt[t], 1);
    }
  }
  grid.sync();

  for (int64_t piece = blockIdx.x; piece < pieces; piece += gridDim.x) {
    const int64_t t = piece * kFusedThreads + threadIdx.x;
    const int32_t v = t < a.T ? a.p.cnt[t] : 0;
    int32_t total;
    const int32_t excl = block_exclusive_scan(v, warp_sums, total);
    if (t < a.T) a.p.cnt[t] = excl;  // the histogram has done its job: keep the piece-local offset in its place
    if (threadIdx.x == 0) piece_total[piece] = total;
  }
  grid.sync();

  {  // first row of every piece: exclusive prefix of the piece totals, by every CTA for itself
    int32_t carry = 0;
    for (int64_t q0 = 0; q0 < pieces; q0 += kFusedThreads) {
      const int64_t q = q0 + threadIdx.x;
      int32_t round_total;
      const int32_t excl = block_exclusive_scan(q < pieces ? piece_total[q] : 0, warp_sums, round_total);
      if (q < pieces) piece_base[q] = carry + excl;
      carry += round_total;
    }
    __syncthreads();
    for (int64_t piece = blockIdx.x; piece < pieces; piece += gridDim.x) {  // final offsets of my pieces
      const int64_t t = piece * kFusedThreads + threadIdx.x;
      if (t < a.T) a.p.seg_off[t] = a.p.cnt[t] + piece_base[piece];
      if (piece == pieces - 1 && threadIdx.x == 0) a.p.seg_off[a.T] = carry;
    }
  }
  for (int64_t g = tid; g < a.N; g += nthreads) {
    const int32_t r = a.p.rank[g];
    if (r < 0) continue;
    const int64_t t = load_index(a.idx, g, a.idx_type);
    a.p.seg_rows[a.p.cnt[t] + piece_base[t / kFusedThreads] + r] = static_cast<int32_t>(g);
  }
  grid.sync();
  // the last step: a kernel launched as a programmatic dependent of this one (the gather) may
  // have its CTAs placed from here on; it still waits for this grid to complete before it reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  for (int64_t g = tid; g < a.N; g += nthreads) {
    int32_t r = a.p.rank[g];
    if (r < 0) continue;
    const int64_t t = load_index(a.idx, g, a.idx_type);
    const int32_t beg = a.p.seg_off[t], end = a.p.seg_off[t + 1];
    if (end - beg <= kPlanStableCap) {
      r = 0;
      for (int32_t j = beg; j < end; ++j) r += (a.p.seg_rows[j] < g) ? 1 : 0;
    }
    const int32_t slot = beg + r;
    int64_t addr = 0;
    const int e = find_expert(a.expert_offsets, a.E, g);
    const int64_t local = g - a.expert_offsets[e];
    if (local < 0 || local >= a.chunk_sizes[e]) {
      flags |= FMOE_STATUS_BAD_EXPERT;
    } else {
      const int64_t base = a.ptr_table[e];
      if (base == 0)
        flags |= FMOE_STATUS_NULL_PTR;
      else
        addr = base + local * a.D * a.elem_bytes;
    }
    // row_of_slot doubles as the piece totals: they were last read before the previous barrier
    a.p.row_of_slot[slot] = static_cast<int32_t>(g);
    a.p.src_sorted[slot] = addr;
    a.p.w_sorted[slot] = load_scalar_as_float(a.w, g, a.w_dtype);
  }
  if (flags != 0 && a.status != nullptr) atomicOr(a.status, flags);
}

// fmoe_tune "plan_rows_per_thread": rows (or targets) each thread of the fused plan kernel
// takes per step. The kernel is bound by the latency of its steps and of the grid barriers
// between them, and a barrier over fewer CTAs is quicker, so a thread may well take several.
int g_plan_rows_per_thread = 1;

// Cooperative grid size for the current device (0 = cooperative launch not usable), cached.
static int fused_grid_limit() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int coop = 0, per_sm = 0, sms = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (coop && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, plan_fused_kernel, kFusedThreads, 0) ==
                    cudaSuccess &&
        per_sm > 0)
      cached[dev] = per_sm * sms;
    else
      cached[dev] = -1;
  }
  return cached[dev] > 0 ? cached[dev] : 0;
}

}  // namespace fmoe

extern "C" size_t fmoe_combine_plan_bytes(int64_t N, int64_t T) {
  if (N < 0 || T < 0) return 0;
  return fmoe::plan_view(nullptr, N, T).bytes;
}

extern "C" int fmoe_combine_plan(const int64_t* ptr_table, const int32_t* chunk_sizes,
                                 const int64_t* expert_offsets, const void* idx, int idx_type,
                                 const void* w, int w_dtype, int64_t E, int64_t N, int64_t T,
                                 int64_t D, int dtype, void* plan, size_t plan_bytes,
                                 int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_combine_plan");
  using namespace fmoe;
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype), FMOE_ERR_ARG,
               "fmoe_combine_plan: bad dtype %d / w_dtype %d", dtype, w_dtype);
  FMOE_REQUIRE(valid_itype(idx_type), FMOE_ERR_ARG, "fmoe_combine_plan: bad idx_type %d", idx_type);
  FMOE_REQUIRE(E >= 0 && N >= 0 && T >= 0 && D >= 0, FMOE_ERR_ARG,
               "fmoe_combine_plan: negative size (E=%lld N=%lld T=%lld D=%lld)", (long long)E,
               (long long)N, (long long)T, (long long)D);
  FMOE_REQUIRE(E < (1ll << 31) && N < (1ll << 31) && T < (1ll << 31) - 1, FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_plan: E, N and T must fit in int32");
  FMOE_REQUIRE(plan != nullptr && aligned_to(plan, 256), FMOE_ERR_WORKSPACE,
               "fmoe_combine_plan: plan scratch is null or not 256-byte aligned");
  PlanView pv = plan_view(plan, N, T);
  FMOE_REQUIRE(plan_bytes >= pv.bytes, FMOE_ERR_WORKSPACE,
               "fmoe_combine_plan: plan scratch has %zu bytes, needs %zu", plan_bytes, pv.bytes);
  FMOE_REQUIRE(N == 0 || T > 0, FMOE_ERR_ARG, "fmoe_combine_plan: N > 0 rows but T == 0");
  FMOE_REQUIRE(N == 0 || (ptr_table && chunk_sizes && expert_offsets && idx && w && E > 0),
               FMOE_ERR_ARG, "fmoe_combine_plan: null pointer argument or E == 0 with N > 0");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  PlanArgs a;
  a.ptr_table = ptr_table;
  a.chunk_sizes = chunk_sizes;
  a.expert_offsets = expert_offsets;
  a.idx = idx;
  a.w = w;
  a.N = N;
  a.T = T;
  a.D = D;
  a.E = static_cast<int>(E);
  a.idx_type = idx_type;
  a.w_dtype = w_dtype;
  a.elem_bytes = dtype_size(dtype);
  a.p = pv;
  a.status = status;

  const int64_t pieces = (T + kFusedThreads - 1) / kFusedThreads;
  const int limit = N > 0 ? fused_grid_limit() : 0;
  if (limit > 0 && pieces <= N && pieces <= kFusedMaxPieces) {
    // one cooperative launch; the piece totals fit into the row_of_slot section (N ints)
    const int64_t per_cta = static_cast<int64_t>(kFusedThreads) * (g_plan_rows_per_thread > 0 ? g_plan_rows_per_thread : 1);
    const int64_t want = ((N > T ? N : T) + per_cta - 1) / per_cta;
    const int grid = static_cast<int>(want < limit ? want : limit);
    void* params[] = {&a};
    FMOE_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(plan_fused_kernel), dim3(grid),
                                          dim3(kFusedThreads), params, 0, s));
    return FMOE_OK;
  }
  // cnt and seg_off are adjacent sections: one memset zeroes both (seg_off must
  // be all zero when N == 0 or T is tiny, the scan overwrites it otherwise)
  FMOE_CUDA(cudaMemsetAsync(pv.seg_off, 0,
                            reinterpret_cast<char*>(pv.rank) - reinterpret_cast<char*>(pv.seg_off),
                            s));
  if (N == 0) return FMOE_OK;
  const int blocks = static_cast<int>((N + 255) / 256);
  plan_hist_kernel<<<blocks, 256, 0, s>>>(a);
  FMOE_CUDA(cudaGetLastError());
  plan_scan_kernel<<<1, 1024, 0, s>>>(pv.cnt, pv.seg_off, T);
  FMOE_CUDA(cudaGetLastError());
  plan_place_kernel<<<blocks, 256, 0, s>>>(a);
  FMOE_CUDA(cudaGetLastError());
  plan_finalize_kernel<<<blocks, 256, 0, s>>>(a);
  return check_launch("plan_finalize_kernel");
}
