// fmoe_combine_fwd_static: the planned combine for callers that must not allocate.
//
// Some hosts of this library cannot hand it scratch memory of their own and cannot
// let it call cudaMalloc either: a plugin running inside a framework whose memory
// pool has already claimed the whole of HBM (a side allocation fails, or is against
// the host's rules), or a latency-critical serving loop where cudaMalloc's implicit
// device-wide synchronisation would stall every other stream. For them the plan
// (the inverse of the index vector) is built in a fixed array that is part of this
// library's device image. Every GPU that loads the library holds that array until
// the process exits, whether or not this entry point is ever called.
#include <mutex>

#include "plan.cuh"

namespace fmoe {

// File-scope device array: the plan scratch of the static entry point. On the host
// this name is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress below and is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_plan[FMOE_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void* g_static_plan_addr[kMaxDevices] = {};
static std::mutex g_static_mutex;

// Device address of the array on the CURRENT device; resolved once per device.
static int static_plan_address(void** out) {
  int dev = -1;
  FMOE_CUDA(cudaGetDevice(&dev));
  FMOE_REQUIRE(dev >= 0 && dev < kMaxDevices, FMOE_ERR_DEVICE,
               "fmoe_combine_fwd_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_plan_addr[dev] == nullptr) {
    void* p = nullptr;
    FMOE_CUDA(cudaGetSymbolAddress(&p, g_static_plan));
    FMOE_REQUIRE(p != nullptr && aligned_to(p, 256), FMOE_ERR_DEVICE,
                 "fmoe_combine_fwd_static: symbol address %p is null or misaligned", p);
    g_static_plan_addr[dev] = p;
  }
  *out = g_static_plan_addr[dev];
  return FMOE_OK;
}

}  // namespace fmoe

extern "C" int fmoe_combine_fwd_static(const int64_t* ptr_table, const int32_t* chunk_sizes,
                                       const int64_t* expert_offsets, const void* idx,
                                       int idx_type, const void* w, int w_dtype, void* out,
                                       int64_t out_row_stride, int64_t E, int64_t N, int64_t T,
                                       int64_t D, int dtype, int accumulate, int32_t* status,
                                       void* stream) {
  FMOE_RANGE("fmoe_combine_fwd_static");
  using namespace fmoe;
  FMOE_REQUIRE(N >= 0 && T >= 0, FMOE_ERR_ARG, "fmoe_combine_fwd_static: negative size");
  const size_t need = fmoe_combine_plan_bytes(N, T);
  FMOE_REQUIRE(need <= static_cast<size_t>(FMOE_STATIC_SCRATCH_BYTES), FMOE_ERR_WORKSPACE,
               "fmoe_combine_fwd_static: N=%lld rows into T=%lld outputs need %zu bytes of plan, the "
               "built-in array holds %d; use fmoe_combine_plan + fmoe_combine_gather with your own "
               "scratch",
               (long long)N, (long long)T, need, FMOE_STATIC_SCRATCH_BYTES);
  void* plan = nullptr;
  int rc = static_plan_address(&plan);
  if (rc != 0) return rc;
  // The array still holds the previous call's plan. fmoe_combine_plan clears the two
  // sections that must start at zero (segment offsets and target histogram) on `stream`
  // and overwrites every other entry that the gather reads.
  rc = fmoe_combine_plan(ptr_table, chunk_sizes, expert_offsets, idx, idx_type, w, w_dtype, E, N, T,
                         D, dtype, plan, FMOE_STATIC_SCRATCH_BYTES, status, stream);
  if (rc != 0) return rc;
  return fmoe_combine_gather(plan, out, out_row_stride, N, T, D, dtype, accumulate, stream);
}
