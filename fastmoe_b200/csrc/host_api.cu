// Host-buffer entry point: the whole combine for a caller that holds host
// memory. Mirrors grouped_weighted_scatter_add(expert_tensors, indices,
// weights, out_shape) of polkadot21/fastmoe (src/fastmoe/kernels/ops.py:365-394)
// for callers outside PyTorch: copies in, plans, gathers, copies out.
#include <mutex>
#include <vector>

#include "plan.cuh"

namespace fmoe {

struct ArenaView {
  size_t ptr_table, chunk_sizes, offsets, idx, w, rows, out, plan, status, total;
};

static ArenaView arena_view(const int64_t* sizes, int64_t E, int64_t N, int64_t T, int64_t D,
                            int dtype, int idx_type, int w_dtype, std::vector<size_t>* row_off) {
  ArenaView a{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t r = off;
    off += round_up(bytes > 0 ? bytes : 1, 256);
    return r;
  };
  const size_t eb = dtype_size(dtype);
  a.ptr_table = take(sizeof(int64_t) * E);
  a.chunk_sizes = take(sizeof(int32_t) * E);
  a.offsets = take(sizeof(int64_t) * E);
  a.idx = take((idx_type == FMOE_I64 ? 8 : 4) * static_cast<size_t>(N));
  a.w = take(dtype_size(w_dtype) * static_cast<size_t>(N));
  a.rows = off;
  for (int64_t e = 0; e < E; ++e) {
    // every expert matrix gets its own 256-byte aligned block: the matrices stay
    // disjoint, as the pointer-table interface has them
    const size_t o = take(static_cast<size_t>(sizes[e]) * D * eb);
    if (row_off) row_off->push_back(o);
  }
  a.out = take(static_cast<size_t>(T) * D * eb);
  a.plan = take(plan_view(nullptr, N, T).bytes);
  a.status = take(sizeof(int32_t));
  a.total = off;
  return a;
}

extern int g_host_chunks;  // token_major.cu (fmoe_tune "host_chunks")

// Events of one pipelined call, destroyed on every exit path.
struct EventSet {
  std::vector<cudaEvent_t> ev;
  ~EventSet() {
    for (cudaEvent_t e : ev) cudaEventDestroy(e);
  }
  cudaError_t add(cudaEvent_t* out) {
    const cudaError_t rc = cudaEventCreateWithFlags(out, cudaEventDisableTiming);
    if (rc == cudaSuccess) ev.push_back(*out);
    return rc;
  }
};

// Waits for both streams of a pipelined call when it is left early (an error part-way through):
// nothing of the call may still be running when the caller sees the status.
struct DrainOnExit {
  cudaStream_t a, b;
  bool armed = true;
  ~DrainOnExit() {
    if (!armed) return;
    cudaStreamSynchronize(b);
    cudaStreamSynchronize(a);
  }
};

// One non-blocking helper stream per device, created on first use and kept for the
// life of the process: the gathers and the copies back run there while the caller's
// stream keeps feeding the copy engine.
static cudaError_t side_stream(cudaStream_t* out) {
  constexpr int kMaxDevices = 64;
  static cudaStream_t streams[kMaxDevices] = {};
  static std::mutex guard;
  const std::lock_guard<std::mutex> lock(guard);
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  if (streams[dev] == nullptr) {
    rc = cudaStreamCreateWithFlags(&streams[dev], cudaStreamNonBlocking);
    if (rc != cudaSuccess) return rc;
  }
  *out = streams[dev];
  return cudaSuccess;
}

// Columns per slice of the pipelined call: whole 256-byte pieces of a row, slices of
// at least 4 KB per row (below that the strided copies stop paying).
static int64_t slice_cols(int64_t D, size_t eb) {
  const int64_t piece = static_cast<int64_t>(256 / eb);
  int chunks = g_host_chunks;
  if (chunks == 0) chunks = static_cast<int64_t>(D * eb) >= 16384 ? 4 : 1;
  if (chunks <= 1) return D;
  int64_t cols = (D + chunks - 1) / chunks;
  cols = (cols + piece - 1) / piece * piece;
  const int64_t min_cols = static_cast<int64_t>(4096 / eb);
  if (cols < min_cols) cols = min_cols;
  return cols < D ? cols : D;
}

}  // namespace fmoe

using namespace fmoe;

extern "C" size_t fmoe_combine_host_arena_bytes(const int64_t* chunk_sizes_host, int64_t E,
                                                int64_t N, int64_t T, int64_t D, int dtype) {
  if (E < 0 || N < 0 || T < 0 || D < 0 || !valid_dtype(dtype) || (E > 0 && !chunk_sizes_host))
    return 0;
  for (int64_t e = 0; e < E; ++e)
    if (chunk_sizes_host[e] < 0) return 0;
  // idx and w are sized for their widest types so the figure does not depend on them
  return arena_view(chunk_sizes_host, E, N, T, D, dtype, FMOE_I64, FMOE_F32, nullptr).total;
}

extern "C" int fmoe_combine_host(const void* const* expert_rows_host,
                                 const int64_t* chunk_sizes_host, const void* idx_host,
                                 int idx_type, const void* w_host, int w_dtype, void* out_host,
                                 int64_t E, int64_t N, int64_t T, int64_t D, int dtype, void* arena,
                                 size_t arena_bytes, void* stream) {
  FMOE_RANGE("fmoe_combine_host");
  FMOE_REQUIRE(valid_dtype(dtype) && valid_dtype(w_dtype) && valid_itype(idx_type), FMOE_ERR_ARG,
               "fmoe_combine_host: bad dtype/w_dtype/idx_type");
  FMOE_REQUIRE(E >= 0 && N >= 0 && T >= 0 && D >= 0, FMOE_ERR_ARG,
               "fmoe_combine_host: negative size");
  FMOE_REQUIRE(N < (1ll << 31) && T < (1ll << 31) - 1 && E < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_combine_host: E, N and T must fit in int32");
  FMOE_REQUIRE(out_host != nullptr || T * D == 0, FMOE_ERR_ARG, "fmoe_combine_host: out_host null");
  FMOE_REQUIRE(E == 0 || (expert_rows_host && chunk_sizes_host), FMOE_ERR_ARG,
               "fmoe_combine_host: null expert table");
  FMOE_REQUIRE(N == 0 || (idx_host && w_host), FMOE_ERR_ARG, "fmoe_combine_host: null idx or w");
  int64_t total_rows = 0;
  for (int64_t e = 0; e < E; ++e) {
    FMOE_REQUIRE(chunk_sizes_host[e] >= 0, FMOE_ERR_ARG, "fmoe_combine_host: negative chunk size");
    FMOE_REQUIRE(chunk_sizes_host[e] == 0 || D == 0 || expert_rows_host[e] != nullptr, FMOE_ERR_ARG,
                 "fmoe_combine_host: expert %lld has rows but a null pointer", (long long)e);
    total_rows += chunk_sizes_host[e];
  }
  FMOE_REQUIRE(total_rows == N, FMOE_ERR_ARG,
               "fmoe_combine_host: chunk sizes sum to %lld but N is %lld", (long long)total_rows,
               (long long)N);
  FMOE_REQUIRE(arena != nullptr && aligned_to(arena, 256), FMOE_ERR_WORKSPACE,
               "fmoe_combine_host: arena null or not 256-byte aligned");
  std::vector<size_t> row_off;
  row_off.reserve(E);
  const ArenaView av = arena_view(chunk_sizes_host, E, N, T, D, dtype, idx_type, w_dtype, &row_off);
  FMOE_REQUIRE(arena_bytes >= av.total, FMOE_ERR_WORKSPACE,
               "fmoe_combine_host: arena has %zu bytes, needs %zu", arena_bytes, av.total);
  if (T == 0 || D == 0) return FMOE_OK;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(arena);
  const size_t eb = dtype_size(dtype);

  std::vector<int64_t> ptrs(E), offs(E);
  std::vector<int32_t> sizes(E);
  int64_t run = 0;
  for (int64_t e = 0; e < E; ++e) {
    ptrs[e] = reinterpret_cast<int64_t>(base + row_off[e]);
    sizes[e] = static_cast<int32_t>(chunk_sizes_host[e]);
    offs[e] = run;
    run += chunk_sizes_host[e];
  }
  if (E > 0) {
    FMOE_CUDA(cudaMemcpyAsync(base + av.ptr_table, ptrs.data(), sizeof(int64_t) * E,
                              cudaMemcpyHostToDevice, s));
    FMOE_CUDA(cudaMemcpyAsync(base + av.chunk_sizes, sizes.data(), sizeof(int32_t) * E,
                              cudaMemcpyHostToDevice, s));
    FMOE_CUDA(cudaMemcpyAsync(base + av.offsets, offs.data(), sizeof(int64_t) * E,
                              cudaMemcpyHostToDevice, s));
  }
  if (N > 0) {
    FMOE_CUDA(cudaMemcpyAsync(base + av.idx, idx_host, (idx_type == FMOE_I64 ? 8 : 4) * N,
                              cudaMemcpyHostToDevice, s));
    FMOE_CUDA(cudaMemcpyAsync(base + av.w, w_host, dtype_size(w_dtype) * N, cudaMemcpyHostToDevice, s));
  }
  FMOE_CUDA(cudaMemsetAsync(base + av.status, 0, sizeof(int32_t), s));
  const int64_t cols = slice_cols(D, eb);
  if (cols < D) {
    // Pipelined form (opt-in, fmoe_tune "host_chunks"). The plan needs only the index, the weights and the tables, so it is
    // built first; the rows then arrive one slice of columns at a time (strided copies on the
    // caller's stream), and as soon as a slice is complete the helper stream gathers those
    // columns and sends them back while the next slice is still on its way in: the copy back
    // travels against the traffic instead of after it.
    int rc = fmoe_combine_plan(reinterpret_cast<const int64_t*>(base + av.ptr_table),
                               reinterpret_cast<const int32_t*>(base + av.chunk_sizes),
                               reinterpret_cast<const int64_t*>(base + av.offsets), base + av.idx,
                               idx_type, base + av.w, w_dtype, E, N, T, D, dtype, base + av.plan,
                               av.total - av.plan, reinterpret_cast<int32_t*>(base + av.status), s);
    if (rc != 0) return rc;
    cudaStream_t side = nullptr;
    FMOE_CUDA(side_stream(&side));
    EventSet events;
    DrainOnExit drain{s, side};
    const size_t pitch = static_cast<size_t>(D) * eb;
    for (int64_t c0 = 0; c0 < D; c0 += cols) {
      const int64_t width = (D - c0 < cols ? D - c0 : cols);
      for (int64_t e = 0; e < E; ++e) {
        if (chunk_sizes_host[e] > 0)
          FMOE_CUDA(cudaMemcpy2DAsync(base + row_off[e] + c0 * eb, pitch,
                                      static_cast<const char*>(expert_rows_host[e]) + c0 * eb, pitch,
                                      width * eb, static_cast<size_t>(chunk_sizes_host[e]),
                                      cudaMemcpyHostToDevice, s));
      }
      cudaEvent_t arrived;
      FMOE_CUDA(events.add(&arrived));
      FMOE_CUDA(cudaEventRecord(arrived, s));
      FMOE_CUDA(cudaStreamWaitEvent(side, arrived, 0));
      rc = combine_gather_window(base + av.plan, base + av.out + c0 * eb, D, N, T, c0, width, dtype, side);
      if (rc != 0) return rc;
      FMOE_CUDA(cudaMemcpy2DAsync(static_cast<char*>(out_host) + c0 * eb, pitch, base + av.out + c0 * eb,
                                  pitch, width * eb, static_cast<size_t>(T), cudaMemcpyDeviceToHost, side));
    }
    cudaEvent_t returned;
    FMOE_CUDA(events.add(&returned));
    FMOE_CUDA(cudaEventRecord(returned, side));
    FMOE_CUDA(cudaStreamWaitEvent(s, returned, 0));
    int32_t status_host = 0;
    FMOE_CUDA(cudaMemcpyAsync(&status_host, base + av.status, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    FMOE_CUDA(cudaStreamSynchronize(s));
    drain.armed = false;  // s has waited for the helper stream: both are idle
    FMOE_REQUIRE((status_host & FMOE_STATUS_BAD_INDEX) == 0, FMOE_ERR_ARG,
                 "fmoe_combine_host: an index lies outside [0, T); that row was skipped");
    return FMOE_OK;
  }
  for (int64_t e = 0; e < E; ++e) {
    const size_t bytes = static_cast<size_t>(chunk_sizes_host[e]) * D * eb;
    if (bytes > 0)
      FMOE_CUDA(cudaMemcpyAsync(base + row_off[e], expert_rows_host[e], bytes,
                                cudaMemcpyHostToDevice, s));
  }
  int rc = fmoe_combine_plan(reinterpret_cast<const int64_t*>(base + av.ptr_table),
                             reinterpret_cast<const int32_t*>(base + av.chunk_sizes),
                             reinterpret_cast<const int64_t*>(base + av.offsets), base + av.idx,
                             idx_type, base + av.w, w_dtype, E, N, T, D, dtype, base + av.plan,
                             av.total - av.plan, reinterpret_cast<int32_t*>(base + av.status), s);
  if (rc != 0) return rc;
  rc = fmoe_combine_gather(base + av.plan, base + av.out, D, N, T, D, dtype, /*accumulate=*/0, s);
  if (rc != 0) return rc;
  int32_t status_host = 0;
  FMOE_CUDA(cudaMemcpyAsync(out_host, base + av.out, static_cast<size_t>(T) * D * eb,
                            cudaMemcpyDeviceToHost, s));
  FMOE_CUDA(cudaMemcpyAsync(&status_host, base + av.status, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  FMOE_CUDA(cudaStreamSynchronize(s));
  FMOE_REQUIRE((status_host & FMOE_STATUS_BAD_INDEX) == 0, FMOE_ERR_ARG,
               "fmoe_combine_host: an index lies outside [0, T); that row was skipped");
  return FMOE_OK;
}
