// Layout of the combine plan (the inverse of the index vector) in caller scratch.
#pragma once
#include "common.cuh"

namespace fmoe {

// Sections, each starting on a 256-byte boundary, in this order:
//   seg_off     int32[T+1]  rows targeting output row t are slots [seg_off[t], seg_off[t+1])
//   cnt         int32[T]    histogram of targets (build-time only)
//   rank        int32[N]    arrival rank of row g among rows with its target (build-time only)
//   seg_rows    int32[N]    global rows by slot in arrival order (build-time only)
//   row_of_slot int32[N]    global row g of each slot, ascending inside a segment
//   src_sorted  int64[N]    address of the source row of each slot (0 = skip)
//   w_sorted    float[N]    gate weight of each slot as fp32
struct PlanView {
  int32_t* seg_off;
  int32_t* cnt;
  int32_t* rank;
  int32_t* seg_rows;
  int32_t* row_of_slot;
  int64_t* src_sorted;
  float* w_sorted;
  size_t bytes;
};

inline PlanView plan_view(void* base, int64_t N, int64_t T) {
  PlanView p;
  char* c = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* r = c + off;
    off += round_up(bytes, 256);
    return r;
  };
  p.seg_off = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * (T + 1)));
  p.cnt = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * (T > 0 ? T : 1)));
  p.rank = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * (N > 0 ? N : 1)));
  p.seg_rows = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * (N > 0 ? N : 1)));
  p.row_of_slot = reinterpret_cast<int32_t*>(take(sizeof(int32_t) * (N > 0 ? N : 1)));
  p.src_sorted = reinterpret_cast<int64_t*>(take(sizeof(int64_t) * (N > 0 ? N : 1)));
  p.w_sorted = reinterpret_cast<float*>(take(sizeof(float) * (N > 0 ? N : 1)));
  p.bytes = off;
  return p;
}

// Segments longer than this keep their arrival order (still correct, but the
// fp32 summation order then varies from run to run).
constexpr int kPlanStableCap = 1024;

// token_major.cu: the gather over a window of columns (see the definition)
int combine_gather_window(const void* plan, void* out, int64_t out_row_stride, int64_t N, int64_t T,
                          int64_t col0, int64_t cols, int dtype, cudaStream_t s);

}  // namespace fmoe
