// Shared device/host helpers for the fastmoe_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include <nvtx3/nvToolsExt.h>

#include "../../include/fastmoe_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "fastmoe_b200 kernels are written for sm_100a (B200) only"
#endif

namespace fmoe {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of it

// ---- host-side error plumbing ---------------------------------------------
void set_error(const char* fmt, ...);  // stores a thread-local message
int fail(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);

#define FMOE_REQUIRE(cond, code, ...)                   \
  do {                                                  \
    if (!(cond)) return ::fmoe::fail((code), __VA_ARGS__); \
  } while (0)

#define FMOE_CUDA(expr)                                            \
  do {                                                             \
    int _rc = ::fmoe::check_cuda((expr), #expr);                   \
    if (_rc != 0) return _rc;                                      \
  } while (0)

inline int check_launch(const char* kernel) { return check_cuda(cudaGetLastError(), kernel); }

// NVTX range around the host side of an entry point (header-only NVTX 3: a no-op unless a
// profiler has injected its library): timelines show which call enqueued which kernels, as
// the reference marks its pipeline stages (src/fastmoe/models/tiny_model.py:527-622).
struct ScopedRange {
  explicit ScopedRange(const char* name) { nvtxRangePushA(name); }
  ~ScopedRange() { nvtxRangePop(); }
  ScopedRange(const ScopedRange&) = delete;
  ScopedRange& operator=(const ScopedRange&) = delete;
};
#define FMOE_RANGE(name) ::fmoe::ScopedRange fmoe_range_(name)

inline bool valid_dtype(int dt) { return dt == FMOE_F32 || dt == FMOE_BF16 || dt == FMOE_F16; }
inline bool valid_itype(int it) { return it == FMOE_I64 || it == FMOE_I32; }
inline int dtype_size(int dt) { return dt == FMOE_F32 ? 4 : 2; }
inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Dispatch a runtime dtype tag to a compile-time one.
#define FMOE_DISPATCH_DTYPE(dt, DT, ...)                      \
  switch (dt) {                                               \
    case FMOE_F32: {                                          \
      constexpr int DT = FMOE_F32;                            \
      __VA_ARGS__;                                            \
    } break;                                                  \
    case FMOE_BF16: {                                         \
      constexpr int DT = FMOE_BF16;                           \
      __VA_ARGS__;                                            \
    } break;                                                  \
    default: {                                                \
      constexpr int DT = FMOE_F16;                            \
      __VA_ARGS__;                                            \
    } break;                                                  \
  }

// ---- element traits ----------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<FMOE_F32> {
  using type = float;
  static constexpr int kBytes = 4;
  static constexpr int kVec = 4;  // elements per 16-byte vector
};
template <>
struct Elem<FMOE_BF16> {
  using type = __nv_bfloat16;
  static constexpr int kBytes = 2;
  static constexpr int kVec = 8;
};
template <>
struct Elem<FMOE_F16> {
  using type = __half;
  static constexpr int kBytes = 2;
  static constexpr int kVec = 8;
};

#ifdef __CUDACC__

// Scalar element <-> fp32.
template <int DT>
__device__ __forceinline__ float to_float(typename Elem<DT>::type v);
template <>
__device__ __forceinline__ float to_float<FMOE_F32>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<FMOE_BF16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<FMOE_F16>(__half v) { return __half2float(v); }

template <int DT>
__device__ __forceinline__ typename Elem<DT>::type from_float(float v);
template <>
__device__ __forceinline__ float from_float<FMOE_F32>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<FMOE_BF16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<FMOE_F16>(float v) { return __float2half_rn(v); }

// Load a gate weight / scalar of runtime dtype as fp32.
__device__ __forceinline__ float load_scalar_as_float(const void* p, int64_t i, int dt) {
  if (dt == FMOE_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == FMOE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_scalar_from_float(void* p, int64_t i, int dt, float v) {
  if (dt == FMOE_F32)
    reinterpret_cast<float*>(p)[i] = v;
  else if (dt == FMOE_BF16)
    reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}
__device__ __forceinline__ int64_t load_index(const void* p, int64_t i, int it) {
  return it == FMOE_I64 ? reinterpret_cast<const int64_t*>(p)[i]
                        : static_cast<int64_t>(reinterpret_cast<const int32_t*>(p)[i]);
}

// 16-byte vector <-> kVec floats.
template <int DT>
__device__ __forceinline__ void unpack16(const uint4& v, float* f);
template <>
__device__ __forceinline__ void unpack16<FMOE_F32>(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x);
  f[1] = __uint_as_float(v.y);
  f[2] = __uint_as_float(v.z);
  f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack16<FMOE_BF16>(const uint4& v, float* f) {
  // bf16 -> fp32 is a 16-bit shift: no conversion instruction needed
  f[0] = __uint_as_float(v.x << 16);
  f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16);
  f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16);
  f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16);
  f[7] = __uint_as_float(v.w & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack16<FMOE_F16>(const uint4& v, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <int DT>
__device__ __forceinline__ uint4 pack16(const float* f);
template <>
__device__ __forceinline__ uint4 pack16<FMOE_F32>(const float* f) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                    __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack16<FMOE_BF16>(const float* f) {
  uint4 r;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(f[0], f[1]);
  r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(f[2], f[3]);
  r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(f[4], f[5]);
  r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(f[6], f[7]);
  r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}
template <>
__device__ __forceinline__ uint4 pack16<FMOE_F16>(const float* f) {
  uint4 r;
  __half2 t;
  t = __floats2half2_rn(f[0], f[1]);
  r.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(f[2], f[3]);
  r.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(f[4], f[5]);
  r.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2half2_rn(f[6], f[7]);
  r.w = *reinterpret_cast<uint32_t*>(&t);
  return r;
}

// Streaming 16-byte global accesses: rows are read once and written once, so
// loads bypass L1 allocation and stores use the streaming (evict-first) policy.
__device__ __forceinline__ uint4 ld_stream16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// Rows that several warps of one CTA read at about the same time: let L1 keep them.
__device__ __forceinline__ uint4 ld_cached16(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(uint4* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Vector reductions to global memory (sm_90+): one 16-byte `red` per vector.
template <int DT>
__device__ __forceinline__ void red_add16(void* p, const float* f);
template <>
__device__ __forceinline__ void red_add16<FMOE_F32>(void* p, const float* f) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(f[0]), "f"(f[1]),
               "f"(f[2]), "f"(f[3])
               : "memory");
}
template <>
__device__ __forceinline__ void red_add16<FMOE_BF16>(void* p, const float* f) {
  uint4 v = pack16<FMOE_BF16>(f);
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
template <>
__device__ __forceinline__ void red_add16<FMOE_F16>(void* p, const float* f) {
  uint4 v = pack16<FMOE_F16>(f);
  asm volatile("red.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// Scalar reduction for the unaligned / odd-width fallback.
template <int DT>
__device__ __forceinline__ void red_add1(typename Elem<DT>::type* p, float v);
template <>
__device__ __forceinline__ void red_add1<FMOE_F32>(float* p, float v) { atomicAdd(p, v); }
template <>
__device__ __forceinline__ void red_add1<FMOE_BF16>(__nv_bfloat16* p, float v) {
  atomicAdd(p, __float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ void red_add1<FMOE_F16>(__half* p, float v) {
  atomicAdd(p, __float2half_rn(v));
}

// Index of the expert that owns global row g: the last e with offsets[e] <= g.
// Empty experts share an offset with their successor, so the last one wins and
// the caller still checks the local row against chunk_sizes.
__device__ __forceinline__ int find_expert(const int64_t* __restrict__ offsets, int E, int64_t g) {
  int lo = 0, hi = E;  // invariant: offsets[lo] <= g, answer in [lo, hi)
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (offsets[mid] <= g)
      lo = mid;
    else
      hi = mid;
  }
  return lo;
}

#endif  // __CUDACC__

}  // namespace fmoe
