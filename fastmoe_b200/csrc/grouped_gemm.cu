// Grouped GEMM for the expert FFN on the 5th-generation tensor cores (tcgen05):
//   C[rows of expert e, :] = A[rows of expert e, :] x W_e^T        (plain)
//   C[rows of expert e, :] = silu(A W_gate_e^T) * (A W_up_e^T)     (SwiGLU, fused epilogue)
// A is [R, K] bf16 with each expert's rows contiguous (offsets/counts on the device, as
// the index builder leaves them), W is [E, N, K] bf16 in nn.Linear layout. Replaces the
// Python loop of per-expert cuBLAS GEMMs in MoEFeedForward.compute_experts of
// polkadot21/fastmoe (src/fastmoe/models/tiny_model.py:282-294): one persistent launch,
// ragged M per expert resolved on the device, no host knowledge of the counts.
//
// Structure per CTA (192 threads, one CTA per SM):
//   warp 0      TMA producer: A tile 128x64 and W tile 256x64 (two 128-row boxes) per stage,
//               128-byte swizzle, 4 stages, mbarrier full/empty pairs
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=256, K=16, bf16 -> fp32)
//               into one of two 256-column TMEM accumulators; tcgen05.commit frees stages
//   warps 2-5   epilogue: tcgen05.ld of the finished accumulator (row = TMEM lane),
//               activation, bf16 rounding, masked stores of the expert's valid rows; runs
//               while the next tile's MMAs fill the other accumulator
// Every mbarrier wait is bounded: on a timeout the kernel sets FMOE_STATUS_WAIT_TIMEOUT in
// the status word, every role leaves its loop, TMEM is released and the kernel returns.
#include <cuda.h>

#include "common.cuh"

namespace fmoe {

constexpr int kBM = 128, kBN = 256, kBK = 64, kStages = 4, kUmmaK = 16;
constexpr int kABytes = kBM * kBK * 2;        // 16 KB
constexpr int kBBytes = kBN * kBK * 2;        // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kGemmThreads = 192;
constexpr int kEpiStageBytes = 4 * 32 * 128;  // epilogue staging: one 32-row x 128-byte block per warp
constexpr int kMaxExperts = 1024;
constexpr uint32_t kSpinLimit = 1u << 24;  // probes per wait before giving up (about a second)

struct GemmArgs {
  const int64_t* offsets;  // [E] first row of each expert in A / C
  const int64_t* counts;   // [E] rows of each expert
  const int64_t* c_row_map;  // optional [R]: row of C that receives the result of A's row r (nullptr = r)
  const int64_t* c_row_ptrs;  // optional [R]: ADDRESS of the output row of A's row r (may be peer memory)
  __nv_bfloat16* C;
  __nv_bfloat16* pre;      // optional [R, N]: the product BEFORE the activation, by A's row (for a backward pass)
  int64_t ldc;             // row stride of C in elements
  int64_t ld_pre;          // row stride of pre in elements (N)
  int64_t R;               // rows of A
  int E;
  int n_blocks;            // column tiles per expert
  int k_blocks;            // K / 64
  int w_rows_per_expert;   // rows of the weight tensor per expert (N, or 2*ff for SwiGLU)
  int up_row_offset;       // SwiGLU: row of the first "up" weight inside an expert (= ff), else 128
  int swiglu;
  int gelu;                // plain product followed by the exact (erf) GELU, as nn.GELU() computes it
  int w_transposed;        // 1: data gradient, C = A x W (W is [E, K_red, N_out]: the reduction runs over W's rows)
  int skip_loads;  // test hook: the producer issues nothing, so every consumer wait runs out
  int prefetch;    // weight k-blocks requested into L2 ahead of the loads (0 = none)
  uint32_t spin_limit;
  int32_t* status;
};

// ---- PTX wrappers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait: false after `limit` unsuccessful probes, or once another role has given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < limit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
// The same without the give-up flag: used on the way out, when the flag may already be set.
__device__ __forceinline__ bool mbar_wait_plain(uint64_t* bar, uint32_t parity, uint32_t limit) {
  int never = 0;
  return mbar_wait(bar, parity, &never, limit);
}
// Leaving the kernel, normally or after a wait gave up: the MMA thread waits (bounded) until
// the tensor core has finished every MMA it issued, so that tensor memory is not released
// under them; after a give-up the producer thread waits (bounded) for the loads it still has
// in flight, so that none lands in shared memory after the CTA has gone.
__device__ __forceinline__ void drain_on_exit(int warp, int lane, int fills, bool mma_issued, uint64_t* full,
                                              uint64_t* drain, const volatile int* abort_flag, int stages,
                                              uint32_t limit) {
  if (warp == 0 && lane == 0 && *abort_flag) {
    for (int s = 0; s < stages && s < fills; ++s) {
      const int last = (fills - 1 - s) / stages * stages + s;  // last fill that used stage s
      mbar_wait_plain(&full[s], (last / stages) & 1, limit);
    }
  }
  if (warp == 1 && lane == 0 && mma_issued) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(drain)))
                 : "memory");
    mbar_wait_plain(drain, 0, limit);
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (the layout a 128B-swizzled TMA box produces).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fff);        // start address
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused here)
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3fff) << 32;    // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                       // 128-byte swizzle
  return d;
}
// The same for an operand whose MN dimension is the contiguous one (a row-major [K, N] weight
// used as B): 64-element (128-byte) pieces of the MN dimension are separate TMA boxes
// `mn_piece_bytes` apart, and inside a box every 8 reduction rows form a 1024-byte group.
__device__ __forceinline__ uint64_t smem_desc_mn(uint32_t saddr, uint32_t mn_piece_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((mn_piece_bytes >> 4) & 0x3fff) << 16;  // leading byte offset: next MN piece
  d |= static_cast<uint64_t>((1024 >> 4) & 0x3fff) << 32;            // stride byte offset: next 8 reduction rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M=128, N=256.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kBN >> 3) << 17) | ((kBM >> 4) << 24);
constexpr uint32_t kIdescBMn = kIdesc | (1u << 16);  // B with the N dimension contiguous

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

// Rows of expert e that lie inside A: a count that would run past the end of A (a caller
// whose receive buffer overflowed, say) is cut there, so no tile reaches beyond row R.
__device__ __forceinline__ int64_t expert_rows(const int64_t* offsets, const int64_t* counts, int64_t R, int e) {
  const int64_t off = offsets[e], n = counts[e];
  if (off < 0 || off >= R || n <= 0) return 0;
  return n < R - off ? n : R - off;
}

// Asks for a tile to be brought into L2; completes on its own, nothing waits for it.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1)
               : "memory");
}
struct TileCoord {
  int expert, mb, nb, rows;  // rows = valid rows of this M block
  int64_t row0;              // first row in A / C
};

// Tiles are numbered expert-major, then column block, then row block: the row blocks that
// share a weight tile are neighbours and run at the same time, so the weight tile comes
// from DRAM once and from L2 afterwards.
__device__ __forceinline__ TileCoord locate_tile(int tile, const int* mb_prefix, const GemmArgs& a) {
  int lo = 0, hi = a.E;  // last e with mb_prefix[e] * n_blocks <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(mb_prefix[mid]) * a.n_blocks <= tile) lo = mid; else hi = mid;
  }
  TileCoord c;
  c.expert = lo;
  const int mblocks = mb_prefix[lo + 1] - mb_prefix[lo];
  const int local = tile - mb_prefix[lo] * a.n_blocks;
  c.nb = local / mblocks;
  c.mb = local - c.nb * mblocks;
  c.row0 = a.offsets[lo] + static_cast<int64_t>(c.mb) * kBM;
  const int64_t left = expert_rows(a.offsets, a.counts, a.R, lo) - static_cast<int64_t>(c.mb) * kBM;
  c.rows = static_cast<int>(left < kBM ? left : kBM);
  return c;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
    grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                        const GemmArgs a) {  // map_w: box 64 x 256 rows (plain), 64 x 128 (SwiGLU) or 64 x 64 (w_transposed)
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern is anchored to
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_base_slot + 1);
  uint64_t* drain = reinterpret_cast<uint64_t*>(abort_flag + 1);  // see drain_on_exit
  uint4* stage = reinterpret_cast<uint4*>(smem + kStages * kStageBytes + 256);  // 4 warps x 32 rows x 128 B
  int* mb_prefix = reinterpret_cast<int*>(smem + kStages * kStageBytes + 256 + kEpiStageBytes);  // [E + 1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int fills = 0;            // producer: stage fills issued so far
  bool mma_issued = false;  // MMA thread: at least one MMA is (or was) in flight

  // ---- set-up: tile table, barriers, TMEM ----------------------------------------------
  for (int e = threadIdx.x; e < a.E; e += kGemmThreads) {
    const int64_t n = expert_rows(a.offsets, a.counts, a.R, e);
    if (n != a.counts[e] && a.counts[e] > 0 && a.status != nullptr && blockIdx.x == 0)
      atomicOr(a.status, FMOE_STATUS_BAD_EXPERT);  // rows past the end of A were cut off
    mb_prefix[e + 1] = static_cast<int>((n + kBM - 1) / kBM);
  }
  if (threadIdx.x == 0) {
    mb_prefix[0] = 0;
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    mbar_init(drain, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {  // inclusive scan of the per-expert block counts, 32 at a time
    int carry = 0;
    for (int base = 0; base < a.E; base += 32) {
      const int e = base + lane;
      int v = e < a.E ? mb_prefix[e + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
      }
      if (e < a.E) mb_prefix[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  if (warp == 1) {  // the MMA warp owns the tensor memory: all 512 columns, two accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_base_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = mb_prefix[a.E] * a.n_blocks;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ---------------------------------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    // Optional (fmoe_tune "gemm_prefetch", off by default): ask for the weight k-blocks
    // `a.prefetch` steps ahead (across the boundary to this CTA's next tile) to be brought
    // into L2, so that the loads themselves find them there.
    auto prefetch_w = [&](int expert, int nb, int kb) {
      if (a.w_transposed) {
        const int red_row = expert * a.w_rows_per_expert + kb * kBK;
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) tma_prefetch_2d(&map_w, nb * kBN + piece * 64, red_row);
      } else {
        const int r0 = expert * a.w_rows_per_expert + nb * (a.swiglu ? 128 : kBN);
        tma_prefetch_2d(&map_w, kb * kBK, r0);
        if (a.swiglu) tma_prefetch_2d(&map_w, kb * kBK, r0 + a.up_row_offset);
      }
    };
    const int ahead = a.prefetch < a.k_blocks ? a.prefetch : a.k_blocks;
    bool first_tile = true;
    for (int tile = blockIdx.x; tile < total_tiles && !a.skip_loads; tile += gridDim.x) {
      const TileCoord c = locate_tile(tile, mb_prefix, a);
      const int w_row0 = c.expert * a.w_rows_per_expert + c.nb * (a.swiglu ? 128 : kBN);
      const int w_row1 = w_row0 + a.up_row_offset;
      int next_expert = -1, next_nb = 0;
      if (ahead > 0) {
        if (first_tile)
          for (int kb = 0; kb < ahead; ++kb) prefetch_w(c.expert, c.nb, kb);
        first_tile = false;
        if (tile + static_cast<int>(gridDim.x) < total_tiles) {
          const TileCoord n = locate_tile(tile + gridDim.x, mb_prefix, a);
          next_expert = n.expert;
          next_nb = n.nb;
        }
      }
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        if (ahead > 0) {
          const int pk = kb + ahead;
          if (pk < a.k_blocks) prefetch_w(c.expert, c.nb, pk);
          else if (next_expert >= 0) prefetch_w(next_expert, next_nb, pk - a.k_blocks);
        }
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, a.spin_limit)) goto timed_out;
        mbar_expect_tx(&full[stage], kStageBytes);
        tma_load_2d(smem_a + stage * kABytes, &map_a, kb * kBK, static_cast<int>(c.row0), &full[stage]);
        if (a.w_transposed) {
          // W[e] is [K_red, N_out] row-major: four boxes of 64 output columns x 64 reduction rows
          const int red_row = c.expert * a.w_rows_per_expert + kb * kBK;
#pragma unroll
          for (int piece = 0; piece < 4; ++piece)
            tma_load_2d(smem_b + stage * kBBytes + piece * (kBBytes / 4), &map_w, c.nb * kBN + piece * 64, red_row,
                        &full[stage]);
        } else if (a.swiglu) {
          tma_load_2d(smem_b + stage * kBBytes, &map_w, kb * kBK, w_row0, &full[stage]);
          tma_load_2d(smem_b + stage * kBBytes + kBBytes / 2, &map_w, kb * kBK, w_row1, &full[stage]);
        } else {  // 256 consecutive weight rows: one box (the TMA unit's cost is per box as well as per byte)
          tma_load_2d(smem_b + stage * kBBytes, &map_w, kb * kBK, w_row0, &full[stage]);
        }
        ++fills;
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer -----------------------------------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, a.spin_limit)) goto timed_out;
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + acc * kBN;
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, a.spin_limit)) goto timed_out;
        tcgen05_fence_after();
        mma_issued = true;
        const uint64_t da = smem_desc(smem_u32(smem_a + stage * kABytes));
        if (a.w_transposed) {
          const uint64_t db = smem_desc_mn(smem_u32(smem_b + stage * kBBytes), kBBytes / 4);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // A: +32 bytes along K; B: 16 reduction rows of 128 bytes further = +2048 bytes
            umma_bf16(tmem_d, da + 2 * k, db + 128 * k, kIdescBMn, (kb | k) != 0 ? 1u : 0u);
          }
        } else {
          const uint64_t db = smem_desc(smem_u32(smem_b + stage * kBBytes));
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // 16 bf16 = 32 bytes along K inside the swizzle atom: +2 in the encoded address
            umma_bf16(tmem_d, da + 2 * k, db + 2 * k, kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&empty[stage]);  // frees the stage when these MMAs have read it
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      umma_commit(&tmem_full[acc]);  // accumulator complete
    }
  } else if (warp >= 2) {
    // ---- epilogue -------------------------------------------------------------------
    const int quarter = warp & 3;  // the TMEM lanes this warp may read: 32*quarter .. +31
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const TileCoord c = locate_tile(tile, mb_prefix, a);
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, a.spin_limit)) goto timed_out;
      tcgen05_fence_after();
      const int row = quarter * 32 + lane;
      const bool valid = row < c.rows && c.row0 + row < a.R;  // never past A's rows, whatever the counts say
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
      // Address of this lane's output row (0 = no row): the same row as in A, the row the map
      // names, or wherever the address table points (possibly another GPU's memory).
      const int out_cols = a.swiglu ? 128 : kBN;
      char* my_row = nullptr;
      if (valid) {
        const int64_t a_row = c.row0 + row;
        if (a.c_row_ptrs != nullptr) my_row = reinterpret_cast<char*>(a.c_row_ptrs[a_row]);
        if (my_row == nullptr) {
          const int64_t out_row = (a.c_row_ptrs == nullptr && a.c_row_map != nullptr) ? a.c_row_map[a_row] : a_row;
          if (a.C != nullptr) my_row = reinterpret_cast<char*>(a.C + out_row * a.ldc);
        }
        if (my_row != nullptr) my_row += static_cast<int64_t>(c.nb) * out_cols * 2;
      }
      // The accumulator arrives one row per lane. Rows are regrouped through a small
      // swizzled staging buffer so that every store instruction writes four complete
      // 128-byte row segments: full lines for HBM, full packets for NVLink peers.
      uint4* stage_w = stage + (warp - 2) * (32 * 8);
      // a training forward keeps the product before the activation: this lane's row of `pre`
#ifdef FMOE_NO_KEEP_PRE  // build switch for A/B measurements of the epilogue without this path
      __nv_bfloat16* pre_row = nullptr;
#else
      __nv_bfloat16* pre_row = (valid && a.pre != nullptr) ? a.pre + (c.row0 + row) * a.ld_pre : nullptr;
#endif
      auto keep = [&](const uint32_t* v, int64_t col) {  // 32 consecutive columns of one row, 64 bytes
        float t[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) t[i] = __uint_as_float(v[i]);
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(pre_row + col + 8 * q) = pack16<FMOE_BF16>(t + 8 * q);
      };
#pragma unroll 1
      for (int c0 = 0; c0 < out_cols; c0 += 64) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float f[32];
          if (a.swiglu) {
            uint32_t g[32], u[32];
            tmem_ld32(taddr + c0 + 32 * h, g);
            tmem_ld32(taddr + 128 + c0 + 32 * h, u);
            tmem_ld_wait();
            if (pre_row != nullptr) {  // gate columns first, up columns behind them, as the weights lie
              const int64_t col = static_cast<int64_t>(c.nb) * 128 + c0 + 32 * h;
              keep(g, col);
              keep(u, a.up_row_offset + col);
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = silu(__uint_as_float(g[i])) * __uint_as_float(u[i]);
          } else {
            uint32_t r[32];
            tmem_ld32(taddr + c0 + 32 * h, r);
            tmem_ld_wait();
            if (pre_row != nullptr) keep(r, static_cast<int64_t>(c.nb) * kBN + c0 + 32 * h);
            if (a.gelu) {
#pragma unroll
              for (int i = 0; i < 32; ++i) f[i] = gelu_erf(__uint_as_float(r[i]));
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
            }
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int q = 4 * h + v;  // 16-byte piece of this row's 128-byte segment
            stage_w[lane * 8 + (q ^ (lane & 7))] = pack16<FMOE_BF16>(f + 8 * v);
          }
        }
        __syncwarp();
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          const int r = step * 4 + (lane >> 3);
          const int q = lane & 7;
          const unsigned long long rp =
              __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_row), r);
          if (rp != 0) {
            const uint4 val = stage_w[r * 8 + (q ^ (r & 7))];
            *reinterpret_cast<uint4*>(reinterpret_cast<char*>(rp) + c0 * 2 + q * 16) = val;
          }
        }
        __syncwarp();
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);  // this warp is done with the accumulator
    }
  }
  goto done;

timed_out:
  *abort_flag = 1;
  if (a.status != nullptr) atomicOr(a.status, FMOE_STATUS_WAIT_TIMEOUT);

done:
  drain_on_exit(warp, lane, fills, mma_issued, full, drain, abort_flag, kStages, a.spin_limit);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---- weight gradient ------------------------------------------------------------------------
// grad_w[e][n, k] = sum over the rows m of expert e of grad_c[m, n] * a[m, k].
// The reduction runs over the ROWS of both operands, so both are used with their
// contiguous dimension as the MN dimension: 64-wide TMA boxes of 64 rows each (two for the
// 128 n of a tile, four for its 256 k). An expert's last 64-row chunk may reach into the
// next expert's rows: the MMA warp zeroes those rows of the grad_c tile in shared memory
// before the MMAs read it (rows past the end of the tensor are zero-filled by TMA). Tiles
// are (expert, n block, k block) with a fixed count per expert, so no tile table is needed;
// an expert without rows gets zeros straight from the epilogue.
struct WgradArgs {
  const int64_t* offsets;
  const int64_t* counts;
  __nv_bfloat16* grad_w;  // [E, N, K]
  int64_t N, K, R;
  int E, n_blocks, k_blocks;  // tiles per expert: N/128 x K/256
  int skip_loads;
  uint32_t spin_limit;
  int32_t* status;
};

constexpr uint32_t kIdescAllMn = kIdesc | (1u << 15) | (1u << 16);  // A and B with MN contiguous

__global__ void __launch_bounds__(kGemmThreads, 1)
    grouped_wgrad_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_a,
                         const WgradArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;                       // grad_c tile: 2 boxes x 8 KB per stage
  uint8_t* smem_b = smem + kStages * kABytes;   // a tile: 4 boxes x 8 KB per stage
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_base_slot + 1);
  uint64_t* drain = reinterpret_cast<uint64_t*>(abort_flag + 1);
  uint4* stage_buf = reinterpret_cast<uint4*>(smem + kStages * kStageBytes + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int fills = 0;
  bool mma_issued = false;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(drain, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_base_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int tiles_per_expert = a.n_blocks * a.k_blocks;
  const int total_tiles = a.E * tiles_per_expert;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ---------------------------------------------------------------
    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !a.skip_loads; tile += gridDim.x) {
      const int e = tile / tiles_per_expert;
      const int local = tile - e * tiles_per_expert;
      const int nb = local / a.k_blocks, kbk = local - nb * a.k_blocks;
      const int64_t row0 = a.offsets[e];
      const int chunks = static_cast<int>((expert_rows(a.offsets, a.counts, a.R, e) + kBK - 1) / kBK);
      for (int kb = 0; kb < chunks; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, a.spin_limit)) goto timed_out;
        mbar_expect_tx(&full[stage], kStageBytes);
        const int row = static_cast<int>(row0) + kb * kBK;
#pragma unroll
        for (int piece = 0; piece < 2; ++piece)
          tma_load_2d(smem_a + stage * kABytes + piece * (kABytes / 2), &map_g, nb * kBM + piece * 64, row,
                      &full[stage]);
#pragma unroll
        for (int piece = 0; piece < 4; ++piece)
          tma_load_2d(smem_b + stage * kBBytes + piece * (kBBytes / 4), &map_a, kbk * kBN + piece * 64, row,
                      &full[stage]);
        ++fills;
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---- MMA warp: all lanes mask a ragged chunk, lane 0 issues the MMAs ----------------
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int e = tile / tiles_per_expert;
      const int64_t rows = expert_rows(a.offsets, a.counts, a.R, e);
      const int chunks = static_cast<int>((rows + kBK - 1) / kBK);
      if (chunks == 0) continue;  // the epilogue writes zeros for this tile on its own
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, a.spin_limit)) goto timed_out;
      tcgen05_fence_after();
      const uint32_t tmem_d = tmem_base + acc * kBN;
      for (int kb = 0; kb < chunks; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, a.spin_limit)) goto timed_out;
        const int valid = static_cast<int>(rows - static_cast<int64_t>(kb) * kBK);
        if (valid < kBK) {
          // rows valid..63 of this chunk belong to the next expert (or to nobody: the unused
          // tail of a capacity-sized buffer, whose bytes may read as NaN or Inf): clear them in
          // BOTH tiles, since 0 x NaN is NaN (each reduction row is one 128-byte line in each
          // of the two grad_c boxes and the four boxes of the other operand)
          uint4* tile_g = reinterpret_cast<uint4*>(smem_a + stage * kABytes);
          const int lines = (kBK - valid) * 2;
          for (int i = lane; i < lines * 8; i += 32) {
            const int line = i >> 3, piece = line & 1, r = valid + (line >> 1);
            tile_g[piece * (kABytes / 2 / 16) + r * 8 + (i & 7)] = make_uint4(0, 0, 0, 0);
          }
          uint4* tile_a = reinterpret_cast<uint4*>(smem_b + stage * kBBytes);
          const int lines_a = (kBK - valid) * 4;
          for (int i = lane; i < lines_a * 8; i += 32) {
            const int line = i >> 3, piece = line & 3, r = valid + (line >> 2);
            tile_a[piece * (kBBytes / 4 / 16) + r * 8 + (i & 7)] = make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor core reads
        }
        __syncwarp();
        tcgen05_fence_after();
        if (lane == 0) {
          mma_issued = true;
          const uint64_t da = smem_desc_mn(smem_u32(smem_a + stage * kABytes), kABytes / 2);
          const uint64_t db = smem_desc_mn(smem_u32(smem_b + stage * kBBytes), kBBytes / 4);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_bf16(tmem_d, da + 128 * k, db + 128 * k, kIdescAllMn, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (kb == chunks - 1) umma_commit(&tmem_full[acc]);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp >= 2) {
    // ---- epilogue -------------------------------------------------------------------
    const int quarter = warp & 3;
    uint4* stage_w = stage_buf + (warp - 2) * (32 * 8);
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int e = tile / tiles_per_expert;
      const int local = tile - e * tiles_per_expert;
      const int nb = local / a.k_blocks, kbk = local - nb * a.k_blocks;
      const bool empty_expert = expert_rows(a.offsets, a.counts, a.R, e) <= 0;
      const int row = quarter * 32 + lane;
      char* my_row = reinterpret_cast<char*>(a.grad_w + (static_cast<int64_t>(e) * a.N + nb * kBM + row) * a.K +
                                             static_cast<int64_t>(kbk) * kBN);
      int acc = 0;
      if (!empty_expert) {
        acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, a.spin_limit)) goto timed_out;
        tcgen05_fence_after();
      }
      const uint32_t taddr = tmem_base + acc * kBN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 64) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float f[32];
          if (empty_expert) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = 0.f;
          } else {
            uint32_t r[32];
            tmem_ld32(taddr + c0 + 32 * h, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) stage_w[lane * 8 + ((4 * h + v) ^ (lane & 7))] = pack16<FMOE_BF16>(f + 8 * v);
        }
        __syncwarp();
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          const int r = step * 4 + (lane >> 3);
          const int q = lane & 7;
          const unsigned long long rp = __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_row), r);
          *reinterpret_cast<uint4*>(reinterpret_cast<char*>(rp) + c0 * 2 + q * 16) = stage_w[r * 8 + (q ^ (r & 7))];
        }
        __syncwarp();
      }
      if (!empty_expert) {
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      }
    }
  }
  goto done;

timed_out:
  *abort_flag = 1;
  if (a.status != nullptr) atomicOr(a.status, FMOE_STATUS_WAIT_TIMEOUT);

done:
  drain_on_exit(warp, lane, fills, mma_issued, full, drain, abort_flag, kStages, a.spin_limit);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---- tokens as the MMA's N dimension, two weight tiles per token tile --------------------------
// The same product with the operands' roles exchanged and a larger tile. WEIGHT rows are the
// MMA's M dimension (the lanes of tensor memory) and an expert's TOKEN rows are its N dimension,
// which comes in steps of 16 instead of blocks of 128: an expert with n <= 256 rows is ONE tile
// of round16(n) tokens, a larger one is cut into ceil(n / 256) tiles of equal size (never a full
// tile plus a sliver, which would pull whole weight tiles through the SM for a fraction of the
// work). With a few hundred rows per expert this issues 3% more MMA work than the rows need,
// where 128-row blocks issue 25% more.
//
// A tile pairs its tokens with TWO weight tiles of 128 rows, each MMA'd into its own 256-column
// accumulator (all 512 columns of tensor memory): 64 KB of operands per k-block feed two
// 128 x n x 64 products, where the kernel above moves 48 KB for one. Both kernels are bound by
// what the TMA unit can bring into an SM, not by the tensor pipe (measured: time per k-block
// grows with bytes and with the number of boxes, about 67 bytes per clock plus 50 clocks per
// box), so operand bytes per MMA are what counts. The price is that the accumulators are not
// double-buffered: a tile's epilogue and the next tile's first MMA do not overlap; the loads
// do run ahead through the three pipeline stages meanwhile.
//   plain / GELU   the two weight tiles are 256 consecutive output columns
//   SwiGLU         128 gate rows and the 128 up rows of the same columns: a column's two
//                  factors sit in the same lane of the two accumulators
// The accumulator arrives transposed (lane = output column, column = token), so the epilogue
// turns 32-token chunks around through shared memory and stores whole 256-byte row segments.
// Tokens are loaded in 64-row boxes (up to four per stage, each issued by its own lane of warp
// 0; rows past the tile's end ride along unused).
struct TnArgs {
  const int64_t* offsets;
  const int64_t* counts;
  const int64_t* c_row_map;
  const int64_t* c_row_ptrs;
  __nv_bfloat16* C;
  int64_t ldc, R;
  int E;
  int m_blocks;           // weight tile pairs per expert: N / 256, or ff / 128 for SwiGLU
  int k_blocks;           // K / 64
  int w_rows_per_expert;  // N (2 * ff for SwiGLU)
  int ff;                 // SwiGLU: row of the first "up" weight inside an expert
  int swiglu, gelu;
  int skip_loads;
  uint32_t spin_limit;
  int32_t* status;
};

constexpr int kTnTokens = 256;                       // most tokens in one tile
constexpr int kTnBox = 16;                           // step of a tile's token count (the MMA's N)
constexpr int kTnLoadRows = 64;                      // token rows per TMA box
constexpr int kTnLoadBytes = kTnLoadRows * kBK * 2;  // 8 KB
constexpr int kTnWBytes = 2 * 128 * kBK * 2;         // 32 KB: two weight tiles per stage
constexpr int kTnTBytes = kTnTokens * kBK * 2;       // up to 32 KB of tokens per stage
constexpr int kTnStages = 3;
static_assert(kTnStages * (kTnWBytes + kTnTBytes) == kStages * kStageBytes, "same pipeline memory as grouped_gemm_kernel");

struct TnTile {
  int expert, mb, rows, n;  // rows = valid tokens, n = rows rounded up to 16 (the MMA's N)
  int64_t row0;             // first token row in A / C
};

__device__ __forceinline__ int tn_splits(int64_t n) { return static_cast<int>((n + kTnTokens - 1) / kTnTokens); }

__device__ __forceinline__ TnTile tn_locate(int tile, const int* split_prefix, const TnArgs& a) {
  int lo = 0, hi = a.E;  // last e with split_prefix[e] * m_blocks <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(split_prefix[mid]) * a.m_blocks <= tile) lo = mid; else hi = mid;
  }
  TnTile c;
  c.expert = lo;
  const int splits = split_prefix[lo + 1] - split_prefix[lo];
  const int local = tile - split_prefix[lo] * a.m_blocks;
  c.mb = local / splits;
  const int sp = local - c.mb * splits;
  const int64_t n = expert_rows(a.offsets, a.counts, a.R, lo);
  const int64_t per = ((n + splits - 1) / splits + kTnBox - 1) / kTnBox * kTnBox;  // equal shares, in steps of 16
  const int64_t begin = sp * per;
  int64_t rows = n - begin;
  rows = rows < 0 ? 0 : (rows < per ? rows : per);
  c.rows = static_cast<int>(rows);
  c.n = static_cast<int>((rows + kTnBox - 1) / kTnBox * kTnBox);
  if (c.n == 0) c.n = kTnBox;
  c.row0 = a.offsets[lo] + begin;
  return c;
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// All 128 epilogue threads learn whether every one of them got through its wait.
__device__ __forceinline__ bool epi_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(ok ? 1u : 0u)
      : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
    grouped_gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                           const TnArgs a) {  // map_a: box 64 x 64 token rows; map_w: box 64 x 128 weight rows
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_w = smem;
  uint8_t* smem_t = smem + kTnStages * kTnWBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* tmem_full = empty + kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  int* abort_flag = reinterpret_cast<int*>(tmem_base_slot + 1);
  uint64_t* drain = reinterpret_cast<uint64_t*>(abort_flag + 1);
  __nv_bfloat16* turn = reinterpret_cast<__nv_bfloat16*>(smem + kStages * kStageBytes + 256);  // [2][32 tokens][128 cols]
  int* split_prefix = reinterpret_cast<int*>(smem + kStages * kStageBytes + 256 + kEpiStageBytes);  // [E + 1]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int fills = 0;
  bool mma_issued = false;

  for (int e = threadIdx.x; e < a.E; e += kGemmThreads) {
    const int64_t n = expert_rows(a.offsets, a.counts, a.R, e);
    if (n != a.counts[e] && a.counts[e] > 0 && a.status != nullptr && blockIdx.x == 0)
      atomicOr(a.status, FMOE_STATUS_BAD_EXPERT);
    split_prefix[e + 1] = tn_splits(n);
  }
  if (threadIdx.x == 0) {
    split_prefix[0] = 0;
    *abort_flag = 0;
    for (int s = 0; s < kTnStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(drain, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < a.E; base += 32) {
      const int e = base + lane;
      int v = e < a.E ? split_prefix[e + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += n;
      }
      if (e < a.E) split_prefix[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_base_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_tiles = split_prefix[a.E] * a.m_blocks;

  if (warp == 0) {
    // ---- TMA producer: lane 0 waits and announces the bytes, six lanes issue one box each ------
    int stage = 0;
    uint32_t phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles && !a.skip_loads; tile += gridDim.x) {
      const TnTile c = tn_locate(tile, split_prefix, a);
      const int boxes = (c.n + kTnLoadRows - 1) / kTnLoadRows;
      const int w_row = c.expert * a.w_rows_per_expert;
      // lane 0: first weight tile, lane 1: second one (the next 128 output columns, or the up rows)
      const int my_w_row = a.swiglu ? w_row + (lane ? a.ff : 0) + c.mb * 128 : w_row + c.mb * 256 + lane * 128;
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&empty[stage], phase ^ 1, abort_flag, a.spin_limit) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) goto timed_out;
        if (lane == 0) {
          mbar_expect_tx(&full[stage], kTnWBytes + boxes * kTnLoadBytes);
          ++fills;
        }
        __syncwarp();
        if (lane < 2)
          tma_load_2d(smem_w + stage * kTnWBytes + lane * (kTnWBytes / 2), &map_w, kb * kBK, my_w_row, &full[stage]);
        if (lane >= 8 && lane - 8 < boxes)
          tma_load_2d(smem_t + stage * kTnTBytes + (lane - 8) * kTnLoadBytes, &map_a, kb * kBK,
                      static_cast<int>(c.row0) + (lane - 8) * kTnLoadRows, &full[stage]);
        if (++stage == kTnStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: two products per k-step, one per weight tile, the tokens shared -----------
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const TnTile c = tn_locate(tile, split_prefix, a);
      // D fp32, A and B bf16, both K-major, M = 128 weight rows, N = this tile's tokens
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(c.n >> 3) << 17) |
                             (static_cast<uint32_t>(128 >> 4) << 24);
      if (!mbar_wait(&tmem_empty[0], (it & 1) ^ 1, abort_flag, a.spin_limit)) goto timed_out;
      tcgen05_fence_after();
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        if (!mbar_wait(&full[stage], phase, abort_flag, a.spin_limit)) goto timed_out;
        tcgen05_fence_after();
        mma_issued = true;
        const uint64_t dw0 = smem_desc(smem_u32(smem_w + stage * kTnWBytes));
        const uint64_t dw1 = smem_desc(smem_u32(smem_w + stage * kTnWBytes + kTnWBytes / 2));
        const uint64_t dt = smem_desc(smem_u32(smem_t + stage * kTnTBytes));
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          umma_bf16(tmem_base, dw0 + 2 * k, dt + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_bf16(tmem_base + kTnTokens, dw1 + 2 * k, dt + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[stage]);
        if (++stage == kTnStages) { stage = 0; phase ^= 1; }
      }
      umma_commit(&tmem_full[0]);
    }
  } else if (warp >= 2) {
    // ---- epilogue: lane = output column, TMEM column = token -----------------------------------
    const int quarter = warp & 3;
    const int tid = threadIdx.x - 64;  // 0..127 among the epilogue threads
    const int halves = a.swiglu ? 1 : 2;  // passes over the tile: one per 128 output columns
    int it = 0;
    uint32_t chunk = 0;  // running count of 32-token chunks: its parity picks the turning buffer
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const TnTile c = tn_locate(tile, split_prefix, a);
      const bool got = mbar_wait(&tmem_full[0], it & 1, abort_flag, a.spin_limit);
      if (!epi_all(got)) goto timed_out;  // the four warps go on, or give up, together
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const int64_t col0 = static_cast<int64_t>(c.mb) * (a.swiglu ? 128 : 256);
#pragma unroll 1
      for (int half = 0; half < halves; ++half) {
#pragma unroll 1
        for (int c0 = 0; c0 < c.n; c0 += 32, ++chunk) {
          __nv_bfloat16* buf = turn + (chunk & 1) * (32 * 128);
          uint32_t r[32];
          if (a.swiglu) {
            uint32_t u[32];
            tmem_ld32(taddr + c0, r);
            tmem_ld32(taddr + kTnTokens + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              buf[j * 128 + quarter * 32 + lane] =
                  __float2bfloat16_rn(silu(__uint_as_float(r[j])) * __uint_as_float(u[j]));
          } else {
            tmem_ld32(taddr + half * kTnTokens + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float v = __uint_as_float(r[j]);
              buf[j * 128 + quarter * 32 + lane] = __float2bfloat16_rn(a.gelu ? gelu_erf(v) : v);
            }
          }
          if (half == halves - 1 && c0 + 32 >= c.n) {
            // the last read of tensor memory for this tile: the next tile's MMAs may start
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[0]);
          }
          epi_bar_sync();  // the chunk is complete in shared memory (the other buffer is refilled next)
#pragma unroll
          for (int r0 = 0; r0 < 32; r0 += 8) {  // 8 token rows per pass, 16 threads x 16 bytes per row
            const int tr = r0 + (tid >> 4), q = tid & 15;
            const int token = c0 + tr;
            const int64_t a_row = c.row0 + token;
            if (token < c.rows && a_row < a.R) {
              char* row = nullptr;
              if (a.c_row_ptrs != nullptr) row = reinterpret_cast<char*>(a.c_row_ptrs[a_row]);
              if (row == nullptr && a.C != nullptr) {
                const int64_t out_row = (a.c_row_ptrs == nullptr && a.c_row_map != nullptr) ? a.c_row_map[a_row] : a_row;
                row = reinterpret_cast<char*>(a.C + out_row * a.ldc);
              }
              if (row != nullptr) {
                const uint4 val = *reinterpret_cast<const uint4*>(buf + tr * 128 + q * 8);
                *reinterpret_cast<uint4*>(row + (col0 + half * 128 + q * 8) * 2) = val;
              }
            }
          }
        }
      }
    }
  }
  goto done;

timed_out:
  *abort_flag = 1;
  if (a.status != nullptr) atomicOr(a.status, FMOE_STATUS_WAIT_TIMEOUT);

done:
  drain_on_exit(warp, lane, fills, mma_issued, full, drain, abort_flag, kTnStages, a.spin_limit);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------
// SMs the persistent grid may occupy (fmoe_tune "gemm_sms"). Leaving a few SMs free lets
// NCCL's copy kernels run beside the GEMM instead of waiting for its CTAs to retire.
int g_gemm_sms = kNumSMs;
// Test hooks (fmoe_tune "gemm_skip_loads", "gemm_spin_limit"): make the bounded waits run out
// on purpose, with a short limit, to exercise the give-up path without hanging anything.
int g_gemm_skip_loads = 0;
// fmoe_tune "gemm_prefetch": weight k-blocks to request into L2 ahead of the loads. Off unless
// asked for: measured on B200 it costs more than it returns in both regimes (256 rows per expert:
// 6.13 ms without, 6.93 / 6.74 / 8.03 ms with 8 / 16 / 32 k-blocks ahead; 2048 rows per expert:
// 4.62 ms without, 5.07-5.15 ms with), because the requests go through the same TMA unit and
// fill path as the loads, which are already close to their per-SM limit.
int g_gemm_prefetch = 0;
static int prefetch_depth(int64_t, int64_t) { return g_gemm_prefetch > 0 ? g_gemm_prefetch : 0; }
int g_gemm_spin_limit = static_cast<int>(kSpinLimit);
// fmoe_tune "gemm_tokens_as_n": which forward kernel fmoe_grouped_gemm launches. 1 = tokens as
// the MMA's N dimension (grouped_gemm_tn_kernel), 0 = tokens in 128-row blocks as its M dimension
// (grouped_gemm_kernel), -1 = choose from the sizes the host knows: tokens as N while the experts
// average fewer than kTnAutoRows rows, where padding to 128-row blocks costs most.
int g_gemm_tokens_as_n = -1;
constexpr int64_t kTnAutoRows = 0;  // rows per expert below which "auto" picks tokens-as-N (0: never)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols], box = 64 columns x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, const char* what,
                    int box_rows = 128) {
  // The encoder is a driver call and wants a current context. A thread that has not yet made
  // a runtime call of this library (an autograd worker, say) may have none bound: bind it.
  FMOE_CUDA(cudaFree(nullptr));
  EncodeTiledFn fn = encode_tiled_fn();
  FMOE_REQUIRE(fn != nullptr, FMOE_ERR_DEVICE, "fmoe_grouped_gemm: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FMOE_REQUIRE(r == CUDA_SUCCESS, FMOE_ERR_ARG, "fmoe_grouped_gemm: cuTensorMapEncodeTiled(%s) failed with %d", what,
               static_cast<int>(r));
  return FMOE_OK;
}

}  // namespace fmoe

using namespace fmoe;

static int grouped_gemm_impl(const void* a, const void* w, void* c, void* pre, const int64_t* offsets,
                             const int64_t* counts, const int64_t* c_row_map, const int64_t* c_row_ptrs,
                             int64_t E, int64_t R, int64_t N, int64_t K, int activation, int32_t* status,
                             void* stream);

extern "C" int fmoe_grouped_gemm(const void* a, const void* w, void* c, const int64_t* offsets,
                                 const int64_t* counts, const int64_t* c_row_map, const int64_t* c_row_ptrs,
                                 int64_t E, int64_t R, int64_t N, int64_t K, int activation, int32_t* status,
                                 void* stream) {
  FMOE_RANGE("fmoe_grouped_gemm");
  return grouped_gemm_impl(a, w, c, nullptr, offsets, counts, c_row_map, c_row_ptrs, E, R, N, K, activation, status,
                           stream);
}

extern "C" int fmoe_grouped_gemm_keep_pre(const void* a, const void* w, void* c, void* pre, const int64_t* offsets,
                                          const int64_t* counts, const int64_t* c_row_map,
                                          const int64_t* c_row_ptrs, int64_t E, int64_t R, int64_t N, int64_t K,
                                          int activation, int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_grouped_gemm_keep_pre");
  FMOE_REQUIRE(pre != nullptr && aligned_to(pre, 16), FMOE_ERR_ARG,
               "fmoe_grouped_gemm_keep_pre: pre must be a 16-byte aligned [R, N] buffer");
  return grouped_gemm_impl(a, w, c, pre, offsets, counts, c_row_map, c_row_ptrs, E, R, N, K, activation, status,
                           stream);
}

static int grouped_gemm_impl(const void* a, const void* w, void* c, void* pre, const int64_t* offsets,
                             const int64_t* counts, const int64_t* c_row_map, const int64_t* c_row_ptrs,
                             int64_t E, int64_t R, int64_t N, int64_t K, int activation, int32_t* status,
                             void* stream) {
  FMOE_REQUIRE(activation >= FMOE_ACT_NONE && activation <= FMOE_ACT_GELU, FMOE_ERR_ARG,
               "fmoe_grouped_gemm: activation must be FMOE_ACT_NONE, FMOE_ACT_SWIGLU or FMOE_ACT_GELU");
  const int swiglu = activation == FMOE_ACT_SWIGLU;
  FMOE_REQUIRE(E >= 0 && R >= 0 && N > 0 && K > 0, FMOE_ERR_ARG, "fmoe_grouped_gemm: bad sizes");
  FMOE_REQUIRE(E <= kMaxExperts, FMOE_ERR_UNSUPPORTED, "fmoe_grouped_gemm: supports E <= %d", kMaxExperts);
  FMOE_REQUIRE(K % kBK == 0, FMOE_ERR_UNSUPPORTED, "fmoe_grouped_gemm: K=%lld must be a multiple of %d",
               (long long)K, kBK);
  if (swiglu) {
    FMOE_REQUIRE(N % 256 == 0, FMOE_ERR_UNSUPPORTED,
                 "fmoe_grouped_gemm: SwiGLU needs N = 2*ff with ff a multiple of 128 (N=%lld)", (long long)N);
  } else {
    FMOE_REQUIRE(N % kBN == 0, FMOE_ERR_UNSUPPORTED, "fmoe_grouped_gemm: N=%lld must be a multiple of %d",
                 (long long)N, kBN);
  }
  FMOE_REQUIRE(R < (1ll << 31) && E * N < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_grouped_gemm: R and E*N must fit in int32");
  if (E == 0 || R == 0) return FMOE_OK;
  FMOE_REQUIRE(a && w && (c || c_row_ptrs) && offsets && counts, FMOE_ERR_ARG,
               "fmoe_grouped_gemm: null pointer argument");
  FMOE_REQUIRE(aligned_to(a, 16) && aligned_to(w, 16) && aligned_to(c, 16), FMOE_ERR_ARG,
               "fmoe_grouped_gemm: a, w and c must be 16-byte aligned");
  // (the tokens-as-N kernel does not keep pre-activations: a training forward takes the other one)
  const bool tokens_as_n =
      pre == nullptr && (g_gemm_tokens_as_n == 1 || (g_gemm_tokens_as_n < 0 && R / E < kTnAutoRows));
  if (tokens_as_n) {
    CUtensorMap map_t, map_wt;
    int rc_t = make_map(&map_t, a, R, K, "A (64-row boxes)", kTnLoadRows);
    if (rc_t != 0) return rc_t;
    rc_t = make_map(&map_wt, w, E * N, K, "W", 128);
    if (rc_t != 0) return rc_t;
    TnArgs t;
    t.offsets = offsets;
    t.counts = counts;
    t.c_row_map = c_row_map;
    t.c_row_ptrs = c_row_ptrs;
    t.C = static_cast<__nv_bfloat16*>(c);
    t.ldc = swiglu ? N / 2 : N;
    t.R = R;
    t.E = static_cast<int>(E);
    t.m_blocks = static_cast<int>(swiglu ? (N / 2) / 128 : N / 256);
    t.k_blocks = static_cast<int>(K / kBK);
    t.w_rows_per_expert = static_cast<int>(N);
    t.ff = static_cast<int>(N / 2);
    t.swiglu = swiglu ? 1 : 0;
    t.gelu = activation == FMOE_ACT_GELU ? 1 : 0;
    t.skip_loads = g_gemm_skip_loads;
    t.spin_limit = static_cast<uint32_t>(g_gemm_spin_limit);
    t.status = status;
    const size_t smem_t = 1024 + static_cast<size_t>(kStages) * kStageBytes + 256 + kEpiStageBytes + sizeof(int) * (E + 2);
    FMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   1024 + kStages * kStageBytes + 256 + kEpiStageBytes +
                                       static_cast<int>(sizeof(int)) * (kMaxExperts + 2)));
    // upper bound of the tile count, known without reading the counts: one partial tile per expert
    const int64_t max_tiles_t = (R / kTnTokens + E) * t.m_blocks;
    const int grid_t = static_cast<int>(max_tiles_t < g_gemm_sms ? max_tiles_t : g_gemm_sms);
    grouped_gemm_tn_kernel<<<grid_t, kGemmThreads, smem_t, static_cast<cudaStream_t>(stream)>>>(map_t, map_wt, t);
    return check_launch("grouped_gemm_tn_kernel");
  }
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, a, R, K, "A");
  if (rc != 0) return rc;
  rc = make_map(&map_w, w, E * N, K, "W", swiglu ? 128 : 256);
  if (rc != 0) return rc;

  GemmArgs g;
  g.offsets = offsets;
  g.counts = counts;
  g.c_row_map = c_row_map;
  g.c_row_ptrs = c_row_ptrs;
  g.C = static_cast<__nv_bfloat16*>(c);
  g.pre = static_cast<__nv_bfloat16*>(pre);
  g.ldc = swiglu ? N / 2 : N;
  g.ld_pre = N;
  g.R = R;
  g.E = static_cast<int>(E);
  g.n_blocks = static_cast<int>(swiglu ? (N / 2) / 128 : N / kBN);
  g.k_blocks = static_cast<int>(K / kBK);
  g.w_rows_per_expert = static_cast<int>(N);
  g.up_row_offset = static_cast<int>(swiglu ? N / 2 : 128);
  g.swiglu = swiglu ? 1 : 0;
  g.gelu = activation == FMOE_ACT_GELU ? 1 : 0;
  g.w_transposed = 0;
  g.skip_loads = g_gemm_skip_loads;
  g.prefetch = prefetch_depth(R, E);
  g.spin_limit = static_cast<uint32_t>(g_gemm_spin_limit);
  g.status = status;

  const size_t smem = 1024 + static_cast<size_t>(kStages) * kStageBytes + 256 + kEpiStageBytes + sizeof(int) * (E + 2);
  // per device and cheap: set on every call rather than caching per device
  FMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 1024 + kStages * kStageBytes + 256 + kEpiStageBytes +
                                     static_cast<int>(sizeof(int)) * (kMaxExperts + 2)));
  // upper bound of the tile count, known without reading the counts: one partial block per expert
  const int64_t max_tiles = (R / kBM + E) * g.n_blocks;
  const int grid = static_cast<int>(max_tiles < g_gemm_sms ? max_tiles : g_gemm_sms);
  grouped_gemm_kernel<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(stream)>>>(map_a, map_w, g);
  return check_launch("grouped_gemm_kernel");
}

extern "C" int fmoe_grouped_gemm_dgrad(const void* grad_c, const void* w, void* grad_a, const int64_t* offsets,
                                       const int64_t* counts, const int64_t* row_ptrs, int64_t E, int64_t R,
                                       int64_t N, int64_t K, int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_grouped_gemm_dgrad");
  FMOE_REQUIRE(E >= 0 && R >= 0 && N > 0 && K > 0, FMOE_ERR_ARG, "fmoe_grouped_gemm_dgrad: bad sizes");
  FMOE_REQUIRE(E <= kMaxExperts, FMOE_ERR_UNSUPPORTED, "fmoe_grouped_gemm_dgrad: supports E <= %d", kMaxExperts);
  FMOE_REQUIRE(N % kBK == 0 && K % kBN == 0, FMOE_ERR_UNSUPPORTED,
               "fmoe_grouped_gemm_dgrad: N=%lld must be a multiple of %d and K=%lld of %d", (long long)N, kBK,
               (long long)K, kBN);
  FMOE_REQUIRE(R < (1ll << 31) && E * N < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_grouped_gemm_dgrad: R and E*N must fit in int32");
  if (E == 0 || R == 0) return FMOE_OK;
  FMOE_REQUIRE(grad_c && w && (grad_a || row_ptrs) && offsets && counts, FMOE_ERR_ARG,
               "fmoe_grouped_gemm_dgrad: null pointer argument");
  FMOE_REQUIRE(aligned_to(grad_c, 16) && aligned_to(w, 16) && aligned_to(grad_a, 16), FMOE_ERR_ARG,
               "fmoe_grouped_gemm_dgrad: grad_c, w and grad_a must be 16-byte aligned");
  CUtensorMap map_a, map_w;
  int rc = make_map(&map_a, grad_c, R, N, "grad_c");
  if (rc != 0) return rc;
  rc = make_map(&map_w, w, E * N, K, "W (transposed use)", 64);
  if (rc != 0) return rc;
  GemmArgs g;
  g.offsets = offsets;
  g.counts = counts;
  g.c_row_map = nullptr;
  g.c_row_ptrs = row_ptrs;
  g.C = static_cast<__nv_bfloat16*>(grad_a);
  g.pre = nullptr;
  g.ld_pre = 0;
  g.ldc = K;
  g.R = R;
  g.E = static_cast<int>(E);
  g.n_blocks = static_cast<int>(K / kBN);   // output columns are W's columns
  g.k_blocks = static_cast<int>(N / kBK);   // the reduction runs over W's rows
  g.w_rows_per_expert = static_cast<int>(N);
  g.up_row_offset = 0;
  g.swiglu = 0;
  g.gelu = 0;
  g.w_transposed = 1;
  g.skip_loads = g_gemm_skip_loads;
  g.prefetch = prefetch_depth(R, E);
  g.spin_limit = static_cast<uint32_t>(g_gemm_spin_limit);
  g.status = status;
  const size_t smem = 1024 + static_cast<size_t>(kStages) * kStageBytes + 256 + kEpiStageBytes + sizeof(int) * (E + 2);
  FMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 1024 + kStages * kStageBytes + 256 + kEpiStageBytes +
                                     static_cast<int>(sizeof(int)) * (kMaxExperts + 2)));
  const int64_t max_tiles = (R / kBM + E) * g.n_blocks;
  const int grid = static_cast<int>(max_tiles < g_gemm_sms ? max_tiles : g_gemm_sms);
  grouped_gemm_kernel<<<grid, kGemmThreads, smem, static_cast<cudaStream_t>(stream)>>>(map_a, map_w, g);
  return check_launch("grouped_gemm_kernel (dgrad)");
}

extern "C" int fmoe_grouped_gemm_wgrad(const void* grad_c, const void* a, void* grad_w, const int64_t* offsets,
                                       const int64_t* counts, int64_t E, int64_t R, int64_t N, int64_t K,
                                       int32_t* status, void* stream) {
  FMOE_RANGE("fmoe_grouped_gemm_wgrad");
  FMOE_REQUIRE(E >= 0 && R >= 0 && N > 0 && K > 0, FMOE_ERR_ARG, "fmoe_grouped_gemm_wgrad: bad sizes");
  FMOE_REQUIRE(N % kBM == 0 && K % kBN == 0, FMOE_ERR_UNSUPPORTED,
               "fmoe_grouped_gemm_wgrad: N=%lld must be a multiple of %d and K=%lld of %d", (long long)N, kBM,
               (long long)K, kBN);
  FMOE_REQUIRE(R < (1ll << 31) && E * (N / kBM) * (K / kBN) < (1ll << 31), FMOE_ERR_UNSUPPORTED,
               "fmoe_grouped_gemm_wgrad: sizes must fit in int32");
  if (E == 0) return FMOE_OK;
  FMOE_REQUIRE(grad_w && offsets && counts && (R == 0 || (grad_c && a)), FMOE_ERR_ARG,
               "fmoe_grouped_gemm_wgrad: null pointer argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (R == 0) {  // no rows at all: every expert's gradient is zero
    FMOE_CUDA(cudaMemsetAsync(grad_w, 0, static_cast<size_t>(E) * N * K * 2, s));
    return FMOE_OK;
  }
  FMOE_REQUIRE(aligned_to(grad_c, 16) && aligned_to(a, 16) && aligned_to(grad_w, 16), FMOE_ERR_ARG,
               "fmoe_grouped_gemm_wgrad: grad_c, a and grad_w must be 16-byte aligned");
  CUtensorMap map_g, map_a;
  int rc = make_map(&map_g, grad_c, R, N, "grad_c (row reduction)", 64);
  if (rc != 0) return rc;
  rc = make_map(&map_a, a, R, K, "a (row reduction)", 64);
  if (rc != 0) return rc;
  WgradArgs g;
  g.offsets = offsets;
  g.counts = counts;
  g.grad_w = static_cast<__nv_bfloat16*>(grad_w);
  g.N = N;
  g.K = K;
  g.R = R;
  g.E = static_cast<int>(E);
  g.n_blocks = static_cast<int>(N / kBM);
  g.k_blocks = static_cast<int>(K / kBN);
  g.skip_loads = g_gemm_skip_loads;
  g.spin_limit = static_cast<uint32_t>(g_gemm_spin_limit);
  g.status = status;
  const int smem = 1024 + kStages * kStageBytes + 256 + kEpiStageBytes;
  FMOE_CUDA(cudaFuncSetAttribute(grouped_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int64_t tiles = E * g.n_blocks * g.k_blocks;
  const int grid = static_cast<int>(tiles < g_gemm_sms ? tiles : g_gemm_sms);
  grouped_wgrad_kernel<<<grid, kGemmThreads, smem, s>>>(map_g, map_a, g);
  return check_launch("grouped_wgrad_kernel");
}
