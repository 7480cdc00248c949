// Shared pieces of the attention kernels: launch parameters, status words,
// bounded mbarrier waits, the three fp32 -> bf16 rounding rules and the
// per-row online-softmax arithmetic.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "sm100_ptx.cuh"

namespace ma {

constexpr int kHeadDim = 128;   // the only head size the operator supports (reference: csrc/attention_kernel.hip:1576)
constexpr int kTileM = 128;     // query rows per tensor-core tile (= TMEM lanes)
constexpr int kTileN = 128;     // key/value rows per block
constexpr int kTaskRows = 256;  // query rows per CTA task in the pipelined kernel (two tiles)
constexpr int kTileBytes = kTileM * kHeadDim * 2;  // 32 KiB: one 128 x 128 bf16 tile

enum RoundMode : int { kRTNE = 0, kRTNA = 1, kRTZ = 2 };

// Device-side status block at the start of the workspace (64 words = 256 bytes).
//   [0] first error code (0 = ok)   [1] wait site | blockIdx.x << 8   [2] detail
constexpr int kStatusWords = 64;
constexpr uint32_t kErrWaitTimeout = 0x57A17u;

// Wall-clock bound of one mbarrier wait.  A healthy wait lasts microseconds; the
// longest legitimate one (an epilogue warp waiting for a whole long task) stays
// far below this.
constexpr uint64_t kWaitLimitNs = 2000ull * 1000ull * 1000ull;

struct AttnParams {
  CUtensorMap tm_q, tm_k, tm_v;  // rank-4 maps, box = 64 head-dim elements x 128 rows, 128-byte swizzle
  __nv_bfloat16* out;
  uint32_t* status;  // may be null
  float* part_o;     // [slots][256][128] un-normalised fp32 partial outputs of KV-split units
  float* part_ml;    // [slots][256][2]   running max (log2 units) and row sum of each partial
  int batch, heads, seq_q, seq_kv;
  int bshd;          // 0: [B,H,S,D]   1: [B,S,H,D]
  int round_mode;    // RoundMode
  int nqb;           // query blocks per (batch, head): ceil(seq_q / rows per task)
  int nkb;           // key/value blocks: ceil(seq_kv / 128)
  int full_units;    // units [0, full_units) are whole tasks (all KV blocks, final output)
  int tail_tasks;    // tasks split along KV
  int split;         // parts per split task (>= 2 when tail_tasks > 0)
  int total_units;   // full_units + tail_tasks * split
  float scale_log2e; // log2(e) / sqrt(head_dim)
  float rescale_tau; // lazy-rescale threshold in log2 units (0 = always track the exact max)
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------
struct WaitCtx {
  uint32_t* status;     // global status block or null
  volatile int* abort;  // shared-memory flag: some thread of this CTA gave up
};

__device__ __forceinline__ void record_error(uint32_t* status, uint32_t code, uint32_t site, uint32_t detail) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = site | (blockIdx.x << 8);
    status[2] = detail;
    __threadfence();
  }
}

// Waits for the phase with the given parity of an mbarrier.  Returns false when
// the wait was abandoned (time limit, or another thread already reported an
// error); the caller must then unwind to the kernel's common exit.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (sm100::mbar_try_wait(bar, parity)) return true;
    if ((it & 0x3FFu) == 0u) {
      if (*ctx.abort) return false;
      if (ctx.status != nullptr && *reinterpret_cast<volatile uint32_t*>(ctx.status) != 0u) {
        *ctx.abort = 1;
        return false;
      }
      const uint64_t now = sm100::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > kWaitLimitNs) {
        record_error(ctx.status, kErrWaitTimeout, site, parity);
        *ctx.abort = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  if (sm100::mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, site, ctx);
}
// Same, with the verdict made uniform over the warp (needed before warp-collective tcgen05.ld/st).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  const bool ok = mbar_wait(bar, parity, site, ctx);
  return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------------------
// fp32 -> bf16, the three rules of the reference (csrc/attention_kernel.hip:110-145),
// NaN always becomes the canonical 0x7FFF.
// ---------------------------------------------------------------------------
template <int kMode>
__device__ __forceinline__ uint32_t bf16_bits(float f) {
  const uint32_t u = __float_as_uint(f);
  uint32_t r;
  if (kMode == kRTNE) {
    r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
  } else if (kMode == kRTNA) {
    r = (u + 0x8000u) >> 16;
  } else {
    r = u >> 16;
  }
  return (f != f) ? 0x7FFFu : r;
}
template <int kMode>
__device__ __forceinline__ uint32_t bf16_pack2(float lo, float hi) {
  return bf16_bits<kMode>(lo) | (bf16_bits<kMode>(hi) << 16);
}

// ---------------------------------------------------------------------------
// arithmetic helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packs two probabilities as bf16 for the P operand of the second MMA (`lo` has the lower key index).
// The tensor core takes A and B of one 16-bit format only: a kind::f16 MMA with fp16 A and bf16 B is
// an illegal instruction on sm_100, so P shares V's bf16.  P is rounded to nearest-even in every
// output rounding mode; the mode applies to the final store only.
__device__ __forceinline__ uint32_t pack_p(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Address (in elements) of output row `row` of slice (b, h).
__device__ __forceinline__ size_t out_row_offset(const AttnParams& p, int b, int h, int row) {
  if (p.bshd) return ((static_cast<size_t>(b) * p.seq_q + row) * p.heads + h) * kHeadDim;
  return ((static_cast<size_t>(b) * p.heads + h) * p.seq_q + row) * kHeadDim;
}

// Scales 32 fp32 accumulator values, rounds them and stores 64 bytes of the output row.
template <int kMode>
__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* dst, const uint32_t (&acc)[32], float inv) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 w;
    w.x = bf16_pack2<kMode>(__uint_as_float(acc[8 * q + 0]) * inv, __uint_as_float(acc[8 * q + 1]) * inv);
    w.y = bf16_pack2<kMode>(__uint_as_float(acc[8 * q + 2]) * inv, __uint_as_float(acc[8 * q + 3]) * inv);
    w.z = bf16_pack2<kMode>(__uint_as_float(acc[8 * q + 4]) * inv, __uint_as_float(acc[8 * q + 5]) * inv);
    w.w = bf16_pack2<kMode>(__uint_as_float(acc[8 * q + 6]) * inv, __uint_as_float(acc[8 * q + 7]) * inv);
    d4[q] = w;
  }
}
__device__ __forceinline__ void store_chunk_bf16(int mode, __nv_bfloat16* dst, const uint32_t (&acc)[32], float inv) {
  if (mode == kRTNE) {
    store_chunk_bf16<kRTNE>(dst, acc, inv);
  } else if (mode == kRTNA) {
    store_chunk_bf16<kRTNA>(dst, acc, inv);
  } else {
    store_chunk_bf16<kRTZ>(dst, acc, inv);
  }
}

// Coordinates of a 64 x 128 TMA box: head-dim offset d0, first row, head, batch.
__device__ __forceinline__ void tma_load_tile_half(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int bshd, int d0,
                                                   int row0, int h, int b) {
  if (bshd) {
    sm100::tma_load_4d(dst, tm, bar, d0, h, row0, b);
  } else {
    sm100::tma_load_4d(dst, tm, bar, d0, row0, h, b);
  }
}
// A whole 128 x 128 tile = two boxes (head-dim halves), 16 KiB each, both on the same barrier.
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int bshd, int row0,
                                              int h, int b) {
  tma_load_tile_half(dst, tm, bar, bshd, 0, row0, h, b);
  tma_load_tile_half(dst + kTileBytes / 2, tm, bar, bshd, 64, row0, h, b);
}

// S[128 x 128] = A_tile (K-major) * B_tile^T (K-major): 8 MMAs of K = 16 over the head dimension.
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_smem, uint32_t k_smem) {
  constexpr uint32_t idesc = sm100::umma_idesc(sm100::kFmtBF16, sm100::kFmtBF16, 0, 0, kTileM, kTileN);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t off = (ks >> 2) * (kTileBytes / 2) + (ks & 3) * 32;
    sm100::umma_ss(d_tmem, sm100::umma_smem_desc(q_smem + off, 16, 1024), sm100::umma_smem_desc(k_smem + off, 16, 1024),
                   idesc, ks > 0 ? 1u : 0u);
  }
}
// O[128 x 128] (+)= P (TMEM, 16-bit pairs) * V_tile (MN-major: head dim contiguous): 8 MMAs of K = 16 keys.
__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_smem, bool accumulate) {
  constexpr uint32_t idesc = sm100::umma_idesc(sm100::kFmtBF16, sm100::kFmtBF16, 0, 1, kTileM, kHeadDim);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    sm100::umma_ts(d_tmem, p_tmem + ks * 8, sm100::umma_smem_desc(v_smem + ks * 2048, kTileBytes / 2, 1024), idesc,
                   (accumulate || ks > 0) ? 1u : 0u);
  }
}

}  // namespace ma
