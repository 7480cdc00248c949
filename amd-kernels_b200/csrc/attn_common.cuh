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

// Default wall-clock bound of one mbarrier wait.  A healthy wait lasts microseconds; the
// longest legitimate one (an epilogue warp waiting for a whole long task) stays
// far below this.  A kernel may run its waits under another bound (WaitCtx::limit_ns).
constexpr uint64_t kWaitLimitNs = 2000ull * 1000ull * 1000ull;

struct AttnParams {
  // rank-4 maps, 128-byte swizzle, box = 64 head-dim elements x 128 rows (Q) or x the kernel's key block rows (K, V)
  CUtensorMap tm_q, tm_k, tm_v;
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

// LiteAttention launch (skip lists: lite_list.h).  `a` carries the tensor maps (K and V with 64-row boxes),
// output, status block, dimensions, layout, rounding and softmax constants; the tail-split fields are unused.
struct LiteParams {
  AttnParams a;
  const int16_t* read_list;  // [tasks][row_width]
  int16_t* write_list;       // [tasks][row_width]
  const int16_t* must_do;    // [len, s0, e0, ...] or null
  const int* order;          // task of each hand-out slot, heaviest first; null = identity
  int* counter;              // hand-out counter, zero at launch
  int num_tasks;             // batch * heads * query blocks
  int row_width;             // 64-key blocks + 2
  int phase;                 // 1: blocks walked upwards, 0: downwards
  float threshold;           // log2 units, negative
};

// MLA absorbed-decode launch (mla_decode.cu).
struct MlaParams {
  CUtensorMap tm_kv, tm_kv_rope;      // contiguous slab only: rank-3 byte map {576, seq, batch}, box 128 bytes x 96 rows, 128-byte swizzle
  int use_tma;            // 1: tiles come by box loads through tm_kv; 0: by 16-byte asynchronous copies (paged pool)
  const void* q_lat;      // bf16 [B, q_len, H, 512]  ([B, H, 512] when q_len = 1)
  const void* q_pe;       // bf16 [B, q_len, H, 64]
  const void* kv;         // fp8 rows of 576 bytes: [B, seq, 576] or a pool [slots, 1, 576]
  void* o_lat;            // bf16, like q_lat
  const int* seq_lens;    // [B] cached tokens per request, or null (= seq)
  const int* rows;        // [B] batch row of q / o for request b, or null (= b)
  const int* kv_indices;  // flat per-token slots, or null (contiguous slab)
  const int* kv_indptr;   // [B + 1] offsets into kv_indices
  uint32_t* status;
  float* part_o;          // [B * groups * parts][16 * pos_per_cta][512] un-normalised partial outputs
  float* part_ml;         // [B * groups * parts][16 * pos_per_cta][2] reference maximum (log2 units), denominator
  int batch, heads, q_len, seq;
  int parts, groups, pos_per_cta;
  int cluster_merge;      // set by the launcher: the parts of a request form a thread-block cluster and merge through shared memory
  int kv_format;          // 0: e4m3-fnuz (the reference's), 1: e4m3 (OCP, what the tensor core reads)
  float scale, kv_scale;
};

// ---------------------------------------------------------------------------
// bounded waits
// ---------------------------------------------------------------------------
struct WaitCtx {
  uint32_t* status;     // global status block or null
  volatile int* abort;  // shared-memory flag: some thread of this CTA gave up
  uint64_t limit_ns = kWaitLimitNs;  // how long one wait may last before it is abandoned
  bool watch_status = true;  // give up as soon as any CTA has reported an error (needs a status word that was zero before the launch)
};

__device__ __forceinline__ void record_error(uint32_t* status, uint32_t code, uint32_t site, uint32_t detail) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = site | (blockIdx.x << 8);
    status[2] = detail;
    __threadfence();
  }
}

// One poll of an mbarrier phase.  The suspend-time hint lets the hardware park the thread until the
// phase completes (or the hint runs out) instead of returning after a short spin: measured on B200 the
// parked MMA issuer and softmax waits leave power and issue slots to the working warps (+7 % at 8 K
// keys under the power cap), and wake-up is not slower.
constexpr uint32_t kPollHintNs = 20000;
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
  return sm100::mbar_try_wait_hint(bar, parity, kPollHintNs);
}

// Waits for the phase with the given parity of an mbarrier.  Returns false when
// the wait was abandoned (time limit, or another thread already reported an
// error); the caller must then unwind to the kernel's common exit.
// `kSleepNs` > 0 puts the thread to sleep between polls: a polling warp otherwise issues an instruction
// every few clocks and takes issue slots from the softmax warps that share its scheduler.  Waits whose
// wake-up latency is on the critical path (MMA issuer) keep kSleepNs = 0.
template <uint32_t kSleepNs>
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_poll(bar, parity)) return true;
    if (kSleepNs > 0) asm volatile("nanosleep.u32 %0;" ::"n"(kSleepNs));
    if ((it & 0x3Fu) == 0u) {
      if (*ctx.abort) return false;
      if (ctx.watch_status && ctx.status != nullptr && *reinterpret_cast<volatile uint32_t*>(ctx.status) != 0u) {
        *ctx.abort = 1;
        return false;
      }
      const uint64_t now = sm100::globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ctx.limit_ns) {
        record_error(ctx.status, kErrWaitTimeout, site, parity);
        *ctx.abort = 1;
        return false;
      }
    }
  }
}
template <uint32_t kSleepNs = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  if (mbar_poll(bar, parity)) return true;
  return mbar_wait_slow<kSleepNs>(bar, parity, site, ctx);
}
// Same, with the verdict made uniform over the warp (needed before warp-collective tcgen05.ld/st).
template <uint32_t kSleepNs = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, uint32_t site, const WaitCtx& ctx) {
  const bool ok = mbar_wait<kSleepNs>(bar, parity, site, ctx);
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

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Three-input maximum in one instruction; NaN operands are ignored (fmaxf semantics).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Packed pairs of fp32 in a 64-bit register: the FMA pipe of sm_100 processes both halves in one instruction.
using f32x2 = uint64_t;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Packs two probabilities as bf16 for the P operand of the second MMA (`lo` has the lower key index).
// The tensor core takes A and B of one 16-bit format only: a kind::f16 MMA with fp16 A and bf16 B is
// an illegal instruction on sm_100, so P shares V's bf16.  P is rounded to nearest-even in every
// output rounding mode; the mode applies to the final store only.
__device__ __forceinline__ uint32_t pack_p(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Precise mode: a probability pair as two bf16 pairs, P_hi + P_lo = p to about 16 significant bits.
// P_hi is p * (1 - 2^-9) truncated to bf16, so that the remainder p - P_hi is positive for every p > 0
// (between 2^-9 p and 2^-6.7 p, exact in fp32), and P_lo is that remainder rounded to bf16.  Both terms then have
// the sign of p: a +-inf in V meets two positive factors and stays +-inf, as in the fp32 formula; a remainder of
// either sign, or one that is exactly zero, would turn it into NaN (inf - inf, 0 * inf).  p = 0 gives 0 + 0.
__device__ __forceinline__ void pack_p_precise(float lo, float hi, uint32_t& p_hi, uint32_t& p_lo) {
  constexpr float kShrink = 1.f - 0.001953125f;  // 1 - 2^-9
  const f32x2 p2 = pack2(lo, hi);
  float a, b;
  unpack2(mul2(p2, pack2(kShrink, kShrink)), a, b);
  p_hi = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x7632);  // upper halves: a >> 16 | b & 0xFFFF0000
  const f32x2 h2 = pack2(__uint_as_float(p_hi << 16), __uint_as_float(p_hi & 0xFFFF0000u));
  float r0, r1;
  unpack2(fma2(h2, pack2(-1.f, -1.f), p2), r0, r1);
  p_lo = pack_p(r0, r1);
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
// A whole kRows x 128 tile = two boxes (head-dim halves) of kRows x 128 bytes each, both on the same barrier.
template <int kRows>
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int bshd, int row0,
                                              int h, int b) {
  tma_load_tile_half(dst, tm, bar, bshd, 0, row0, h, b);
  tma_load_tile_half(dst + kRows * 128, tm, bar, bshd, 64, row0, h, b);
}

// ---------------------------------------------------------------------------
// MMA issue.  One thread issues every tcgen05.mma of a CTA, and that thread's
// instruction stream is the pace-maker of the kernel: descriptors are therefore
// split into a constant high word and a low word that is a 32-bit add away from
// a per-tile base computed once.
//   low word : [0,14) start address >> 4, [16,30) leading byte offset >> 4
//   high word: [0,14) stride byte offset >> 4, [14,16) version = 1, [29,32) swizzle = 2 (128 bytes)
// ---------------------------------------------------------------------------
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO = 1024 bytes (8 rows of 128 bytes)
constexpr uint32_t kDescLoKMajor = (16u >> 4) << 16;                  // LBO unused (1)

// Low descriptor word of a tile at shared address `smem` read as a K-major operand (Q, K) ...
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t smem) { return ((smem & 0x3FFFFu) >> 4) | kDescLoKMajor; }
// ... or as an MN-major operand (V: head dimension contiguous); LBO = distance of the second 64-column half.
template <int kRows>
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t smem) {
  return ((smem & 0x3FFFFu) >> 4) | ((static_cast<uint32_t>(kRows * 128) >> 4) << 16);
}

__device__ __forceinline__ uint64_t make_desc(uint32_t lo) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(kDescHi));
  return d;
}

// S[128 x kKeys] = Q_tile * K_tile^T, both K-major: 8 MMAs of K = 16 over the head dimension.
// k-step ks lives in 64-column half (ks >> 2) of each tile, 32 bytes per step inside the 128-byte swizzle row.
template <int kKeys>
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_lo, uint32_t k_lo) {
  constexpr uint32_t idesc = sm100::umma_idesc(sm100::kFmtBF16, sm100::kFmtBF16, 0, 0, kTileM, kKeys);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint32_t q_off = ((ks >> 2) * (kTileM * 128) + (ks & 3) * 32) >> 4;
    const uint32_t k_off = ((ks >> 2) * (kKeys * 128) + (ks & 3) * 32) >> 4;
    sm100::umma_ss(d_tmem, make_desc(q_lo + q_off), make_desc(k_lo + k_off), idesc, ks > 0 ? 1u : 0u);
  }
}
// O[128 x 128] (+)= P (TMEM, bf16 pairs, 8 columns per step) * V_tile (MN-major): kKeys / 16 MMAs of K = 16 keys,
// 16 key rows = 2048 bytes per step.
template <int kKeys, int kFirstStep = 0, int kSteps = kKeys / 16>
__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_lo, bool accumulate) {
  constexpr uint32_t idesc = sm100::umma_idesc(sm100::kFmtBF16, sm100::kFmtBF16, 0, 1, kTileM, kHeadDim);
#pragma unroll
  for (int ks = kFirstStep; ks < kFirstStep + kSteps; ++ks) {
    sm100::umma_ts(d_tmem, p_tmem + ks * 8, make_desc(v_lo + ks * (2048 >> 4)), idesc,
                   (accumulate || ks > kFirstStep) ? 1u : 0u);
  }
}

}  // namespace ma
