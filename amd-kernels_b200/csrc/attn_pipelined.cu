// The production kernel: a persistent, warp-specialised flash-attention forward
// for sm_100a.  One CTA per SM walks a list of units; a unit is a 256-row query
// block (two 128-row tiles) of one (batch, head) slice against a contiguous
// range of 128-row key/value blocks.
//
//   warps  0- 3  softmax of tile 0     (one thread per query row, fp32 online softmax)
//   warps  4- 7  softmax of tile 1
//   warps  8-11  epilogue              (normalise, round to bf16, store; or fp32 partials)
//   warp  12     MMA issuer            (one thread issues every tcgen05.mma)
//   warp  13     TMA producer          (Q tiles and the K/V ring, either native layout)
//   warps 14-15  idle
//
// Tensor memory (512 columns x 128 lanes x 32 bit):
//   [  0,128) S0   [128,256) S1   [256,384) O0   [384,512) O1
//   P_t (16-bit pairs, 64 columns) overwrites the first half of S_t and feeds the
//   second MMA straight from tensor memory.
//
// The two tiles ping-pong: while the softmax warps work on S_t the tensor core
// runs the other tile's P*V and next Q*K^T, in the issue order
//   PV0(j)  QK0(j+1)  PV1(j)  QK1(j+1)  PV0(j+1) ...
// MMAs complete in issue order, which is what makes the S/P aliasing safe.
//
// Precise mode (MA_FLAG_PRECISE_P): the probabilities reach the tensor core as the sum of two bf16 terms,
// P = P_hi + P_lo (pack_p_precise), P_hi in columns [0, 64) and P_lo in columns [64, 128) of S_t
// (all scores are in registers by then), and P*V is issued twice into the same accumulator.  That carries
// 16 significant bits of p instead of 8 for 25 % more tensor work.
//
// All synchronisation is CTA-local mbarriers; every wait is bounded.
#include "attn_common.cuh"
#include "attn_launch.h"

namespace ma {
namespace {

using namespace sm100;

constexpr int kThreads = 512;
constexpr int kStages = 4;  // K/V ring, 32 KiB each
constexpr uint32_t kTmemCols = 512;
// Sleep between polls of a barrier that is not complete yet, per role (ns): waiting warps then leave the
// issue slots (and the power budget) to the working ones.  The MMA issuer does not sleep (its wake-up
// latency is on the critical path); every poll, its own included, carries a suspend-time hint.
constexpr uint32_t kSleepProducer = 128, kSleepSoftmax = 32, kSleepEpilogue = 1000;

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffQ = 0;                                    // 2 tiles
constexpr uint32_t kOffKV = 2 * kTileBytes;                      // kStages tiles
constexpr uint32_t kOffStats = kOffKV + kStages * kTileBytes;    // float [2 parity][2 tile][128 rows][2: max, sum]
constexpr uint32_t kOffBars = kOffStats + 2 * 2 * 128 * 2 * 4;   // mbarriers, 8 bytes each
enum Bar : uint32_t {
  kBarQFull = 0,                       // [2]       TMA -> MMA
  kBarQEmpty = 2,                      //           MMA -> TMA (both Q tiles consumed)
  kBarKvFull = 3,                      // [kStages] TMA -> MMA
  kBarKvEmpty = kBarKvFull + kStages,  // [kStages] MMA -> TMA
  kBarSFull = kBarKvEmpty + kStages,   // [2]       MMA -> softmax
  kBarPFull = kBarSFull + 2,           // [2]       softmax -> MMA (128 arrivals)
  kBarOFull = kBarPFull + 2,           // [2]       MMA -> epilogue
  kBarOFree = kBarOFull + 2,           // [2]       epilogue -> MMA (128 arrivals)
  kBarLReady = kBarOFree + 2,          // [2]       softmax -> epilogue (128 arrivals)
  kNumBars = kBarLReady + 2
};
constexpr uint32_t kOffTmemSlot = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemSlot + 4;
constexpr size_t kSmemBytes = kOffAbort + 4 + 1024;  // + alignment slack

struct Unit {
  int qb, b, h;      // query block, batch, head
  int kb_begin, kb_end;
  int part;          // partial-result slot, or -1 when the unit produces final output
};

__device__ __forceinline__ Unit decode_unit(const AttnParams& p, int u) {
  Unit r;
  int task;
  if (u < p.full_units) {
    task = u;
    r.kb_begin = 0;
    r.kb_end = p.nkb;
    r.part = -1;
  } else {
    const int v = u - p.full_units;
    task = p.full_units + v / p.split;
    const int g = v % p.split;
    r.kb_begin = static_cast<int>((static_cast<long long>(g) * p.nkb) / p.split);
    r.kb_end = static_cast<int>((static_cast<long long>(g + 1) * p.nkb) / p.split);
    r.part = v;
  }
  // Head-major order: consecutive tasks share a (batch, head) so that concurrently
  // running CTAs read the same K/V and find it in L2.
  r.qb = task % p.nqb;
  const int bh = task / p.nqb;
  r.b = bh / p.heads;
  r.h = bh % p.heads;
  return r;
}


#define MA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), (site), ctx)) return
#define MA_WAIT_WARP(bar, parity, site) \
  if (!mbar_wait_warp((bar), (parity), (site), ctx)) return
#define MA_WAIT_SLEEP(ns, bar, parity, site) \
  if (!mbar_wait<ns>((bar), (parity), (site), ctx)) return
#define MA_WAIT_WARP_SLEEP(ns, bar, parity, site) \
  if (!mbar_wait_warp<ns>((bar), (parity), (site), ctx)) return

// ---------------------------------------------------------------------------
// TMA producer (one thread)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void role_producer(const AttnParams& p, uint32_t base, const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  uint32_t fill = 0;  // K/V ring fills so far
  uint32_t it = 0;    // units so far
  for (int u = blockIdx.x; u < p.total_units; u += gridDim.x, ++it) {
    const Unit un = decode_unit(p, u);
    const int q_row0 = un.qb * kTaskRows;
    if (it > 0) MA_WAIT_SLEEP(kSleepProducer, bars + 8 * kBarQEmpty, (it - 1) & 1, 0x10);
    mbar_arrive_expect_tx(bars + 8 * (kBarQFull + 0), kTileBytes);
    tma_load_tile<kTileM>(base + kOffQ, &p.tm_q, bars + 8 * (kBarQFull + 0), p.bshd, q_row0, un.h, un.b);
    for (int kb = un.kb_begin; kb < un.kb_end; ++kb) {
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        const uint32_t stage = fill % kStages, use = fill / kStages;
        if (use > 0) MA_WAIT_SLEEP(kSleepProducer, bars + 8 * (kBarKvEmpty + stage), (use - 1) & 1, 0x11 + kv);
        const uint32_t full = bars + 8 * (kBarKvFull + stage);
        mbar_arrive_expect_tx(full, kTileBytes);
        tma_load_tile<kTileN>(base + kOffKV + stage * kTileBytes, kv == 0 ? &p.tm_k : &p.tm_v, full, p.bshd, kb * kTileN, un.h,
                      un.b);
        ++fill;
        if (kv == 0 && kb == un.kb_begin) {  // second Q tile right behind the first K block
          mbar_arrive_expect_tx(bars + 8 * (kBarQFull + 1), kTileBytes);
          tma_load_tile<kTileM>(base + kOffQ + kTileBytes, &p.tm_q, bars + 8 * (kBarQFull + 1), p.bshd, q_row0 + kTileM, un.h,
                        un.b);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// MMA issuer (one thread)
// ---------------------------------------------------------------------------
template <bool kPrecise>
__device__ __forceinline__ void role_mma(const AttnParams& p, uint32_t base, uint32_t tmem, const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  const uint32_t q_lo = desc_lo_kmajor(base + kOffQ);      // + tile  * (kTileBytes >> 4)
  const uint32_t kv_lo_k = desc_lo_kmajor(base + kOffKV);  // + stage * (kTileBytes >> 4)
  const uint32_t kv_lo_v = desc_lo_mnmajor<kTileN>(base + kOffKV);
  constexpr uint32_t kTileLo = kTileBytes >> 4;
  uint32_t fill = 0;   // K/V ring fills consumed before this unit
  uint32_t it = 0;     // units so far
  uint32_t blk = 0;    // key/value blocks so far (phase of s_full / p_full)
  for (int u = blockIdx.x; u < p.total_units; u += gridDim.x, ++it) {
    const Unit un = decode_unit(p, u);
    const int n = un.kb_end - un.kb_begin;

    // S0(0), S1(0)
    {
      const uint32_t st = fill % kStages;
      MA_WAIT(bars + 8 * (kBarKvFull + st), (fill / kStages) & 1, 0x21);
      const uint32_t k_lo = kv_lo_k + st * kTileLo;
#pragma unroll 1
      for (uint32_t t = 0; t < 2; ++t) {
        MA_WAIT(bars + 8 * (kBarQFull + t), it & 1, 0x20 + t);
        tc_fence_after_sync();
        issue_qk<kTileN>(tmem + t * 128, q_lo + t * kTileLo, k_lo);
        umma_commit(bars + 8 * (kBarSFull + t));
      }
      umma_commit(bars + 8 * (kBarKvEmpty + st));
      if (n == 1) umma_commit(bars + 8 * kBarQEmpty);
    }
    for (int j = 0; j < n; ++j, ++blk) {
      const uint32_t fv = fill + 2 * j + 1, sv = fv % kStages;   // V(j)
      const uint32_t fk = fill + 2 * j + 2, sk = fk % kStages;   // K(j+1)
      const uint32_t v_lo = kv_lo_v + sv * kTileLo;
      const uint32_t k_lo = kv_lo_k + sk * kTileLo;
      const bool more = (j + 1 < n);
      // Operand tiles first: these waits are normally long satisfied and must not sit between
      // "P is ready" and the issue of the MMAs that consume it.
      MA_WAIT(bars + 8 * (kBarKvFull + sv), (fv / kStages) & 1, 0x23);
      if (more) MA_WAIT(bars + 8 * (kBarKvFull + sk), (fk / kStages) & 1, 0x26);
#pragma unroll 1
      for (uint32_t t = 0; t < 2; ++t) {
        // O_t (+)= P_t(j) V(j);  S_t(j+1) = Q_t K(j+1)^T
        if (j == 0 && it > 0) MA_WAIT(bars + 8 * (kBarOFree + t), (it - 1) & 1, 0x25);
        MA_WAIT(bars + 8 * (kBarPFull + t), blk & 1, 0x24);
        tc_fence_after_sync();
        issue_pv<kTileN>(tmem + 256 + t * 128, tmem + t * 128, v_lo, j > 0);
        if constexpr (kPrecise) issue_pv<kTileN>(tmem + 256 + t * 128, tmem + t * 128 + 64, v_lo, true);
        if (t == 1) umma_commit(bars + 8 * (kBarKvEmpty + sv));
        if (more) {
          issue_qk<kTileN>(tmem + t * 128, q_lo + t * kTileLo, k_lo);
          umma_commit(bars + 8 * (kBarSFull + t));
        } else {
          umma_commit(bars + 8 * (kBarOFull + t));
        }
      }
      if (more) {
        umma_commit(bars + 8 * (kBarKvEmpty + sk));
        if (j + 2 == n) umma_commit(bars + 8 * kBarQEmpty);
      }
    }
    fill += 2 * static_cast<uint32_t>(n);
  }
}

// Reads this thread's 128 scores of the current block; keys past the end of the sequence become -inf.
__device__ __forceinline__ void load_scores(uint32_t tS, uint32_t (&s)[128], int valid) {
  tmem_ld128_sync(tS, s);
  if (valid < kTileN) {
#pragma unroll
    for (int i = 0; i < 128; ++i)
      if (i >= valid) s[i] = __float_as_uint(-INFINITY);
  }
}
// Row maximum that ignores NaN scores (fmaxf semantics), for the slow path.
__device__ __forceinline__ float row_max(const uint32_t (&s)[128]) {
  float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    mx0 = fmaxf(mx0, __uint_as_float(s[i]));
    mx1 = fmaxf(mx1, __uint_as_float(s[32 + i]));
    mx2 = fmaxf(mx2, __uint_as_float(s[64 + i]));
    mx3 = fmaxf(mx3, __uint_as_float(s[96 + i]));
  }
  return fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
}

// Largest row sum of one block (relative to the reference maximum) the speculative pass accepts:
// p <= 2^40, so P and the accumulators stay far inside bf16 and fp32 range.
constexpr float kSumHard = 1.099511627776e12f;  // 2^40

// O_row *= alpha for this thread's accumulator row (128 fp32 columns in tensor memory).
__device__ __forceinline__ void rescale_accumulator(uint32_t tO, float alpha) {
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    uint32_t o[32];
    tmem_ld32_sync(tO + c * 32, o);
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
    tmem_st32(tO + c * 32, o);
  }
}

// ---------------------------------------------------------------------------
// softmax warps (128 threads per tile, one query row each)
// ---------------------------------------------------------------------------
template <bool kPrecise>
__device__ __forceinline__ void role_softmax(const AttnParams& p, uint8_t* smem, uint32_t base, uint32_t tmem, int tile,
                                             int row, const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  const uint32_t lane_sel = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t tS = tmem + tile * 128 + lane_sel;
  const uint32_t tO = tmem + 256 + tile * 128 + lane_sel;
  const uint32_t bar_s = bars + 8 * (kBarSFull + tile), bar_p = bars + 8 * (kBarPFull + tile);
  float* stats = reinterpret_cast<float*>(smem + kOffStats);
  const float scale = p.scale_log2e;
  uint32_t blk = 0, it = 0;
  for (int u = blockIdx.x; u < p.total_units; u += gridDim.x, ++it) {
    const Unit un = decode_unit(p, u);
    const int n = un.kb_end - un.kb_begin;
    float m_ref = 0.f, m_seen = 0.f, l_run = 0.f;
    for (int j = 0; j < n; ++j, ++blk) {
      MA_WAIT_WARP_SLEEP(kSleepSoftmax, bar_s, blk & 1, 0x30 + tile);
      tc_fence_after_sync();
      uint32_t s[128];
      const int valid = p.seq_kv - (un.kb_begin + j) * kTileN;
      load_scores(tS, s, valid);
      uint32_t pk[64];  // P of this block as bf16 pairs; written to tensor memory once the block is known to be safe
      uint32_t pl[kPrecise ? 64 : 1];  // precise mode: the bf16 pairs of what rounding p to P left over

      // Speculative pass (every block but the first of a unit): exponentiate against the reference
      // maximum as it stands, without looking for the block's maximum first.  The result of softmax
      // does not depend on the reference, only overflow does: if the block's row sum is NaN, +inf or
      // above kSumHard, nothing has been stored yet and the block is redone on the exact path.
      bool exact = (j == 0) || p.rescale_tau == 0.f;
      if (!exact) {
        // Lazy rescale, one block late: move the reference when the maximum seen so far exceeds it by
        // more than tau.  The accumulator is stable here: S(j) complete implies P V (j-1) complete.
        const bool need = (m_seen - m_ref) > p.rescale_tau;
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = fmaxf(m_ref, m_seen);
          const float alpha = ex2_approx(m_ref - m_new);
          m_ref = m_new;
          l_run *= alpha;
          rescale_accumulator(tO, alpha);
        }
        const f32x2 scale2 = pack2(scale, scale), negm2 = pack2(-m_ref, -m_ref);
        f32x2 sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const f32x2 x = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, negm2);
          float x0, x1;
          unpack2(x, x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          sum2[i & 1] = add2(sum2[i & 1], pack2(p0, p1));
          if constexpr (kPrecise) {
            pack_p_precise(p0, p1, pk[i], pl[i]);
          } else {
            pk[i] = pack_p(p0, p1);
          }
        }
        float sa, sb, sc, sd;
        unpack2(sum2[0], sa, sb);
        unpack2(sum2[1], sc, sd);
        const float sum_blk = (sa + sb) + (sc + sd);
        // The block's row sum doubles as overflow guard and as estimate of the block maximum: with 128
        // keys, max x <= log2(sum) <= max x + 7.  NaN (a NaN score) and +inf (an overflow or a +inf
        // score) fail the comparison too.  No instruction of the sweep is spent on the maximum: a warp
        // cannot overlap its own special-function issue with other work, so every one counts.
        const bool bad = !(sum_blk <= kSumHard);
        if (__any_sync(0xffffffffu, bad)) {
          exact = true;
          load_scores(tS, s, valid);
        } else {
          l_run += sum_blk;
          m_seen = fmaxf(m_seen, m_ref + lg2_approx(sum_blk));
        }
      }
      if (exact) {
        // Exact path: maximum first (NaN scores ignored by the maximum, then propagated by ex2), plain
        // special-function exponentials: IEEE propagation of NaN and infinities throughout.
        const float m_blk = row_max(s) * scale;
        if (j == 0) {
          // First block of the unit: the accumulator is overwritten, nothing to rescale.
          m_ref = (m_blk == -INFINITY) ? 0.f : m_blk;
        } else {
          const bool need = (m_blk - m_ref) > p.rescale_tau;
          if (__any_sync(0xffffffffu, need)) {
            const float m_new = fmaxf(m_ref, m_blk);
            const float alpha = ex2_approx(m_ref - m_new);
            m_ref = m_new;
            l_run *= alpha;
            rescale_accumulator(tO, alpha);
            // The scores were dropped to make room for the accumulator row; fetch them again.
            load_scores(tS, s, valid);
          }
        }
        m_seen = fmaxf(m_ref, m_blk);
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(s[2 * i]), scale, -m_ref));
          const float p1 = ex2_approx(fmaf(__uint_as_float(s[2 * i + 1]), scale, -m_ref));
          sum0 += p0;
          sum1 += p1;
          if constexpr (kPrecise) {
            pack_p_precise(p0, p1, pk[i], pl[i]);
          } else {
            pk[i] = pack_p(p0, p1);
          }
        }
        l_run += sum0 + sum1;
      }
      // P overwrites the first 64 columns of S, whose scores are all in registers (or dead) by now.
      tmem_st32_at<0>(tS, pk);
      tmem_st32_at<32>(tS + 32, pk);
      if constexpr (kPrecise) {
        tmem_st32_at<0>(tS + 64, pl);
        tmem_st32_at<32>(tS + 96, pl);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
    }
    // The epilogue must have consumed the previous unit's l_ready phase before this one
    // completes; with single-block units nothing else orders the two.
    if (it > 0) MA_WAIT_WARP(bars + 8 * (kBarOFree + tile), (it - 1) & 1, 0x34 + tile);
    float* st = stats + (((it & 1) * 2 + tile) * 128 + row) * 2;
    st[0] = m_ref;
    st[1] = l_run;
    mbar_arrive(bars + 8 * (kBarLReady + tile));
  }
}

// ---------------------------------------------------------------------------
// epilogue warps (128 threads, both tiles)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void role_epilogue(const AttnParams& p, uint8_t* smem, uint32_t base, uint32_t tmem, int row,
                                              const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  const uint32_t lane_sel = static_cast<uint32_t>(row & ~31) << 16;
  const float* stats = reinterpret_cast<const float*>(smem + kOffStats);
  uint32_t it = 0;
  for (int u = blockIdx.x; u < p.total_units; u += gridDim.x, ++it) {
    const Unit un = decode_unit(p, u);
#pragma unroll 1
    for (int tile = 0; tile < 2; ++tile) {
      MA_WAIT_WARP_SLEEP(kSleepEpilogue, bars + 8 * (kBarOFull + tile), it & 1, 0x40 + tile);
      MA_WAIT_WARP(bars + 8 * (kBarLReady + tile), it & 1, 0x42 + tile);
      tc_fence_after_sync();
      const float* st = stats + (((it & 1) * 2 + tile) * 128 + row) * 2;
      const float m_ref = st[0], l_run = st[1];
      const uint32_t tO = tmem + 256 + tile * 128 + lane_sel;
      const int q_row = un.qb * kTaskRows + tile * kTileM + row;
      if (un.part < 0) {
        const float inv = 1.0f / l_run;
        const bool live = q_row < p.seq_q;
        __nv_bfloat16* dst = p.out + out_row_offset(p, un.b, un.h, live ? q_row : 0);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32_sync(tO + c * 32, o);
          if (live) store_chunk_bf16(p.round_mode, dst + c * 32, o, inv);
        }
      } else {
        const size_t prow = static_cast<size_t>(un.part) * kTaskRows + tile * kTileM + row;
        float4* dst = reinterpret_cast<float4*>(p.part_o + prow * kHeadDim);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32_sync(tO + c * 32, o);
#pragma unroll
          for (int q = 0; q < 8; ++q)
            dst[c * 8 + q] = make_float4(__uint_as_float(o[4 * q]), __uint_as_float(o[4 * q + 1]),
                                         __uint_as_float(o[4 * q + 2]), __uint_as_float(o[4 * q + 3]));
        }
        reinterpret_cast<float2*>(p.part_ml)[prow] = make_float2(m_ref, l_run);
      }
      tc_fence_before_sync();
      mbar_arrive(bars + 8 * (kBarOFree + tile));
    }
  }
}

template <bool kPrecise>
__global__ void __launch_bounds__(kThreads, 1) attn_pipelined_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const WaitCtx ctx{p.status, abort_flag};

  if (tid == 0) {
    const uint32_t bars = base + kOffBars;
    for (uint32_t i = 0; i < kNumBars; ++i) {
      const bool many = (i >= kBarPFull && i < kBarPFull + 2) || (i >= kBarOFree && i < kBarOFree + 2) ||
                        (i >= kBarLReady && i < kBarLReady + 2);
      mbar_init(bars + 8 * i, many ? 128u : 1u);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 13 && lane == 0) {
    tma_prefetch_desc(&p.tm_q);
    tma_prefetch_desc(&p.tm_k);
    tma_prefetch_desc(&p.tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < 8) {
    setmaxnreg_inc<192>();
    role_softmax<kPrecise>(p, smem, base, tmem, warp >> 2, tid & 127, ctx);
  } else if (warp < 12) {
    setmaxnreg_dec<80>();
    role_epilogue(p, smem, base, tmem, tid & 127, ctx);
  } else {
    setmaxnreg_dec<48>();
    if (warp == 12 && lane == 0) role_mma<kPrecise>(p, base, tmem, ctx);
    if (warp == 13 && lane == 0) role_producer(p, base, ctx);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, kTmemCols);
}

}  // namespace


cudaError_t launch_attn_pipelined(const AttnParams& p, int grid, bool precise_p, cudaStream_t stream) {
  auto kernel = precise_p ? attn_pipelined_kernel<true> : attn_pipelined_kernel<false>;
  cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ma
