// LiteAttention forward for sm_100a: the dense kernel's pipeline driven by a skip list.
//
// Behaviour follows the reference's `isLite` kernel (csrc/attention_kernel.hip:629-716 list cursor and
// emitter, :981-1004 vote, :1056-1086 loop and final record, :1604-1681 launch) with this kernel's own tile
// geometry: a task is a 256-row query block of one (batch, head); its read-list row names the 64-key
// blocks to compute; the blocks are taken two at a time, in list order, as one 128-key tensor-core block
// (each half fetched by its own TMA box, so any two kept blocks pair up).  For every processed 64-key
// block each softmax warp (32 query rows) votes "keep" when some live row's block maximum lies within
// `threshold` (log2 units, negative) of that row's reference maximum; a warp that votes "skip" contributes
// nothing for that block, and a block every warp of the task skips is left out of the list written for
// the next call (unless the must-do list pins it).  The first processed block of a task is never skipped.
//
//   warps  0- 3  softmax of tile 0 (thread 0 also emits the write list, two steps late)
//   warps  4- 7  softmax of tile 1
//   warps  8-11  epilogue
//   warp  12     MMA issuer
//   warp  13     task fetch (atomic counter over the optional longest-first order) + TMA producer
//
// Tensor memory and the S/P aliasing are those of the dense kernel.  All waits are bounded.
#include "attn_common.cuh"
#include "attn_launch.h"
#include "lite_list.h"

namespace ma {
namespace {

using namespace sm100;

constexpr int kThreads = 512;
constexpr int kStages = 4;  // K/V ring, 32 KiB each
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSleepProducer = 128, kSleepSoftmax = 32, kSleepEpilogue = 1000;
constexpr int kTaskRing = 4;     // task descriptors in flight: producer, MMA, softmax and epilogue span < 4 tasks
// Steps whose votes are kept.  Slots are indexed by the CTA-wide step counter, not the step within a task: the
// emitter reads steps c - 2 and c - 1 while the warps it does not gate may already vote on step c of the
// next task (never c + 1: that needs the emitter's own arrival on p_full), so four slots never collide.
constexpr int kVerdictRing = 4;

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffQ = 0;                                    // 2 tiles
constexpr uint32_t kOffKV = 2 * kTileBytes;                      // kStages tiles
constexpr uint32_t kOffStats = kOffKV + kStages * kTileBytes;    // float [2 parity][2 tile][128 rows][2: max, sum]
constexpr uint32_t kOffTasks = kOffStats + 2 * 2 * 128 * 2 * 4;  // int [kTaskRing][2: task or -1, kept blocks]
constexpr uint32_t kOffVerdict = kOffTasks + kTaskRing * 8;      // uint32 [kVerdictRing][8 warps]: bit h = skip half h
constexpr uint32_t kOffBars = kOffVerdict + kVerdictRing * 8 * 4;
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
  kBarTask = kBarLReady + 2,           // [kTaskRing] producer -> everyone: task descriptor written
  kBarVotes = kBarTask + kTaskRing,    //           softmax -> list emitter: a task's votes are all in (256 arrivals)
  kNumBars = kBarVotes + 1
};
constexpr uint32_t kOffTmemSlot = kOffBars + kNumBars * 8;
constexpr uint32_t kOffAbort = kOffTmemSlot + 4;
constexpr size_t kSmemBytes = kOffAbort + 4 + 1024;  // + alignment slack


#define MA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), (site), ctx)) return
#define MA_WAIT_WARP(bar, parity, site) \
  if (!mbar_wait_warp((bar), (parity), (site), ctx)) return
#define MA_WAIT_SLEEP(ns, bar, parity, site) \
  if (!mbar_wait<ns>((bar), (parity), (site), ctx)) return
#define MA_WAIT_WARP_SLEEP(ns, bar, parity, site) \
  if (!mbar_wait_warp<ns>((bar), (parity), (site), ctx)) return

struct Task {
  int id;     // list row = (batch * heads + head) * query blocks + query block; -1: no more work
  int kept;   // 64-key blocks its read list names
  int steps;  // 128-key tensor-core blocks: ceil(kept / 2), and 1 (fully masked) when the list is empty
  int qb, b, h;
};

__device__ __forceinline__ Task decode_task(const LiteParams& p, int id, int kept) {
  Task t;
  t.id = id;
  t.kept = kept;
  t.steps = kept > 0 ? (kept + 1) >> 1 : 1;
  t.qb = id % p.a.nqb;
  const int bh = id / p.a.nqb;
  t.b = bh / p.a.heads;
  t.h = bh % p.a.heads;
  return t;
}

// Every consumer role starts a task by reading its descriptor from the ring (`WAIT` is the wait macro that
// suits the caller: whole warps or a single thread).
#define MA_NEXT_TASK(WAIT, task_var, site)                                                        \
  WAIT(bars + 8 * (kBarTask + (it % kTaskRing)), (it / kTaskRing) & 1, (site));                   \
  const int task_id_ = tasks[(it % kTaskRing) * 2], task_kept_ = tasks[(it % kTaskRing) * 2 + 1]; \
  if (task_id_ < 0) break;                                                                        \
  const Task task_var = decode_task(p, task_id_, task_kept_)

// ---------------------------------------------------------------------------
// task fetch + TMA producer (one thread)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void role_producer(const LiteParams& p, uint8_t* smem, uint32_t base, const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  volatile int* tasks = reinterpret_cast<volatile int*>(smem + kOffTasks);
  uint32_t fill = 0;  // K/V ring fills so far
  // Tasks are handed out in the order of an atomic counter, heaviest first when an order is given.  The next
  // task is fetched while the current one is being loaded, so that its latency stays off the pipeline.
  auto fetch = [&](int& id, int& kept) {
    const int slot = atomicAdd(p.counter, 1);
    id = -1;
    kept = 0;
    if (slot < p.num_tasks) {
      id = p.order != nullptr ? p.order[slot] : slot;
      kept = list_kept_blocks(p.read_list + static_cast<size_t>(id) * p.row_width, p.phase);
    }
  };
  int id, kept;
  fetch(id, kept);
  for (uint32_t it = 0;; ++it) {
    tasks[(it % kTaskRing) * 2] = id;
    tasks[(it % kTaskRing) * 2 + 1] = kept;
    mbar_arrive(bars + 8 * (kBarTask + (it % kTaskRing)));
    if (id < 0) return;
    const int16_t* row = p.read_list + static_cast<size_t>(id) * p.row_width;
    const Task t = decode_task(p, id, kept);
    const int q_row0 = t.qb * kTaskRows;
    if (it > 0) MA_WAIT_SLEEP(kSleepProducer, bars + 8 * kBarQEmpty, (it - 1) & 1, 0x10);
    mbar_arrive_expect_tx(bars + 8 * (kBarQFull + 0), kTileBytes);
    tma_load_tile<kTileM>(base + kOffQ, &p.a.tm_q, bars + 8 * (kBarQFull + 0), p.a.bshd, q_row0, t.h, t.b);
    ListCursor cur;
    cur.init(row, p.phase);
    for (int j = 0; j < t.steps; ++j) {
      // Two kept blocks per step.  A missing second block (odd count) repeats the first: its scores are
      // masked, and P = 0 against a copy of rows already in the product cannot introduce a value that is
      // not there anyway.  An empty list loads block 0 for a fully masked step whose result is discarded.
      int b0 = cur.block;
      if (b0 >= 0) {
        cur.advance();
      } else {
        b0 = 0;
      }
      int b1 = cur.block;
      if (b1 >= 0) {
        cur.advance();
      } else {
        b1 = b0;
      }
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        const uint32_t stage = fill % kStages, use = fill / kStages;
        if (use > 0) MA_WAIT_SLEEP(kSleepProducer, bars + 8 * (kBarKvEmpty + stage), (use - 1) & 1, 0x11 + kv);
        const uint32_t full = bars + 8 * (kBarKvFull + stage);
        const uint32_t dst = base + kOffKV + stage * kTileBytes;
        const CUtensorMap* tm = kv == 0 ? &p.a.tm_k : &p.a.tm_v;
        mbar_arrive_expect_tx(full, kTileBytes);
        // tile = [head-dim half][128 rows][128 bytes]; rows 0-63 from block b0, rows 64-127 from block b1
        tma_load_tile_half(dst, tm, full, p.a.bshd, 0, b0 * kLiteKeyBlock, t.h, t.b);
        tma_load_tile_half(dst + kLiteKeyBlock * 128, tm, full, p.a.bshd, 0, b1 * kLiteKeyBlock, t.h, t.b);
        tma_load_tile_half(dst + kTileN * 128, tm, full, p.a.bshd, 64, b0 * kLiteKeyBlock, t.h, t.b);
        tma_load_tile_half(dst + kTileN * 128 + kLiteKeyBlock * 128, tm, full, p.a.bshd, 64, b1 * kLiteKeyBlock, t.h, t.b);
        ++fill;
        if (kv == 0 && j == 0) {  // second Q tile right behind the first K block
          mbar_arrive_expect_tx(bars + 8 * (kBarQFull + 1), kTileBytes);
          tma_load_tile<kTileM>(base + kOffQ + kTileBytes, &p.a.tm_q, bars + 8 * (kBarQFull + 1), p.a.bshd,
                                q_row0 + kTileM, t.h, t.b);
        }
      }
      if (j == 0) {
        fetch(id, kept);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// MMA issuer (one thread): the dense kernel's order  PV0(j) QK0(j+1) PV1(j) QK1(j+1)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void role_mma(const LiteParams& p, uint8_t* smem, uint32_t base, uint32_t tmem,
                                         const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  volatile int* tasks = reinterpret_cast<volatile int*>(smem + kOffTasks);
  const uint32_t q_lo = desc_lo_kmajor(base + kOffQ);
  const uint32_t kv_lo_k = desc_lo_kmajor(base + kOffKV);
  const uint32_t kv_lo_v = desc_lo_mnmajor<kTileN>(base + kOffKV);
  constexpr uint32_t kTileLo = kTileBytes >> 4;
  uint32_t fill = 0, blk = 0;
  for (uint32_t it = 0;; ++it) {
    MA_NEXT_TASK(MA_WAIT, t, 0x2F);
    const int n = t.steps;
    {
      const uint32_t st = fill % kStages;
      MA_WAIT(bars + 8 * (kBarKvFull + st), (fill / kStages) & 1, 0x21);
      const uint32_t k_lo = kv_lo_k + st * kTileLo;
#pragma unroll 1
      for (uint32_t tl = 0; tl < 2; ++tl) {
        MA_WAIT(bars + 8 * (kBarQFull + tl), it & 1, 0x20 + tl);
        tc_fence_after_sync();
        issue_qk<kTileN>(tmem + tl * 128, q_lo + tl * kTileLo, k_lo);
        umma_commit(bars + 8 * (kBarSFull + tl));
      }
      umma_commit(bars + 8 * (kBarKvEmpty + st));
      if (n == 1) umma_commit(bars + 8 * kBarQEmpty);
    }
    for (int j = 0; j < n; ++j, ++blk) {
      const uint32_t fv = fill + 2 * j + 1, sv = fv % kStages;  // V(j)
      const uint32_t fk = fill + 2 * j + 2, sk = fk % kStages;  // K(j+1)
      const uint32_t v_lo = kv_lo_v + sv * kTileLo;
      const uint32_t k_lo = kv_lo_k + sk * kTileLo;
      const bool more = (j + 1 < n);
      MA_WAIT(bars + 8 * (kBarKvFull + sv), (fv / kStages) & 1, 0x23);
      if (more) MA_WAIT(bars + 8 * (kBarKvFull + sk), (fk / kStages) & 1, 0x26);
#pragma unroll 1
      for (uint32_t tl = 0; tl < 2; ++tl) {
        if (j == 0 && it > 0) MA_WAIT(bars + 8 * (kBarOFree + tl), (it - 1) & 1, 0x25);
        MA_WAIT(bars + 8 * (kBarPFull + tl), blk & 1, 0x24);
        tc_fence_after_sync();
        issue_pv<kTileN>(tmem + 256 + tl * 128, tmem + tl * 128, v_lo, j > 0);
        if (tl == 1) umma_commit(bars + 8 * (kBarKvEmpty + sv));
        if (more) {
          issue_qk<kTileN>(tmem + tl * 128, q_lo + tl * kTileLo, k_lo);
          umma_commit(bars + 8 * (kBarSFull + tl));
        } else {
          umma_commit(bars + 8 * (kBarOFull + tl));
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

// Maximum of 64 scores (NaN ignored, as fmaxf does).
__device__ __forceinline__ float half_max(const uint32_t* s) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    m0 = fmax3(m0, __uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
    m1 = fmax3(m1, __uint_as_float(s[16 + 2 * i]), __uint_as_float(s[16 + 2 * i + 1]));
    m2 = fmax3(m2, __uint_as_float(s[32 + 2 * i]), __uint_as_float(s[32 + 2 * i + 1]));
    m3 = fmax3(m3, __uint_as_float(s[48 + 2 * i]), __uint_as_float(s[48 + 2 * i + 1]));
  }
  return fmax3(fmaxf(m0, m1), m2, m3);
}

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

// One step of the list as the softmax threads see it.
struct StepBlocks {
  int b0, b1;    // 64-key blocks of the two halves (-1: none)
  bool e0, e1;   // the block closed its range of the read list
};

// Write-list state of the emitting thread.
struct Recorder {
  ListEmitter out;
  MustDo pin;
  __device__ __forceinline__ void step(const StepBlocks& sb, const volatile uint32_t* verdict, bool last_step) {
    // A block is left out only when every warp of the task voted "skip" (reference: vote, hip:692-701).
    uint32_t all = 3u;
#pragma unroll
    for (int w = 0; w < 8; ++w) all &= verdict[w];
    const bool has1 = sb.b1 >= 0;
    if (sb.b0 >= 0) out.record(sb.b0, (all & 1u) != 0u && !pin.forced(sb.b0), sb.e0 || (last_step && !has1));
    if (has1) out.record(sb.b1, (all & 2u) != 0u && !pin.forced(sb.b1), sb.e1 || last_step);
  }
};

// ---------------------------------------------------------------------------
// softmax warps (128 threads per tile, one query row each)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void role_softmax(const LiteParams& p, uint8_t* smem, uint32_t base, uint32_t tmem, int tile,
                                             int row, const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  volatile int* tasks = reinterpret_cast<volatile int*>(smem + kOffTasks);
  volatile uint32_t* verdict = reinterpret_cast<volatile uint32_t*>(smem + kOffVerdict);
  const uint32_t lane_sel = static_cast<uint32_t>(row & ~31) << 16;
  const uint32_t tS = tmem + tile * 128 + lane_sel;
  const uint32_t tO = tmem + 256 + tile * 128 + lane_sel;
  const uint32_t bar_s = bars + 8 * (kBarSFull + tile), bar_p = bars + 8 * (kBarPFull + tile);
  float* stats = reinterpret_cast<float*>(smem + kOffStats);
  const float scale = p.a.scale_log2e, thr = p.threshold;
  const int warp8 = tile * 4 + (row >> 5);
  const bool lane0 = (row & 31) == 0;
  const bool emits = tile == 0 && row == 0;
  uint32_t blk = 0;
  for (uint32_t it = 0;; ++it) {
    MA_NEXT_TASK(MA_WAIT_WARP, t, 0x3F);
    const int n = t.steps;
    const bool live = t.qb * kTaskRows + tile * kTileM + row < p.a.seq_q;
    ListCursor cur;
    cur.init(p.read_list + static_cast<size_t>(t.id) * p.row_width, p.phase);
    Recorder rec;
    if (emits) {
      rec.out.init(p.write_list + static_cast<size_t>(t.id) * p.row_width, p.phase, p.row_width);
      rec.pin.init(p.must_do, p.phase);
    }
    StepBlocks hist1{-1, -1, false, false}, hist2{-1, -1, false, false};  // steps j - 1 and j - 2
    float m_ref = 0.f, l_run = 0.f;
    constexpr float kSlack = 1.f / 1024.f;
    const float sum_keep = ex2_approx(thr + 6.f + kSlack);
    for (int j = 0; j < n; ++j, ++blk) {
      StepBlocks sb{-1, -1, false, false};
      sb.b0 = cur.block;
      if (sb.b0 >= 0) sb.e0 = cur.advance();
      sb.b1 = cur.block;
      if (sb.b1 >= 0) sb.e1 = cur.advance();

      MA_WAIT_WARP_SLEEP(kSleepSoftmax, bar_s, blk & 1, 0x30 + tile);
      tc_fence_after_sync();

      uint32_t s[128];
      tmem_ld128_sync(tS, s);
      // keys of each half that exist (the last block of the sequence may be ragged; a half may be absent)
      const int valid0 = sb.b0 >= 0 ? p.a.seq_kv - sb.b0 * kLiteKeyBlock : 0;
      const int valid1 = sb.b1 >= 0 ? p.a.seq_kv - sb.b1 * kLiteKeyBlock : 0;
      if (valid0 < kLiteKeyBlock || valid1 < kLiteKeyBlock) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          if (i >= valid0) s[i] = __float_as_uint(-INFINITY);
          if (i >= valid1) s[64 + i] = __float_as_uint(-INFINITY);
        }
      }
      const bool first = j == 0;
      uint32_t pk[64];
      bool exact = first;
      if (!first) {
        // Speculative sweep, as in the dense kernel: exponentiate against the reference maximum as it stands and
        // read the votes off the two half sums instead of looking for the half maxima first.  With 64 keys,
        // max <= log2(sum) <= max + 6 (all in units relative to the reference), so
        //   log2(sum) > threshold + 6  : this row's maximum is above the threshold  ->  the vote is "keep",
        // exactly what the exact maxima would give.  A half no row is certain about, a sum that might move the
        // reference maximum (> 2^tau), or a NaN / inf, sends the warp to the exact path below; nothing has been
        // stored by then.
        const f32x2 scale2 = pack2(scale, scale), negm2 = pack2(-m_ref, -m_ref);
        f32x2 sum2[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};  // two per half
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const f32x2 x = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, negm2);
          float x0, x1;
          unpack2(x, x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          sum2[(i >> 5) * 2 + (i & 1)] = add2(sum2[(i >> 5) * 2 + (i & 1)], pack2(p0, p1));
          pk[i] = pack_p(p0, p1);
        }
        float sa, sb2, sc, sd;
        unpack2(add2(sum2[0], sum2[1]), sa, sb2);
        unpack2(add2(sum2[2], sum2[3]), sc, sd);
        const float sum_h0 = sa + sb2, sum_h1 = sc + sd;
        // The threshold is compared in the linear domain: log2(sum) > t  <=>  sum > 2^t (computed once per task;
        // 2^-1000 is 0, so "sum > 0" then).  kSlack covers what the approximate exponentials and the fp32 sums
        // can be off.
        const bool moves = !(sum_h0 + sum_h1 <= 255.f);  // the block maximum may exceed the reference by tau = 8 (or NaN)
        uint32_t bits = moves ? 16u : 0u;
        if (live) bits |= (sum_h0 > sum_keep ? 1u : 0u) | (sb.b1 >= 0 && sum_h1 > sum_keep ? 4u : 0u);
        bits = __reduce_or_sync(0xffffffffu, bits);
        // The sweep's result stands only when every half that exists is certainly kept: a half some warp skips
        // has to be taken out of P and of the row sum, which the exact path below does (it is the rarer case: a
        // skipped block leaves the list).  An absent second half has scores of -inf, p = 0 and sum 0 already.
        const bool keep0 = (bits & 1u) != 0u, keep1 = (bits & 4u) != 0u;
        if ((bits & 16u) != 0u || !keep0 || (!keep1 && sb.b1 >= 0)) {
          exact = true;
          tmem_ld128_sync(tS, s);
          if (valid0 < kLiteKeyBlock || valid1 < kLiteKeyBlock) {
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if (i >= valid0) s[i] = __float_as_uint(-INFINITY);
              if (i >= valid1) s[64 + i] = __float_as_uint(-INFINITY);
            }
          }
        } else {
          if (lane0) verdict[(blk % kVerdictRing) * 8 + warp8] = keep1 ? 0u : 2u;
          l_run += sum_h0 + sum_h1;
        }
      }
      if (exact) {
        const float m0 = half_max(s) * scale, m1 = half_max(s + 64) * scale;

        // Votes (reference: hip:981-993).  The first processed block of a task is always kept; its successor in
        // the same step is judged against the maximum the first block establishes.
        const float ref1 = first ? ((m0 == -INFINITY) ? 0.f : m0) : m_ref;
        const bool want0 = live && (m0 - m_ref) > thr;
        const bool want1 = live && sb.b1 >= 0 && (m1 - ref1) > thr;
        const bool keep0 = first || __any_sync(0xffffffffu, want0);
        const bool keep1 = __any_sync(0xffffffffu, want1);
        if (lane0) verdict[(blk % kVerdictRing) * 8 + warp8] = (keep0 ? 0u : 1u) | (keep1 ? 0u : 2u);
        if (!keep0 || !keep1) {
          // A skipping warp contributes nothing for the block and its state does not see it.
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            if (!keep0) s[i] = __float_as_uint(-INFINITY);
            if (!keep1) s[64 + i] = __float_as_uint(-INFINITY);
          }
        }
        const float m_blk = fmaxf(keep0 ? m0 : -INFINITY, keep1 ? m1 : -INFINITY);
        if (first) {
          m_ref = (m_blk == -INFINITY) ? 0.f : m_blk;
        } else {
          const bool need = (m_blk - m_ref) > p.a.rescale_tau;
          if (__any_sync(0xffffffffu, need)) {
            const float m_new = fmaxf(m_ref, m_blk);
            const float alpha = ex2_approx(m_ref - m_new);
            m_ref = m_new;
            l_run *= alpha;
            rescale_accumulator(tO, alpha);
          }
        }
        // p = 2^(s * scale - m_ref), two keys per FMA / add instruction; the row sum uses the unrounded values
        const f32x2 scale2 = pack2(scale, scale), negm2 = pack2(-m_ref, -m_ref);
        f32x2 sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const f32x2 x = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, negm2);
          float x0, x1;
          unpack2(x, x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          sum2[i & 1] = add2(sum2[i & 1], pack2(p0, p1));
          pk[i] = pack_p(p0, p1);
        }
        float sa, sb2, sc, sd;
        unpack2(sum2[0], sa, sb2);
        unpack2(sum2[1], sc, sd);
        l_run += (sa + sb2) + (sc + sd);
      }
      tmem_st32_at<0>(tS, pk);
      tmem_st32_at<32>(tS + 32, pk);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(bar_p);
      // The list entry of step j - 2, written off the critical path (the thread has until the next S arrives).
      // S(j) of tile 0 followed P V (j-1) of tile 0 in the MMA order, which followed P V (j-2) of tile 1: every
      // warp's votes of step j - 2 are in shared memory, and no warp can be at step j + 2 yet (that needs this
      // tile's P of step j + 1), so the slot has not been reused.
      if (emits && j >= 2) rec.step(hist2, verdict + ((blk - 2) % kVerdictRing) * 8, false);
      hist2 = hist1;
      hist1 = sb;
    }
    // One phase of the votes barrier per task: it completes when all 256 softmax threads have cast their
    // last vote of this task, and cannot run ahead (the next phase needs the emitter's own arrival).
    mbar_arrive(bars + 8 * kBarVotes);
    if (emits && t.kept > 0) {
      MA_WAIT(bars + 8 * kBarVotes, it & 1, 0x38);
      if (n >= 2) rec.step(hist2, verdict + ((blk - 2) % kVerdictRing) * 8, false);
      rec.step(hist1, verdict + ((blk - 1) % kVerdictRing) * 8, true);
      rec.out.finish();
    }
    // The epilogue must have consumed the previous task's l_ready phase before this one completes.
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
__device__ __forceinline__ void role_epilogue(const LiteParams& p, uint8_t* smem, uint32_t base, uint32_t tmem, int row,
                                              const WaitCtx& ctx) {
  const uint32_t bars = base + kOffBars;
  volatile int* tasks = reinterpret_cast<volatile int*>(smem + kOffTasks);
  const uint32_t lane_sel = static_cast<uint32_t>(row & ~31) << 16;
  const float* stats = reinterpret_cast<const float*>(smem + kOffStats);
  for (uint32_t it = 0;; ++it) {
    MA_NEXT_TASK(MA_WAIT_WARP, t, 0x4F);
#pragma unroll 1
    for (int tile = 0; tile < 2; ++tile) {
      MA_WAIT_WARP_SLEEP(kSleepEpilogue, bars + 8 * (kBarOFull + tile), it & 1, 0x40 + tile);
      MA_WAIT_WARP(bars + 8 * (kBarLReady + tile), it & 1, 0x42 + tile);
      tc_fence_after_sync();
      const float* st = stats + (((it & 1) * 2 + tile) * 128 + row) * 2;
      const float l_run = st[1];
      const uint32_t tO = tmem + 256 + tile * 128 + lane_sel;
      const int q_row = t.qb * kTaskRows + tile * kTileM + row;
      // An empty read list computes nothing: the output rows are zero (reference: inv_sum = 0, hip:1088-1090).
      const float inv = t.kept > 0 ? 1.0f / l_run : 0.f;
      const bool live = q_row < p.a.seq_q;
      __nv_bfloat16* dst = p.a.out + out_row_offset(p.a, t.b, t.h, live ? q_row : 0);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32_sync(tO + c * 32, o);
        if (t.kept == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (live) store_chunk_bf16(p.a.round_mode, dst + c * 32, o, inv);
      }
      tc_fence_before_sync();
      mbar_arrive(bars + 8 * (kBarOFree + tile));
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) attn_lite_kernel(const __grid_constant__ LiteParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = smem_u32(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffTmemSlot);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const WaitCtx ctx{p.a.status, abort_flag};

  if (tid == 0) {
    const uint32_t bars = base + kOffBars;
    for (uint32_t i = 0; i < kNumBars; ++i) {
      const bool many = (i >= kBarPFull && i < kBarPFull + 2) || (i >= kBarOFree && i < kBarOFree + 2) ||
                        (i >= kBarLReady && i < kBarLReady + 2);
      mbar_init(bars + 8 * i, i == kBarVotes ? 256u : (many ? 128u : 1u));
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 12) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 13 && lane == 0) {
    tma_prefetch_desc(&p.a.tm_q);
    tma_prefetch_desc(&p.a.tm_k);
    tma_prefetch_desc(&p.a.tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp < 8) {
    setmaxnreg_inc<192>();
    role_softmax(p, smem, base, tmem, warp >> 2, tid & 127, ctx);
  } else if (warp < 12) {
    setmaxnreg_dec<80>();
    role_epilogue(p, smem, base, tmem, tid & 127, ctx);
  } else {
    setmaxnreg_dec<48>();
    if (warp == 12 && lane == 0) role_mma(p, smem, base, tmem, ctx);
    if (warp == 13 && lane == 0) role_producer(p, smem, base, ctx);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, kTmemCols);
}

// ---------------------------------------------------------------------------
// Longest-first task order (reference: plan_lite_order, hip:1296-1347): a counting sort of the tasks by
// the number of key blocks their read list keeps, 256 buckets, heaviest bucket first.  The order only
// changes which CTA runs a task and when; every task's result is the same.  Also resets the task counter.
// ---------------------------------------------------------------------------
constexpr int kWorkBuckets = 256;

__global__ void __launch_bounds__(256, 1) lite_order_kernel(const int16_t* __restrict__ read_list, int* __restrict__ order,
                                                             int* __restrict__ counter, int num_tasks, int row_width,
                                                             int key_blocks, int phase) {
  __shared__ int count[kWorkBuckets];
  __shared__ int slot[kWorkBuckets];
  for (int b = threadIdx.x; b < kWorkBuckets; b += blockDim.x) count[b] = 0;
  if (threadIdx.x == 0) *counter = 0;
  __syncthreads();
  auto bucket_of = [&](int task) {
    const int kept = list_kept_blocks(read_list + static_cast<size_t>(task) * row_width, phase);
    const long long b = static_cast<long long>(kept) * kWorkBuckets / (key_blocks + 1);
    return static_cast<int>(b < kWorkBuckets ? b : kWorkBuckets - 1);
  };
  for (int task = threadIdx.x; task < num_tasks; task += blockDim.x) atomicAdd(&count[bucket_of(task)], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int b = kWorkBuckets - 1; b >= 0; --b) {
      slot[b] = s;
      s += count[b];
    }
  }
  __syncthreads();
  for (int task = threadIdx.x; task < num_tasks; task += blockDim.x) order[atomicAdd(&slot[bucket_of(task)], 1)] = task;
}

}  // namespace

cudaError_t launch_lite_order(const LiteParams& p, int* order, cudaStream_t stream) {
  lite_order_kernel<<<1, 256, 0, stream>>>(p.read_list, order, p.counter, p.num_tasks, p.row_width, p.row_width - 2,
                                           p.phase);
  return cudaGetLastError();
}


cudaError_t launch_attn_lite(const LiteParams& p, int grid, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(attn_lite_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes));
  if (e != cudaSuccess) return e;
  attn_lite_kernel<<<grid, kThreads, kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ma
