// Tail KV-split planner for a persistent grid of `num_sms` CTAs.
//
// A task is one 256-row query block of one (batch, head) slice walking all key /
// value blocks.  CTA c runs units c, c + grid, c + 2*grid, ...  When the task
// count is not a multiple of the SM count the last round leaves SMs idle; the
// planner then cuts each task of that last partial round into `split`
// contiguous key/value ranges ("parts") whose fp32 partial results a merge
// kernel combines.  Same idea and the same shape of cost model as the
// reference's plan_tail_split (csrc/attention_kernel.hip:1349-1393, constants
// :1292-1294, restated in tools/tail_speedup.py:33-73), with the constants
// re-derived for 148 SMs, 128-row key/value blocks and a schedule that is pure
// arithmetic on the unit index (no schedule table, no global state).
#pragma once

#include <cstddef>
#include <cstdint>

namespace ma {

struct TailPlan {
  int nqb;          // 256-row query blocks per (batch, head)
  int nkb;          // 128-row key/value blocks
  int tasks;        // nqb * batch * heads
  int full_units;   // tasks run whole (multiple of the grid, or all tasks when no split)
  int tail_tasks;   // tasks of the last partial round that are split (0 = no split)
  int split;        // parts per split task (1 when tail_tasks == 0)
  int total_units;  // full_units + tail_tasks * split
  int grid;         // CTAs to launch
  long long span_nosplit;  // modelled cost of the last round without / with the split, in block times
  long long span_split;
};

constexpr int kPlanTaskRows = 256;
constexpr int kPlanKvRows = 128;
constexpr int kMinKvBlocksToSplit = 8;   // below this a task is too short for a split to pay for the merge
constexpr int kMinBlocksPerPart = 2;     // floor on key/value blocks per part
constexpr int kPartOverheadBlocks = 1;   // per-part prologue + fp32 partial write, in block times
constexpr int kMergeCostBlocks = 4;      // merge launch + traffic, in block times
constexpr int kMaxSplit = 16;

inline TailPlan plan_tail(int batch, int heads, int seq_q, int seq_kv, int num_sms, bool enable_split) {
  TailPlan t{};
  t.nqb = (seq_q + kPlanTaskRows - 1) / kPlanTaskRows;
  t.nkb = (seq_kv + kPlanKvRows - 1) / kPlanKvRows;
  t.tasks = t.nqb * batch * heads;
  t.full_units = t.tasks;
  t.tail_tasks = 0;
  t.split = 1;
  t.total_units = t.tasks;
  t.grid = t.tasks < num_sms ? t.tasks : num_sms;
  t.span_nosplit = t.nkb + kPartOverheadBlocks;
  t.span_split = t.span_nosplit;

  const int tail = t.tasks % num_sms;
  if (!enable_split || tail == 0 || tail > num_sms * 19 / 20 || t.nkb < kMinKvBlocksToSplit) return t;

  int best_g = 1;
  long long best = t.span_nosplit;
  for (int g = 2; g <= kMaxSplit && t.nkb / g >= kMinBlocksPerPart; ++g) {
    const long long rounds = (static_cast<long long>(tail) * g + num_sms - 1) / num_sms;
    const long long per_part = (t.nkb + g - 1) / g + kPartOverheadBlocks;
    const long long span = rounds * per_part + kMergeCostBlocks;
    // A split must beat the unsplit last round by a margin (10 %): measured on B200, marginal
    // predictions (e.g. 108 stranded tasks of 32 blocks) lose to the extra partial traffic and merge.
    if (span < best && span * 11 < t.span_nosplit * 10) {
      best = span;
      best_g = g;
    }
  }
  if (best_g == 1) return t;
  t.full_units = t.tasks - tail;
  t.tail_tasks = tail;
  t.split = best_g;
  t.total_units = t.full_units + tail * best_g;
  t.grid = t.total_units < num_sms ? t.total_units : num_sms;
  t.span_split = best;
  return t;
}

// fp32 words one part writes: 256 rows x 128 accumulators, plus (max, sum) per row.
constexpr size_t kPartOFloats = static_cast<size_t>(kPlanTaskRows) * 128;
constexpr size_t kPartMlFloats = static_cast<size_t>(kPlanTaskRows) * 2;
constexpr size_t kStatusBytes = 256;

inline size_t plan_workspace_bytes(const TailPlan& t) {
  const size_t slots = static_cast<size_t>(t.tail_tasks) * t.split;
  return kStatusBytes + slots * (kPartOFloats + kPartMlFloats) * sizeof(float);
}

}  // namespace ma
