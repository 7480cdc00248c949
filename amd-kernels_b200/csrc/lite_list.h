// LiteAttention skip lists: the run-length format the reference kernel reads and writes
// (csrc/attention_kernel.hip:629-716; moonmath_attention/lite.py:108-128), restated for host and device.
//
// One row of int16 per (batch, head, query block): [len, m_1, ..., m_len], row width = key blocks + 2.
// The markers are read from the back, in pairs: the range that starts at m_i + step and ends before
// m_(i-1) + step, for i = len, len - 2, ..., where step = +1 when `phase` is 1 (blocks walked upwards) and
// -1 when it is 0 (downwards).  A kernel call walks the read row in its direction and writes, in that same
// order, the markers of the blocks it wants computed next time; the next call reads that row from the back
// in the opposite direction, so the two directions alternate from call to call.
// The compute-all seed for a first call with phase 1 is [2, key_blocks - 1, -1].
//
// A key block here is 64 keys (the reference's KvBlockRows), whatever the tensor-core tile of the kernel.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define MA_HD __host__ __device__ __forceinline__
#else
#define MA_HD inline
#endif

namespace ma {

constexpr int kLiteKeyBlock = 64;     // keys per skip-list block
constexpr int kLiteQueryBlock = 256;  // query rows per skip-list row (one CTA task)
constexpr int kLiteVoteRows = 32;     // query rows that vote together (one warp)

// Read cursor over one row (reference: open_range / next_kept, hip:645-664).
struct ListCursor {
  const int16_t* row;
  int step;   // +1 / -1
  int idx;    // next marker pair
  int block;  // current block, -1 when exhausted
  int end;    // exclusive end of the current range, in walk direction

  MA_HD void open() {
    block = static_cast<int>(row[idx]) + step;
    end = static_cast<int>(row[idx - 1]) + step;
    idx -= 2;
  }
  MA_HD void init(const int16_t* r, int phase) {
    row = r;
    step = phase ? 1 : -1;
    idx = static_cast<int>(r[0]);
    block = -1;
    end = 0;
    if (idx >= 2) open();
  }
  // Moves to the next kept block; returns true when the block just left was the last of its range.
  MA_HD bool advance() {
    const int next = block + step;
    if (step > 0 ? next < end : next > end) {
      block = next;
      return false;
    }
    if (idx >= 2) {
      open();
    } else {
      block = -1;
    }
    return true;
  }
};

// Blocks a cursor over this row will yield (every pair yields at least its first block, as the walk does).
MA_HD int list_kept_blocks(const int16_t* row, int phase) {
  const int step = phase ? 1 : -1;
  int kept = 0;
  for (int i = static_cast<int>(row[0]); i >= 2; i -= 2) {
    const int first = static_cast<int>(row[i]) + step, end = static_cast<int>(row[i - 1]) + step;
    const int n = step > 0 ? end - first : first - end;
    kept += n > 1 ? n : 1;
  }
  return kept;
}

// Global force-compute ranges [len, s0, e0, s1, e1, ...] ([s, e) key blocks), walked monotonically in the
// direction of the call (reference: md_force, hip:676-691).  Null or len 0: nothing is forced.
struct MustDo {
  const int16_t* list;
  int step, ranges, cur;
  MA_HD void init(const int16_t* l, int phase) {
    list = l;
    step = phase ? 1 : -1;
    ranges = (l != nullptr && static_cast<int>(l[0]) > 0) ? (static_cast<int>(l[0]) >> 1) : 0;
    cur = step > 0 ? 0 : ranges - 1;
  }
  MA_HD bool forced(int block) {
    if (ranges == 0) return false;
    if (step > 0) {
      while (cur < ranges && block >= static_cast<int>(list[2 + 2 * cur])) ++cur;
    } else {
      while (cur >= 0 && block < static_cast<int>(list[1 + 2 * cur])) --cur;
    }
    return cur >= 0 && cur < ranges && block >= static_cast<int>(list[1 + 2 * cur]) &&
           block < static_cast<int>(list[2 + 2 * cur]);
  }
};

// Write-list emitter (reference: record, hip:703-713, and the final length store, hip:1081-1084):
// a marker at every change between "skip" and "compute", and a closing marker when a range of the
// read list ends while computing.
struct ListEmitter {
  int16_t* row;
  int step;
  int idx;     // next slot (slot 0 receives the length)
  int width;   // slots of the row (key blocks + 2); a well-formed read list never produces more markers
  bool skip;   // running state
  MA_HD void init(int16_t* r, int phase, int row_width) {
    row = r;
    step = phase ? 1 : -1;
    idx = 1;
    width = row_width;
    skip = true;
  }
  MA_HD void put(int marker) {
    if (idx < width) row[idx++] = static_cast<int16_t>(marker);  // overlapping ranges of a malformed list: drop
  }
  MA_HD void record(int block, bool skip_block, bool range_end) {
    if (skip_block != skip) {
      put(block);
      skip = skip_block;
    }
    if (range_end) {
      skip = true;
      if (!skip_block) put(block + step);
    }
  }
  MA_HD void finish() { row[0] = static_cast<int16_t>(idx - 1); }
};

}  // namespace ma
