// Host build of the skip-list helpers the CUDA kernels use (amd-kernels_b200/csrc/lite_list.h), exported
// with C linkage so that the CPU tests can compare them with the Python restatement in oracle/lite_oracle.py.
#include "../../amd-kernels_b200/csrc/lite_list.h"

extern "C" {

// Walks `row`; writes up to `cap` (block, closes) pairs; returns the number of blocks.
int harness_walk(const int16_t* row, int phase, int* blocks, int* closes, int cap) {
  ma::ListCursor cur;
  cur.init(row, phase);
  int n = 0;
  while (cur.block >= 0 && n < cap) {
    blocks[n] = cur.block;
    closes[n] = cur.advance() ? 1 : 0;
    ++n;
  }
  return n;
}

int harness_kept(const int16_t* row, int phase) { return ma::list_kept_blocks(row, phase); }

// Emits the list for `n` processed blocks with the given votes (1 = every group skipped) and range ends.
void harness_emit(const int* blocks, const int* skips, const int* closes, int n, int width, int phase,
                  const int16_t* must_do, int16_t* out_row) {
  ma::ListEmitter e;
  e.init(out_row, phase, width);
  ma::MustDo pin;
  pin.init(must_do, phase);
  for (int i = 0; i < n; ++i) e.record(blocks[i], skips[i] != 0 && !pin.forced(blocks[i]), closes[i] != 0 || i + 1 == n);
  e.finish();
}

}  // extern "C"
