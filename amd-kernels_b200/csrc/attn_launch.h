// Host-side declarations shared by the C-ABI translation unit and the kernel
// translation units.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

#include "tail_plan.h"

namespace ma {

struct AttnParams;
struct LiteParams;
struct MlaParams;

// One CTA per 128-row query tile, fully serialised (cross-check kernel).
cudaError_t launch_attn_simple(const AttnParams& p, cudaStream_t stream);

// Persistent warp-specialised kernel; `grid` CTAs walk the unit list of the plan.
// `precise_p`: feed the probabilities to the second MMA as a sum of two bf16 terms (MA_FLAG_PRECISE_P).
cudaError_t launch_attn_pipelined(const AttnParams& p, int grid, bool precise_p, cudaStream_t stream);

// Combines the partial results of KV-split tasks into the bf16 output.
cudaError_t launch_merge_parts(const AttnParams& p, cudaStream_t stream);

// LiteAttention: the skip-list driven kernel, and the kernel that sorts its tasks longest-first into `order`
// (and zeroes the hand-out counter).
cudaError_t launch_attn_lite(const LiteParams& p, int grid, cudaStream_t stream);
cudaError_t launch_lite_order(const LiteParams& p, int* order, cudaStream_t stream);

// MLA absorbed decode: one CTA per (request, group of draft positions, KV part), then the merge of the parts.
cudaError_t launch_mla_decode(const MlaParams& p, cudaStream_t stream);
// Clusters of `parts` decode CTAs (2..8) that the current device holds at once; 0: no such cluster.  A request's
// parts are launched as one cluster, and merged through shared memory, while batch x groups is within this.
int mla_cluster_capacity(int pos_per_cta, bool slab, int parts);

// One CTA that waits, under `limit_ns`, on a barrier nobody arrives on: exercises the time-out branch of the
// bounded waits, the status words and the unwind that frees tensor memory.  `status`: 64 zeroed words.
cudaError_t launch_wait_timeout_selftest(uint32_t* status, uint64_t limit_ns, cudaStream_t stream);

// dst[i] = bf16(src[i]) with the given rounding mode (device pointers); exposes the
// epilogue's rounding code for exhaustive bit-pattern tests.
cudaError_t launch_round_bf16(const float* src, uint16_t* dst, size_t n, int round_mode, cudaStream_t stream);

}  // namespace ma
