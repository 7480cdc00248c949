// Small memory-bound kernels beside the attention kernels:
//  * merge_parts: combines the fp32 partial results of KV-split tasks
//    (same formulae as the reference's merge_parts, csrc/attention_kernel.hip:1242-1279);
//  * round_bf16: applies the epilogue's fp32 -> bf16 rounding rules to an array,
//    so that tests can sweep bit patterns through the exact device code.
#include "attn_common.cuh"
#include "attn_launch.h"

namespace ma {
namespace {

constexpr int kMergeThreads = 256;   // 8 rows x 32 threads, 4 head-dim values per thread
constexpr int kMergeRowsPerBlock = 8;

template <int kMode>
__global__ void __launch_bounds__(kMergeThreads) merge_parts_kernel(const __grid_constant__ AttnParams p) {
  const int blocks_per_task = kTaskRows / kMergeRowsPerBlock;
  const int tail_task = blockIdx.x / blocks_per_task;
  const int row = (blockIdx.x % blocks_per_task) * kMergeRowsPerBlock + (threadIdx.x >> 5);
  const int c4 = threadIdx.x & 31;
  const int task = p.full_units + tail_task;
  const int qb = task % p.nqb, bh = task / p.nqb;
  const int q_row = qb * kTaskRows + row;
  if (q_row >= p.seq_q) return;

  const size_t slot0 = static_cast<size_t>(tail_task) * p.split;
  const float2* ml = reinterpret_cast<const float2*>(p.part_ml);
  float m_max = -INFINITY;
  for (int g = 0; g < p.split; ++g) m_max = fmaxf(m_max, ml[(slot0 + g) * kTaskRows + row].x);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float den = 0.f;
  for (int g = 0; g < p.split; ++g) {
    const size_t prow = (slot0 + g) * kTaskRows + row;
    const float2 st = ml[prow];
    const float w = ex2_approx(st.x - m_max);
    const float4 o = reinterpret_cast<const float4*>(p.part_o + prow * kHeadDim)[c4];
    acc.x = fmaf(w, o.x, acc.x);
    acc.y = fmaf(w, o.y, acc.y);
    acc.z = fmaf(w, o.z, acc.z);
    acc.w = fmaf(w, o.w, acc.w);
    den = fmaf(w, st.y, den);
  }
  const float inv = 1.0f / den;
  uint2 w2;
  w2.x = bf16_pack2<kMode>(acc.x * inv, acc.y * inv);
  w2.y = bf16_pack2<kMode>(acc.z * inv, acc.w * inv);
  __nv_bfloat16* dst = p.out + out_row_offset(p, bh / p.heads, bh % p.heads, q_row) + c4 * 4;
  *reinterpret_cast<uint2*>(dst) = w2;
}

template <int kMode>
__global__ void round_bf16_kernel(const float* __restrict__ src, uint16_t* __restrict__ dst, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = static_cast<uint16_t>(bf16_bits<kMode>(src[i]));
}

}  // namespace

cudaError_t launch_merge_parts(const AttnParams& p, cudaStream_t stream) {
  if (p.tail_tasks <= 0) return cudaSuccess;
  const int grid = p.tail_tasks * (kTaskRows / kMergeRowsPerBlock);
  if (p.round_mode == kRTNE) {
    merge_parts_kernel<kRTNE><<<grid, kMergeThreads, 0, stream>>>(p);
  } else if (p.round_mode == kRTNA) {
    merge_parts_kernel<kRTNA><<<grid, kMergeThreads, 0, stream>>>(p);
  } else {
    merge_parts_kernel<kRTZ><<<grid, kMergeThreads, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

cudaError_t launch_round_bf16(const float* src, uint16_t* dst, size_t n, int round_mode, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int threads = 256;
  size_t blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (round_mode == kRTNE) {
    round_bf16_kernel<kRTNE><<<static_cast<int>(blocks), threads, 0, stream>>>(src, dst, n);
  } else if (round_mode == kRTNA) {
    round_bf16_kernel<kRTNA><<<static_cast<int>(blocks), threads, 0, stream>>>(src, dst, n);
  } else {
    round_bf16_kernel<kRTZ><<<static_cast<int>(blocks), threads, 0, stream>>>(src, dst, n);
  }
  return cudaGetLastError();
}

}  // namespace ma
