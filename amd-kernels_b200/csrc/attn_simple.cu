// Bring-up / cross-check kernel: one CTA of 128 threads per 128-row query tile,
// everything serialised (load K,V -> S = Q K^T -> softmax -> O += P V).  It uses
// the same TMA maps, shared-memory descriptors, TMEM layouts and rounding code
// as the pipelined kernel but none of its concurrency, so a disagreement
// between the two isolates a synchronisation fault from a layout fault.
// It always tracks the exact running maximum (no lazy rescale).
#include "attn_common.cuh"
#include "attn_launch.h"

namespace ma {
namespace {

using namespace sm100;

constexpr int kSimpleThreads = 128;
constexpr int kSimpleTmemCols = 256;
constexpr uint32_t kOffQ = 0, kOffK = kTileBytes, kOffV = 2 * kTileBytes, kOffMisc = 3 * kTileBytes;
constexpr size_t kSimpleSmemBytes = 3 * kTileBytes + 64 + 1024;  // + misc + alignment slack

__global__ void __launch_bounds__(kSimpleThreads, 1) attn_simple_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sQ = base + kOffQ, sK = base + kOffK, sV = base + kOffV;
  const uint32_t bar_q = base + kOffMisc, bar_kv = bar_q + 8, bar_mma = bar_q + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffMisc + 28);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int q_tile = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.heads, h = bh % p.heads;
  const int row0 = q_tile * kTileM;
  const WaitCtx ctx{p.status, abort_flag};

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_kv, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), kSimpleTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
  const uint32_t tS = tmem_base, tO = tmem_base + 128;

  if (tid == 0) {
    mbar_arrive_expect_tx(bar_q, kTileBytes);
    tma_load_tile<kTileM>(sQ, &p.tm_q, bar_q, p.bshd, row0, h, b);
  }

  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;
  uint32_t mma_phase = 0;
  for (int j = 0; j < p.nkb && ok; ++j) {
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
      tma_load_tile<kTileN>(sK, &p.tm_k, bar_kv, p.bshd, j * kTileN, h, b);
      tma_load_tile<kTileN>(sV, &p.tm_v, bar_kv, p.bshd, j * kTileN, h, b);
    }
    if (j == 0) ok = mbar_wait_warp(bar_q, 0, 1, ctx);
    ok = ok && mbar_wait_warp(bar_kv, j & 1, 2, ctx);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (tid == 0) {
      tc_fence_after_sync();
      issue_qk<kTileN>(tS, desc_lo_kmajor(sQ), desc_lo_kmajor(sK));
      umma_commit(bar_mma);
    }
    ok = mbar_wait_warp(bar_mma, mma_phase, 3, ctx);
    mma_phase ^= 1;
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after_sync();

    // ---- softmax of this thread's row ----
    uint32_t s[4][32];
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld32(tS + lane_sel + c * 32, s[c]);
#pragma unroll
    for (int c = 0; c < 4; ++c) tmem_ld_wait32(s[c]);

    const int valid = p.seq_kv - j * kTileN;  // keys of this block that exist
    if (valid < kTileN) {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i >= valid) s[c][i] = __float_as_uint(-INFINITY);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(s[c][i]));
    const float m_new = fmaxf(m_run, mx * p.scale_log2e);
    const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = ex2_approx(m_run - m_safe);
    m_run = m_new;
    l_run *= alpha;

    if (j > 0) {  // rescale the accumulator row
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + lane_sel + c * 32, o);
        tmem_ld_wait32(o);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st32(tO + lane_sel + c * 32, o);
      }
    }

    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(s[c][2 * i]), p.scale_log2e, -m_safe));
        const float p1 = ex2_approx(fmaf(__uint_as_float(s[c][2 * i + 1]), p.scale_log2e, -m_safe));
        sum += p0 + p1;
        pk[i] = pack_p(p0, p1);
      }
      tmem_st16(tS + lane_sel + c * 16, pk);  // P overwrites the first 64 columns of S
    }
    l_run += sum;
    tmem_st_wait();
    tc_fence_before_sync();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after_sync();
      issue_pv<kTileN>(tO, tS, desc_lo_mnmajor<kTileN>(sV), j > 0);
      umma_commit(bar_mma);
    }
    ok = mbar_wait_warp(bar_mma, mma_phase, 4, ctx);
    mma_phase ^= 1;
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after_sync();
  }

  if (ok) {
    const int row = row0 + tid;
    const float inv = 1.0f / l_run;
    __nv_bfloat16* dst = p.out + out_row_offset(p, b, h, row < p.seq_q ? row : 0);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      tmem_ld32(tO + lane_sel + c * 32, o);
      tmem_ld_wait32(o);
      if (row < p.seq_q) store_chunk_bf16(p.round_mode, dst + c * 32, o, inv);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kSimpleTmemCols);
}

}  // namespace

cudaError_t launch_attn_simple(const AttnParams& p, cudaStream_t stream) {
  auto kernel = attn_simple_kernel;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSimpleSmemBytes));
  if (e != cudaSuccess) return e;
  const dim3 grid((p.seq_q + kTileM - 1) / kTileM, p.batch * p.heads);
  kernel<<<grid, kSimpleThreads, kSimpleSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace ma
