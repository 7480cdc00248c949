// Self-test of the failure path every kernel of this library shares: a bounded mbarrier wait that
// runs out, the status words it leaves, and the unwind to the common exit that frees tensor memory.
//
// Nothing faults and nothing waits for ever: the kernel waits on a barrier that by construction
// nobody arrives on, under a limit the caller chooses (a millisecond in the tests), and returns.
// The reference reports failures through return codes only (csrc/attention_kernel.hip:1573-1576,
// :1588); this library adds the device status block because its kernels synchronise through
// mbarriers, where a lost arrival would otherwise be a hang.
#include "attn_common.cuh"
#include "attn_launch.h"

namespace ma {
namespace {

using namespace sm100;

constexpr uint32_t kSelftestTmemCols = 64;

// One CTA, four warps, laid out like the attention kernels: barriers and the abort flag in shared
// memory, tensor memory allocated by one warp, roles that leave through `return` when a wait gives
// up, and a common exit that releases tensor memory.
__global__ void __launch_bounds__(128, 1) wait_timeout_kernel(uint32_t* status, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t bar_never;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  const WaitCtx ctx{status, &abort_flag, limit_ns};
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_never), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), kSelftestTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  // The roles: warp 1 waits as a whole warp (the form the softmax and epilogue warps use), one thread
  // of warp 2 waits alone (the form the MMA issuer and the TMA producer use).  Both waits must end by
  // the limit; the second usually ends early because the first has raised the abort flag.
  [&] {
    if (warp == 1) {
      if (!mbar_wait_warp<32>(smem_u32(&bar_never), 0, 0x71, ctx)) return;
      status[8] = 0xBADu;  // unreachable: the barrier never completes
    } else if (warp == 2 && (threadIdx.x & 31) == 0) {
      if (!mbar_wait(smem_u32(&bar_never), 0, 0x72, ctx)) return;
      status[8] = 0xBADu;
    }
  }();

  // common exit
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, kSelftestTmemCols);
  if (threadIdx.x == 0) status[9] = static_cast<uint32_t>(abort_flag);  // 1: the roles unwound through the abort path
}

}  // namespace

cudaError_t launch_wait_timeout_selftest(uint32_t* status, uint64_t limit_ns, cudaStream_t stream) {
  wait_timeout_kernel<<<1, 128, 0, stream>>>(status, limit_ns);
  return cudaGetLastError();
}

}  // namespace ma
