// C ABI of the library (declared in include/moonmath_attention.h): argument
// checks, tensor maps, tail plan, kernel launches.  Keeps no state between
// calls apart from the lazily resolved driver entry point and, for
// ma_attention_forward_static only, the static scratch array and its cached
// per-device address.
#include <cmath>
#include <cstring>
#include <mutex>

#include "../../include/moonmath_attention.h"
#include "attn_common.cuh"
#include "attn_launch.h"
#include "lite_list.h"

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Rank-4 map over a contiguous bf16 tensor, rows of 128 head-dim elements.
// The sequence axis is a dimension of its own, so a box that runs past the end
// of a sequence reads zeros instead of the next head or batch.
int make_tensor_map(CUtensorMap* tm, const void* ptr, int batch, int heads, int seq, int bshd, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return MA_ERR_DRIVER;
  const cuuint64_t row = ma::kHeadDim * 2;  // bytes
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
  if (bshd) {  // [B, S, H, D]
    dims[0] = ma::kHeadDim, dims[1] = heads, dims[2] = seq, dims[3] = batch;
    strides[0] = row, strides[1] = row * heads, strides[2] = row * heads * seq;
    box[0] = 64, box[1] = 1, box[2] = box_rows, box[3] = 1;
  } else {  // [B, H, S, D]
    dims[0] = ma::kHeadDim, dims[1] = seq, dims[2] = heads, dims[3] = batch;
    strides[0] = row, strides[1] = row * seq, strides[2] = row * seq * heads;
    box[0] = 64, box[1] = box_rows, box[2] = 1, box[3] = 1;
  }
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MA_OK : MA_ERR_TENSOR_MAP;
}

// Rank-3 byte map over a contiguous MLA cache slab [batch][seq][576]: box = one 128-byte column chunk of 96 token
// rows; rows past `seq` and bytes past 576 read as zeros.
// Box of `width` byte columns x 96 token rows of a [batch][seq][576 B] slab; 128 wide under the 128-byte swizzle
// (latent chunks), 64 wide under the 64-byte swizzle (rope chunk).
int make_kv_slab_map(CUtensorMap* tm, const void* ptr, int batch, int seq, int width) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return MA_ERR_DRIVER;
  const cuuint64_t dims[3] = {576, static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch)};
  const cuuint64_t strides[2] = {576, static_cast<cuuint64_t>(576) * seq};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(width), 96, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, width == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MA_OK : MA_ERR_TENSOR_MAP;
}

int cuda_rc(cudaError_t e) { return e == cudaSuccess ? MA_OK : MA_ERR_CUDA_BASE + static_cast<int>(e); }

// Flag bits each entry point understands; anything else is refused rather than ignored.
constexpr int kForwardFlags = MA_FLAG_NO_TAIL | MA_FLAG_SIMPLE | MA_FLAG_EXACT_MAX | MA_FLAG_PRECISE_P;
constexpr int kLiteFlags = MA_FLAG_LITE_PLAIN;

int check_dims(int batch, int heads, int seq_len, int seq_len_kv) {
  if (batch <= 0 || heads <= 0) return MA_ERR_BATCH_HEADS;
  if (seq_len <= 0) return MA_ERR_SEQ_Q;
  if (seq_len_kv <= 0) return MA_ERR_SEQ_KV;
  // Unit indices and grid.y are 32-bit / 16-bit quantities.
  const long long bh = static_cast<long long>(batch) * heads;
  const long long tasks = bh * ((seq_len + ma::kPlanTaskRows - 1) / ma::kPlanTaskRows);
  if (bh > 65535 || tasks > (1ll << 30)) return MA_ERR_TOO_LARGE;
  return MA_OK;
}

// Scratch of ma_attention_forward_static: lives in the library image, so no call ever allocates it.
// Every device that loads the library holds one copy until the process exits.
constexpr size_t kStaticScratchBytes = MA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_addr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
int static_scratch_address(int dev, void** out) {
  if (dev < 0 || dev >= kMaxDevices) return MA_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_addr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_rc(e);
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255u)) return MA_ERR_WORKSPACE;
    g_static_addr[dev] = ptr;
  }
  *out = g_static_addr[dev];
  return MA_OK;
}

// Forgets the cached address of a device, so that the next call asks the runtime again.  Called when a
// launch through the cached address failed: after cudaDeviceReset the old address is stale.
void forget_static_scratch_address(int dev) {
  if (dev < 0 || dev >= kMaxDevices) return;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  g_static_addr[dev] = nullptr;
}

int resolve_sms(int num_sms) {
  if (num_sms > 0) return num_sms;
  return ma_device_sms();
}

}  // namespace

extern "C" {

int ma_abi_version(void) { return MA_ABI_VERSION; }

const char* ma_error_string(int rc) {
  switch (rc) {
    case MA_OK: return "ok";
    case MA_ERR_BATCH_HEADS: return "batch and heads must be positive";
    case MA_ERR_SEQ_Q: return "seq_len must be positive";
    case MA_ERR_HEAD_DIM: return "head_dim must be 128";
    case MA_ERR_LISTS: return "read_list and write_list must not be null";
    case MA_ERR_SEQ_KV: return "seq_len_kv must be positive";
    case MA_ERR_PLAN: return "tail plan could not be set up";
    case MA_ERR_LAYOUT: return "layout must be 0 (bhsd) or 1 (bshd)";
    case MA_ERR_ROUND_MODE: return "round_mode must be 0 (rtne), 1 (rtna) or 2 (rtz)";
    case MA_ERR_NULL_POINTER: return "q, k, v and out must not be null";
    case MA_ERR_ALIGNMENT: return "q, k, v and out must be 16-byte aligned";
    case MA_ERR_WORKSPACE: return "workspace too small or not 256-byte aligned";
    case MA_ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected a tensor";
    case MA_ERR_DRIVER: return "cuTensorMapEncodeTiled not found in the driver";
    case MA_ERR_DEVICE: return "current CUDA device is not an sm_100 GPU";
    case MA_ERR_TOO_LARGE: return "problem exceeds the kernel's index range";
    case MA_ERR_LITE_ARGS: return "threshold must be negative, phase 0 or 1, at most 32766 key blocks of 64";
    case MA_ERR_MLA_ARGS: return "parts must be in [1, MA_MLA_MAX_PARTS], kv_format 0 (e4m3-fnuz) or 1 (e4m3)";
    case MA_ERR_FLAGS: return "flags holds a bit this entry point does not define";
    case MA_ERR_STATIC_SCRATCH:
      return "problem needs more scratch than the built-in static buffer holds (pass MA_FLAG_NO_TAIL or use "
             "ma_attention_forward with a workspace)";
    default: return rc >= MA_ERR_CUDA_BASE ? "CUDA runtime error (code - 1000 is the cudaError_t)" : "unknown error";
  }
}

int ma_device_sms(void) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return -(MA_ERR_CUDA_BASE + static_cast<int>(e));
  return sms;
}

size_t ma_workspace_bytes(int batch, int heads, int seq_len, int seq_len_kv, int num_sms, int flags) {
  if (check_dims(batch, heads, seq_len, seq_len_kv) != MA_OK) return ma::kStatusBytes;
  const int sms = resolve_sms(num_sms);
  if (sms <= 0) return ma::kStatusBytes;
  const bool split = !(flags & (MA_FLAG_NO_TAIL | MA_FLAG_SIMPLE));
  return ma::plan_workspace_bytes(ma::plan_tail(batch, heads, seq_len, seq_len_kv, sms, split));
}

int ma_plan_tail(int batch, int heads, int seq_len, int seq_len_kv, int num_sms, int flags, int plan[8]) {
  if (plan == nullptr) return MA_ERR_NULL_POINTER;
  const int rc = check_dims(batch, heads, seq_len, seq_len_kv);
  if (rc != MA_OK) return rc;
  const int sms = resolve_sms(num_sms);
  if (sms <= 0) return sms < 0 ? -sms : MA_ERR_PLAN;
  const bool split = !(flags & (MA_FLAG_NO_TAIL | MA_FLAG_SIMPLE));
  const ma::TailPlan t = ma::plan_tail(batch, heads, seq_len, seq_len_kv, sms, split);
  plan[0] = t.tasks, plan[1] = t.full_units, plan[2] = t.tail_tasks, plan[3] = t.split;
  plan[4] = t.total_units, plan[5] = t.grid, plan[6] = t.nqb, plan[7] = t.nkb;
  return MA_OK;
}

int ma_attention_forward(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                         int seq_len_kv, int head_dim, int layout, int round_mode, void* workspace,
                         size_t workspace_bytes, int flags, void* stream_) {
  int rc = check_dims(batch, heads, seq_len, seq_len_kv);
  if (rc != MA_OK) return rc;
  if (head_dim != ma::kHeadDim) return MA_ERR_HEAD_DIM;
  if (layout != MA_LAYOUT_BHSD && layout != MA_LAYOUT_BSHD) return MA_ERR_LAYOUT;
  if (round_mode < MA_ROUND_RTNE || round_mode > MA_ROUND_RTZ) return MA_ERR_ROUND_MODE;
  if (flags & ~kForwardFlags) return MA_ERR_FLAGS;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return MA_ERR_NULL_POINTER;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                         reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out);
  if (bits & 15u) return MA_ERR_ALIGNMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  int dev = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (major != 10) return MA_ERR_DEVICE;

  const bool want_split = workspace != nullptr && !(flags & (MA_FLAG_NO_TAIL | MA_FLAG_SIMPLE));
  const ma::TailPlan plan = ma::plan_tail(batch, heads, seq_len, seq_len_kv, sms, want_split);
  if (plan.total_units <= 0 || plan.grid <= 0) return MA_ERR_PLAN;
  if (workspace != nullptr) {
    if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < ma::plan_workspace_bytes(plan))
      return MA_ERR_WORKSPACE;
  }

  ma::AttnParams p;
  std::memset(&p, 0, sizeof(p));
  const bool simple = (flags & MA_FLAG_SIMPLE) != 0;
  const int kv_rows = ma::kTileN;
  rc = make_tensor_map(&p.tm_q, q, batch, heads, seq_len, layout, ma::kTileM);
  if (rc == MA_OK) rc = make_tensor_map(&p.tm_k, k, batch, heads, seq_len_kv, layout, kv_rows);
  if (rc == MA_OK) rc = make_tensor_map(&p.tm_v, v, batch, heads, seq_len_kv, layout, kv_rows);
  if (rc != MA_OK) return rc;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = static_cast<uint32_t*>(workspace);
  if (workspace != nullptr) {
    float* parts = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ma::kStatusBytes);
    const size_t slots = static_cast<size_t>(plan.tail_tasks) * plan.split;
    p.part_o = parts;
    p.part_ml = parts + slots * ma::kPartOFloats;
  }
  p.batch = batch, p.heads = heads, p.seq_q = seq_len, p.seq_kv = seq_len_kv;
  p.bshd = layout, p.round_mode = round_mode;
  p.nqb = plan.nqb, p.nkb = plan.nkb;
  p.full_units = plan.full_units, p.tail_tasks = plan.tail_tasks, p.split = plan.split;
  p.total_units = plan.total_units;
  // Same constant as the reference (csrc/attention_kernel.hip:59, :1582): log2(e) / sqrt(head_dim), in fp32.
  p.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(ma::kHeadDim));
  p.rescale_tau = (flags & MA_FLAG_EXACT_MAX) ? 0.f : 8.f;

  if (workspace != nullptr) {
    e = cudaMemsetAsync(workspace, 0, ma::kStatusBytes, stream);
    if (e != cudaSuccess) return cuda_rc(e);
  }
  if (simple) return cuda_rc(ma::launch_attn_simple(p, stream));
  e = ma::launch_attn_pipelined(p, plan.grid, (flags & MA_FLAG_PRECISE_P) != 0, stream);
  if (e == cudaSuccess && plan.tail_tasks > 0) e = ma::launch_merge_parts(p, stream);
  return cuda_rc(e);
}

int ma_attention_forward_static(const void* q, const void* k, const void* v, void* out, int batch, int heads,
                                int seq_len, int seq_len_kv, int head_dim, int layout, int round_mode, int flags,
                                void* stream) {
  int rc = check_dims(batch, heads, seq_len, seq_len_kv);
  if (rc != MA_OK) return rc;
  if (flags & ~kForwardFlags) return MA_ERR_FLAGS;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_rc(e);
  // Reject before anything is launched: the scratch this problem's plan wants must fit the static buffer.
  const bool split = !(flags & (MA_FLAG_NO_TAIL | MA_FLAG_SIMPLE));
  const size_t need = ma::plan_workspace_bytes(ma::plan_tail(batch, heads, seq_len, seq_len_kv, sms, split));
  if (need > kStaticScratchBytes) return MA_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  const int arc = static_scratch_address(dev, &scratch);  // first call on a device: symbol lookup
  if (arc != MA_OK) return arc;
  // Same kernels and plan as ma_attention_forward, with the static buffer as its workspace.  That
  // call clears the status block; the partial results are fully rewritten before the merge reads them.
  rc = ma_attention_forward(q, k, v, out, batch, heads, seq_len, seq_len_kv, head_dim, layout, round_mode, scratch,
                            kStaticScratchBytes, flags, stream);
  // A CUDA error on the way may mean that the cached address went stale (cudaDeviceReset since the
  // look-up): drop it, so that the next call asks the runtime again.
  if (rc >= MA_ERR_CUDA_BASE) forget_static_scratch_address(dev);
  return rc;
}

int ma_static_status(uint32_t* host_words, int n, void* stream_) {
  if (host_words == nullptr) return MA_ERR_NULL_POINTER;
  if (n < 0 || n > ma::kStatusWords) return MA_ERR_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_rc(e);
  void* scratch = nullptr;
  const int arc = static_scratch_address(dev, &scratch);
  if (arc != MA_OK) return arc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  e = cudaMemcpyAsync(host_words, scratch, sizeof(uint32_t) * n, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  return cuda_rc(e);
}

size_t ma_lite_workspace_bytes(int batch, int heads, int seq_len) {
  if (batch <= 0 || heads <= 0 || seq_len <= 0) return ma::kStatusBytes + 256;
  const size_t tasks = static_cast<size_t>(batch) * heads * ((seq_len + ma::kLiteQueryBlock - 1) / ma::kLiteQueryBlock);
  return ma::kStatusBytes + 256 + ((tasks * sizeof(int) + 255) & ~static_cast<size_t>(255));
}

void ma_lite_tile(int* query_rows, int* key_rows) {
  if (query_rows != nullptr) *query_rows = ma::kLiteQueryBlock;
  if (key_rows != nullptr) *key_rows = ma::kLiteKeyBlock;
}

int ma_attention_forward_lite(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                              int seq_len_kv, int head_dim, int layout, int round_mode, const void* read_list,
                              void* write_list, const void* must_do_list, float threshold, int phase, void* workspace,
                              size_t workspace_bytes, int flags, void* stream_) {
  int rc = check_dims(batch, heads, seq_len, seq_len_kv);
  if (rc != MA_OK) return rc;
  if (head_dim != ma::kHeadDim) return MA_ERR_HEAD_DIM;
  if (read_list == nullptr || write_list == nullptr) return MA_ERR_LISTS;
  if (layout != MA_LAYOUT_BHSD && layout != MA_LAYOUT_BSHD) return MA_ERR_LAYOUT;
  if (round_mode < MA_ROUND_RTNE || round_mode > MA_ROUND_RTZ) return MA_ERR_ROUND_MODE;
  if (flags & ~kLiteFlags) return MA_ERR_FLAGS;
  if (q == nullptr || k == nullptr || v == nullptr || out == nullptr) return MA_ERR_NULL_POINTER;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                         reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out);
  if (bits & 15u) return MA_ERR_ALIGNMENT;
  const int key_blocks = (seq_len_kv + ma::kLiteKeyBlock - 1) / ma::kLiteKeyBlock;
  if (!(threshold < 0.f) || (phase != 0 && phase != 1) || key_blocks > 32766) return MA_ERR_LITE_ARGS;
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) ||
      workspace_bytes < ma_lite_workspace_bytes(batch, heads, seq_len))
    return MA_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  int dev = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (major != 10) return MA_ERR_DEVICE;

  ma::LiteParams p;
  std::memset(&p, 0, sizeof(p));
  rc = make_tensor_map(&p.a.tm_q, q, batch, heads, seq_len, layout, ma::kTileM);
  if (rc == MA_OK) rc = make_tensor_map(&p.a.tm_k, k, batch, heads, seq_len_kv, layout, ma::kLiteKeyBlock);
  if (rc == MA_OK) rc = make_tensor_map(&p.a.tm_v, v, batch, heads, seq_len_kv, layout, ma::kLiteKeyBlock);
  if (rc != MA_OK) return rc;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.a.out = static_cast<__nv_bfloat16*>(out);
  p.a.status = reinterpret_cast<uint32_t*>(ws);
  p.a.batch = batch, p.a.heads = heads, p.a.seq_q = seq_len, p.a.seq_kv = seq_len_kv;
  p.a.bshd = layout, p.a.round_mode = round_mode;
  p.a.nqb = (seq_len + ma::kLiteQueryBlock - 1) / ma::kLiteQueryBlock;
  p.a.nkb = key_blocks;
  p.a.scale_log2e = 1.4426950408889634f / sqrtf(static_cast<float>(ma::kHeadDim));
  p.a.rescale_tau = 8.f;
  p.read_list = static_cast<const int16_t*>(read_list);
  p.write_list = static_cast<int16_t*>(write_list);
  p.must_do = static_cast<const int16_t*>(must_do_list);
  p.counter = reinterpret_cast<int*>(ws + ma::kStatusBytes);
  p.num_tasks = batch * heads * p.a.nqb;
  p.row_width = key_blocks + 2;
  p.phase = phase;
  p.threshold = threshold;

  // status block and hand-out counter
  e = cudaMemsetAsync(workspace, 0, ma::kStatusBytes + 256, stream);
  if (e != cudaSuccess) return cuda_rc(e);
  if (!(flags & MA_FLAG_LITE_PLAIN)) {
    int* order = reinterpret_cast<int*>(ws + ma::kStatusBytes + 256);
    e = ma::launch_lite_order(p, order, stream);
    if (e != cudaSuccess) return cuda_rc(e);
    p.order = order;
  }
  const int grid = p.num_tasks < sms ? p.num_tasks : sms;
  return cuda_rc(ma::launch_attn_lite(p, grid, stream));
}

// ---- MLA absorbed decode -------------------------------------------------------------------------------
namespace {
// Draft positions per CTA: two for a window (a second group of softmax warps on the same tiles), the way the
// reference's multi-query kernel keeps a window resident (csrc/mla_decode_a16w8_multiq.hip:722).
int mla_pos_per_cta(int q_len) { return q_len >= 2 ? 2 : 1; }
int mla_groups(int q_len, int per) { return (q_len + per - 1) / per; }
}  // namespace

namespace {
int mla_plan(int batch, int q_len, int max_seq_len, int num_sms) {
  if (batch <= 0 || q_len < 1 || q_len > 8 || max_seq_len <= 0) return 1;
  const int sms = resolve_sms(num_sms);
  if (sms <= 0) return 1;
  const int base = batch * mla_groups(q_len, mla_pos_per_cta(q_len));  // CTAs before any split
  const int tiles = (max_seq_len + 127) / 128;            // planning unit: 128 tokens of the longest request
  int parts = sms / base;                                 // fill the GPU once ...
  const int by_length = (tiles + 3) / 4;                  // ... with at least four tiles (512 tokens) per part
  if (parts > by_length) parts = by_length;
  if (parts > MA_MLA_MAX_PARTS) parts = MA_MLA_MAX_PARTS;
  return parts < 1 ? 1 : parts;
}
}  // namespace

int ma_mla_plan_parts(int batch, int q_len, int max_seq_len, int num_sms) {
  return mla_plan(batch, q_len, max_seq_len, num_sms);
}
int ma_mla_plan_parts_contiguous(int batch, int q_len, int seq_len, int num_sms) {
  return mla_plan(batch, q_len, seq_len, num_sms);
}

int ma_mla_cluster_capacity(int q_len, int paged, int parts) {
  if (q_len < 1 || q_len > 8) return 0;
  return ma::mla_cluster_capacity(mla_pos_per_cta(q_len), paged == 0, parts);
}

size_t ma_mla_workspace_bytes(int batch, int q_len, int parts) {
  if (batch <= 0 || q_len < 1 || q_len > 8 || parts < 1) return ma::kStatusBytes;
  // one slot of 16 rows per (request, position, part); positions are rounded up to even, which also covers
  // CTAs that take two positions (32 rows per slot)
  const size_t slots = static_cast<size_t>(batch) * (q_len == 1 ? 1 : (q_len + 1) / 2 * 2) * parts;
  return ma::kStatusBytes + slots * 16u * (512 + 2) * sizeof(float);
}

int ma_mla_decode_a16w8(const void* q_lat, const void* q_pe, const void* kv, void* o_lat, const int* seq_lens,
                        const int* rows, const int* kv_indices, const int* kv_indptr, int batch, int heads, int q_len,
                        int seq_len, int parts, float scale, float kv_scale, int kv_format, void* workspace,
                        size_t workspace_bytes, void* stream_) {
  if (batch <= 0 || heads < 1 || heads > 16) return MA_ERR_BATCH_HEADS;
  if (q_len < 1 || q_len > 8) return MA_ERR_SEQ_Q;
  const bool paged = kv_indices != nullptr;
  if (paged ? (kv_indptr == nullptr || seq_lens == nullptr) : seq_len <= 0) return MA_ERR_SEQ_KV;
  if (parts < 1 || parts > MA_MLA_MAX_PARTS || (kv_format != 0 && kv_format != 1)) return MA_ERR_MLA_ARGS;
  if (q_lat == nullptr || q_pe == nullptr || kv == nullptr || o_lat == nullptr) return MA_ERR_NULL_POINTER;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(q_lat) | reinterpret_cast<uintptr_t>(q_pe) |
                         reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(o_lat);
  if (bits & 15u) return MA_ERR_ALIGNMENT;
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) ||
      workspace_bytes < ma_mla_workspace_bytes(batch, q_len, parts))
    return MA_ERR_WORKSPACE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int dev = 0, major = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (major != 10) return MA_ERR_DEVICE;

  ma::MlaParams p;
  std::memset(&p, 0, sizeof(p));
  p.q_lat = q_lat, p.q_pe = q_pe, p.kv = kv, p.o_lat = o_lat;
  p.seq_lens = seq_lens, p.rows = rows, p.kv_indices = kv_indices, p.kv_indptr = kv_indptr;
  p.batch = batch, p.heads = heads, p.q_len = q_len, p.seq = seq_len;
  const bool slab = !paged;
  p.parts = parts, p.pos_per_cta = mla_pos_per_cta(q_len), p.groups = mla_groups(q_len, p.pos_per_cta);
  p.kv_format = kv_format, p.scale = scale, p.kv_scale = kv_scale;
  if (slab) {
    int rc = make_kv_slab_map(&p.tm_kv, kv, batch, seq_len, 128);
    if (rc == MA_OK) rc = make_kv_slab_map(&p.tm_kv_rope, kv, batch, seq_len, 64);
    if (rc != MA_OK) return rc;
    p.use_tma = 1;
  }
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.status = reinterpret_cast<uint32_t*>(ws);
  const size_t slots = static_cast<size_t>(batch) * p.groups * parts, r = 16u * p.pos_per_cta;
  p.part_ml = reinterpret_cast<float*>(ws + ma::kStatusBytes);
  p.part_o = p.part_ml + slots * r * 2;
  // (the status word is cleared by the kernel itself: a memset in front of it would cost two microseconds and
  // keep the kernel from lining up behind its predecessor in the stream)
  return cuda_rc(ma::launch_mla_decode(p, stream));
}

int ma_selftest_wait_timeout(uint64_t limit_ns, void* workspace, size_t workspace_bytes, void* stream_) {
  if (workspace == nullptr) return MA_ERR_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < ma::kStatusBytes) return MA_ERR_WORKSPACE;
  // The limit is the caller's, but never long: this entry point exists to show that a wait that runs
  // out ends the kernel, not to occupy an SM.
  if (limit_ns == 0 || limit_ns > 100ull * 1000ull * 1000ull) return MA_ERR_TOO_LARGE;
  int dev = 0, major = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_rc(e);
  if (major != 10) return MA_ERR_DEVICE;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  e = cudaMemsetAsync(workspace, 0, ma::kStatusBytes, stream);
  if (e != cudaSuccess) return cuda_rc(e);
  return cuda_rc(ma::launch_wait_timeout_selftest(static_cast<uint32_t*>(workspace), limit_ns, stream));
}

int ma_round_bf16(const float* src, uint16_t* dst, size_t n, int round_mode, void* stream) {
  if (round_mode < MA_ROUND_RTNE || round_mode > MA_ROUND_RTZ) return MA_ERR_ROUND_MODE;
  if (n > 0 && (src == nullptr || dst == nullptr)) return MA_ERR_NULL_POINTER;
  return cuda_rc(ma::launch_round_bf16(src, dst, n, round_mode, static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
