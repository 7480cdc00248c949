/*
 * C ABI of libmoonmath_attention_sm100.so: dense bf16 flash-attention forward
 * for NVIDIA B200 (sm_100a).
 *
 * These entry points take the place of the per-rounding-mode native interface
 * that the reference's torch binding calls (csrc/attention_api.cpp:17-64 and
 * :122-125 declare it; csrc/attention_kernel.hip:1546-1597 and :1685-1715
 * define it):
 *
 *     int    launch_v_transpose_<mode>(v, v_t, n_rows, seq_len_per_head, heads, layout, stream)
 *     int    launch_attention_forward_<mode>(q, k, v_t, out, batch, heads, seq_len, seq_len_kv,
 *                                            head_dim, layout, workspace, stream)
 *     size_t tail_workspace_bytes_<mode>(void)
 *
 * Differences a binding author must know:
 *   - one library, the rounding mode is an argument (no _rtne/_rtna/_rtz copies);
 *   - no V pre-transpose pass and no V_t buffer: K and V are read in place in
 *     either layout;
 *   - the workspace is sized per problem (ma_workspace_bytes) and starts with a
 *     256-byte status block that the kernels fill in when a bounded wait gives up;
 *   - the library keeps no state between calls: calls on different streams or
 *     devices may run concurrently (the reference keeps a static schedule,
 *     csrc/attention_kernel.hip:1375-1378).  The one exception is
 *     ma_attention_forward_static, which owns a static device array and a
 *     cached address per device; its comment states the rules.
 *
 * All pointers are device pointers on the current CUDA device; `stream` is a
 * cudaStream_t.  Every call is asynchronous on `stream` and never synchronises.
 * There is no CPU path: without an sm_100 device the calls fail with an error code.
 */
#ifndef MOONMATH_ATTENTION_H_
#define MOONMATH_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MA_ABI_VERSION 1

/* layout (reference: csrc/attention_kernel.hip:1581 "0 = BHSD, 1 = BSHD") */
#define MA_LAYOUT_BHSD 0
#define MA_LAYOUT_BSHD 1

/* round_mode (reference: BF16Round, csrc/attention_kernel.hip:37-38) */
#define MA_ROUND_RTNE 0
#define MA_ROUND_RTNA 1
#define MA_ROUND_RTZ 2

/* flags */
#define MA_FLAG_NO_TAIL 0x1      /* never split the last partial round along KV (reference: null workspace /
                                    MOONMATH_NO_TAIL, csrc/attention_api.cpp:258-267) */
#define MA_FLAG_SIMPLE 0x2       /* run the serialised cross-check kernel instead of the pipelined one */
#define MA_FLAG_EXACT_MAX 0x8    /* rescale the accumulator whenever the running maximum rises (tau = 0) */
#define MA_FLAG_PRECISE_P 0x10   /* accuracy mode: the softmax probabilities enter the second matrix product as the
                                    sum of two bf16 terms (16 significant bits instead of the 8 the reference keeps,
                                    csrc/attention_kernel.hip:446-448), for 25 % more tensor-core work */
#define MA_FLAG_LITE_PLAIN 0x20  /* ma_attention_forward_lite: hand tasks out in index order, not longest-first
                                    (reference: MOONMATH_LITE_PLAIN / null workspace, csrc/attention_api.cpp:400-407) */
/* ma_attention_forward(_static) accepts NO_TAIL, SIMPLE, EXACT_MAX and PRECISE_P; ma_attention_forward_lite accepts
   LITE_PLAIN; any other bit is refused with MA_ERR_FLAGS. */

/* return codes: 1, 2, 3, 5, 6 keep the reference's meaning (csrc/attention_kernel.hip:1573-1576, :1588) */
#define MA_OK 0
#define MA_ERR_BATCH_HEADS 1     /* batch <= 0 or heads <= 0 */
#define MA_ERR_SEQ_Q 2           /* seq_len <= 0 */
#define MA_ERR_HEAD_DIM 3        /* head_dim != 128 */
#define MA_ERR_LISTS 4           /* ma_attention_forward_lite: read_list or write_list is null
                                    (reference: csrc/attention_kernel.hip:1627) */
#define MA_ERR_SEQ_KV 5          /* seq_len_kv <= 0 */
#define MA_ERR_PLAN 6            /* the tail plan could not be set up */
#define MA_ERR_LAYOUT 7
#define MA_ERR_ROUND_MODE 8
#define MA_ERR_NULL_POINTER 9
#define MA_ERR_ALIGNMENT 10      /* q, k, v, out must be 16-byte aligned */
#define MA_ERR_WORKSPACE 11      /* workspace smaller than ma_workspace_bytes() or misaligned */
#define MA_ERR_TENSOR_MAP 12     /* cuTensorMapEncodeTiled refused the tensor */
#define MA_ERR_DRIVER 13         /* driver entry point not found */
#define MA_ERR_DEVICE 14         /* current device is not sm_100 */
#define MA_ERR_TOO_LARGE 15      /* a dimension exceeds what the kernel indexes */
#define MA_ERR_STATIC_SCRATCH 16 /* ma_attention_forward_static: the plan needs more than MA_STATIC_SCRATCH_BYTES */
#define MA_ERR_LITE_ARGS 17      /* threshold >= 0, phase not 0 / 1, or more than 32766 key blocks of 64 */
#define MA_ERR_MLA_ARGS 18       /* ma_mla_decode_a16w8: parts or kv_format out of range */
#define MA_ERR_FLAGS 19          /* a flag bit the entry point does not define */
#define MA_ERR_CUDA_BASE 1000    /* 1000 + cudaError_t of a failed runtime call or launch */

/* Value of MA_ABI_VERSION the library was built with. */
int ma_abi_version(void);

/* Static text for a return code. */
const char* ma_error_string(int rc);

/* Number of SMs of the current device, or a negative return code. */
int ma_device_sms(void);

/*
 * Bytes of workspace ma_attention_forward needs for this problem on a device
 * with `num_sms` SMs (<= 0: query the current device).  Always >= 256.
 * Replaces tail_workspace_bytes (csrc/attention_kernel.hip:1549-1551), which
 * returns a shape-independent 121 405 440.
 */
size_t ma_workspace_bytes(int batch, int heads, int seq_len, int seq_len_kv, int num_sms, int flags);

/*
 * The tail KV-split decision for a problem (pure host arithmetic; replaces
 * plan_tail_split, csrc/attention_kernel.hip:1349-1393).  Fills
 *   plan[0] tasks          256-row query blocks x batch x heads
 *   plan[1] full_units     tasks run whole
 *   plan[2] tail_tasks     tasks of the last partial round that are split (0: no split)
 *   plan[3] split          parts per split task
 *   plan[4] total_units
 *   plan[5] grid           CTAs launched
 *   plan[6] nqb            query blocks per (batch, head)
 *   plan[7] nkb            128-row key/value blocks
 */
int ma_plan_tail(int batch, int heads, int seq_len, int seq_len_kv, int num_sms, int flags, int plan[8]);

/*
 * out = softmax(q k^T / sqrt(128)) v, bf16 in / bf16 out, fp32 accumulation.
 * Replaces launch_v_transpose + launch_attention_forward
 * (csrc/attention_kernel.hip:1560-1597, :1685-1715).
 *   layout 0: q,out [batch, heads, seq_len, 128], k,v [batch, heads, seq_len_kv, 128]
 *   layout 1: q,out [batch, seq_len, heads, 128], k,v [batch, seq_len_kv, heads, 128]
 * All tensors contiguous.  `workspace` may be null (then no KV split and no
 * status reporting); otherwise it holds at least ma_workspace_bytes(...) bytes,
 * 256-byte aligned, and its first 256 bytes are cleared by this call and hold
 * the device status afterwards (word 0 != 0: a kernel gave up, output invalid).
 */
int ma_attention_forward(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                         int seq_len_kv, int head_dim, int layout, int round_mode, void* workspace,
                         size_t workspace_bytes, int flags, void* stream);

/*
 * The same operation as ma_attention_forward for callers that must not allocate device memory
 * and have nowhere to keep a workspace: code running inside another framework's memory pool or
 * under a fixed memory budget, plug-ins handed only the input and output buffers, and anything
 * that runs where cudaMalloc is forbidden or would synchronise the device.  (No counterpart in
 * the reference, whose binding allocates its 121 MB workspace on every call.)
 *
 * The scratch (status block + KV-split partial results) is a static device array inside the
 * library, MA_STATIC_SCRATCH_BYTES large; every GPU that loads the library carries it until the
 * process exits.  The call performs no cudaMalloc / cudaFree and calls no allocating library
 * routine.  Limits and rules:
 *   - a problem whose tail plan wants more scratch than that returns MA_ERR_STATIC_SCRATCH and
 *     launches nothing; with MA_FLAG_NO_TAIL every problem fits (256 bytes are used);
 *   - the first call on each device looks up the array's device address (a host-side set-up step);
 *     make that first call before any stream capture begins;
 *   - the address is cached per device ordinal for the life of the process.  It belongs to the device's
 *     primary context as the CUDA runtime sets it up; after cudaDeviceReset the cache is stale (a call that
 *     then fails with a CUDA error drops it, the next call looks the address up again), and contexts other
 *     than the primary one are not supported;
 *   - all calls on one device share the one array: calls whose kernels can overlap on the GPU
 *     (different streams, no ordering between them) race on it and must be serialised by the
 *     caller.  Calls ordered on one stream are safe; the array keeps the previous call's contents
 *     and this call rewrites everything it reads (the status block is cleared first).
 * After the stream has drained, ma_static_status() tells whether the kernels reported a fault.
 */
#define MA_STATIC_SCRATCH_BYTES (40u << 20)
int ma_attention_forward_static(const void* q, const void* k, const void* v, void* out, int batch, int heads,
                                int seq_len, int seq_len_kv, int head_dim, int layout, int round_mode, int flags,
                                void* stream);

/*
 * Copies the first `n` (<= 64) device status words of the static scratch of the current device to
 * `host_words` (synchronises `stream`).  Word 0 is 0 when the last ma_attention_forward_static on
 * this device ran clean.  No counterpart in the reference.
 */
int ma_static_status(uint32_t* host_words, int n, void* stream);

/*
 * LiteAttention forward.  Replaces launch_attention_forward_lite_{rtna,rtne,rtz}
 * (csrc/attention_kernel.hip:1604-1681; bound from csrc/attention_api.cpp:287-434) together with the
 * V transpose and the allocations of its caller.
 *
 * read_list / write_list: int16 device arrays [batch][heads][query blocks][key blocks + 2], one
 * run-length row per task in the reference's format (csrc/attention_kernel.hip:629-716;
 * moonmath_attention/lite.py:108-128): [len, markers...], read from the back in the direction `phase`
 * names (1 upwards, 0 downwards).  Only the key blocks the read row names are loaded and computed; the
 * row written for the next call keeps the blocks for which some group of query rows found a score
 * within `threshold` (log2 units, negative) of its running maximum.  The block geometry is this
 * library's (ma_lite_tile): 256 query rows per list row where the reference has 384
 * (moonmath_attention/lite.py:36-37), 64 keys per block as in the reference, votes per 32 query rows
 * where the reference votes per 48; lists are therefore exchanged only between calls of this library.
 * must_do_list: optional global [len, s0, e0, s1, e1, ...] of key-block ranges [s, e) always written as
 * "compute" (csrc/attention_kernel.hip:676-701), or null.
 * workspace: ma_lite_workspace_bytes() bytes, 256-byte aligned, required (status block, hand-out
 * counter, longest-first order: plan_lite_order, csrc/attention_kernel.hip:1296-1347).
 * Return codes as ma_attention_forward, plus MA_ERR_LISTS (4, the reference's code) and MA_ERR_LITE_ARGS.
 */
size_t ma_lite_workspace_bytes(int batch, int heads, int seq_len);
/* Query rows per list row and keys per list block (reference: KBLOCK_M, KBLOCK_N, moonmath_attention/lite.py:36-37). */
void ma_lite_tile(int* query_rows, int* key_rows);
int ma_attention_forward_lite(const void* q, const void* k, const void* v, void* out, int batch, int heads, int seq_len,
                              int seq_len_kv, int head_dim, int layout, int round_mode, const void* read_list,
                              void* write_list, const void* must_do_list, float threshold, int phase, void* workspace,
                              size_t workspace_bytes, int flags, void* stream);

/*
 * MLA absorbed-decode attention, bf16 queries against an fp8 KV cache.  One entry point for what the
 * reference exports as launch_mla_decode_a16w8, launch_mla_decode_a16w8_paged_dev
 * (csrc/mla_decode_a16w8.hip:784-876, bound from csrc/mla_decode_a16w8_api.cpp:76-150) and the multi-query
 * pair (csrc/mla_decode_a16w8_multiq.hip:946-1001).
 *   q_lat [batch][q_len][heads][512], q_pe [batch][q_len][heads][64], o_lat like q_lat: bf16, q_len 1..8,
 *   heads 1..16.  Draft position t of request b attends the first len_b - q_len + t + 1 cached tokens.
 *   kv: fp8 rows of 576 bytes ([0,512) latent, [512,576) rope), one per-tensor kv_scale.
 *     contiguous: kv_indices = kv_indptr = null, kv is [batch][seq_len][576], len_b = seq_lens ? seq_lens[b] : seq_len;
 *     paged:      kv is a pool [slots][576]; token i of request b lives in slot kv_indices[kv_indptr[b] + i];
 *                 seq_lens is required.  All index arrays are int32 device memory, read by the kernel only
 *                 (no host read, fixed grid: the call can be captured in a CUDA graph with `parts` fixed).
 *   rows: optional int32[batch], batch row of q_lat / o_lat that request b uses (null: b).
 *   kv_format: 0 = e4m3-fnuz, the reference's cache format; 1 = e4m3 (OCP).  The tensor core reads e4m3: fnuz
 *     bytes are reinterpreted (every finite value is exactly half).  0x7F / 0xFF (+-240), which are NaN in e4m3,
 *     are fed as +-224 and corrected by hand: exact for up to 640 such entries per 96 consecutive tokens of a
 *     request (256 when q_len > 1), +-224 for the surplus.  0x80 (NaN in fnuz) reads as zero.  An e4m3 cache is
 *     read as it is; a NaN code in it reaches both draft positions of the CTA that reads the row (positions are
 *     processed in pairs), also the one whose causal limit lies before that token.
 *   parts: KV split per request, 1..MA_MLA_MAX_PARTS (ma_mla_plan_parts); workspace: ma_mla_workspace_bytes.
 *   Stream order: the kernel is launched as a programmatic dependent of whatever kernel precedes it in the stream
 *     (it sets up while that kernel drains, then waits for it to complete before it reads or writes global
 *     memory), and it lets a kernel launched the same way behind it do the same.  No memset precedes it: the
 *     first word of the status block is cleared by the kernel.
 */
#define MA_MLA_MAX_PARTS 256
int ma_mla_plan_parts(int batch, int q_len, int max_seq_len, int num_sms);
/* The split the contiguous entry points of the Python package choose for themselves (same rule). */
int ma_mla_plan_parts_contiguous(int batch, int q_len, int seq_len, int num_sms);
size_t ma_mla_workspace_bytes(int batch, int q_len, int parts);
/* With 2..8 parts, the parts of a request run as one thread-block cluster and merge their results through
 * shared memory, as long as all clusters of the call are resident at once: batch x ceil(q_len / 2) (batch when
 * q_len = 1) <= this number, which depends on the device, the cluster size and the kernel variant (paged: 0 for
 * a contiguous cache, 1 for a pool).  Otherwise, and with more parts, a merge kernel follows.  Results are the
 * same either way up to fp32 summation order.  0: no GPU, or no such cluster.  No counterpart in the reference. */
int ma_mla_cluster_capacity(int q_len, int paged, int parts);
int ma_mla_decode_a16w8(const void* q_lat, const void* q_pe, const void* kv, void* o_lat, const int* seq_lens,
                        const int* rows, const int* kv_indices, const int* kv_indptr, int batch, int heads, int q_len,
                        int seq_len, int parts, float scale, float kv_scale, int kv_format, void* workspace,
                        size_t workspace_bytes, void* stream);

/*
 * Self-test of the failure path: launches one CTA that waits, for at most `limit_ns` (1 .. 100 000 000), on
 * a barrier nobody arrives on.  The wait gives up, the kernel leaves through its common exit (tensor memory
 * freed) and returns; nothing faults.  Afterwards (stream drained) the first words of `workspace`
 * (>= 256 bytes, 256-byte aligned, cleared by this call) read
 *   [0] 0x57A17 (a bounded wait ran out)   [1] wait site | CTA << 8   [9] 1 (the CTA unwound through its abort flag)
 * exactly what a production kernel leaves in its status block when a wait times out.  The reference has
 * no counterpart (it reports through return codes only, csrc/attention_kernel.hip:1573-1576, :1588).
 */
int ma_selftest_wait_timeout(uint64_t limit_ns, void* workspace, size_t workspace_bytes, void* stream);

/*
 * dst[i] = bf16 bits of src[i] under round_mode, NaN -> 0x7FFF; device pointers.
 * Exposes the output rounding of the attention epilogue (reference:
 * bf16_round_one, csrc/attention_kernel.hip:110-145) for bit-pattern tests.
 */
int ma_round_bf16(const float* src, uint16_t* dst, size_t n, int round_mode, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOONMATH_ATTENTION_H_ */
