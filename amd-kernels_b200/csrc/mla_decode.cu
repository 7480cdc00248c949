// MLA absorbed-decode attention, bf16 queries against an fp8 KV cache ("A16W8"), for sm_100a.
//
// What it computes is the reference's mla_decode_a16w8 / _multiq operators (csrc/mla_decode_a16w8.hip:186,
// csrc/mla_decode_a16w8_multiq.hip:722; semantics stated in moonmath_attention/mla.py:41-186 and
// tests/test_mla_decode.py:52-68): per request b and draft position t, softmax over the first
// len_b - q_len + t + 1 cached tokens of (q_lat . kv[:512] + q_pe . kv[512:576]) * scale, times kv[:512],
// with kv stored as fp8 rows of 576 bytes at one per-tensor scale, contiguous or paged one token per slot.
//
// How: the KV bytes go to the tensor core as they are.  The reference unpacks fp8 to bf16 on the way into
// LDS; here a tile of 96 tokens x 576 bytes is the A operand of fp8 MMAs (kind::f8f6f4) twice:
//   S^T[tokens x N]       = KV[96 x 576] (K-major)  x  Q^T[576 x N]
//   O^T[4 x 128 dims x N] = KV^T (same bytes, MN-major, 128 latent bytes of a row per M tile)  x  P^T[96 tokens x N]
// The 16-bit operands become sums of two e4m3 terms, stacked along N (N = 2 x rows): a query row scaled by a
// power of two splits exactly into q1 + q2 (8 significant bits = 4 + 4); a probability splits the same
// way (the reference rounds it to bf16, also 8 bits).  The terms' partial sums sit in separate accumulator
// columns and are added by the thread that reads them.  With tokens on the lanes of tensor memory, a thread
// owns one token (softmax) or one output dimension (rescale, epilogue).
//
// e4m3-fnuz (the reference's format) differs from the e4m3 the tensor core reads by a factor of two in
// every finite value, folded into the scales, and in two codes: 0x7F / 0xFF are +-240 there and NaN here.
// Nobody looks for them in advance: a token row that holds one gives NaN scores, and only then does the
// softmax thread of that token rewrite them to 0x7E / 0xFE (+-224) in shared memory, list them and have the
// tile's Q K^T run again; the softmax warps add the missing +-16 x q to the scores and +-16 x p to the outputs
// by hand, so the result is exact for up to 640 such entries per tile of 96 tokens (beyond that the rest stay
// at +-224).  0x80 (NaN there) reads as zero.  e4m3 caches (kv_format 1) are read unchanged.
//
// One CTA per (request, group of draft positions, KV part).  Up to eight parts of a request form a thread-block
// cluster: each leaves its partial result in its own shared memory and, after a cluster barrier, merges a share
// of the rows from all of them (distributed shared memory, no trip through L2, no second launch).  More parts
// (a few long requests) go through global memory and mla_merge_kernel.
//   warps 0-3  softmax / rescale / epilogue    warp 4  MMA issuer    warps 5-12 (or 5)  copy
// All waits are bounded mbarrier waits.
#include <cuda_fp8.h>

#include <atomic>
#include <type_traits>

#include "attn_common.cuh"
#include "attn_launch.h"

namespace ma {
namespace {

using namespace sm100;

constexpr int kLat = 512, kRowBytes = 576;
constexpr int kTok = 96;                         // tokens per tile
constexpr int kMmaM = 128;                       // rows of an MMA; S^T rows 96..127 are never looked at (see role_mma)
constexpr int kChunks = 5;                       // column chunks of a row: 4 latent of 128 bytes + rope of 64
constexpr int kChunkBytes = kTok * 128;          // 12 KiB: a latent chunk, [96 rows][128 B], 128-byte swizzle
constexpr int kRopeBytes = kTok * 64;            //  6 KiB: the rope chunk, [96 rows][64 B], 64-byte swizzle
constexpr int kTileBytesMla = 4 * kChunkBytes + kRopeBytes;  // 55296 = 96 x 576: nothing is padded
constexpr int kMaxStagesMla = 3;                 // a tile spends about as long being loaded as being used
constexpr int kHeadsMax = 16;
constexpr int kSoftmaxThreads = 128;             // per draft position of the CTA
// Copy warps: eight for the 16-byte copies of a paged pool, one (one thread of it) for box loads; the block is
// launched with as many threads as its roles need, so the box-load variant has twice the registers per thread.
constexpr int copy_threads(bool tma, int pos) { return tma ? 32 : (pos == 1 ? 256 : 192); }
// slab: 192 threads (two positions: 320); pool: 416 (two positions: 480) rounded up to whole warpgroups = 512,
// because the pool variants move registers between warpgroups (setmaxnreg) and every warpgroup that takes part
// is complete; the padding warps do nothing.
constexpr int block_threads(bool tma, int pos) {
  const int used = pos * kSoftmaxThreads + 32 + copy_threads(tma, pos);
  return tma ? used : (used + 127) / 128 * 128;
}
constexpr float kTauMla = 8.f;                   // lazy rescale: p <= 2^8 = 256 < 448
constexpr float kSatResidual = 32.f;             // +-240 fnuz = +-480 as e4m3; the tensor core gets +-448; the rest by hand

template <int kPos>
struct Cfg {
  static constexpr int kRows = kHeadsMax * kPos;  // query rows per CTA
  static constexpr int kN = 2 * kRows;            // two e4m3 terms per row
  static constexpr uint32_t kTmemCols = kPos == 1 ? 256 : 512;  // S x 2 + O^T x 4 = 6 * kN = 192 / 384
  static constexpr int kStages = 3;
  static constexpr int kSatCap = kPos == 1 ? 640 : 256;         // saturated e4m3-fnuz entries of one tile that are corrected exactly
  static constexpr uint32_t kOffKV = 0;
  // After the last P V the stages are idle; a part of a cluster leaves its result there for the merge:
  // float [kRows][512] un-normalised outputs, then float2 [kRows] (reference maximum, denominator).
  static constexpr uint32_t kOffPartO = kOffKV;
  static constexpr uint32_t kOffPartMl = kOffPartO + kRows * kLat * 4;
  static constexpr uint32_t kOffQT = kStages * kTileBytesMla;       // [5 chunks][kN rows][128 B]
  static constexpr uint32_t kOffPT = kOffQT + kChunks * kN * 128;      // [2][128 token rows][kN B], kN-byte swizzle (96 rows used)
  static constexpr uint32_t kOffRowScale = kOffPT + 2 * kN * 128;      // float [kRows]: score = (S1 + S2) * this
  static constexpr uint32_t kOffMx = kOffRowScale + kRows * 4;         // float [2][4 warps][kRows]
  static constexpr uint32_t kOffL = kOffMx + 2 * 4 * kRows * 4;        // float [4 warps][kRows]: denominators (epilogue)
  static constexpr uint32_t kOffFlags = kOffL + 4 * kRows * 4;         // int [2][4 kPos softmax warps]
  static constexpr uint32_t kOffSatCnt = kOffFlags + 2 * 4 * kPos * 4; // int [kStages]: saturated entries of the tile in a stage; [3]: first P V accumulates
  static constexpr uint32_t kOffSat = kOffSatCnt + 16;                 // uint32 [kStages][kSatCap]: token | column << 7 | negative << 17
  static constexpr uint32_t kOffBars = kOffSat + kStages * kSatCap * 4;
};
enum MlaBar : uint32_t {
  kMTileEmpty = 0,  // [3] MMA -> copy warps
  kMTileRaw = 3,    // [3] copy warps -> MMA: the tile has landed (256 copy threads, or 1 + bytes for box loads)
  kMSFull = 6,      // [2] MMA -> softmax
  kMPFull = 8,      // [2] softmax -> MMA (every softmax thread arrives)
  kMPvDone = 10,    // [2] MMA -> softmax: P V of the tile complete (P buffer free, O stable)
  kMMx = 12,        // [2][2 groups] softmax warps of a group among themselves: row maxima written (4 arrivals)
  kMFlag = 16,      // [2] all softmax warps: overflow and NaN flags written (one arrival per warp)
  kMEpi = 18,       // [2 groups] softmax warps of a group: denominators written (4 arrivals)
  kMSat = 20,       // [2] all softmax warps: P^T written, before a saturation correction (one arrival per warp)
  kMRedoReq = 22,   //     softmax warps -> MMA: rows of the oldest tile were rewritten, run its Q K^T again (one arrival per warp)
  kMRedoDone = 23,  //     MMA -> softmax: that Q K^T has completed
  kMNumBars = 24
};


#define MA_WAIT(bar, parity, site) \
  if (!mbar_wait((bar), (parity), (site), ctx)) return
#define MA_WAIT_WARP(bar, parity, site) \
  if (!mbar_wait_warp((bar), (parity), (site), ctx)) return
#define MA_WAIT_SLEEP(ns, bar, parity, site) \
  if (!mbar_wait<ns>((bar), (parity), (site), ctx)) return

__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Two floats -> two e4m3 bytes (round to nearest, saturating), low byte = first argument; and back.
__device__ __forceinline__ uint32_t to_e4m3x2(float lo, float hi) {
  return __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float2 from_e4m3x2(uint32_t v) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(v), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Byte offset of (row, byte column) inside a [rows][128 B] block with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 4) ^ (row & 7u)) << 4) | (col & 15u));
}
// The same for a [rows][64 B] block with the 64-byte swizzle (16-byte pieces xor-ed with bits 1-2 of the row).
__device__ __forceinline__ uint32_t swz64(uint32_t row, uint32_t col) {
  return row * 64u + ((((col >> 4) ^ ((row >> 1) & 3u)) << 4) | (col & 15u));
}
// P of a tile is stored token-major, [tokens][N bytes] under the N-byte swizzle (N = 32 or 64), so that a
// softmax thread (one token) writes its probabilities with 16-byte stores; the tensor core reads it as an
// MN-major B operand.  Byte offset of (token, accumulator column n):
template <int N>
__device__ __forceinline__ uint32_t p_off(uint32_t tok, uint32_t n) {
  static_assert(N == 32 || N == 64, "one swizzle row per token");
  const uint32_t x = N == 32 ? (tok >> 2) & 1u : (tok >> 1) & 3u;
  return tok * N + ((((n >> 4) ^ x) << 4) | (n & 15u));
}
// Byte offset of (token row, byte column 0..575) inside a KV tile.
__device__ __forceinline__ uint32_t kv_off(uint32_t row, uint32_t col) {
  return col < static_cast<uint32_t>(kLat) ? (col >> 7) * kChunkBytes + swz128(row, col & 127u)
                                           : 4u * kChunkBytes + swz64(row, col - kLat);
}

struct Work {
  int b, brow, group, part;
  int q_len, heads;
  int pos0, npos;       // draft positions of this CTA
  int len;              // cached tokens of the request
  int tile0, tiles;     // tiles [tile0, tile0 + tiles) of 96 tokens
  int idx0;             // paged pool: where the request's slot numbers begin in kv_indices
  int end_max;          // tokens the last position of the group may see
};

__device__ __forceinline__ Work decode_work(const MlaParams& p, int kpos) {
  Work w;
  const int cta = blockIdx.x;
  w.part = cta % p.parts;
  const int bg = cta / p.parts;
  w.group = bg % p.groups;
  w.b = bg / p.groups;
  w.brow = p.rows != nullptr ? p.rows[w.b] : w.b;
  w.q_len = p.q_len;
  w.heads = p.heads;
  w.pos0 = w.group * kpos;
  w.npos = min(kpos, p.q_len - w.pos0);
  // (the three loads are independent of one another: one trip to memory, not three)
  w.idx0 = p.kv_indptr != nullptr ? p.kv_indptr[w.b] : 0;
  w.len = p.seq_lens != nullptr ? p.seq_lens[w.b] : p.seq;
  w.end_max = w.len - p.q_len + w.pos0 + w.npos;  // last position of the group, inclusive limit + 1
  const int total = w.end_max > 0 ? (w.end_max + kTok - 1) / kTok : 0;
  const int per = (total + p.parts - 1) / p.parts;
  w.tile0 = min(w.part * per, total);
  w.tiles = min(per, total - w.tile0);
  return w;
}

// loaders.  Pools: eight (six) "copy" warps stream a tile of 96 token rows into the swizzled chunks with 16-byte
// loaders.  Eight "copy" warps stream a tile of 128 token rows into the swizzled chunks with 16-byte
// asynchronous copies (no registers in between) and hand completion to an mbarrier, so they never wait for
// data and the next tile's copies start the moment its stage is free.  The MMA thread takes the landed tile
// (after a proxy fence for the 16-byte copies, which are generic-proxy writes; box loads need none).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// The mbarrier receives one arrival once every copy this thread has issued so far has landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

template <int kPos, bool kTma>
__device__ __forceinline__ void role_copy(const MlaParams& p, const Work& w, uint32_t base, int lt, const WaitCtx& ctx) {
  using C = Cfg<kPos>;
  constexpr int kCopyThreads = copy_threads(kTma, kPos);
  const uint32_t bars = base + C::kOffBars;
  if constexpr (kTma) {
    // Contiguous slab: five box loads per tile (one per column chunk, 96 rows each), issued by one
    // thread.  Rows past the slab and the columns past byte 576 of the rope chunk arrive as zeros.
    if (lt != 0) return;
    for (int j = 0; j < w.tiles; ++j) {
      const int st = j % C::kStages;
      if (j >= C::kStages) MA_WAIT_SLEEP(64, bars + 8 * (kMTileEmpty + st), ((j / C::kStages) - 1) & 1, 0x50);
      const uint32_t tile = base + C::kOffKV + st * kTileBytesMla;
      const uint32_t bar = bars + 8 * (kMTileRaw + st);
      mbar_arrive_expect_tx(bar, kTileBytesMla);
#pragma unroll
      for (int c = 0; c < 4; ++c) tma_load_3d(tile + c * kChunkBytes, &p.tm_kv, bar, c * 128, (w.tile0 + j) * kTok, w.b);
      tma_load_3d(tile + 4 * kChunkBytes, &p.tm_kv_rope, bar, kLat, (w.tile0 + j) * kTok, w.b);
    }
    return;
  } else {
  // Paged pool (or a slab sent this way): a warp copies 12 (or 16) whole token rows of the tile, 36 pieces of
  // 16 bytes each.  Lane k < 12 holds the pool slot of the warp's k-th row, fetched one tile ahead, so that no
  // copy waits for an index load of its own.
  const uint8_t* kv = static_cast<const uint8_t*>(p.kv);
  const int idx0 = w.idx0;
  const int warp = lt >> 5, lane = lt & 31;
  constexpr int kRowsPerWarp = kTok / (kCopyThreads / 32);  // 12 (eight warps) or 16 (six)
  constexpr int kPiecesPerWarp = kRowsPerWarp * 36;         // 432 = 13.5 warp-wide copies, or 576 = 18
  auto slot_of = [&](int j) -> long long {  // slot of row `lane` of this warp in tile j; -1: past the end
    const int tok_abs = (w.tile0 + j) * kTok + warp * kRowsPerWarp + lane;
    if (lane >= kRowsPerWarp || j >= w.tiles || tok_abs >= w.end_max) return -1;
    return p.kv_indices != nullptr ? static_cast<long long>(p.kv_indices[idx0 + tok_abs])
                                   : static_cast<long long>(w.b) * p.seq + tok_abs;
  };
  // where this lane's pieces go and come from does not change from tile to tile
  constexpr int kRoundsCopy = (kPiecesPerWarp + 31) / 32;  // 14 or 18
  uint32_t dst_off[kRoundsCopy];
#pragma unroll
  for (int i = 0; i < kRoundsCopy; ++i) {
    const int piece = i * 32 + lane;
    const int row = piece / 36;  // row == kRowsPerWarp only in the last, half-empty round
    dst_off[i] = kv_off(warp * kRowsPerWarp + (row < kRowsPerWarp ? row : 0), static_cast<uint32_t>(piece % 36) * 16u);
  }
  long long slot_next = slot_of(0);
  for (int j = 0; j < w.tiles; ++j) {
    const int st = j % C::kStages;
    const long long slot_mine = slot_next;
    slot_next = slot_of(j + 1);
    if (j >= C::kStages) MA_WAIT_SLEEP(64, bars + 8 * (kMTileEmpty + st), ((j / C::kStages) - 1) & 1, 0x50);
    const uint32_t tile = base + C::kOffKV + st * kTileBytesMla;
#pragma unroll
    for (int i = 0; i < kRoundsCopy; ++i) {
      const int piece = i * 32 + lane;
      const int row = piece / 36, q = piece % 36;
      const long long slot = __shfl_sync(0xffffffffu, slot_mine, row < kRowsPerWarp ? row : 0);
      // rows past the end are zero-filled (source size 0)
      if (piece < kPiecesPerWarp)
        cp_async16(tile + dst_off[i], kv + (slot < 0 ? 0 : slot) * kRowBytes + static_cast<uint32_t>(q) * 16u,
                   slot < 0 ? 0u : 16u);
    }
    cp_async_arrive(bars + 8 * (kMTileRaw + st));
  }
  }
}

__device__ __forceinline__ uint64_t make_desc_hi(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
// Shared-memory descriptor of a K-major operand stored as [rows][64 B] under the 64-byte swizzle.
__device__ __forceinline__ uint64_t make_desc_sw64(uint32_t lo) {
  return make_desc_hi(lo, (512u >> 4) | (1u << 14) | (4u << 29));  // SBO = 8 rows x 64 B, version 1, swizzle mode 64 B
}

// ---------------------------------------------------------------------------
// MMA issuer (one thread)
// ---------------------------------------------------------------------------
template <int kPos, bool kTma>
__device__ __forceinline__ void role_mma(const Work& w, uint8_t* smem, uint32_t base, uint32_t tmem, const WaitCtx& ctx) {
  using C = Cfg<kPos>;
  constexpr uint32_t kFmtE4M3 = 0;
  constexpr uint32_t idesc_qk = umma_idesc(kFmtE4M3, kFmtE4M3, 0, 0, kMmaM, C::kN);
  constexpr uint32_t idesc_pv = umma_idesc(kFmtE4M3, kFmtE4M3, 1, 1, kMmaM, C::kN);
  const uint32_t bars = base + C::kOffBars;
  const uint32_t qt_lo = desc_lo_kmajor(base + C::kOffQT);
  const int n = w.tiles;
  // Q K^T runs with M = 128 over chunks of 96 token rows: rows 96..127 of the A operand are the first 32 rows
  // of whatever follows the chunk in shared memory.  A row of D depends on its own row of A only, so this
  // fills S^T rows 96..127 with numbers nobody reads.  P V has the tokens on K: three steps of 32, exact.
  auto issue_qk = [&](int j, uint32_t done_bar) {
    const uint32_t tile = base + C::kOffKV + (j % C::kStages) * kTileBytesMla;
    const uint32_t a_lo = desc_lo_kmajor(tile);
    const uint32_t d = tmem + (j & 1) * C::kN;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        umma_ss_f8(d, make_desc(a_lo + ((c * kChunkBytes + ks * 32) >> 4)),
                   make_desc(qt_lo + ((c * C::kN * 128 + ks * 32) >> 4)), idesc_qk, (c | ks) != 0 ? 1u : 0u);
      }
    }
    // the rope chunk: 64-byte rows under the 64-byte swizzle (8 rows = 512 bytes); Q^T keeps 128-byte rows
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      umma_ss_f8(d, make_desc_sw64(a_lo + ((4 * kChunkBytes + ks * 32) >> 4)),
                 make_desc(qt_lo + ((4 * C::kN * 128 + ks * 32) >> 4)), idesc_qk, 1u);
    }
    umma_commit(done_bar);
  };
  auto issue_pv = [&](int j) {
    // a saturation correction may have put something into O^T before the first P V (role_softmax)
    const bool keep = j > 0 || *reinterpret_cast<volatile int*>(smem + C::kOffSatCnt + 4 * kMaxStagesMla) != 0;
    const uint32_t tile = base + C::kOffKV + (j % C::kStages) * kTileBytesMla;
    // B = P, MN-major: rows of kN bytes per token, 8 tokens per swizzle atom, 32 tokens per step
    constexpr uint32_t pt_hi = ((8u * C::kN) >> 4) | (1u << 14) | ((C::kN == 32 ? 6u : 4u) << 29);
    const uint32_t pt_lo = (((base + C::kOffPT + (j & 1) * C::kN * 128) & 0x3FFFFu) >> 4) | (1u << 16);
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      // A = 128 latent bytes of every token row (M), 32 token rows per step (K): MN-major, one swizzle atom wide
      const uint32_t a_lo = desc_lo_mnmajor<kTok>(tile + mt * kChunkBytes);
#pragma unroll
      for (int ks = 0; ks < kTok / 32; ++ks) {
        umma_ss_f8(tmem + (2 + mt) * C::kN, make_desc(a_lo + ((ks * 32 * 128) >> 4)),
                   make_desc_hi(pt_lo + ((ks * 32 * C::kN) >> 4), pt_hi),
                   idesc_pv, (keep || ks > 0) ? 1u : 0u);
      }
    }
    umma_commit(bars + 8 * (kMTileEmpty + (j % C::kStages)));
    umma_commit(bars + 8 * (kMPvDone + (j & 1)));
  };
  // Whatever is ready is issued: Q K^T of tile i needs the tile and the S buffer (read out by the softmax of
  // tile i - 2, known from its P arrival, i.e. once P V (i - 2) has been issued); P V of tile j needs P(j).
  int qk_i = 0, pv_i = 0;
  uint32_t redos = 0;
  uint32_t idle = 0;
  uint64_t t0 = 0;
  while (pv_i < n) {
    bool progressed = false;
    if (qk_i < n && qk_i - pv_i < 2 &&
        mbar_test_wait(bars + 8 * (kMTileRaw + (qk_i % C::kStages)), (qk_i / C::kStages) & 1)) {
      if constexpr (!kTma) fence_proxy_async_smem();
      tc_fence_after_sync();
      issue_qk(qk_i, bars + 8 * (kMSFull + (qk_i & 1)));
      ++qk_i;
      progressed = true;
    }
    auto try_pv = [&]() {
      if (pv_i < qk_i && mbar_test_wait(bars + 8 * (kMPFull + (pv_i & 1)), (pv_i >> 1) & 1)) {
        tc_fence_after_sync();
        issue_pv(pv_i);
        ++pv_i;
        progressed = true;
      }
    };
    try_pv();
    // The softmax warps rewrote rows of the tile they hold (saturated e4m3-fnuz codes): its scores once more.
    // They hold the oldest tile without P V; the P of the tile before it is complete by now, but this thread may
    // not have seen it yet, hence the second look.
    if (mbar_test_wait(bars + 8 * kMRedoReq, redos & 1)) {
      try_pv();
      tc_fence_after_sync();
      issue_qk(pv_i, bars + 8 * kMRedoDone);
      ++redos;
      progressed = true;
    }
    if (progressed) {
      idle = 0;
      t0 = 0;
    } else if ((++idle & 0x3FFu) == 0u) {  // bounded like every other wait
      if (*ctx.abort) return;
      if (ctx.watch_status && ctx.status != nullptr && *reinterpret_cast<volatile uint32_t*>(ctx.status) != 0u) {
        *ctx.abort = 1;
        return;
      }
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > ctx.limit_ns) {
        record_error(ctx.status, kErrWaitTimeout, 0x60, (static_cast<uint32_t>(qk_i) << 16) | static_cast<uint32_t>(pv_i));
        *ctx.abort = 1;
        return;
      }
    }
  }
}

// Orders floats as signed integers (for redux.sync.max).
__device__ __forceinline__ int float_key(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7FFFFFFF);
}
__device__ __forceinline__ float key_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7FFFFFFF)); }

template <int kCols>
__device__ __forceinline__ void tmem_load_cols(uint32_t taddr, uint32_t (&d)[kCols]) {
  if constexpr (kCols == 32) {
    tmem_ld32_sync(taddr, d);
  } else {
    tmem_ld64_sync(taddr, d);
  }
}

// ---------------------------------------------------------------------------
// softmax warps: thread = token of the tile (S^T lanes) and = output dimension (O^T lanes)
//
// The reference maximum of a row moves lazily (by more than tau above it, and on the first tile), so that
// p <= 2^tau = 256 fits e4m3.  A tile normally needs no maximum at all: every thread checks its own scores
// against reference + tau, the four warps exchange one flag, and only a raised flag sends the CTA through
// the exact row maxima (redux + a second exchange) and the rescale of O^T.  All of this is uniform over the
// CTA: every thread holds the same reference maxima.  The softmax denominator is summed per thread (one
// token each) over all tiles and reduced across the threads once, in the epilogue.
// ---------------------------------------------------------------------------
template <int kPos>
__device__ __forceinline__ void role_softmax(const MlaParams& p, const Work& w, uint8_t* smem, uint32_t base,
                                             uint32_t tmem, int tid, const WaitCtx& ctx) {
  using C = Cfg<kPos>;
  // A group of four warps owns one draft position: R = 16 query rows (heads), whose two e4m3 terms sit in
  // accumulator columns [row0, row0 + 16) and [RT + row0, RT + row0 + 16) of S^T and of every O^T tile.
  constexpr int R = kHeadsMax, RT = C::kRows, N = C::kN, kW = 4 * kPos;
  const int group = tid >> 7, tl = tid & 127;
  const int warp = tl >> 5, lane = tl & 31, gwarp = tid >> 5;
  const uint32_t row0 = group * R;
  const uint32_t bars = base + C::kOffBars;
  const uint32_t lane_sel = static_cast<uint32_t>(tl & ~31) << 16;
  const float* row_scale = reinterpret_cast<const float*>(smem + C::kOffRowScale) + row0;
  float* mx = reinterpret_cast<float*>(smem + C::kOffMx);          // [2][groups][4][R] row maxima of a tile, per warp
  volatile int* flags = reinterpret_cast<volatile int*>(smem + C::kOffFlags);  // [2][kW] bit 0: a score is above reference + tau; bit 1: NaN
  float* l_part = reinterpret_cast<float*>(smem + C::kOffL) + group * 4 * R;  // [4][R] per-warp denominators (epilogue)
  const int n = w.tiles;
  // tokens [0, limit) are visible to this group's position; a group past the window sees none and writes nothing
  const bool pos_live = w.pos0 + group < w.q_len;
  const int limit = pos_live ? w.len - w.q_len + w.pos0 + group + 1 : 0;
  auto ld_pair = [&](uint32_t taddr, uint32_t (&r)[2 * R]) {  // taddr: column 0 of an N-column block
    if constexpr (kPos == 1) {
      tmem_ld32_sync(taddr, r);
    } else {
      tmem_ld16x2_sync(taddr + row0, taddr + RT + row0, r);
    }
  };
  auto st_pair = [&](uint32_t taddr, const uint32_t (&r)[2 * R]) {
    if constexpr (kPos == 1) {
      tmem_st32(taddr, r);
    } else {
      tmem_st16x2(taddr + row0, taddr + RT + row0, r);
    }
  };
  float m_ref[R], l_sum[R];
#pragma unroll
  for (int r = 0; r < R; ++r) m_ref[r] = 0.f, l_sum[r] = 0.f;
  uint32_t slow = 0;          // exact-maximum rounds so far (phase of their barrier)
  uint32_t n_sat_rounds = 0;  // tiles with saturated entries so far (phase of their barrier)
  uint32_t redos = 0;         // Q K^T repetitions so far (phase of their barriers)

  for (int j = 0; j < n; ++j) {
    const int buf = j & 1, par = (j >> 1) & 1;
    MA_WAIT_WARP(bars + 8 * (kMSFull + buf), par, 0x70);
    tc_fence_after_sync();
    uint32_t d[2 * R];
    ld_pair(tmem + buf * N + lane_sel, d);
    const int tok_abs = (w.tile0 + j) * kTok + tl;
    const int st = j % C::kStages;
    const uint32_t* sat = reinterpret_cast<const uint32_t*>(smem + C::kOffSat) + st * C::kSatCap;
    // e4m3-fnuz: a byte 0x7F / 0xFF (+-240 there, NaN to the tensor core) in this thread's token row shows as NaN
    // scores of the token.
    bool tok_nan = false;
    if (p.use_tma && tl < kTok && tok_abs >= w.end_max) {
      // Box loads bring whole rows, also those between the end of what this CTA may see and the end of the slab:
      // another position's tokens, or bytes nobody wrote.  Their scores are masked below, but P V would multiply
      // p = 0 with whatever NaN code they hold: zero the row (the 16-byte copies of a pool do that themselves).
      uint8_t* tile = smem + C::kOffKV + st * kTileBytesMla;
#pragma unroll 4
      for (uint32_t col0 = 0; col0 < kRowBytes; col0 += 16)
        *reinterpret_cast<uint4*>(tile + kv_off(tl, col0)) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (p.kv_format == 0 && tl < kTok && tok_abs < limit) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = __uint_as_float(d[r]) + __uint_as_float(d[R + r]);
        tok_nan = tok_nan || (v != v);
      }
    }
    int n_sat = 0;
    float s[R];
    float over = -INFINITY;
    float scale_r[R];  // four 16-byte loads instead of sixteen scalar ones: shared-memory instructions are what this loop waits for
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const float4 q4 = *reinterpret_cast<const float4*>(row_scale + r);
      scale_r[r] = q4.x, scale_r[r + 1] = q4.y, scale_r[r + 2] = q4.z, scale_r[r + 3] = q4.w;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float v = (__uint_as_float(d[r]) + __uint_as_float(d[R + r])) * scale_r[r];
      s[r] = (tl < kTok && tok_abs < limit) ? v : -INFINITY;
      over = fmaxf(over, s[r] - m_ref[r]);
    }
    const bool warp_over = __any_sync(0xffffffffu, over > kTauMla) || j == 0;
    const bool warp_nan = __any_sync(0xffffffffu, tok_nan);
    if (lane == 0) {
      flags[buf * kW + gwarp] = (warp_over ? 1 : 0) | (warp_nan ? 2 : 0);
      mbar_arrive(bars + 8 * (kMFlag + buf));
    }
    MA_WAIT_WARP(bars + 8 * (kMFlag + buf), par, 0x71);
    // overflow is this group's own business, a NaN (the tile is rewritten and multiplied again) everybody's
    int tile_flags = 0;
#pragma unroll
    for (int k = 0; k < kW; ++k) tile_flags |= flags[buf * kW + k] & ((k >> 2) == group ? 3 : 2);
    if (tile_flags & 2) {  // uniform over the CTA
      // Rewrite the two codes one down (+-224) in the rows that showed NaN, list the entries for the corrections
      // by hand, and have the MMA thread run the tile's Q K^T again on the rewritten bytes.
      // (a token that several positions see is rewritten by the first of them)
      if (tok_nan && (group == 0 || tok_abs >= limit - group)) {
        int* sat_cnt = reinterpret_cast<int*>(smem + C::kOffSatCnt) + st;
        uint32_t* sat_w = reinterpret_cast<uint32_t*>(smem + C::kOffSat) + st * C::kSatCap;
        uint8_t* tile = smem + C::kOffKV + st * kTileBytesMla;
        for (int piece = 0; piece < kRowBytes / 16; ++piece) {
          const uint32_t col0 = piece * 16;
          uint4* ptr = reinterpret_cast<uint4*>(tile + kv_off(tl, col0));
          uint4 v = *ptr;
          uint32_t* x = reinterpret_cast<uint32_t*>(&v);
          bool any = false;
          for (int k = 0; k < 4; ++k) {
            const uint32_t hit = ((x[k] & 0x7F7F7F7Fu) + 0x01010101u) & 0x80808080u;
            if (hit == 0u) continue;
            any = true;
            for (int b = 0; b < 4; ++b) {
              if (((hit >> (8 * b)) & 0x80u) == 0u) continue;
              const int slot = atomicAdd(sat_cnt, 1);
              if (slot < C::kSatCap) sat_w[slot] = tl | ((col0 + k * 4 + b) << 7) | (((x[k] >> (8 * b + 7)) & 1u) << 17);
            }
            x[k] -= hit >> 7;
          }
          if (any) *ptr = v;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * kMRedoReq);
      MA_WAIT_WARP(bars + 8 * kMRedoDone, redos & 1, 0x7A);
      ++redos;
      tc_fence_after_sync();
      ld_pair(tmem + buf * N + lane_sel, d);
      n_sat = min(*reinterpret_cast<volatile int*>(smem + C::kOffSatCnt + 4 * st), C::kSatCap);
      // the tensor core saw +-448 where the cache says +-480 (in e4m3 units): add the rest of this token by hand
      for (int e = 0; e < n_sat; ++e) {
        const uint32_t ent = sat[e];
        if (static_cast<int>(ent & 127u) != tl) continue;
        const uint32_t col = (ent >> 7) & 1023u;
        const float rest = (ent >> 17) ? -kSatResidual : kSatResidual;
        const uint8_t* qt = smem + C::kOffQT + (col >> 7) * (N * 128);
#pragma unroll
        for (int r = 0; r < R; r += 2) {  // the two terms of rows r and r + 1 at this column
          const float2 a = from_e4m3x2(qt[swz128(row0 + r, col & 127u)] | (qt[swz128(row0 + r + 1, col & 127u)] << 8));
          const float2 b = from_e4m3x2(qt[swz128(RT + row0 + r, col & 127u)] | (qt[swz128(RT + row0 + r + 1, col & 127u)] << 8));
          d[r] = __float_as_uint(__uint_as_float(d[r]) + rest * (a.x + b.x));
          d[r + 1] = __float_as_uint(__uint_as_float(d[r + 1]) + rest * (a.y + b.y));
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = (__uint_as_float(d[r]) + __uint_as_float(d[R + r])) * scale_r[r];
        s[r] = (tl < kTok && tok_abs < limit) ? v : -INFINITY;
      }
      tile_flags |= 1;  // the maxima were judged on NaN: take the exact path
    }
    if ((tile_flags & 1) != 0) {
      // exact row maxima of the tile: redux within the warp, shared memory across the four warps
      const int sb = slow & 1;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int k = __reduce_max_sync(0xffffffffu, float_key(s[r]));
        if (lane == (r & 31)) mx[((sb * kPos + group) * 4 + warp) * R + r] = key_float(k);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kMMx + sb + 2 * group));
      MA_WAIT_WARP(bars + 8 * (kMMx + sb + 2 * group), (slow >> 1) & 1, 0x75);
      ++slow;
      float alpha[R];
      bool moved = false;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float* m4 = mx + (sb * kPos + group) * 4 * R + r;
        const float m_tile = fmaxf(fmaxf(m4[0], m4[R]), fmaxf(m4[2 * R], m4[3 * R]));
        float m_new = m_ref[r];
        if (j == 0) {
          m_new = (m_tile == -INFINITY) ? 0.f : m_tile;
        } else if (m_tile - m_ref[r] > kTauMla) {
          m_new = m_tile;
        }
        alpha[r] = ex2_approx(m_ref[r] - m_new);
        moved = moved || (m_new != m_ref[r]);
        m_ref[r] = m_new;
        l_sum[r] *= alpha[r];
      }
      if (j > 0 && moved) {
        MA_WAIT_WARP(bars + 8 * (kMPvDone + ((j - 1) & 1)), ((j - 1) >> 1) & 1, 0x72);
        tc_fence_after_sync();
#pragma unroll 1
        for (int mt = 0; mt < 4; ++mt) {
          uint32_t o[2 * R];
          ld_pair(tmem + (2 + mt) * N + lane_sel, o);
#pragma unroll
          for (int c = 0; c < 2 * R; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c % R]);
          st_pair(tmem + (2 + mt) * N + lane_sel, o);
        }
        tmem_st_wait();
        tc_fence_before_sync();
      }
    }
    // probabilities as two e4m3 terms each; rows are converted in pairs
    uint32_t t1[R / 2], t2[R / 2];
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      const float p0 = ex2_approx(s[r] - m_ref[r]), p1 = ex2_approx(s[r + 1] - m_ref[r + 1]);
      l_sum[r] += p0;
      l_sum[r + 1] += p1;
      t1[r / 2] = to_e4m3x2(p0, p1);
      const float2 back = from_e4m3x2(t1[r / 2]);
      t2[r / 2] = to_e4m3x2(p0 - back.x, p1 - back.y);
    }
    if (j >= 2) MA_WAIT_WARP(bars + 8 * (kMPvDone + buf), ((j - 2) >> 1) & 1, 0x73);
    uint8_t* pt = smem + C::kOffPT + buf * N * 128;
    if (tl < kTok) {  // the token's 16 first terms and 16 second terms: two 16-byte stores
      *reinterpret_cast<uint4*>(pt + p_off<N>(tl, row0)) =
          make_uint4(t1[0] | (t1[1] << 16), t1[2] | (t1[3] << 16), t1[4] | (t1[5] << 16), t1[6] | (t1[7] << 16));
      *reinterpret_cast<uint4*>(pt + p_off<N>(tl, RT + row0)) =
          make_uint4(t2[0] | (t2[1] << 16), t2[2] | (t2[3] << 16), t2[4] | (t2[5] << 16), t2[6] | (t2[7] << 16));
    }
    if (n_sat > 0) {  // uniform over the CTA
      // O^T misses p * (+-32) for every listed entry with a latent column.  The entry's output dimension is a
      // lane of tensor memory: the warp that owns the lane patches it, with p read back from P^T (both terms
      // keep their own accumulator column).  P^T must be complete, and no P V may be in flight on O^T.
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kMSat + (n_sat_rounds & 1)));
      MA_WAIT_WARP(bars + 8 * (kMSat + (n_sat_rounds & 1)), (n_sat_rounds >> 1) & 1, 0x77);
      ++n_sat_rounds;
      if (j > 0) {
        MA_WAIT_WARP(bars + 8 * (kMPvDone + ((j - 1) & 1)), ((j - 1) >> 1) & 1, 0x78);
        tc_fence_after_sync();
      } else {
        // The first P V of a part normally overwrites O^T.  Start it from zero here and tell the MMA thread to
        // accumulate instead, so that the patches below survive.
        uint32_t zero[2 * R];
#pragma unroll
        for (int c = 0; c < 2 * R; ++c) zero[c] = 0u;
#pragma unroll 1
        for (int mt = 0; mt < 4; ++mt) st_pair(tmem + (2 + mt) * N + lane_sel, zero);
        tmem_st_wait();
        if (tl == 0) *reinterpret_cast<volatile int*>(smem + C::kOffSatCnt + 4 * kMaxStagesMla) = 1;
      }
      for (int e = 0; e < n_sat; ++e) {
        const uint32_t ent = sat[e];
        const uint32_t tok = ent & 127u, col = (ent >> 7) & 1023u;
        if (col >= static_cast<uint32_t>(kLat) || ((col >> 5) & 3u) != static_cast<uint32_t>(warp)) continue;  // warp-uniform
        const float rest = (ent >> 17) ? -kSatResidual : kSatResidual;
        const uint32_t taddr = tmem + (2 + (col >> 7)) * N + lane_sel;
        uint32_t o[2 * R];
        ld_pair(taddr, o);
        if (static_cast<uint32_t>(lane) == (col & 31u)) {
#pragma unroll
          for (int c = 0; c < 2 * R; c += 2) {
            const uint32_t pcol = (c < R ? row0 : RT + row0 - R) + c;  // accumulator column c of this group within P
            const float2 pq = from_e4m3x2(*reinterpret_cast<const uint16_t*>(pt + p_off<N>(tok, pcol)));
            o[c] = __float_as_uint(__uint_as_float(o[c]) + rest * pq.x);
            o[c + 1] = __float_as_uint(__uint_as_float(o[c + 1]) + rest * pq.y);
          }
        }
        st_pair(taddr, o);
        tmem_st_wait();
      }
      tc_fence_before_sync();
      if (tl == 0) *reinterpret_cast<volatile int*>(smem + C::kOffSatCnt + 4 * st) = 0;  // the stage's next tile starts empty
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    mbar_arrive(bars + 8 * (kMPFull + buf));
  }

  // epilogue.  With one KV part the CTA finishes its rows itself (normalise, scale back, round to bf16); with
  // several it leaves un-normalised fp32 outputs, reference maxima and denominators: in its own shared memory
  // for the merge inside the cluster (cluster_merge below), else in global memory for mla_merge_kernel.
  const size_t slot = blockIdx.x;
  const bool direct = p.parts == 1, in_smem = p.cluster_merge != 0;
  float* part_o = in_smem ? reinterpret_cast<float*>(smem + C::kOffPartO) + row0 * kLat
                          : p.part_o + (slot * RT + row0) * kLat;  // this group's 16 rows
  float2* part_ml = in_smem ? reinterpret_cast<float2*>(smem + C::kOffPartMl) + row0
                            : reinterpret_cast<float2*>(p.part_ml) + slot * RT + row0;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.o_lat);
  auto out_row = [&](int r) {  // row r of this group: its position, head r
    return ((static_cast<size_t>(w.brow) * w.q_len + w.pos0 + group) * w.heads + r) * kLat;
  };
  auto row_live = [&](int r) { return r < w.heads && pos_live; };
  if (n == 0) {  // no token in range (an empty part, or a request without tokens)
    if (direct) {
      for (int r = 0; r < R; ++r)
        if (row_live(r))
          for (int mt = 0; mt < 4; ++mt) out[out_row(r) + mt * 128 + tl] = __float2bfloat16_rn(0.f);
    } else if (tl < R) {
      part_ml[tl] = make_float2(-INFINITY, 0.f);
    }
    return;
  }
  // denominators: sum over the 128 tokens-of-a-tile threads, then across the four warps through shared memory
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v = l_sum[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == (r & 31)) l_part[warp * R + r] = v;
  }
  __syncwarp();
  if (lane == 0) mbar_arrive(bars + 8 * (kMEpi + group));
  MA_WAIT_WARP(bars + 8 * (kMEpi + group), 0, 0x76);
  const float fmt = p.kv_format == 0 ? 2.f : 1.f;
  float inv[R];  // per row: kv_scale / (format factor x denominator); 0 for a row without tokens
  bool live[R];
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    float4 l4 = *reinterpret_cast<const float4*>(l_part + r);
#pragma unroll
    for (int q = 1; q < 4; ++q) {
      const float4 x = *reinterpret_cast<const float4*>(l_part + q * R + r);
      l4.x += x.x, l4.y += x.y, l4.z += x.z, l4.w += x.w;
    }
    const float l[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      inv[r + q] = (l[q] > 0.f || l[q] != l[q]) ? p.kv_scale / (fmt * l[q]) : 0.f;
      live[r + q] = row_live(r + q);
    }
  }
  // (all of the above ran while the last P V was still at work)
  MA_WAIT_WARP(bars + 8 * (kMPvDone + ((n - 1) & 1)), ((n - 1) >> 1) & 1, 0x74);
  tc_fence_after_sync();
#pragma unroll 1
  for (int mt = 0; mt < 4; ++mt) {
    uint32_t o[2 * R];
    ld_pair(tmem + (2 + mt) * N + lane_sel, o);
    if (direct) {
      __nv_bfloat16* dst = out + out_row(0) + mt * 128 + tl;  // rows of one position are consecutive heads
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float v = __uint_as_float(o[r]) + __uint_as_float(o[R + r]);
        if (live[r]) dst[static_cast<size_t>(r) * kLat] = __float2bfloat16_rn(v * inv[r]);
      }
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r)
        part_o[static_cast<size_t>(r) * kLat + mt * 128 + tl] = __uint_as_float(o[r]) + __uint_as_float(o[R + r]);
    }
  }
  if (!direct && tl < R) {
    const float l = (l_part[tl] + l_part[R + tl]) + (l_part[2 * R + tl] + l_part[3 * R + tl]);
    float m = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (r == tl) m = m_ref[r];
    part_ml[tl] = make_float2(m, l);
  }
}

// ---------------------------------------------------------------------------
// merge inside a cluster: the P parts of a request are the CTAs of one thread-block cluster; each has left its
// partial result in its own shared memory (role_softmax) and all have passed a cluster barrier.  Part c finishes
// head rows c, c + P, ... of every position of the CTA: out = sum_q 2^(m_q - M) O_q / sum_q 2^(m_q - M) l_q,
// scaled back, rounded to bf16.  A thread takes four dimensions of a row; the loads of a chunk of rows from all
// parts (at most 16 x 16 bytes and 16 x 8 bytes per thread) are issued together.
// ---------------------------------------------------------------------------
template <int kPos, int P>
__device__ __forceinline__ void cluster_merge_rows(const MlaParams& p, const Work& w, uint32_t base, int tid) {
  using C = Cfg<kPos>;
  constexpr int R = kHeadsMax, kRowsMax = (R + P - 1) / P, kChunk = R / P;
  static_assert(P >= 2 && P <= 8 && kChunk >= 2, "cluster of two to eight parts");
  const int group = tid >> 7, tl = tid & 127;
  if (w.pos0 + group >= w.q_len) return;  // a position past the window has no output rows
  uint32_t o_at[P], ml_at[P];
#pragma unroll
  for (int q = 0; q < P; ++q) {
    const uint32_t there = cluster_map(base, q);
    o_at[q] = there + C::kOffPartO + (group * R * kLat + tl * 4) * 4;
    ml_at[q] = there + C::kOffPartMl + group * R * 8;
  }
  const float scale_back = p.kv_scale / (p.kv_format == 0 ? 2.f : 1.f);
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.o_lat) +
                       (static_cast<size_t>(w.brow) * w.q_len + w.pos0 + group) * w.heads * kLat + tl * 4;
  auto part_live = [](float2 v) { return v.y > 0.f || v.y != v.y; };  // a part without tokens has denominator 0
#pragma unroll
  for (int k0 = 0; k0 < kRowsMax; k0 += kChunk) {
    float2 ml[kChunk][P];
    float4 o[kChunk][P];
#pragma unroll
    for (int k = 0; k < kChunk; ++k) {
      const int r = w.part + (k0 + k) * P;
      const bool row = k0 + k < kRowsMax && r < w.heads;  // uniform over the CTA
#pragma unroll
      for (int q = 0; q < P; ++q) {
        ml[k][q] = make_float2(-INFINITY, 0.f);
        o[k][q] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row) {
          ml[k][q] = ld_cluster_f32x2(ml_at[q] + r * 8);
          o[k][q] = ld_cluster_f32x4(o_at[q] + r * (kLat * 4));  // never written by a part without tokens: not used then
        }
      }
    }
#pragma unroll
    for (int k = 0; k < kChunk; ++k) {
      const int r = w.part + (k0 + k) * P;
      if (!(k0 + k < kRowsMax && r < w.heads)) continue;
      float m_all = -INFINITY;
#pragma unroll
      for (int q = 0; q < P; ++q)
        if (part_live(ml[k][q])) m_all = fmaxf(m_all, ml[k][q].x);
      float l_all = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < P; ++q) {
        if (!part_live(ml[k][q])) continue;
        const float wgt = ex2_approx(ml[k][q].x - m_all);
        l_all += wgt * ml[k][q].y;
        acc.x += wgt * o[k][q].x, acc.y += wgt * o[k][q].y, acc.z += wgt * o[k][q].z, acc.w += wgt * o[k][q].w;
      }
      const float inv = (l_all > 0.f || l_all != l_all) ? scale_back / l_all : 0.f;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      *reinterpret_cast<uint2*>(out + static_cast<size_t>(r) * kLat) =
          make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
  }
}

__device__ __forceinline__ void cluster_sync() {
  __syncwarp();
  cluster_arrive_release();
  cluster_wait_acquire();
}

template <int kPos>
__device__ __forceinline__ void cluster_merge(const MlaParams& p, const Work& w, uint32_t base, int tid) {
  switch (p.parts) {
    case 2: cluster_merge_rows<kPos, 2>(p, w, base, tid); break;
    case 3: cluster_merge_rows<kPos, 3>(p, w, base, tid); break;
    case 4: cluster_merge_rows<kPos, 4>(p, w, base, tid); break;
    case 5: cluster_merge_rows<kPos, 5>(p, w, base, tid); break;
    case 6: cluster_merge_rows<kPos, 6>(p, w, base, tid); break;
    case 7: cluster_merge_rows<kPos, 7>(p, w, base, tid); break;
    case 8: cluster_merge_rows<kPos, 8>(p, w, base, tid); break;
    default: break;
  }
}

template <int kPos, bool kTma>
__global__ void __launch_bounds__(block_threads(kTma, kPos), 1) mla_decode_kernel(const __grid_constant__ MlaParams p) {
  using C = Cfg<kPos>;
  constexpr int kCopyThreads = copy_threads(kTma, kPos);
  constexpr int R = C::kRows, N = C::kN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = smem_u32(smem);
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Errors of other CTAs are not watched: the status word is cleared by CTA 0 of this launch (below), not before it.
  const WaitCtx ctx{p.status, abort_flag, kWaitLimitNs, false};
  // Programmatic dependent launch, in both directions.  The kernel behind this one in the stream may take its
  // places as SMs become free (a decode call behind a decode call: one CTA per SM, so a CTA of the next call
  // moves in when the one before it leaves; a merge kernel: beside the decode CTAs).  And this kernel sets up
  // barriers and tensor memory while the kernel before it still runs, then waits for it to complete before it
  // touches global memory: the queries, the cache, the lengths and the status word may all be its results.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kMmaWarp = 4 * kPos, kFirstCopyWarp = kMmaWarp + 1;  // softmax warps, MMA warp, copy warps
  if (tid < static_cast<int>(kMNumBars)) {  // one barrier per thread
    const uint32_t i = tid;
    uint32_t count = 1;
    if (i >= kMTileRaw && i < kMTileRaw + kMaxStagesMla) count = kTma ? 1u : static_cast<uint32_t>(kCopyThreads);
    if (i >= kMPFull && i < kMPFull + 2) count = kPos * kSoftmaxThreads;
    if ((i >= kMMx && i < kMMx + 4) || (i >= kMEpi && i < kMEpi + 2)) count = 4;
    if ((i >= kMFlag && i < kMFlag + 2) || (i >= kMSat && i < kMSat + 2) || i == kMRedoReq) count = 4 * kPos;
    mbar_init(base + C::kOffBars + 8 * i, count);
    if (i == 0) abort_flag_s = 0;
    if (i < 4) reinterpret_cast<int*>(smem + C::kOffSatCnt)[i] = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  if constexpr (kTma) {
    if (tid == kFirstCopyWarp * 32) {  // the thread that issues the box loads: their descriptors are kernel parameters
      tma_prefetch_desc(&p.tm_kv);
      tma_prefetch_desc(&p.tm_kv_rope);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const Work w = decode_work(p, kPos);
  // The status word of the call: errors are recorded by compare-and-swap against zero, and the first of them
  // comes after a wait has run out, long after this store.  (Nobody watches the word for other CTAs' errors:
  // a CTA whose wait runs out ends by itself.)
  if (blockIdx.x == 0 && tid == 0) *reinterpret_cast<volatile uint32_t*>(p.status) = 0u;

  // The query rows are fetched first of all, before any KV copy is on its way: behind three tiles of every CTA
  // (25 MB on the whole GPU) these few loads would wait for microseconds.  All are issued before the barrier below.
  const __nv_bfloat16* q_lat = static_cast<const __nv_bfloat16*>(p.q_lat);
  const __nv_bfloat16* q_pe = static_cast<const __nv_bfloat16*>(p.q_pe);
  constexpr int kPrepWarps = kMmaWarp;  // the softmax warps
  const int prep_warp = warp;
  constexpr int kRounds = (R + kPrepWarps - 1) / kPrepWarps;  // 4: a warp takes rows prep_warp, + kPrepWarps, ...
  // A row is 72 pieces of 8 elements (16 bytes): a lane takes pieces lane, lane + 32 and (lanes 0-7) lane + 64.
  // All loads are issued before any is used.
  uint4 vin[kRounds][3];
#pragma unroll
  for (int k = 0; k < kRounds; ++k) {
    const int r = prep_warp + k * kPrepWarps;
    const int pos = w.pos0 + r / kHeadsMax, h = r % kHeadsMax;
    const bool live = warp < kPrepWarps && r < R && h < w.heads && pos < w.q_len;
    const size_t qrow = (static_cast<size_t>(w.brow) * w.q_len + pos) * w.heads + h;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int x = (i * 32 + lane) * 8;
      vin[k][i] = make_uint4(0u, 0u, 0u, 0u);
      if (live && x < kRowBytes)
        vin[k][i] = x < kLat ? *reinterpret_cast<const uint4*>(q_lat + qrow * kLat + x)
                             : *reinterpret_cast<const uint4*>(q_pe + qrow * 64 + (x - kLat));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  // The copy warps start fetching at once; the softmax warps first turn the query rows into Q^T.
  // Pools: the copy warps need few registers, the softmax warps many (setmaxnreg, each inside its own branch so
  // that every role is compiled for its own budget).  The warpgroup that holds the MMA warp (descriptors kept in
  // registers) and the first three copy warps keeps what it was launched with (128).
  if (warp >= kMmaWarp + 4) {  // pools only: warpgroups of copy warps (and the padding warps behind them)
    if constexpr (!kTma) {
      setmaxnreg_dec<kPos == 1 ? 96 : 80>();
      if (warp < kFirstCopyWarp + kCopyThreads / 32) role_copy<kPos, kTma>(p, w, base, tid - kFirstCopyWarp * 32, ctx);
    }
  } else if (warp >= kFirstCopyWarp) {
    role_copy<kPos, kTma>(p, w, base, tid - kFirstCopyWarp * 32, ctx);
  } else if (warp == kMmaWarp) {
    asm volatile("bar.sync 1, %0;" ::"n"((kPrepWarps + 1) * 32) : "memory");  // Q^T is ready
    if (lane == 0) role_mma<kPos, kTma>(w, smem, base, tmem, ctx);
  } else {
    if constexpr (!kTma) setmaxnreg_inc<kPos == 1 ? 192 : 152>();
    // The query data is first looked at from here on (keeps the compiler from waiting for it above the barrier).
#pragma unroll
    for (int k = 0; k < kRounds; ++k)
#pragma unroll
      for (int i = 0; i < 3; ++i)
        asm volatile("" : "+r"(vin[k][i].x), "+r"(vin[k][i].y), "+r"(vin[k][i].z), "+r"(vin[k][i].w));
    // Query rows -> Q^T as two e4m3 terms per row.  Row r = position (r / 16) of the group, head (r % 16); a
    // row is scaled by the power of two that puts its largest magnitude into [128, 256), which makes
    // q * f = q1 + q2 exact for every element within 2^-7 of the largest (8 significant bits = 4 + 4).
    float* row_scale = reinterpret_cast<float*>(smem + C::kOffRowScale);
    uint8_t* qt = smem + C::kOffQT;
    const float fmt = p.kv_format == 0 ? 2.f : 1.f;  // e4m3-fnuz bytes read as e4m3 are twice their value
#pragma unroll
    for (int k = 0; k < kRounds; ++k) {
      const int r = prep_warp + k * kPrepWarps;
      if (r >= R) break;
      float v[3][8];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const uint32_t in[4] = {vin[k][i].x, vin[k][i].y, vin[k][i].z, vin[k][i].w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 two = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[q]));
          v[i][2 * q] = two.x, v[i][2 * q + 1] = two.y;
          amax = fmaxf(amax, fmaxf(fabsf(two.x), fabsf(two.y)));
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      // f = 2^(7 - exponent(amax)); NaN / inf / zero rows keep f = 1
      float f = 1.f;
      if (amax > 0.f && amax < INFINITY) {
        const int e = static_cast<int>((__float_as_uint(amax) >> 23) & 0xFF) - 127;
        f = __uint_as_float(static_cast<uint32_t>(127 + 7 - e) << 23);
      }
      if (lane == 0) row_scale[r] = p.scale * 1.4426950408889634f * p.kv_scale / (fmt * f);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const uint32_t x = (i * 32 + lane) * 8;
        if (x >= kRowBytes) break;
        uint32_t t1[4], t2[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float a = v[i][2 * q] * f, b = v[i][2 * q + 1] * f;
          t1[q] = to_e4m3x2(a, b);
          const float2 back = from_e4m3x2(t1[q]);
          t2[q] = to_e4m3x2(a - back.x, b - back.y);
        }
        const uint32_t chunk = x >> 7, col = x & 127u;  // eight adjacent bytes of one 16-byte piece
        *reinterpret_cast<uint2*>(qt + chunk * (N * 128) + swz128(r, col)) =
            make_uint2(t1[0] | (t1[1] << 16), t1[2] | (t1[3] << 16));
        *reinterpret_cast<uint2*>(qt + chunk * (N * 128) + swz128(R + r, col)) =
            make_uint2(t2[0] | (t2[1] << 16), t2[2] | (t2[3] << 16));
      }
    }
    fence_proxy_async_smem();
    // every one of these warps gets here unconditionally: a plain named barrier is safe
    asm volatile("bar.sync 1, %0;" ::"n"((kPrepWarps + 1) * 32) : "memory");
    role_softmax<kPos>(p, w, smem, base, tmem, tid, ctx);
    if (p.cluster_merge) {
      // Every thread of every part of the request passes two cluster barriers, also after a wait that gave up (its
      // role returned): the first says that all partial results lie in shared memory, the second that nobody reads
      // this CTA's shared memory any more.  Between them the softmax warps merge (here, with their register budget).
      cluster_sync();
      cluster_merge<kPos>(p, w, base, tid);
      cluster_sync();
    }
  }
  tc_fence_before_sync();
  if (p.cluster_merge && warp >= kMmaWarp) {  // the softmax warps' two barriers: see their branch above
    cluster_sync();
    cluster_sync();
  }
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, C::kTmemCols);
}

// ---------------------------------------------------------------------------
// merge of the KV parts: out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p, scaled back, rounded to bf16
// ---------------------------------------------------------------------------
// One CTA per (output row, quarter of the 512 dimensions); its warps (8, or 32 for more than 64 parts) take every
// n-th part, a lane four dimensions (16-byte loads), and the warps' sums meet in shared memory.  With 148 parts of
// one long request every warp then has at most five parts, whose loads are issued together: two trips to L2 (the
// maxima, then the rows) instead of six.
constexpr int kMergeWarps = 8, kMergeWarpsMany = 32;
__global__ void __launch_bounds__(kMergeWarpsMany * 32) mla_merge_kernel(const MlaParams p, int kpos) {
  const int R = kHeadsMax * kpos;
  const int row = blockIdx.x >> 2, quarter = blockIdx.x & 3;  // row = (b, pos, h)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int h = row % p.heads, pos = (row / p.heads) % p.q_len, b = row / (p.heads * p.q_len);
  const int brow = p.rows != nullptr ? p.rows[b] : b;
  const int group = pos / kpos, r = (pos % kpos) * kHeadsMax + h;
  const size_t slot0 = (static_cast<size_t>(b) * p.groups + group) * p.parts;
  const float2* ml = reinterpret_cast<const float2*>(p.part_ml);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the decode grid has completed and its partials are visible
  auto live = [](float2 v) { return v.y > 0.f || v.y != v.y; };  // a part without tokens has denominator 0
  float m_all = -INFINITY;
#pragma unroll 8
  for (int q = lane; q < p.parts; q += 32) {
    const float2 v = ml[(slot0 + q) * R + r];
    if (live(v)) m_all = fmaxf(m_all, v.x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l_all = 0.f;
#pragma unroll 5
  for (int q = warp; q < p.parts; q += nwarps) {
    const float2 v = ml[(slot0 + q) * R + r];
    const bool on = live(v);
    const float wgt = on ? ex2_approx(v.x - m_all) : 0.f;
    // (the outputs of a part without tokens were never written: read all the same, so that no load waits for another)
    const float4 o = *reinterpret_cast<const float4*>(p.part_o + ((slot0 + q) * R + r) * kLat + quarter * 128 + lane * 4);
    l_all += wgt * v.y;
    if (on) acc.x += wgt * o.x, acc.y += wgt * o.y, acc.z += wgt * o.z, acc.w += wgt * o.w;
  }
  __shared__ float4 acc_s[kMergeWarpsMany][32];
  __shared__ float l_s[kMergeWarpsMany];
  acc_s[warp][lane] = acc;
  if (lane == 0) l_s[warp] = l_all;
  __syncthreads();
  if (warp != 0) return;
  for (int k = 1; k < nwarps; ++k) {
    const float4 x = acc_s[k][lane];
    acc.x += x.x, acc.y += x.y, acc.z += x.z, acc.w += x.w;
    l_all += l_s[k];
  }
  const float fmt = p.kv_format == 0 ? 2.f : 1.f;
  const float inv = l_all > 0.f || l_all != l_all ? p.kv_scale / (fmt * l_all) : 0.f;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.o_lat) +
                       ((static_cast<size_t>(brow) * p.q_len + pos) * p.heads + h) * kLat + quarter * 128 + lane * 4;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// The same for up to eight parts that could not be one cluster (more requests than the device holds clusters of
// that size): one CTA of 128 threads per output row, a thread four dimensions, all parts' loads issued together,
// so that the whole merge is one wave of CTAs and one trip to L2.
constexpr int kMergeFewParts = 8;
__global__ void __launch_bounds__(128) mla_merge_few_kernel(const MlaParams p, int kpos) {
  const int R = kHeadsMax * kpos;
  const int row = blockIdx.x;  // (b, pos, h)
  const int h = row % p.heads, pos = (row / p.heads) % p.q_len, b = row / (p.heads * p.q_len);
  const int brow = p.rows != nullptr ? p.rows[b] : b;
  const int group = pos / kpos, r = (pos % kpos) * kHeadsMax + h;
  const size_t slot0 = (static_cast<size_t>(b) * p.groups + group) * p.parts;
  const float2* ml = reinterpret_cast<const float2*>(p.part_ml);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the decode grid has completed and its partials are visible
  float2 v[kMergeFewParts];
  float4 o[kMergeFewParts];
#pragma unroll
  for (int q = 0; q < kMergeFewParts; ++q) {
    const size_t at = (slot0 + (q < p.parts ? q : 0)) * R + r;  // a part without tokens never wrote its outputs: read, not used
    v[q] = ml[at];
    o[q] = *reinterpret_cast<const float4*>(p.part_o + at * kLat + threadIdx.x * 4);
    if (q >= p.parts) v[q] = make_float2(-INFINITY, 0.f);
  }
  auto live = [](float2 x) { return x.y > 0.f || x.y != x.y; };
  float m_all = -INFINITY;
#pragma unroll
  for (int q = 0; q < kMergeFewParts; ++q)
    if (live(v[q])) m_all = fmaxf(m_all, v[q].x);
  float l_all = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int q = 0; q < kMergeFewParts; ++q) {
    if (!live(v[q])) continue;
    const float wgt = ex2_approx(v[q].x - m_all);
    l_all += wgt * v[q].y;
    acc.x += wgt * o[q].x, acc.y += wgt * o[q].y, acc.z += wgt * o[q].z, acc.w += wgt * o[q].w;
  }
  const float fmt = p.kv_format == 0 ? 2.f : 1.f;
  const float inv = l_all > 0.f || l_all != l_all ? p.kv_scale / (fmt * l_all) : 0.f;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.o_lat) +
                       ((static_cast<size_t>(brow) * p.q_len + pos) * p.heads + h) * kLat + threadIdx.x * 4;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

constexpr int kClusterPartsMax = 8;  // the portable cluster size

// How many clusters of `parts` CTAs of this kernel the device holds at once (0: such a cluster cannot be launched).
// Asked once per device and size.
template <int kPos, bool kTma>
int active_clusters(int parts, size_t smem_bytes) {
  constexpr int kDevices = 64;
  static std::atomic<int> known[kDevices][kClusterPartsMax + 1];  // answer + 1; 0: not asked yet
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kDevices) return 0;
  const int have = known[dev][parts].load(std::memory_order_relaxed);
  if (have != 0) return have - 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(parts), cfg.blockDim = dim3(block_threads(kTma, kPos)), cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = parts, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  int n = 0;
  if (cudaFuncSetAttribute(mla_decode_kernel<kPos, kTma>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem_bytes)) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, mla_decode_kernel<kPos, kTma>, &cfg) != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  known[dev][parts].store(n + 1, std::memory_order_relaxed);
  return n;
}

template <int kPos, bool kTma>
cudaError_t launch_one(const MlaParams& params, cudaStream_t stream) {
  using C = Cfg<kPos>;
  constexpr size_t smem_bytes = C::kOffBars + kMNumBars * 8 + 1024;
  static_assert(smem_bytes <= 232448, "shared memory budget of one CTA on sm_100");
  static_assert(C::kOffPartMl + C::kRows * 8 <= C::kStages * kTileBytesMla, "a part's result fits the idle stages");
  cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel<kPos, kTma>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem_bytes));
  if (e != cudaSuccess) return e;
  MlaParams p = params;
  // The parts of a request as one cluster, when all clusters of the call are resident together (a cluster that
  // had to wait for a free group of SMs would cost more than the merge kernel does).
  p.cluster_merge = p.parts >= 2 && p.parts <= kClusterPartsMax &&
                    p.batch * p.groups <= active_clusters<kPos, kTma>(p.parts, smem_bytes);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.batch * p.groups * p.parts), cfg.blockDim = dim3(block_threads(kTma, kPos));
  cfg.dynamicSmemBytes = smem_bytes, cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.cluster_merge ? p.parts : 1, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see the head of the kernel
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 2;
  e = cudaLaunchKernelEx(&cfg, mla_decode_kernel<kPos, kTma>, p);
  if (e != cudaSuccess || p.parts == 1 || p.cluster_merge) return e;  // the decode kernel has written the final output itself
  // The merge is launched as a programmatic dependent: its CTAs may take their places while the parts still
  // run (they are small enough to sit beside a decode CTA) and wait there for the decode grid to complete.
  const bool few = p.parts <= kMergeFewParts;
  cudaLaunchConfig_t mcfg = {};
  mcfg.gridDim = dim3(p.batch * p.q_len * p.heads * (few ? 1 : 4));
  mcfg.blockDim = dim3(few ? 128 : (p.parts > 64 ? kMergeWarpsMany : kMergeWarps) * 32);
  mcfg.stream = stream;
  cudaLaunchAttribute mattr[1];
  mattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  mattr[0].val.programmaticStreamSerializationAllowed = 1;
  mcfg.attrs = mattr, mcfg.numAttrs = 1;
  return few ? cudaLaunchKernelEx(&mcfg, mla_merge_few_kernel, p, static_cast<int>(kPos))
             : cudaLaunchKernelEx(&mcfg, mla_merge_kernel, p, static_cast<int>(kPos));
}

}  // namespace


int mla_cluster_capacity(int pos_per_cta, bool slab, int parts) {
  if (parts < 2 || parts > kClusterPartsMax) return 0;
  auto ask = [&](auto kpos, auto tma) {
    using C = Cfg<decltype(kpos)::value>;
    return active_clusters<decltype(kpos)::value, decltype(tma)::value>(parts, C::kOffBars + kMNumBars * 8 + 1024);
  };
  using One = std::integral_constant<int, 1>;
  using Two = std::integral_constant<int, 2>;
  if (pos_per_cta == 2) return slab ? ask(Two{}, std::true_type{}) : ask(Two{}, std::false_type{});
  return slab ? ask(One{}, std::true_type{}) : ask(One{}, std::false_type{});
}

cudaError_t launch_mla_decode(const MlaParams& p, cudaStream_t stream) {
  if (p.pos_per_cta == 2) return p.use_tma ? launch_one<2, true>(p, stream) : launch_one<2, false>(p, stream);
  if (p.pos_per_cta != 1) return cudaErrorInvalidValue;
  return p.use_tma ? launch_one<1, true>(p, stream) : launch_one<1, false>(p, stream);
}

}  // namespace ma
