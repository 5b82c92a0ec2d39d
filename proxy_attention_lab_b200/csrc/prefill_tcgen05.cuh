// Paged-attention prefill on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// operands staged by TMA / bulk copies, for head_dim 32 / 64 / 80 / 96 / 128 / 256 and tokens_per_page 16 / 32.
//
// Replaces pal_paged_attention_prefill (src/pal_core/kernels/paged_attention/prefill/
// paged_attention_prefill.h.metal:28-389), which handles one key per iteration per simdgroup with
// scalar FMAs, and its launcher (src/pal_core/src/paged_attention_prefill_primitive.cpp:63-167); the
// instantiation grid is the reference's (paged_attention_kernels.metal:111-131): head dims that are not whole
// 64-element swizzle blocks (32, 80, 96) use tiles padded to the next one, whose padding is neither computed on nor stored.
//
// One CTA owns NQ (1 or 2) accumulator tiles of M = 128 rows that read the same K / V tiles: 128 consecutive new
// tokens of two query heads that share a kv head, or - when the heads per kv head are odd in number, e.g. one -
// two consecutive 128-token query tiles of one head.  Keys arrive in tiles of 128 tokens: first the
// paged history, then the dense prompt keys up to the diagonal tile.
//
//   warp 0        producer: Q / dense K / dense V tiles by TMA (128-byte swizzle); history K by TMA gather4
//                 requests, one per (8-element chunk, four pages), each lane issuing its own; history V pages by TMA
//                 with the 32- or 64-byte swizzle (a page row is TPP * 2 bytes); K ring and V ring of kStages each.
//   warp 1        issues every tcgen05.mma and tcgen05.commit: the warp stays converged and the thread picked by
//                 elect.sync issues, which lets the compiler keep descriptors in uniform registers (a branch
//                 on lane 0 instead costs several hundred cycles of the issuing thread per key tile).
//   warps 2..     one softmax warpgroup (128 threads = 128 rows = 128 TMEM lanes) per accumulator tile; at the end
//                 it scales O by 1/l, stages the tile in the tile's (by then unused) Q buffer and writes it out
//                 with TMA stores.
//
// Shared-memory operand layouts and their UMMA descriptors (D = head_dim, B = D / 64 blocks of 64 elements)
//   Q, dense K   [B k-blocks][128 rows][64 el]  K-major, SWIZZLE_128B, SBO 1024; +32 B per K=16 step
//   paged K      The pool keeps a page as [D/8 chunks of 8 el][TPP tokens][16 B]; every (chunk, 8 tokens) is one
//                contiguous 128-byte core matrix.  A page copied whole would put the 8-token groups of a 128-key tile at
//                two different strides (inside a page, across pages), which one descriptor cannot express: with 16-token
//                pages that costs two N = 64 MMAs per K step and permuted S columns (measured: 920 against 968
//                TFLOP/s on the chunked-prefill configuration).  Instead the tile is gathered: viewing the pool as a
//                2-D tensor of (page, kv head, chunk) rows of TPP*16 bytes, one gather4 request puts the same chunk of
//                four pages back to back, so the tile lands as [D/8 chunks][128 tokens][16 B]: K-major, no swizzle,
//                LBO 2048 (next chunk), SBO 128 (next 8 tokens), one N = 128 MMA per K step, S columns in token order,
//                for either page size.
//   paged V      page p at +D*TPP*2 p: [D rows][TPP tokens], rows of TPP*2 bytes, SWIZZLE_32B / 64B K-major,
//                SBO 8 rows; one K = 16 MMA per 16 tokens of a page, N = D.
//   dense V      [B n-blocks][128 tokens][64 el] MN-major, SWIZZLE_128B, LBO 16384, SBO 1024, N = D.
//
// TMEM (512 columns): the S tiles first (fp32 scores, 128 columns each; P, packed two per column in the input type,
// overwrites the first 64 columns of its S tile and is the A operand of the PV MMAs), then the O tiles (D columns
// each).  With two accumulator tiles there is one S tile each (S, then P, then the next S: the chain
// softmax -> PV -> next QK^T of a tile is serial and the two tiles run in anti-phase).  With one accumulator tile
// (SBUF = 2) S is double-buffered: QK^T of key tile j + 1 is issued before PV of tile j and runs under softmax j.
//
// P has the input type (an fp16 A with a bf16 B is rejected by the hardware as an illegal
// instruction).  bf16 rounds P by up to 2^-8 relative; query tiles whose rows see fewer than 256 keys
// get the rounding residual of P through a second set of PV MMAs (see split_p below).
//
// Softmax keeps a possibly stale running maximum and only rescales O when the true maximum has grown
// by more than 2^8 (the result is exact either way: numerator and denominator use the same
// reference point).  Every wait is bounded; on expiry the CTA records a timeout in the workspace
// status word, still releases its TMEM and returns.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

#include "common.cuh"
#include "launch.h"

namespace pal {
namespace {

constexpr int kTile = 128;                      // query rows per accumulator tile and keys per KV tile
constexpr int kBlockBytes = kTile * 64 * 2;     // one 64-element block of a 128-row tile: 128 rows x 128 bytes
constexpr float kRescaleThreshold = 8.0f;       // log2 units

// Everything that depends on the shape: head_dim D, tokens per page TPP, accumulator tiles per CTA NQ, S tiles per
// accumulator SBUF.
template <int D_, int TPP_, int NQ_, int SBUF_>
struct TcCfg {
  static constexpr int D = D_, TPP = TPP_, NQ = NQ_, SBUF = SBUF_;
  static_assert(D == 32 || D == 64 || D == 80 || D == 96 || D == 128 || D == 256, "head_dim must be 32, 64, 80, 96, 128 or 256");
  // Shared-memory tiles are laid out for the head dim rounded up to whole 64-element swizzle blocks (32 -> 64; 80, 96 ->
  // 128).  The tensor maps carry the real head dim, so the columns past it arrive as zeros and leave clipped; the MMAs
  // only step over the real ones (K steps of 16 for QK^T, N = head_dim for PV), so nothing is computed on the padding.
  static constexpr int DP = (D + 63) / 64 * 64;
  static constexpr int kOChunk = D % 32 == 0 ? 32 : 16;  // columns of O moved per tcgen05.ld / st in the rescale and epilogue
  static_assert(TPP == 16 || TPP == 32, "tokens_per_page must be 16 or 32");
  static_assert(SBUF == 1 || (SBUF == 2 && NQ == 1), "S is double-buffered only with one accumulator tile per CTA");
  static constexpr int kBlocks = DP / 64;             // 64-element blocks of a (padded) row
  static constexpr int kPagesPerTile = kTile / TPP;
  static constexpr int kPageBytes = D * TPP * 2;
  static constexpr int kTileBytes = kTile * DP * 2;   // a Q tile, and a ring stage of K or V
  static constexpr int kStages = D <= 128 ? 2 : 1;    // K ring and V ring depth (head_dim 256: 64 KB per tile)
  static constexpr int kChunkBytes = kTile * 16;      // one 8-element chunk of all 128 tokens of a history K tile
  // TMEM columns
  static constexpr int kSCols = NQ * SBUF * kTile;
  static constexpr int kOBase = kSCols;
  static_assert(kSCols + NQ * DP <= 512, "TMEM holds 512 columns");
  // shared memory
  static constexpr int kQ = 0;
  static constexpr int kK = NQ * kTileBytes;
  static constexpr int kV = kK + kStages * kTileBytes;
  static constexpr int kBars = kV + kStages * kTileBytes;
  static constexpr int kUsed = kBars + 256 + 1024;  // + alignment slack
  // at least half of an SM's shared memory, so that two CTAs (each allocating all 512 TMEM columns) never share an SM
  static constexpr int kTotal = kUsed < 116 * 1024 ? 116 * 1024 : kUsed;
};

struct TcParams {
  const void* k_pool;
  const uint32_t* page_table;
  const int32_t* hist_lens;
  const int32_t* cu_seqlens;  // ragged batches: first row of each sequence; null = every sequence has n_new rows
  void* out;
  WaitCtx status;
  int out_f32;  // out holds float32 instead of the input type (stored row by row, not through the TMA path)
  int num_seqs, n_new, num_q_heads, num_kv_heads, group, max_pages_per_seq;
  long long num_pages;
  float scale_log2;
  // History split across CTAs (parts > 1): blockIdx.z counts (sequence, part); part k attends to history tiles
  // [k * split_tiles, (k + 1) * split_tiles), the last part also to the new tokens; every CTA writes the un-normalised
  // fp32 triple of its rows - acc [row][part][D], m (natural-log units) and l [row][part] - and a combine kernel merges them.
  int parts, split_tiles;
  float* part_acc;
  float* part_m;
  float* part_l;
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Four rows of a 2-D tensor (row indices r0..r3, starting at column c0) land back to back in shared memory.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* map, int c0, int r0, int r1, int r2, int r3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_stw(uint32_t taddr, const uint32_t (&r)[32]) { tmem_st32(taddr, r); }
__device__ __forceinline__ void tmem_stw(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st16(taddr, r); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Shared-memory matrix descriptor (start address, leading / stride byte offsets, Blackwell version bit, layout)
enum : uint64_t { kLayoutNone = 0, kLayoutSw128 = 2, kLayoutSw64 = 4, kLayoutSw32 = 6 };
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (layout << 61);
}
// Instruction descriptor for kind::f16 with fp32 accumulation, M = 128, A K-major, N up to 256
__host__ __device__ constexpr uint32_t make_idesc(int n, int a_fmt, int b_fmt, int b_mn_major) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);
}


// ---- softmax building blocks ------------------------------------------------------------------
// Column c of an S tile holds key c of the key tile, for history tiles as well as dense ones.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Row maximum of one thread's 128 raw scores; columns past rel_limit are ignored.
// Four independent chains, the next 32 columns in flight while the current ones are reduced.
template <bool MASK>
__device__ __forceinline__ float tile_row_max(uint32_t tS, int rel_limit) {
  float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  uint32_t cur[32], nxt[32];
  tmem_ld32(tS, cur);
  tmem_wait_ld();
#pragma unroll
  for (int c4 = 0; c4 < 4; ++c4) {
    if (c4 < 3) tmem_ld32(tS + (c4 + 1) * 32, nxt);
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a = __uint_as_float(cur[i + 2 * k]), b = __uint_as_float(cur[i + 2 * k + 1]);
        if (MASK) {
          if (c4 * 32 + i + 2 * k > rel_limit) a = -INFINITY;
          if (c4 * 32 + i + 2 * k + 1 > rel_limit) b = -INFINITY;
        }
        m[k] = max3(m[k], a, b);
      }
    }
    if (c4 < 3) {
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) cur[i] = nxt[i];
    }
  }
  return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// P = exp2(s * scale - m_ref) for one row, written as packed 16-bit pairs over S's first 64 columns,
// a quarter (32 keys -> 16 columns) at a time so that P never overtakes S columns still to be read,
// with the next quarter's scores in flight.  SPLIT also writes the rounding residual P - round(P)
// to columns 64..127 (after the scores living there have been consumed).
template <typename T, bool MASK, bool SPLIT>
__device__ __forceinline__ void tile_exp_store(uint32_t tS, float scale_log2, float m_ref, int rel_limit, float& l_run) {
  using PK = Mma16816<T>;
  float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
  const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_ref, -m_ref);
  uint32_t cur[32], nxt[32];
  uint32_t lo_hold0[16], lo_hold1[16];
  tmem_ld32(tS, cur);
  tmem_wait_ld();
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    if (u < 3) tmem_ld32(tS + 32 * (u + 1), nxt);
    uint32_t hi[16], lo[16];
#pragma unroll
    for (int w = 0; w < 16; ++w) {
      float2 x = __ffma2_rn(make_float2(__uint_as_float(cur[2 * w]), __uint_as_float(cur[2 * w + 1])), sc2, nm2);
      if (MASK) {
        if (32 * u + 2 * w > rel_limit) x.x = -INFINITY;
        if (32 * u + 2 * w + 1 > rel_limit) x.y = -INFINITY;
      }
      const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
      hi[w] = PK::pack(e.x, e.y);
      if (SPLIT) lo[w] = PK::pack_residual(e.x, e.y, hi[w]);
      if (w & 1)
        acc1 = __fadd2_rn(acc1, e);
      else
        acc0 = __fadd2_rn(acc0, e);
    }
    tmem_st16(tS + 16 * u, hi);
    if (SPLIT) {
      if (u == 0) {
#pragma unroll
        for (int w = 0; w < 16; ++w) lo_hold0[w] = lo[w];
      } else if (u == 1) {
#pragma unroll
        for (int w = 0; w < 16; ++w) lo_hold1[w] = lo[w];
      } else if (u == 2) {
        // S columns 64..95 are in `cur`, 96..127 are being fetched: 64..95 may be overwritten now
        tmem_st16(tS + 64, lo_hold0);
        tmem_st16(tS + 80, lo_hold1);
#pragma unroll
        for (int w = 0; w < 16; ++w) lo_hold0[w] = lo[w];
      } else {
        tmem_st16(tS + 96, lo_hold0);
        tmem_st16(tS + 112, lo);
      }
    }
    if (u < 3) {
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) cur[i] = nxt[i];
    }
  }
  l_run += (acc0.x + acc0.y) + (acc1.x + acc1.y);
}

template <typename T>
struct Fmt;
template <>
struct Fmt<__half> {
  static constexpr int kCode = 0;
};
template <>
struct Fmt<__nv_bfloat16> {
  static constexpr int kCode = 1;
};

// The grid's z index counts sequences in order of decreasing work (history plus new tokens), so that the CTAs launched
// last - the ones that run while the SMs drain - belong to the sequence whose CTAs are shortest.  With the sequences in
// the caller's order a long last sequence leaves a tail in which most SMs idle (simulated for the benchmark batch, whose
// last sequence is its longest: 95 % -> 97 % of the SM-time used).  The order inside a sequence is unchanged: its query
// tiles stay neighbours in launch order and share its history tiles in L2.  Every warp computes the mapping for itself
// (batches of up to 32 sequences: one key per lane, ranked with shuffles); larger batches keep the caller's order.
// (In two steps, so that the loads of the keys can be in flight while the CTA sets itself up.)
__device__ __forceinline__ int sequence_rank_key(const TcParams& p, int lane) {
  if (p.num_seqs > 32 || p.num_seqs < 2 || lane >= p.num_seqs) return -1;
  int h = p.hist_lens[lane];
  h = h < 0 ? 0 : h;
  const int n = p.cu_seqlens ? p.cu_seqlens[lane + 1] - p.cu_seqlens[lane] : 0;
  return min(h, 0x3fffffff) + min(max(n, 0), 0x3fffffff);
}
__device__ __forceinline__ int sequence_of_rank(const TcParams& p, int z, int lane, int key) {
  if (p.num_seqs > 32 || p.num_seqs < 2) return z;
  int rank = 0;
  for (int j = 0; j < p.num_seqs; ++j) {
    const int kj = __shfl_sync(0xffffffffu, key, j);
    rank += (kj > key || (kj == key && j < lane)) ? 1 : 0;
  }
  const unsigned hit = __ballot_sync(0xffffffffu, lane < p.num_seqs && rank == z);
  return hit ? __ffs(hit) - 1 : z;
}

// NQ accumulator tiles per CTA.  PAIR_TILES = false: tile q is query head h0 + q of one 128-token query tile (heads that
// share a kv head).  PAIR_TILES = true (NQ = 2): both tiles belong to head h0, tile q holds query tile 2 * blockIdx.x' + q;
// they share every K / V tile, and the earlier one sees its last key tile fully masked.
template <typename T, int D, int TPP, int NQ, bool PAIR_TILES, int SBUF>
__global__ void __launch_bounds__(64 + 128 * NQ, 1)
    prefill_tcgen05_kernel(const TcParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_vpool,
                           const __grid_constant__ CUtensorMap tm_kpool, const __grid_constant__ CUtensorMap tm_out) {
  using C = TcCfg<D, TPP, NQ, SBUF>;
  constexpr int kBlocks = C::kBlocks, kPagesPerTile = C::kPagesPerTile, kPageBytes = C::kPageBytes, kTileBytes = C::kTileBytes;
  constexpr int ST = C::kStages, kOC = C::kOChunk;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + C::kQ;
  unsigned char* sK = smem + C::kK;
  unsigned char* sV = smem + C::kV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBars);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // NS
  uint64_t* p_full = bars + 11;       // NS
  uint64_t* o_done = bars + 13;       // NQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Launch order (x fastest): all heads of a sequence's heaviest (latest) query tile, then its next query tile, ... so
  // the CTAs of one sequence run together (its K / V tiles are shared in L2) and the last ones of the grid are light.
  const int qt_cta = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int qt = PAIR_TILES ? 2 * qt_cta : qt_cta;   // the CTA's first (or only) query tile
  const int t0 = qt * kTile;
  const int h0 = PAIR_TILES ? blockIdx.x : blockIdx.x * NQ;
  constexpr int kHeadStep = PAIR_TILES ? 0 : 1;         // head of accumulator tile q = h0 + q * kHeadStep
  constexpr int kRowStep = PAIR_TILES ? kTile : 0;      // its first query token = t0 + q * kRowStep
  // Barriers and tensor memory; for uniform batches this runs while the keys that order the sequences are being loaded.
  auto set_up = [&] {
    if (tid == 0) {
      mbar_init(q_full, 1);
      for (int i = 0; i < 2; ++i) {
        mbar_init(&k_full[i], 1);
        mbar_init(&k_empty[i], 1);
        mbar_init(&v_full[i], 1);
        mbar_init(&v_empty[i], 1);
        mbar_init(&s_full[i], 1);
        mbar_init(&p_full[i], 4);
        mbar_init(&o_done[i], 1);
      }
      fence_mbar_init();
    }
    if (warp == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  };
  const bool ragged = p.cu_seqlens != nullptr;
  const int rank_key = sequence_rank_key(p, lane);
  if (!ragged) {
    if (t0 >= p.n_new) return;
    set_up();
  }
  const int part = p.parts > 1 ? (int)(blockIdx.z % (unsigned)p.parts) : 0;
  const int s = sequence_of_rank(p, p.parts > 1 ? (int)(blockIdx.z / (unsigned)p.parts) : (int)blockIdx.z, lane, rank_key);
  const int kvh = h0 / p.group;
  // Uniform batches index the prompt tensors as [sequence][token] (rows past N read as zero); ragged batches as one
  // flat row axis starting at the sequence's first row (rows past N belong to the next sequence and are masked).
  const int N = ragged ? p.cu_seqlens[s + 1] - p.cu_seqlens[s] : p.n_new;
  const int row0 = ragged ? p.cu_seqlens[s] : 0;
  const int tma_seq = ragged ? 0 : s;
  const size_t out_row0 = ragged ? (size_t)row0 : (size_t)s * N;
  if (ragged) {
    if (t0 >= N) return;  // the grid is sized for the longest sequence (nothing is allocated yet)
    set_up();
  }
  // The Q tiles are requested by the thread that initialised their barrier, before the CTA-wide barrier below: the load
  // travels while tensor memory is being allocated and the history length is fetched.
  if (tid == 0) {
    mbar_arrive_expect_tx(q_full, NQ * kTileBytes);
    for (int q = 0; q < NQ; ++q)
      for (int kb = 0; kb < kBlocks; ++kb)
        tma_load_4d(sQ + q * kTileBytes + kb * kBlockBytes, &tm_q, kb * 64, h0 + q * kHeadStep, row0 + t0 + q * kRowStep, tma_seq, q_full);
  }
  int H = p.hist_lens[s];
  if (H < 0 || p.num_pages <= 0) H = 0;
  {
    const long long cap = (long long)p.max_pages_per_seq * TPP;
    if (H > cap) H = (int)cap;
  }
  const int H_total = H;
  int page0 = 0;           // first page of the history this CTA reads
  bool with_new = true;    // ... and whether it also attends to the new tokens
  if (p.parts > 1) {
    const int first = part * p.split_tiles * kTile;
    const int last = min(H_total, first + p.split_tiles * kTile);
    H = last > first ? last - first : 0;
    page0 = first / TPP;
    with_new = part == p.parts - 1;
  }
  const int hist_tiles = (H + kTile - 1) / kTile;
  // key tiles of the new tokens up to the diagonal of the CTA's last query tile that exists
  const int dense_tiles = with_new ? (PAIR_TILES && t0 + kTile < N ? qt + 1 : qt) + 1 : 0;
  const int num_tiles = hist_tiles + dense_tiles;  // (0 for a part that lies past the end of a short history)
  // bf16 rounds P with a relative error of up to 2^-8; summed over n keys that leaves about
  // 0.002 / sqrt(n / 3) of absolute error per unit of |v|, which only drops below the 2e-3 target
  // (at the 6-sigma level) once a row sees a few hundred keys.  CTAs that hold rows with fewer than
  // 256 visible keys - the first one or two query tiles of sequences with little history, the
  // lightest CTAs of the causal schedule - feed the residual P - bf16(P) through a second set of
  // PV MMAs.
  // A caller that asks for a float32 output asks for the arithmetic error alone to stay within tolerance on every row,
  // including rows dominated by a single key, where the rounding of P shows undiluted: the residual is then always fed.
  const bool split_p = Mma16816<T>::kSplitP && (p.out_f32 != 0 || H_total + t0 < 256);

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =============================== producer ===============================
    int ok = 1;
    // Key tile j lives in ring stage j % ST; its full / empty barriers are those of index j & 1, used for the
    // (j >> 1)-th time (two barriers per kind even when the ring has one stage, so that nobody ever waits on a barrier
    // that may be more than one phase away from the one it names - a parity wait cannot tell phases two apart).
    for (int j = 0; j < num_tiles && ok; ++j) {
      const int st = j % ST;
      const int jb = j & 1;
      const int jr = j - ST;  // the tile whose consumption frees this stage
      const bool paged = j < hist_tiles;
      int npg = 0;
      uint32_t my_pid = 0;
      if (paged) {
        npg = min(kPagesPerTile, (H - j * kTile + TPP - 1) / TPP);
        if (lane < npg) {
          my_pid = p.page_table[(size_t)s * p.max_pages_per_seq + page0 + j * kPagesPerTile + lane];
          if ((long long)my_pid >= p.num_pages) my_pid = (uint32_t)(p.num_pages - 1);
        }
      }
      // ---- K ----
      if (lane == 0 && jr >= 0) ok = mbar_wait(&k_empty[jr & 1], (jr >> 1) & 1, p.status);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (paged) {
        // The pool keeps a page as [chunk of 8 elements][token][16 B].  For each chunk, one gather4 request brings the
        // chunk's TPP * 16-byte rows of four pages and puts them back to back: the tile becomes [chunk][128 tokens][16 B],
        // tokens in order, whatever the page size.  One request per lane at a time; groups of four pages that lie wholly
        // past the history are not fetched (their S columns are masked), pages past it inside a group repeat page 0.
        constexpr int kChunks = D / 8, kGroups = kPagesPerTile / 4;     // requests per tile = kChunks * kGroups
        constexpr int kGroupBytes = 4 * TPP * 16;
        const int groups_used = (npg + 3) >> 2;
        if (lane == 0) mbar_arrive_expect_tx(&k_full[jb], kChunks * groups_used * kGroupBytes);
        __syncwarp();
        const int pid0 = __shfl_sync(0xffffffffu, (int)my_pid, 0);
#pragma unroll
        for (int op0 = 0; op0 < kChunks * kGroups; op0 += 32) {
          const int op = op0 + lane;
          const int c = op / kGroups, g = op % kGroups;
          int rows[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int pg = 4 * g + i;  // page of the tile; every lane takes part in the shuffle
            const int pid = __shfl_sync(0xffffffffu, (int)my_pid, pg & 31);
            rows[i] = ((pg < npg ? pid : pid0) * p.num_kv_heads + kvh) * kChunks + c;
          }
          if (op < kChunks * kGroups && g < groups_used)
            tma_gather4(sK + st * kTileBytes + c * C::kChunkBytes + g * kGroupBytes, &tm_kpool, 0, rows[0], rows[1], rows[2], rows[3],
                        &k_full[jb]);
        }
      } else if (lane == 0) {
        const int jd = j - hist_tiles;
        mbar_arrive_expect_tx(&k_full[jb], kTileBytes);
        for (int kb = 0; kb < kBlocks; ++kb)
          tma_load_4d(sK + st * kTileBytes + kb * kBlockBytes, &tm_k, kb * 64, kvh, row0 + jd * kTile, tma_seq, &k_full[jb]);
      }
      // ---- V ----
      if (lane == 0 && jr >= 0) ok = mbar_wait(&v_empty[jr & 1], (jr >> 1) & 1, p.status);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (paged) {
        if (lane == 0) mbar_arrive_expect_tx(&v_full[jb], npg * kPageBytes);
        __syncwarp();
        if (lane < npg)
          tma_load_3d(sV + st * kTileBytes + lane * kPageBytes, &tm_vpool, 0, 0, (int)(my_pid * p.num_kv_heads + kvh), &v_full[jb]);
      } else if (lane == 0) {
        const int jd = j - hist_tiles;
        mbar_arrive_expect_tx(&v_full[jb], kTileBytes);
        for (int nb = 0; nb < kBlocks; ++nb)
          tma_load_4d(sV + st * kTileBytes + nb * kBlockBytes, &tm_v, nb * 64, kvh, row0 + jd * kTile, tma_seq, &v_full[jb]);
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    {
      constexpr int F = Fmt<T>::kCode;
      constexpr uint32_t idesc_qk128 = make_idesc(128, F, F, 0);
      constexpr uint32_t idesc_pv_paged = make_idesc(D, F, F, 0);  // A = P (TMEM), B = V K-major, N = head_dim
      constexpr uint32_t idesc_pv_dense = make_idesc(D, F, F, 1);  // B = V MN-major
      const uint32_t sQ_u = smem_u32(sQ), sK_u = smem_u32(sK), sV_u = smem_u32(sV);
      // Descriptors of the operand tiles, built once; an MMA's descriptor is one of these plus a constant
      // (the start-address field counts 16-byte units and sits in the low bits, so a byte offset adds >> 4).
      uint64_t q_desc[NQ], k_dense[ST], k_hist[ST], v_dense[ST], v_hist[ST];
#pragma unroll
      for (int q = 0; q < NQ; ++q) q_desc[q] = make_desc(sQ_u + q * kTileBytes, 16, 1024, kLayoutSw128);
#pragma unroll
      for (int st = 0; st < ST; ++st) {
        k_dense[st] = make_desc(sK_u + st * kTileBytes, 16, 1024, kLayoutSw128);
        // gathered history K: chunks of 8 elements are 2048 bytes apart, 8-token core matrices 128 bytes
        k_hist[st] = make_desc(sK_u + st * kTileBytes, C::kChunkBytes, 128, kLayoutNone);
        v_dense[st] = make_desc(sV_u + st * kTileBytes, kBlockBytes, 1024, kLayoutSw128);
        v_hist[st] = make_desc(sV_u + st * kTileBytes, 16, 8 * TPP * 2, TPP == 16 ? kLayoutSw32 : kLayoutSw64);
      }
      // Every lane waits (each needs to observe the barrier itself), and the outcomes are combined so that the warp
      // leaves together if a wait expires: elect.sync below names all 32 lanes.
      auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status)) != 0; };
      bool ok = wait_all(q_full, 0);
      // (a register array must not be indexed with a run-time value: pick the stage's descriptor with a select)
      auto pick = [&](const uint64_t (&d)[ST], int st) { return ST == 1 ? d[0] : (st ? d[ST - 1] : d[0]); };

      // S tile of accumulator q for key tile j, as (index of its barriers, TMEM column)
      auto s_index = [&](int q, int j) { return SBUF == 2 ? (j & 1) : q; };
      // S_q(j) = Q_q . K(j)^T
      auto issue_qk = [&](int q, int j) {
        if (!elect_one()) return;
        const int st = j % ST;
        const int si = s_index(q, j);
        const uint32_t d_tmem = tmem_base + si * kTile;
        const uint64_t qa = q == 0 ? q_desc[0] : q_desc[NQ - 1];
        if (j < hist_tiles) {
          const uint64_t kb = pick(k_hist, st);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t a = qa + (uint64_t)(((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4);
            // chunks 2 ks and 2 ks + 1 of all 128 tokens
            tc_mma_ss(d_tmem, a, kb + (uint64_t)((ks * 2 * C::kChunkBytes) >> 4), idesc_qk128, ks > 0);
          }
        } else {
          const uint64_t kb = pick(k_dense, st);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t off = (uint64_t)(((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4);
            tc_mma_ss(d_tmem, qa + off, kb + off, idesc_qk128, ks > 0);
          }
        }
        tc_commit(&s_full[si]);
      };
      // O_q += P_q(j) . V(j)
      auto issue_pv = [&](int q, int j) {
        if (!elect_one()) return;
        const int st = j % ST;
        const uint32_t d_tmem = tmem_base + C::kOBase + q * C::DP;
        const uint32_t a_tmem = tmem_base + s_index(q, j) * kTile;  // P over the first 64 columns of the S tile
        for (int part = 0; part < (split_p ? 2 : 1); ++part) {  // part 1: the residual of P, 64 columns on
          const uint32_t a_part = a_tmem + part * 64;
          if (j < hist_tiles) {
            const uint64_t vb = pick(v_hist, st);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
              // 16 tokens: page kk (TPP = 16), or half kk & 1 of page kk >> 1 (TPP = 32: 32 bytes further inside the swizzled row)
              const int off = TPP == 16 ? kk * kPageBytes : (kk >> 1) * kPageBytes + (kk & 1) * 32;
              tc_mma_ts(d_tmem, a_part + kk * 8, vb + (uint64_t)(off >> 4), idesc_pv_paged, (j > 0 || kk > 0 || part > 0));
            }
          } else {
            const uint64_t vb = pick(v_dense, st);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              tc_mma_ts(d_tmem, a_part + kk * 8, vb + (uint64_t)((kk * 2048) >> 4), idesc_pv_dense, (j > 0 || kk > 0 || part > 0));
          }
        }
        tc_commit(&o_done[SBUF == 2 ? (j & 1) : q]);  // one accumulator tile: the two barriers alternate by key tile
      };

      if (num_tiles == 0) ok = false;  // a part past the end of a short history: Q has landed, there is nothing to multiply
      if (ok) ok = wait_all(&k_full[0], 0);
      if (ok) {
        tc_fence_after();
        for (int q = 0; q < NQ; ++q) issue_qk(q, 0);
        if (elect_one()) tc_commit(&k_empty[0]);
      }
      // (all barrier indices below are key tile & 1, all parities (key tile >> 1) & 1; the ring stage is key tile % ST)
      if (SBUF == 2) {
        // One accumulator tile, two S tiles: QK^T of key tile j + 1 goes into the other S tile before PV of tile j is
        // issued, so it runs while the softmax warps work on tile j.  (The tensor pipe executes in issue order: QK^T(j+1)
        // overwrites the S tile whose P was read by PV(j-1), issued before it.)
        for (int j = 0; j < num_tiles && ok; ++j) {
          if (j + 1 < num_tiles) {
            ok = wait_all(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
            if (!ok) break;
            tc_fence_after();
            issue_qk(0, j + 1);
            if (elect_one()) tc_commit(&k_empty[(j + 1) & 1]);
          }
          ok = wait_all(&v_full[j & 1], (j >> 1) & 1);
          if (ok) ok = wait_all(&p_full[j & 1], (j >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_pv(0, j);
          __syncwarp();
          if (elect_one()) tc_commit(&v_empty[j & 1]);
        }
      } else {
        for (int j = 0; j < num_tiles && ok; ++j) {
          ok = wait_all(&v_full[j & 1], (j >> 1) & 1);
          for (int q = 0; q < NQ && ok; ++q) {
            ok = wait_all(&p_full[q], j & 1);
            if (!ok) break;
            tc_fence_after();
            issue_pv(q, j);
            if (j + 1 < num_tiles) {
              if (q == 0) {
                ok = wait_all(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
                if (!ok) break;
                tc_fence_after();
              }
              issue_qk(q, j + 1);
              if (q == NQ - 1 && elect_one()) tc_commit(&k_empty[(j + 1) & 1]);
            }
          }
          __syncwarp();
          if (ok && elect_one()) tc_commit(&v_empty[j & 1]);
        }
      }
    }
  } else {
    // =============================== softmax warpgroups ===============================
    const int q = (warp - 2) >> 2;
    const int lane_group = warp & 3;            // the TMEM sub-partition this warp may touch
    const int row = lane_group * 32 + lane;     // row of the 128-row tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const uint32_t tO = tmem_base + lane_addr + C::kOBase + q * C::DP;
    const int t0q = t0 + q * kRowStep;          // first query token of this accumulator tile
    const int diag = t0q / kTile;               // its diagonal key tile among the new tokens
    const int qi = t0q + row;                   // index of this row's query token in its sequence
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    // PV of key tile `tile` of this accumulator is complete.  (Valid where it is used: when S of key tile j is ready, PV of
    // tile j - 2 is complete with S double-buffered, PV of tile j - 1 otherwise, so the barrier named here is at most one
    // phase behind.  With S double-buffered the two o_done barriers alternate by key tile.)
    auto wait_pv_done = [&](int tile) {
      return SBUF == 2 ? mbar_wait(&o_done[tile & 1], (tile >> 1) & 1, p.status) : mbar_wait(&o_done[q], tile & 1, p.status);
    };
    auto wait_v_landed = [&](int tile) { return mbar_wait(&v_full[tile & 1], (tile >> 1) & 1, p.status); };
    for (int j = 0; j < num_tiles; ++j) {
      const bool paged = j < hist_tiles;
      const int jd = j - hist_tiles;
      const int si = SBUF == 2 ? (j & 1) : q;                        // which S tile, and which of its barriers
      const uint32_t s_par = SBUF == 2 ? ((j >> 1) & 1) : (j & 1);   // parity of this use of the S tile
      const uint32_t tS = tmem_base + lane_addr + si * kTile;
      const int vst = j % ST;
      if (!(ok = mbar_wait(&s_full[si], s_par, p.status))) break;
      tc_fence_after();
      // which columns need masking at all (warp-uniform), and up to which key offset this row sees
      const bool need_mask = paged ? ((j + 1) * kTile > H) : (jd >= diag || (jd + 1) * kTile > N);
      const int rel_limit = paged ? (H - 1 - j * kTile) : (min(qi, N - 1) - jd * kTile);

      // ---- pass 1: row maximum of the scaled scores ----
      float mx;
      mx = need_mask ? tile_row_max<true>(tS, rel_limit) : tile_row_max<false>(tS, rel_limit);
      mx *= p.scale_log2;  // scale > 0, so the maximum commutes with the scaling
      const float m_new = fmaxf(m_used, mx);
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
        // O_q must be stable: PV(j-1) of this accumulator has to be complete
        if (!(ok = wait_pv_done(j - 1))) break;
        tc_fence_after();
        const float f = fast_exp2(m_used - m_new);
#pragma unroll
        for (int c4 = 0; c4 < D / kOC; ++c4) {
          uint32_t v[kOC];
          tmem_ldw(tO + c4 * kOC, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < kOC; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_stw(tO + c4 * kOC, v);
        }
        tmem_wait_st();
        l_run *= f;
        m_used = m_new;
      }
      const float m_ref = m_used > -INFINITY ? m_used : 0.f;

      // ---- pass 2: P = exp2(s * scale - m), packed over S's first 64 columns ----
      if (split_p)
        tile_exp_store<T, true, Mma16816<T>::kSplitP>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      else if (need_mask)
        tile_exp_store<T, true, false>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      else
        tile_exp_store<T, false, false>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      tmem_wait_st();

      // The last history tile may hold slots past the history length, and pages that were never
      // loaded: zero those V tokens in shared memory, because 0 * NaN would poison the accumulator.
      if (q == 0 && paged && need_mask) {
        if (!(ok = wait_v_landed(j))) break;
        unsigned char* vt = sV + vst * kTileBytes;
        constexpr int kRowBytes = TPP * 2;  // one head-dim row of a page: 32 bytes (32-byte swizzle) or 64 (64-byte swizzle)
        for (int dr = row; dr < D; dr += kTile) {
          // the swizzle xors the 16-byte chunk index of a row with address bits 7 and up
          const int sw = TPP == 16 ? ((dr >> 2) & 1) : ((dr >> 1) & 3);
          for (int pg = 0; pg < kPagesPerTile; ++pg) {
            int nv = H - j * kTile - pg * TPP;
            nv = nv < 0 ? 0 : nv;
            unsigned char* vrow = vt + pg * kPageBytes + dr * kRowBytes;
            for (int slot = nv; slot < TPP; ++slot)
              *reinterpret_cast<uint16_t*>(vrow + ((((slot >> 3) ^ sw) << 4) | ((slot & 7) << 1))) = 0;
          }
        }
        fence_proxy_async_smem();
      }
      // In a ragged batch the dense tile that holds a sequence's last new tokens also holds rows of the next sequence.
      // Their keys are masked, but their V rows would still be multiplied by P = 0: zero them (0 * NaN again).
      if (q == 0 && !paged && p.cu_seqlens != nullptr && (jd + 1) * kTile > N) {
        if (!(ok = wait_v_landed(j))) break;
        if (jd * kTile + row >= N) {
          // dense V tile: [blocks of 64 head-dim elements][128 tokens][128 bytes]; the swizzle permutes within a row
          unsigned char* vt = sV + vst * kTileBytes + row * 128;
#pragma unroll
          for (int nb = 0; nb < kBlocks; ++nb)
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(vt + nb * kBlockBytes + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[si]);
    }

    // ---- epilogue: O / l -> out[((s*N + qi)*Hq + h0 + q)*D + d] ----
    if (ok && num_tiles > 0) ok = wait_pv_done(num_tiles - 1);
    if (p.parts > 1) {
      // this CTA's share of the keys: the un-normalised triple of every row goes to the partial buffers
      // (the TMEM loads are warp-wide instructions: every lane takes part, only the stores depend on the row)
      if (ok) {
        tc_fence_after();
        const size_t prow = ((out_row0 + qi) * p.num_q_heads + h0 + q * kHeadStep) * (size_t)p.parts + part;
        const bool any = num_tiles > 0 && m_used > -INFINITY;
        if (qi < N) {
          p.part_m[prow] = any ? m_used * kLn2 : -INFINITY;
          p.part_l[prow] = any ? l_run : 0.f;
        }
        if (num_tiles > 0) {
          float4* pacc = reinterpret_cast<float4*>(p.part_acc + prow * D);
#pragma unroll
          for (int c4 = 0; c4 < D / kOC; ++c4) {
            uint32_t v[kOC];
            tmem_ldw(tO + c4 * kOC, v);
            tmem_wait_ld();
            if (qi < N && any) {
#pragma unroll
              for (int i = 0; i < kOC / 4; ++i)
                pacc[c4 * (kOC / 4) + i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i + 2]),
                                                       __uint_as_float(v[4 * i + 3]));
            }
          }
        }
      }
      ok = false;  // nothing else to store
    }
    // Full tiles (and partial ones of uniform batches, which the tensor map clips at the sequence's end) leave through
    // shared memory: the tile's Q buffer is no longer read by any MMA, has exactly the size and swizzled layout of the
    // output tile, and TMA stores write it out in whole lines.  A partial tile of a ragged batch would run into the
    // next sequence's rows, so it is stored row by row from registers; so is a float32 output.
    const bool tma_out = !p.out_f32 && (p.cu_seqlens == nullptr || t0q + kTile <= N);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const size_t out_off = ((out_row0 + qi) * p.num_q_heads + h0 + q * kHeadStep) * D;
      T* orow = static_cast<T*>(p.out) + out_off;
      unsigned char* stage = sQ + q * kTileBytes + row * 128;
#pragma unroll
      for (int c4 = 0; c4 < D / kOC; ++c4) {
        uint32_t v[kOC];
        tmem_ldw(tO + c4 * kOC, v);
        tmem_wait_ld();
        if (p.out_f32) {
          if (qi < N) {
            float4* o32 = reinterpret_cast<float4*>(static_cast<float*>(p.out) + out_off + c4 * kOC);
#pragma unroll
            for (int i = 0; i < kOC / 4; ++i)
              o32[i] = make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                                   __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv);
          }
          continue;
        }
#pragma unroll
        for (int i = 0; i < kOC / 8; ++i) {
          uint4 w;
          w.x = Mma16816<T>::pack(__uint_as_float(v[8 * i + 0]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
          w.y = Mma16816<T>::pack(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
          w.z = Mma16816<T>::pack(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
          w.w = Mma16816<T>::pack(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
          // 16-byte chunk c of the row: 64-element block c / 8, chunk c % 8 xor-swizzled with the row
          const int c = (kOC / 8) * c4 + i;
          if (tma_out) {
            *reinterpret_cast<uint4*>(stage + (c >> 3) * kBlockBytes + (((c & 7) ^ (row & 7)) << 4)) = w;
          } else if (qi < N) {
            *reinterpret_cast<uint4*>(orow + c * 8) = w;
          }
        }
      }
      if (tma_out) {
        fence_proxy_async_smem();
        __syncwarp();
        // one more phase of a barrier that counts the tile's four warps: the one the last key tile used, advanced once
        const int se = SBUF == 2 ? ((num_tiles - 1) & 1) : q;
        const uint32_t e_par = SBUF == 2 ? ((((num_tiles - 1) >> 1) + 1) & 1) : (num_tiles & 1);
        if (lane == 0) mbar_arrive(&p_full[se]);
        // (a paired CTA's second query tile may lie entirely past the sequence's end: nothing to write then)
        if (lane_group == 0 && lane == 0 && mbar_wait(&p_full[se], e_par, p.status) && t0q < N) {
          for (int kb = 0; kb < kBlocks; ++kb)
            tma_store_4d(&tm_out, sQ + q * kTileBytes + kb * kBlockBytes, kb * 64, h0 + q * kHeadStep, row0 + t0q, tma_seq);
          tma_store_commit_and_wait_read();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------
inline PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  // resolved once; the initialisation of a function-local static is safe against concurrent first calls
  static const PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }();
  return fn;
}

inline bool encode_map(CUtensorMap* map, int dtype, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
                       const cuuint32_t* box, CUtensorMapSwizzle swizzle) {
  auto fn = get_encode_fn();
  if (!fn) {
    set_error("paged_attention_prefill: cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  const cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(map, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                  const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("paged_attention_prefill: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return false;
  }
  return true;
}

// The five tensor maps of a call.  Encoding them costs several microseconds of host time, and a serving loop calls with
// the same buffers and shapes step after step, so each host thread remembers the maps of its last few distinct calls.
struct TcMaps {
  CUtensorMap q, k, v, vpool, kpool, out;
};
struct TcMapKey {
  const void *q, *k, *v, *vpool, *kpool, *out;
  long long rows, seqs, pages;
  int hq, hkv, d, tpp, dtype;
  bool operator==(const TcMapKey& o) const {
    return q == o.q && k == o.k && v == o.v && vpool == o.vpool && kpool == o.kpool && out == o.out && rows == o.rows && seqs == o.seqs &&
           pages == o.pages && hq == o.hq && hkv == o.hkv && d == o.d && tpp == o.tpp && dtype == o.dtype;
  }
};

template <int D, int TPP>
const TcMaps* tensor_maps_for(const PrefillArgs& a) {
  constexpr int kSlots = 8;
  struct Slot {
    bool used = false;
    TcMapKey key;
    TcMaps maps;
  };
  thread_local Slot cache[kSlots];
  thread_local int next = 0;
  // ragged batches: one flat row axis of total_tokens rows (the kernel adds each sequence's first row)
  const cuuint64_t S = a.cu_seqlens ? 1 : a.num_seqs, N = a.cu_seqlens ? (cuuint64_t)a.total_tokens : a.tokens_per_seq;
  const cuuint64_t Hq = a.num_q_heads, Hkv = a.num_kv_heads;
  const TcMapKey key{a.q_prompt, a.k_prompt, a.v_prompt, a.num_pages > 0 ? a.v_pool : nullptr, a.num_pages > 0 ? a.k_pool : nullptr,
                     a.out, (long long)N, (long long)S,
                     a.num_pages, a.num_q_heads, a.num_kv_heads, D, TPP, a.dtype};
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].used && cache[i].key == key) return &cache[i].maps;
  Slot& slot = cache[next];
  next = (next + 1) % kSlots;
  slot.used = false;
  TcMaps& m = slot.maps;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, Hq, N, S};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, Hq * D * 2, N * Hq * D * 2};
    const cuuint32_t box[4] = {64, 1, kTile, 1};
    if (!encode_map(&m.q, a.dtype, 4, a.q_prompt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
    if (!encode_map(&m.out, a.dtype, 4, a.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;  // out has q's layout
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, Hkv, N, S};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, Hkv * D * 2, N * Hkv * D * 2};
    const cuuint32_t box[4] = {64, 1, kTile, 1};
    if (!encode_map(&m.k, a.dtype, 4, a.k_prompt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
    if (!encode_map(&m.v, a.dtype, 4, a.v_prompt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
  }
  if (a.num_pages > 0) {
    // one page of one kv head: [D rows][TPP tokens]; the third dimension counts (page, kv head) blocks
    const cuuint64_t dims[3] = {(cuuint64_t)TPP, (cuuint64_t)D, (cuuint64_t)a.num_pages * Hkv};
    const cuuint64_t strides[2] = {(cuuint64_t)TPP * 2, (cuuint64_t)D * TPP * 2};
    const cuuint32_t box[3] = {(cuuint32_t)TPP, (cuuint32_t)D, 1};
    if (!encode_map(&m.vpool, a.dtype, 3, a.v_pool, dims, strides, box, TPP == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B))
      return nullptr;
    // the K pool as rows of one (page, kv head, chunk) each: TPP tokens x 8 elements = TPP * 16 contiguous bytes
    const cuuint64_t kdims[2] = {(cuuint64_t)TPP * 8, (cuuint64_t)a.num_pages * Hkv * (D / 8)};
    const cuuint64_t kstrides[1] = {(cuuint64_t)TPP * 16};
    const cuuint32_t kbox[2] = {(cuuint32_t)TPP * 8, 1};  // gather4 takes four such rows per request
    if (!encode_map(&m.kpool, a.dtype, 2, a.k_pool, kdims, kstrides, kbox, CU_TENSOR_MAP_SWIZZLE_NONE)) return nullptr;
  } else {
    m.vpool = m.v;  // never dereferenced: without pages every history length is treated as 0
    m.kpool = m.k;
  }
  slot.key = key;
  slot.used = true;
  return &m;
}

template <typename T, int D, int TPP, int NQ, bool PAIR_TILES, int SBUF>
int launch_tc(const TcParams& p, const TcMaps& m, cudaStream_t stream) {
  using C = TcCfg<D, TPP, NQ, SBUF>;
  static_assert(C::kTotal <= 227 * 1024, "prefill shared memory exceeds the per-CTA limit");
  auto kern = prefill_tcgen05_kernel<T, D, TPP, NQ, PAIR_TILES, SBUF>;
  static DeviceOnce configured;  // one per instantiation
  const int rc = configured.run([&] { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal); });
  if (rc != 0) return rc;
  const int num_qt = (p.n_new + kTile - 1) / kTile;
  dim3 grid(PAIR_TILES ? p.num_q_heads : p.num_q_heads / NQ, PAIR_TILES ? (num_qt + 1) / 2 : num_qt, p.num_seqs * p.parts);
  if (grid.y > 65535) {
    set_error("paged_attention_prefill: more than 65535 query tiles per sequence");
    return -2;
  }
  kern<<<grid, 64 + 128 * NQ, C::kTotal, stream>>>(p, m.q, m.k, m.v, m.vpool, m.kpool, m.out);
  return (int)cudaGetLastError();
}

// How the accumulator tiles are put on CTAs.  Heads that share a kv head go two to a CTA; with an odd number of heads per
// kv head two consecutive query tiles of one head do; a sequence of a single query tile with an odd group, head_dim 256
// (whose O tile takes half of TMEM), or an explicit request leave one accumulator tile per CTA, with S double-buffered.
template <typename T, int D, int TPP>
int launch_tc_dtype(const PrefillArgs& a, const TcParams& p, const TcMaps& m, cudaStream_t stream) {
  if constexpr (D <= 128) {
    const bool single = a.impl == 3;
    const bool pair_heads = !single && (p.group % 2) == 0;
    const bool pair_tiles = !single && !pair_heads && a.tokens_per_seq > kTile;
    if (pair_heads) return launch_tc<T, D, TPP, 2, false, 1>(p, m, stream);
    if (pair_tiles) return launch_tc<T, D, TPP, 2, true, 1>(p, m, stream);
  }
  return launch_tc<T, D, TPP, 1, false, 2>(p, m, stream);
}

template <int D, int TPP>
int launch_tc_shape(const PrefillArgs& a, cudaStream_t stream) {
  if (a.num_seqs > 65535 || a.num_q_heads > 65535) {
    set_error("paged_attention_prefill: num_seqs and num_q_heads are limited to 65535");
    return -1;
  }
  if ((long long)a.num_pages * a.num_kv_heads * (D / 8) > 0x7fffffffLL) {
    set_error("paged_attention_prefill: pool too large for the tcgen05 kernel (pages * kv_heads * head_dim / 8 must fit 31 bits)");
    return -2;
  }
  TcParams p;
  p.k_pool = a.k_pool;
  p.page_table = a.page_table;
  p.hist_lens = a.history_lens;
  p.cu_seqlens = a.cu_seqlens;
  p.out = a.out;
  p.status = WaitCtx{&static_cast<WorkspaceHeader*>(a.workspace)->status, wait_limit_cycles()};
  p.out_f32 = a.out_f32 ? 1 : 0;
  p.num_seqs = a.num_seqs;
  p.n_new = a.tokens_per_seq;
  p.num_q_heads = a.num_q_heads;
  p.num_kv_heads = a.num_kv_heads;
  p.group = a.num_q_heads / a.num_kv_heads;
  p.max_pages_per_seq = a.max_pages_per_seq;
  p.num_pages = a.num_pages;
  p.scale_log2 = a.scale * kLog2e;
  // A batch that gives the GPU less than one CTA per SM has every CTA walk its sequence's whole history alone.  Such a
  // batch is cut along the history instead (as the decode kernel's split pass does): parts x as many CTAs, each with
  // 1 / parts of the history tiles, fp32 partial triples in the caller's workspace, one combine launch.  The workspace
  // size the caller was told (pal_prefill_workspace_bytes) plans for it; a smaller workspace simply runs unsplit.
  p.parts = 1;
  p.split_tiles = 0;
  p.part_acc = p.part_m = p.part_l = nullptr;
  const long long rows = (a.cu_seqlens ? a.total_tokens : (long long)a.num_seqs * a.tokens_per_seq) * a.num_q_heads;
  const int planned = prefill_split_parts(a.num_seqs, a.tokens_per_seq, a.num_q_heads, a.num_kv_heads, D);
  const int hist_tiles_max = (int)(((long long)a.max_pages_per_seq * TPP + kTile - 1) / kTile);
  if (planned > 1 && hist_tiles_max >= 2 && a.num_pages > 0 && rows > 0) {
    int split_tiles = (hist_tiles_max + planned - 1) / planned;
    if (split_tiles < 2) split_tiles = 2;  // a CTA's fixed cost is worth several key tiles
    const int parts = (hist_tiles_max + split_tiles - 1) / split_tiles;
    const size_t need = sizeof(WorkspaceHeader) + (size_t)rows * parts * (D + 2) * sizeof(float);
    if (parts >= 2 && a.workspace_bytes >= need && (long long)a.num_seqs * parts <= 65535) {
      p.parts = parts;
      p.split_tiles = split_tiles;
      p.part_acc = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) + sizeof(WorkspaceHeader));
      p.part_m = p.part_acc + (size_t)rows * parts * D;
      p.part_l = p.part_m + (size_t)rows * parts;
    }
  }
  const TcMaps* m = tensor_maps_for<D, TPP>(a);
  if (!m) return -3;
  const int rc = a.dtype == 0 ? launch_tc_dtype<__half, D, TPP>(a, p, *m, stream) : launch_tc_dtype<__nv_bfloat16, D, TPP>(a, p, *m, stream);
  if (rc != 0 || p.parts == 1) return rc;
  const PartialsView in{p.part_m, p.part_l, p.part_acc, 1, p.parts, D, (long long)p.parts * D};
  return launch_lse_combine(in, a.out, a.out_f32, TripleOut{}, p.parts, rows, D, a.dtype, stream);
}

}  // namespace
}  // namespace pal
