// Paged-attention prefill with tcgen05.mma.cta_group::2: two CTAs on the two SMs of a TPC work as one M = 256 MMA.
//
// Same operator as prefill_tcgen05.cuh (the reference's pal_paged_attention_prefill,
// src/pal_core/kernels/paged_attention/prefill/paged_attention_prefill.h.metal:28-389), for head_dim 256 and - with an
// even number of query heads per kv head - head_dim 128.
//
// A cluster of two CTAs owns two accumulator tiles that read the same K / V tiles: 128 new tokens of two query heads that
// share a kv head or, when the heads per kv head are odd in number (head_dim 256 only), two consecutive 128-token query
// tiles of one head.  CTA r holds the 128 rows of tile r (Q in its
// shared memory, S / P / O in its TMEM), and every MMA is issued once, by CTA 0, with M = 256.  The B operand of such an
// MMA is split between the CTAs - each supplies half of the N rows from its own shared memory - so CTA r loads only
// keys [64 r, 64 r + 64) of a K tile and head-dim columns [D/2 r, D/2 r + D/2) of a V tile.  Against one accumulator
// tile per CTA on its own (what head_dim 256 otherwise needs, because its O tile takes half of TMEM) that halves the
// bytes each SM pulls from L2 per flop and the shared memory a ring stage takes, which buys a second stage.
// With head_dim 128 the one-CTA kernel with two accumulator tiles per SM is faster (its two softmax warpgroups per SM
// hide each other's latency; here each SM has one), so this kernel is the default for head_dim 256 only.
//
//   warp 0   producer (both CTAs): its half of each tile by TMA with .cta_group::2, whose transaction bytes are
//            counted on CTA 0's "full" barriers (CTA 0 posts the expected total).  Every load is an ordinary
//            single-destination copy into the executing CTA's own shared memory.
//   warp 1   CTA 0: issues every tcgen05.mma.cta_group::2 and the commits, which arrive on the same barrier of both
//            CTAs.  Both CTAs: TMEM allocation and release.
//   warps 2-5 softmax warpgroup of the CTA's 128 rows; P-ready arrivals of both CTAs go to CTA 0's barrier.
//
// Shared-memory operand layouts per CTA (UMMA descriptors name the same offsets in both CTAs), B = D / 64
//   Q            [B k-blocks][128 rows][64 el]     K-major SWIZZLE_128B, SBO 1024
//   dense K half [B k-blocks][64 keys][64 el]      K-major SWIZZLE_128B, SBO 1024 (k-block stride 8192)
//   paged K half [D/8 chunks][64 tokens][16 B]     gathered 16 tokens x 4 per request; no swizzle, LBO 1024, SBO 128
//   paged V half page p at +D/2 * TPP * 2 p: [D/2 head-dim rows][TPP tokens], SWIZZLE_32B / 64B, SBO 8 rows
//   dense V half [B/2 n-blocks][128 tokens][64 el] MN-major SWIZZLE_128B, LBO 16384, SBO 1024
// TMEM: kSBuf S tiles of 128 columns (three with head_dim 128, two with 256), then O (D columns).  QK^T runs kSBuf key
// tiles ahead of PV.
//
// Every wait on a barrier is bounded; the two cluster-wide rendezvous (after barrier initialisation, before TMEM is
// released) are hardware barriers that every thread of both CTAs reaches because nothing before them can block forever.
#pragma once

#include "prefill_tcgen05.cuh"

namespace pal {
namespace {

template <int D_, int TPP_>
struct PairCfg {
  static constexpr int D = D_, TPP = TPP_;
  static_assert(D == 128 || D == 256, "the two-CTA kernel covers head_dim 128 and 256");
  static constexpr int kBlocks = D / 64;
  static constexpr int kStages = D == 128 ? 4 : 2;
  static constexpr int kSBuf = D == 128 ? 3 : 2;
  static constexpr int kHalfBytes = 64 * D * 2;            // one CTA's half of a K or V tile
  static constexpr int kQBytes = kTile * D * 2;
  static constexpr int kPagesPerTile = kTile / TPP;
  static constexpr int kPageHalfBytes = (D / 2) * TPP * 2;  // D/2 head-dim rows of one page
  static constexpr int kOBase = kSBuf * kTile;
  static_assert(kOBase + D <= 512, "TMEM holds 512 columns");
  static constexpr int kQ = 0;
  static constexpr int kK = kQBytes;
  static constexpr int kV = kK + kStages * kHalfBytes;
  static constexpr int kBars = kV + kStages * kHalfBytes;
  static constexpr int kTotal = kBars + 512 + 1024;
};

// ---- cluster / cta_group::2 PTX -------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier of a CTA of the cluster, with the default (CTA-scope) ordering: a cluster-scope release costs
// about a thousand cycles per arrival (measured), and what is handed over here lives in tensor memory, whose stores have
// been waited for.  The one hand-over through shared memory (the zero fill of V) is fenced explicitly.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// TMA loads of a CTA pair: the data lands in the executing CTA's shared memory, the bytes are counted on the barrier
// at `bar_cluster_addr`, which may live in the peer CTA.
__device__ __forceinline__ void tma2_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma2_gather4(void* dst, const CUtensorMap* map, int c0, int r0, int r1, int r2, int r3, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
// Arrives, once every MMA issued so far has completed, on the barrier at this offset in both CTAs of the pair.
__device__ __forceinline__ void tc2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tc2_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of the pair's MMA: M = 256 (128 rows per CTA), N counts both CTAs' halves of B.
__host__ __device__ constexpr uint32_t make_idesc_pair(int n, int a_fmt, int b_fmt, int b_mn_major) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(256 >> 4) << 24);
}

// PAIR_TILES = false: the pair's two accumulator tiles are one 128-token query tile of query heads 2k and 2k + 1 (which
// share a kv head).  PAIR_TILES = true (odd numbers of query heads per kv head): they are query tiles 2t and 2t + 1 of one
// head; both read every K / V tile up to the later tile's diagonal, and the earlier one sees its last key tile fully masked.
template <typename T, int D, int TPP, bool PAIR_TILES>
__global__ void __launch_bounds__(192, 1)
    prefill_tcgen05_pair_kernel(const TcParams p, const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_khalf,
                                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_vhalf,
                                const __grid_constant__ CUtensorMap tm_kpool16, const __grid_constant__ CUtensorMap tm_out) {
  using C = PairCfg<D, TPP>;
  constexpr int ST = C::kStages, SB = C::kSBuf, kHalf = C::kHalfBytes, kPagesPerTile = C::kPagesPerTile, kBlocks = C::kBlocks;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + C::kQ;
  unsigned char* sK = smem + C::kK;
  unsigned char* sV = smem + C::kV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kBars);
  uint64_t* q_full = bars;         // 1   (CTA 0's is used)
  uint64_t* k_full = bars + 1;     // 4   (CTA 0's)
  uint64_t* k_empty = bars + 5;    // 4   (each CTA's own, signalled by commits)
  uint64_t* v_full = bars + 9;     // 4   (CTA 0's)
  uint64_t* v_empty = bars + 13;   // 4
  uint64_t* s_full = bars + 17;    // 3
  uint64_t* p_full = bars + 20;    // 3   (CTA 0's; eight warps arrive)
  uint64_t* o_done = bars + 23;    // 3
  uint64_t* v_local = bars + 26;   // 2   (own V half landed, for the two tiles whose V needs zero-filling)
  uint64_t* e_bar = bars + 28;     // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();
  // Launch order (x fastest): the head pairs of a sequence's heaviest query tile, then its next query tile, ...;
  // sequences in order of decreasing work (see sequence_of_rank).  blockIdx.x = 2 * head pair + rank in the pair.
  const int qt_pair = (int)gridDim.y - 1 - (int)blockIdx.y;
  const int qt = PAIR_TILES ? 2 * qt_pair + (int)rank : qt_pair;     // this CTA's query tile
  const int t0 = qt * kTile;
  const int t0_first = PAIR_TILES ? 2 * qt_pair * kTile : t0;        // the pair's first query token
  const int h = PAIR_TILES ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;  // heads 2k and 2k + 1 form the pair, or one head does
  const int s = sequence_of_rank(p, blockIdx.z, lane, sequence_rank_key(p, lane));
  const int kvh = h / p.group;
  const bool ragged = p.cu_seqlens != nullptr;
  const int N = ragged ? p.cu_seqlens[s + 1] - p.cu_seqlens[s] : p.n_new;
  const int row0 = ragged ? p.cu_seqlens[s] : 0;
  const int tma_seq = ragged ? 0 : s;
  const size_t out_row0 = ragged ? (size_t)row0 : (size_t)s * N;
  if (t0_first >= N) return;  // both CTAs of a pair take the same branch; nothing is allocated yet
  int H = p.hist_lens[s];
  if (H < 0 || p.num_pages <= 0) H = 0;
  {
    const long long cap = (long long)p.max_pages_per_seq * TPP;
    if (H > cap) H = (int)cap;
  }
  const int hist_tiles = (H + kTile - 1) / kTile;
  // key tiles of the new tokens up to the diagonal of the pair's last query tile that exists
  const int dense_tiles = PAIR_TILES ? (t0_first + kTile < N ? 2 * qt_pair + 2 : 2 * qt_pair + 1) : qt + 1;
  const int num_tiles = hist_tiles + dense_tiles;
  // the rounding residual of P goes through a second set of PV MMAs where rows see few keys, or for float32 outputs
  // (decided for the pair as a whole: CTA 0 issues the MMAs of both)
  const bool split_p = Mma16816<T>::kSplitP && (p.out_f32 != 0 || H + t0_first < 256);
  // Tiles whose V holds slots that must read as zero (0 * NaN would poison O): the last history tile when the history
  // ends inside it, and in ragged batches the dense tile that runs into the next sequence's rows.  Their V halves are
  // counted on the CTA's own v_local barrier (index 0 / 1), so that the CTA's softmax warps can wait for them.
  auto needs_zero = [&](int j) { return j < hist_tiles ? (j + 1) * kTile > H : (ragged && (j - hist_tiles + 1) * kTile > N); };

  if (tid == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 8);
      mbar_init(&o_done[i], 1);
    }
    mbar_init(&v_local[0], 1);
    mbar_init(&v_local[1], 1);
    mbar_init(e_bar, 4);
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // =============================== producer ===============================
    int ok = 1;
    if (lane == 0) {
      if (rank == 0) mbar_arrive_expect_tx(q_full, 2 * C::kQBytes);
      const uint32_t qb = map_to_cta(q_full, 0);
      for (int kb = 0; kb < kBlocks; ++kb) tma2_load_4d(sQ + kb * kBlockBytes, &tm_q, kb * 64, h, row0 + t0, tma_seq, qb);
    }
    // Key tile j lives in ring stage j % ST and uses that stage's barriers for the (j / ST)-th time.
    for (int j = 0; j < num_tiles && ok; ++j) {
      const int st = j % ST;
      const uint32_t ph = (j / ST) & 1;
      const bool paged = j < hist_tiles;
      const int jd = j - hist_tiles;
      int npg = 0, units_valid = 0;  // pages / 16-token units of the tile that hold history
      uint32_t my_pid = 0;
      if (paged) {
        npg = min(kPagesPerTile, (H - j * kTile + TPP - 1) / TPP);
        units_valid = min(8, (H - j * kTile + 15) / 16);
        if (lane < npg) {
          my_pid = p.page_table[(size_t)s * p.max_pages_per_seq + j * kPagesPerTile + lane];
          if ((long long)my_pid >= p.num_pages) my_pid = (uint32_t)(p.num_pages - 1);
        }
      }
      // ---- K: keys [64 rank, 64 rank + 64) of the tile ----
      if (lane == 0 && j >= ST) ok = mbar_wait(&k_empty[st], ph ^ 1, p.status);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const uint32_t kb_addr = map_to_cta(&k_full[st], 0);
      if (paged) {
        // The pool viewed as rows of 16 tokens of one (page, kv head, 8-element chunk): 256 bytes each.  One gather4
        // request per chunk brings this CTA's four 16-token units and puts them back to back: [chunk][64 tokens][16 B].
        // A CTA whose units all lie past the history fetches nothing (its S columns are masked); units past the history
        // inside a fetched group repeat the tile's first unit.
        constexpr int kChunks = D / 8;  // 16 or 32: one request per lane
        const bool peer_active = units_valid > 4;
        if (rank == 0 && lane == 0) mbar_arrive_expect_tx(&k_full[st], (peer_active ? 2 : 1) * kHalf);
        __syncwarp();
        const int pid0 = __shfl_sync(0xffffffffu, (int)my_pid, 0);
        int rows[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int u = 4 * (int)rank + i;
          const int pg = TPP == 16 ? u : (u >> 1);
          const int pid = __shfl_sync(0xffffffffu, (int)my_pid, pg);
          const bool valid = u < units_valid;
          const int sub = (TPP == 16 || !valid) ? 0 : (u & 1);
          rows[i] = (((valid ? pid : pid0) * p.num_kv_heads + kvh) * kChunks + (lane % kChunks)) * (TPP / 16) + sub;
        }
        if ((rank == 0 || peer_active) && lane < kChunks)
          tma2_gather4(sK + st * kHalf + lane * 1024, &tm_kpool16, 0, rows[0], rows[1], rows[2], rows[3], kb_addr);
      } else if (lane == 0) {
        if (rank == 0) mbar_arrive_expect_tx(&k_full[st], 2 * kHalf);
        for (int kb = 0; kb < kBlocks; ++kb)
          tma2_load_4d(sK + st * kHalf + kb * 8192, &tm_khalf, kb * 64, kvh, row0 + jd * kTile + (int)rank * 64, tma_seq, kb_addr);
      }
      // ---- V: head-dim columns [D/2 rank, D/2 rank + D/2) of the tile's tokens ----
      if (lane == 0 && j >= ST) ok = mbar_wait(&v_empty[st], ph ^ 1, p.status);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const uint32_t vb_addr = map_to_cta(&v_full[st], 0);
      const bool fix = needs_zero(j);
      if (paged) {
        const uint32_t bytes = (uint32_t)npg * C::kPageHalfBytes;
        if (lane == 0) {
          if (fix) {
            mbar_arrive_expect_tx(&v_local[0], bytes);
            if (rank == 0) mbar_arrive(&v_full[st]);  // completes at once: the P-ready arrivals vouch for both halves
          } else if (rank == 0) {
            mbar_arrive_expect_tx(&v_full[st], 2 * bytes);
          }
        }
        __syncwarp();
        if (lane < npg) {
          unsigned char* dst = sV + st * kHalf + lane * C::kPageHalfBytes;
          const int blk = (int)(my_pid * p.num_kv_heads + kvh);
          if (fix)
            tma_load_3d(dst, &tm_vhalf, 0, (int)rank * (D / 2), blk, &v_local[0]);
          else
            tma2_load_3d(dst, &tm_vhalf, 0, (int)rank * (D / 2), blk, vb_addr);
        }
      } else if (lane == 0) {
        if (fix) {
          mbar_arrive_expect_tx(&v_local[1], kHalf);
          if (rank == 0) mbar_arrive(&v_full[st]);
        } else if (rank == 0) {
          mbar_arrive_expect_tx(&v_full[st], 2 * kHalf);
        }
        for (int nb = 0; nb < kBlocks / 2; ++nb) {
          unsigned char* dst = sV + st * kHalf + nb * kBlockBytes;
          const int c0 = (int)rank * (D / 2) + nb * 64;
          if (fix)
            tma_load_4d(dst, &tm_v, c0, kvh, row0 + jd * kTile, tma_seq, &v_local[1]);
          else
            tma2_load_4d(dst, &tm_v, c0, kvh, row0 + jd * kTile, tma_seq, vb_addr);
        }
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer (CTA 0) ===============================
    if (rank == 0) {
      constexpr int F = Fmt<T>::kCode;
      constexpr uint32_t idesc_qk = make_idesc_pair(128, F, F, 0);
      constexpr uint32_t idesc_pv_paged = make_idesc_pair(D, F, F, 0);
      constexpr uint32_t idesc_pv_dense = make_idesc_pair(D, F, F, 1);
      const uint32_t sQ_u = smem_u32(sQ), sK_u = smem_u32(sK), sV_u = smem_u32(sV);
      // descriptors of ring stage 0; stage st adds st * kHalf to the start-address field (16-byte units, low bits)
      const uint64_t q_desc = make_desc(sQ_u, 16, 1024, kLayoutSw128);
      const uint64_t k_dense = make_desc(sK_u, 16, 1024, kLayoutSw128);
      const uint64_t k_hist = make_desc(sK_u, 1024, 128, kLayoutNone);
      const uint64_t v_dense = make_desc(sV_u, kBlockBytes, 1024, kLayoutSw128);
      const uint64_t v_hist = make_desc(sV_u, 16, 8 * TPP * 2, TPP == 16 ? kLayoutSw32 : kLayoutSw64);
      auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar, parity, p.status)) != 0; };
      // S(j) = Q . K(j)^T into S tile j % SB; frees K stage j % ST
      auto issue_qk = [&](int j) {
        if (!elect_one()) return;
        const int st = j % ST;
        const uint32_t d_tmem = tmem_base + (j % SB) * kTile;
        const uint64_t stage = (uint64_t)((st * kHalf) >> 4);
        if (j < hist_tiles) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t a = q_desc + (uint64_t)(((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4);
            tc2_mma_ss(d_tmem, a, k_hist + stage + (uint64_t)((ks * 2 * 1024) >> 4), idesc_qk, ks > 0);
          }
        } else {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t a = q_desc + (uint64_t)(((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4);
            tc2_mma_ss(d_tmem, a, k_dense + stage + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4), idesc_qk, ks > 0);
          }
        }
        tc2_commit_both(&s_full[j % SB]);
        tc2_commit_both(&k_empty[st]);
      };
      // O += P(j) . V(j); frees V stage j % ST and S tile j % SB
      auto issue_pv = [&](int j) {
        if (!elect_one()) return;
        const int st = j % ST;
        const uint32_t d_tmem = tmem_base + C::kOBase;
        const uint32_t a_tmem = tmem_base + (j % SB) * kTile;
        const uint64_t stage = (uint64_t)((st * kHalf) >> 4);
        for (int part = 0; part < (split_p ? 2 : 1); ++part) {
          const uint32_t a_part = a_tmem + part * 64;
          if (j < hist_tiles) {
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
              const int off = TPP == 16 ? kk * C::kPageHalfBytes : (kk >> 1) * C::kPageHalfBytes + (kk & 1) * 32;
              tc2_mma_ts(d_tmem, a_part + kk * 8, v_hist + stage + (uint64_t)(off >> 4), idesc_pv_paged, (j > 0 || kk > 0 || part > 0));
            }
          } else {
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              tc2_mma_ts(d_tmem, a_part + kk * 8, v_dense + stage + (uint64_t)((kk * 2048) >> 4), idesc_pv_dense,
                         (j > 0 || kk > 0 || part > 0));
          }
        }
        tc2_commit_both(&o_done[j % SB]);
        tc2_commit_both(&v_empty[st]);
      };

      bool ok = wait_all(q_full, 0);
      for (int j = 0; j < SB && j < num_tiles && ok; ++j) {
        ok = wait_all(&k_full[j % ST], (j / ST) & 1);
        if (!ok) break;
        tc_fence_after();
        issue_qk(j);
        __syncwarp();
      }
      // S tile (j + SB) % SB is the one PV(j) has just read: QK^T runs SB key tiles ahead of PV.
      for (int j = 0; j < num_tiles && ok; ++j) {
        ok = wait_all(&v_full[j % ST], (j / ST) & 1);
        if (ok) ok = wait_all(&p_full[j % SB], (j / SB) & 1);
        if (!ok) break;
        if (needs_zero(j)) fence_acq_rel_cluster();  // pairs with the fence after the peer's zero fill of its V half
        tc_fence_after();
        issue_pv(j);
        __syncwarp();
        if (j + SB < num_tiles) {
          ok = wait_all(&k_full[(j + SB) % ST], ((j + SB) / ST) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + SB);
          __syncwarp();
        }
      }
    }
  } else {
    // =============================== softmax warpgroup ===============================
    const int lane_group = warp & 3;
    const int row = lane_group * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(lane_group * 32) << 16;
    const uint32_t tO = tmem_base + lane_addr + C::kOBase;
    const int diag = qt;
    const int qi = t0 + row;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < num_tiles; ++j) {
      const bool paged = j < hist_tiles;
      const int jd = j - hist_tiles;
      const int si = j % SB;
      const uint32_t s_par = (j / SB) & 1;
      const uint32_t tS = tmem_base + lane_addr + si * kTile;
      const int vst = j % ST;
      if (!(ok = mbar_wait(&s_full[si], s_par, p.status))) break;
      tc_fence_after();
      const bool need_mask = paged ? ((j + 1) * kTile > H) : (jd >= diag || (jd + 1) * kTile > N);
      const int rel_limit = paged ? (H - 1 - j * kTile) : (min(qi, N - 1) - jd * kTile);

      float mx = need_mask ? tile_row_max<true>(tS, rel_limit) : tile_row_max<false>(tS, rel_limit);
      mx *= p.scale_log2;
      const float m_new = fmaxf(m_used, mx);
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
        // PV(j - 1) must be complete.  When S(j) is ready PV(j - SB) is, so the barrier of tile j - 1 (index (j - 1) % SB,
        // shared with tiles j - 1 - SB and j - 1 + SB) is at most one phase behind the one named here.
        if (!(ok = mbar_wait(&o_done[(j - 1) % SB], ((j - 1) / SB) & 1, p.status))) break;
        tc_fence_after();
        const float f = fast_exp2(m_used - m_new);
#pragma unroll
        for (int c4 = 0; c4 < D / 32; ++c4) {
          uint32_t v[32];
          tmem_ld32(tO + c4 * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st32(tO + c4 * 32, v);
        }
        tmem_wait_st();
        l_run *= f;
        m_used = m_new;
      }
      const float m_ref = m_used > -INFINITY ? m_used : 0.f;

      if (split_p)
        tile_exp_store<T, true, Mma16816<T>::kSplitP>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      else if (need_mask)
        tile_exp_store<T, true, false>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      else
        tile_exp_store<T, false, false>(tS, p.scale_log2, m_ref, rel_limit, l_run);
      tmem_wait_st();

      if (needs_zero(j)) {
        if (paged) {
          // slots past the history, and pages never loaded, of this CTA's D/2 head-dim rows
          if (!(ok = mbar_wait(&v_local[0], 0, p.status))) break;
          unsigned char* vt = sV + vst * kHalf;
          constexpr int kRowBytes = TPP * 2;
          for (int idx = row; idx < (D / 2) * kPagesPerTile; idx += kTile) {
            const int dr = idx % (D / 2), pg = idx / (D / 2);
            // the swizzle xors the 16-byte chunk index of a row with address bits 7 and up
            const int sw = TPP == 16 ? ((dr >> 2) & 1) : ((dr >> 1) & 3);
            int nv = H - j * kTile - pg * TPP;
            nv = nv < 0 ? 0 : nv;
            unsigned char* vrow = vt + pg * C::kPageHalfBytes + dr * kRowBytes;
            for (int slot = nv; slot < TPP; ++slot)
              *reinterpret_cast<uint16_t*>(vrow + ((((slot >> 3) ^ sw) << 4) | ((slot & 7) << 1))) = 0;
          }
        } else {
          // rows of the next sequence in the dense tile: [n-blocks][128 tokens][128 bytes], the swizzle permutes within a row
          if (!(ok = mbar_wait(&v_local[1], 0, p.status))) break;
          if (jd * kTile + row >= N) {
            unsigned char* vt = sV + vst * kHalf + row * 128;
#pragma unroll
            for (int nb = 0; nb < kBlocks / 2; ++nb)
#pragma unroll
              for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(vt + nb * kBlockBytes + c * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        fence_proxy_async_smem();
        fence_acq_rel_cluster();  // the zero fill is read by an MMA that the other CTA issues
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&p_full[si], 0));
    }

    // ---- epilogue ----
    if (ok) ok = mbar_wait(&o_done[(num_tiles - 1) % SB], ((num_tiles - 1) / SB) & 1, p.status);
    const bool tma_out = !p.out_f32 && (!ragged || t0 + kTile <= N);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const size_t out_off = ((out_row0 + qi) * p.num_q_heads + h) * D;
      T* orow = static_cast<T*>(p.out) + out_off;
      unsigned char* stage = sQ + row * 128;  // Q is no longer read by any MMA
#pragma unroll
      for (int c4 = 0; c4 < D / 32; ++c4) {
        uint32_t v[32];
        tmem_ld32(tO + c4 * 32, v);
        tmem_wait_ld();
        if (p.out_f32) {
          if (qi < N) {
            float4* o32 = reinterpret_cast<float4*>(static_cast<float*>(p.out) + out_off + c4 * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              o32[i] = make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                                   __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv);
          }
          continue;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w;
          w.x = Mma16816<T>::pack(__uint_as_float(v[8 * i + 0]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
          w.y = Mma16816<T>::pack(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
          w.z = Mma16816<T>::pack(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
          w.w = Mma16816<T>::pack(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
          if (tma_out) {
            const int c = 4 * c4 + i;
            *reinterpret_cast<uint4*>(stage + (c >> 3) * kBlockBytes + (((c & 7) ^ (row & 7)) << 4)) = w;
          } else if (qi < N) {
            *reinterpret_cast<uint4*>(orow + c4 * 32 + i * 8) = w;
          }
        }
      }
      if (tma_out) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(e_bar);
        // (with query tiles paired, the second one may lie entirely past the sequence's end: nothing to write then)
        if (lane_group == 0 && lane == 0 && mbar_wait(e_bar, 0, p.status) && t0 < N) {
          for (int kb = 0; kb < kBlocks; ++kb) tma_store_4d(&tm_out, sQ + kb * kBlockBytes, kb * 64, h, row0 + t0, tma_seq);
          tma_store_commit_and_wait_read();
        }
      }
    }
  }

  // Neither CTA may release TMEM (or exit, taking its shared memory along) while the other still reads its accumulator
  // or while MMAs of the pair are in flight: the softmax warps above leave only after the last PV has completed.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------
struct PairMaps {
  CUtensorMap q, khalf, v, vhalf, kpool16, out;
};

template <int D, int TPP>
const PairMaps* pair_maps_for(const PrefillArgs& a) {
  constexpr int kSlots = 8;
  struct Slot {
    bool used = false;
    TcMapKey key;
    PairMaps maps;
  };
  thread_local Slot cache[kSlots];
  thread_local int next = 0;
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
  PairMaps& m = slot.maps;
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, Hq, N, S};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, Hq * D * 2, N * Hq * D * 2};
    const cuuint32_t box[4] = {64, 1, kTile, 1};
    if (!encode_map(&m.q, a.dtype, 4, a.q_prompt, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
    if (!encode_map(&m.out, a.dtype, 4, a.out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
  }
  {
    const cuuint64_t dims[4] = {(cuuint64_t)D, Hkv, N, S};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, Hkv * D * 2, N * Hkv * D * 2};
    const cuuint32_t box_k[4] = {64, 1, 64, 1};     // 64 keys x 64 elements
    const cuuint32_t box_v[4] = {64, 1, kTile, 1};  // 128 tokens x 64 head-dim columns
    if (!encode_map(&m.khalf, a.dtype, 4, a.k_prompt, dims, strides, box_k, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
    if (!encode_map(&m.v, a.dtype, 4, a.v_prompt, dims, strides, box_v, CU_TENSOR_MAP_SWIZZLE_128B)) return nullptr;
  }
  if (a.num_pages > 0) {
    // D/2 head-dim rows of one page of one kv head
    const cuuint64_t dims[3] = {(cuuint64_t)TPP, (cuuint64_t)D, (cuuint64_t)a.num_pages * Hkv};
    const cuuint64_t strides[2] = {(cuuint64_t)TPP * 2, (cuuint64_t)D * TPP * 2};
    const cuuint32_t box[3] = {(cuuint32_t)TPP, (cuuint32_t)D / 2, 1};
    if (!encode_map(&m.vhalf, a.dtype, 3, a.v_pool, dims, strides, box, TPP == 16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B))
      return nullptr;
    // the K pool as rows of 16 tokens of one (page, kv head, chunk): 128 elements = 256 contiguous bytes
    const cuuint64_t kdims[2] = {128, (cuuint64_t)a.num_pages * Hkv * (D / 8) * (TPP / 16)};
    const cuuint64_t kstrides[1] = {256};
    const cuuint32_t kbox[2] = {128, 1};
    if (!encode_map(&m.kpool16, a.dtype, 2, a.k_pool, kdims, kstrides, kbox, CU_TENSOR_MAP_SWIZZLE_NONE)) return nullptr;
  } else {
    m.vhalf = m.v;
    m.kpool16 = m.khalf;
  }
  slot.key = key;
  slot.used = true;
  return &m;
}

template <typename T, int D, int TPP, bool PAIR_TILES>
int launch_pair(const TcParams& p, const PairMaps& m, cudaStream_t stream) {
  using C = PairCfg<D, TPP>;
  static_assert(C::kTotal <= 227 * 1024, "prefill shared memory exceeds the per-CTA limit");
  auto kern = prefill_tcgen05_pair_kernel<T, D, TPP, PAIR_TILES>;
  static DeviceOnce configured;
  const int rc = configured.run([&] { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kTotal); });
  if (rc != 0) return rc;
  const int num_qt = (p.n_new + kTile - 1) / kTile;
  if (num_qt > 65535) {
    set_error("paged_attention_prefill: more than 65535 query tiles per sequence");
    return -2;
  }
  // (a cluster dimension given at compile time with a <<<>>> launch was rejected by the driver for the (1, 2, 1) shape;
  // the launch attribute with the pair along x is accepted)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = PAIR_TILES ? dim3(2 * p.num_q_heads, (num_qt + 1) / 2, p.num_seqs) : dim3(p.num_q_heads, num_qt, p.num_seqs);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = C::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, p, m.q, m.khalf, m.v, m.vhalf, m.kpool16, m.out);
}

template <int D, int TPP>
int launch_pair_shape(const PrefillArgs& a, cudaStream_t stream) {
  if (a.num_seqs > 65535 || a.num_q_heads > 32767) {
    set_error("paged_attention_prefill: num_seqs is limited to 65535 and num_q_heads to 32767");
    return -1;
  }
  if ((long long)a.num_pages * a.num_kv_heads * (D / 8) * (TPP / 16) > 0x7fffffffLL) {
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
  p.parts = 1;  // (the history split of the one-CTA kernel is not used here)
  p.split_tiles = 0;
  p.part_acc = p.part_m = p.part_l = nullptr;
  const PairMaps* m = pair_maps_for<D, TPP>(a);
  if (!m) return -3;
  // heads that share a kv head pair up; with an odd number of heads per kv head two consecutive query tiles of one head do
  if (p.group % 2 == 0)
    return a.dtype == 0 ? launch_pair<__half, D, TPP, false>(p, *m, stream) : launch_pair<__nv_bfloat16, D, TPP, false>(p, *m, stream);
  if constexpr (D == 256)
    return a.dtype == 0 ? launch_pair<__half, D, TPP, true>(p, *m, stream) : launch_pair<__nv_bfloat16, D, TPP, true>(p, *m, stream);
  set_error("paged_attention_prefill: the two-CTA tcgen05 kernel needs an even number of query heads per kv head at this head_dim");
  return -2;
}

}  // namespace
}  // namespace pal
