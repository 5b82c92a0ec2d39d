// Paged-attention decode for sm_100a: fused single-pass kernel, split-KV variant and the
// log-sum-exp combine kernel.
//
// Replaces pal_paged_attention_decode (src/pal_core/kernels/paged_attention/decode/
// paged_attention_decode.h.metal:29-412), pal_paged_reduce_decode (.../paged_reduce_decode.h.metal:27-129)
// and the launcher PagedAttentionDecodePrimitive::eval_gpu
// (src/pal_core/src/paged_attention_decode_primitive.cpp:71-266).
//
// Design (not a translation of the Metal kernel, which launches one threadgroup per query head and
// therefore re-reads every KV page Hq/Hkv times):
//  * One work item = (sequence, kv head, group of <= 8 query heads [, partition]).  The query heads of
//    a GQA group are the N dimension of the MMAs, so each KV page is read from HBM once per kv head.
//  * Persistent CTAs pull work items from an atomic counter; in single-pass mode the items are served
//    longest sequence first (every CTA ranks the sequence lengths in shared memory), which keeps the
//    tail of a ragged batch short.
//  * A producer warp walks the page table (32 page ids per coalesced load, one batch prefetched ahead)
//    and streams each page's contiguous K block and V block (D*TPP*2 bytes each) into a ring of
//    shared-memory stages with cp.async.bulk + mbarrier transaction counts; as many of its lanes as the ring has
//    stages each issue one page's copies at a time.  No multicast.
//  * Four consumer warps take the pages round robin.  Per 16 tokens a warp computes
//        S^T[16 tok x 8 heads] = K[16 tok x D] . Q^T            (mma.sync m16n8k16, A via ldmatrix)
//        online softmax over tokens (warp shuffles across the 8 token lanes)
//        O^T[D x 8 heads]     += V^T[D x 16 tok] . P^T           (A via ldmatrix, B via movmatrix)
//    The striped K block [D/8][TPP][8] and the transposed V block [D][TPP] are exactly the row-major
//    8x8 tiles ldmatrix wants, so the pools' native layouts are consumed without any re-tiling.
//  * The four warps' (m, l, O) are merged through shared memory at the end of an item; in split mode
//    the merged un-normalised triple goes to the workspace and the combine kernel finishes the job.
//  * Every mbarrier wait is bounded; on expiry the kernel records a timeout in the workspace status
//    word and returns.
#include <math.h>

#include "common.cuh"
#include "launch.h"

namespace pal {

namespace {

constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kDecodeThreads = kConsumerThreads + 32;
constexpr int kMaxSort = 512;        // rank sequence lengths in-kernel up to this batch size
constexpr int kHeadsPerItem = 8;     // N of the m16n8k16 MMA: one head set; a work item holds HS (1 or 2) of them
constexpr int kSmemBudget = 113 * 1024;  // per CTA, so that two CTAs fit one SM

struct DecodeParams {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const void* new_k;  // append form only: [S, Hkv, D] K and V of each sequence's last token
  const void* new_v;
  const uint32_t* page_table;
  const int32_t* seq_lens;
  void* out;
  float* part_m;
  float* part_l;
  float* part_acc;
  WorkspaceHeader* hdr;
  long long wait_limit;  // cycles any single device-side wait may last
  int out_f32;           // out is float32 instead of the query dtype
  int num_seqs, num_q_heads, num_kv_heads, group, head_groups;
  int max_pages_per_seq;
  long long num_pages;
  int partition_pages, num_parts;
  int num_items;
  float scale_log2;
};

template <int D, int TPP, int HS>
struct DecodeSmem {
  static constexpr int kBlockBytes = D * TPP * 2;       // one (page, kv head) block of K or of V
  static constexpr int kStageBytes = 2 * kBlockBytes;
  static constexpr int kPitch = D + 4;                  // fp32 row pitch of the merge buffer
  static constexpr int kHeads = kHeadsPerItem * HS;     // query heads of one work item
  static constexpr int kMergeBytes = kConsumerWarps * kHeads * kPitch * 4 + 2 * kConsumerWarps * kHeads * 4;
  static constexpr int kSortBytes = kMaxSort * 4 + kMaxSort * 2;
  static constexpr int kFixedBytes = kMergeBytes + kSortBytes + 1024;
  // A stage is always consumed by warp (stage % 4): the ring length is a multiple of the consumer
  // warp count, so a warp meets the phases of its own stages strictly in order.
  static constexpr int kStagesRaw = ((kSmemBudget - kFixedBytes) / kStageBytes) / kConsumerWarps * kConsumerWarps;
  static constexpr int kStages = kStagesRaw > 16 ? 16 : (kStagesRaw < kConsumerWarps ? kConsumerWarps : kStagesRaw);
  static constexpr int kTotalBytes = kStages * kStageBytes + kFixedBytes;
};

struct ItemCoord {
  int seq, kvh, hg, part;
};

template <bool SPLIT>
__device__ __forceinline__ ItemCoord decode_item(int item, const DecodeParams& p, const uint16_t* sm_order, bool sorted) {
  ItemCoord c;
  c.hg = item % p.head_groups;
  int r = item / p.head_groups;
  c.kvh = r % p.num_kv_heads;
  r /= p.num_kv_heads;
  if (SPLIT) {
    c.part = r % p.num_parts;
    c.seq = r / p.num_parts;
  } else {
    c.part = 0;
    c.seq = sorted ? (int)sm_order[r] : r;
  }
  return c;
}

template <bool SPLIT>
__device__ __forceinline__ void page_range(const DecodeParams& p, int len, int part, int tpp, int& pb, int& pe) {
  int npages = (len > 0 && p.num_pages > 0) ? (len + tpp - 1) / tpp : 0;
  if (npages > p.max_pages_per_seq) npages = p.max_pages_per_seq;
  if (SPLIT) {
    pb = part * p.partition_pages;
    pe = min(pb + p.partition_pages, npages);
    if (pe < pb) pe = pb;
  } else {
    pb = 0;
    pe = npages;
  }
}

// HS = 2: a work item covers 16 query heads of one kv head (two N = 8 MMA column sets fed from the same K / V fragments),
// so that groups of more than 8 heads per kv head still read every page once.
template <typename T, int D, int TPP, bool SPLIT, bool APPEND, int HS>
__global__ void __launch_bounds__(kDecodeThreads, 2) paged_decode_kernel(const DecodeParams p) {
  using SM = DecodeSmem<D, TPP, HS>;
  constexpr int HPI = SM::kHeads;
  using MMA = Mma16816<T>;
  constexpr int NST = SM::kStages;
  constexpr int KSTEPS = D / 16;
  constexpr int MTILES = D / 16;
  constexpr int UNITS = TPP / 16;

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* stages = smem;
  float* sm_O = reinterpret_cast<float*>(smem + NST * SM::kStageBytes);
  float* sm_m = sm_O + kConsumerWarps * HPI * SM::kPitch;
  float* sm_l = sm_m + kConsumerWarps * HPI;
  int* sm_len = reinterpret_cast<int*>(sm_l + kConsumerWarps * HPI);
  uint16_t* sm_order = reinterpret_cast<uint16_t*>(sm_len + kMaxSort);
  uint64_t* bars = reinterpret_cast<uint64_t*>(
      (reinterpret_cast<uintptr_t>(sm_order + kMaxSort) + 15) & ~uintptr_t(15));
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + NST;
  uint64_t* item_full = bars + 2 * NST;
  uint64_t* item_empty = item_full + 2;
  uint64_t* merge_bar = item_empty + 2;  // [0]: all warps wrote their state, [1]: all warps read it
  int* item_ring = reinterpret_cast<int*>(merge_bar + 2);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const WaitCtx status{&p.hdr->status, p.wait_limit};

  if (tid == 0) {
    for (int i = 0; i < NST; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&item_full[i], 1);
      mbar_init(&item_empty[i], kConsumerWarps);
      mbar_init(&merge_bar[i], kConsumerWarps);
    }
    fence_mbar_init();
  }
  const bool sorted = !SPLIT && p.num_seqs <= kMaxSort;
  if (sorted) {
    for (int s = tid; s < p.num_seqs; s += kDecodeThreads) sm_len[s] = p.seq_lens[s];
    __syncthreads();
    for (int s = tid; s < p.num_seqs; s += kDecodeThreads) {
      const int ls = sm_len[s];
      int rank = 0;
      for (int j = 0; j < p.num_seqs; ++j) {
        const int lj = sm_len[j];
        rank += (lj > ls) || (lj == ls && j < s);
      }
      sm_order[rank] = (uint16_t)s;
    }
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer warp ------------------------------
    const unsigned char* kp = static_cast<const unsigned char*>(p.k_pool);
    const unsigned char* vp = static_cast<const unsigned char*>(p.v_pool);
    uint32_t n_item = 0, it = 0;
    for (;;) {
      int item = 0;
      if (lane == 0) item = (int)atomicAdd(&p.hdr->work_counter, 1u);
      item = __shfl_sync(0xffffffffu, item, 0);
      int ok = 1;
      if (lane == 0) {
        const int slot = n_item & 1;
        ok = mbar_wait(&item_empty[slot], ((n_item >> 1) & 1) ^ 1, status);
        if (ok) {
          item_ring[slot] = item;
          mbar_arrive(&item_full[slot]);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      ++n_item;
      if (item >= p.num_items) break;

      const ItemCoord c = decode_item<SPLIT>(item, p, sm_order, sorted);
      const int len = sorted ? sm_len[c.seq] : p.seq_lens[c.seq];
      int pb, pe;
      page_range<SPLIT>(p, len, c.part, TPP, pb, pe);
      const int npg = pe - pb;
      const uint32_t* row = p.page_table + (size_t)c.seq * p.max_pages_per_seq + pb;
      uint32_t pid_next = lane < npg ? row[lane] : 0u;
      for (int j0 = 0; j0 < npg; j0 += 32) {
        const uint32_t pid_cur = pid_next;
        if (j0 + 32 + lane < npg) pid_next = row[j0 + 32 + lane];
        const int cnt = min(32, npg - j0);
        // NST consecutive pages go to NST different stages, so NST lanes each take one: wait for the stage, announce
        // the bytes, issue the two copies.  (A single issuing lane costs ~600 cycles per page, which caps small blocks -
        // head_dim 32..64 with 16-token pages - far below the memory bandwidth.)
        for (int b0 = 0; b0 < cnt; b0 += NST) {
          const int k = b0 + lane;
          uint32_t pid = __shfl_sync(0xffffffffu, pid_cur, k & 31);
          if (lane < NST && k < cnt) {
            const uint32_t n = it + j0 + k;
            const uint32_t stage = n % NST;
            ok = mbar_wait(&empty_bar[stage], ((n / NST) & 1) ^ 1, status);
            if (ok) {
              if ((long long)pid >= p.num_pages) pid = (uint32_t)(p.num_pages - 1);
              const size_t off = ((size_t)pid * p.num_kv_heads + c.kvh) * SM::kBlockBytes;
              unsigned char* dst = stages + stage * SM::kStageBytes;
              mbar_arrive_expect_tx(&full_bar[stage], SM::kStageBytes);
              bulk_g2s(dst, kp + off, SM::kBlockBytes, &full_bar[stage]);
              bulk_g2s(dst + SM::kBlockBytes, vp + off, SM::kBlockBytes, &full_bar[stage]);
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) return;
        }
      }
      // Pad the item to a multiple of four pages with empty hand-shakes, so that local page j always
      // goes to warp j % 4 whatever the CTA processed before: the summation order of a work item, and
      // with it every output bit, is then independent of how items were scheduled.
      const int npg_pad = (npg + kConsumerWarps - 1) & ~(kConsumerWarps - 1);
      if (lane == 0) {
        for (int j = npg; j < npg_pad && ok; ++j) {
          const uint32_t n = it + j;
          const uint32_t stage = n % NST;
          ok = mbar_wait(&empty_bar[stage], ((n / NST) & 1) ^ 1, status);
          if (ok) mbar_arrive(&full_bar[stage]);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) return;
      it += npg_pad;
    }
    // Every CTA has drawn its last item before it gets here, so the CTA that arrives last can put the scheduler's
    // counters back to zero for the next launch that uses this workspace.
    if (lane == 0) {
      __threadfence();
      if (atomicAdd(&p.hdr->done_counter, 1u) == gridDim.x - 1) {
        p.hdr->work_counter = 0u;
        p.hdr->done_counter = 0u;
      }
    }
    return;
  }

  // -------------------------------- consumer warps --------------------------------
  const int g = lane >> 2;
  const int t = lane & 3;
  const T* qbase = static_cast<const T*>(p.q);
  uint32_t n_item = 0, it = 0, n_merge = 0;
  for (;;) {
    const int slot = n_item & 1;
    if (!mbar_wait(&item_full[slot], (n_item >> 1) & 1, status)) return;
    const int item = item_ring[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(&item_empty[slot]);
    ++n_item;
    if (item >= p.num_items) break;

    const ItemCoord c = decode_item<SPLIT>(item, p, sm_order, sorted);
    const int len = sorted ? sm_len[c.seq] : p.seq_lens[c.seq];
    int pb, pe;
    page_range<SPLIT>(p, len, c.part, TPP, pb, pe);
    const int npg = pe - pb;
    const int head0 = c.kvh * p.group + c.hg * HPI;
    const int nheads = min(HPI, p.group - c.hg * HPI);

    // Q^T as the B operand: b0 = Q[head g][16ks + 2t, +1], b1 = Q[head g][16ks + 8 + 2t, +1]
    uint32_t qf[HS][KSTEPS][2];
#pragma unroll
    for (int hs = 0; hs < HS; ++hs) {
      const bool valid = 8 * hs + g < nheads;
      const uint32_t* qrow =
          reinterpret_cast<const uint32_t*>(qbase + ((size_t)c.seq * p.num_q_heads + head0 + (valid ? 8 * hs + g : 0)) * D);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        qf[hs][ks][0] = valid ? qrow[ks * 8 + t] : 0u;
        qf[hs][ks][1] = valid ? qrow[ks * 8 + 4 + t] : 0u;
      }
    }
    // Append form: the sequence's last token (position len - 1) is not in the pool yet.  The warp that owns its page
    // fetches the token's K and V rows here, and when the page lands in shared memory it overwrites the token's slot
    // there before using it; the item of the first head group also stores the rows into the pool.
    int last_j = -1, last_slot = 0;
    uint4 app_k = make_uint4(0u, 0u, 0u, 0u), app_v = make_uint4(0u, 0u, 0u, 0u);
    long long app_block = -1;  // byte offset of the (page, kv head) block in the pools, -1 = do not store
    if (APPEND && len > 0) {
      const int last_page = (len - 1) / TPP;
      if (last_page >= pb && last_page < pe && ((last_page - pb) & (kConsumerWarps - 1)) == warp) {
        last_j = last_page - pb;
        last_slot = (len - 1) - last_page * TPP;
        const size_t row = ((size_t)c.seq * p.num_kv_heads + c.kvh) * D;
        if (lane < D / 8) {
          app_k = reinterpret_cast<const uint4*>(static_cast<const T*>(p.new_k) + row)[lane];
          app_v = reinterpret_cast<const uint4*>(static_cast<const T*>(p.new_v) + row)[lane];
        }
        if (c.hg == 0) {
          const uint32_t pid = p.page_table[(size_t)c.seq * p.max_pages_per_seq + last_page];
          if ((long long)pid < p.num_pages) app_block = ((long long)pid * p.num_kv_heads + c.kvh) * SM::kBlockBytes;
        }
      }
    }
    float m_run[HS][2], l_run[HS][2];
    float o[HS][MTILES][4];
#pragma unroll
    for (int hs = 0; hs < HS; ++hs) {
      m_run[hs][0] = m_run[hs][1] = -INFINITY;
      l_run[hs][0] = l_run[hs][1] = 0.f;
#pragma unroll
      for (int i = 0; i < MTILES; ++i) o[hs][i][0] = o[hs][i][1] = o[hs][i][2] = o[hs][i][3] = 0.f;
    }

    // Page n (counted over the whole kernel, items padded to multiples of four) lives in stage n % NST
    // and belongs to warp n % 4; `it` is a multiple of four, so local page j goes to warp j % 4.
    const int npg_pad = (npg + kConsumerWarps - 1) & ~(kConsumerWarps - 1);
    for (int j = warp; j < npg_pad; j += kConsumerWarps) {
      const uint32_t n = it + j;
      const uint32_t stage = n % NST;
      if (!mbar_wait(&full_bar[stage], (n / NST) & 1, status)) return;
      if (j >= npg) {  // padding hand-shake: nothing was copied
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        continue;
      }
      if (APPEND && j == last_j) {
        unsigned char* ks = stages + stage * SM::kStageBytes;
        unsigned char* vs = ks + SM::kBlockBytes;
        if (lane < D / 8) {
          // K block [D/8][TPP][8]: chunk `lane` of the token; V block [D][TPP]: elements 8 lane .. 8 lane + 7
          const int k_off = lane * (TPP * 16) + last_slot * 16;
          *reinterpret_cast<uint4*>(ks + k_off) = app_k;
          const uint32_t w[4] = {app_v.x, app_v.y, app_v.z, app_v.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const uint16_t val = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
            *reinterpret_cast<uint16_t*>(vs + (lane * 8 + e) * (TPP * 2) + last_slot * 2) = val;
          }
          if (app_block >= 0) {
            unsigned char* kg = static_cast<unsigned char*>(const_cast<void*>(p.k_pool)) + app_block;
            unsigned char* vg = static_cast<unsigned char*>(const_cast<void*>(p.v_pool)) + app_block;
            *reinterpret_cast<uint4*>(kg + k_off) = app_k;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const uint16_t val = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
              *reinterpret_cast<uint16_t*>(vg + (lane * 8 + e) * (TPP * 2) + last_slot * 2) = val;
            }
          }
        }
        // the stage is refilled later by an asynchronous copy: order these generic writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
      }
      const uint32_t kb = smem_u32(stages + stage * SM::kStageBytes);
      const uint32_t vb = kb + SM::kBlockBytes;
      const int tok0 = (pb + j) * TPP;
#pragma unroll
      for (int u = 0; u < UNITS; ++u) {
        const int nvalid = len - (tok0 + 16 * u);
        if (nvalid <= 0) break;
        // ---- S^T = K . Q^T (the K fragments serve every head set) ----
        float s[HS][4];
#pragma unroll
        for (int hs = 0; hs < HS; ++hs) s[hs][0] = s[hs][1] = s[hs][2] = s[hs][3] = 0.f;
        {
          // matrix i = lane/8: chunk 2ks + (i>>1), tokens 8*(i&1) + lane%8
          const int mi = lane >> 3, r = lane & 7;
          const uint32_t a_lane = kb + (uint32_t)((mi >> 1) * (TPP * 16) + (16 * u + (mi & 1) * 8 + r) * 16);
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, a_lane + ks * 2 * (TPP * 16));
#pragma unroll
            for (int hs = 0; hs < HS; ++hs) MMA::run(s[hs], a, qf[hs][ks][0], qf[hs][ks][1]);
          }
        }
        // s[0],s[1]: token g, heads 2t,2t+1 of the set;  s[2],s[3]: token g+8
        const bool v_lo = g < nvalid, v_hi = g + 8 < nvalid;
        uint32_t b0[HS], b1[HS], r0[HS], r1[HS];
#pragma unroll
        for (int hs = 0; hs < HS; ++hs) {
          s[hs][0] = v_lo ? s[hs][0] * p.scale_log2 : -INFINITY;
          s[hs][1] = v_lo ? s[hs][1] * p.scale_log2 : -INFINITY;
          s[hs][2] = v_hi ? s[hs][2] * p.scale_log2 : -INFINITY;
          s[hs][3] = v_hi ? s[hs][3] * p.scale_log2 : -INFINITY;
          float mx0 = fmaxf(s[hs][0], s[hs][2]), mx1 = fmaxf(s[hs][1], s[hs][3]);
#pragma unroll
          for (int sh = 4; sh <= 16; sh <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
          }
          const float mn0 = fmaxf(m_run[hs][0], mx0), mn1 = fmaxf(m_run[hs][1], mx1);
          // token 0 of a processed unit is always valid, so mn0/mn1 are finite here unless the
          // data itself is non-finite
          const float c0 = fast_exp2(m_run[hs][0] - mn0), c1 = fast_exp2(m_run[hs][1] - mn1);
          m_run[hs][0] = mn0;
          m_run[hs][1] = mn1;
          const float p0 = fast_exp2(s[hs][0] - mn0), p1 = fast_exp2(s[hs][1] - mn1);
          const float p2 = fast_exp2(s[hs][2] - mn0), p3 = fast_exp2(s[hs][3] - mn1);
          l_run[hs][0] = l_run[hs][0] * c0 + p0 + p2;
          l_run[hs][1] = l_run[hs][1] * c1 + p1 + p3;
          if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {
#pragma unroll
            for (int i = 0; i < MTILES; ++i) {
              o[hs][i][0] *= c0;
              o[hs][i][1] *= c1;
              o[hs][i][2] *= c0;
              o[hs][i][3] *= c1;
            }
          }
          // P^T as the B operand of the PV MMA.  bf16 keeps only 8 bits of P, so there the residual
          // P - bf16(P) goes through a second MMA and the product is accurate to ~2^-17.
          const uint32_t pk0 = MMA::pack(p0, p1), pk1 = MMA::pack(p2, p3);
          b0[hs] = movmatrix_trans(pk0);
          b1[hs] = movmatrix_trans(pk1);
          r0[hs] = r1[hs] = 0;
          if (MMA::kSplitP) {
            r0[hs] = movmatrix_trans(MMA::pack_residual(p0, p1, pk0));
            r1[hs] = movmatrix_trans(MMA::pack_residual(p2, p3, pk1));
          }
        }
        // ---- O^T += V^T . P^T (the V fragments serve every head set) ----
        {
          // matrix i = lane/8: d rows 8*(i&1) + lane%8 of the m-tile, token half i>>1
          const int mi = lane >> 3, r = lane & 7;
          const uint32_t a_lane = vb + (uint32_t)(((mi & 1) * 8 + r) * (TPP * 2) + 32 * u + (mi >> 1) * 16);
          uint32_t mask_lo = 0xffffffffu, mask_hi = 0xffffffffu;
          if (nvalid < 16) {
            // a0/a1 hold tokens 2t,2t+1 and a2/a3 tokens 2t+8,2t+9: zero what lies past the length
            const int ta = 2 * t, tb = 2 * t + 8;
            mask_lo = (ta < nvalid ? 0x0000ffffu : 0u) | (ta + 1 < nvalid ? 0xffff0000u : 0u);
            mask_hi = (tb < nvalid ? 0x0000ffffu : 0u) | (tb + 1 < nvalid ? 0xffff0000u : 0u);
          }
#pragma unroll
          for (int mt = 0; mt < MTILES; ++mt) {
            uint32_t a[4];
            ldmatrix_x4(a, a_lane + mt * 16 * (TPP * 2));
            if (nvalid < 16) {
              a[0] &= mask_lo;
              a[1] &= mask_lo;
              a[2] &= mask_hi;
              a[3] &= mask_hi;
            }
#pragma unroll
            for (int hs = 0; hs < HS; ++hs) {
              MMA::run(o[hs][mt], a, b0[hs], b1[hs]);
              if (MMA::kSplitP) MMA::run(o[hs][mt], a, r0[hs], r1[hs]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
    it += npg_pad;

    // ---- merge the four warps' partial states ----
#pragma unroll
    for (int hs = 0; hs < HS; ++hs) {
#pragma unroll
      for (int sh = 4; sh <= 16; sh <<= 1) {
        l_run[hs][0] += __shfl_xor_sync(0xffffffffu, l_run[hs][0], sh);
        l_run[hs][1] += __shfl_xor_sync(0xffffffffu, l_run[hs][1], sh);
      }
      const int hcol = warp * HPI + 8 * hs + 2 * t;  // this thread's two heads of the set
      if (g == 0) {
        sm_m[hcol] = m_run[hs][0];
        sm_m[hcol + 1] = m_run[hs][1];
        sm_l[hcol] = l_run[hs][0];
        sm_l[hcol + 1] = l_run[hs][1];
      }
      float* ow = sm_O + hcol * SM::kPitch;
#pragma unroll
      for (int mt = 0; mt < MTILES; ++mt) {
        ow[16 * mt + g] = o[hs][mt][0];
        ow[SM::kPitch + 16 * mt + g] = o[hs][mt][1];
        ow[16 * mt + g + 8] = o[hs][mt][2];
        ow[SM::kPitch + 16 * mt + g + 8] = o[hs][mt][3];
      }
    }
    // consumer-only barrier built on an mbarrier so that, like every other wait here, it is bounded
    __syncwarp();
    if (lane == 0) mbar_arrive(&merge_bar[0]);
    if (!mbar_wait(&merge_bar[0], n_merge & 1, status)) return;
    for (int idx = tid; idx < nheads * D; idx += kConsumerThreads) {
      const int h = idx / D, d = idx - h * D;
      float mw[kConsumerWarps];
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        mw[w] = sm_m[w * HPI + h];
        M = fmaxf(M, mw[w]);
      }
      float num = 0.f, den = 0.f;
      if (M > -INFINITY) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          const float wgt = fast_exp2(mw[w] - M);
          num += wgt * sm_O[(w * HPI + h) * SM::kPitch + d];
          den += wgt * sm_l[w * HPI + h];
        }
      }
      const size_t row = (size_t)c.seq * p.num_q_heads + head0 + h;
      if (SPLIT) {
        const size_t prow = row * p.num_parts + c.part;
        p.part_acc[prow * D + d] = num;
        if (d == 0) {
          p.part_m[prow] = M > -INFINITY ? M * kLn2 : -INFINITY;
          p.part_l[prow] = den;
        }
      } else {
        const float val = den > 0.f ? num / den : 0.f;
        if (p.out_f32)
          static_cast<float*>(p.out)[row * D + d] = val;
        else
          static_cast<T*>(p.out)[row * D + d] = MMA::from_float(val);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&merge_bar[1]);
    if (!mbar_wait(&merge_bar[1], n_merge & 1, status)) return;
    ++n_merge;
  }
}

// Merge num_parts partial triples per row.  One CTA per row, one thread per head-dim element pair.
// m/l/acc are addressed with explicit strides so the same kernel serves the in-workspace layout
// [row][part], the part-major layout [part][row] of gathered per-GPU triples and the packed layout
// [part][row][D + 2] (acc, m, l in one row) that a single collective moves.
template <typename T>
__global__ void __launch_bounds__(128) lse_combine_kernel(const PartialsView in, void* __restrict__ out, int out_f32,
                                                          const TripleOut triple, int num_parts, int head_dim) {
  const long long row = blockIdx.x;
  const float* mr = in.m + row * in.row_stride_ml;
  const float* lr = in.l + row * in.row_stride_ml;
  __shared__ float s_w[1024];
  __shared__ float s_red[8];
  // pass 1: global max over partitions
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < num_parts; j += blockDim.x) mx = fmaxf(mx, mr[j * in.part_stride_ml]);
#pragma unroll
  for (int sh = 16; sh >= 1; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mx;
  __syncthreads();
  float M = s_red[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w) M = fmaxf(M, s_red[w]);
  __syncthreads();
  // pass 2: weights and denominator
  float den = 0.f;
  for (int j = threadIdx.x; j < num_parts; j += blockDim.x) {
    const float mj = mr[j * in.part_stride_ml];
    const float w = (mj > -INFINITY) ? __expf(mj - M) : 0.f;
    if (j < 1024) s_w[j] = w;
    den += w * lr[j * in.part_stride_ml];
  }
#pragma unroll
  for (int sh = 16; sh >= 1; sh >>= 1) den += __shfl_xor_sync(0xffffffffu, den, sh);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = den;
  __syncthreads();
  float den_all = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) den_all += s_red[w];
  const float* ar = in.acc + row * in.row_stride_acc;
  auto weight = [&](int j) {
    if (j < 1024) return s_w[j];
    const float mj = mr[j * in.part_stride_ml];
    return (mj > -INFINITY) ? __expf(mj - M) : 0.f;
  };
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    // Eight partitions' values are requested before the first is used: the loop is bound by the latency of its loads,
    // not by their number.  The sum is still taken in partition order.
    float num = 0.f;
    int j = 0;
    for (; j + 8 <= num_parts; j += 8) {
      float a[8], w[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        w[k] = weight(j + k);
        a[k] = ar[(long long)(j + k) * in.part_stride_acc + d];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (w[k] != 0.f) num = fmaf(w[k], a[k], num);
    }
    for (; j < num_parts; ++j) {
      const float w = weight(j);
      if (w != 0.f) num = fmaf(w, ar[(long long)j * in.part_stride_acc + d], num);
    }
    if (out) {
      const float v = den_all > 0.f ? num / den_all : 0.f;
      if (out_f32)
        static_cast<float*>(out)[row * head_dim + d] = v;
      else
        static_cast<T*>(out)[row * head_dim + d] = Mma16816<T>::from_float(v);
    }
    if (triple.acc) triple.acc[row * triple.row_stride_acc + d] = num;
  }
  if (threadIdx.x == 0 && triple.m) {
    triple.m[row * triple.row_stride_ml] = M;
    triple.l[row * triple.row_stride_ml] = den_all;
  }
}

template <typename T, int D, int TPP, bool SPLIT, bool APPEND, int HS>
int launch_decode_inst(const DecodeParams& p, int num_sms, cudaStream_t stream) {
  using SM = DecodeSmem<D, TPP, HS>;
  static_assert(SM::kTotalBytes <= 227 * 1024, "decode shared memory exceeds the per-CTA limit");
  auto kern = paged_decode_kernel<T, D, TPP, SPLIT, APPEND, HS>;
  static DeviceOnce configured;  // one per instantiation
  const int rc = configured.run(
      [&] { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotalBytes); });
  if (rc != 0) return rc;
  const int ctas_per_sm = SM::kTotalBytes <= kSmemBudget ? 2 : 1;
  int grid = num_sms * ctas_per_sm;
  if (grid > p.num_items) grid = p.num_items;
  if (grid < 1) grid = 1;
  kern<<<grid, kDecodeThreads, SM::kTotalBytes, stream>>>(p);
  return (int)cudaGetLastError();
}

template <typename T, bool SPLIT, int HS>
int dispatch_shape(const DecodeParams& p, int head_dim, int tpp, int num_sms, cudaStream_t stream) {
#define PAL_DECODE_CASE(DD, TT)                                                                        \
  if (head_dim == DD && tpp == TT)                                                                     \
    return p.new_k ? launch_decode_inst<T, DD, TT, SPLIT, true, (DD <= 128 ? HS : 1)>(p, num_sms, stream)   \
                   : launch_decode_inst<T, DD, TT, SPLIT, false, (DD <= 128 ? HS : 1)>(p, num_sms, stream);
  PAL_DECODE_CASE(32, 16)
  PAL_DECODE_CASE(64, 16)
  PAL_DECODE_CASE(80, 16)
  PAL_DECODE_CASE(96, 16)
  PAL_DECODE_CASE(128, 16)
  PAL_DECODE_CASE(256, 16)
  PAL_DECODE_CASE(32, 32)
  PAL_DECODE_CASE(64, 32)
  PAL_DECODE_CASE(80, 32)
  PAL_DECODE_CASE(96, 32)
  PAL_DECODE_CASE(128, 32)
  PAL_DECODE_CASE(256, 32)
#undef PAL_DECODE_CASE
  set_error("paged_attention_decode: no kernel for head_dim=%d tokens_per_page=%d "
            "(head_dim in {32,64,80,96,128,256}, tokens_per_page in {16,32})", head_dim, tpp);
  return -2;
}

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// Work items hold 16 query heads when a kv head serves more than 8 (and the accumulators fit: head_dim <= 128), else 8.
int heads_per_item(int group, int head_dim) { return group > kHeadsPerItem && head_dim <= 128 ? 2 * kHeadsPerItem : kHeadsPerItem; }

}  // namespace

int cached_sm_count() {
  static std::atomic<int> sms[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  int n = sms[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev].store(n, std::memory_order_relaxed);  // every thread computes the same value
  }
  return n;
}

int decode_num_partitions(int max_pages_per_seq, int partition_pages) {
  if (partition_pages <= 0) return 1;
  int n = (max_pages_per_seq + partition_pages - 1) / partition_pages;
  return n < 1 ? 1 : n;
}

// Two-pass when the batch alone cannot give every resident CTA (two per SM) a work item.  The number of partitions per
// sequence is then the one with the least modelled step time.  Measured on B200 (8 sequences x 131072 tokens, whole and
// under 8-way kv-head / context sharding): a step costs the larger of the HBM time of all its pages and the time the
// busiest CTA needs for its own pages (with ~200 CTAs active one CTA sustains about 28 GB/s: 64 KB in flight per ~2 us),
// plus about 1.3 us per work item a CTA handles and 75 ns per partition in the combine kernel.  So partitions should be
// as few as still give the memory system enough CTAs: e.g. one kv head per GPU runs 256-page partitions (256 items) in
// 92.7 us, 512-page ones (128 items, too few CTAs) in ~118 us and 64-page ones (1024 items) in 109 us.
int decode_auto_partition_pages(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                int max_pages_per_seq) {
  const int group = num_q_heads / num_kv_heads;
  const int hpi = heads_per_item(group, head_dim);
  const long long base = (long long)num_seqs * num_kv_heads * ((group + hpi - 1) / hpi);
  const long long slots = 2LL * cached_sm_count();
  if (base >= slots || max_pages_per_seq <= 32) return 0;
  const double page_bytes = (double)head_dim * tokens_per_page * 4.0;  // K and V block of one page
  const double hbm_ns = (double)base * max_pages_per_seq * page_bytes / 6600.0;  // 6.6 TB/s = 6600 bytes per ns
  const double page_ns = page_bytes / 28.0;                                       // one CTA among ~200 active: 28 GB/s
  int best_parts = 1;
  double best = 1e30;
  const int max_parts = max_pages_per_seq / 16;
  for (int parts = 1; parts <= max_parts && parts <= 4096; ++parts) {
    const int pp = (max_pages_per_seq + parts - 1) / parts;
    const int real_parts = (max_pages_per_seq + pp - 1) / pp;
    const long long items = base * real_parts;
    const long long waves = (items + slots - 1) / slots;
    const double stream = fmax(hbm_ns, (double)waves * pp * page_ns);
    const double t = stream + waves * 1300.0 + real_parts * 75.0;
    if (t < best * 0.995) {  // ties go to fewer, larger partitions
      best = t;
      best_parts = parts;
    }
    if (items > 16 * slots) break;
  }
  const int pp = (max_pages_per_seq + best_parts - 1) / best_parts;
  return pp >= max_pages_per_seq ? 0 : pp;
}

size_t decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                              int max_pages_per_seq, int partition_pages) {
  if (partition_pages < 0)
    partition_pages = decode_auto_partition_pages(num_seqs, num_q_heads, num_kv_heads, head_dim, tokens_per_page, max_pages_per_seq);
  size_t bytes = sizeof(WorkspaceHeader);
  if (partition_pages > 0) {
    const size_t rows = (size_t)num_seqs * num_q_heads * decode_num_partitions(max_pages_per_seq, partition_pages);
    bytes += 2 * align256(rows * 4) + align256(rows * head_dim * 4);
  }
  return bytes;
}

int launch_lse_combine(const PartialsView& in, void* out, bool out_f32, const TripleOut& triple, int num_parts,
                       long long rows, int head_dim, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (dtype == 0)
    lse_combine_kernel<__half><<<(unsigned)rows, 128, 0, stream>>>(in, out, out_f32 ? 1 : 0, triple, num_parts, head_dim);
  else
    lse_combine_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, stream>>>(in, out, out_f32 ? 1 : 0, triple, num_parts,
                                                                         head_dim);
  return (int)cudaGetLastError();
}

PartialsView decode_partials_view(const DecodeArgs& a, int* num_parts) {
  const int parts = decode_num_partitions(a.max_pages_per_seq, a.partition_pages);
  const size_t rows = (size_t)a.num_seqs * a.num_q_heads * parts;
  unsigned char* ws = static_cast<unsigned char*>(a.workspace);
  PartialsView v;
  v.m = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader));
  v.l = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader) + align256(rows * 4));
  v.acc = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader) + 2 * align256(rows * 4));
  v.part_stride_ml = 1;
  v.row_stride_ml = parts;
  v.part_stride_acc = a.head_dim;
  v.row_stride_acc = (long long)parts * a.head_dim;
  *num_parts = parts;
  return v;
}

int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
  DecodeParams p;
  p.q = a.queries;
  p.k_pool = a.k_pool;
  p.v_pool = a.v_pool;
  p.new_k = a.new_keys;
  p.new_v = a.new_values;
  p.page_table = a.page_table;
  p.seq_lens = a.sequence_lengths;
  p.out = a.out;
  p.hdr = static_cast<WorkspaceHeader*>(a.workspace);
  p.wait_limit = wait_limit_cycles();
  p.out_f32 = a.out_f32 ? 1 : 0;
  p.num_seqs = a.num_seqs;
  p.num_q_heads = a.num_q_heads;
  p.num_kv_heads = a.num_kv_heads;
  p.group = a.num_q_heads / a.num_kv_heads;
  const int hpi = heads_per_item(p.group, a.head_dim);
  p.head_groups = (p.group + hpi - 1) / hpi;
  p.max_pages_per_seq = a.max_pages_per_seq;
  p.num_pages = a.num_pages;
  p.partition_pages = a.partition_pages;
  p.num_parts = decode_num_partitions(a.max_pages_per_seq, a.partition_pages);
  p.scale_log2 = a.scale * kLog2e;
  const bool split = a.partition_pages > 0;
  const long long items =
      (long long)a.num_seqs * a.num_kv_heads * p.head_groups * (split ? p.num_parts : 1);
  if (items > 0x7fffffffLL) {
    set_error("paged_attention_decode: too many work items (%lld)", items);
    return -1;
  }
  p.num_items = (int)items;
  const size_t rows = (size_t)a.num_seqs * a.num_q_heads * p.num_parts;
  unsigned char* ws = static_cast<unsigned char*>(a.workspace);
  p.part_m = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader));
  p.part_l = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader) + align256(rows * 4));
  p.part_acc = reinterpret_cast<float*>(ws + sizeof(WorkspaceHeader) + 2 * align256(rows * 4));

  const int sms = cached_sm_count();
  int rc;
  if (a.dtype == 0)
    rc = hpi > kHeadsPerItem ? (split ? dispatch_shape<__half, true, 2>(p, a.head_dim, a.tokens_per_page, sms, stream)
                                      : dispatch_shape<__half, false, 2>(p, a.head_dim, a.tokens_per_page, sms, stream))
                             : (split ? dispatch_shape<__half, true, 1>(p, a.head_dim, a.tokens_per_page, sms, stream)
                                      : dispatch_shape<__half, false, 1>(p, a.head_dim, a.tokens_per_page, sms, stream));
  else
    rc = hpi > kHeadsPerItem
             ? (split ? dispatch_shape<__nv_bfloat16, true, 2>(p, a.head_dim, a.tokens_per_page, sms, stream)
                      : dispatch_shape<__nv_bfloat16, false, 2>(p, a.head_dim, a.tokens_per_page, sms, stream))
             : (split ? dispatch_shape<__nv_bfloat16, true, 1>(p, a.head_dim, a.tokens_per_page, sms, stream)
                      : dispatch_shape<__nv_bfloat16, false, 1>(p, a.head_dim, a.tokens_per_page, sms, stream));
  if (rc != 0) return rc;
  if (split && !a.skip_combine) {
    const long long out_rows = (long long)a.num_seqs * a.num_q_heads;
    const PartialsView in{p.part_m, p.part_l, p.part_acc, 1, p.num_parts, a.head_dim, (long long)p.num_parts * a.head_dim};
    TripleOut triple;
    if (a.packed_out) {
      // one row = head_dim values of acc, then m, then l
      triple.acc = a.packed_out;
      triple.m = a.packed_out + a.head_dim;
      triple.l = a.packed_out + a.head_dim + 1;
      triple.row_stride_ml = triple.row_stride_acc = a.head_dim + 2;
    } else {
      triple.m = a.m_out;
      triple.l = a.l_out;
      triple.acc = a.acc_out;
      triple.row_stride_ml = 1;
      triple.row_stride_acc = a.head_dim;
    }
    rc = launch_lse_combine(in, a.out, a.out_f32, triple, p.num_parts, out_rows, a.head_dim, a.dtype, stream);
  }
  return rc;
}

}  // namespace pal
