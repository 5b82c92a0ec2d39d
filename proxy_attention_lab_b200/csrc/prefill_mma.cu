// Paged-attention prefill, general-shape kernel (mma.sync m16n8k16, fp32 online softmax).
//
// Replaces pal_paged_attention_prefill (src/pal_core/kernels/paged_attention/prefill/
// paged_attention_prefill.h.metal:28-389) and PagedAttentionPrefillPrimitive::eval_gpu
// (src/pal_core/src/paged_attention_prefill_primitive.cpp:63-167) for every head_dim that is a
// multiple of 16 and tokens_per_page in {16, 32}.  The tcgen05 kernel covers the
// head_dim = 128 / tokens_per_page = 16 case that matters for throughput; this one is the
// reference-complete path.
//
// One CTA = 64 query tokens of one (sequence, query head); each of its 4 warps owns 16 rows.
// Keys come in tiles of 64 tokens: first the paged history (all visible, read through the page
// table in the pools' native striped-K / transposed-V layouts, which ldmatrix consumes
// directly), then the dense prompt K/V with the causal mask `key <= query`.
#include <math.h>

#include "common.cuh"
#include "launch.h"

namespace pal {
namespace {

constexpr int kBM = 64;
constexpr int kBN = 64;
constexpr int kPrefillThreads = 128;

struct PrefillParams {
  const void* q;
  const void* k_new;
  const void* v_new;
  const void* k_pool;
  const void* v_pool;
  const uint32_t* page_table;
  const int32_t* hist_lens;
  const int32_t* cu_seqlens;  // ragged batches: first row of each sequence in q / k_new / v_new / out; null = uniform n_new
  void* out;
  int out_f32;  // out holds float32 instead of the input type
  int num_seqs, n_new, num_q_heads, num_kv_heads, group, max_pages_per_seq;
  long long num_pages;
  float scale_log2;
};

template <typename T, int D, int TPP>
__global__ void __launch_bounds__(kPrefillThreads) prefill_mma_kernel(const PrefillParams p) {
  using MMA = Mma16816<T>;
  constexpr int DP = D + 8;                 // padded row pitch (elements) of dense tiles
  constexpr int KSTEPS = D / 16;
  constexpr int NDT = D / 8;                // output n-tiles of 8 head-dim columns
  constexpr int VEC_PER_ROW = D / 8;        // 16-byte vectors per dense row
  constexpr int PAGES_PER_TILE = kBN / TPP;
  constexpr int BLOCK_ELEMS = D * TPP;      // one (page, kv head) block

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + kBM * DP;
  T* sV = sK + kBN * DP;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int mi = lane >> 3, r8 = lane & 7;
  const int q0 = blockIdx.x * kBM;
  const int h = blockIdx.y;
  const int s = blockIdx.z;
  const int kvh = h / p.group;
  const int N = p.cu_seqlens ? p.cu_seqlens[s + 1] - p.cu_seqlens[s] : p.n_new;
  const size_t row0 = p.cu_seqlens ? (size_t)p.cu_seqlens[s] : (size_t)s * N;  // the sequence's first row
  if (q0 >= N) return;  // ragged: the grid is sized for the longest sequence
  int H = p.hist_lens[s];
  if (H < 0) H = 0;
  if (p.num_pages <= 0) H = 0;
  {
    const long long cap = (long long)p.max_pages_per_seq * TPP;
    if (H > cap) H = (int)cap;
  }

  const T* qg = static_cast<const T*>(p.q);
  const T* kg = static_cast<const T*>(p.k_new);
  const T* vg = static_cast<const T*>(p.v_new);
  const T* kpool = static_cast<const T*>(p.k_pool);
  const T* vpool = static_cast<const T*>(p.v_pool);

  // ---- Q tile -> shared (rows past N are zero) ----
  for (int v = tid; v < kBM * VEC_PER_ROW; v += kPrefillThreads) {
    const int row = v / VEC_PER_ROW, cv = v - row * VEC_PER_ROW;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (q0 + row < N)
      val = *reinterpret_cast<const uint4*>(qg + ((row0 + q0 + row) * p.num_q_heads + h) * D + cv * 8);
    *reinterpret_cast<uint4*>(sQ + row * DP + cv * 8) = val;
  }

  float o[NDT][4];
#pragma unroll
  for (int i = 0; i < NDT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int row_lo = warp * 16 + g;           // this thread's two rows inside the tile
  const int i_lo = q0 + row_lo, i_hi = i_lo + 8;  // query token indices

  const uint32_t sQ_u = smem_u32(sQ), sK_u = smem_u32(sK), sV_u = smem_u32(sV);
  const uint32_t q_lane = sQ_u + (uint32_t)(((warp * 16 + (mi & 1) * 8 + r8) * DP + (mi >> 1) * 8) * 2);

  const int hist_tiles = (H + kBN - 1) / kBN;
  const int last_q = min(q0 + kBM, N) - 1;
  const int prompt_tiles = last_q / kBN + 1;

  for (int tile = 0; tile < hist_tiles + prompt_tiles; ++tile) {
    const bool paged = tile < hist_tiles;
    const int j0 = paged ? tile * kBN : (tile - hist_tiles) * kBN;
    __syncthreads();  // previous tile fully consumed (and the Q tile written, first time round)
    if (paged) {
      // copy the tile's pages: K block and V block, D*TPP elements each, contiguous in the pools
      for (int pi = 0; pi < PAGES_PER_TILE; ++pi) {
        const int tok = j0 + pi * TPP;
        T* dk = sK + pi * BLOCK_ELEMS;
        T* dv = sV + pi * BLOCK_ELEMS;
        if (tok < H) {
          long long pid = p.page_table[(size_t)s * p.max_pages_per_seq + tok / TPP];
          if (pid >= p.num_pages) pid = p.num_pages - 1;
          const size_t off = ((size_t)pid * p.num_kv_heads + kvh) * BLOCK_ELEMS;
          for (int v = tid; v < BLOCK_ELEMS / 8; v += kPrefillThreads) {
            *reinterpret_cast<uint4*>(dk + v * 8) = *reinterpret_cast<const uint4*>(kpool + off + v * 8);
            *reinterpret_cast<uint4*>(dv + v * 8) = *reinterpret_cast<const uint4*>(vpool + off + v * 8);
          }
        } else {
          for (int v = tid; v < BLOCK_ELEMS / 8; v += kPrefillThreads) {
            *reinterpret_cast<uint4*>(dk + v * 8) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(dv + v * 8) = make_uint4(0, 0, 0, 0);
          }
        }
      }
      if (j0 + kBN > H) {
        __syncthreads();
        // zero V for the slots past the history length: they may hold anything, and 0 * NaN = NaN
        const int pi = (H - j0) / TPP;
        const int first_bad = (H - j0) - pi * TPP;
        if (pi < PAGES_PER_TILE && first_bad > 0) {
          T* dv = sV + pi * BLOCK_ELEMS;
          for (int d = tid; d < D; d += kPrefillThreads)
            for (int x = first_bad; x < TPP; ++x) dv[d * TPP + x] = MMA::from_float(0.f);
        }
      }
    } else {
      for (int v = tid; v < kBN * VEC_PER_ROW; v += kPrefillThreads) {
        const int row = v / VEC_PER_ROW, cv = v - row * VEC_PER_ROW;
        uint4 kk = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
        if (j0 + row < N) {
          const size_t off = ((row0 + j0 + row) * p.num_kv_heads + kvh) * D + cv * 8;
          kk = *reinterpret_cast<const uint4*>(kg + off);
          vv = *reinterpret_cast<const uint4*>(vg + off);
        }
        *reinterpret_cast<uint4*>(sK + row * DP + cv * 8) = kk;
        *reinterpret_cast<uint4*>(sV + row * DP + cv * 8) = vv;
      }
    }
    __syncthreads();

    // ---- S = Q K^T for this warp's 16 rows x 64 keys ----
    float sacc[kBN / 8][4];
#pragma unroll
    for (int i = 0; i < kBN / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, q_lane + ks * 32);
#pragma unroll
      for (int nt = 0; nt < kBN / 8; nt += 2) {
        uint32_t b[4];
        const int ntile = nt + (mi >> 1);
        uint32_t addr;
        if (paged) {
          const int tok = ntile * 8;
          const int pi = tok / TPP, tp = tok - pi * TPP;
          addr = sK_u + (uint32_t)((pi * BLOCK_ELEMS) * 2 + (2 * ks + (mi & 1)) * (TPP * 16) + (tp + r8) * 16);
        } else {
          addr = sK_u + (uint32_t)(((ntile * 8 + r8) * DP + ks * 16 + (mi & 1) * 8) * 2);
        }
        ldmatrix_x4(b, addr);
        MMA::run(sacc[nt], a, b[0], b[1]);
        MMA::run(sacc[nt + 1], a, b[2], b[3]);
      }
    }

    // ---- mask + online softmax ----
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < kBN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = j0 + nt * 8 + 2 * t + (e & 1);
        const int qi = (e & 2) ? i_hi : i_lo;
        const bool vis = paged ? (key < H) : (key <= qi && key < N);
        const float v = vis ? sacc[nt][e] * p.scale_log2 : -INFINITY;
        sacc[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
    }
    float corr[2], mnew[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      mnew[rr] = fmaxf(m_run[rr], mx[rr]);
      // a row that has seen no visible key yet keeps m = -inf; use 0 as the subtrahend there
      const float msafe = mnew[rr] > -INFINITY ? mnew[rr] : 0.f;
      corr[rr] = fast_exp2(m_run[rr] - msafe);
      m_run[rr] = mnew[rr];
      mnew[rr] = msafe;
    }
    float lsum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < kBN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(sacc[nt][e] - mnew[e >> 1]);
        sacc[nt][e] = pv;
        lsum[e >> 1] += pv;
      }
    }
    l_run[0] = l_run[0] * corr[0] + lsum[0];
    l_run[1] = l_run[1] * corr[1] + lsum[1];
#pragma unroll
    for (int i = 0; i < NDT; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < kBN / 16; ++kk) {
      uint32_t a[4];
      a[0] = MMA::pack(sacc[2 * kk][0], sacc[2 * kk][1]);
      a[1] = MMA::pack(sacc[2 * kk][2], sacc[2 * kk][3]);
      a[2] = MMA::pack(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
      a[3] = MMA::pack(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
      // bf16 keeps 8 bits of P; the residual P - bf16(P) goes through a second MMA (see decode.cu)
      uint32_t ar[4] = {0u, 0u, 0u, 0u};
      if (MMA::kSplitP) {
        ar[0] = MMA::pack_residual(sacc[2 * kk][0], sacc[2 * kk][1], a[0]);
        ar[1] = MMA::pack_residual(sacc[2 * kk][2], sacc[2 * kk][3], a[1]);
        ar[2] = MMA::pack_residual(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], a[2]);
        ar[3] = MMA::pack_residual(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], a[3]);
      }
#pragma unroll
      for (int nd = 0; nd < NDT; nd += 2) {
        uint32_t b[4];
        if (paged) {
          const int tok = kk * 16;
          const int pi = tok / TPP, tp = tok - pi * TPP;
          const uint32_t addr = sV_u + (uint32_t)((pi * BLOCK_ELEMS) * 2 + ((nd + (mi >> 1)) * 8 + r8) * (TPP * 2) +
                                                  tp * 2 + (mi & 1) * 16);
          ldmatrix_x4(b, addr);
        } else {
          const uint32_t addr =
              sV_u + (uint32_t)(((kk * 16 + (mi & 1) * 8 + r8) * DP + (nd + (mi >> 1)) * 8) * 2);
          ldmatrix_x4_trans(b, addr);
        }
        MMA::run(o[nd], a, b[0], b[1]);
        MMA::run(o[nd + 1], a, b[2], b[3]);
        if (MMA::kSplitP) {
          MMA::run(o[nd], ar, b[0], b[1]);
          MMA::run(o[nd + 1], ar, b[2], b[3]);
        }
      }
    }
  }

  // ---- normalise and store: out[((s*N + i)*Hq + h)*D + d] ----
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
    l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
  }
  T* outp = static_cast<T*>(p.out);
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int qi = rr ? i_hi : i_lo;
    if (qi >= N) continue;
    const float inv = l_run[rr] > 0.f ? 1.f / l_run[rr] : 0.f;
    const size_t off = ((row0 + qi) * p.num_q_heads + h) * D;
    if (p.out_f32) {
      float2* orow = reinterpret_cast<float2*>(static_cast<float*>(p.out) + off);
#pragma unroll
      for (int nd = 0; nd < NDT; ++nd) orow[nd * 4 + t] = make_float2(o[nd][2 * rr] * inv, o[nd][2 * rr + 1] * inv);
    } else {
      uint32_t* orow = reinterpret_cast<uint32_t*>(outp + off);
#pragma unroll
      for (int nd = 0; nd < NDT; ++nd) orow[nd * 4 + t] = MMA::pack(o[nd][2 * rr] * inv, o[nd][2 * rr + 1] * inv);
    }
  }
}

template <typename T, int D, int TPP>
int launch_inst(const PrefillParams& p, cudaStream_t stream) {
  constexpr int smem = 3 * kBM * (D + 8) * 2;
  auto kern = prefill_mma_kernel<T, D, TPP>;
  static DeviceOnce configured;  // one per instantiation
  const int rc = configured.run([&] { return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  if (rc != 0) return rc;
  dim3 grid((p.n_new + kBM - 1) / kBM, p.num_q_heads, p.num_seqs);
  kern<<<grid, kPrefillThreads, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

template <typename T>
int dispatch(const PrefillParams& p, int d, int tpp, cudaStream_t stream) {
#define PAL_PREFILL_CASE(DD, TT) \
  if (d == DD && tpp == TT) return launch_inst<T, DD, TT>(p, stream);
  PAL_PREFILL_CASE(32, 16)
  PAL_PREFILL_CASE(64, 16)
  PAL_PREFILL_CASE(80, 16)
  PAL_PREFILL_CASE(96, 16)
  PAL_PREFILL_CASE(128, 16)
  PAL_PREFILL_CASE(256, 16)
  PAL_PREFILL_CASE(32, 32)
  PAL_PREFILL_CASE(64, 32)
  PAL_PREFILL_CASE(80, 32)
  PAL_PREFILL_CASE(96, 32)
  PAL_PREFILL_CASE(128, 32)
  PAL_PREFILL_CASE(256, 32)
#undef PAL_PREFILL_CASE
  set_error("paged_attention_prefill: no kernel for head_dim=%d tokens_per_page=%d "
            "(head_dim in {32,64,80,96,128,256}, tokens_per_page in {16,32})", d, tpp);
  return -2;
}

}  // namespace

int launch_prefill_mma(const PrefillArgs& a, cudaStream_t stream) {
  PrefillParams p;
  p.q = a.q_prompt;
  p.k_new = a.k_prompt;
  p.v_new = a.v_prompt;
  p.k_pool = a.k_pool;
  p.v_pool = a.v_pool;
  p.page_table = a.page_table;
  p.hist_lens = a.history_lens;
  p.cu_seqlens = a.cu_seqlens;
  p.out = a.out;
  p.out_f32 = a.out_f32 ? 1 : 0;
  p.num_seqs = a.num_seqs;
  p.n_new = a.tokens_per_seq;
  p.num_q_heads = a.num_q_heads;
  p.num_kv_heads = a.num_kv_heads;
  p.group = a.num_q_heads / a.num_kv_heads;
  p.max_pages_per_seq = a.max_pages_per_seq;
  p.num_pages = a.num_pages;
  p.scale_log2 = a.scale * kLog2e;
  if (a.num_seqs > 65535 || a.num_q_heads > 65535) {
    set_error("paged_attention_prefill: num_seqs and num_q_heads are limited to 65535");
    return -1;
  }
  return a.dtype == 0 ? dispatch<__half>(p, a.head_dim, a.tokens_per_page, stream)
                      : dispatch<__nv_bfloat16>(p, a.head_dim, a.tokens_per_page, stream);
}

}  // namespace pal
