// fill_kv_pages for sm_100a: scatter new K/V tokens [T, Hkv, D] into the striped-K /
// transposed-V page pools, in place and bit-exact.
//
// Replaces fill_kv_pages_kernel (src/pal_core/kernels/paged_attention/fill_kv_pages.h.metal:30-121)
// and its launcher (src/pal_core/src/fill_kv_pages_primitive.cpp:70-170).  Unlike the reference
// launcher, the pools are not copied first.
//
// Scattered tokens (fill_kv_pages_kernel): one thread moves one 16-byte vector (8 elements) of one
// token's K and of its V:
//   K[page, h, d/8, slot, 0..7] <- new_keys[t, h, d..d+7]        one 16-byte store
//   V[page, h, d+j, slot]       <- new_values[t, h, d+j], j<8    eight 2-byte stores, TPP apart
// The V stores cannot be widened for a single token: consecutive d are TPP elements apart in the
// pool, so each element lives in its own 32-byte sector.  Loads of the source are fully coalesced.
//
// Appended runs (fill_kv_pages_grouped_kernel): a CTA takes 16 consecutive tokens of the list.  Where
// 2, 4 or 8 of them go to consecutive slots of one page starting at a multiple of that count - what a
// prefill append looks like - their K vectors are contiguous per (head, chunk) and their V elements are
// 4, 8 or 16 contiguous bytes per (head, d): the tokens are staged in shared memory and written back
// transposed with one wide store per chunk.  Groups without any such chunk take the scattered path.
#include "common.cuh"
#include "launch.h"

namespace pal {

template <bool kSlots>
__global__ void __launch_bounds__(256) fill_kv_pages_kernel(
    const uint4* __restrict__ new_keys, const uint4* __restrict__ new_values, uint16_t* __restrict__ k_pool,
    uint16_t* __restrict__ v_pool, const int64_t* __restrict__ slot_mapping, const uint32_t* __restrict__ page_table,
    const int32_t* __restrict__ write_positions, const uint32_t* __restrict__ query_to_seq_map, long long num_tokens,
    int num_seqs, int num_kv_heads, int head_dim, int tokens_per_page, long long num_pages, int max_pages_per_seq) {
  const int vec_per_head = head_dim >> 3;
  const int vec_per_token = num_kv_heads * vec_per_head;
  const long long total_vecs = num_tokens * vec_per_token;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total_vecs; v += stride) {
    const long long t = v / vec_per_token;
    const int in_token = (int)(v - t * vec_per_token);
    const int h = in_token / vec_per_head;
    const int c = in_token - h * vec_per_head;

    long long page;
    int slot;
    if (kSlots) {
      const long long s = slot_mapping[t];
      if (s < 0 || s >= num_pages * tokens_per_page) continue;
      page = s / tokens_per_page;
      slot = (int)(s - page * tokens_per_page);
    } else {
      // fill_kv_pages.h.metal:64-72
      const uint32_t seq = query_to_seq_map[t];
      const int pos = write_positions[t];
      if (pos < 0 || seq >= (uint32_t)num_seqs) continue;
      const int block = pos / tokens_per_page;
      if (block >= max_pages_per_seq) continue;
      slot = pos - block * tokens_per_page;
      page = page_table[(long long)seq * max_pages_per_seq + block];
      if (page >= num_pages) continue;
    }

    const uint4 kv = new_keys[v];
    const uint4 vv = new_values[v];
    const long long head_base = (page * num_kv_heads + h) * (long long)head_dim * tokens_per_page;
    // K: [.., d/8, TPP, 8]  (fill_kv_pages.h.metal:94-101)
    *reinterpret_cast<uint4*>(k_pool + head_base + ((long long)c * tokens_per_page + slot) * 8) = kv;
    // V: [.., d, TPP]       (fill_kv_pages.h.metal:106-114)
    uint16_t* vp = v_pool + head_base + (long long)c * 8 * tokens_per_page + slot;
    const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      vp[(2 * j) * tokens_per_page] = (uint16_t)(w[j] & 0xffffu);
      vp[(2 * j + 1) * tokens_per_page] = (uint16_t)(w[j] >> 16);
    }
  }
}


constexpr int kGroupTokens = 16;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
               : "memory");
}

// (page, slot) of token t, or page = -1 when the token has to be skipped
template <bool kSlots>
__device__ __forceinline__ void token_destination(long long t, const int64_t* slot_mapping, const uint32_t* page_table,
                                                  const int32_t* write_positions, const uint32_t* query_to_seq_map,
                                                  int num_seqs, int tokens_per_page, long long num_pages,
                                                  int max_pages_per_seq, long long& page, int& slot) {
  page = -1;
  slot = 0;
  if (kSlots) {
    const long long s = slot_mapping[t];
    if (s < 0 || s >= num_pages * tokens_per_page) return;
    page = s / tokens_per_page;
    slot = (int)(s - page * tokens_per_page);
  } else {
    const uint32_t seq = query_to_seq_map[t];
    const int pos = write_positions[t];
    if (pos < 0 || seq >= (uint32_t)num_seqs) return;
    const int block = pos / tokens_per_page;
    if (block >= max_pages_per_seq) return;
    const long long pg = page_table[(long long)seq * max_pages_per_seq + block];
    if (pg >= num_pages) return;
    page = pg;
    slot = pos - block * tokens_per_page;
  }
}

template <bool kSlots>
__global__ void __launch_bounds__(256) fill_kv_pages_grouped_kernel(
    const uint4* __restrict__ new_keys, const uint4* __restrict__ new_values, uint16_t* __restrict__ k_pool,
    uint16_t* __restrict__ v_pool, const int64_t* __restrict__ slot_mapping, const uint32_t* __restrict__ page_table,
    const int32_t* __restrict__ write_positions, const uint32_t* __restrict__ query_to_seq_map, long long num_tokens,
    int num_seqs, int num_kv_heads, int head_dim, int tokens_per_page, long long num_pages, int max_pages_per_seq,
    int parts) {
  extern __shared__ __align__(16) unsigned char fill_smem[];
  __shared__ long long s_page[kGroupTokens];
  __shared__ int s_slot[kGroupTokens];
  __shared__ int s_chunk[kGroupTokens];  // tokens i..i+chunk-1 fill an aligned stretch of slots of one page
  __shared__ int s_any_wide;
  const int row_elems = num_kv_heads * head_dim;
  const int vec_per_token = row_elems >> 3;
  const int vec_per_head = head_dim >> 3;
  // A work item is a group of tokens x one of `parts` equal slices of the token row: smaller items, more CTAs per SM.
  const int part_vecs = vec_per_token / parts;
  const int pitch = part_vecs * 16 + 16;  // bytes; the 16-byte skew keeps the transposed reads off one bank group
  unsigned char* sK = fill_smem;
  unsigned char* sV = fill_smem + kGroupTokens * pitch;
  const long long num_groups = (num_tokens + kGroupTokens - 1) / kGroupTokens;

  for (long long item = blockIdx.x; item < num_groups * parts; item += gridDim.x) {
    const long long grp = item / parts;
    const int vec0 = (int)(item - grp * parts) * part_vecs;  // first 16-byte vector of this slice within a token row
    const long long t0 = grp * kGroupTokens;
    const int ntok = (int)min((long long)kGroupTokens, num_tokens - t0);
    __syncthreads();  // the previous group's shared data is no longer needed
    // The token rows do not depend on where they go: their staging copies (coalesced 16-byte asynchronous copies, all
    // in flight at once) are issued first, and the destinations are looked up while they travel.
    for (int v = threadIdx.x; v < ntok * part_vecs; v += blockDim.x) {
      const int i = v / part_vecs, in_part = v - i * part_vecs;
      cp_async_16(sK + i * pitch + in_part * 16, new_keys + (t0 + i) * vec_per_token + vec0 + in_part);
      cp_async_16(sV + i * pitch + in_part * 16, new_values + (t0 + i) * vec_per_token + vec0 + in_part);
    }
    if (threadIdx.x < kGroupTokens) {
      long long page = -1;
      int slot = 0;
      if ((int)threadIdx.x < ntok)
        token_destination<kSlots>(t0 + threadIdx.x, slot_mapping, page_table, write_positions, query_to_seq_map, num_seqs,
                                  tokens_per_page, num_pages, max_pages_per_seq, page, slot);
      s_page[threadIdx.x] = page;
      s_slot[threadIdx.x] = slot;
    }
    if (threadIdx.x == 0) s_any_wide = 0;
    __syncthreads();
    if (threadIdx.x < kGroupTokens) {
      // largest power-of-two chunk (8, 4, 2, 1 tokens) that starts at token i, stays in one page on consecutive
      // slots and whose first slot is a multiple of its size: V stores of 16, 8, 4 or 2 bytes
      const int i = threadIdx.x;
      int run = 0;
      if (i < ntok && s_page[i] >= 0) {
        run = 1;
        while (run < 8 && i + run < ntok && s_page[i + run] == s_page[i] && s_slot[i + run] == s_slot[i] + run) ++run;
      }
      int chunk = 0;  // 0 = nothing to write for this token
      if (run >= 1) chunk = 1;
      if (run >= 2 && (s_slot[i] & 1) == 0) chunk = 2;
      if (run >= 4 && (s_slot[i] & 3) == 0) chunk = 4;
      if (run >= 8 && (s_slot[i] & 7) == 0) chunk = 8;
      s_chunk[i] = chunk;
      if (chunk > 1) s_any_wide = 1;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();

    if (!s_any_wide) {
      // scattered path for this group (same stores as fill_kv_pages_kernel, fed from the staged rows)
      for (int v = threadIdx.x; v < ntok * part_vecs; v += blockDim.x) {
        const int i = v / part_vecs, in_part = v - i * part_vecs, in_token = vec0 + in_part;
        const long long page = s_page[i];
        if (page < 0) continue;
        const int h = in_token / vec_per_head, c = in_token - h * vec_per_head, slot = s_slot[i];
        const uint4 kv = *reinterpret_cast<const uint4*>(sK + i * pitch + in_part * 16);
        const uint4 vv = *reinterpret_cast<const uint4*>(sV + i * pitch + in_part * 16);
        const long long head_base = (page * num_kv_heads + h) * (long long)head_dim * tokens_per_page;
        *reinterpret_cast<uint4*>(k_pool + head_base + ((long long)c * tokens_per_page + slot) * 8) = kv;
        uint16_t* vp = v_pool + head_base + (long long)c * 8 * tokens_per_page + slot;
        const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          vp[(2 * j) * tokens_per_page] = (uint16_t)(w[j] & 0xffffu);
          vp[(2 * j + 1) * tokens_per_page] = (uint16_t)(w[j] >> 16);
        }
      }
      continue;
    }

    // K: consecutive threads take consecutive tokens of one (head, chunk): 16-byte stores that are contiguous
    // in the pool wherever the slots are
    for (int u = threadIdx.x; u < part_vecs * kGroupTokens; u += blockDim.x) {
      const int i = u & (kGroupTokens - 1), in_part = u >> 4, in_token = vec0 + in_part;
      if (i >= ntok) continue;
      const long long page = s_page[i];
      if (page < 0) continue;
      const int h = in_token / vec_per_head, c = in_token - h * vec_per_head;
      const long long head_base = (page * num_kv_heads + h) * (long long)head_dim * tokens_per_page;
      *reinterpret_cast<uint4*>(k_pool + head_base + ((long long)c * tokens_per_page + s_slot[i]) * 8) =
          *reinterpret_cast<const uint4*>(sK + i * pitch + in_part * 16);
    }
    // V: one thread per (head, d) row; a chunk of 8, 4 or 2 tokens becomes one 16-, 8- or 4-byte store
    for (int el = threadIdx.x; el < part_vecs * 8; el += blockDim.x) {
      const int e = vec0 * 8 + el;
      const int h = e / head_dim, d = e - h * head_dim;
      const unsigned char* col = sV + el * 2;
      int i = 0;
      while (i < ntok) {
        const int chunk = s_chunk[i];
        if (chunk == 0) {
          ++i;
          continue;
        }
        uint16_t* dst = v_pool + ((s_page[i] * num_kv_heads + h) * (long long)head_dim + d) * tokens_per_page + s_slot[i];
        const unsigned char* src = col + i * pitch;
        auto pair = [&](int k) {
          return (uint32_t) * reinterpret_cast<const uint16_t*>(src + k * pitch) |
                 ((uint32_t) * reinterpret_cast<const uint16_t*>(src + (k + 1) * pitch) << 16);
        };
        if (chunk == 8)
          *reinterpret_cast<uint4*>(dst) = make_uint4(pair(0), pair(2), pair(4), pair(6));
        else if (chunk == 4)
          *reinterpret_cast<uint2*>(dst) = make_uint2(pair(0), pair(2));
        else if (chunk == 2)
          *reinterpret_cast<uint32_t*>(dst) = pair(0);
        else
          *dst = *reinterpret_cast<const uint16_t*>(src);
        i += chunk;
      }
    }
  }
}

int launch_fill(const FillArgs& a, cudaStream_t stream) {
  const long long total_vecs = a.num_tokens * a.num_kv_heads * (a.head_dim / 8);
  if (total_vecs == 0) return 0;
  // Enough tokens for runs to exist and rows that fit shared memory: the grouped kernel (it falls back
  // to scattered stores group by group).  V's 16-byte stores need TPP to be a multiple of 8.
  // The token row is cut into `parts` slices so that one work item stages about 32 KiB (several CTAs per SM).
  const int vec_per_token = a.num_kv_heads * a.head_dim / 8;
  int parts = 1;
  while (parts < 8 && vec_per_token % (parts * 2) == 0 && vec_per_token / parts > 64) parts *= 2;
  const size_t grouped_smem = 2 * (size_t)kGroupTokens * ((size_t)(vec_per_token / parts) * 16 + 16);
  // Below a few hundred tokens (a decode step appends one token per sequence) the call is latency-bound and the
  // scattered kernel, with its single dependent load per thread, finishes sooner.
  if (a.num_tokens >= 256 && a.tokens_per_page % 8 == 0 && grouped_smem <= 160 * 1024) {
    long long groups = (a.num_tokens + kGroupTokens - 1) / kGroupTokens * parts;
    const long long max_groups = 148LL * 32;
    if (groups > max_groups) groups = max_groups;
    static DeviceOnce configured;
    const int rc = configured.run([] {
      cudaError_t e = cudaFuncSetAttribute(fill_kv_pages_grouped_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(fill_kv_pages_grouped_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
      return (int)e;
    });
    if (rc != 0) return rc;
    if (a.slot_mapping)
      fill_kv_pages_grouped_kernel<true><<<(unsigned)groups, 256, grouped_smem, stream>>>(
          (const uint4*)a.new_keys, (const uint4*)a.new_values, (uint16_t*)a.k_pool, (uint16_t*)a.v_pool,
          a.slot_mapping, nullptr, nullptr, nullptr, a.num_tokens, a.num_seqs, a.num_kv_heads, a.head_dim,
          a.tokens_per_page, a.num_pages, a.max_pages_per_seq, parts);
    else
      fill_kv_pages_grouped_kernel<false><<<(unsigned)groups, 256, grouped_smem, stream>>>(
          (const uint4*)a.new_keys, (const uint4*)a.new_values, (uint16_t*)a.k_pool, (uint16_t*)a.v_pool, nullptr,
          (const uint32_t*)a.page_table, a.write_positions, (const uint32_t*)a.query_to_seq_map, a.num_tokens,
          a.num_seqs, a.num_kv_heads, a.head_dim, a.tokens_per_page, a.num_pages, a.max_pages_per_seq, parts);
    return (int)cudaGetLastError();
  }
  long long blocks = (total_vecs + 255) / 256;
  const long long max_blocks = 148LL * 8 * 4;
  if (blocks > max_blocks) blocks = max_blocks;
  if (a.slot_mapping) {
    fill_kv_pages_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(
        (const uint4*)a.new_keys, (const uint4*)a.new_values, (uint16_t*)a.k_pool, (uint16_t*)a.v_pool,
        a.slot_mapping, nullptr, nullptr, nullptr, a.num_tokens, a.num_seqs, a.num_kv_heads, a.head_dim,
        a.tokens_per_page, a.num_pages, a.max_pages_per_seq);
  } else {
    fill_kv_pages_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(
        (const uint4*)a.new_keys, (const uint4*)a.new_values, (uint16_t*)a.k_pool, (uint16_t*)a.v_pool, nullptr,
        (const uint32_t*)a.page_table, a.write_positions, (const uint32_t*)a.query_to_seq_map, a.num_tokens,
        a.num_seqs, a.num_kv_heads, a.head_dim, a.tokens_per_page, a.num_pages, a.max_pages_per_seq);
  }
  return (int)cudaGetLastError();
}

}  // namespace pal
