// fill_kv_pages for sm_100a: scatter new K/V tokens [T, Hkv, D] into the striped-K /
// transposed-V page pools, in place and bit-exact.
//
// Replaces fill_kv_pages_kernel (src/pal_core/kernels/paged_attention/fill_kv_pages.h.metal:30-121)
// and its launcher (src/pal_core/src/fill_kv_pages_primitive.cpp:70-170).  Unlike the reference
// launcher, the pools are not copied first.
//
// One thread moves one 16-byte vector (8 elements) of one token's K and of its V:
//   K[page, h, d/8, slot, 0..7] <- new_keys[t, h, d..d+7]        one 16-byte store
//   V[page, h, d+j, slot]       <- new_values[t, h, d+j], j<8    eight 2-byte stores, TPP apart
// The V stores cannot be widened for a single token: consecutive d are TPP elements apart in the
// pool, so each element lives in its own 32-byte sector.  Loads of the source are fully coalesced.
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

int launch_fill(const FillArgs& a, cudaStream_t stream) {
  const long long total_vecs = a.num_tokens * a.num_kv_heads * (a.head_dim / 8);
  if (total_vecs == 0) return 0;
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
