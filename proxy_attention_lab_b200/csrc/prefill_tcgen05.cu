// Dispatch of the tcgen05 prefill kernel over its instantiations (head_dim 32 / 64 / 80 / 96 / 128 / 256 x tokens_per_page 16 / 32);
// the kernel itself is in prefill_tcgen05.cuh, one translation unit per shape.
#include "common.cuh"
#include "launch.h"

namespace pal {

#define PAL_TC_SHAPES(X) X(32, 16) X(32, 32) X(64, 16) X(64, 32) X(80, 16) X(80, 32) X(96, 16) X(96, 32) X(128, 16) X(128, 32) X(256, 16) X(256, 32)
#define PAL_TC_DECLARE(DD, TT) int launch_prefill_tcgen05_d##DD##_t##TT(const PrefillArgs& a, cudaStream_t stream);
PAL_TC_SHAPES(PAL_TC_DECLARE)
#undef PAL_TC_DECLARE

bool prefill_tcgen05_supports(int head_dim, int tokens_per_page) {
#define PAL_TC_TEST(DD, TT) \
  if (head_dim == DD && tokens_per_page == TT) return true;
  PAL_TC_SHAPES(PAL_TC_TEST)
#undef PAL_TC_TEST
  return false;
}

int prefill_split_parts(int num_seqs, int tokens_per_seq, int num_q_heads, int num_kv_heads, int head_dim) {
  if (head_dim == 256 || num_seqs <= 0 || tokens_per_seq <= 0 || num_q_heads <= 0 || num_kv_heads <= 0) return 1;  // 256: the two-CTA kernel
  const long long qt = (tokens_per_seq + 127) / 128;
  const int group = num_q_heads / num_kv_heads;
  // CTAs of the unsplit launch: two heads of a kv head per CTA, or (odd groups) two query tiles of one head, or one tile
  const long long ctas = group % 2 == 0 ? (long long)num_seqs * qt * (num_q_heads / 2)
                                        : (tokens_per_seq > 128 ? (long long)num_seqs * ((qt + 1) / 2) * num_q_heads : (long long)num_seqs * num_q_heads);
  // Cutting pays while all parts still run at once: every CTA carries ~9 us of fixed cost, so a second wave of smaller
  // CTAs is slower than one wave of whole ones (measured: 8 sequences x 16 tokens over 2048, 128 CTAs: 45 us whole, 68 us in
  // three parts).
  constexpr long long kSms = 148;
  if (2 * ctas > kSms) return 1;
  long long parts = kSms / ctas;
  if (parts > 16) parts = 16;
  const long long rows = (long long)num_seqs * tokens_per_seq * num_q_heads;
  while (parts > 1 && rows * parts * (head_dim + 2) * 4 > (32ll << 20)) --parts;  // partial triples: at most 32 MB
  return parts < 2 ? 1 : (int)parts;
}

size_t prefill_workspace_bytes(int num_seqs, int tokens_per_seq, int num_q_heads, int num_kv_heads, int head_dim) {
  const int parts = prefill_split_parts(num_seqs, tokens_per_seq, num_q_heads, num_kv_heads, head_dim);
  if (parts < 2) return sizeof(WorkspaceHeader);
  return sizeof(WorkspaceHeader) + (size_t)num_seqs * tokens_per_seq * num_q_heads * parts * (head_dim + 2) * sizeof(float);
}

// The two-CTA form (prefill_tcgen05_pair.cuh): head_dim 128 / 256, an even number of query heads per kv head.
int launch_prefill_tcgen05_pair_d128(const PrefillArgs& a, cudaStream_t stream);
int launch_prefill_tcgen05_pair_d256(const PrefillArgs& a, cudaStream_t stream);

bool prefill_tcgen05_pair_supports(int head_dim, int tokens_per_page, int num_q_heads, int num_kv_heads) {
  if (!(head_dim == 128 || head_dim == 256) || !(tokens_per_page == 16 || tokens_per_page == 32) || num_kv_heads <= 0 ||
      num_q_heads % num_kv_heads != 0)
    return false;
  // head_dim 256 also pairs two query tiles of one head, which serves odd numbers of query heads per kv head
  return head_dim == 256 || (num_q_heads / num_kv_heads) % 2 == 0;
}

int launch_prefill_tcgen05(const PrefillArgs& a, cudaStream_t stream) {
  const bool pair_ok = prefill_tcgen05_pair_supports(a.head_dim, a.tokens_per_page, a.num_q_heads, a.num_kv_heads);
  // impl 4 asks for the two-CTA form; head_dim 256 takes it by default (impl 3 keeps the one-CTA kernel)
  if (a.impl == 4 && !pair_ok) {
    set_error("paged_attention_prefill: the two-CTA tcgen05 kernel covers head_dim 256, and head_dim 128 with an even number of query heads per kv head (tokens_per_page 16 / 32)");
    return -2;
  }
  // (odd groups with a single query tile per sequence gain nothing from pairing query tiles: the one-CTA kernel keeps them)
  const bool odd_single_tile = (a.num_q_heads / a.num_kv_heads) % 2 != 0 && a.tokens_per_seq <= 128;
  if (pair_ok && (a.impl == 4 || (a.head_dim == 256 && a.impl != 3 && !odd_single_tile)))
    return a.head_dim == 128 ? launch_prefill_tcgen05_pair_d128(a, stream) : launch_prefill_tcgen05_pair_d256(a, stream);
#define PAL_TC_CALL(DD, TT) \
  if (a.head_dim == DD && a.tokens_per_page == TT) return launch_prefill_tcgen05_d##DD##_t##TT(a, stream);
  PAL_TC_SHAPES(PAL_TC_CALL)
#undef PAL_TC_CALL
  set_error("paged_attention_prefill: the tcgen05 kernel covers head_dim in {32, 64, 80, 96, 128, 256} with tokens_per_page in {16, 32}");
  return -2;
}

}  // namespace pal
