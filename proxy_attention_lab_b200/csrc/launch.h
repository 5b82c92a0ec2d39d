// Host-side argument blocks shared by the C-ABI translation unit and the kernel files.
//
// These play the role of PagedAttentionParams / FillKVPagesParams in the reference
// (src/pal_core/include/kernels/paged_attention_types.h:50-60,84-92), widened with the pointers
// the CUDA launchers need.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace pal {

struct FillArgs {
  const void* new_keys;
  const void* new_values;
  void* k_pool;
  void* v_pool;
  const int64_t* slot_mapping;  // either this ...
  const void* page_table;       // ... or these three
  const int32_t* write_positions;
  const void* query_to_seq_map;
  long long num_tokens;
  int num_seqs;
  int num_kv_heads;
  int head_dim;
  int tokens_per_page;
  long long num_pages;
  int max_pages_per_seq;
};

struct DecodeArgs {
  const void* queries;
  const void* k_pool;
  const void* v_pool;
  const void* new_keys = nullptr;    // both set = append form: the pools are written as well (see decode.cu)
  const void* new_values = nullptr;
  const uint32_t* page_table;
  const int32_t* sequence_lengths;
  void* out;            // [S, Hq, D] in the query dtype (null when only the triple is wanted)
  float* m_out;         // optional un-normalised triple [S, Hq], [S, Hq], [S, Hq, D]
  float* l_out;
  float* acc_out;
  int num_seqs;
  int num_q_heads;
  int num_kv_heads;
  int head_dim;
  int tokens_per_page;
  long long num_pages;
  int max_pages_per_seq;
  float scale;
  int dtype;
  int partition_pages;  // 0 = fused single pass, > 0 = two-pass
  void* workspace;
  size_t workspace_bytes;
};

struct PrefillArgs {
  const void* q_prompt;
  const void* k_prompt;
  const void* v_prompt;
  const void* k_pool;
  const void* v_pool;
  const uint32_t* page_table;
  const int32_t* history_lens;
  const int32_t* cu_seqlens = nullptr;  // ragged form: [S + 1] row offsets; tokens_per_seq is then the longest sequence
  long long total_tokens = 0;           // ragged form: rows of q_prompt / k_prompt / v_prompt
  void* out;
  int num_seqs;
  int tokens_per_seq;
  int num_q_heads;
  int num_kv_heads;
  int head_dim;
  int tokens_per_page;
  long long num_pages;
  int max_pages_per_seq;
  float scale;
  int dtype;
  int impl;
  void* workspace;
  size_t workspace_bytes;
};

// Each returns a cudaError_t value as int (0 = success) or a negative PAL_ERR_* code, and
// leaves a message via set_error() on failure.
int launch_fill(const FillArgs& a, cudaStream_t stream);
int launch_decode(const DecodeArgs& a, cudaStream_t stream);
int launch_lse_combine(const float* m, const float* l, const float* acc, void* out, float* m_out, float* l_out,
                       float* acc_out, int num_parts, long long rows, int head_dim, int dtype, long long part_stride_ml,
                       long long row_stride_ml, long long part_stride_acc, long long row_stride_acc,
                       cudaStream_t stream);
int launch_prefill_mma(const PrefillArgs& a, cudaStream_t stream);
int launch_prefill_tcgen05(const PrefillArgs& a, cudaStream_t stream);

size_t decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                              int max_pages_per_seq, int partition_pages);
int decode_num_partitions(int max_pages_per_seq, int partition_pages);
int decode_auto_partition_pages(int num_seqs, int num_q_heads, int num_kv_heads, int max_pages_per_seq);

void set_error(const char* fmt, ...);

}  // namespace pal
