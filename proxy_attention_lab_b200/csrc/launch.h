// Host-side argument blocks shared by the C-ABI translation unit and the kernel files.
//
// These play the role of PagedAttentionParams / FillKVPagesParams in the reference
// (src/pal_core/include/kernels/paged_attention_types.h:50-60,84-92), widened with the pointers
// the CUDA launchers need.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <mutex>

namespace pal {

constexpr int kMaxDevices = 64;

// One-time, per-device set-up (kernel attributes, device properties) that any host thread may trigger:
// the first caller on a device runs `fn` under a lock, later callers see the flag and skip it.
class DeviceOnce {
 public:
  // fn() returns a cudaError_t as int; a failure is returned and the set-up is retried by the next call.
  template <typename F>
  int run(F&& fn) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return fn();
    if (done_[dev].load(std::memory_order_acquire)) return 0;
    std::lock_guard<std::mutex> lock(mu_);
    if (done_[dev].load(std::memory_order_relaxed)) return 0;
    const int rc = fn();
    if (rc == 0) done_[dev].store(true, std::memory_order_release);
    return rc;
  }

 private:
  std::mutex mu_;
  std::atomic<bool> done_[kMaxDevices] = {};
};

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
  void* out;            // [S, Hq, D] in the query dtype or float32 (null when only the triple is wanted)
  bool out_f32 = false;
  float* m_out;         // optional un-normalised triple [S, Hq], [S, Hq], [S, Hq, D]
  float* l_out;
  float* acc_out;
  float* packed_out = nullptr;  // or the same triple as one [S*Hq, D + 2] buffer: acc, then m, then l
  bool skip_combine = false;    // two-pass only: leave the per-partition partials in the workspace (see decode_partials_view)
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
  bool out_f32 = false;
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
// Strided views of a set of partial triples (element strides): partition j of row r has its m / l at
// m[j * part_stride_ml + r * row_stride_ml] and its acc row at acc + j * part_stride_acc + r * row_stride_acc.
struct PartialsView {
  const float* m;
  const float* l;
  const float* acc;
  long long part_stride_ml, row_stride_ml, part_stride_acc, row_stride_acc;
};
// Where a merged, still un-normalised triple goes (all optional): row r's acc at acc + r * row_stride_acc, its m / l at
// m[r * row_stride_ml].
struct TripleOut {
  float* m = nullptr;
  float* l = nullptr;
  float* acc = nullptr;
  long long row_stride_ml = 1, row_stride_acc = 0;
};
// The per-partition partials a two-pass launch_decode leaves in `workspace` for this problem, and their count per row.
PartialsView decode_partials_view(const DecodeArgs& a, int* num_parts);
int launch_lse_combine(const PartialsView& in, void* out, bool out_f32, const TripleOut& triple, int num_parts,
                       long long rows, int head_dim, int dtype, cudaStream_t stream);
// Context-sharded decode, second half: merge this GPU's partitions, store the merged triple into every peer's exchange
// buffer, wait (bounded) for all peers' triples and merge them into `out`.  `peer_bases[r]` is rank r's exchange buffer as
// mapped into this process (see decode_exchange.cu for its layout).
struct ExchangeArgs {
  PartialsView in;
  int num_parts;
  long long rows;
  int head_dim;
  void* out;
  bool out_f32;
  int dtype;
  int world_size, rank;
  long long rows_capacity;
  const void* const* peer_bases;
  void* workspace;  // its status word receives a timeout
};
size_t exchange_bytes(int world_size, long long rows_capacity, int head_dim);
int launch_exchange_combine(const ExchangeArgs& a, cudaStream_t stream);
int launch_prefill_mma(const PrefillArgs& a, cudaStream_t stream);
int launch_prefill_tcgen05(const PrefillArgs& a, cudaStream_t stream);
bool prefill_tcgen05_supports(int head_dim, int tokens_per_page);
// Parts into which the tcgen05 prefill kernel would cut the history of this batch (1 = not at all), and the workspace
// that takes: a function of the shape alone, so that the size can be asked for before the page table exists.
int prefill_split_parts(int num_seqs, int tokens_per_seq, int num_q_heads, int num_kv_heads, int head_dim);
size_t prefill_workspace_bytes(int num_seqs, int tokens_per_seq, int num_q_heads, int num_kv_heads, int head_dim);
bool prefill_tcgen05_pair_supports(int head_dim, int tokens_per_page, int num_q_heads, int num_kv_heads);

size_t decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                              int max_pages_per_seq, int partition_pages);
int decode_num_partitions(int max_pages_per_seq, int partition_pages);
int decode_auto_partition_pages(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                int max_pages_per_seq);

void set_error(const char* fmt, ...);
// cudaError_t (as int) or negative PAL_ERR_* -> PAL_* return code, with the message set
int cuda_rc(int rc, const char* what);

// Limit, in SM clock cycles, of every bounded device-side wait of the launches that follow (process-wide).
long long wait_limit_cycles();
int cached_sm_count();

}  // namespace pal
