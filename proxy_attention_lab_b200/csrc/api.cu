// C ABI of the library: argument validation, error strings, and dispatch to the launchers.
//
// Stands where the reference has its nanobind module and op builders
// (src/pal_core/bindings.cpp:40-222, src/pal_core/src/ops.cpp:36-239): shape rules are checked
// here, before any launch, and failures come back as an error code plus a thread-local message
// instead of a C++ exception.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>

#include "../../include/pal_b200.h"
#include "common.cuh"
#include "launch.h"

namespace pal {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_wait_limit{kDefaultWaitLimitCycles};

long long wait_limit_cycles() { return g_wait_limit.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int cuda_rc(int rc, const char* what) {
  if (rc == 0) return PAL_OK;
  if (rc < 0) return rc;  // already a PAL_ERR_* with a message
  if (rc == (int)cudaErrorMemoryAllocation) {
    set_error("%s: out of device memory (%s)", what, cudaGetErrorString((cudaError_t)rc));
    return PAL_ERR_WORKSPACE;
  }
  set_error("%s: CUDA error %d (%s)", what, rc, cudaGetErrorString((cudaError_t)rc));
  return PAL_ERR_LAUNCH;
}

static bool check_dtype(int dtype, const char* what) {
  if (dtype == PAL_DTYPE_F16 || dtype == PAL_DTYPE_BF16) return true;
  set_error("%s: dtype %d is not supported (0 = float16, 1 = bfloat16)", what, dtype);
  return false;
}

// The attention entry points take the element type with PAL_OUT_F32 optionally OR'ed in.
static bool split_dtype(int dtype_arg, const char* what, int* dtype, bool* out_f32) {
  *out_f32 = (dtype_arg & PAL_OUT_F32) != 0;
  *dtype = dtype_arg & ~PAL_OUT_F32;
  return check_dtype(*dtype, what);
}

// One CTA that waits on an mbarrier nobody ever arrives at: the wait runs into its limit, records the
// timeout in the workspace status word and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(WorkspaceHeader* hdr, long long limit_cycles) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
    const WaitCtx ctx{&hdr->status, limit_cycles};
    mbar_wait(&bar, 0, ctx);
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_heads(const char* what, int hq, int hkv, int d, int tpp) {
  if (hq <= 0 || hkv <= 0 || d <= 0 || tpp <= 0) {
    set_error("%s: head counts, head_dim and tokens_per_page must be positive", what);
    return PAL_ERR_BAD_ARG;
  }
  // src/pal_core/src/paged_attention_decode_primitive.cpp:156-159
  if (hq % hkv != 0) {
    set_error("%s: num_q_heads (%d) must be a multiple of num_kv_heads (%d)", what, hq, hkv);
    return PAL_ERR_BAD_ARG;
  }
  return PAL_OK;
}

}  // namespace pal

using namespace pal;

extern "C" {

const char* pal_last_error(void) { return g_error; }
const char* pal_version(void) { return "pal_b200 0.1.0 (sm_100a)"; }

int pal_get_k_cache_stripe_size(int dtype) {
  if (!check_dtype(dtype, "get_k_cache_stripe_size")) return PAL_ERR_UNSUPPORTED;
  return 16 / 2;
}

int pal_get_optimal_page_size(void) { return 16; }

int pal_get_k_cache_shape(int64_t num_pages, int num_kv_heads, int head_dim, int tokens_per_page, int dtype,
                          int64_t shape_out[5]) {
  if (!check_dtype(dtype, "get_k_cache_shape")) return PAL_ERR_UNSUPPORTED;
  if (!shape_out) {
    set_error("get_k_cache_shape: shape_out is null");
    return PAL_ERR_BAD_ARG;
  }
  const int x = 8;
  shape_out[0] = num_pages;
  shape_out[1] = num_kv_heads;
  shape_out[2] = head_dim / x;
  shape_out[3] = tokens_per_page;
  shape_out[4] = x;
  return PAL_OK;
}

int pal_get_v_cache_shape(int64_t num_pages, int num_kv_heads, int head_dim, int tokens_per_page, int dtype,
                          int64_t shape_out[4]) {
  if (!check_dtype(dtype, "get_v_cache_shape")) return PAL_ERR_UNSUPPORTED;
  if (!shape_out) {
    set_error("get_v_cache_shape: shape_out is null");
    return PAL_ERR_BAD_ARG;
  }
  shape_out[0] = num_pages;
  shape_out[1] = num_kv_heads;
  shape_out[2] = head_dim;
  shape_out[3] = tokens_per_page;
  return PAL_OK;
}

static int fill_common(FillArgs& a, int dtype, void* stream) {
  if (!check_dtype(dtype, "fill_kv_pages")) return PAL_ERR_UNSUPPORTED;
  if (a.num_tokens < 0 || a.num_pages < 0) {
    set_error("fill_kv_pages: negative token or page count");
    return PAL_ERR_BAD_ARG;
  }
  if (a.num_tokens == 0) return PAL_OK;  // src/pal_core/src/fill_kv_pages_primitive.cpp:94-96
  if (a.num_kv_heads <= 0 || a.head_dim <= 0 || a.tokens_per_page <= 0) {
    set_error("fill_kv_pages: num_kv_heads, head_dim and tokens_per_page must be positive");
    return PAL_ERR_BAD_ARG;
  }
  // src/pal_core/kernels/paged_attention/fill_kv_pages.h.metal:53,88-94 (16-byte vectors)
  if (a.head_dim % 8 != 0) {
    set_error("fill_kv_pages: head_dim (%d) must be a multiple of 8", a.head_dim);
    return PAL_ERR_UNSUPPORTED;
  }
  if (!a.new_keys || !a.new_values || !a.k_pool || !a.v_pool) {
    set_error("fill_kv_pages: null data pointer");
    return PAL_ERR_BAD_ARG;
  }
  if (!aligned16(a.new_keys) || !aligned16(a.new_values) || !aligned16(a.k_pool) || !aligned16(a.v_pool)) {
    set_error("fill_kv_pages: data pointers must be 16-byte aligned");
    return PAL_ERR_BAD_ARG;
  }
  return cuda_rc(launch_fill(a, (cudaStream_t)stream), "fill_kv_pages");
}

int pal_fill_kv_pages(const void* new_keys, const void* new_values, void* k_pool, void* v_pool,
                      const void* page_table, const int32_t* write_positions, const void* query_to_seq_map,
                      int64_t num_tokens, int num_seqs, int num_kv_heads, int head_dim, int tokens_per_page,
                      int64_t num_pages, int max_pages_per_seq, int dtype, void* stream) {
  FillArgs a{};
  a.new_keys = new_keys;
  a.new_values = new_values;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.slot_mapping = nullptr;
  a.page_table = page_table;
  a.write_positions = write_positions;
  a.query_to_seq_map = query_to_seq_map;
  a.num_tokens = num_tokens;
  a.num_seqs = num_seqs;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  if (num_tokens > 0 && (!page_table || !write_positions || !query_to_seq_map)) {
    set_error("fill_kv_pages: page_table, write_positions and query_to_seq_map are required");
    return PAL_ERR_BAD_ARG;
  }
  return fill_common(a, dtype, stream);
}

int pal_fill_kv_pages_slots(const void* new_keys, const void* new_values, void* k_pool, void* v_pool,
                            const int64_t* slot_mapping, int64_t num_tokens, int num_kv_heads, int head_dim,
                            int tokens_per_page, int64_t num_pages, int dtype, void* stream) {
  FillArgs a{};
  a.new_keys = new_keys;
  a.new_values = new_values;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.slot_mapping = slot_mapping;
  a.num_tokens = num_tokens;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  if (num_tokens > 0 && !slot_mapping) {
    set_error("fill_kv_pages: slot_mapping is null");
    return PAL_ERR_BAD_ARG;
  }
  return fill_common(a, dtype, stream);
}

size_t pal_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                  int tokens_per_page, int max_pages_per_seq, int partition_pages) {
  if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return sizeof(WorkspaceHeader);
  return decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim, tokens_per_page, max_pages_per_seq,
                                partition_pages);
}

int pal_decode_auto_partition_pages(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                    int max_pages_per_seq) {
  if (num_seqs <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || tokens_per_page <= 0 || max_pages_per_seq <= 0)
    return 0;
  return decode_auto_partition_pages(num_seqs, num_q_heads, num_kv_heads, head_dim, tokens_per_page, max_pages_per_seq);
}

static int decode_common(DecodeArgs& a, void* stream, const char* what) {
  if (!split_dtype(a.dtype, what, &a.dtype, &a.out_f32)) return PAL_ERR_UNSUPPORTED;
  int rc = check_heads(what, a.num_q_heads, a.num_kv_heads, a.head_dim, a.tokens_per_page);
  if (rc != PAL_OK) return rc;
  if (a.num_seqs < 0 || a.num_pages < 0 || a.max_pages_per_seq < 0) {
    set_error("%s: negative size", what);
    return PAL_ERR_BAD_ARG;
  }
  if (a.num_seqs == 0) return PAL_OK;
  if (!a.queries || !a.sequence_lengths || (a.num_pages > 0 && (!a.k_pool || !a.v_pool)) ||
      (a.max_pages_per_seq > 0 && !a.page_table)) {
    set_error("%s: null input pointer", what);
    return PAL_ERR_BAD_ARG;
  }
  if (!aligned16(a.k_pool) || !aligned16(a.v_pool) || (reinterpret_cast<uintptr_t>(a.queries) & 3)) {
    set_error("%s: pools must be 16-byte aligned and queries 4-byte aligned", what);
    return PAL_ERR_BAD_ARG;
  }
  if (a.partition_pages < 0)
    a.partition_pages =
        decode_auto_partition_pages(a.num_seqs, a.num_q_heads, a.num_kv_heads, a.head_dim, a.tokens_per_page, a.max_pages_per_seq);
  if (a.max_pages_per_seq == 0) a.partition_pages = (a.m_out || a.packed_out) ? 1 : 0;
  const size_t need = decode_workspace_bytes(a.num_seqs, a.num_q_heads, a.num_kv_heads, a.head_dim,
                                             a.tokens_per_page, a.max_pages_per_seq, a.partition_pages);
  if (!a.workspace || a.workspace_bytes < need || (reinterpret_cast<uintptr_t>(a.workspace) & 255)) {
    set_error("%s: workspace of %zu bytes (256-byte aligned) required, got %zu", what, need,
              a.workspace ? a.workspace_bytes : (size_t)0);
    return PAL_ERR_WORKSPACE;
  }
  if (!(a.scale > 0.f)) a.scale = 1.0f / sqrtf((float)a.head_dim);
  return cuda_rc(launch_decode(a, (cudaStream_t)stream), what);
}

int pal_paged_attention_decode(const void* queries, const void* k_pool, const void* v_pool,
                               const void* page_table, const int32_t* sequence_lengths, void* out, int num_seqs,
                               int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                               int64_t num_pages, int max_pages_per_seq, float scale, int dtype,
                               int partition_pages, void* workspace, size_t workspace_bytes, void* stream) {
  DecodeArgs a{};
  a.queries = queries;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.sequence_lengths = sequence_lengths;
  a.out = out;
  a.num_seqs = num_seqs;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale;
  a.dtype = dtype;
  a.partition_pages = partition_pages;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (num_seqs > 0 && !out) {
    set_error("paged_attention_decode: out is null");
    return PAL_ERR_BAD_ARG;
  }
  return decode_common(a, stream, "paged_attention_decode");
}

int pal_paged_attention_decode_append(const void* new_keys, const void* new_values, const void* queries, void* k_pool,
                                      void* v_pool, const void* page_table, const int32_t* sequence_lengths, void* out,
                                      int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                      int64_t num_pages, int max_pages_per_seq, float scale, int dtype,
                                      int partition_pages, void* workspace, size_t workspace_bytes, void* stream) {
  DecodeArgs a{};
  a.queries = queries;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.new_keys = new_keys;
  a.new_values = new_values;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.sequence_lengths = sequence_lengths;
  a.out = out;
  a.num_seqs = num_seqs;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale;
  a.dtype = dtype;
  a.partition_pages = partition_pages;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (num_seqs > 0 && (!out || !new_keys || !new_values)) {
    set_error("paged_attention_decode_append: out, new_keys or new_values is null");
    return PAL_ERR_BAD_ARG;
  }
  if (!aligned16(new_keys) || !aligned16(new_values)) {
    set_error("paged_attention_decode_append: new_keys and new_values must be 16-byte aligned");
    return PAL_ERR_BAD_ARG;
  }
  return decode_common(a, stream, "paged_attention_decode_append");
}

int pal_paged_attention_decode_partials(const void* queries, const void* k_pool, const void* v_pool,
                                        const void* page_table, const int32_t* sequence_lengths, float* m_out,
                                        float* l_out, float* acc_out, int num_seqs, int num_q_heads,
                                        int num_kv_heads, int head_dim, int tokens_per_page, int64_t num_pages,
                                        int max_pages_per_seq, float scale, int dtype, int partition_pages,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  DecodeArgs a{};
  a.queries = queries;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.sequence_lengths = sequence_lengths;
  a.out = nullptr;
  a.m_out = m_out;
  a.l_out = l_out;
  a.acc_out = acc_out;
  a.num_seqs = num_seqs;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale;
  a.dtype = dtype;
  a.partition_pages = partition_pages;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (partition_pages <= 0) {
    set_error("paged_attention_decode_partials: partition_pages must be > 0");
    return PAL_ERR_BAD_ARG;
  }
  if (num_seqs > 0 && (!m_out || !l_out || !acc_out)) {
    set_error("paged_attention_decode_partials: null output pointer");
    return PAL_ERR_BAD_ARG;
  }
  return decode_common(a, stream, "paged_attention_decode_partials");
}

int pal_paged_attention_decode_partials_packed(const void* queries, const void* k_pool, const void* v_pool,
                                               const void* page_table, const int32_t* sequence_lengths,
                                               float* packed_out, int num_seqs, int num_q_heads, int num_kv_heads,
                                               int head_dim, int tokens_per_page, int64_t num_pages,
                                               int max_pages_per_seq, float scale, int dtype, int partition_pages,
                                               void* workspace, size_t workspace_bytes, void* stream) {
  DecodeArgs a{};
  a.queries = queries;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.sequence_lengths = sequence_lengths;
  a.out = nullptr;
  a.packed_out = packed_out;
  a.num_seqs = num_seqs;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale;
  a.dtype = dtype;
  a.partition_pages = partition_pages;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (partition_pages <= 0) {
    set_error("paged_attention_decode_partials_packed: partition_pages must be > 0");
    return PAL_ERR_BAD_ARG;
  }
  if (num_seqs > 0 && !packed_out) {
    set_error("paged_attention_decode_partials_packed: null output pointer");
    return PAL_ERR_BAD_ARG;
  }
  return decode_common(a, stream, "paged_attention_decode_partials_packed");
}

size_t pal_exchange_bytes(int world_size, int64_t rows_capacity, int head_dim) {
  if (world_size < 1 || rows_capacity < 0 || head_dim <= 0) return 0;
  return exchange_bytes(world_size, rows_capacity, head_dim);
}

int pal_paged_attention_decode_ctx_exchange(const void* queries, const void* k_pool, const void* v_pool,
                                            const void* page_table, const int32_t* sequence_lengths, void* out,
                                            int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                            int tokens_per_page, int64_t num_pages, int max_pages_per_seq, float scale,
                                            int dtype, int partition_pages, void* workspace, size_t workspace_bytes,
                                            const void* const* peer_bases, int world_size, int rank,
                                            int64_t rows_capacity, void* stream) {
  const char* what = "paged_attention_decode_ctx_exchange";
  DecodeArgs a{};
  a.queries = queries;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.sequence_lengths = sequence_lengths;
  a.out = nullptr;
  a.skip_combine = true;
  a.num_seqs = num_seqs;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale;
  a.dtype = dtype;
  a.partition_pages = partition_pages;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  if (partition_pages <= 0) {
    set_error("%s: partition_pages must be > 0", what);
    return PAL_ERR_BAD_ARG;
  }
  if (num_seqs <= 0 || !out || !peer_bases) {
    // every rank has to take part in every step: an empty batch is an error here, not a no-op
    set_error("%s: num_seqs must be positive and out / peer_bases non-null", what);
    return PAL_ERR_BAD_ARG;
  }
  if (max_pages_per_seq <= 0) {
    set_error("%s: max_pages_per_seq must be positive (a rank without context passes lengths of 0)", what);
    return PAL_ERR_BAD_ARG;
  }
  int rc = decode_common(a, stream, what);  // split-KV pass over this GPU's slice; a.dtype / a.out_f32 are split there
  if (rc != PAL_OK) return rc;
  ExchangeArgs x{};
  x.in = decode_partials_view(a, &x.num_parts);
  x.rows = (long long)num_seqs * num_q_heads;
  x.head_dim = head_dim;
  x.out = out;
  x.out_f32 = a.out_f32;
  x.dtype = a.dtype;
  x.world_size = world_size;
  x.rank = rank;
  x.rows_capacity = rows_capacity;
  x.peer_bases = peer_bases;
  x.workspace = workspace;
  return cuda_rc(launch_exchange_combine(x, (cudaStream_t)stream), what);
}

static int combine_common(const char* what, const PartialsView& in, void* out, int num_parts, int64_t rows, int head_dim,
                          int dtype_arg, void* stream) {
  int dtype;
  bool out_f32;
  if (!split_dtype(dtype_arg, what, &dtype, &out_f32)) return PAL_ERR_UNSUPPORTED;
  if (num_parts <= 0 || rows < 0 || head_dim <= 0) {
    set_error("%s: num_parts and head_dim must be positive, rows non-negative", what);
    return PAL_ERR_BAD_ARG;
  }
  if (rows == 0) return PAL_OK;
  if (rows > 0x7fffffffLL) {
    set_error("%s: rows must be below 2^31", what);
    return PAL_ERR_BAD_ARG;
  }
  if (!in.m || !in.l || !in.acc || !out) {
    set_error("%s: null pointer", what);
    return PAL_ERR_BAD_ARG;
  }
  return cuda_rc(launch_lse_combine(in, out, out_f32, TripleOut{}, num_parts, rows, head_dim, dtype, (cudaStream_t)stream), what);
}

int pal_lse_combine(const float* m, const float* l, const float* acc, void* out, int num_parts, int64_t rows,
                    int head_dim, int dtype, void* stream) {
  const PartialsView in{m, l, acc, rows, 1, rows * head_dim, head_dim};
  return combine_common("lse_combine", in, out, num_parts, rows, head_dim, dtype, stream);
}

int pal_lse_combine_packed(const float* packed, void* out, int num_parts, int64_t rows, int head_dim, int dtype,
                           void* stream) {
  const long long pitch = head_dim + 2;
  const PartialsView in{packed ? packed + head_dim : nullptr, packed ? packed + head_dim + 1 : nullptr, packed,
                        rows * pitch, pitch, rows * pitch, pitch};
  return combine_common("lse_combine_packed", in, out, num_parts, rows, head_dim, dtype, stream);
}

// The prefill kernels keep everything in shared memory and TMEM: the workspace is only the 256-byte header with the
// status word, whatever the problem size (the arguments exist so that a later kernel may need more without an ABI change).
size_t pal_prefill_workspace_bytes(int num_seqs, int tokens_per_seq, int num_q_heads, int num_kv_heads,
                                   int head_dim) {
  return prefill_workspace_bytes(num_seqs, tokens_per_seq, num_q_heads, num_kv_heads, head_dim);
}

// tokens_per_seq is the uniform count, or with cu_seqlens (ragged form) the longest sequence's count
static int prefill_common(const char* what, const void* q_prompt, const void* k_prompt, const void* v_prompt,
                          const void* k_pool, const void* v_pool, const void* page_table, const int32_t* history_lens,
                          const int32_t* cu_seqlens, int64_t total_tokens, void* out, int num_seqs, int tokens_per_seq,
                          int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page, int64_t num_pages,
                          int max_pages_per_seq, float scale, int dtype_arg, int impl, void* workspace,
                          size_t workspace_bytes, void* stream) {
  int dtype;
  bool out_f32;
  if (!split_dtype(dtype_arg, what, &dtype, &out_f32)) return PAL_ERR_UNSUPPORTED;
  int rc = check_heads(what, num_q_heads, num_kv_heads, head_dim, tokens_per_page);
  if (rc != PAL_OK) return rc;
  if (num_seqs < 0 || tokens_per_seq < 0 || num_pages < 0 || max_pages_per_seq < 0) {
    set_error("%s: negative size", what);
    return PAL_ERR_BAD_ARG;
  }
  if (num_seqs == 0 || tokens_per_seq == 0) return PAL_OK;
  if (!q_prompt || !k_prompt || !v_prompt || !history_lens || !out) {
    set_error("%s: null pointer", what);
    return PAL_ERR_BAD_ARG;
  }
  if (!aligned16(q_prompt) || !aligned16(k_prompt) || !aligned16(v_prompt) || !aligned16(k_pool) ||
      !aligned16(v_pool) || !aligned16(out)) {
    set_error("%s: data pointers must be 16-byte aligned", what);
    return PAL_ERR_BAD_ARG;
  }
  if (!workspace || workspace_bytes < sizeof(WorkspaceHeader) || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("%s: workspace of %zu bytes (256-byte aligned) required", what, sizeof(WorkspaceHeader));
    return PAL_ERR_WORKSPACE;
  }
  PrefillArgs a{};
  a.q_prompt = q_prompt;
  a.k_prompt = k_prompt;
  a.v_prompt = v_prompt;
  a.k_pool = k_pool;
  a.v_pool = v_pool;
  a.page_table = static_cast<const uint32_t*>(page_table);
  a.history_lens = history_lens;
  a.cu_seqlens = cu_seqlens;
  a.total_tokens = total_tokens;
  a.out = out;
  a.out_f32 = out_f32;
  a.num_seqs = num_seqs;
  a.tokens_per_seq = tokens_per_seq;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.head_dim = head_dim;
  a.tokens_per_page = tokens_per_page;
  a.num_pages = num_pages;
  a.max_pages_per_seq = max_pages_per_seq;
  a.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)head_dim);
  a.dtype = dtype;
  a.impl = impl;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  const bool tc_ok = prefill_tcgen05_supports(head_dim, tokens_per_page);
  if (impl < 0 || impl > 4) {
    set_error("%s: impl must be 0 (auto), 1 (mma.sync), 2 (tcgen05), 3 (tcgen05, one accumulator tile per CTA) or 4 (tcgen05, two CTAs per MMA)", what);
    return PAL_ERR_BAD_ARG;
  }
  if (impl == 4 && !prefill_tcgen05_pair_supports(head_dim, tokens_per_page, num_q_heads, num_kv_heads)) {
    set_error("%s: the two-CTA tcgen05 kernel covers head_dim 256, and head_dim 128 with an even number of query heads per kv head (tokens_per_page 16 / 32)", what);
    return PAL_ERR_UNSUPPORTED;
  }
  if (impl >= 2 && !tc_ok) {
    set_error("%s: the tcgen05 kernel covers head_dim in {32, 64, 80, 96, 128, 256} with tokens_per_page in {16, 32}", what);
    return PAL_ERR_UNSUPPORTED;
  }
  // The tcgen05 kernels are the launcher's choice for every shape they cover, down to a single new token per sequence
  // (measured 2-6x faster than the mma.sync kernel from 1 to 63 new tokens per sequence; equal at the launch floor).
  const bool use_tc = impl >= 2 || (impl == 0 && tc_ok);
  return cuda_rc(use_tc ? launch_prefill_tcgen05(a, (cudaStream_t)stream) : launch_prefill_mma(a, (cudaStream_t)stream),
                 what);
}

int pal_paged_attention_prefill(const void* q_prompt, const void* k_prompt, const void* v_prompt,
                                const void* k_pool, const void* v_pool, const void* page_table,
                                const int32_t* history_lens, void* out, int num_seqs, int tokens_per_seq,
                                int num_q_heads, int num_kv_heads, int head_dim, int tokens_per_page,
                                int64_t num_pages, int max_pages_per_seq, float scale, int dtype, int impl,
                                void* workspace, size_t workspace_bytes, void* stream) {
  return prefill_common("paged_attention_prefill", q_prompt, k_prompt, v_prompt, k_pool, v_pool, page_table,
                        history_lens, nullptr, (int64_t)num_seqs * tokens_per_seq, out, num_seqs, tokens_per_seq,
                        num_q_heads, num_kv_heads, head_dim, tokens_per_page, num_pages, max_pages_per_seq, scale, dtype,
                        impl, workspace, workspace_bytes, stream);
}

int pal_paged_attention_prefill_ragged(const void* q_prompt, const void* k_prompt, const void* v_prompt,
                                       const void* k_pool, const void* v_pool, const void* page_table,
                                       const int32_t* history_lens, const int32_t* cu_seqlens, void* out,
                                       int num_seqs, int64_t total_tokens, int max_new_tokens, int num_q_heads,
                                       int num_kv_heads, int head_dim, int tokens_per_page, int64_t num_pages,
                                       int max_pages_per_seq, float scale, int dtype, int impl, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  const char* what = "paged_attention_prefill_ragged";
  if (total_tokens < 0 || total_tokens > 0x7fffffffLL) {
    set_error("%s: total_tokens must be in [0, 2^31)", what);
    return PAL_ERR_BAD_ARG;
  }
  if (num_seqs > 0 && total_tokens > 0 && max_new_tokens > 0 && !cu_seqlens) {
    set_error("%s: cu_seqlens is null", what);
    return PAL_ERR_BAD_ARG;
  }
  if (total_tokens == 0) return num_seqs < 0 ? PAL_ERR_BAD_ARG : PAL_OK;
  return prefill_common(what, q_prompt, k_prompt, v_prompt, k_pool, v_pool, page_table, history_lens, cu_seqlens,
                        total_tokens, out, num_seqs, max_new_tokens, num_q_heads, num_kv_heads, head_dim, tokens_per_page,
                        num_pages, max_pages_per_seq, scale, dtype, impl, workspace, workspace_bytes, stream);
}

int pal_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  if (!workspace || workspace_bytes < sizeof(WorkspaceHeader) || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("workspace_init: a 256-byte aligned workspace of at least %zu bytes is required", sizeof(WorkspaceHeader));
    return PAL_ERR_WORKSPACE;
  }
  return cuda_rc((int)cudaMemsetAsync(workspace, 0, sizeof(WorkspaceHeader), (cudaStream_t)stream), "workspace_init");
}

int64_t pal_set_wait_limit_cycles(int64_t cycles) {
  if (cycles <= 0) cycles = kDefaultWaitLimitCycles;
  return g_wait_limit.exchange(cycles, std::memory_order_relaxed);
}

int pal_selftest_bounded_wait(void* workspace, int64_t limit_cycles, void* stream) {
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255)) {
    set_error("selftest_bounded_wait: a 256-byte aligned workspace is required");
    return PAL_ERR_WORKSPACE;
  }
  if (limit_cycles <= 0 || limit_cycles > kDefaultWaitLimitCycles) {
    set_error("selftest_bounded_wait: limit_cycles must be in (0, %lld]", kDefaultWaitLimitCycles);
    return PAL_ERR_BAD_ARG;
  }
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(static_cast<WorkspaceHeader*>(workspace), limit_cycles);
  return cuda_rc((int)cudaGetLastError(), "selftest_bounded_wait");
}

int pal_check_status(void* workspace, void* stream) {
  if (!workspace) {
    set_error("check_status: workspace is null");
    return PAL_ERR_BAD_ARG;
  }
  WorkspaceHeader h;
  cudaError_t e = cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_rc((int)e, "check_status");
  if (h.status == kStatusTimeout) {
    // a kernel that gave up left the scheduler's counters wherever they were: make the workspace usable again
    e = cudaMemsetAsync(workspace, 0, sizeof(WorkspaceHeader), (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_rc((int)e, "check_status");
    set_error("a bounded device-side wait timed out");
    return PAL_ERR_TIMEOUT;
  }
  return PAL_OK;
}

}  // extern "C"
