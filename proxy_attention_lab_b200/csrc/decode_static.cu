// paged_attention_decode for callers that cannot hand the library any scratch memory.
//
// Some hosts only ever own the tensors their framework gave them: an engine whose device memory is
// fully committed to the KV page pools, or a plugin interface that passes inputs and outputs but has
// no call for requesting temporaries.  They cannot supply the workspace pal_paged_attention_decode
// asks for.  This entry point runs the same two kernels (split-KV pass + log-sum-exp combine, or the
// fused single pass) with the workspace taken from an array that is part of the library image, so the
// call allocates nothing: no cudaMalloc / cudaFree, no allocating library routine.
//
// Consequences of the array being shared and permanent:
//  * every GPU that loads the library holds PAL_STATIC_SCRATCH_BYTES of device memory until exit;
//  * problems whose workspace exceeds that size are refused with PAL_ERR_WORKSPACE (use
//    pal_paged_attention_decode with a caller-owned workspace instead);
//  * the array keeps whatever the previous call left in it - the launcher clears the work counter and
//    status word at the start of each call, nothing else needs to start at zero - and two calls that
//    overlap on one GPU (different streams, or different host threads) race on it.  Serialise them.
//
// The first call on each device looks up the device address of the array (the array's name in host
// code is only a handle, not a device pointer).  Make that first call outside any stream capture.
#include <mutex>

#include "../../include/pal_b200.h"
#include "launch.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[PAL_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of this device's copy of the array; looked up once per device, with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    pal::set_error("paged_attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
    return PAL_ERR_LAUNCH;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    pal::set_error("paged_attention_decode_static: device ordinal %d is outside the supported range [0, %d)", dev, kMaxDevices);
    return PAL_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      pal::set_error("paged_attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                     cudaGetErrorString(e));
      return PAL_ERR_LAUNCH;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return PAL_OK;
}

}  // namespace

extern "C" int pal_paged_attention_decode_static(const void* queries, const void* k_pool, const void* v_pool,
                                                 const void* page_table, const int32_t* sequence_lengths, void* out,
                                                 int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                                                 int tokens_per_page, int64_t num_pages, int max_pages_per_seq,
                                                 float scale, int dtype, int partition_pages, void* stream) {
  if (num_seqs > 0 && num_q_heads > 0 && num_kv_heads > 0 && head_dim > 0) {
    const size_t need = pal_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim, tokens_per_page,
                                                   max_pages_per_seq, partition_pages);
    if (need > (size_t)PAL_STATIC_SCRATCH_BYTES) {
      pal::set_error("paged_attention_decode_static: this problem needs %zu bytes of workspace but the built-in scratch "
                     "holds %zu; call pal_paged_attention_decode with a caller-owned workspace",
                     need, (size_t)PAL_STATIC_SCRATCH_BYTES);
      return PAL_ERR_WORKSPACE;
    }
  }
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != PAL_OK) return rc;
  return pal_paged_attention_decode(queries, k_pool, v_pool, page_table, sequence_lengths, out, num_seqs, num_q_heads,
                                    num_kv_heads, head_dim, tokens_per_page, num_pages, max_pages_per_seq, scale, dtype,
                                    partition_pages, scratch, (size_t)PAL_STATIC_SCRATCH_BYTES, stream);
}
