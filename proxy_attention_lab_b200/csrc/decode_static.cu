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
//  * CUDA loads this file's module lazily, at the first pal_static_scratch_init (or first decode_static call) on
//    a device: that is the moment the device sets PAL_STATIC_SCRATCH_BYTES aside, and it keeps them until the
//    process exits.  A host that is about to commit all remaining device memory calls pal_static_scratch_init
//    first; if the memory is already gone the call fails with PAL_ERR_WORKSPACE.
//  * problems whose workspace exceeds that size are refused with PAL_ERR_WORKSPACE (use
//    pal_paged_attention_decode with a caller-owned workspace instead);
//  * the first call on a device zeroes the array's 256-byte header and the kernels put the scheduler's counters
//    back to zero when they finish, which is all that has to start at zero; partial results of the previous
//    call are overwritten before they are read.  Two calls that overlap on one GPU (different streams, or
//    different host threads) race on the array.  Serialise them.
//  * the device address is looked up once per device and kept; cudaDeviceReset invalidates it, so a
//    process that resets a device must not call these entry points for it afterwards.
//
// The array's name in host code is only a handle, not a device pointer: the address the kernels get
// comes from cudaGetSymbolAddress, called with the device current.  Make the first call on a device
// outside any stream capture.
#include <mutex>

#include "../../include/pal_b200.h"
#include "common.cuh"
#include "launch.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[PAL_STATIC_SCRATCH_BYTES];

void* g_scratch_ptr[pal::kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of this device's copy of the array; looked up once per device, with that device current.
int static_scratch_for_current_device(const char* what, void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return pal::cuda_rc((int)e, what);
  if (dev < 0 || dev >= pal::kMaxDevices) {
    pal::set_error("%s: device ordinal %d is outside the supported range [0, %d)", what, dev, pal::kMaxDevices);
    return PAL_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return pal::cuda_rc((int)e, what);  // out of memory comes back as PAL_ERR_WORKSPACE
    if (ptr == nullptr) {
      pal::set_error("%s: cudaGetSymbolAddress returned a null address on device %d", what, dev);
      return PAL_ERR_LAUNCH;
    }
    // the header must start at zero; this runs once per device, before any kernel has seen the array
    e = cudaMemset(ptr, 0, sizeof(pal::WorkspaceHeader));
    if (e != cudaSuccess) return pal::cuda_rc((int)e, what);
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return PAL_OK;
}

}  // namespace

extern "C" int pal_static_scratch_init(void) {
  void* scratch = nullptr;
  return static_scratch_for_current_device("static_scratch_init", &scratch);
}

extern "C" int pal_check_status_static(void* stream) {
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device("check_status_static", &scratch);
  if (rc != PAL_OK) return rc;
  return pal_check_status(scratch, stream);
}

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
  const int rc = static_scratch_for_current_device("paged_attention_decode_static", &scratch);
  if (rc != PAL_OK) return rc;
  return pal_paged_attention_decode(queries, k_pool, v_pool, page_table, sequence_lengths, out, num_seqs, num_q_heads,
                                    num_kv_heads, head_dim, tokens_per_page, num_pages, max_pages_per_seq, scale, dtype,
                                    partition_pages, scratch, (size_t)PAL_STATIC_SCRATCH_BYTES, stream);
}
