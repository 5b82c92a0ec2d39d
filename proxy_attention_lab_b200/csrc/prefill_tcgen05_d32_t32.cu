// prefill_tcgen05_kernel for head_dim = 32, tokens_per_page = 32 (a translation unit per shape keeps the build parallel).
#include "prefill_tcgen05.cuh"

namespace pal {

int launch_prefill_tcgen05_d32_t32(const PrefillArgs& a, cudaStream_t stream) { return launch_tc_shape<32, 32>(a, stream); }

}  // namespace pal
