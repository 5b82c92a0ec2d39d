// prefill_tcgen05_kernel for head_dim = 96, tokens_per_page = 16 (a translation unit per shape keeps the build parallel).
#include "prefill_tcgen05.cuh"

namespace pal {

int launch_prefill_tcgen05_d96_t16(const PrefillArgs& a, cudaStream_t stream) { return launch_tc_shape<96, 16>(a, stream); }

}  // namespace pal
