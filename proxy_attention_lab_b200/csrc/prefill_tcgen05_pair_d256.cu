// prefill_tcgen05_pair_kernel (two CTAs per MMA) for head_dim = 256, tokens_per_page = 16 / 32.
#include "prefill_tcgen05_pair.cuh"

namespace pal {

int launch_prefill_tcgen05_pair_d256(const PrefillArgs& a, cudaStream_t stream) {
  return a.tokens_per_page == 16 ? launch_pair_shape<256, 16>(a, stream) : launch_pair_shape<256, 32>(a, stream);
}

}  // namespace pal
