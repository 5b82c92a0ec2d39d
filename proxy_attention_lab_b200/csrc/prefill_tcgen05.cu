// placeholder until the tcgen05 kernel lands
#include "launch.h"
namespace pal {
int launch_prefill_tcgen05(const PrefillArgs&, cudaStream_t) {
  set_error("paged_attention_prefill: the tcgen05 kernel is not built in this library");
  return -2;
}
}  // namespace pal
