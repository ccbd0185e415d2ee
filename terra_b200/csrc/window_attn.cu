#include "common.cuh"
#include "host_api.h"
namespace tb {
int window_attn_fwd(const WindowAttnArgs&, cudaStream_t) { return -999; }
int window_attn_bwd(const WindowAttnArgs&, cudaStream_t) { return -999; }
}  // namespace tb
