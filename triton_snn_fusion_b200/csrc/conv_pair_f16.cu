// f16 instantiations of the timestep-pair conv kernel (one translation unit per activation type so
// that the two compile in parallel).
#include "conv_pair_impl.cuh"

namespace snnb {
int conv3x3_pair_f16(const ConvArgs &a, cudaStream_t stream) { return dispatch<__half>(a, stream); }
int pair_status_f16(int *out) { return pair_tu_status(out); }
}  // namespace snnb
