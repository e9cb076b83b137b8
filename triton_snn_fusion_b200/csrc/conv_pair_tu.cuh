// One translation unit of the timestep-pair conv kernel: the kernels for one combination of activation, spike and
// membrane type (SNNB_PAIR_XT / _ST / _VT, named by SNNB_PAIR_TAG), so that the eight combinations compile in
// parallel. Each unit has its own device status word.
#include "conv_pair_impl.cuh"

#define SNNB_PAIR_CAT2(a, b) a##b
#define SNNB_PAIR_CAT(a, b) SNNB_PAIR_CAT2(a, b)

namespace snnb {
int SNNB_PAIR_CAT(conv3x3_pair_, SNNB_PAIR_TAG)(const ConvArgs &a, cudaStream_t stream) {
  return launch<SNNB_PAIR_XT, SNNB_PAIR_ST, SNNB_PAIR_VT>(a, stream);
}
int SNNB_PAIR_CAT(pair_status_, SNNB_PAIR_TAG)(int *out) { return pair_tu_status(out); }
}  // namespace snnb
