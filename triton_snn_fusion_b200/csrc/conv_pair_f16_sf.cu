// Timestep-pair conv kernel, f16 activations: spikes in the activation type, fp32 membrane.
#define SNNB_PAIR_XT __half
#define SNNB_PAIR_ST __half
#define SNNB_PAIR_VT float
#define SNNB_PAIR_TAG f16_sf
#include "conv_pair_tu.cuh"
