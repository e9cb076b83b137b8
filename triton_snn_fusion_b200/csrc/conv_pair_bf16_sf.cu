// Timestep-pair conv kernel, bf16 activations: spikes in the activation type, fp32 membrane.
#define SNNB_PAIR_XT __nv_bfloat16
#define SNNB_PAIR_ST __nv_bfloat16
#define SNNB_PAIR_VT float
#define SNNB_PAIR_TAG bf16_sf
#include "conv_pair_tu.cuh"
