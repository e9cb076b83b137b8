// Timestep-pair conv kernel, bf16 activations: spikes and membrane in the activation type.
#define SNNB_PAIR_XT __nv_bfloat16
#define SNNB_PAIR_ST __nv_bfloat16
#define SNNB_PAIR_VT __nv_bfloat16
#define SNNB_PAIR_TAG bf16_ss
#include "conv_pair_tu.cuh"
