// Timestep-pair conv kernel, bf16 activations: one-byte spikes, membrane in the activation type.
#define SNNB_PAIR_XT __nv_bfloat16
#define SNNB_PAIR_ST uint8_t
#define SNNB_PAIR_VT __nv_bfloat16
#define SNNB_PAIR_TAG bf16_us
#include "conv_pair_tu.cuh"
