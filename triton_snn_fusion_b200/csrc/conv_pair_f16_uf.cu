// Timestep-pair conv kernel, f16 activations: one-byte spikes, fp32 membrane.
#define SNNB_PAIR_XT __half
#define SNNB_PAIR_ST uint8_t
#define SNNB_PAIR_VT float
#define SNNB_PAIR_TAG f16_uf
#include "conv_pair_tu.cuh"
