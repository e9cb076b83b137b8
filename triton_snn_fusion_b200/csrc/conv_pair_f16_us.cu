// Timestep-pair conv kernel, f16 activations: one-byte spikes, membrane in the activation type.
#define SNNB_PAIR_XT __half
#define SNNB_PAIR_ST uint8_t
#define SNNB_PAIR_VT __half
#define SNNB_PAIR_TAG f16_us
#include "conv_pair_tu.cuh"
