// Timestep-pair conv kernel, f16 activations: spikes and membrane in the activation type.
#define SNNB_PAIR_XT __half
#define SNNB_PAIR_ST __half
#define SNNB_PAIR_VT __half
#define SNNB_PAIR_TAG f16_ss
#include "conv_pair_tu.cuh"
