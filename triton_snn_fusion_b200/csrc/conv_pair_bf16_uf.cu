// Timestep-pair conv kernel, bf16 activations: one-byte spikes, fp32 membrane.
#define SNNB_PAIR_XT __nv_bfloat16
#define SNNB_PAIR_ST uint8_t
#define SNNB_PAIR_VT float
#define SNNB_PAIR_TAG bf16_uf
#include "conv_pair_tu.cuh"
