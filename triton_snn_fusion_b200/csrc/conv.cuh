// Argument block shared by the dense conv / linear + LIF implementations.
#pragma once
#include "common.cuh"

namespace snnb {

struct ConvArgs {
  const void *x;        // [T][B][H][W][Cin], frames x_t_stride elements apart (0: one frame for all t)
  int64_t x_t_stride;
  const void *w;        // [Cout][KH][KW][Cin]
  const void *b;        // [Cout] or null
  const void *res;      // null or [T][B][Ho][Wo][Cout]
  const void *v_init;   // null or [B][Ho][Wo][Cout]
  void *spikes;         // [T][B][Ho][Wo][Cout]
  void *v_out;          // [B][Ho][Wo][Cout]
  int T, B, Cin, H, W, Cout, KH, KW, stride, pad, Ho, Wo;
  int lif;              // 0: write conv + bias (+ residual) instead of spikes, no state
  int dtype, spike_dtype, v_dtype;
  LifParams p;
  // Optional strided view of x for the tensor-core path (all 0 = the dense [B][H][W][Cin] frame):
  // element strides between neighbouring pixels / rows / images and the number of valid
  // coordinates along W and H. Used to read overlapping windows as if they were pixels.
  long long xs_w = 0, xs_h = 0, xs_b = 0;
  int xd_w = 0, xd_h = 0;
  // Optional shortcut branch accumulated into the same output before the LIF: a 1x1 conv with stride
  // sc_stride over a second input sc_x [T][B][sc_H][sc_W][sc_cin] (frames sc_t_stride elements apart),
  // weights sc_w [Cout][sc_cin]; its bias is folded into b by the caller. Output pixel (h, w) reads
  // sc_x at (h * sc_stride, w * sc_stride). Only the timestep-pair kernel implements it.
  const void *sc_x = nullptr;
  const void *sc_w = nullptr;
  const void *b2 = nullptr;   // bias of the shortcut conv, [Cout] or null: added to b in fp32
  int64_t sc_t_stride = 0;
  int sc_cin = 0, sc_H = 0, sc_W = 0, sc_stride = 1;
};

// CUDA-core implicit GEMM (any shape, fp32 accumulate).
int conv_lif_simt(const ConvArgs &a, cudaStream_t stream);

// Direct CUDA-core kernel for 3x3 convs over images with at most four channels (the first layer of a network).
bool conv_smallcin_supported(const ConvArgs &a);
int conv_smallcin(const ConvArgs &a, cudaStream_t stream);

// tcgen05 / TMEM implicit GEMM fed by TMA. `why` receives the reason when unsupported.
bool conv_lif_tc_supported(const ConvArgs &a, const char **why);
int conv_lif_tc(const ConvArgs &a, cudaStream_t stream);

// tcgen05 implicit GEMM for 3x3 / stride 1 / padding 1 that reads all nine taps from one
// shared-memory halo tile (far less L2 traffic than conv_lif_tc). Preferred when supported.
bool conv3x3_halo_supported(const ConvArgs &a);
int conv3x3_halo(const ConvArgs &a, cudaStream_t stream);
int halo_device_status(int *out);

// tcgen05 implicit GEMM for 3x3 (stride 1 or 2) and 1x1 convs, T = 1 or even: weights as the M operand and
// the pixels of two timesteps as a 256-wide N operand (the only shape that runs the tensor pipe at
// its full rate), halo tiles in shared memory. Preferred over conv3x3_halo when supported.
bool conv3x3_pair_supported(const ConvArgs &a);
int conv3x3_pair(const ConvArgs &a, cudaStream_t stream);
int pair_device_status(int *out);
// Self-test of the bounded waits (snnb_selftest_arm_wait_timeout): if armed, hands the shortened limit and the
// "drop one load" switch to the next launch of the timestep-pair kernel and disarms.
void consume_wait_selftest(long long *limit_cycles, int *drop_load);

// GEMM + LIF stage of the 7x7 / stride 2 stem on the re-laid image (stem.cu): persistent tcgen05 kernel
// with the packed weight resident in shared memory.
struct StemGemmArgs {
  const void *s2d;        // re-laid input [frames * B][Hb][Wb][16]
  const void *w_packed;   // [Cout][4][4][16]
  const void *b, *v_init;
  void *spikes, *v_out;
  int T, frames, B, Ho, Wo, Hb, Wb, Cout;   // frames = 1 (one frame for every step) or T
  int dtype, spike_dtype, v_dtype;
  LifParams p;
};
bool stem_gemm_supported(const StemGemmArgs &a);
int stem_gemm_lif(const StemGemmArgs &a, cudaStream_t stream);
int stem_device_status(int *out);
int dw_device_status(int *out);   // depthwise tile kernel (dwconv_tile.cu)

}  // namespace snnb
