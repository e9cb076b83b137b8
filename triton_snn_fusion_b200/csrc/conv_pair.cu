// Host-side gate of the timestep-pair conv kernel (conv_pair_impl.cuh): which calls it takes, and the
// routing to the per-dtype translation units.
#include "conv.cuh"

#include <atomic>

namespace snnb {

namespace {
std::atomic<long long> g_selftest_limit{0};
}

void consume_wait_selftest(long long *limit_cycles, int *drop_load) {
  const long long armed = g_selftest_limit.exchange(0);
  if (armed > 0) {
    *limit_cycles = armed;
    *drop_load = 1;
  }
}

// one translation unit per (activation, spike, membrane) type combination: s = the activation type, u = one-byte
// spikes, f = fp32 membrane
#define SNNB_PAIR_UNITS(X) X(bf16_ss) X(bf16_sf) X(bf16_us) X(bf16_uf) X(f16_ss) X(f16_sf) X(f16_us) X(f16_uf)
#define SNNB_PAIR_DECL(tag)                                        \
  int conv3x3_pair_##tag(const ConvArgs &a, cudaStream_t stream);  \
  int pair_status_##tag(int *out);
SNNB_PAIR_UNITS(SNNB_PAIR_DECL)
#undef SNNB_PAIR_DECL

bool conv3x3_pair_supported(const ConvArgs &a) {
  if (a.dtype != SNNB_BF16 && a.dtype != SNNB_F16) return false;
  const bool k3 = a.KH == 3 && a.KW == 3 && a.stride == 1 && a.pad == 1;
  const bool k1 = a.KH == 1 && a.KW == 1 && a.stride == 1 && a.pad == 0;   // reads only the centre of each halo tile
  // stride 2: four phase views of the input per slab; the base of the odd-column views must stay 16-byte aligned
  const bool k3s2 = a.KH == 3 && a.KW == 3 && a.stride == 2 && a.pad == 1 && a.Cout > 64 && a.H >= 2 && a.W >= 2;
  if (!k3 && !k1 && !k3s2) return false;
  if (a.sc_x != nullptr && !k3) return false;
  // input channels come in slabs of 64; a last slab that is only partly inside the tensor is completed with
  // zeros by the TMA copies of both operands (activations and weights), so any multiple of 8 channels (the
  // 16-byte granularity of a copy) works, at the price of multiplying the zeros
  if (a.Cin % 8 != 0) return false;
  if (a.Cin % 64 != 0 && (a.KH != 1 || a.sc_x != nullptr)) return false;   // only the 1x1 form has been checked on partial slabs
  if (a.x_t_stride == 0 && a.T > 1) return false;   // one frame for all steps: left to the other kernels
  // T = 1, or an even number of steps: they are processed as pairs that alternate between two accumulators in
  // tensor memory while the membrane stays in registers, so any number of pairs fits
  if (a.T != 1 && (a.T % 2 != 0 || a.T > 64)) return false;
  // maps of at least 8 x 8 (one image per tile) or at most 7 x 8 (two images per tile, Cout > 64); what lies
  // in between goes to conv_halo.cu
  const bool one_image = a.Ho >= 8 && a.Wo >= 8;
  const bool two_images = a.Ho <= 7 && a.Wo <= 8 && a.Cout > 64;
  if (!one_image && !two_images) return false;
  if (a.xs_w || a.xs_h || a.xs_b || a.xd_w || a.xd_h) return false;
  if (a.x_t_stride % 8 != 0) return false;
  if (!aligned16(a.x) || !aligned16(a.w)) return false;
  if (a.sc_x != nullptr) {   // fused 1x1 shortcut conv
    if (a.res != nullptr || a.Cout <= 64 || a.sc_cin % 64 != 0 || a.sc_stride < 1) return false;
    if ((a.sc_H - 1) / a.sc_stride + 1 != a.Ho || (a.sc_W - 1) / a.sc_stride + 1 != a.Wo) return false;
    if (a.sc_t_stride % 8 != 0 || a.sc_t_stride <= 0 || !aligned16(a.sc_x) || !aligned16(a.sc_w)) return false;
  }
  return true;
}

int conv3x3_pair(const ConvArgs &a, cudaStream_t stream) {
  const bool s_u8 = a.lif && a.spike_dtype == SNNB_U8;
  const bool v_f32 = a.lif && a.v_dtype == SNNB_F32;
  if (a.dtype == SNNB_BF16) {
    if (s_u8) return v_f32 ? conv3x3_pair_bf16_uf(a, stream) : conv3x3_pair_bf16_us(a, stream);
    return v_f32 ? conv3x3_pair_bf16_sf(a, stream) : conv3x3_pair_bf16_ss(a, stream);
  }
  if (s_u8) return v_f32 ? conv3x3_pair_f16_uf(a, stream) : conv3x3_pair_f16_us(a, stream);
  return v_f32 ? conv3x3_pair_f16_sf(a, stream) : conv3x3_pair_f16_ss(a, stream);
}

int pair_device_status(int *out) {
  int all = 0;
#define SNNB_PAIR_STATUS(tag)                   \
  {                                             \
    int h = 0;                                  \
    const int rc = pair_status_##tag(&h);       \
    if (rc != SNNB_OK) return rc;               \
    all |= h;                                   \
  }
  SNNB_PAIR_UNITS(SNNB_PAIR_STATUS)
#undef SNNB_PAIR_STATUS
  *out = all;
  return SNNB_OK;
}

}  // namespace snnb

extern "C" int snnb_selftest_arm_wait_timeout(long long limit_cycles) {
  using namespace snnb;
  SNNB_CHECK_ARG(limit_cycles >= 1000 && limit_cycles <= 4000000000ll, "selftest_arm_wait_timeout: limit out of range");
  g_selftest_limit.store(limit_cycles);
  return SNNB_OK;
}
