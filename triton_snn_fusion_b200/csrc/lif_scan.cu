// Standalone temporal LIF scan: one thread owns VEC consecutive neurons, keeps
// their membrane potential in registers and walks the T timesteps.
//
// HBM-bound streaming kernel. Per neuron it moves T*(s_x + s_spike) bytes plus
// the membrane state once in (if given) and once out; all accesses are 128-bit
// (or the widest the dtype allows), issued for all T steps before the first
// use when T is a compile-time constant so that each thread keeps T
// independent loads in flight.
#include "common.cuh"

namespace snnb {
namespace {

constexpr int kThreads = 256;

template <typename XT, typename ST, typename VT, int VEC, int TS>
__global__ void __launch_bounds__(kThreads)
lif_scan_kernel(const XT *__restrict__ x, const VT *__restrict__ v_init, ST *__restrict__ spikes,
                VT *__restrict__ v_out, int T, int64_t n, LifParams p) {
  const int64_t pack = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const int64_t i0 = pack * VEC;
  if (i0 >= n) return;

  float v[VEC];
  if (v_init != nullptr) {
    load_pack_stream<VT, VEC>(v_init + i0, v);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = 0.f;
  }

  if constexpr (TS > 0) {
    // All T loads are issued before the first use; they stay packed (16 bytes per step)
    // until their step is evaluated so that 16-bit inputs do not double the live registers.
    Pack<XT, VEC> raw[TS];
#pragma unroll
    for (int t = 0; t < TS; ++t)
      *reinterpret_cast<int4 *>(&raw[t]) = __ldcs(reinterpret_cast<const int4 *>(x + (int64_t)t * n + i0));
#pragma unroll
    for (int t = 0; t < TS; ++t) {
      float s[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) s[i] = lif_step(DT<XT>::to_f(raw[t].v[i]), v[i], p);
      store_pack<ST, VEC>(spikes + (int64_t)t * n + i0, s);
    }
  } else {
    float xr[VEC], xn[VEC];
    load_pack_stream<XT, VEC>(x + i0, xr);
    for (int t = 0; t < T; ++t) {
      if (t + 1 < T) load_pack_stream<XT, VEC>(x + (int64_t)(t + 1) * n + i0, xn);
      float s[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) s[i] = lif_step(xr[i], v[i], p);
      store_pack<ST, VEC>(spikes + (int64_t)t * n + i0, s);
#pragma unroll
      for (int i = 0; i < VEC; ++i) xr[i] = xn[i];
    }
  }
  store_pack<VT, VEC>(v_out + i0, v);
}

// Scalar variant for sizes / addresses that do not allow vector access.
template <typename XT, typename ST, typename VT>
__global__ void __launch_bounds__(kThreads)
lif_scan_scalar_kernel(const XT *__restrict__ x, const VT *__restrict__ v_init,
                       ST *__restrict__ spikes, VT *__restrict__ v_out, int T, int64_t n,
                       LifParams p) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  float v = v_init != nullptr ? DT<VT>::to_f(v_init[i]) : 0.f;
  for (int t = 0; t < T; ++t) {
    const float s = lif_step(DT<XT>::to_f(x[(int64_t)t * n + i]), v, p);
    spikes[(int64_t)t * n + i] = DT<ST>::from_f(s);
  }
  v_out[i] = DT<VT>::from_f(v);
}

template <typename XT, typename ST, typename VT>
int launch(const void *x, const void *v_init, void *spikes, void *v_out, int T, int64_t n,
           const LifParams &p, cudaStream_t stream) {
  constexpr int VEC = 16 / sizeof(XT);
  const XT *xp = static_cast<const XT *>(x);
  const VT *vi = static_cast<const VT *>(v_init);
  ST *sp = static_cast<ST *>(spikes);
  VT *vo = static_cast<VT *>(v_out);
  auto al = [](const void *q, size_t a) { return (reinterpret_cast<uintptr_t>(q) % a) == 0; };
  constexpr size_t SA = sizeof(ST) * VEC >= 16 ? 16 : sizeof(ST) * VEC;
  constexpr size_t VA = sizeof(VT) * VEC >= 16 ? 16 : sizeof(VT) * VEC;
  const bool vec_ok = (n % VEC == 0) && al(x, 16) && al(spikes, SA) && al(v_out, VA) &&
                      (v_init == nullptr || al(v_init, VA));
  if (vec_ok) {
    const int64_t packs = n / VEC;
    const int64_t blocks = (packs + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "lif_scan: n too large");
    dim3 grid((unsigned)blocks), block(kThreads);
#define SNNB_LIF_CASE(TS) \
  lif_scan_kernel<XT, ST, VT, VEC, TS><<<grid, block, 0, stream>>>(xp, vi, sp, vo, T, n, p)
    switch (T) {
      case 1: SNNB_LIF_CASE(1); break;
      case 2: SNNB_LIF_CASE(2); break;
      case 4: SNNB_LIF_CASE(4); break;
      case 8: SNNB_LIF_CASE(8); break;
      case 16: SNNB_LIF_CASE(16); break;
      default: SNNB_LIF_CASE(0); break;
    }
#undef SNNB_LIF_CASE
  } else {
    const int64_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "lif_scan: n too large");
    lif_scan_scalar_kernel<XT, ST, VT><<<(unsigned)blocks, kThreads, 0, stream>>>(xp, vi, sp, vo, T, n, p);
  }
  SNNB_CHECK_LAUNCH("lif_scan");
  return SNNB_OK;
}

template <typename XT>
int dispatch(const void *x, const void *v_init, void *spikes, void *v_out, int T, int64_t n,
             int x_dtype, int spike_dtype, int v_dtype, const LifParams &p, cudaStream_t stream) {
  const bool s_u8 = spike_dtype == SNNB_U8;
  const bool v_f32 = v_dtype == SNNB_F32;
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(x, v_init, spikes, v_out, T, n, p, stream);
  if (s_u8) return launch<XT, uint8_t, XT>(x, v_init, spikes, v_out, T, n, p, stream);
  if (v_f32) return launch<XT, XT, float>(x, v_init, spikes, v_out, T, n, p, stream);
  return launch<XT, XT, XT>(x, v_init, spikes, v_out, T, n, p, stream);
}

}  // namespace
}  // namespace snnb

extern "C" int snnb_lif_scan(const void *x_seq, const void *v_init, void *spikes, void *v_out,
                             int T, int64_t n, int x_dtype, int spike_dtype, int v_dtype,
                             float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && spikes && v_out, "lif_scan: null pointer");
  SNNB_CHECK_ARG(T >= 1, "lif_scan: T must be >= 1, got %d", T);
  SNNB_CHECK_ARG(n >= 0, "lif_scan: n must be >= 0");
  SNNB_CHECK_ARG(is_act_dtype(x_dtype), "lif_scan: unsupported x dtype %d", x_dtype);
  SNNB_CHECK_ARG(spike_dtype == x_dtype || spike_dtype == SNNB_U8,
                 "lif_scan: spike dtype must be the x dtype or u8");
  SNNB_CHECK_ARG(v_dtype == x_dtype || v_dtype == SNNB_F32, "lif_scan: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(tau != 0.0f, "lif_scan: unsupported_tau: tau must be nonzero");
  if (n == 0) return SNNB_OK;
  const LifParams p = make_lif_params(v_th, v_reset, tau);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case SNNB_F32: return dispatch<float>(x_seq, v_init, spikes, v_out, T, n, x_dtype, spike_dtype, v_dtype, p, s);
    case SNNB_BF16: return dispatch<__nv_bfloat16>(x_seq, v_init, spikes, v_out, T, n, x_dtype, spike_dtype, v_dtype, p, s);
    default: return dispatch<__half>(x_seq, v_init, spikes, v_out, T, n, x_dtype, spike_dtype, v_dtype, p, s);
  }
}
