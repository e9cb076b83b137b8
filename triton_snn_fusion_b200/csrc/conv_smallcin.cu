// 3x3 conv over an image with at most four channels (+ bias) + LIF over T: the first layer of a network that
// reads RGB frames (CNN-small 3 -> 64 stride 1, MobileNet 3 -> 32 stride 2).
//
// K = 9 * Cin <= 36 is far too small for the tensor-core kernels and the layer is bound by its output stream
// (T spike frames per input frame), so this is a direct CUDA-core kernel: a thread owns eight consecutive output
// channels of one output pixel, reads the window's 9 * Cin input values (lanes that share a pixel read the same
// addresses), takes its weights from a [tap][Cout] copy in shared memory with two 16-byte reads per tap, and keeps
// the eight membrane potentials in registers over the T steps. When all T steps see the same frame (direct
// encoding, x_t_stride == 0) the conv is evaluated once and only the LIF runs T times. Each step's eight spikes
// leave as one 16-byte (16-bit data) store.
#include "conv.cuh"

namespace snnb {
namespace {

constexpr int kMaxTaps = 36;

// CIN: the channel count as a compile-time constant, which unrolls the whole window (all 9 * CIN input loads are
// issued before the first multiply-add and out-of-image taps become predicated zero loads); FAST: tau a power of
// two with hard reset, evaluated without lif_step's run-time mode switch.
template <typename XT, typename ST, typename VT, int CIN, bool FAST>
__global__ void __launch_bounds__(256)
conv3x3_smallcin_kernel(const XT *__restrict__ x, long long x_t_stride, const XT *__restrict__ w,
                        const XT *__restrict__ bias, const VT *v_init, ST *__restrict__ spikes, VT *v_out,
                        int T, int B, int H, int W, int Cout, int stride, int Ho, int Wo, int lif,
                        LifParams p) {
  extern __shared__ __align__(16) float ws[];   // [9 * Cin][Cout]
  constexpr int Cin = CIN;
  constexpr int ntaps = 9 * Cin;
  for (int i = threadIdx.x; i < ntaps * Cout; i += blockDim.x) {
    const int tap = i / Cout, co = i - tap * Cout;
    ws[i] = DT<XT>::to_f(w[(size_t)co * ntaps + tap]);   // [Cout][3][3][Cin] -> [tap][Cout]
  }
  __syncthreads();
  const int groups = Cout >> 3;
  const long long total = (long long)B * Ho * Wo * groups;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int cg = (int)(idx % groups);
  long long pix = idx / groups;
  const int wo = (int)(pix % Wo); pix /= Wo;
  const int ho = (int)(pix % Ho);
  const int b = (int)(pix / Ho);
  const int c0 = cg * 8;
  float bs[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) bs[i] = bias != nullptr ? DT<XT>::to_f(bias[c0 + i]) : 0.f;
  const size_t o0 = (((size_t)b * Ho + ho) * Wo + wo) * Cout + c0;
  const size_t frame_out = (size_t)B * Ho * Wo * Cout;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.f;
  if (lif && v_init != nullptr) load_pack_stream<VT, 8>(v_init + o0, v);

  const int h0 = ho * stride - 1, w0 = wo * stride - 1;
  const int frames = x_t_stride == 0 ? 1 : T;
  float y[8];
  for (int t = 0; t < T; ++t) {
    if (t < frames) {   // a new input frame: evaluate the conv
      const XT *xf = x + (size_t)t * (size_t)x_t_stride + (size_t)b * H * W * Cin;
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = bs[i];
      float xv[ntaps];
#pragma unroll
      for (int kh = 0; kh < 3; ++kh)
#pragma unroll
        for (int kw = 0; kw < 3; ++kw) {
          const int h = h0 + kh, wi = w0 + kw;
          const bool in = h >= 0 && h < H && wi >= 0 && wi < W;
          const XT *px = xf + ((size_t)(in ? h : 0) * W + (in ? wi : 0)) * Cin;
#pragma unroll
          for (int ci = 0; ci < Cin; ++ci) xv[(kh * 3 + kw) * Cin + ci] = in ? DT<XT>::to_f(px[ci]) : 0.f;
        }
#pragma unroll
      for (int tp = 0; tp < ntaps; ++tp) {
        const float4 wa = *reinterpret_cast<const float4 *>(ws + (size_t)tp * Cout + c0);
        const float4 wb = *reinterpret_cast<const float4 *>(ws + (size_t)tp * Cout + c0 + 4);
        const float xt = xv[tp];
        y[0] = fmaf(wa.x, xt, y[0]); y[1] = fmaf(wa.y, xt, y[1]); y[2] = fmaf(wa.z, xt, y[2]); y[3] = fmaf(wa.w, xt, y[3]);
        y[4] = fmaf(wb.x, xt, y[4]); y[5] = fmaf(wb.y, xt, y[5]); y[6] = fmaf(wb.z, xt, y[6]); y[7] = fmaf(wb.w, xt, y[7]);
      }
    }
    if (lif) {
      float s[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] = FAST ? lif_step_t<1, true>(y[i], v[i], p) : lif_step(y[i], v[i], p);
      store_pack<ST, 8>(spikes + (size_t)t * frame_out + o0, s);
    } else {
      store_pack<XT, 8>(reinterpret_cast<XT *>(spikes) + (size_t)t * frame_out + o0, y);
    }
  }
  if (lif && v_out != nullptr) store_pack<VT, 8>(v_out + o0, v);
}

template <typename XT, typename ST, typename VT, int CIN, bool FAST>
int launch_cin(const ConvArgs &a, cudaStream_t stream) {
  const long long total = (long long)a.B * a.Ho * a.Wo * (a.Cout / 8);
  const long long blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "conv_lif: problem too large");
  const size_t smem = (size_t)9 * a.Cin * a.Cout * sizeof(float);
  conv3x3_smallcin_kernel<XT, ST, VT, CIN, FAST><<<(unsigned)blocks, 256, smem, stream>>>(
      static_cast<const XT *>(a.x), (long long)a.x_t_stride, static_cast<const XT *>(a.w), static_cast<const XT *>(a.b),
      static_cast<const VT *>(a.v_init), static_cast<ST *>(a.spikes), static_cast<VT *>(a.v_out), a.T, a.B,
      a.H, a.W, a.Cout, a.stride, a.Ho, a.Wo, a.lif, a.p);
  SNNB_CHECK_LAUNCH("conv3x3_smallcin");
  return SNNB_OK;
}

template <typename XT, typename ST, typename VT>
int launch(const ConvArgs &a, cudaStream_t stream) {
  const bool fast = a.lif && a.p.mode == 1 && a.p.hard;
  switch (a.Cin * 2 + (fast ? 1 : 0)) {
    case 2: return launch_cin<XT, ST, VT, 1, false>(a, stream);
    case 3: return launch_cin<XT, ST, VT, 1, true>(a, stream);
    case 4: return launch_cin<XT, ST, VT, 2, false>(a, stream);
    case 5: return launch_cin<XT, ST, VT, 2, true>(a, stream);
    case 6: return launch_cin<XT, ST, VT, 3, false>(a, stream);
    case 7: return launch_cin<XT, ST, VT, 3, true>(a, stream);
    case 8: return launch_cin<XT, ST, VT, 4, false>(a, stream);
    default: return launch_cin<XT, ST, VT, 4, true>(a, stream);
  }
}

template <typename XT>
int dispatch(const ConvArgs &a, cudaStream_t stream) {
  const bool s_u8 = a.lif && a.spike_dtype == SNNB_U8;
  const bool v_f32 = a.lif && a.v_dtype == SNNB_F32 && a.dtype != SNNB_F32;
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(a, stream);
  if (s_u8) return launch<XT, uint8_t, XT>(a, stream);
  if (v_f32) return launch<XT, XT, float>(a, stream);
  return launch<XT, XT, XT>(a, stream);
}

}  // namespace

bool conv_smallcin_supported(const ConvArgs &a) {
  if (a.KH != 3 || a.KW != 3 || a.pad != 1 || (a.stride != 1 && a.stride != 2)) return false;
  if (a.Cin < 1 || a.Cin > 4 || a.Cout % 8 != 0 || 9 * a.Cin > kMaxTaps) return false;
  if ((size_t)9 * a.Cin * a.Cout * sizeof(float) > 40 * 1024) return false;
  if (a.res != nullptr || a.sc_x != nullptr) return false;
  if (a.xs_w || a.xs_h || a.xs_b || a.xd_w || a.xd_h) return false;
  if (!aligned16(a.spikes) || (a.v_out && !aligned16(a.v_out)) || (a.v_init && !aligned16(a.v_init))) return false;
  return true;
}

int conv_smallcin(const ConvArgs &a, cudaStream_t stream) {
  switch (a.dtype) {
    case SNNB_F32: return dispatch<float>(a, stream);
    case SNNB_BF16: return dispatch<__nv_bfloat16>(a, stream);
    default: return dispatch<__half>(a, stream);
  }
}

}  // namespace snnb
