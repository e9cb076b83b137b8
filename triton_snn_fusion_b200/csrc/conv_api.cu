// extern "C" entry points of the dense conv / linear + LIF ops: argument validation and
// the choice between the tensor-core and the CUDA-core implementation.

#include "conv.cuh"

namespace snnb {
namespace {

// v_init and v_out may be one and the same buffer (the membrane is then updated in place, as the reference's
// in/out membrane buffer is); two different buffers that overlap would be read and written by different threads.
bool membranes_overlap_partially(const ConvArgs &a) {
  if (!a.lif || a.v_init == nullptr || a.v_out == nullptr || a.v_init == a.v_out) return false;
  const size_t bytes = (size_t)a.B * a.Ho * a.Wo * a.Cout * dtype_size(a.v_dtype);
  const char *p = static_cast<const char *>(a.v_init), *q = static_cast<const char *>(a.v_out);
  return p < q + bytes && q < p + bytes;
}

int run(const ConvArgs &a, int path, cudaStream_t stream, const char *what) {
  if (membranes_overlap_partially(a))
    return fail(SNNB_ERR_INVALID, "%s: v_init and v_out overlap without being the same buffer", what);
  if (path == SNNB_PATH_AUTO && conv_smallcin_supported(a)) return conv_smallcin(a, stream);   // RGB first layers
  if (path == SNNB_PATH_SIMT) return conv_lif_simt(a, stream);
  const bool taps_only = path == SNNB_PATH_TCGEN05_TAPS;
  if (!taps_only && path != SNNB_PATH_TCGEN05_HALO && conv3x3_pair_supported(a)) return conv3x3_pair(a, stream);
  if (!taps_only && conv3x3_halo_supported(a)) return conv3x3_halo(a, stream);
  const char *why = "";
  if (conv_lif_tc_supported(a, &why)) return conv_lif_tc(a, stream);
  if (path == SNNB_PATH_AUTO) return conv_lif_simt(a, stream);
  return fail(SNNB_ERR_UNSUPPORTED, "%s: tcgen05 path not available for this call: %s", what, why);
}

}  // namespace
}  // namespace snnb

extern "C" int snnb_conv_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                             const void *residual, const void *v_init, void *spikes, void *v_out,
                             int T, int B, int Cin, int H, int W, int Cout, int KH, int KW,
                             int stride, int pad, int lif, int dtype, int spike_dtype, int v_dtype,
                             float v_th, float v_reset, float tau, int path, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && w && spikes, "conv_lif: null pointer");
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && Cin >= 1 && Cout >= 1 && H >= 1 && W >= 1, "conv_lif: sizes must be positive");
  SNNB_CHECK_ARG(KH >= 1 && KW >= 1 && stride >= 1 && pad >= 0, "conv_lif: bad kernel/stride/padding");
  SNNB_CHECK_ARG(is_act_dtype(dtype), "conv_lif: unsupported dtype %d", dtype);
  SNNB_CHECK_ARG(!lif || spike_dtype == dtype || spike_dtype == SNNB_U8, "conv_lif: spike dtype must be the x dtype or u8");
  SNNB_CHECK_ARG(!lif || v_dtype == dtype || v_dtype == SNNB_F32, "conv_lif: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(path >= SNNB_PATH_AUTO && path <= SNNB_PATH_TCGEN05_HALO, "conv_lif: bad path %d", path);
  SNNB_CHECK_ARG(x_t_stride >= 0, "conv_lif: negative frame stride");
  SNNB_CHECK_ARG(!lif || tau != 0.0f, "conv_lif: unsupported_tau: tau must be nonzero");
  const int Ho = (H + 2 * pad - KH) / stride + 1;
  const int Wo = (W + 2 * pad - KW) / stride + 1;
  SNNB_CHECK_ARG(H + 2 * pad >= KH && W + 2 * pad >= KW && Ho >= 1 && Wo >= 1, "conv_lif: empty output");
  SNNB_CHECK_ARG((int64_t)B * Ho * Wo < (1LL << 31) && (int64_t)KH * KW * Cin < (1LL << 31), "conv_lif: problem too large");
  ConvArgs a;
  a.x = x_seq; a.x_t_stride = x_t_stride; a.w = w; a.b = b; a.res = residual;
  a.v_init = lif ? v_init : nullptr; a.spikes = spikes; a.v_out = v_out;
  a.T = T; a.B = B; a.Cin = Cin; a.H = H; a.W = W; a.Cout = Cout; a.KH = KH; a.KW = KW;
  a.stride = stride; a.pad = pad; a.Ho = Ho; a.Wo = Wo; a.lif = lif ? 1 : 0;
  a.dtype = dtype; a.spike_dtype = lif ? spike_dtype : dtype; a.v_dtype = lif ? v_dtype : dtype;
  a.p = make_lif_params(v_th, v_reset, lif ? tau : 2.0f);
  return run(a, path, static_cast<cudaStream_t>(stream), "conv_lif");
}

extern "C" int snnb_conv_lif_which(int T, int B, int Cin, int H, int W, int Cout, int KH, int KW, int stride, int pad,
                                   int lif, int dtype, int one_frame, int has_residual, int path, char *name, int name_len) {
  using namespace snnb;
  SNNB_CHECK_ARG(name != nullptr && name_len >= 8, "conv_lif_which: name buffer too small");
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && Cin >= 1 && Cout >= 1 && H >= 1 && W >= 1 && KH >= 1 && KW >= 1 && stride >= 1 && pad >= 0,
                 "conv_lif_which: bad sizes");
  SNNB_CHECK_ARG(is_act_dtype(dtype), "conv_lif_which: unsupported dtype %d", dtype);
  ConvArgs a;
  // stand-in addresses: 16-byte aligned and distinct, which is all the support gates look at
  a.x = reinterpret_cast<const void *>(uintptr_t(0x1000)); a.w = reinterpret_cast<const void *>(uintptr_t(0x2000));
  a.b = reinterpret_cast<const void *>(uintptr_t(0x3000)); a.res = has_residual ? reinterpret_cast<const void *>(uintptr_t(0x4000)) : nullptr;
  a.v_init = nullptr; a.spikes = reinterpret_cast<void *>(uintptr_t(0x5000)); a.v_out = reinterpret_cast<void *>(uintptr_t(0x6000));
  a.T = T; a.B = B; a.Cin = Cin; a.H = H; a.W = W; a.Cout = Cout; a.KH = KH; a.KW = KW; a.stride = stride; a.pad = pad;
  a.Ho = (H + 2 * pad - KH) / stride + 1; a.Wo = (W + 2 * pad - KW) / stride + 1;
  SNNB_CHECK_ARG(a.Ho >= 1 && a.Wo >= 1, "conv_lif_which: empty output");
  a.x_t_stride = one_frame ? 0 : (int64_t)B * H * W * Cin;
  a.lif = lif ? 1 : 0; a.dtype = dtype; a.spike_dtype = dtype; a.v_dtype = dtype;
  a.p = make_lif_params(1.0f, 0.0f, 2.0f);
  const char *k = "conv_lif_simt";
  const bool taps_only = path == SNNB_PATH_TCGEN05_TAPS;
  const char *why = "";
  if (path == SNNB_PATH_AUTO && conv_smallcin_supported(a)) k = "conv3x3_smallcin";
  else if (path == SNNB_PATH_SIMT) k = "conv_lif_simt";
  else if (!taps_only && path != SNNB_PATH_TCGEN05_HALO && conv3x3_pair_supported(a)) k = "conv3x3_pair";
  else if (!taps_only && conv3x3_halo_supported(a)) k = "conv3x3_halo";
  else if (conv_lif_tc_supported(a, &why)) k = "conv_lif_tc";
  else if (path != SNNB_PATH_AUTO) return fail(SNNB_ERR_UNSUPPORTED, "conv_lif_which: no tensor-core kernel takes this call: %s", why);
  snprintf(name, (size_t)name_len, "%s", k);
  return SNNB_OK;
}

extern "C" int snnb_conv3x3_shortcut_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                                         const void *sc_x, int64_t sc_t_stride, const void *sc_w, const void *sc_b,
                                         int sc_cin, int sc_H, int sc_W, int sc_stride,
                                         const void *v_init, void *spikes, void *v_out,
                                         int T, int B, int Cin, int H, int W, int Cout,
                                         int dtype, int spike_dtype, int v_dtype,
                                         float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && w && sc_x && sc_w && spikes, "conv3x3_shortcut_lif: null pointer");
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && Cin >= 1 && Cout >= 1 && H >= 1 && W >= 1, "conv3x3_shortcut_lif: sizes must be positive");
  SNNB_CHECK_ARG(sc_cin >= 1 && sc_H >= 1 && sc_W >= 1 && sc_stride >= 1, "conv3x3_shortcut_lif: bad shortcut geometry");
  SNNB_CHECK_ARG(dtype == SNNB_BF16 || dtype == SNNB_F16, "conv3x3_shortcut_lif: dtype must be bf16 or f16");
  SNNB_CHECK_ARG(spike_dtype == dtype || spike_dtype == SNNB_U8, "conv3x3_shortcut_lif: spike dtype must be the x dtype or u8");
  SNNB_CHECK_ARG(v_dtype == dtype || v_dtype == SNNB_F32, "conv3x3_shortcut_lif: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(x_t_stride > 0 && sc_t_stride > 0 && tau != 0.0f, "conv3x3_shortcut_lif: bad frame stride or tau");
  SNNB_CHECK_ARG((int64_t)B * H * W < (1LL << 31), "conv3x3_shortcut_lif: problem too large");
  ConvArgs a;
  a.x = x_seq; a.x_t_stride = x_t_stride; a.w = w; a.b = b; a.res = nullptr;
  a.v_init = v_init; a.spikes = spikes; a.v_out = v_out;
  a.T = T; a.B = B; a.Cin = Cin; a.H = H; a.W = W; a.Cout = Cout; a.KH = 3; a.KW = 3;
  a.stride = 1; a.pad = 1; a.Ho = H; a.Wo = W; a.lif = 1;
  a.dtype = dtype; a.spike_dtype = spike_dtype; a.v_dtype = v_dtype;
  a.p = make_lif_params(v_th, v_reset, tau);
  a.sc_x = sc_x; a.sc_w = sc_w; a.b2 = sc_b; a.sc_t_stride = sc_t_stride;
  a.sc_cin = sc_cin; a.sc_H = sc_H; a.sc_W = sc_W; a.sc_stride = sc_stride;
  if (!conv3x3_pair_supported(a))
    return fail(SNNB_ERR_UNSUPPORTED,
                "conv3x3_shortcut_lif: needs Cin %% 64 == 0, sc_cin %% 64 == 0, Cout > 64, T = 1 or even, a map of at "
                "least 8x8 or at most 7x8 and a shortcut input whose strided size equals the output; run the shortcut "
                "conv and snnb_conv_lif with a residual instead");
  if (membranes_overlap_partially(a))
    return fail(SNNB_ERR_INVALID, "conv3x3_shortcut_lif: v_init and v_out overlap without being the same buffer");
  return conv3x3_pair(a, static_cast<cudaStream_t>(stream));
}

extern "C" int snnb_linear_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                               const void *v_init, void *spikes, void *v_out,
                               int T, int M, int K, int N, int dtype, int spike_dtype, int v_dtype,
                               float v_th, float v_reset, float tau, int path, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && w && spikes, "linear_lif: null pointer");
  SNNB_CHECK_ARG(T >= 1 && M >= 1 && K >= 1 && N >= 1, "linear_lif: sizes must be positive");
  SNNB_CHECK_ARG(is_act_dtype(dtype), "linear_lif: unsupported dtype %d", dtype);
  SNNB_CHECK_ARG(spike_dtype == dtype || spike_dtype == SNNB_U8, "linear_lif: spike dtype must be the x dtype or u8");
  SNNB_CHECK_ARG(v_dtype == dtype || v_dtype == SNNB_F32, "linear_lif: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(path >= SNNB_PATH_AUTO && path <= SNNB_PATH_TCGEN05_HALO, "linear_lif: bad path %d", path);
  SNNB_CHECK_ARG(x_t_stride >= 0, "linear_lif: negative frame stride");
  SNNB_CHECK_ARG(tau != 0.0f, "linear_lif: unsupported_tau: tau must be nonzero");
  // A linear layer over [M][K] rows is a 1x1 convolution over one [1][M] frame with K channels.
  ConvArgs a;
  a.x = x_seq; a.x_t_stride = x_t_stride; a.w = w; a.b = b; a.res = nullptr;
  a.v_init = v_init; a.spikes = spikes; a.v_out = v_out;
  // a 1x1 conv over the tokens laid out as an image: 8 tokens per row when that divides (the shape the
  // timestep-pair kernel tiles), else one row of M tokens
  const bool rows8 = M % 8 == 0 && M >= 64;
  a.T = T; a.B = 1; a.Cin = K; a.H = rows8 ? M / 8 : 1; a.W = rows8 ? 8 : M; a.Cout = N; a.KH = 1; a.KW = 1;
  a.stride = 1; a.pad = 0; a.Ho = a.H; a.Wo = a.W; a.lif = 1;
  a.dtype = dtype; a.spike_dtype = spike_dtype; a.v_dtype = v_dtype;
  a.p = make_lif_params(v_th, v_reset, tau);
  return run(a, path, static_cast<cudaStream_t>(stream), "linear_lif");
}
