// 3x3 depthwise conv (+ bias, + residual) + LIF over T, channels-last.
//
// HBM-bound: per output element it needs 1 (stride 1) or 4 (stride 2) input elements,
// one spike per step and the membrane once. A thread owns VEC consecutive channels of
// a strip of S consecutive output pixels of one output row; lanes run over channels
// first, so every load/store instruction of a warp covers contiguous memory. Along the
// strip the 3x3 window slides in registers: only the new input column(s) are fetched
// for each output, the rest is reused, which keeps the load-unit traffic at ~4.5
// (stride 1) accesses per output instead of 9. The T steps are the outer loop; the S
// membrane vectors of the strip stay in registers for the whole call.
#include "common.cuh"

namespace snnb {

// shared-memory tile kernel (dwconv_tile.cu): preferred whenever it applies
bool dwconv_tile_supported(const void *x, int64_t xts, const void *res, const void *v_init, const void *spikes,
                           const void *v_out, int C, int H, int W, int dtype);
int dwconv_tile(const void *x, int64_t xts, const void *w, const void *b, const void *res, const void *v_init,
                void *spikes, void *v_out, int T, int B, int C, int H, int W, int stride, int dtype, int spike_dtype,
                int v_dtype, const LifParams &p, cudaStream_t stream);

namespace {

constexpr int NT = 128;
constexpr int S = 4;  // output pixels per thread

template <typename XT, typename ST, typename VT, int VEC, int STRIDE>
__global__ void __launch_bounds__(NT, 3)
dwconv3x3_lif_kernel(const XT *__restrict__ x, int64_t x_t_stride, const XT *__restrict__ w,
                     const XT *__restrict__ bias, const XT *__restrict__ res,
                     const VT *__restrict__ v_init, ST *__restrict__ spikes, VT *__restrict__ v_out,
                     int T, int B, int C, int H, int W, int Ho, int Wo, LifParams p) {
  const int CV = C / VEC;
  const int nstrips = (Wo + S - 1) / S;
  const int64_t total = (int64_t)B * Ho * nstrips * CV;
  int64_t idx = (int64_t)blockIdx.x * NT + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % CV);
  idx /= CV;
  const int strip = (int)(idx % nstrips);
  idx /= nstrips;
  const int ho = (int)(idx % Ho);
  const int b = (int)(idx / Ho);
  const int c0 = cv * VEC;
  const int wo0 = strip * S;

  float wr[9][VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i)
#pragma unroll
    for (int k = 0; k < 9; ++k) wr[k][i] = DT<XT>::to_f(w[(int64_t)(c0 + i) * 9 + k]);
  float bs[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) bs[i] = bias != nullptr ? DT<XT>::to_f(bias[c0 + i]) : 0.f;

  const int64_t orow = ((int64_t)b * Ho + ho) * Wo;  // first output pixel of this row
  const int64_t frame_out = (int64_t)B * Ho * Wo * C;

  float v[S][VEC];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    if (v_init != nullptr && wo0 + s < Wo) {
      load_pack_stream<VT, VEC>(v_init + (orow + wo0 + s) * C + c0, v[s]);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[s][i] = 0.f;
    }
  }

  const int hi0 = ho * STRIDE - 1;
  for (int t = 0; t < T; ++t) {
    const XT *xt = x + (int64_t)t * x_t_stride + (int64_t)b * H * W * C + c0;
    auto load_col = [&](int wi, float (&col)[3][VEC]) {
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        const int hi = hi0 + r;
        if (hi >= 0 && hi < H && wi >= 0 && wi < W) {
          load_pack<XT, VEC>(xt + ((int64_t)hi * W + wi) * C, col[r]);
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) col[r][i] = 0.f;
        }
      }
    };
    float c0v[3][VEC], c1v[3][VEC], c2v[3][VEC];
    if constexpr (STRIDE == 1) {
      load_col(wo0 - 1, c0v);
      load_col(wo0, c1v);
    } else {
      load_col(2 * wo0 - 1, c0v);
    }
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int wo = wo0 + s;
      if (wo >= Wo) break;
      if constexpr (STRIDE == 1) {
        load_col(wo + 1, c2v);
      } else {
        load_col(2 * wo, c1v);
        load_col(2 * wo + 1, c2v);
      }
      float y[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float a = 0.f;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
          a = fmaf(c0v[r][i], wr[r * 3 + 0][i], a);
          a = fmaf(c1v[r][i], wr[r * 3 + 1][i], a);
          a = fmaf(c2v[r][i], wr[r * 3 + 2][i], a);
        }
        y[i] = a + bs[i];
      }
      const int64_t o = (int64_t)t * frame_out + (orow + wo) * C + c0;
      if (res != nullptr) {
        float rr[VEC];
        load_pack<XT, VEC>(res + o, rr);
#pragma unroll
        for (int i = 0; i < VEC; ++i) y[i] += rr[i];
      }
      float sp[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) sp[i] = lif_step(y[i], v[s][i], p);
      store_pack<ST, VEC>(spikes + o, sp);
      // slide the window
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          if constexpr (STRIDE == 1) {
            c0v[r][i] = c1v[r][i];
            c1v[r][i] = c2v[r][i];
          } else {
            c0v[r][i] = c2v[r][i];
          }
        }
    }
  }
#pragma unroll
  for (int s = 0; s < S; ++s)
    if (wo0 + s < Wo) store_pack<VT, VEC>(v_out + (orow + wo0 + s) * C + c0, v[s]);
}

// Fast path: 4 channels per thread (a warp's load covers 32 x 4 consecutive channels), a strip of SS
// output pixels, and per timestep ALL window loads of the strip issued before the first use, with the
// loads of step t+1 in flight while step t is evaluated. Bounds, offsets and the LIF flavour are
// resolved once per thread / at compile time; the window stays packed (16-bit) until it is used.
template <typename XT> struct Raw4 { using type = uint2; };        // four 16-bit values
template <> struct Raw4<float> { using type = uint4; };            // four fp32 values

template <typename XT>
__device__ __forceinline__ void unpack4(const typename Raw4<XT>::type &r, float (&f)[4]) {
  if constexpr (sizeof(XT) == 4) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  } else {
    const XT *h = reinterpret_cast<const XT *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = DT<XT>::to_f(h[i]);
  }
}

template <typename XT, typename ST, typename VT, int STRIDE, bool FAST>
__global__ void __launch_bounds__(NT, 3)
dwconv3x3_lif_fast_kernel(const XT *__restrict__ x, int64_t x_t_stride, const XT *__restrict__ w,
                          const XT *__restrict__ bias, const XT *__restrict__ res,
                          const VT *__restrict__ v_init, ST *__restrict__ spikes, VT *__restrict__ v_out,
                          int T, int B, int C, int H, int W, int Ho, int Wo, LifParams p) {
  using Raw = typename Raw4<XT>::type;
  constexpr int SS = STRIDE == 1 ? 4 : 2;                  // output pixels per thread
  constexpr int NCOL = STRIDE == 1 ? SS + 2 : 2 * SS + 1;  // input columns the strip touches
  const int CV = C / 4;
  const int nstrips = (Wo + SS - 1) / SS;
  const int64_t total = (int64_t)B * Ho * nstrips * CV;
  int64_t idx = (int64_t)blockIdx.x * NT + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % CV);
  idx /= CV;
  const int strip = (int)(idx % nstrips);
  idx /= nstrips;
  const int ho = (int)(idx % Ho);
  const int b = (int)(idx / Ho);
  const int c0 = cv * 4;
  const int wo0 = strip * SS;

  float wr[9][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int k = 0; k < 9; ++k) wr[k][i] = DT<XT>::to_f(w[(int64_t)(c0 + i) * 9 + k]);
  float bs[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) bs[i] = bias != nullptr ? DT<XT>::to_f(bias[c0 + i]) : 0.f;

  // window geometry, fixed for the whole call: element offsets inside a frame and validity bits
  const int hi0 = ho * STRIDE - 1, wi0 = wo0 * STRIDE - 1;
  unsigned ok_bits = 0;
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int j = 0; j < NCOL; ++j) {
      const int hi = hi0 + r, wi = wi0 + j;
      const bool ok = hi >= 0 && hi < H && wi >= 0 && wi < W;
      if (ok) ok_bits |= 1u << (r * NCOL + j);
    }
  const int off0 = (hi0 * W + wi0) * C, row_step = W * C;   // offset of window element (r, j): off0 + r * row_step + j * C
  const XT *xb = x + (int64_t)b * H * W * C + c0;
  auto load_window = [&](int t, Raw (&win)[3][NCOL]) {
    const XT *xt = xb + (int64_t)t * x_t_stride;
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int j = 0; j < NCOL; ++j) {
        if ((ok_bits >> (r * NCOL + j)) & 1u) win[r][j] = __ldg(reinterpret_cast<const Raw *>(xt + (off0 + r * row_step + j * C)));
        else win[r][j] = Raw{};
      }
  };

  const int64_t orow = ((int64_t)b * Ho + ho) * Wo;
  const int64_t frame_out = (int64_t)B * Ho * Wo * C;
  float v[SS][4];
#pragma unroll
  for (int s = 0; s < SS; ++s) {
    if (v_init != nullptr && wo0 + s < Wo) {
      load_pack_stream<VT, 4>(v_init + (orow + wo0 + s) * C + c0, v[s]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) v[s][i] = 0.f;
    }
  }

  // 16-bit data: the window of step t+1 is fetched while step t is evaluated (fp32 windows are too
  // large to hold twice)
  constexpr bool PF = sizeof(XT) == 2;
  Raw cur[3][NCOL], nxt[PF ? 3 : 1][PF ? NCOL : 1];
  load_window(0, cur);
#pragma unroll 1
  for (int t = 0; t < T; ++t) {
    if constexpr (PF) {
      if (t + 1 < T) load_window(t + 1, nxt);
    }
    // column by column: a window column is unpacked once and feeds every output of the strip that
    // touches it, so only one column of fp32 values is live besides the accumulators
    float y[SS][4];
#pragma unroll
    for (int s = 0; s < SS; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i) y[s][i] = bs[i];
#pragma unroll
    for (int j = 0; j < NCOL; ++j) {
      float f[3][4];
#pragma unroll
      for (int r = 0; r < 3; ++r) unpack4<XT>(cur[r][j], f[r]);
#pragma unroll
      for (int s = 0; s < SS; ++s) {
        const int k = j - s * STRIDE;
        if (k >= 0 && k < 3) {
#pragma unroll
          for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i) y[s][i] = fmaf(f[r][i], wr[r * 3 + k][i], y[s][i]);
        }
      }
    }
#pragma unroll
    for (int s = 0; s < SS; ++s) {
      if (wo0 + s < Wo) {
        const int64_t o = (int64_t)t * frame_out + (orow + wo0 + s) * C + c0;
        if (res != nullptr) {
          float rr[4];
          load_pack<XT, 4>(res + o, rr);
#pragma unroll
          for (int i = 0; i < 4; ++i) y[s][i] += rr[i];
        }
        float sp[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) sp[i] = FAST ? lif_step_t<1, true>(y[s][i], v[s][i], p) : lif_step(y[s][i], v[s][i], p);
        store_pack<ST, 4>(spikes + o, sp);
      }
    }
    if constexpr (PF) {
#pragma unroll
      for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int j = 0; j < NCOL; ++j) cur[r][j] = nxt[r][j];
    } else {
      if (t + 1 < T) load_window(t + 1, cur);
    }
  }
#pragma unroll
  for (int s = 0; s < SS; ++s)
    if (wo0 + s < Wo) store_pack<VT, 4>(v_out + (orow + wo0 + s) * C + c0, v[s]);
}

template <typename XT, typename ST, typename VT>
int launch(const void *x, int64_t xts, const void *w, const void *b, const void *res, const void *v_init,
           void *spikes, void *v_out, int T, int B, int C, int H, int W, int stride, const LifParams &p,
           cudaStream_t stream) {
  const int Ho = (H + 2 - 3) / stride + 1;
  const int Wo = (W + 2 - 3) / stride + 1;
  const int nstrips = (Wo + S - 1) / S;
  const bool vec = (C % 4 == 0) && aligned16(x) && aligned16(spikes) && aligned16(v_out) &&
                   (v_init == nullptr || aligned16(v_init)) && (res == nullptr || aligned16(res)) &&
                   (xts % 4 == 0);
  const int VEC = vec ? 4 : 1;
  // the fast kernel keeps 32-bit element offsets inside one image
  if (vec && (int64_t)H * W * C < 0x7fffffffLL) {
    const int SS = stride == 1 ? 4 : 2;
    const int64_t tot = (int64_t)B * Ho * ((Wo + SS - 1) / SS) * (C / 4);
    const int64_t nb = (tot + NT - 1) / NT;
    if (nb > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "dwconv3x3_lif: problem too large");
    const bool fast = p.mode == 1 && p.hard;
#define SNNB_DWF(STR, FAST)                                                                            \
  dwconv3x3_lif_fast_kernel<XT, ST, VT, STR, FAST><<<(unsigned)nb, NT, 0, stream>>>(                  \
      static_cast<const XT *>(x), xts, static_cast<const XT *>(w), static_cast<const XT *>(b),         \
      static_cast<const XT *>(res), static_cast<const VT *>(v_init), static_cast<ST *>(spikes),        \
      static_cast<VT *>(v_out), T, B, C, H, W, Ho, Wo, p)
    if (stride == 1) { if (fast) SNNB_DWF(1, true); else SNNB_DWF(1, false); }
    else { if (fast) SNNB_DWF(2, true); else SNNB_DWF(2, false); }
#undef SNNB_DWF
    SNNB_CHECK_LAUNCH("dwconv3x3_lif");
    return SNNB_OK;
  }
  const int64_t total = (int64_t)B * Ho * nstrips * (C / VEC);
  const int64_t blocks = (total + NT - 1) / NT;
  if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "dwconv3x3_lif: problem too large");
#define SNNB_DW(VECN, STR)                                                                             \
  dwconv3x3_lif_kernel<XT, ST, VT, VECN, STR><<<(unsigned)blocks, NT, 0, stream>>>(                    \
      static_cast<const XT *>(x), xts, static_cast<const XT *>(w), static_cast<const XT *>(b),         \
      static_cast<const XT *>(res), static_cast<const VT *>(v_init), static_cast<ST *>(spikes),        \
      static_cast<VT *>(v_out), T, B, C, H, W, Ho, Wo, p)
  if (vec) {
    if (stride == 1) SNNB_DW(4, 1); else SNNB_DW(4, 2);
  } else {
    if (stride == 1) SNNB_DW(1, 1); else SNNB_DW(1, 2);
  }
#undef SNNB_DW
  SNNB_CHECK_LAUNCH("dwconv3x3_lif");
  return SNNB_OK;
}

template <typename XT>
int dispatch(const void *x, int64_t xts, const void *w, const void *b, const void *res, const void *v_init,
             void *spikes, void *v_out, int T, int B, int C, int H, int W, int stride, int spike_dtype,
             int v_dtype, const LifParams &p, cudaStream_t stream) {
  const bool s_u8 = spike_dtype == SNNB_U8;
  const bool v_f32 = v_dtype == SNNB_F32;
#define SNNB_ARGS x, xts, w, b, res, v_init, spikes, v_out, T, B, C, H, W, stride, p, stream
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(SNNB_ARGS);
  if (s_u8) return launch<XT, uint8_t, XT>(SNNB_ARGS);
  if (v_f32) return launch<XT, XT, float>(SNNB_ARGS);
  return launch<XT, XT, XT>(SNNB_ARGS);
#undef SNNB_ARGS
}

}  // namespace
}  // namespace snnb

extern "C" int snnb_dwconv3x3_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                                  const void *residual, const void *v_init, void *spikes, void *v_out,
                                  int T, int B, int C, int H, int W, int stride,
                                  int dtype, int spike_dtype, int v_dtype,
                                  float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && w && spikes && v_out, "dwconv3x3_lif: null pointer");
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && C >= 1 && H >= 1 && W >= 1, "dwconv3x3_lif: sizes must be positive");
  SNNB_CHECK_ARG(stride == 1 || stride == 2, "dwconv3x3_lif: unsupported_stride: stride must be 1 or 2, got %d", stride);
  SNNB_CHECK_ARG(is_act_dtype(dtype), "dwconv3x3_lif: unsupported dtype %d", dtype);
  SNNB_CHECK_ARG(spike_dtype == dtype || spike_dtype == SNNB_U8, "dwconv3x3_lif: spike dtype must be the x dtype or u8");
  SNNB_CHECK_ARG(v_dtype == dtype || v_dtype == SNNB_F32, "dwconv3x3_lif: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(x_t_stride >= 0, "dwconv3x3_lif: negative frame stride");
  SNNB_CHECK_ARG(tau != 0.0f, "dwconv3x3_lif: unsupported_tau: tau must be nonzero");
  const LifParams p = make_lif_params(v_th, v_reset, tau);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (v_init != nullptr && v_init != v_out) {
    const size_t bytes = (size_t)B * ((H - 1) / stride + 1) * ((W - 1) / stride + 1) * C * dtype_size(v_dtype);
    const char *pi = static_cast<const char *>(v_init), *po = static_cast<const char *>(v_out);
    SNNB_CHECK_ARG(!(pi < po + bytes && po < pi + bytes), "dwconv3x3_lif: v_init and v_out overlap without being the same buffer");
  }
  if (dwconv_tile_supported(x_seq, x_t_stride, residual, v_init, spikes, v_out, C, H, W, dtype))
    return dwconv_tile(x_seq, x_t_stride, w, b, residual, v_init, spikes, v_out, T, B, C, H, W, stride, dtype, spike_dtype,
                       v_dtype, p, s);
#define SNNB_ARGS x_seq, x_t_stride, w, b, residual, v_init, spikes, v_out, T, B, C, H, W, stride, spike_dtype, v_dtype, p, s
  switch (dtype) {
    case SNNB_F32: return dispatch<float>(SNNB_ARGS);
    case SNNB_BF16: return dispatch<__nv_bfloat16>(SNNB_ARGS);
    default: return dispatch<__half>(SNNB_ARGS);
  }
#undef SNNB_ARGS
}
