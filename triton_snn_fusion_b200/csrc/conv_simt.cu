// Dense conv (+ bias, + residual) + LIF over T on CUDA cores: an implicit GEMM with
// M = B*Ho*Wo output pixels, N = Cout, K = KH*KW*Cin (Cin innermost, matching the
// channels-last weight layout), fp32 accumulation, 64x64 tiles, 4x4 outputs per thread.
//
// This is the general path: fp32 activations (where the 1e-4 membrane tolerance rules
// out TF32), channel counts the tensor-core path does not take (e.g. the Cin=3 stem),
// and linear layers (a 1x1 conv over a [1,1,M] frame). The membrane potential of the
// thread's 16 outputs stays in registers across the T steps. When every step sees the
// same frame (x_t_stride == 0) the convolution is evaluated once and only the LIF is
// repeated.
#include "conv.cuh"

namespace snnb {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, NT = 256;

template <typename XT, typename ST, typename VT>
__global__ void __launch_bounds__(NT)
conv_lif_simt_kernel(const XT *__restrict__ x, int64_t x_t_stride, const XT *__restrict__ w,
                     const XT *__restrict__ bias, const XT *__restrict__ res,
                     const VT *__restrict__ v_init, ST *__restrict__ spikes, VT *__restrict__ v_out,
                     int T, int B, int Cin, int H, int W, int Cout, int KH, int KW, int stride, int pad,
                     int Ho, int Wo, int lif, int vec_ok, LifParams p) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int64_t M = (int64_t)B * Ho * Wo;
  const int K = KH * KW * Cin;
  const int64_t m0 = (int64_t)blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;

  // A-tile loader: this thread always fetches pixel `lm`, k offsets lk0..lk0+3
  const int lm = tid % BM;
  const int lk0 = (tid / BM) * 4;
  const int64_t gm = m0 + lm;
  const bool m_ok = gm < M;
  int hi0 = 0, wi0 = 0;
  int64_t xb = 0;
  if (m_ok) {
    const int wo = (int)(gm % Wo);
    const int ho = (int)((gm / Wo) % Ho);
    const int bb = (int)(gm / ((int64_t)Wo * Ho));
    hi0 = ho * stride - pad;
    wi0 = wo * stride - pad;
    xb = (int64_t)bb * H * W * Cin;
  }
  // B-tile loader: cout `ln`, k offsets lkb..lkb+3
  const int ln = tid / 4;
  const int lkb = (tid % 4) * 4;
  const bool n_ok = (n0 + ln) < Cout;
  const XT *wrow = w + (int64_t)(n0 + ln) * K;

  float acc[4][4];
  float v[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) v[i][j] = 0.f;

  const int64_t frame_out = M * Cout;
  if (lif && v_init != nullptr) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t m = m0 + ty * 4 + i;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (n < Cout) v[i][j] = DT<VT>::to_f(v_init[m * Cout + n]);
      }
    }
  }
  float bj[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + tx * 4 + j;
    bj[j] = (bias != nullptr && n < Cout) ? DT<XT>::to_f(bias[n]) : 0.f;
  }

  const bool alias = (x_t_stride == 0);
  for (int t = 0; t < T; ++t) {
    if (t == 0 || !alias) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
      const XT *xt = x + (int64_t)t * x_t_stride + xb;
      for (int k0 = 0; k0 < K; k0 += BK) {
        // ---- stage tiles
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + lk0 + j;
          float val = 0.f;
          if (m_ok && k < K) {
            const int ci = k % Cin;
            const int tap = k / Cin;
            const int kh = tap / KW, kw = tap % KW;
            const int hi = hi0 + kh, wi = wi0 + kw;
            if (hi >= 0 && hi < H && wi >= 0 && wi < W)
              val = DT<XT>::to_f(xt[((int64_t)hi * W + wi) * Cin + ci]);
          }
          As[lk0 + j][lm] = val;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = k0 + lkb + j;
          Bs[lkb + j][ln] = (n_ok && k < K) ? DT<XT>::to_f(wrow[k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
          const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
          const float av[4] = {a4.x, a4.y, a4.z, a4.w};
          const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
      }
    }
    // ---- epilogue for step t
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t m = m0 + ty * 4 + i;
      if (m >= M) continue;
      const int nb = n0 + tx * 4;
      const int64_t o = (int64_t)t * frame_out + m * Cout + nb;
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = acc[i][j] + bj[j];
      if (vec_ok && nb + 3 < Cout) {
        if (res != nullptr) {
          float r[4];
          load_pack<XT, 4>(res + o, r);
#pragma unroll
          for (int j = 0; j < 4; ++j) y[j] += r[j];
        }
        if (lif) {
          float s[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) s[j] = lif_step(y[j], v[i][j], p);
          store_pack<ST, 4, false>(spikes + o, s);
        } else {
          store_pack<XT, 4, false>(reinterpret_cast<XT *>(spikes) + o, y);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (nb + j >= Cout) continue;
          float yy = y[j];
          if (res != nullptr) yy += DT<XT>::to_f(res[o + j]);
          if (lif) spikes[o + j] = DT<ST>::from_f(lif_step(yy, v[i][j], p));
          else reinterpret_cast<XT *>(spikes)[o + j] = DT<XT>::from_f(yy);
        }
      }
    }
  }
  if (lif) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t m = m0 + ty * 4 + i;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (v_out != nullptr && n < Cout) v_out[m * Cout + n] = DT<VT>::from_f(v[i][j]);
      }
    }
  }
}

template <typename XT, typename ST, typename VT>
int launch(const ConvArgs &a, cudaStream_t stream) {
  const int64_t M = (int64_t)a.B * a.Ho * a.Wo;
  const int64_t gx = (M + BM - 1) / BM;
  const int gy = (a.Cout + BN - 1) / BN;
  if (gx > 0x7fffffffLL || gy > 65535) return fail(SNNB_ERR_INVALID, "conv_lif: problem too large for the grid");
  const int vec_ok = (a.Cout % 4 == 0) && aligned16(a.spikes) && (a.res == nullptr || aligned16(a.res));
  conv_lif_simt_kernel<XT, ST, VT><<<dim3((unsigned)gx, (unsigned)gy), NT, 0, stream>>>(
      static_cast<const XT *>(a.x), a.x_t_stride, static_cast<const XT *>(a.w), static_cast<const XT *>(a.b),
      static_cast<const XT *>(a.res), static_cast<const VT *>(a.v_init), static_cast<ST *>(a.spikes),
      static_cast<VT *>(a.v_out), a.T, a.B, a.Cin, a.H, a.W, a.Cout, a.KH, a.KW, a.stride, a.pad, a.Ho, a.Wo,
      a.lif, vec_ok, a.p);
  SNNB_CHECK_LAUNCH("conv_lif_simt");
  return SNNB_OK;
}

template <typename XT>
int dispatch(const ConvArgs &a, cudaStream_t stream) {
  const bool s_u8 = a.lif && a.spike_dtype == SNNB_U8;
  const bool v_f32 = a.v_dtype == SNNB_F32;
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(a, stream);
  if (s_u8) return launch<XT, uint8_t, XT>(a, stream);
  if (v_f32) return launch<XT, XT, float>(a, stream);
  return launch<XT, XT, XT>(a, stream);
}

}  // namespace

int conv_lif_simt(const ConvArgs &a, cudaStream_t stream) {
  switch (a.dtype) {
    case SNNB_F32: return dispatch<float>(a, stream);
    case SNNB_BF16: return dispatch<__nv_bfloat16>(a, stream);
    case SNNB_F16: return dispatch<__half>(a, stream);
    default: return fail(SNNB_ERR_INVALID, "conv_lif: unsupported dtype %d", a.dtype);
  }
}

}  // namespace snnb
