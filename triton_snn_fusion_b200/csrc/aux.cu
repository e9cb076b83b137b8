// Stateless channels-last helpers around the fused ops: layout transposes, the 3x3/s2
// max pool after a ResNet stem, and the avgpool + linear head averaged over T.
#include "common.cuh"

namespace snnb {
namespace {

// [frames][R][Ccols] -> [frames][Ccols][R] for 2- or 4-byte elements (32x32 smem tiles).
template <typename E>
__global__ void transpose_kernel(const E *__restrict__ src, E *__restrict__ dst, int R, int Cc) {
  __shared__ E tile[32][33];
  const int64_t f = blockIdx.z;
  const E *s = src + f * (int64_t)R * Cc;
  E *d = dst + f * (int64_t)R * Cc;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < R && c < Cc) tile[i][threadIdx.x] = s[(int64_t)r * Cc + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < R && c < Cc) d[(int64_t)c * R + r] = tile[threadIdx.x][i];
  }
}

int transpose(const void *src, void *dst, int64_t frames, int R, int Cc, int dtype, cudaStream_t st, const char *what) {
  if (!src || !dst) return fail(SNNB_ERR_INVALID, "%s: null pointer", what);
  if (frames < 0 || R < 1 || Cc < 1) return fail(SNNB_ERR_INVALID, "%s: bad sizes", what);
  if (!is_act_dtype(dtype) && dtype != SNNB_U8) return fail(SNNB_ERR_INVALID, "%s: unsupported dtype", what);
  if (frames == 0) return SNNB_OK;
  const dim3 block(32, 8);
  const unsigned gx = (Cc + 31) / 32, gy = (R + 31) / 32;
  for (int64_t f0 = 0; f0 < frames; f0 += 65535) {
    const unsigned nf = (unsigned)((frames - f0) < 65535 ? (frames - f0) : 65535);
    const dim3 grid(gx, gy, nf);
    const int64_t off = f0 * (int64_t)R * Cc;
    const int es = dtype_size(dtype);
    if (es == 4) transpose_kernel<uint32_t><<<grid, block, 0, st>>>(static_cast<const uint32_t *>(src) + off, static_cast<uint32_t *>(dst) + off, R, Cc);
    else if (es == 2) transpose_kernel<uint16_t><<<grid, block, 0, st>>>(static_cast<const uint16_t *>(src) + off, static_cast<uint16_t *>(dst) + off, R, Cc);
    else transpose_kernel<uint8_t><<<grid, block, 0, st>>>(static_cast<const uint8_t *>(src) + off, static_cast<uint8_t *>(dst) + off, R, Cc);
  }
  SNNB_CHECK_LAUNCH(what);
  return SNNB_OK;
}

template <typename XT, int VEC>
__global__ void __launch_bounds__(256)
maxpool3x3s2_kernel(const XT *__restrict__ x, XT *__restrict__ y, int64_t frames, int H, int W, int C, int Ho, int Wo) {
  const int CV = C / VEC;
  const int64_t total = frames * Ho * Wo * CV;
  int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % CV); idx /= CV;
  const int wo = (int)(idx % Wo); idx /= Wo;
  const int ho = (int)(idx % Ho);
  const int64_t f = idx / Ho;
  float m[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) m[i] = -INFINITY;
  const XT *xf = x + f * (int64_t)H * W * C + cv * VEC;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const int hi = ho * 2 - 1 + r;
    if (hi < 0 || hi >= H) continue;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const int wi = wo * 2 - 1 + c;
      if (wi < 0 || wi >= W) continue;
      float v[VEC];
      load_pack<XT, VEC>(xf + ((int64_t)hi * W + wi) * C, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) m[i] = fmaxf(m[i], v[i]);
    }
  }
  store_pack<XT, VEC, false>(y + ((f * Ho + ho) * (int64_t)Wo + wo) * C + cv * VEC, m);
}

template <typename XT>
int maxpool(const void *x, void *y, int64_t frames, int H, int W, int C, cudaStream_t st) {
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  constexpr int V = 16 / sizeof(XT);
  const bool vec = (C % V == 0) && aligned16(x) && aligned16(y);
  const int64_t total = frames * Ho * Wo * (vec ? C / V : C);
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "maxpool3x3s2: problem too large");
  if (blocks == 0) return SNNB_OK;
  if (vec) maxpool3x3s2_kernel<XT, V><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const XT *>(x), static_cast<XT *>(y), frames, H, W, C, Ho, Wo);
  else maxpool3x3s2_kernel<XT, 1><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const XT *>(x), static_cast<XT *>(y), frames, H, W, C, Ho, Wo);
  SNNB_CHECK_LAUNCH("maxpool3x3s2");
  return SNNB_OK;
}

// The same pooling over one-byte spikes (0 / 1), written out in the activation dtype: a thread owns
// 16 channels of one output pixel (16 bytes in, 32 bytes out for 16-bit activations). Bytes are
// combined with a per-byte unsigned max, four at a time.
template <typename XT>
__global__ void __launch_bounds__(256)
maxpool3x3s2_u8_kernel(const uint8_t *__restrict__ x, XT *__restrict__ y, int64_t frames, int H, int W, int C, int Ho, int Wo) {
  const int CV = C / 16;
  const int64_t total = frames * Ho * Wo * CV;
  int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total) return;
  const int cv = (int)(idx % CV); idx /= CV;
  const int wo = (int)(idx % Wo); idx /= Wo;
  const int ho = (int)(idx % Ho);
  const int64_t f = idx / Ho;
  uint4 m = make_uint4(0u, 0u, 0u, 0u);
  const uint8_t *xf = x + f * (int64_t)H * W * C + cv * 16;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const int hi = ho * 2 - 1 + r;
    if (hi < 0 || hi >= H) continue;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const int wi = wo * 2 - 1 + c;
      if (wi < 0 || wi >= W) continue;
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(xf + ((int64_t)hi * W + wi) * C));
      m.x = __vmaxu4(m.x, v.x); m.y = __vmaxu4(m.y, v.y); m.z = __vmaxu4(m.z, v.z); m.w = __vmaxu4(m.w, v.w);
    }
  }
  const uint32_t words[4] = {m.x, m.y, m.z, m.w};
  float out[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) out[i] = (float)((words[i >> 2] >> ((i & 3) * 8)) & 0xffu);
  store_pack<XT, 16, false>(y + ((f * Ho + ho) * (int64_t)Wo + wo) * C + cv * 16, out);
}

// 3x3 / stride 2 / padding 1 max-pool of bit-packed spikes: the max of 0 / 1 values is the OR of the words.
// A thread ORs the nine 64-bit words (64 channels) of one output pixel: a warp's load covers 32 neighbouring
// pixels, i.e. a few contiguous lines. The 64 results of a pixel are 128 bytes of 16-bit output, so the warp then
// writes its 32 pixels as 4096 contiguous bytes in eight fully coalesced 16-byte-per-lane stores, each lane
// fetching the eight bits it needs from the lane that owns the pixel (two shuffles per store). Spikes are written
// as the bit patterns of 0.0 / 1.0 directly; all index arithmetic is 32-bit.
template <typename XT> struct OneBits;
template <> struct OneBits<__nv_bfloat16> { static constexpr uint32_t v = 0x3F80u; };
template <> struct OneBits<__half> { static constexpr uint32_t v = 0x3C00u; };

template <typename XT>
__global__ void __launch_bounds__(256)
maxpool3x3s2_bits_kernel(const uint2 *__restrict__ x, XT *__restrict__ y, unsigned npix, int H, int W, int G, int Ho, int Wo) {
  // x: [frames][H][W][G] 64-bit words (G = C / 64 channel groups); y: [frames][Ho][Wo][C]; blockIdx.y = channel group
  const int g = blockIdx.y;
  const unsigned pix = blockIdx.x * 256u + threadIdx.x;     // this thread's output pixel (frame, ho, wo) flattened
  const unsigned pc = pix < npix ? pix : npix - 1;          // lanes past the end repeat the last pixel and store nothing
  const int wo = (int)(pc % (unsigned)Wo);
  const unsigned fr = pc / (unsigned)Wo;
  const int ho = (int)(fr % (unsigned)Ho);
  const unsigned f = fr / (unsigned)Ho;
  uint32_t lo = 0u, hi = 0u;
  const uint2 *xf = x + (size_t)f * H * W * G + g;
#pragma unroll
  for (int r = 0; r < 3; ++r) {
    const int hi_ = ho * 2 - 1 + r;
    if (hi_ < 0 || hi_ >= H) continue;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      const int wi = wo * 2 - 1 + c;
      if (wi < 0 || wi >= W) continue;
      const uint2 v = __ldg(xf + (size_t)(hi_ * W + wi) * G);
      lo |= v.x;
      hi |= v.y;
    }
  }
  const int lane = threadIdx.x & 31;
  const unsigned warp_pix0 = pix - (unsigned)lane;          // first pixel of this warp
  const int C = G * 64;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    // store k of the warp: lane L writes channels 8 * (L % 8) .. + 7 of pixel warp_pix0 + 4 * k + L / 8
    const int src = 4 * k + (lane >> 3);
    const uint32_t wl = __shfl_sync(0xffffffffu, lo, src), wh = __shfl_sync(0xffffffffu, hi, src);
    const uint32_t m = (((lane & 4) ? wh : wl) >> ((lane & 3) * 8)) & 0xffu;
    const unsigned p = warp_pix0 + (unsigned)src;
    if (p < npix) {
      XT *dst = y + (size_t)p * C + g * 64 + (lane & 7) * 8;
      if constexpr (sizeof(XT) == 2) {
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          o[i] = ((m >> (2 * i)) & 1u) * OneBits<XT>::v | ((m >> (2 * i + 1)) & 1u) * (OneBits<XT>::v << 16);
        *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
#pragma unroll
        for (int i = 0; i < 2; ++i)
          *reinterpret_cast<float4 *>(dst + 4 * i) = make_float4(((m >> (4 * i)) & 1u) ? 1.f : 0.f, ((m >> (4 * i + 1)) & 1u) ? 1.f : 0.f,
                                                                  ((m >> (4 * i + 2)) & 1u) ? 1.f : 0.f, ((m >> (4 * i + 3)) & 1u) ? 1.f : 0.f);
      }
    }
  }
}

// One CTA per (group of SB samples, chunk of classes): channel sums over (t, pixel) into shared memory,
// then a warp-per-class mat-vec for the SB samples with the fc row read once. The sums are cheap and
// latency-bound (T*HW strided rows per channel), so the threads of a CTA split the pixels as well as
// the channels (16 bytes of channels per load, PG pixel groups whose partial sums are added in a fixed
// order), and CTAs that differ only in their class chunk simply repeat them.
constexpr int SB = 2;
template <typename XT>
__global__ void __launch_bounds__(256)
avgpool_linear_mean_kernel(const XT *__restrict__ x, const XT *__restrict__ w, const XT *__restrict__ b,
                           float *__restrict__ out, int T, int N, int C, int HW, int K, int Kc, int PG, int vec) {
  extern __shared__ float sums[];  // [PG][SB][C]
  constexpr int V = 16 / sizeof(XT);
  const int n0 = blockIdx.x * SB;
  const int ns = min(SB, N - n0);
  const int tid = threadIdx.x;
  const int64_t frame = (int64_t)N * HW * C;
  if (vec) {
    const int groups = C / V, rows = T * HW;
    for (int item = tid; item < ns * PG * groups; item += 256) {
      const int cg = item % groups;
      const int pg = (item / groups) % PG;
      const int s = item / (groups * PG);
      const XT *px = x + (int64_t)(n0 + s) * HW * C + cg * V;
      float acc[4][V];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < V; ++i) acc[u][i] = 0.f;
      for (int q0 = pg; q0 < rows; q0 += 4 * PG) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {   // four independent rows in flight
          const int q = q0 + u * PG;
          if (q < rows) {
            const int t = q / HW, pp = q - t * HW;
            float v[V];
            load_pack<XT, V>(px + (int64_t)t * frame + (int64_t)pp * C, v);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[u][i] += v[i];
          }
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) sums[(pg * SB + s) * C + cg * V + i] = (acc[0][i] + acc[1][i]) + (acc[2][i] + acc[3][i]);
    }
  } else {
    for (int i = tid; i < ns * C; i += 256) {
      const int s = i / C, c = i % C;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      for (int t = 0; t < T; ++t) {
        const XT *px = x + (int64_t)t * frame + (int64_t)(n0 + s) * HW * C + c;
        int pp = 0;
        for (; pp + 4 <= HW; pp += 4) {
          a0 += DT<XT>::to_f(px[(int64_t)pp * C]);
          a1 += DT<XT>::to_f(px[(int64_t)(pp + 1) * C]);
          a2 += DT<XT>::to_f(px[(int64_t)(pp + 2) * C]);
          a3 += DT<XT>::to_f(px[(int64_t)(pp + 3) * C]);
        }
        for (; pp < HW; ++pp) a0 += DT<XT>::to_f(px[(int64_t)pp * C]);
      }
      sums[s * C + c] = (a0 + a1) + (a2 + a3);
    }
  }
  __syncthreads();
  if (vec && PG > 1) {
    for (int i = tid; i < ns * C; i += 256) {
      float a = sums[i];
      for (int pg = 1; pg < PG; ++pg) a += sums[pg * SB * C + i];
      sums[i] = a;
    }
    __syncthreads();
  }
  const int warp = tid / 32, lane = tid % 32;
  const float scale = 1.0f / ((float)T * (float)HW);
  const int k_end = min(K, (int)(blockIdx.y + 1) * Kc);
  for (int k = blockIdx.y * Kc + warp; k < k_end; k += 8) {
    float acc[SB];
#pragma unroll
    for (int s = 0; s < SB; ++s) acc[s] = 0.f;
    const XT *wk = w + (int64_t)k * C;
    for (int c = lane; c < C; c += 32) {
      const float wv = DT<XT>::to_f(wk[c]);
#pragma unroll
      for (int s = 0; s < SB; ++s)
        if (s < ns) acc[s] = fmaf(wv, sums[s * C + c], acc[s]);
    }
    const float bk = b != nullptr ? DT<XT>::to_f(b[k]) : 0.f;
#pragma unroll
    for (int s = 0; s < SB; ++s) {
      float a = acc[s];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (lane == 0 && s < ns) out[(int64_t)(n0 + s) * K + k] = a * scale + bk;
    }
  }
}

template <typename XT>
int head(const void *x, const void *w, const void *b, float *out, int T, int N, int C, int HW, int K, cudaStream_t st) {
  if ((size_t)SB * C * sizeof(float) > 48 * 1024) return fail(SNNB_ERR_UNSUPPORTED, "avgpool_linear_mean: C=%d too large", C);
  constexpr int V = 16 / sizeof(XT);
  const int vec = (C % V == 0 && aligned16(x)) ? 1 : 0;
  int PG = 1;   // pixel groups: fill the 256 threads, within 48 KB of partial sums
  if (vec) {
    PG = 256 / (C / V) > 1 ? 256 / (C / V) : 1;
    if (PG > 8) PG = 8;
    while (PG > 1 && (size_t)PG * SB * C * sizeof(float) > 48 * 1024) --PG;
  }
  const int gx = (N + SB - 1) / SB;
  const int sms = sm_count() > 0 ? sm_count() : 128;
  int ks = (2 * sms + gx - 1) / gx;   // class chunks: about two CTAs per SM in flight
  ks = ks < 1 ? 1 : (ks > 8 ? 8 : ks);
  const int Kc = (K + ks - 1) / ks;
  const size_t smem = (size_t)PG * SB * C * sizeof(float);
  avgpool_linear_mean_kernel<XT><<<dim3((unsigned)gx, (unsigned)((K + Kc - 1) / Kc)), 256, smem, st>>>(
      static_cast<const XT *>(x), static_cast<const XT *>(w), static_cast<const XT *>(b), out, T, N, C, HW, K, Kc, PG, vec);
  SNNB_CHECK_LAUNCH("avgpool_linear_mean");
  return SNNB_OK;
}

}  // namespace
}  // namespace snnb

extern "C" int snnb_nchw_to_nhwc(const void *src, void *dst, int64_t frames, int C, int HW, int dtype, void *stream) {
  return snnb::transpose(src, dst, frames, C, HW, dtype, static_cast<cudaStream_t>(stream), "nchw_to_nhwc");
}

extern "C" int snnb_nhwc_to_nchw(const void *src, void *dst, int64_t frames, int C, int HW, int dtype, void *stream) {
  return snnb::transpose(src, dst, frames, HW, C, dtype, static_cast<cudaStream_t>(stream), "nhwc_to_nchw");
}

extern "C" int snnb_maxpool3x3s2(const void *x, void *y, int64_t frames, int H, int W, int C, int dtype, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x && y, "maxpool3x3s2: null pointer");
  SNNB_CHECK_ARG(frames >= 0 && H >= 1 && W >= 1 && C >= 1, "maxpool3x3s2: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SNNB_F32: return maxpool<float>(x, y, frames, H, W, C, st);
    case SNNB_BF16: return maxpool<__nv_bfloat16>(x, y, frames, H, W, C, st);
    case SNNB_F16: return maxpool<__half>(x, y, frames, H, W, C, st);
    default: return fail(SNNB_ERR_INVALID, "maxpool3x3s2: unsupported dtype %d", dtype);
  }
}

extern "C" int snnb_maxpool3x3s2_u8(const void *x, void *y, int64_t frames, int H, int W, int C, int out_dtype, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x && y, "maxpool3x3s2_u8: null pointer");
  SNNB_CHECK_ARG(frames >= 0 && H >= 1 && W >= 1 && C >= 16 && C % 16 == 0, "maxpool3x3s2_u8: bad sizes (C must be a multiple of 16)");
  SNNB_CHECK_ARG(is_act_dtype(out_dtype), "maxpool3x3s2_u8: unsupported output dtype %d", out_dtype);
  SNNB_CHECK_ARG(aligned16(x) && aligned16(y), "maxpool3x3s2_u8: buffers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  const int64_t total = frames * Ho * Wo * (C / 16);
  const int64_t blocks = (total + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "maxpool3x3s2_u8: problem too large");
  if (blocks == 0) return SNNB_OK;
  const uint8_t *xs = static_cast<const uint8_t *>(x);
  if (out_dtype == SNNB_F32) maxpool3x3s2_u8_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(xs, static_cast<float *>(y), frames, H, W, C, Ho, Wo);
  else if (out_dtype == SNNB_BF16) maxpool3x3s2_u8_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(xs, static_cast<__nv_bfloat16 *>(y), frames, H, W, C, Ho, Wo);
  else maxpool3x3s2_u8_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(xs, static_cast<__half *>(y), frames, H, W, C, Ho, Wo);
  SNNB_CHECK_LAUNCH("maxpool3x3s2_u8");
  return SNNB_OK;
}

extern "C" int snnb_maxpool3x3s2_bits(const void *x, void *y, int64_t frames, int H, int W, int C, int out_dtype, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x && y, "maxpool3x3s2_bits: null pointer");
  SNNB_CHECK_ARG(frames >= 0 && H >= 1 && W >= 1 && C >= 64 && C % 64 == 0, "maxpool3x3s2_bits: bad sizes (C must be a multiple of 64)");
  SNNB_CHECK_ARG(is_act_dtype(out_dtype), "maxpool3x3s2_bits: unsupported output dtype %d", out_dtype);
  SNNB_CHECK_ARG(aligned16(x) && aligned16(y), "maxpool3x3s2_bits: buffers must be 16-byte aligned");
  const int Ho = (H - 1) / 2 + 1, Wo = (W - 1) / 2 + 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t npix = frames * Ho * Wo;
  if (npix >= (1LL << 31)) return fail(SNNB_ERR_INVALID, "maxpool3x3s2_bits: problem too large");
  if (npix == 0) return SNNB_OK;
  const dim3 grid((unsigned)((npix + 255) / 256), (unsigned)(C / 64));
  const uint2 *xs = static_cast<const uint2 *>(x);
  if (out_dtype == SNNB_F32) maxpool3x3s2_bits_kernel<float><<<grid, 256, 0, st>>>(xs, static_cast<float *>(y), (unsigned)npix, H, W, C / 64, Ho, Wo);
  else if (out_dtype == SNNB_BF16) maxpool3x3s2_bits_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(xs, static_cast<__nv_bfloat16 *>(y), (unsigned)npix, H, W, C / 64, Ho, Wo);
  else maxpool3x3s2_bits_kernel<__half><<<grid, 256, 0, st>>>(xs, static_cast<__half *>(y), (unsigned)npix, H, W, C / 64, Ho, Wo);
  SNNB_CHECK_LAUNCH("maxpool3x3s2_bits");
  return SNNB_OK;
}

extern "C" int snnb_avgpool_linear_mean(const void *x_seq, const void *fc_w, const void *fc_b, float *out,
                                        int T, int N, int C, int HW, int K, int dtype, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && fc_w && out, "avgpool_linear_mean: null pointer");
  SNNB_CHECK_ARG(T >= 1 && N >= 1 && C >= 1 && HW >= 1 && K >= 1, "avgpool_linear_mean: sizes must be positive");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case SNNB_F32: return head<float>(x_seq, fc_w, fc_b, out, T, N, C, HW, K, st);
    case SNNB_BF16: {
      bool taken = false;
      const int rc = head_pool_linear_bf16(x_seq, fc_w, fc_b, out, T, N, C, HW, K, st, &taken);
      if (taken || rc != SNNB_OK) return rc;
      return head<__nv_bfloat16>(x_seq, fc_w, fc_b, out, T, N, C, HW, K, st);
    }
    case SNNB_F16: return head<__half>(x_seq, fc_w, fc_b, out, T, N, C, HW, K, st);
    default: return fail(SNNB_ERR_INVALID, "avgpool_linear_mean: unsupported dtype %d", dtype);
  }
}
