// 7x7 / stride 2 / padding 3 stem conv (3 input channels) + folded BN + LIF on the tensor cores.
//
// A 3-channel image cannot feed 64-channel TMA rows directly, so the input is first re-laid
// ("space to depth"): every 2x2 pixel block becomes one 16-channel pixel (12 real values + 4
// zeros), with a 2-block zero border on the top/left and 1 on the bottom/right. In that layout
// the 7x7/s2 window of an output pixel is 4 block-rows of 4 consecutive blocks, i.e. 4 runs of
// 64 contiguous values — exactly the 128-byte rows the implicit-GEMM kernel consumes. The conv
// becomes a GEMM with K = 4 x 64 (49*3 = 147 real taps, the rest multiply zero weights) read
// through a tensor map whose "pixel" stride is one block (32 bytes): overlapping windows.
// The re-laid image lives in caller-provided scratch memory.
#include <mutex>

#include "conv.cuh"

// Built-in scratch for snnb_stem7x7_lif_static: lives in every GPU's memory from the moment the
// library is loaded there until the process exits.
#define SNNB_STEM_STATIC_SCRATCH_BYTES (16 * 1024 * 1024)
static __device__ __align__(256) unsigned char g_stem_static_scratch[SNNB_STEM_STATIC_SCRATCH_BYTES];

namespace snnb {
namespace {

// x [B][H][W][3] -> s [B][H/2+3][W/2+3][16], zero padded. One thread per 2x2 block of pixels: the block's two image
// rows are 12 contiguous bytes each (two pixels x three 16-bit channels, 4-byte aligned because W is even), read as
// three 32-bit words, and leave as the block's 32 bytes: channel (dr * 2 + dc) * 3 + c for c < 3, four zero channels.
template <typename XT>
__global__ void __launch_bounds__(256)
stem_s2d_kernel(const XT *__restrict__ x, XT *__restrict__ s, int B, int H, int W) {
  const int Hb = H / 2 + 3, Wb = W / 2 + 3;
  const long long total = (long long)B * Hb * Wb;
  long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  if (idx >= total) return;
  const long long out_idx = idx;
  const int bw = (int)(idx % Wb);
  idx /= Wb;
  const int bh = (int)(idx % Hb);
  const long long b = idx / Hb;
  uint32_t r0[3] = {0u, 0u, 0u}, r1[3] = {0u, 0u, 0u};
  const int ph = bh - 2, pw = bw - 2;  // block coordinates in the image
  if (ph >= 0 && ph < H / 2 && pw >= 0 && pw < W / 2) {
    const uint32_t *p0 = reinterpret_cast<const uint32_t *>(x + ((b * H + 2 * ph) * W + 2 * pw) * 3);
    const uint32_t *p1 = reinterpret_cast<const uint32_t *>(x + ((b * H + 2 * ph + 1) * W + 2 * pw) * 3);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      r0[i] = __ldg(p0 + i);
      r1[i] = __ldg(p1 + i);
    }
  }
  // 16-bit channels 0..5 = row 0 (pixel 0: c0 c1 c2, pixel 1: c0 c1 c2), 6..11 = row 1, 12..15 = 0
  int4 *dst = reinterpret_cast<int4 *>(s + out_idx * 16);
  dst[0] = make_int4((int)r0[0], (int)r0[1], (int)r0[2], (int)r1[0]);
  dst[1] = make_int4((int)r1[1], (int)r1[2], 0, 0);
}

// w [Cout][7][7][3] -> wp [Cout][4 block-rows][4 block-cols][16]; tap (kh, kw) = (2i + dr - 1, 2j + dc - 1).
template <typename XT>
__global__ void stem_pack_weight_kernel(const XT *__restrict__ w, XT *__restrict__ wp, int Cout) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= Cout * 256) return;
  const int ch = idx & 15, j = (idx >> 4) & 3, i = (idx >> 6) & 3, co = idx >> 8;
  XT val = DT<XT>::from_f(0.f);
  if (ch < 12) {
    const int q = ch / 3, c = ch - q * 3;
    const int kh = 2 * i + (q >> 1) - 1, kw = 2 * j + (q & 1) - 1;
    if (kh >= 0 && kh < 7 && kw >= 0 && kw < 7) val = w[((co * 7 + kh) * 7 + kw) * 3 + c];
  }
  wp[idx] = val;
}

}  // namespace
}  // namespace snnb

extern "C" int64_t snnb_stem7x7_scratch_bytes(int frames, int H, int W) {
  if (frames < 1 || H < 2 || W < 2) return 0;
  return (int64_t)frames * (H / 2 + 3) * (W / 2 + 3) * 16 * 2;
}

extern "C" int snnb_stem7x7_pack_weight(const void *w, void *w_packed, int Cout, int dtype, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(w && w_packed && Cout >= 1, "stem7x7_pack_weight: bad arguments");
  SNNB_CHECK_ARG(dtype == SNNB_BF16 || dtype == SNNB_F16, "stem7x7_pack_weight: dtype must be bf16 or f16");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = Cout * 256;
  if (dtype == SNNB_BF16)
    stem_pack_weight_kernel<__nv_bfloat16><<<(n + 255) / 256, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(w), static_cast<__nv_bfloat16 *>(w_packed), Cout);
  else
    stem_pack_weight_kernel<__half><<<(n + 255) / 256, 256, 0, st>>>(static_cast<const __half *>(w), static_cast<__half *>(w_packed), Cout);
  SNNB_CHECK_LAUNCH("stem7x7_pack_weight");
  return SNNB_OK;
}

extern "C" int snnb_stem7x7_lif(const void *x_seq, int64_t x_t_stride, const void *w_packed, const void *b,
                                const void *v_init, void *spikes, void *v_out, void *scratch, int64_t scratch_bytes,
                                int T, int B, int H, int W, int Cout, int dtype, int spike_dtype, int v_dtype,
                                float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && w_packed && spikes && scratch, "stem7x7_lif: null pointer");
  SNNB_CHECK_ARG(dtype == SNNB_BF16 || dtype == SNNB_F16, "stem7x7_lif: dtype must be bf16 or f16");
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && Cout >= 16 && Cout % 16 == 0, "stem7x7_lif: bad T/B/Cout");
  SNNB_CHECK_ARG(H >= 2 && W >= 2 && H % 2 == 0 && W % 2 == 0, "stem7x7_lif: H and W must be even");
  SNNB_CHECK_ARG(spike_dtype == dtype || spike_dtype == SNNB_U8 || (spike_dtype == SNNB_B1 && Cout == 64),
                 "stem7x7_lif: spike dtype must be the x dtype, u8, or (with 64 output channels) bit-packed");
  SNNB_CHECK_ARG(v_dtype == dtype || v_dtype == SNNB_F32, "stem7x7_lif: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(x_t_stride >= 0 && tau != 0.0f, "stem7x7_lif: bad frame stride or tau");
  SNNB_CHECK_ARG(aligned16(scratch) && aligned16(w_packed), "stem7x7_lif: scratch and weights must be 16-byte aligned");
  SNNB_CHECK_ARG((reinterpret_cast<uintptr_t>(x_seq) & 3u) == 0 && x_t_stride % 2 == 0,
                 "stem7x7_lif: the input must be 4-byte aligned and its frame stride even (it is read in 32-bit words)");
  const int frames = (x_t_stride == 0) ? 1 : T;  // one frame reused for all steps: re-laid (and convolved) once
  SNNB_CHECK_ARG((int64_t)frames * B <= 0x7fffffffLL, "stem7x7_lif: too many frames");
  const int64_t need = snnb_stem7x7_scratch_bytes(frames * B, H, W);
  SNNB_CHECK_ARG(need > 0, "stem7x7_lif: bad sizes");
  SNNB_CHECK_ARG(scratch_bytes >= need, "stem7x7_lif: scratch too small: %lld bytes given, %lld needed",
                 (long long)scratch_bytes, (long long)need);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int Hb = H / 2 + 3, Wb = W / 2 + 3;
  for (int f = 0; f < frames; ++f) {
    const long long total = (long long)B * Hb * Wb;
    const long long blocks = (total + 255) / 256;
    SNNB_CHECK_ARG(blocks <= 0x7fffffffLL, "stem7x7_lif: problem too large");
    if (dtype == SNNB_BF16)
      stem_s2d_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(
          static_cast<const __nv_bfloat16 *>(x_seq) + (int64_t)f * x_t_stride,
          static_cast<__nv_bfloat16 *>(scratch) + (int64_t)f * B * Hb * Wb * 16, B, H, W);
    else
      stem_s2d_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(
          static_cast<const __half *>(x_seq) + (int64_t)f * x_t_stride,
          static_cast<__half *>(scratch) + (int64_t)f * B * Hb * Wb * 16, B, H, W);
    SNNB_CHECK_LAUNCH("stem7x7_s2d");
  }
  {
    StemGemmArgs sa;
    sa.s2d = scratch; sa.w_packed = w_packed; sa.b = b; sa.v_init = v_init; sa.spikes = spikes; sa.v_out = v_out;
    sa.T = T; sa.frames = frames; sa.B = B; sa.Ho = H / 2; sa.Wo = W / 2; sa.Hb = Hb; sa.Wb = Wb; sa.Cout = Cout;
    sa.dtype = dtype; sa.spike_dtype = spike_dtype; sa.v_dtype = v_dtype;
    sa.p = make_lif_params(v_th, v_reset, tau);
    if (stem_gemm_supported(sa)) return stem_gemm_lif(sa, st);
  }
  // other channel counts / many real frames: the general implicit-GEMM kernel on a strided view
  ConvArgs a;
  a.x = scratch;
  a.x_t_stride = frames > 1 ? (int64_t)B * Hb * Wb * 16 : 0;
  a.w = w_packed; a.b = b; a.res = nullptr; a.v_init = v_init; a.spikes = spikes; a.v_out = v_out;
  a.T = T; a.B = B; a.Cin = 64; a.H = Hb; a.W = Wb; a.Cout = Cout; a.KH = 4; a.KW = 1; a.stride = 1; a.pad = 0;
  a.Ho = H / 2; a.Wo = W / 2; a.lif = 1;
  a.dtype = dtype; a.spike_dtype = spike_dtype; a.v_dtype = v_dtype;
  a.p = make_lif_params(v_th, v_reset, tau);
  a.xs_w = 16; a.xs_h = (long long)Wb * 16; a.xs_b = (long long)Hb * Wb * 16;
  a.xd_w = W / 2; a.xd_h = Hb;
  const char *why = "";
  if (!conv_lif_tc_supported(a, &why)) return fail(SNNB_ERR_UNSUPPORTED, "stem7x7_lif: %s", why);
  return conv_lif_tc(a, st);
}

namespace snnb {
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void *g_static_ptr[kMaxDevices] = {};

// Device address of the built-in scratch array on the current device. In host code the array's
// name is only a handle, so the address is asked from the runtime once per device (with that
// device current) and remembered.
int static_scratch(void **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "stem7x7_lif_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(SNNB_ERR_UNSUPPORTED, "stem7x7_lif_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_stem_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(SNNB_ERR_CUDA, "stem7x7_lif_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return SNNB_OK;
}

}  // namespace
}  // namespace snnb

extern "C" int64_t snnb_stem7x7_static_scratch_bytes(void) { return SNNB_STEM_STATIC_SCRATCH_BYTES; }

extern "C" int snnb_stem7x7_lif_static(const void *x_seq, int64_t x_t_stride, const void *w_packed, const void *b,
                                       const void *v_init, void *spikes, void *v_out,
                                       int T, int B, int H, int W, int Cout, int dtype, int spike_dtype, int v_dtype,
                                       float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(T >= 1 && B >= 1 && H >= 2 && W >= 2, "stem7x7_lif_static: bad sizes");
  SNNB_CHECK_ARG(x_t_stride >= 0, "stem7x7_lif_static: negative frame stride");
  const int64_t frames = (x_t_stride == 0 ? 1 : (int64_t)T) * (int64_t)B;   // 64-bit: T * B may not fit an int
  SNNB_CHECK_ARG(frames <= 0x7fffffffLL, "stem7x7_lif_static: too many frames");
  const int64_t need = snnb_stem7x7_scratch_bytes((int)frames, H, W);
  SNNB_CHECK_ARG(need > 0, "stem7x7_lif_static: bad sizes");
  if (need > (int64_t)SNNB_STEM_STATIC_SCRATCH_BYTES)
    return fail(SNNB_ERR_UNSUPPORTED,
                "stem7x7_lif_static: this call needs %lld bytes of scratch but the built-in array holds %lld; "
                "use a smaller batch or snnb_stem7x7_lif with caller-provided scratch",
                (long long)need, (long long)SNNB_STEM_STATIC_SCRATCH_BYTES);
  void *scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != SNNB_OK) return rc;
  return snnb_stem7x7_lif(x_seq, x_t_stride, w_packed, b, v_init, spikes, v_out, scratch,
                          (int64_t)SNNB_STEM_STATIC_SCRATCH_BYTES, T, B, H, W, Cout, dtype, spike_dtype, v_dtype,
                          v_th, v_reset, tau, stream);
}
