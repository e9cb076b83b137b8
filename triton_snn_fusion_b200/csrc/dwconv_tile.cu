// 3x3 depthwise conv (+ bias, + residual) + LIF over T from shared-memory halo tiles.
//
// The op is HBM-bound by bytes (one input element per output at stride 1, four at stride 2, one spike per
// step, the membrane once), but a kernel that fetches its nine taps straight from global memory spends its
// time on address arithmetic, border predicates and 16-bit unpacking instead. Here:
//   * a thread block owns R output rows x (NS * PW) output columns x CS channels of one image. For each
//     timestep ONE tiled TMA copy (cp.async.bulk.tensor, no multicast) brings the input pixels those outputs
//     need - the tile plus its one-pixel halo - into shared memory as a dense [row][col][channel] array;
//     pixels outside the image arrive as zeros, which is the conv's padding, so no load is predicated.
//     Two buffers: the copy of step t + 1 runs under the arithmetic of step t;
//   * a thread owns 4 consecutive channels of a strip of PW = 4 consecutive output pixels of one row. Lanes run
//     over channels first, so a warp's shared-memory reads and global stores cover whole 128-byte rows. The
//     3x3 window slides along the strip: every input vector is read from shared memory and widened to fp32
//     once and feeds up to three accumulators, two channels per instruction (fma.rn.f32x2);
//   * the PW x 4 membrane potentials of a thread stay in registers for all T steps.
// Algorithmic bytes per call: T*B*C*(H*W*s_x + Ho*Wo*s_s [+ Ho*Wo*s_x residual]) + B*C*Ho*Wo*s_v*(1 or 2).
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace snnb {

static __device__ int g_dw_status = 0;

namespace {

constexpr int kDwThreads = 256;

struct DwGeom {
  int T, Tx, B, C, H, W, Ho, Wo;
  int cs;        // channels per block: 64 or 32
  int ns;        // strips per tile row: 1 or 2
  int rows;      // output rows per tile = threads / (cs / 4 * ns)
  int hw, hr;    // halo tile: columns, rows
  int nct, nrt, nslab, total_tiles;
  int tx_bytes;    // size of one halo tile = bytes one copy delivers
  int buf_pitch;   // distance between the two buffers (tx_bytes rounded up to 128)
};

template <typename XT> struct Vec4;   // four consecutive channels in shared memory -> two float2
template <> struct Vec4<float> {
  static __device__ __forceinline__ void load(uint32_t addr, float2 &a, float2 &b) {
    float4 r;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "r"(addr));
    a = make_float2(r.x, r.y);
    b = make_float2(r.z, r.w);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(uint32_t addr, float2 &a, float2 &b) {
    uint32_t lo, hi;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
    a = make_float2(__uint_as_float(lo << 16), __uint_as_float(lo & 0xffff0000u));
    b = make_float2(__uint_as_float(hi << 16), __uint_as_float(hi & 0xffff0000u));
  }
};
template <> struct Vec4<__half> {
  static __device__ __forceinline__ void load(uint32_t addr, float2 &a, float2 &b) {
    uint32_t lo, hi;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
    a = __half22float2(*reinterpret_cast<const __half2 *>(&lo));
    b = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
  }
};

// one LIF step on two channels. KIND 0: any LIF (run-time lif_step); 1: tau a power of two and hard reset, with the
// charge step on the packed fp32 pipe; 2: additionally v_reset == 0, where the reset is one packed multiply-add.
// h = v + (y - v) * inv_tau is evaluated as three separately rounded operations exactly as lif_step does
// (x - v and x + (-v) round identically); with s in {0, 1}, h - s * h is exactly 0 or h.
template <int KIND>
__device__ __forceinline__ float2 lif2(float2 y, float2 &v, const LifParams &p) {
  float2 s;
  if constexpr (KIND == 0) {
    s.x = lif_step(y.x, v.x, p);
    s.y = lif_step(y.y, v.y, p);
  } else {
    const float2 d = __fadd2_rn(y, make_float2(-v.x, -v.y));
    const float2 h = __fadd2_rn(v, __fmul2_rn(d, make_float2(p.inv_tau, p.inv_tau)));
    s = make_float2(h.x >= p.v_th ? 1.f : 0.f, h.y >= p.v_th ? 1.f : 0.f);
    if constexpr (KIND == 2) {
      v = __ffma2_rn(make_float2(-s.x, -s.y), h, h);
    } else {
      v.x = s.x != 0.f ? p.v_reset : h.x;
      v.y = s.y != 0.f ? p.v_reset : h.y;
    }
  }
  return s;
}

// Persistent: a block walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... and treats (tile, timestep) pairs as one
// stream of work items, so the copy of the next item - the next timestep, or the first timestep of the next tile -
// always runs under the arithmetic of the current one and only the very first copy of a block is exposed.
// The tile geometry is fixed at compile time (strips of PW = 4 pixels, NS = 2 strips per tile row, CS channels), so
// every shared-memory read of the inner loop is "window base + constant": the loop body is the 16-byte-free
// sequence load, widen, multiply-add with no address arithmetic left in it.
constexpr int PW = 4, NS = 2;

template <typename XT, typename ST, typename VT, int STRIDE, int CS, int KIND>
__global__ void __launch_bounds__(kDwThreads, 2)
dwconv_tile_kernel(const __grid_constant__ CUtensorMap xmap, const XT *__restrict__ w, const XT *__restrict__ bias,
                   const XT *__restrict__ res, const VT *v_init, ST *__restrict__ spikes, VT *v_out,
                   const DwGeom g, const LifParams p) {
  extern __shared__ uint8_t dw_smem_raw[];
  __shared__ __align__(8) uint64_t full[2];
  __shared__ int abort_s;
  const uint32_t smem = (umma::smem_u32(dw_smem_raw) + 127u) & ~127u;
  const uint32_t bar = umma::smem_u32(full);
  volatile int *abort_flag = &abort_s;

  constexpr int CGN = CS / 4;                                  // channel quads per pixel
  constexpr int HWD = (NS * PW - 1) * STRIDE + 3;              // halo tile width in pixels
  constexpr uint32_t PXB = CS * sizeof(XT);                    // bytes per pixel
  constexpr uint32_t ROWB = HWD * PXB;                         // bytes per halo row
  constexpr int NCOL = (PW - 1) * STRIDE + 3;                  // input columns a strip needs
  const int tid = threadIdx.x;
  const int cg = tid % CGN;
  const int strip = (tid / CGN) % NS;
  const int row = tid / (CGN * NS);
  // copies of the launch constants the loops use (kept in registers instead of re-read from the parameter bank)
  const int T = g.T, Ho = g.Ho, Wo = g.Wo, C = g.C, nct = g.nct, nrt = g.nrt, nB = g.B, rows = g.rows;
  const uint32_t pitch = (uint32_t)g.buf_pitch, tx_bytes = (uint32_t)g.tx_bytes;
  const bool many_frames = g.Tx > 1;

  // tile index -> (column tile, row tile, image, channel block); the channel block is slowest, so a block's
  // consecutive tiles nearly always share their weights
  auto decode = [&](int tile, int &ct, int &rt, int &b, int &slab) {
    ct = tile % nct; tile /= nct;
    rt = tile % nrt; tile /= nrt;
    b = tile % nB;
    slab = tile / nB;
  };
  const int my_tiles = (int)blockIdx.x < g.total_tiles ? (g.total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int n_items = my_tiles * T;

  if (tid == 0) {
    abort_s = 0;
    umma::mbar_init(bar, 1);
    umma::mbar_init(bar + 8, 1);
    umma::fence_mbar_init();
    umma::prefetch_tensormap(&xmap);
  }
  __syncthreads();
  // producer state (thread 0): the next work item to copy, as (tile ordinal, timestep) and its tile coordinates
  int p_i = 0, p_t = 0, p_ct = 0, p_rt = 0, p_b = 0, p_slab = 0, p_item = 0;
  auto issue_next = [&]() {   // one thread: start the copy of work item p_item into buffer p_item & 1
    if (p_t == 0) decode((int)blockIdx.x + p_i * (int)gridDim.x, p_ct, p_rt, p_b, p_slab);
    const uint32_t nb = (uint32_t)(p_item & 1);
    umma::mbar_expect_tx(bar + 8 * nb, tx_bytes);
    umma::tma_load_5d(smem + nb * pitch, &xmap, bar + 8 * nb, p_slab * CS, p_ct * (NS * PW * STRIDE) - 1,
                      p_rt * rows * STRIDE - 1, p_b, many_frames ? p_t : 0);
    ++p_item;
    if (++p_t == T) { p_t = 0; ++p_i; }
  };
  if (tid == 0 && n_items > 0) issue_next();

  // this thread's window inside a halo tile: rows row*STRIDE .., columns strip*PW*STRIDE ..
  const uint32_t win0 = smem + (uint32_t)(row * STRIDE) * ROWB + (uint32_t)(strip * PW * STRIDE) * PXB + (uint32_t)cg * 4u * sizeof(XT);
  const size_t frame_out = (size_t)nB * Ho * Wo * C;

  float2 wq[9][2];   // weights and bias of this thread's four channels, as channel pairs
  float2 bq[2];
  int cur_slab = -1;
  int item = 0;
  bool ok = true;
  for (int i = 0; i < my_tiles && ok; ++i) {
    int ct, rt, b, slab;
    decode((int)blockIdx.x + i * (int)gridDim.x, ct, rt, b, slab);
    const int c = slab * CS + cg * 4;
    if (slab != cur_slab) {
      cur_slab = slab;
#pragma unroll
      for (int k = 0; k < 9; ++k) {
        wq[k][0] = make_float2(DT<XT>::to_f(w[(size_t)(c + 0) * 9 + k]), DT<XT>::to_f(w[(size_t)(c + 1) * 9 + k]));
        wq[k][1] = make_float2(DT<XT>::to_f(w[(size_t)(c + 2) * 9 + k]), DT<XT>::to_f(w[(size_t)(c + 3) * 9 + k]));
      }
      bq[0] = bq[1] = make_float2(0.f, 0.f);
      if (bias != nullptr) {
        bq[0] = make_float2(DT<XT>::to_f(bias[c]), DT<XT>::to_f(bias[c + 1]));
        bq[1] = make_float2(DT<XT>::to_f(bias[c + 2]), DT<XT>::to_f(bias[c + 3]));
      }
    }
    const int ho = rt * rows + row;
    const int wo0 = (ct * NS + strip) * PW;
    // which of the strip's PW outputs exist (bit j), and where the first of them lives in a frame
    int live = 0;
#pragma unroll
    for (int j = 0; j < PW; ++j)
      if (ho < Ho && wo0 + j < Wo) live |= 1 << j;
    const size_t out0 = (((size_t)b * Ho + (ho < Ho ? ho : 0)) * Wo + (wo0 < Wo ? wo0 : 0)) * C + c;   // (b, ho, wo0, c)

    float2 v[PW][2];
#pragma unroll
    for (int j = 0; j < PW; ++j) {
      v[j][0] = v[j][1] = make_float2(0.f, 0.f);
      if (v_init != nullptr && ((live >> j) & 1)) {
        float t4[4];
        load_pack_stream<VT, 4>(v_init + out0 + (size_t)j * C, t4);
        v[j][0] = make_float2(t4[0], t4[1]);
        v[j][1] = make_float2(t4[2], t4[3]);
      }
    }
    ST *sp = spikes + out0;
    const XT *rp = res != nullptr ? res + out0 : nullptr;

    for (int t = 0; t < T; ++t, ++item) {
      // buffer (item + 1) & 1 was last read by item - 1, which ended with a barrier
      if (tid == 0 && item + 1 < n_items) issue_next();
      ok = umma::mbar_wait(bar + 8 * (uint32_t)(item & 1), (uint32_t)((item >> 1) & 1), abort_flag);
      if (!ok) break;
      const uint32_t base = win0 + (uint32_t)(item & 1) * pitch;

      float2 acc[PW][2];
#pragma unroll
      for (int j = 0; j < PW; ++j) { acc[j][0] = bq[0]; acc[j][1] = bq[1]; }
#pragma unroll
      for (int kh = 0; kh < 3; ++kh) {
#pragma unroll
        for (int col = 0; col < NCOL; ++col) {
          float2 x0, x1;
          Vec4<XT>::load(base + (uint32_t)kh * ROWB + (uint32_t)col * PXB, x0, x1);
#pragma unroll
          for (int kw = 0; kw < 3; ++kw) {
            // input column col = j * STRIDE + kw
            if ((col - kw) >= 0 && (col - kw) % STRIDE == 0 && (col - kw) / STRIDE < PW) {   // resolved when unrolled
              const int j = (col - kw) / STRIDE;
              acc[j][0] = __ffma2_rn(wq[kh * 3 + kw][0], x0, acc[j][0]);
              acc[j][1] = __ffma2_rn(wq[kh * 3 + kw][1], x1, acc[j][1]);
            }
          }
        }
      }

      if (live == (1 << PW) - 1 && rp == nullptr) {
        // the common case: every output of the strip exists and there is no residual: straight-line code
        ST *spj = sp;
#pragma unroll
        for (int j = 0; j < PW; ++j) {
          const float2 s0 = lif2<KIND>(acc[j][0], v[j][0], p);
          const float2 s1 = lif2<KIND>(acc[j][1], v[j][1], p);
          const float s4[4] = {s0.x, s0.y, s1.x, s1.y};
          store_pack<ST, 4>(spj, s4);
          spj += C;
        }
      } else {
        ST *spj = sp;
        const XT *rpj = rp;
#pragma unroll
        for (int j = 0; j < PW; ++j) {
          if ((live >> j) & 1) {
            if (rpj != nullptr) {
              float r4[4];
              load_pack<XT, 4>(rpj, r4);
              acc[j][0] = __fadd2_rn(acc[j][0], make_float2(r4[0], r4[1]));
              acc[j][1] = __fadd2_rn(acc[j][1], make_float2(r4[2], r4[3]));
            }
            const float2 s0 = lif2<KIND>(acc[j][0], v[j][0], p);
            const float2 s1 = lif2<KIND>(acc[j][1], v[j][1], p);
            const float s4[4] = {s0.x, s0.y, s1.x, s1.y};
            store_pack<ST, 4>(spj, s4);
          }
          spj += C;
          if (rpj != nullptr) rpj += C;
        }
      }
      sp += frame_out;
      if (rp != nullptr) rp += frame_out;
      __syncthreads();   // everyone is done with buffer item & 1 before the copy of item + 2 may overwrite it
    }

    if (ok) {
#pragma unroll
      for (int j = 0; j < PW; ++j) {
        if ((live >> j) & 1) {
          const float v4[4] = {v[j][0].x, v[j][0].y, v[j][1].x, v[j][1].y};
          store_pack<VT, 4>(v_out + out0 + (size_t)j * C, v4);
        }
      }
    }
  }
  if (!ok && tid == 0) atomicExch(&g_dw_status, 1);
}

struct DwCall {
  const void *x; int64_t xts; const void *w, *b, *res, *v_init; void *spikes, *v_out;
  int T, B, C, H, W, stride, dtype;
  LifParams p;
};

template <typename XT, typename ST, typename VT>
int launch_tile(const DwCall &a, cudaStream_t stream) {
  DwGeom g;
  g.T = a.T; g.Tx = a.xts == 0 ? 1 : a.T; g.B = a.B; g.C = a.C; g.H = a.H; g.W = a.W;
  g.Ho = (a.H + 2 - 3) / a.stride + 1;
  g.Wo = (a.W + 2 - 3) / a.stride + 1;
  g.cs = a.C % 64 == 0 ? 64 : 32;
  g.ns = NS;
  int threads = kDwThreads;
  g.rows = threads / ((g.cs / 4) * NS);
  // stride 2 reads four input pixels per output: half the rows keep two buffers of a tile small
  if (a.stride == 2) { g.rows /= 2; threads /= 2; }
  while (g.rows > 1 && g.rows / 2 >= g.Ho) { g.rows /= 2; threads /= 2; }   // short maps: no idle rows
  g.hw = (NS * PW - 1) * a.stride + 3;
  g.hr = (g.rows - 1) * a.stride + 3;
  g.nct = (g.Wo + NS * PW - 1) / (NS * PW);
  g.nrt = (g.Ho + g.rows - 1) / g.rows;
  g.nslab = a.C / g.cs;
  g.tx_bytes = g.hr * g.hw * g.cs * (int)sizeof(XT);
  g.buf_pitch = (g.tx_bytes + 127) & ~127;
  const long long tiles = (long long)a.B * g.nslab * g.nrt * g.nct;
  if (tiles * a.T > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "dwconv3x3_lif: problem too large");
  g.total_tiles = (int)tiles;
  const int sms = sm_count() > 0 ? sm_count() : 128;
  const int per_sm = 2 * (kDwThreads / threads);   // resident blocks per SM (register budget: two blocks of 256 threads)
  const long long grid = tiles < (long long)sms * per_sm ? tiles : (long long)sms * per_sm;
  const size_t smem = 2 * (size_t)g.buf_pitch + 128;
  if (smem > 100 * 1024) return fail(SNNB_ERR_UNSUPPORTED, "dwconv3x3_lif: tile does not fit shared memory");
  CUtensorMap xm;
  {
    const int es = (int)sizeof(XT);
    cuuint64_t dims[5] = {(cuuint64_t)a.C, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.B, (cuuint64_t)g.Tx};
    cuuint64_t strides[4] = {(cuuint64_t)a.C * es, (cuuint64_t)a.W * a.C * es, (cuuint64_t)a.H * a.W * a.C * es,
                             g.Tx > 1 ? (cuuint64_t)a.xts * es : (cuuint64_t)a.B * a.H * a.W * a.C * es};
    cuuint32_t box[5] = {(cuuint32_t)g.cs, (cuuint32_t)g.hw, (cuuint32_t)g.hr, 1, 1};
    const int rc = encode_tmap(&xm, a.dtype, 5, a.x, dims, strides, box, 0);
    if (rc != SNNB_OK) return rc;
  }
  const DwGeom gk = g;
  const int kind = (a.p.mode == 1 && a.p.hard) ? (a.p.v_reset == 0.f ? 2 : 1) : 0;
#define SNNB_DWT2(STR, CSV, KINDV)                                                                                  \
  do {                                                                                                              \
    auto kern = dwconv_tile_kernel<XT, ST, VT, STR, CSV, KINDV>;                                                    \
    static bool attr_done[64] = {};                                                                                 \
    int dev = 0;                                                                                                    \
    cudaGetDevice(&dev);                                                                                            \
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {                                                                  \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)       \
        return fail(SNNB_ERR_CUDA, "dwconv3x3_lif: cannot raise the shared-memory limit");                          \
      if (dev >= 0 && dev < 64) attr_done[dev] = true;                                                              \
    }                                                                                                               \
    kern<<<(unsigned)grid, threads, smem, stream>>>(xm, static_cast<const XT *>(a.w), static_cast<const XT *>(a.b), \
                                                    static_cast<const XT *>(a.res), static_cast<const VT *>(a.v_init), \
                                                    static_cast<ST *>(a.spikes), static_cast<VT *>(a.v_out), gk, a.p); \
  } while (0)
#define SNNB_DWT(STR, CSV)                                                           \
  do {                                                                               \
    if (kind == 2) SNNB_DWT2(STR, CSV, 2);                                           \
    else if (kind == 1) SNNB_DWT2(STR, CSV, 1);                                      \
    else SNNB_DWT2(STR, CSV, 0);                                                     \
  } while (0)
  if (a.stride == 1) {
    if (g.cs == 64) SNNB_DWT(1, 64); else SNNB_DWT(1, 32);
  } else {
    if (g.cs == 64) SNNB_DWT(2, 64); else SNNB_DWT(2, 32);
  }
#undef SNNB_DWT2
#undef SNNB_DWT
  SNNB_CHECK_LAUNCH("dwconv3x3_lif (tile kernel)");
  return SNNB_OK;
}

template <typename XT>
int dispatch_tile(const DwCall &a, int spike_dtype, int v_dtype, cudaStream_t stream) {
  const bool s_u8 = spike_dtype == SNNB_U8, v_f32 = v_dtype == SNNB_F32 && !std::is_same<XT, float>::value;
  if (s_u8 && v_f32) return launch_tile<XT, uint8_t, float>(a, stream);
  if (s_u8) return launch_tile<XT, uint8_t, XT>(a, stream);
  if (v_f32) return launch_tile<XT, XT, float>(a, stream);
  return launch_tile<XT, XT, XT>(a, stream);
}

}  // namespace

// Which calls the tile kernel takes: channel counts that split into 32- or 64-channel blocks, 16-byte aligned
// buffers (the TMA copy and the 8-byte channel-quad accesses need it) and a frame stride the tensor map can express.
bool dwconv_tile_supported(const void *x, int64_t xts, const void *res, const void *v_init, const void *spikes,
                           const void *v_out, int C, int H, int W, int dtype) {
  if (C % 32 != 0) return false;
  const int es = dtype == SNNB_F32 ? 4 : 2;
  if (!aligned16(x) || !aligned16(spikes) || !aligned16(v_out) || (res && !aligned16(res)) || (v_init && !aligned16(v_init)))
    return false;
  if ((xts * es) % 16 != 0) return false;
  if ((long long)W * C * es >= (1ll << 40)) return false;
  return H >= 1 && W >= 1;
}

int dwconv_tile(const void *x, int64_t xts, const void *w, const void *b, const void *res, const void *v_init,
                void *spikes, void *v_out, int T, int B, int C, int H, int W, int stride, int dtype, int spike_dtype,
                int v_dtype, const LifParams &p, cudaStream_t stream) {
  DwCall a{x, xts, w, b, res, v_init, spikes, v_out, T, B, C, H, W, stride, dtype, p};
  switch (dtype) {
    case SNNB_F32: return dispatch_tile<float>(a, spike_dtype, v_dtype, stream);
    case SNNB_BF16: return dispatch_tile<__nv_bfloat16>(a, spike_dtype, v_dtype, stream);
    default: return dispatch_tile<__half>(a, spike_dtype, v_dtype, stream);
  }
}

int dw_device_status(int *out) {
  int h = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&h, g_dw_status, sizeof(int));
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_dw_status, &zero, sizeof(int));
  }
  *out = h;
  return SNNB_OK;
}

}  // namespace snnb
