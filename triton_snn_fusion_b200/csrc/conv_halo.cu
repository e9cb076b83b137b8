// 3x3 / stride 1 / padding 1 conv (+ bias, + residual) + LIF over T as a tcgen05 implicit GEMM whose
// nine taps are read from ONE shared-memory copy of the input tile.
//
// The general kernel (conv_tc.cu) fetches the activation tile of every tap from L2 again: nine loads
// of the same pixels shifted by one, which makes 3x3 layers L2-bandwidth bound. Here a CTA owns an
// 8 (wide) x 16 (high) block of output pixels and loads, per timestep and 64-channel slab, the
// 10 x 18 input pixels that block needs (its halo tile, 23 KB) with one TMA box; out-of-image pixels
// arrive as zeros, which is the padding. Row r = 8*g + i of the MMA's A operand is output pixel
// (row g, column i) of the block; for tap (kh, kw) its input pixel sits at halo row g + kh, halo
// column i + kw, i.e. at byte offset ((g + kh) * 10 + i + kw) * 128 of the halo tile. That is exactly
// what a K-major 128-byte-swizzle operand descriptor can express: start address shifted by
// (kh * 10 + kw) rows, 8-row groups 1280 bytes (one halo row) apart. The swizzle phase of a row is a
// function of its shared-memory address for both TMA and the MMA unit, so no row needs to be aligned
// to the 1024-byte swizzle period. L2 -> SM traffic per tile drops from 9 activation tiles to one
// halo tile (1.4 activation tiles) per (t, slab).
//
// Small feature maps: when (n - 1) * (H + 2) + H <= 16, n images are stacked in one tile (image i
// occupies halo rows i*(H+2) .. and output-row groups i*(H+2) .. i*(H+2)+H-1; the groups in between
// compute junk that is never stored), so 7x7 maps still fill 14 of the 16 groups.
//
// Loop order per tile: slab -> tap -> t. The weight tile of a (tap, slab) is loaded once and used by
// all T timesteps; the T halo tiles of a slab stay resident for its nine taps and are released after
// the last one, while a ring of up to 2T halo slots lets the next slab's tiles stream in meanwhile.
// Warp roles: 0-7 epilogue (shared with conv_tc.cu), 8 halo producer, 9 weight producer, 10 MMA.
#include <type_traits>

#include "conv.cuh"
#include "tc_epilogue.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace snnb {

static __device__ int g_halo_status = 0;

namespace {

constexpr int kHaloW = 10, kHaloH = 18;
constexpr int kHaloRowBytes = kHaloW * 128;                 // 1280: distance between 8-row groups
constexpr int kHaloBytes = kHaloW * kHaloH * 128;           // 23040
constexpr int kMaxHaloSlots = 9;
constexpr int kWRing = 3;
constexpr int kEpiWarpsH = 8;
constexpr int kMmaWarps = 4;   // MMA issuers: warp j issues the MMAs of timesteps j, j + 4, ...
constexpr int kHaloWarp = kEpiWarpsH, kWWarp = kEpiWarpsH + 1, kMmaWarpH = kEpiWarpsH + 2;   // first MMA warp
constexpr int kThreadsH = 32 * (kEpiWarpsH + 2 + kMmaWarps);

struct HaloGeom {
  int T, Tacc, B, Cin, Cout, Ho, Wo;
  int BN, n_tiles_n, kslabs;
  int n_img;        // images stacked in one tile (1 = a tile is 16 rows of one image)
  int img_rows;     // halo rows per stacked image (Ho + 2); box height in stacked mode
  int row_tiles;    // tiles per image column (1 in stacked mode)
  int w_strips;     // 8-pixel column strips per image row
  int halo_slots, w_slot_bytes, tmem_cols, lif, has_res;
  int n_mma;        // active MMA-issuing warps = min(kMmaWarps, Tacc)
};

template <typename XT, typename ST, typename VT>
__global__ void __launch_bounds__(kThreadsH)
conv3x3_halo_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                    const XT *__restrict__ bias, const XT *__restrict__ res, const VT *__restrict__ v_init,
                    ST *__restrict__ spikes, VT *__restrict__ v_out, const HaloGeom g, const LifParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kMaxHaloSlots + 2 * kWRing + 1];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x % g.n_tiles_n;
  int m = blockIdx.x / g.n_tiles_n;
  const int strip = m % g.w_strips;
  m /= g.w_strips;
  const int rt = m % g.row_tiles;
  const int ig = m / g.row_tiles;
  const int n0 = n_tile * g.BN;
  const int w0 = strip * 8;
  const int h0 = rt * 16;          // first output row of the tile (row-tiled mode)
  const int b0 = ig * g.n_img;     // first image of the tile

  const uint32_t smem_base = (umma::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_base = smem_base;
  const uint32_t h_base = smem_base + (uint32_t)kWRing * (uint32_t)g.w_slot_bytes;
  const uint32_t bar_base = umma::smem_u32(bars);
  auto hfull = [&](uint32_t s) { return bar_base + 8u * s; };
  auto hempty = [&](uint32_t s) { return bar_base + 8u * ((uint32_t)kMaxHaloSlots + s); };
  auto wfull = [&](uint32_t s) { return bar_base + 8u * (2u * kMaxHaloSlots + s); };
  auto wempty = [&](uint32_t s) { return bar_base + 8u * (2u * kMaxHaloSlots + kWRing + s); };
  const uint32_t acc_bar = bar_base + 8u * (2u * kMaxHaloSlots + 2u * kWRing);
  volatile int *abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < g.halo_slots; ++s) {
      umma::mbar_init(hfull(s), 1);
      umma::mbar_init(hempty(s), 1);
    }
    for (int s = 0; s < kWRing; ++s) {
      umma::mbar_init(wfull(s), 1);
      umma::mbar_init(wempty(s), (uint32_t)g.n_mma);   // every MMA warp releases a weight tile
    }
    umma::mbar_init(acc_bar, (uint32_t)g.n_mma);
    umma::fence_mbar_init();
  }
  if (warp == kMmaWarpH) {
    umma::tmem_alloc(umma::smem_u32(&tmem_base_s), (uint32_t)g.tmem_cols);
    umma::tmem_relinquish();
  }
  if (warp == kHaloWarp && lane == 0) {
    umma::prefetch_tensormap(&xmap);
    umma::prefetch_tensormap(&wmap);
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  umma::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == kHaloWarp) {
    // ------------------------------------------------------------ halo producer
    // One TMA box per (slab, t) — or one per stacked image, issued by lane i for image i.
    const bool stacked = g.n_img > 1;
    const bool mine = stacked ? (lane < g.n_img && b0 + lane < g.B) : (lane == 0);
    const uint32_t box_bytes = stacked ? (uint32_t)g.img_rows * kHaloRowBytes : (uint32_t)kHaloBytes;
    const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, mine)) * box_bytes;
    const uint32_t my_off = stacked ? (uint32_t)lane * box_bytes : 0u;
    const int my_b = stacked ? b0 + lane : b0;
    const int ch = stacked ? -1 : h0 - 1;
    uint32_t slot = 0, phase = 1;
    bool ok = true;
    for (int slab = 0; slab < g.kslabs && ok; ++slab) {
      for (int t = 0; t < g.Tacc; ++t) {
        if (lane == 0) {
          ok = umma::mbar_wait(hempty(slot), phase, abort_flag);
          if (ok) umma::mbar_expect_tx(hfull(slot), bytes);
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (mine)
          umma::tma_load_5d(h_base + slot * (uint32_t)kHaloBytes + my_off, &xmap, hfull(slot), slab * 64, w0 - 1, ch,
                            my_b, t);
        if (++slot == (uint32_t)g.halo_slots) { slot = 0; phase ^= 1u; }
      }
    }
  } else if (warp == kWWarp) {
    // ---------------------------------------------------------- weight producer
    if (lane == 0) {
      const uint32_t w_bytes = (uint32_t)g.BN * 128u;
      uint32_t ws = 0, wphase = 1;
      const int nw = g.kslabs * 9;
      for (int i = 0, slab = 0, tap = 0; i < nw; ++i) {
        if (!umma::mbar_wait(wempty(ws), wphase, abort_flag)) break;
        umma::mbar_expect_tx(wfull(ws), w_bytes);
        // weight matrix is [Cout][tap][Cin]: K index of (tap, slab) = tap * Cin + slab * 64
        umma::tma_load_2d(w_base + ws * (uint32_t)g.w_slot_bytes, &wmap, wfull(ws), tap * g.Cin + slab * 64, n0);
        if (++ws == (uint32_t)kWRing) { ws = 0; wphase ^= 1u; }
        if (++tap == 9) { tap = 0; ++slab; }
      }
    }
    __syncwarp();
  } else if (warp >= kMmaWarpH) {
    // ------------------------------------------------------------- MMA issuers
    // Issuing one tcgen05.mma costs its thread on the order of a hundred cycles, more than a
    // 128x128x16 MMA occupies the tensor pipe, so a single issuer cannot keep the pipe busy. The T
    // accumulators are independent, so timestep t is issued by warp t mod n_mma; every issuer waits
    // for the weight tile itself and releases it (the weight barriers count n_mma arrivals).
    const int j = warp - kMmaWarpH;
    if (lane == 0 && j < g.n_mma) {
      const uint32_t idesc = umma::make_idesc_f16(128, g.BN, std::is_same<XT, __nv_bfloat16>::value);
      // operand descriptor of a halo tile: 8-row groups one halo row (1280 bytes) apart
      uint64_t hdesc0 = umma::make_sw128_kmajor_desc(h_base);
      hdesc0 = (hdesc0 & ~((uint64_t)0x3FFF << 32)) | ((uint64_t)(kHaloRowBytes >> 4) << 32);
      const uint64_t wdesc0 = umma::make_sw128_kmajor_desc(w_base);
      uint32_t s0 = 0, p0 = 0;   // ring slot / phase of this slab's t = 0 halo tile
      uint32_t ws = 0, wphase = 0;
      bool ok = true;
      for (int slab = 0; slab < g.kslabs && ok; ++slab) {
        for (int tap = 0; tap < 9 && ok; ++tap) {
          ok = umma::mbar_wait(wfull(ws), wphase, abort_flag);
          if (!ok) break;
          umma::tc_fence_after_sync();
          const uint64_t wdesc = wdesc0 + (uint64_t)((ws * (uint32_t)g.w_slot_bytes) >> 4);
          const int kh = tap / 3, kw = tap - kh * 3;
          const uint32_t tap_off = (uint32_t)(kh * kHaloW + kw) * 128u;
          uint32_t slot = s0, phase = p0;
          for (int t = 0; t < g.Tacc; ++t) {
            if (t % g.n_mma == j) {
              if (tap == 0) {
                ok = umma::mbar_wait(hfull(slot), phase, abort_flag);
                if (!ok) break;
                umma::tc_fence_after_sync();
              }
              const uint64_t adesc = hdesc0 + (uint64_t)((slot * (uint32_t)kHaloBytes + tap_off) >> 4);
              const uint32_t d = tmem_base + (uint32_t)(t * g.BN);
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma::mma_f16_ss(d, adesc + (uint64_t)(2 * k), wdesc + (uint64_t)(2 * k), idesc,
                                 (slab > 0 || tap > 0 || k > 0) ? 1u : 0u);
              if (tap == 8) umma::mma_commit(hempty(slot));   // last use of this halo tile
            }
            if (++slot == (uint32_t)g.halo_slots) { slot = 0; phase ^= 1u; }
          }
          if (ok) umma::mma_commit(wempty(ws));
          if (++ws == (uint32_t)kWRing) { ws = 0; wphase ^= 1u; }
          if (tap == 8) { s0 = slot; p0 = phase; }
        }
      }
      if (ok) {
        umma::mma_commit(acc_bar);
        if (j == 0) umma::mbar_wait(acc_bar, 0u, abort_flag);   // all issuers' MMAs are complete
      }
    }
    __syncwarp();
    if (j == 0) {
      umma::tc_fence_before_sync();
      asm volatile("bar.arrive 1, %0;" ::"r"(32 * (kEpiWarpsH + 1)) : "memory");
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;   // tile row: group (output row) r / 8, column r % 8
    const int grp = r >> 3, pw = r & 7;
    int b, ho;
    bool valid;
    if (g.n_img > 1) {
      const int i = grp / g.img_rows;
      ho = grp - i * g.img_rows;
      b = b0 + i;
      valid = (i < g.n_img) && (ho < g.Ho) && (b < g.B);
    } else {
      b = b0;
      ho = h0 + grp;
      valid = ho < g.Ho;
    }
    const int wo = w0 + pw;
    valid = valid && (wo < g.Wo);
    const long long pix = valid ? ((long long)b * g.Ho + ho) * g.Wo + wo : 0;
    asm volatile("bar.sync 1, %0;" ::"r"(32 * (kEpiWarpsH + 1)) : "memory");  // released by the MMA warp
    const bool ok = (*abort_flag == 0);
    umma::tc_fence_after_sync();
    if (ok) {
      const int nch = g.BN / 16, half = (nch + 1) / 2;
      const int c_begin = (warp < 4) ? 0 : half;
      const int c_end = (warp < 4) ? half : nch;
      EpiArgs<XT, ST, VT> ea{bias, res, v_init, spikes, v_out, tmem_base + ((uint32_t)(quarter * 32) << 16),
                             pix, (long long)g.B * g.Ho * g.Wo * g.Cout, n0, c_begin, c_end, valid};
      const EpiGeom eg{g.T, g.Tacc, g.BN, g.Cout, g.has_res};
      epilogue_dispatch<XT, ST, VT>(ea, eg, g.lif, p);
    }
  }

  umma::tc_fence_before_sync();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) atomicExch(&g_halo_status, 1);
  if (warp == kMmaWarpH) {
    umma::tc_fence_after_sync();
    umma::tmem_dealloc(tmem_base, (uint32_t)g.tmem_cols);
  }
}

int halo_bn(int Cout, int Tacc) {
  int bn = Cout >= 128 ? 128 : ((Cout + 15) / 16) * 16;
  while (bn > 16 && Tacc * bn > 512) bn /= 2;
  return bn;
}

bool fill_geom(const ConvArgs &a, HaloGeom &g) {
  g.T = a.T;
  g.Tacc = (a.x_t_stride == 0) ? 1 : a.T;
  g.B = a.B; g.Cin = a.Cin; g.Cout = a.Cout; g.Ho = a.Ho; g.Wo = a.Wo;
  g.BN = halo_bn(a.Cout, g.Tacc);
  g.n_tiles_n = (a.Cout + g.BN - 1) / g.BN;
  g.kslabs = a.Cin / 64;
  g.img_rows = a.Ho + 2;
  int n = 1;
  while (n < 8 && n * g.img_rows + a.Ho <= 16) ++n;   // largest n with (n-1)*(H+2) + H <= 16
  g.n_img = n;
  g.row_tiles = n > 1 ? 1 : (a.Ho + 15) / 16;
  g.w_strips = (a.Wo + 7) / 8;
  g.lif = a.lif;
  g.has_res = a.res != nullptr;
  int cols = 32;
  while (cols < g.Tacc * g.BN) cols *= 2;
  g.tmem_cols = cols;
  g.w_slot_bytes = ((g.BN * 128 + 1023) / 1024) * 1024;
  int slots = (208 * 1024 - kWRing * g.w_slot_bytes) / kHaloBytes;
  if (slots > 2 * g.Tacc) slots = 2 * g.Tacc;
  if (slots > kMaxHaloSlots) slots = kMaxHaloSlots;
  g.halo_slots = slots;
  g.n_mma = g.Tacc < kMmaWarps ? g.Tacc : kMmaWarps;
  return slots >= g.Tacc && slots >= 2;
}

template <typename XT, typename ST, typename VT>
int launch(const ConvArgs &a, cudaStream_t stream) {
  HaloGeom g;
  if (!fill_geom(a, g)) return fail(SNNB_ERR_UNSUPPORTED, "conv_lif: halo tiles of all T steps do not fit shared memory");
  const long long img_groups = (a.B + g.n_img - 1) / g.n_img;
  const long long grid = img_groups * g.row_tiles * g.w_strips * g.n_tiles_n;
  if (grid > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "conv_lif: problem too large for the grid");
  const int es = 2;
  CUtensorMap xm, wm;
  {
    cuuint64_t dims[5] = {(cuuint64_t)a.Cin, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.B, (cuuint64_t)g.Tacc};
    const cuuint64_t frame_bytes = (cuuint64_t)a.B * a.H * a.W * a.Cin * es;
    cuuint64_t strides[4] = {(cuuint64_t)a.Cin * es, (cuuint64_t)a.W * a.Cin * es, (cuuint64_t)a.H * a.W * a.Cin * es,
                             g.Tacc > 1 ? (cuuint64_t)a.x_t_stride * es : frame_bytes};
    cuuint32_t box[5] = {64, (cuuint32_t)kHaloW, (cuuint32_t)(g.n_img > 1 ? g.img_rows : kHaloH), 1, 1};
    const int rc = encode_tmap(&xm, a.dtype, 5, a.x, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  {
    const cuuint64_t K = (cuuint64_t)9 * a.Cin;
    cuuint64_t dims[2] = {K, (cuuint64_t)a.Cout};
    cuuint64_t strides[1] = {K * es};
    cuuint32_t box[2] = {64, (cuuint32_t)g.BN};
    const int rc = encode_tmap(&wm, a.dtype, 2, a.w, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  const size_t smem = (size_t)g.halo_slots * kHaloBytes + (size_t)kWRing * g.w_slot_bytes + 1024;
  auto kern = conv3x3_halo_kernel<XT, ST, VT>;
  const cudaError_t e = raise_smem_limit_once<conv3x3_halo_kernel<XT, ST, VT>>(225 * 1024);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "conv_lif: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
  kern<<<(unsigned)grid, kThreadsH, smem, stream>>>(xm, wm, static_cast<const XT *>(a.b), static_cast<const XT *>(a.res),
                                                    static_cast<const VT *>(a.v_init), static_cast<ST *>(a.spikes),
                                                    static_cast<VT *>(a.v_out), g, a.p);
  SNNB_CHECK_LAUNCH("conv3x3_halo");
  return SNNB_OK;
}

template <typename XT>
int dispatch(const ConvArgs &a, cudaStream_t stream) {
  const bool s_u8 = a.lif && a.spike_dtype == SNNB_U8;
  const bool v_f32 = a.lif && a.v_dtype == SNNB_F32;
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(a, stream);
  if (s_u8) return launch<XT, uint8_t, XT>(a, stream);
  if (v_f32) return launch<XT, XT, float>(a, stream);
  return launch<XT, XT, XT>(a, stream);
}

}  // namespace

bool conv3x3_halo_supported(const ConvArgs &a) {
  if (a.dtype != SNNB_BF16 && a.dtype != SNNB_F16) return false;
  if (a.KH != 3 || a.KW != 3 || a.stride != 1 || a.pad != 1) return false;
  if (a.Cin % 64 != 0 || a.Cout % 16 != 0 || a.T > 32) return false;
  if (a.xs_w || a.xs_h || a.xs_b || a.xd_w || a.xd_h) return false;
  if (a.x_t_stride % 8 != 0) return false;
  if (!aligned16(a.x) || !aligned16(a.w) || !aligned16(a.spikes) || (a.b && !aligned16(a.b)) ||
      (a.res && !aligned16(a.res)) || (a.v_init && !aligned16(a.v_init)) || (a.v_out && !aligned16(a.v_out)))
    return false;
  HaloGeom g;
  if (!fill_geom(a, g)) return false;
  return g.Tacc * g.BN <= 512;
}

int conv3x3_halo(const ConvArgs &a, cudaStream_t stream) {
  if (a.dtype == SNNB_BF16) return dispatch<__nv_bfloat16>(a, stream);
  return dispatch<__half>(a, stream);
}

int halo_device_status(int *out) {
  int h = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&h, g_halo_status, sizeof(int));
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_halo_status, &zero, sizeof(int));
  }
  *out = h;
  return SNNB_OK;
}

}  // namespace snnb

