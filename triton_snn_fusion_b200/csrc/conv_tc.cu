// Dense conv / linear (+ bias, + residual) + LIF over T as a tcgen05 implicit GEMM.
//
//   D[pixel][cout] (one fp32 accumulator per timestep, all T resident in tensor memory)
//     = sum over (tap, 64-channel slab) of  A_t[pixel][slab] * W[cout][tap, slab]^T
//
// One CTA owns a tile of up to 128 output pixels x BN output channels for ALL timesteps:
//   warp 4  TMA producer. Per K step it loads the weight tile once and then the activation
//           tile of each timestep, so a weight tile fetched from L2 is reused T times.
//           The activation tile of a (tap, slab) is the output-pixel tile shifted by the
//           tap offset, fetched as a few boxes of a 5-D (C, W, H, B, T) tensor map; TMA's
//           out-of-bounds zero fill is the conv padding. Stride-2 convs read four
//           "phase" views of the input (even/odd rows x even/odd columns), each an
//           ordinary dense tensor map with doubled strides.
//   warp 5  MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16, bf16/f16 in,
//           fp32 accumulate) into accumulator t at TMEM columns [t*BN, (t+1)*BN).
//   warps 0-3  epilogue: thread r owns output pixel r of the tile (TMEM lane r). For each
//           16-channel group it walks t = 0..T-1 in order: tcgen05.ld the accumulator
//           slice, add bias (+ residual[t]), run the LIF update with the membrane
//           potential held in registers across t, and store the spikes; the membrane is
//           written once at the end.
// Shared-memory operands use the 128-byte swizzle (64 16-bit channels per row), which is
// what both TMA writes and the MMA descriptors describe. Every mbarrier wait is bounded:
// on a timeout the CTA raises a device status word, skips the rest of its work, releases
// its tensor memory and exits.
#include <type_traits>

#include "conv.cuh"
#include "tc_epilogue.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace snnb {

static __device__ int g_tc_status = 0;

namespace {

constexpr int kSlotBytes = 16384;  // one 128-row x 128-byte operand tile
constexpr int kMaxSlots = 13;
constexpr int kMaxBoxes = 32;
constexpr int kWSlots = 4;  // weight tiles in flight: a weight load takes longer than one K step of MMAs
constexpr int kEpiWarps = 8;                      // two per TMEM lane quarter, splitting the columns
constexpr int kAProducers = 4;                    // warps that issue activation-tile loads, round robin
constexpr int kProducerWarp = kEpiWarps;          // first activation producer (warps 8..11)
constexpr int kWProducerWarp = kEpiWarps + kAProducers;      // weight-tile producer (warp 12)
constexpr int kMmaWarp = kEpiWarps + kAProducers + 1;        // MMA issuer (warp 13)
constexpr int kThreads = 32 * (kEpiWarps + kAProducers + 2);

struct TcGeom {
  int T, Tacc, B, Cin, Cout, Ho, Wo, KH, KW, stride, pad;
  int BN, BW, BH, nbox, WB, HB;
  long long total_boxes;
  int n_tiles_n, kchunks, slots, lif, tmem_cols, has_res, w_slot_bytes, nprod;
};

template <typename XT, typename ST, typename VT>
__global__ void __launch_bounds__(kThreads)
conv_lif_tc_kernel(const __grid_constant__ CUtensorMap xmap0, const __grid_constant__ CUtensorMap xmap1,
                   const __grid_constant__ CUtensorMap xmap2, const __grid_constant__ CUtensorMap xmap3,
                   const __grid_constant__ CUtensorMap wmap, const XT *__restrict__ bias,
                   const XT *__restrict__ res, const VT *__restrict__ v_init, ST *__restrict__ spikes,
                   VT *__restrict__ v_out, const TcGeom g, const LifParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kMaxSlots + 1 + 2 * kWSlots];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ int box_w0[kMaxBoxes], box_h0[kMaxBoxes], box_b[kMaxBoxes];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x % g.n_tiles_n;
  const long long m_tile = blockIdx.x / g.n_tiles_n;
  const int n0 = n_tile * g.BN;
  const uint32_t smem_base = (umma::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = umma::smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(kMaxSlots + s); };
  const uint32_t acc_bar = bar_base + 8u * (uint32_t)(2 * kMaxSlots);
  auto wfull_bar = [&](int s) { return bar_base + 8u * (uint32_t)(2 * kMaxSlots + 1 + s); };
  auto wempty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(2 * kMaxSlots + 1 + kWSlots + s); };
  // shared memory: a ring of kWSlots weight tiles, then the ring of activation tiles
  const uint32_t w_base = smem_base;
  const uint32_t a_base = smem_base + (uint32_t)kWSlots * (uint32_t)g.w_slot_bytes;
  volatile int *abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < g.slots; ++s) {
      umma::mbar_init(full_bar(s), 1);
      umma::mbar_init(empty_bar(s), 1);
    }
    umma::mbar_init(acc_bar, 1);
    for (int s = 0; s < kWSlots; ++s) {
      umma::mbar_init(wfull_bar(s), 1);
      umma::mbar_init(wempty_bar(s), 1);
    }
    umma::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    umma::tmem_alloc(umma::smem_u32(&tmem_base_s), (uint32_t)g.tmem_cols);
    umma::tmem_relinquish();
  }
  if (warp == kProducerWarp) {
    if (lane == 0) {
      umma::prefetch_tensormap(&xmap0);
      umma::prefetch_tensormap(&wmap);
    }
    for (int j = lane; j < g.nbox; j += 32) {
      const long long gi = m_tile * g.nbox + j;
      if (gi < g.total_boxes) {
        box_w0[j] = (int)(gi % g.WB) * g.BW;
        box_h0[j] = (int)((gi / g.WB) % g.HB) * g.BH;
        box_b[j] = (int)(gi / ((long long)g.WB * g.HB));
      } else {
        box_b[j] = -1;
      }
    }
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  umma::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  const int ksteps = g.KH * g.KW * g.kchunks;
  const uint32_t box_bytes = (uint32_t)(g.BW * g.BH) * 128u;

  if (warp >= kProducerWarp && warp < kProducerWarp + kAProducers) {
    // -------------------------------------------------- TMA producers, activations
    // Activation tiles are numbered n = kstep * Tacc + t; producer p issues tiles p, p + nprod, ... One
    // warp needs several hundred cycles per tile (barrier wait, expect_tx, TMA issue are dependent
    // long-latency steps), more than the MMAs of a tile take, so the issue work is spread over four
    // warps. The loop carries no divisions and no shared-memory reads: ring position, phase and the
    // (tap, slab, t) of the next tile advance incrementally, lane j keeps box j in registers.
    const int p = warp - kProducerWarp;
    const bool mine = lane < g.nbox && box_b[lane] >= 0;
    const int my_w0 = mine ? box_w0[lane] : 0, my_h0 = mine ? box_h0[lane] : 0, my_b = mine ? box_b[lane] : 0;
    const uint32_t my_off = (uint32_t)lane * box_bytes;
    const uint32_t a_bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, mine)) * box_bytes;
    const CUtensorMap *xmaps[4] = {&xmap0, &xmap1, &xmap2, &xmap3};
    const int ntiles = ksteps * g.Tacc;
    int t = 0, c0 = 0, kh = 0, kw = 0;          // state of tile n
    uint32_t slot = 0, phase = 1;               // waiting on parity 1 of a fresh barrier passes at once
    auto advance = [&](int steps) {
      for (int i = 0; i < steps; ++i) {
        if (++t == g.Tacc) {
          t = 0;
          if ((c0 += 64) == g.Cin) {
            c0 = 0;
            if (++kw == g.KW) { kw = 0; ++kh; }
          }
        }
        if (++slot == (uint32_t)g.slots) { slot = 0; phase ^= 1u; }
      }
    };
    advance(p);
    bool ok = true;
    for (int n = p; n < ntiles && p < g.nprod; n += g.nprod) {
      int dh = kh - g.pad, dw = kw - g.pad, which = 0;
      if (g.stride == 2) {
        const int ph = dh & 1, pw = dw & 1;
        which = ph * 2 + pw;
        dh = (dh - ph) / 2;
        dw = (dw - pw) / 2;
      }
      if (lane == 0) {
        ok = umma::mbar_wait(empty_bar(slot), phase, abort_flag);
        if (ok) umma::mbar_expect_tx(full_bar(slot), a_bytes);
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      if (mine)
        umma::tma_load_5d(a_base + slot * kSlotBytes + my_off, xmaps[which], full_bar(slot), c0, my_w0 + dw, my_h0 + dh,
                          my_b, t);
      advance(g.nprod);
    }
  } else if (warp == kWProducerWarp) {
    // ------------------------------------------------------ TMA producer, weights
    if (lane == 0) {
      const uint32_t w_bytes = (uint32_t)g.BN * 128u;
      uint32_t ws = 0, wphase = 1;
      for (int ks = 0; ks < ksteps; ++ks) {
        if (!umma::mbar_wait(wempty_bar(ws), wphase, abort_flag)) break;
        umma::mbar_expect_tx(wfull_bar(ws), w_bytes);
        umma::tma_load_2d(w_base + ws * (uint32_t)g.w_slot_bytes, &wmap, wfull_bar(ws), ks * 64, n0);
        if (++ws == (uint32_t)kWSlots) { ws = 0; wphase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == kMmaWarp) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma::make_idesc_f16(128, g.BN, std::is_same<XT, __nv_bfloat16>::value);
      const uint64_t adesc0 = umma::make_sw128_kmajor_desc(a_base);
      const uint64_t bdesc0 = umma::make_sw128_kmajor_desc(w_base);
      uint32_t slot = 0, phase = 0, ws = 0, wphase = 0;
      bool ok = true;
      for (int ks = 0; ks < ksteps && ok; ++ks) {
        ok = umma::mbar_wait(wfull_bar(ws), wphase, abort_flag);
        if (!ok) break;
        const uint64_t bdesc = bdesc0 + (uint64_t)((ws * (uint32_t)g.w_slot_bytes) >> 4);
        for (int t = 0; t < g.Tacc; ++t) {
          ok = umma::mbar_wait(full_bar(slot), phase, abort_flag);
          if (!ok) break;
          umma::tc_fence_after_sync();
          const uint64_t adesc = adesc0 + (uint64_t)((slot * kSlotBytes) >> 4);
          const uint32_t d = tmem_base + (uint32_t)(t * g.BN);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 4 x K=16 per 64-channel slab: +32 bytes along the swizzled row
            umma::mma_f16_ss(d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (ks > 0 || k > 0) ? 1u : 0u);
          umma::mma_commit(empty_bar(slot));
          if (++slot == (uint32_t)g.slots) { slot = 0; phase ^= 1u; }
        }
        if (ok) umma::mma_commit(wempty_bar(ws));
        if (++ws == (uint32_t)kWSlots) { ws = 0; wphase ^= 1u; }
      }
      if (ok) {
        umma::mma_commit(acc_bar);
        umma::mbar_wait(acc_bar, 0u, abort_flag);  // the accumulators are complete
      }
    }
    __syncwarp();
    // Wake the epilogue warps. They sleep on a hardware named barrier instead of polling the
    // mbarrier: polling warps share issue slots with this warp and the producer and slow them down.
    umma::tc_fence_before_sync();
    asm volatile("bar.arrive 1, %0;" ::"r"(32 * (kEpiWarps + 1)) : "memory");
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    const int r = quarter * 32 + lane;     // row of the tile = output pixel owned by this thread
    const int per_box = g.BW * g.BH;
    const int j = r / per_box, pp = r - j * per_box;
    const int ph = pp / g.BW, pw = pp - ph * g.BW;
    const long long gi = m_tile * g.nbox + j;
    bool valid = (j < g.nbox) && (gi < g.total_boxes);
    long long pix = 0;
    if (valid) {
      const int wo = (int)(gi % g.WB) * g.BW + pw;
      const int ho = (int)((gi / g.WB) % g.HB) * g.BH + ph;
      const long long b = gi / ((long long)g.WB * g.HB);
      valid = (ho < g.Ho) && (wo < g.Wo);
      pix = (b * g.Ho + ho) * g.Wo + wo;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(32 * (kEpiWarps + 1)) : "memory");  // released by the MMA warp
    const bool ok = (*abort_flag == 0);
    umma::tc_fence_after_sync();
    if (ok) {
      // the two warps of a lane quarter split the 16-column groups of the tile
      const int nch = g.BN / 16, half = (nch + 1) / 2;
      const int c_begin = (warp < 4) ? 0 : half;
      const int c_end = (warp < 4) ? half : nch;
      EpiArgs<XT, ST, VT> ea{bias, res, v_init, spikes, v_out, tmem_base + ((uint32_t)(quarter * 32) << 16),
                             pix, (long long)g.B * g.Ho * g.Wo * g.Cout, n0, c_begin, c_end, valid};
      const EpiGeom eg{g.T, g.Tacc, g.BN, g.Cout, g.has_res};
      epilogue_dispatch<XT, ST, VT>(ea, eg, g.lif, p);
    }
  }

  // ------------------------------------------------------------------ teardown
  umma::tc_fence_before_sync();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) atomicExch(&g_tc_status, 1);
  if (warp == kMmaWarp) {
    umma::tc_fence_after_sync();
    umma::tmem_dealloc(tmem_base, (uint32_t)g.tmem_cols);
  }
}

// ------------------------------------------------------------------- host ----
// Output-pixel tile = nbox boxes of BW x BH pixels (<= 128 pixels). Picks the geometry that wastes the
// fewest MMA rows (partial boxes at image edges + unfilled tile rows), mildly preferring fewer boxes.
void choose_boxes(int Ho, int Wo, int &BW, int &BH, int &nbox) {
  double best = -1.0;
  BW = 1; BH = 1; nbox = 1;
  for (int bw = 1; bw <= Wo && bw <= 128; ++bw) {
    for (int bh = 1; bh <= Ho && bw * bh <= 128; ++bh) {
      const int per = bw * bh;
      int nb = 128 / per;
      if (nb > kMaxBoxes) nb = kMaxBoxes;
      const double cover = (double)Wo * Ho / ((double)((Wo + bw - 1) / bw * bw) * ((Ho + bh - 1) / bh * bh));
      const double score = cover * (per * nb / 128.0) - 0.004 * nb;
      if (score > best + 1e-9) {
        best = score;
        BW = bw; BH = bh; nbox = nb;
      }
    }
  }
}

// Output-channel tile: as wide as the T accumulators allow in the 512 TMEM columns (a wider tile
// re-reads the activations fewer times), at most 256.
int pick_bn(int Cout, int Tacc) {
  int bn = Cout >= 256 ? 256 : (Cout >= 128 ? 128 : ((Cout + 15) / 16) * 16);
  while (bn > 16 && Tacc * bn > 512) bn /= 2;
  return bn;
}

template <typename XT, typename ST, typename VT>
int launch(const ConvArgs &a, cudaStream_t stream) {
  TcGeom g;
  g.T = a.T;
  g.Tacc = (a.x_t_stride == 0) ? 1 : a.T;
  g.B = a.B; g.Cin = a.Cin; g.Cout = a.Cout; g.Ho = a.Ho; g.Wo = a.Wo; g.KH = a.KH; g.KW = a.KW;
  g.stride = a.stride; g.pad = a.pad;
  g.BN = pick_bn(a.Cout, g.Tacc);
  choose_boxes(a.Ho, a.Wo, g.BW, g.BH, g.nbox);
  g.WB = (a.Wo + g.BW - 1) / g.BW;
  g.HB = (a.Ho + g.BH - 1) / g.BH;
  g.total_boxes = (long long)a.B * g.WB * g.HB;
  g.n_tiles_n = (a.Cout + g.BN - 1) / g.BN;
  g.kchunks = a.Cin / 64;
  g.lif = a.lif;
  g.has_res = a.res != nullptr;
  int cols = 32;
  while (cols < g.Tacc * g.BN) cols *= 2;
  g.tmem_cols = cols;
  // Shared memory: kWSlots weight tiles + a ring of 16 KB activation tiles. With <= 256 TMEM columns two
  // CTAs can share an SM (one's epilogue overlaps the other's MMAs), so each takes half the budget.
  g.w_slot_bytes = ((g.BN * 128 + 1023) / 1024) * 1024;
  int budget = (cols <= 256 ? 112 : 208) * 1024;
  g.slots = (budget - kWSlots * g.w_slot_bytes) / kSlotBytes;
  if (g.slots < kAProducers + 2) {  // too shallow to share an SM: take the whole SM instead
    budget = 208 * 1024;
    g.slots = (budget - kWSlots * g.w_slot_bytes) / kSlotBytes;
  }
  if (g.slots > kMaxSlots) g.slots = kMaxSlots;
  // A producer only waits on the ring slots of its own tiles, and an mbarrier wait tells phases
  // apart by parity alone. That is sound while no producer can run two laps ahead of the MMA
  // warp, which holds when the ring has more slots than there are producers.
  g.nprod = g.slots - 1 < kAProducers ? g.slots - 1 : kAProducers;
  if (g.nprod < 1) return fail(SNNB_ERR_UNSUPPORTED, "conv_lif: not enough shared memory for the operand ring");
  const long long m_tiles = (g.total_boxes + g.nbox - 1) / g.nbox;
  const long long grid = m_tiles * g.n_tiles_n;
  if (grid > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "conv_lif: problem too large for the grid");

  // ---- tensor maps
  const int es = 2;
  CUtensorMap xm[4], wm;
  const int nphase = a.stride == 2 ? 4 : 1;
  const long long xs_w = a.xs_w ? a.xs_w : a.Cin;
  const long long xs_h = a.xs_h ? a.xs_h : (long long)a.W * a.Cin;
  const long long xs_b = a.xs_b ? a.xs_b : (long long)a.H * a.W * a.Cin;
  const int xd_w = a.xd_w ? a.xd_w : a.W, xd_h = a.xd_h ? a.xd_h : a.H;
  const cuuint64_t frame_bytes = (cuuint64_t)a.B * xs_b * es;
  for (int q = 0; q < 4; ++q) {
    const int ph = nphase == 4 ? q / 2 : 0, pw = nphase == 4 ? q % 2 : 0;
    const int s = a.stride;
    if (q >= nphase) { xm[q] = xm[0]; continue; }
    cuuint64_t dims[5] = {(cuuint64_t)a.Cin, (cuuint64_t)((xd_w - pw + s - 1) / s), (cuuint64_t)((xd_h - ph + s - 1) / s),
                          (cuuint64_t)a.B, (cuuint64_t)g.Tacc};
    cuuint64_t strides[4] = {(cuuint64_t)(s * xs_w * es), (cuuint64_t)(s * xs_h * es), (cuuint64_t)(xs_b * es),
                             g.Tacc > 1 ? (cuuint64_t)a.x_t_stride * es : frame_bytes};
    cuuint32_t box[5] = {64, (cuuint32_t)g.BW, (cuuint32_t)g.BH, 1, 1};
    const char *base = static_cast<const char *>(a.x) + ((size_t)ph * xs_h + (size_t)pw * xs_w) * es;
    const int rc = encode_tmap(&xm[q], a.dtype, 5, base, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  {
    const cuuint64_t K = (cuuint64_t)a.KH * a.KW * a.Cin;
    cuuint64_t dims[2] = {K, (cuuint64_t)a.Cout};
    cuuint64_t strides[1] = {K * es};
    cuuint32_t box[2] = {64, (cuuint32_t)g.BN};
    const int rc = encode_tmap(&wm, a.dtype, 2, a.w, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  const size_t smem = (size_t)g.slots * kSlotBytes + kWSlots * (size_t)g.w_slot_bytes + 1024;
  auto kern = conv_lif_tc_kernel<XT, ST, VT>;
  {
    const cudaError_t e = raise_smem_limit_once<conv_lif_tc_kernel<XT, ST, VT>>(225 * 1024);
    if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "conv_lif: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
  }
  kern<<<(unsigned)grid, kThreads, smem, stream>>>(
      xm[0], xm[1], xm[2], xm[3], wm, static_cast<const XT *>(a.b), static_cast<const XT *>(a.res),
      static_cast<const VT *>(a.v_init), static_cast<ST *>(a.spikes), static_cast<VT *>(a.v_out), g, a.p);
  SNNB_CHECK_LAUNCH("conv_lif_tc");
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

bool conv_lif_tc_supported(const ConvArgs &a, const char **why) {
  *why = "";
  if (a.dtype != SNNB_BF16 && a.dtype != SNNB_F16) { *why = "activations must be bf16 or f16"; return false; }
  if (a.Cin % 64 != 0) { *why = "Cin must be a multiple of 64"; return false; }
  if (a.Cout % 16 != 0) { *why = "Cout must be a multiple of 16"; return false; }
  if (a.KH > 11 || a.KW > 11) { *why = "kernel must be at most 11x11"; return false; }
  if (a.stride != 1 && a.stride != 2) { *why = "stride must be 1 or 2"; return false; }
  if (a.stride == 2 && (a.H < 2 || a.W < 2)) { *why = "stride 2 needs H, W >= 2"; return false; }
  if (a.T > 32) { *why = "T must be at most 32"; return false; }
  if (a.x_t_stride % 8 != 0) { *why = "frame stride must be a multiple of 8 elements"; return false; }
  if (!aligned16(a.x) || !aligned16(a.w) || !aligned16(a.spikes) || (a.b && !aligned16(a.b)) ||
      (a.res && !aligned16(a.res)) || (a.v_init && !aligned16(a.v_init)) || (a.v_out && !aligned16(a.v_out))) {
    *why = "pointers must be 16-byte aligned";
    return false;
  }
  const int tacc = (a.x_t_stride == 0) ? 1 : a.T;
  if (tacc * pick_bn(a.Cout, tacc) > 512) { *why = "T accumulators do not fit tensor memory"; return false; }
  return true;
}

int conv_lif_tc(const ConvArgs &a, cudaStream_t stream) {
  if (a.dtype == SNNB_BF16) return dispatch<__nv_bfloat16>(a, stream);
  return dispatch<__half>(a, stream);
}

}  // namespace snnb

extern "C" int snnb_device_status(int *status_out) {
  using namespace snnb;
  SNNB_CHECK_ARG(status_out != nullptr, "device_status: null pointer");
  int h = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(&h, g_tc_status, sizeof(int));
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  }
  int h2 = 0;
  const int rc = halo_device_status(&h2);
  if (rc != SNNB_OK) return rc;
  int h3 = 0;
  const int rc3 = pair_device_status(&h3);
  if (rc3 != SNNB_OK) return rc3;
  int h4 = 0;
  const int rc4 = stem_device_status(&h4);
  if (rc4 != SNNB_OK) return rc4;
  int h5 = 0;
  const int rc5 = dw_device_status(&h5);
  if (rc5 != SNNB_OK) return rc5;
  *status_out = h | h2 | h3 | h4 | h5;
  return SNNB_OK;
}

