// 3x3 / stride 1 / padding 1 conv (+ bias, + residual) + LIF over T steps (T = 1 or even) with the operand roles
// swapped so that one tcgen05.mma covers 256 output pixels.
//
// Measured on B200: a tcgen05.mma (cta_group::1, K = 16) occupies the tensor pipe for ~128 cycles
// whether its N is 64, 128 or 256, so only N = 256 instructions reach the pipe's rate. With output
// pixels as the M dimension (conv_tc.cu, conv_halo.cu) N is the channel tile and T accumulators of
// 256 columns do not fit the 512 TMEM columns. Here the weight tile is the M operand (128 output
// channels, rows beyond Cout are zero) and the pixels of TWO consecutive timesteps are the N operand:
//
//   D_pair[cout][tq * 128 + pixel] = sum_(tap, slab)  W[cout][tap, slab] . X_(2*pair+tq)[pixel + tap][slab]^T
//
// A CTA owns 8 (wide) x 14 (high) output pixels. Per 64-channel slab and timestep it keeps the
// 10 x 16 input pixels those need (a 20 KB halo tile; out-of-image pixels arrive as zeros = padding);
// the halo tiles of a timestep pair are adjacent in shared memory, so a K-major operand descriptor
// with its start shifted by (kh * 10 + kw) rows and 8-row groups one halo row (1280 bytes) apart
// addresses 32 groups = 16 output rows x 8 pixels for each of the two timesteps (rows 14, 15 of each
// are junk and never stored). All nine taps are read from that one copy.
//
// Maps of at most 7 rows x 8 columns (the last stage of a ResNet) put two images into one tile: image b
// uses row groups 0..6 and image b + 1 groups 8..14, each loaded as a box of 9 halo rows (rows 0..8 and
// 8..16 of the region; rows 8 and 16 are zero padding shared with the neighbour).
//
// Timestep pairs are processed one after the other and alternate between two accumulators: pair 0 (t = 0, 1)
// is accumulated over all slabs and taps into TMEM columns 0..255, pair 1 into 256..511, pair 2 into 0..255
// again, and so on for any even T. The epilogue warps convert pair p (bias, residual, two LIF steps, spikes out)
// while the MMA warp works on pair p + 1 and keep the membrane potentials in registers over all pairs of a tile. TMEM lane = output channel, so a thread owns one
// channel of 64 pixels and a warp's stores cover 32 consecutive channels of one pixel.
#pragma once
#include <type_traits>

#include "conv.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace snnb {

static __device__ int g_pair_status = 0;

namespace {

constexpr int kPW = 10, kPH = 16;                      // halo tile: 10 x 16 pixels
constexpr int kRowBytes = kPW * 128;                   // 1280
constexpr int kHaloT = kPW * kPH * 128;                // 20480 bytes per timestep
constexpr int kTileRows = 14;                          // valid output rows per tile
constexpr int kPairRing = 3;                           // halo (pair) slots
constexpr int kPairRingMax = 4;                        // ... four of the smaller halo-free tiles of 1x1 convs, which each feed one MMA group only
constexpr int kIdentBytes = 192 * 128;                 // zero rows / 64x64 identity / zero rows, see the residual path
constexpr int kWRingP = 5;                             // weight-tile slots (16 KB each): a load must cover ~1 us of L2 latency
constexpr int kWBarsP = 8;                             // barrier pairs reserved for weight slots (the resident form uses six)
constexpr int kWSlot = 128 * 128;
constexpr int kEpiW = 8;
// "twin" mode (3x3 / stride 1 conv with at most 64 output channels): see PairGeom::twin
constexpr int kTwinIdentBytes = 128 * 128;             // identity rows for D1, zero rows for D2
constexpr int kEpiWTwin = 16;                          // twin mode runs 16 epilogue warps of 16 pixels each
constexpr int kXchgWarp = 32 * 64;                     // one epilogue warp's outgoing values of one timestep: 16 floats per lane
constexpr int kXchgBytes = kEpiWTwin * kXchgWarp;      // 32768
// warp roles: epilogue warps first, then halo producer, weight producer, MMA issuer
template <bool TWIN> struct Roles {
  static constexpr int kEpi = TWIN ? kEpiWTwin : kEpiW;
  static constexpr int kHalo = kEpi, kW = kEpi + 1, kMma = kEpi + 2;
  static constexpr int kThreads = 32 * (kEpi + 3);
};

struct PairGeom {
  int T, Tacc, B, Cin, Cout, Ho, Wo;
  int kslabs, npairs, tq;   // tq = timesteps per pair (1 or 2)
  int n_tiles_n, row_tiles, w_strips;
  int tmem_cols, lif, has_res, total_tiles;
  int s2;         // 3x3 / stride 2 / padding 1: per slab four halo tiles, one per phase (row parity a, column
                  // parity b) of the input, each seen through a tensor map with doubled strides; input row
                  // 2i - 1 + kh is phase row i - 1 (kh = 0, a = 1), i (kh = 1, a = 0) or i (kh = 2, a = 1)
  int ntaps;      // 9 (3x3 conv) or 1 (1x1 conv / linear: only the centre of the halo tile is used)
  int sc_slabs;   // > 0: instead of a residual tensor, a 1x1 shortcut conv over sc_slabs 64-channel slabs of a
                  // second input is accumulated (its pixel tiles come through rmap, its weights through scwmap)
  int flat;       // 1x1 conv on a map of at least 16 rows: the pixel tile is loaded without a halo (8 x 16 pixels, all
                  // of them outputs) instead of as the centre of a 10 x 16 halo tile
  int pw;         // pixels per tile row in shared memory: 10 (with halo) or 8 (flat)
  int row_bytes;  // pw * 128
  int halo_t;     // bytes of one timestep's tile: pw * 16 * 128
  int tile_rows;  // output rows a tile produces: 14 (with halo) or 16 (flat)
  int ring;   // halo slots in use
  int wring;  // weight slots in use (<= kWBarsP)
  int wres;   // twin form without residual, one channel slab: the six weight tiles (96 KB) are loaded once per block and
              // stay in shared memory for all its tiles (two halo slots instead of three make the room)
  int stack;  // maps of at most 7 x 8: two images per tile, image b in row groups 0.., image b + 1 in groups 8..
              // (halo rows 0..8 and 8..16 of a timestep's region: row 8 is the zero padding of both, row 16
              // is row 0 of the next region, which is the zero top padding of whatever is stored there)
  int twin;   // 3x3 / stride 1 with Cout <= 64 (the TWIN instantiation of the kernel): instead of duplicating the 64
              // weight rows, the M rows carry the weights of TWO kernel rows against the same pixel operand. M rows
              // [0,32) and [64,96) ("D1", channels 0..31 / 32..63) hold kernel row 0, rows [32,64) and [96,128)
              // ("D2", same channels) kernel row 1, both multiplied with halo row R for pixel row R; three more
              // groups hold zeros in D1 and kernel row 2 in D2 and read halo row R + 1. Then
              // out[R] = D1[R] + D2[R + 1]: 6 MMA groups per slab instead of 9. In TMEM each lane quarter holds one
              // of D1 / D2 for 32 channels; the warps of quarters q and q ^ 1 pass each other through shared memory
              // the halves the other one needs and each runs the LIF for a quarter of the tile's rows.
  int stage_off;   // twin: byte offset of the exchange buffers from the aligned start of dynamic shared memory
  int dup;    // Cout <= 64 (shapes twin mode does not take): the 64 weight rows are loaded twice (M rows 64..127 repeat 0..63) so that all
              // eight epilogue warps can read the accumulator and split the pixels four ways
  long long wait_limit;   // bound of every mbarrier wait, in SM cycles (about two seconds unless a self-test shortens it)
  int drop_load;          // self-test: CTA 0 announces its first weight tile but never loads it, so that its waits run out
  int own;    // v_init and v_out are the same buffer: a tile that was shifted back inside the image leaves the
              // pixels it shares with its neighbour to that neighbour (no load, no store), so every membrane
              // value is read and written by exactly one thread
};

// The taps served by halo tile `ph` of a slab: all of them for stride 1 (ph = 0); for stride 2 the taps
// whose input rows / columns have the parity of phase ph = 2a + b.
template <bool S2, bool TWIN>
__device__ __forceinline__ int phase_ntaps(const PairGeom &g, int ph) {
  return S2 ? ((ph & 2) ? 2 : 1) * ((ph & 1) ? 2 : 1) : (TWIN ? 6 : g.ntaps);
}
// j-th tap of phase ph: its index in the weight tensor (kh * 3 + kw) and its row offset inside the halo tile.
template <bool S2, bool TWIN>
__device__ __forceinline__ void phase_tap(const PairGeom &g, int ph, int j, int &wtap, int &off) {
  if constexpr (!S2) {
    if constexpr (TWIN) {
      // group j < 3: kernel rows 0 (D1 rows) and 1 (D2 rows) against halo row R of pixel row R; group j >= 3:
      // zero weights (D1 rows) and kernel row 2 (D2 rows) against halo row R + 1. With out[R] = D1[R] + D2[R + 1]
      // every (kernel row, halo row) product lands once, and no accumulator that is used reads past the halo
      // tile. wtap = kernel column.
      wtap = j < 3 ? j : j - 3;
      off = (j < 3 ? 0 : kPW) + wtap;
      return;
    }
    const int kh = g.ntaps == 1 ? 1 : j / 3, kw = g.ntaps == 1 ? 1 : j - kh * 3;
    wtap = g.ntaps == 1 ? 0 : j;
    off = g.flat ? 0 : kh * kPW + kw;
  } else {
    const int a = ph >> 1, b = ph & 1, nc = b ? 2 : 1;
    const int jr = j / nc, jc = j - jr * nc;
    const int kh = a ? (jr ? 2 : 0) : 1, kw = b ? (jc ? 2 : 0) : 1;
    const int du = (a && jr == 0) ? -1 : 0, dv = (b && jc == 0) ? -1 : 0;   // phase pixel relative to the output pixel
    wtap = kh * 3 + kw;
    off = (du + 1) * kPW + (dv + 1);
  }
}

// LIF flavours compiled into the epilogue: the common one (tau a power of two, hard reset) with its
// branches resolved at compile time, every other kind through the run-time lif_step, or no LIF.
enum : int { kLifFast = 0, kLifAny = 1, kLifOff = 2 };

// Where this thread's 64 pixels of the current tile live in the output.
struct PixMap {
  long long row0_off;   // element offset of (tile row 0 of this thread, column w0, channel c) inside a frame
  int row_stride;       // Wo * Cout
  int Cout;
  int rows_ok;          // bit r set: this thread's r-th tile row (0..7) exists in the image and in the tile
  int cols_ok;          // bit j set: column w0 + j exists
};

// Converts one timestep pair for the 64 pixels of this thread's channel: TMEM -> + bias (+ residual)
// -> LIF (membrane in v[]) -> spikes. TQ2: the pair holds two timesteps; RES: a residual is added.
// General version: every pixel is predicated on the tile / image edges.
template <typename XT, typename ST, int KIND, bool TQ2, bool RES, int NV>
__device__ __forceinline__ void pair_epilogue(const LifParams &p, uint32_t tmem_addr, float bias_c,
                                              const XT *__restrict__ res, ST *__restrict__ out, long long frame_out,
                                              const PixMap &pm, float (&v)[NV], int nchunks) {
  // out / res already point at (timestep t0 of the pair, this thread's first row, column w0, channel c)
#pragma unroll
  for (int chunk = 0; chunk < NV / 16; ++chunk) {
    if (chunk < nchunks) {   // warp-uniform; written as a guard so that the loop stays fully unrolled
    uint32_t a0[16], a1[16];
    umma::tmem_ld_x16(tmem_addr + (uint32_t)(chunk * 16), a0);
    if (TQ2) umma::tmem_ld_x16(tmem_addr + (uint32_t)(128 + chunk * 16), a1);
    umma::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int r = chunk * 2 + (i >> 3), j = i & 7;   // a chunk of 16 pixels is two tile rows of 8
      const bool ok = ((pm.rows_ok >> r) & 1) && ((pm.cols_ok >> j) & 1);
      const long long o = pm.row0_off + (long long)r * pm.row_stride + j * pm.Cout;
      float y0 = __uint_as_float(a0[i]) + bias_c;
      float y1 = TQ2 ? __uint_as_float(a1[i]) + bias_c : 0.f;
      if (ok) {
        if (RES && res != nullptr) {
          y0 += DT<XT>::to_f(res[o]);
          if (TQ2) y1 += DT<XT>::to_f(res[o + frame_out]);
        }
        if constexpr (KIND == kLifOff) {
          reinterpret_cast<XT *>(out)[o] = DT<XT>::from_f(y0);
          if (TQ2) reinterpret_cast<XT *>(out)[o + frame_out] = DT<XT>::from_f(y1);
        } else {
          float &vv = v[chunk * 16 + i];
          const float s0 = (KIND == kLifFast) ? lif_step_t<1, true>(y0, vv, p) : lif_step(y0, vv, p);
          out[o] = DT<ST>::from_f(s0);
          if (TQ2) {
            const float s1 = (KIND == kLifFast) ? lif_step_t<1, true>(y1, vv, p) : lif_step(y1, vv, p);
            out[o + frame_out] = DT<ST>::from_f(s1);
          }
        }
      }
    }
    }
  }
}

// Hot version: two timesteps, tau a power of two, hard reset, a valid channel and a tile that lies
// completely inside the image, so nothing is predicated. NROWS = tile rows of this thread. The tile
// grid is laid out so that (for maps of at least 14 x 8) every tile is such a tile.
// Code size matters here: eight warps stream through this body once per pair, and when all of a
// thread's pixels are unrolled (several thousand instructions) the warps mostly wait for instruction
// fetch. So the loop over 16-pixel chunks stays a real loop. The membrane potentials must be
// registers, which cannot be indexed by the loop counter: each trip works on v[0..15] and then
// rotates the thread's NROWS * 8 potentials by 16, so they are back in place after the last trip.
template <typename XT, typename ST, int NROWS, int NV>
__device__ __forceinline__ void pair_epilogue_full(const LifParams &p, uint32_t tmem_addr, float bias_c,
                                                   ST *__restrict__ out, long long frame_out, const PixMap &pm,
                                                   float (&v)[NV]) {
  constexpr int NPIX = NROWS * 8;
  ST *p0 = out + pm.row0_off;
  ST *p1 = p0 + frame_out;
  const int two_rows = 2 * pm.row_stride;
#pragma unroll 1
  for (int chunk = 0; chunk < NROWS / 2; ++chunk) {
    uint32_t a0[16], a1[16];
    umma::tmem_ld_x16(tmem_addr, a0);
    umma::tmem_ld_x16(tmem_addr + 128u, a1);
    umma::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int o = (i >> 3) * pm.row_stride + (i & 7) * pm.Cout;   // fits 32 bits: one tile
      const float s0 = lif_step_t<1, true>(__uint_as_float(a0[i]) + bias_c, v[i], p);
      const float s1 = lif_step_t<1, true>(__uint_as_float(a1[i]) + bias_c, v[i], p);
      p0[o] = DT<ST>::from_f(s0);
      p1[o] = DT<ST>::from_f(s1);
    }
    if (NPIX > 16) {
      float head[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) head[i] = v[i];
#pragma unroll
      for (int i = 0; i < NPIX - 16; ++i) v[i] = v[i + 16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[NPIX - 16 + i] = head[i];
    }
    p0 += two_rows;
    p1 += two_rows;
    tmem_addr += 16u;
  }
}

// ---------------------------------------------------------------------------------------------------------
// Lean epilogue bodies for the common case: two timesteps per pair, tau a power of two, hard reset to zero, a
// tile that lies completely inside the image. Two neighbouring pixels share each packed-fp32 instruction, the
// chunk loop is unrolled (no register rotation), and with COUT known at compile time every store address is
// "row pointer + constant" (COUT = 0: the stride is a run-time value).
//
// h = v + (y - v) * inv_tau: the product with a power of two is exact, so the fused multiply-add rounds the same
// sum as lif_step's separately rounded multiply and add; with s in {0, 1}, h - s * h is exactly 0 or h.
__device__ __forceinline__ float2 lif_fast2(float2 y, float &vx, float &vy, float v_th, float2 inv_tau2) {
  const float2 v = make_float2(vx, vy);
  const float2 d = __fadd2_rn(y, make_float2(-vx, -vy));
  const float2 h = __ffma2_rn(d, inv_tau2, v);
  const float2 s = make_float2(h.x >= v_th ? 1.f : 0.f, h.y >= v_th ? 1.f : 0.f);
  const float2 vn = __ffma2_rn(make_float2(-s.x, -s.y), h, h);
  vx = vn.x;
  vy = vn.y;
  return s;
}

template <typename ST, int NROWS, int COUT, int NV>
__device__ __forceinline__ void pair_epilogue_lean(const LifParams &p, uint32_t tmem_addr, float bias_c,
                                                   ST *__restrict__ out, long long frame_out, const PixMap &pm,
                                                   float (&v)[NV]) {
  constexpr int NCH = NROWS / 2;   // chunks of 16 pixels = two tile rows
  const float2 b2 = make_float2(bias_c, bias_c), it2 = make_float2(p.inv_tau, p.inv_tau);
  const float v_th = p.v_th;
  const int cs = COUT ? COUT : pm.Cout;
  ST *row = out + pm.row0_off;
  uint32_t ab[2][2][16];   // [buffer][timestep][pixel]: the next 16 pixels travel while these are evaluated
  umma::tmem_ld_x16(tmem_addr, ab[0][0]);
  umma::tmem_ld_x16(tmem_addr + 128u, ab[0][1]);
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    umma::tmem_ld_wait();
    uint32_t (&a)[2][16] = ab[c & 1];
    if (c + 1 < NCH) {
      umma::tmem_ld_x16(tmem_addr + (uint32_t)((c + 1) * 16), ab[(c + 1) & 1][0]);
      umma::tmem_ld_x16(tmem_addr + (uint32_t)(128 + (c + 1) * 16), ab[(c + 1) & 1][1]);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      ST *q0 = row, *q1 = row + frame_out;
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const int i = rr * 8 + j, k = c * 16 + i;
        const float2 y0 = __fadd2_rn(make_float2(__uint_as_float(a[0][i]), __uint_as_float(a[0][i + 1])), b2);
        const float2 y1 = __fadd2_rn(make_float2(__uint_as_float(a[1][i]), __uint_as_float(a[1][i + 1])), b2);
        const float2 s0 = lif_fast2(y0, v[k], v[k + 1], v_th, it2);
        const float2 s1 = lif_fast2(y1, v[k], v[k + 1], v_th, it2);
        q0[j * cs] = DT<ST>::from_f(s0.x);
        q0[(j + 1) * cs] = DT<ST>::from_f(s0.y);
        q1[j * cs] = DT<ST>::from_f(s1.x);
        q1[(j + 1) * cs] = DT<ST>::from_f(s1.y);
      }
      row += pm.row_stride;
    }
  }
}

template <typename ST, int NROWS, int NV>
__device__ __forceinline__ void pair_epilogue_lean_any(const LifParams &p, uint32_t tmem_addr, float bias_c,
                                                       ST *__restrict__ out, long long frame_out, const PixMap &pm,
                                                       float (&v)[NV]) {
  switch (pm.Cout) {
    case 128: pair_epilogue_lean<ST, NROWS, 128, NV>(p, tmem_addr, bias_c, out, frame_out, pm, v); break;
    default: pair_epilogue_lean<ST, NROWS, 0, NV>(p, tmem_addr, bias_c, out, frame_out, pm, v); break;
  }
}

// Exchange buffers of twin mode: 64 bytes per lane (16 floats), the four 16-byte pieces of a lane stored at
// piece ^ ((lane >> 1) & 3) so that the 16-byte accesses of eight neighbouring lanes fall on different banks.
__device__ __forceinline__ uint32_t xchg_piece(uint32_t lane_row, int lane, int q) {
  return lane_row + (uint32_t)((q ^ ((lane >> 1) & 3)) << 4);
}

// Twin mode, same case: one timestep for this thread's 16 pixels (64 output channels: the pixel stride is a
// constant). Own accumulator half (tensor memory) + the partner's half (shared memory) + bias -> LIF -> spikes.
template <typename ST>
__device__ __forceinline__ void twin_step_lean(const LifParams &p, uint32_t tmem_addr, uint32_t in_row, int lane,
                                               float bias_c, ST *__restrict__ out, const PixMap &pm, float (&v)[16]) {
  constexpr int cs = 64;
  const float2 b2 = make_float2(bias_c, bias_c), it2 = make_float2(p.inv_tau, p.inv_tau);
  const float v_th = p.v_th;
  uint32_t a[16];
  float d[16];
  umma::tmem_ld_x16(tmem_addr, a);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(d[4 * q]), "=f"(d[4 * q + 1]), "=f"(d[4 * q + 2]), "=f"(d[4 * q + 3])
                 : "r"(xchg_piece(in_row, lane, q)));
  umma::tmem_ld_wait();
  ST *row = out + pm.row0_off;
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      const int i = rr * 8 + j;
      const float2 acc = __fadd2_rn(make_float2(__uint_as_float(a[i]), __uint_as_float(a[i + 1])), make_float2(d[i], d[i + 1]));
      const float2 s = lif_fast2(__fadd2_rn(acc, b2), v[i], v[i + 1], v_th, it2);
      row[j * cs] = DT<ST>::from_f(s.x);
      row[(j + 1) * cs] = DT<ST>::from_f(s.y);
    }
    row += pm.row_stride;
  }
}

// Twin mode, any case: every pixel predicated on the tile / image edges and on the channel count.
template <typename XT, typename ST, int KIND>
__device__ __forceinline__ void twin_step(const LifParams &p, uint32_t tmem_addr, uint32_t in_row, int lane, float bias_c,
                                          ST *__restrict__ out, const PixMap &pm, float (&v)[16]) {
  uint32_t a[16];
  float d[16];
  umma::tmem_ld_x16(tmem_addr, a);
#pragma unroll
  for (int q = 0; q < 4; ++q)
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(d[4 * q]), "=f"(d[4 * q + 1]), "=f"(d[4 * q + 2]), "=f"(d[4 * q + 3])
                 : "r"(xchg_piece(in_row, lane, q)));
  umma::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int r = i >> 3, j = i & 7;   // 16 pixels are two tile rows of 8
    const bool ok = ((pm.rows_ok >> r) & 1) && ((pm.cols_ok >> j) & 1);
    const long long o = pm.row0_off + (long long)r * pm.row_stride + j * pm.Cout;
    const float y = (__uint_as_float(a[i]) + d[i]) + bias_c;
    if (ok) {
      if constexpr (KIND == kLifOff) {
        reinterpret_cast<XT *>(out)[o] = DT<XT>::from_f(y);
      } else {
        const float s = (KIND == kLifFast) ? lif_step_t<1, true>(y, v[i], p) : lif_step(y, v[i], p);
        out[o] = DT<ST>::from_f(s);
      }
    }
  }
}

// DUP: the instantiation for duplicated weight rows at stride 1 (a thread owns four tile rows, 32 membrane values);
// strided convs with at most 64 outputs run the S2 instantiation, which handles that case at run time.
template <typename XT, typename ST, typename VT, bool S2, bool TWIN, bool DUP>
__global__ void __launch_bounds__(Roles<TWIN>::kThreads)
conv3x3_pair_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                    const __grid_constant__ CUtensorMap rmap, const __grid_constant__ CUtensorMap wmap64,
                    const __grid_constant__ CUtensorMap scwmap, const __grid_constant__ CUtensorMap xmap01,
                    const __grid_constant__ CUtensorMap xmap10, const __grid_constant__ CUtensorMap xmap11,
                    const XT *__restrict__ bias, const XT *__restrict__ bias2, const VT *v_init,
                    ST *__restrict__ spikes, VT *v_out, const PairGeom g, const LifParams p) {
  using R = Roles<TWIN>;
  const bool dup = DUP || (S2 && g.dup);
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kPairRingMax + 2 * kWBarsP + 4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  umma::pdl_trigger();   // the next kernel's blocks may take over SMs as this grid drains; they wait for its end themselves

  const uint32_t smem_base = (umma::smem_u32(smem_raw) + 1023u) & ~1023u;
  // [identity block (residual path only)] [weight ring] [halo ring]
  const uint32_t ident_base = smem_base;
  const uint32_t w_base = smem_base + ((g.has_res && !g.sc_slabs) ? (uint32_t)(TWIN ? kTwinIdentBytes : kIdentBytes) : 0u);
  const uint32_t h_base = w_base + (uint32_t)(g.wring * kWSlot);
  const uint32_t slot_bytes = (uint32_t)(g.tq * g.halo_t);
  const uint32_t bar_base = umma::smem_u32(bars);
  auto hfull = [&](uint32_t s) { return bar_base + 8u * s; };
  auto hempty = [&](uint32_t s) { return bar_base + 8u * ((uint32_t)kPairRingMax + s); };
  auto wfull = [&](uint32_t s) { return bar_base + 8u * (2u * kPairRingMax + s); };
  auto wempty = [&](uint32_t s) { return bar_base + 8u * (2u * kPairRingMax + kWBarsP + s); };
  auto accfull = [&](uint32_t s) { return bar_base + 8u * (2u * kPairRingMax + 2u * kWBarsP + s); };
  auto accempty = [&](uint32_t s) { return bar_base + 8u * (2u * kPairRingMax + 2u * kWBarsP + 2u + s); };
  volatile int *abort_flag = &abort_s;
  const long long wl = g.wait_limit;   // SM cycles after which a wait on an mbarrier gives up

  // A CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; tile index -> (image, row tile, column
  // strip, channel tile) with the channel tile fastest so neighbouring CTAs share their halo tiles in L2.
  // wlo / hlo: first column / row of the tile that no other tile computes
  auto decode = [&](int tile, int &n0, int &w0, int &h0, int &b, int &wlo, int &hlo) {
    const int n_tile = tile % g.n_tiles_n;
    int m = tile / g.n_tiles_n;
    if (g.stack) {   // a tile is a pair of whole images
      n0 = n_tile * 128; w0 = 0; h0 = 0; b = 2 * m; wlo = 0; hlo = 0;
      return;
    }
    const int strip = m % g.w_strips;
    m /= g.w_strips;
    const int rt = m % g.row_tiles;
    b = m / g.row_tiles;
    n0 = n_tile * 128;
    // The last strip / row tile is shifted back inside the image instead of sticking out of it: it then
    // recomputes a few pixels of its neighbour (both write the same values) and every tile is complete.
    w0 = min(strip * 8, max(g.Wo - 8, 0));
    h0 = min(rt * g.tile_rows, max(g.Ho - g.tile_rows, 0));
    wlo = strip * 8;
    hlo = rt * g.tile_rows;
  };

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < g.ring; ++s) { umma::mbar_init(hfull(s), 1); umma::mbar_init(hempty(s), 1); }
    for (int s = 0; s < g.wring; ++s) { umma::mbar_init(wfull(s), 1); umma::mbar_init(wempty(s), 1); }
    for (int s = 0; s < 2; ++s) { umma::mbar_init(accfull(s), 1); umma::mbar_init(accempty(s), R::kEpi); }
    umma::fence_mbar_init();
  }
  if (warp == R::kMma) {
    umma::tmem_alloc(umma::smem_u32(&tmem_base_s), (uint32_t)g.tmem_cols);
    umma::tmem_relinquish();
  }
  if (warp == R::kHalo && lane == 0) {
    umma::prefetch_tensormap(&xmap);
    umma::prefetch_tensormap(&wmap);
    if (g.has_res) umma::prefetch_tensormap(&rmap);
    if (g.sc_slabs) umma::prefetch_tensormap(&scwmap);
  }
  if (g.has_res && !g.sc_slabs && warp < R::kEpi) {
    // Residual add on the tensor cores: D += I . R with a 64x64 identity as the weight operand. The block
    // is 192 rows of 128 bytes: 64 zero rows, the identity (row 64 + k has a one in column k, stored where
    // the 128-byte swizzle puts it), 64 zero rows. Read from row 64 it is [I; 0] (channels n0..n0+63 of the
    // tile), read from row 0 it is [0; I] (channels n0+64..n0+127).
    uint4 *blk = reinterpret_cast<uint4 *>(smem_raw + (ident_base - umma::smem_u32(smem_raw)));
    const int ident_bytes = TWIN ? kTwinIdentBytes : kIdentBytes;
    for (int i = threadIdx.x; i < ident_bytes / 16; i += 32 * R::kEpi) blk[i] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("bar.sync 2, %0;" ::"r"(32 * R::kEpi) : "memory");
    if (dup ? threadIdx.x < 128 : threadIdx.x < 64) {
      // dup mode: rows 0..127 carry the identity twice (row r has its one in column r % 64); twin mode: the D1 row
      // of channel k (row k for k < 32, row k + 32 above) has its one in column k, the D2 rows stay zero
      const int k = threadIdx.x & 63, r = dup ? (int)threadIdx.x : (TWIN ? (k < 32 ? k : k + 32) : 64 + k);
      uint8_t *row = smem_raw + (ident_base - umma::smem_u32(smem_raw)) + r * 128;
      *reinterpret_cast<XT *>(row + (((k >> 3) ^ (r & 7)) << 4) + (k & 7) * 2) = DT<XT>::from_f(1.0f);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // make the writes visible to the MMA unit
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  umma::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  // Set-up (barriers, tensor memory, identity tile, tensor-map prefetch) is done; from here on the kernel reads
  // what its predecessor in the stream wrote and writes buffers that predecessor may read.
  umma::pdl_wait();

  if (warp == R::kHalo) {
    // ------------------------------------------------- halo producer: lane q loads timestep q of the pair
    // bytes one slot receives: a full halo per timestep, or (two images per tile) a box of 9 rows per image
    auto tx_bytes = [&](int b) {
      return g.stack ? (uint32_t)g.tq * (uint32_t)(b + 1 < g.B ? 2 : 1) * 9u * (uint32_t)kRowBytes : slot_bytes;
    };
    uint32_t slot = 0, phase = 1;
    bool ok = true;
    const int org = g.flat ? 0 : 1;   // the halo tile starts one pixel up and to the left of the output tile
    constexpr int nph = S2 ? 4 : 1;
    for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x) {
      int n0, w0, h0, b, wlo_unused, hlo_unused;
      decode(tile, n0, w0, h0, b, wlo_unused, hlo_unused);
      for (int pair = 0; pair < g.npairs && ok; ++pair) {
        for (int sp = 0; sp < g.kslabs * nph && ok; ++sp) {
          const int slab = sp / nph, ph = sp - slab * nph;
          const CUtensorMap *xm = ph == 0 ? &xmap : (ph == 1 ? &xmap01 : (ph == 2 ? &xmap10 : &xmap11));
          if (lane == 0) {
            ok = umma::mbar_wait(hempty(slot), phase, abort_flag, wl);
            if (ok) umma::mbar_expect_tx(hfull(slot), tx_bytes(b));
          }
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          if (!ok) break;
          if (lane < g.tq) {
            const uint32_t dst = h_base + slot * slot_bytes + (uint32_t)lane * (uint32_t)g.halo_t;
            umma::tma_load_5d(dst, xm, hfull(slot), slab * 64, w0 - org, h0 - org, b, pair * g.tq + lane);
            if (g.stack && b + 1 < g.B)
              umma::tma_load_5d(dst + 8u * kRowBytes, xm, hfull(slot), slab * 64, -1, -1, b + 1, pair * g.tq + lane);
          }
          if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
        }
        // residual tiles of this pair: one per 64-channel half of the output-channel tile; with a shortcut
        // conv instead: one pixel tile of the shortcut input per 64-channel slab of ITS channels
        const int n_res = g.sc_slabs ? g.sc_slabs : 2;
        for (int rs = 0; rs < n_res && g.has_res && ok; ++rs) {
          if (!g.sc_slabs && n0 + rs * 64 >= g.Cout) break;
          const int res_c0 = g.sc_slabs ? rs * 64 : n0 + rs * 64;
          if (lane == 0) {
            ok = umma::mbar_wait(hempty(slot), phase, abort_flag, wl);
            if (ok) umma::mbar_expect_tx(hfull(slot), tx_bytes(b));
          }
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          if (!ok) break;
          if (lane < g.tq) {
            const uint32_t dst = h_base + slot * slot_bytes + (uint32_t)lane * (uint32_t)g.halo_t;
            umma::tma_load_5d(dst, &rmap, hfull(slot), res_c0, w0 - org, h0 - org, b, pair * g.tq + lane);
            if (g.stack && b + 1 < g.B)
              umma::tma_load_5d(dst + 8u * kRowBytes, &rmap, hfull(slot), res_c0, -1, -1, b + 1, pair * g.tq + lane);
          }
          if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == R::kW) {
    // ---------------------------------------------------------- weight producer
    if (lane == 0) {
      uint32_t ws = 0, wphase = 1;
      bool ok = true;
      for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x) {
        const int n0 = (tile % g.n_tiles_n) * 128;
        for (int pair = 0; pair < g.npairs && ok; ++pair) {
          if (TWIN && g.wres && (tile != (int)blockIdx.x || pair != 0)) continue;   // resident weights: loaded once
          for (int sp = 0; sp < g.kslabs * (S2 ? 4 : 1) && ok; ++sp) {
            const int slab = S2 ? sp >> 2 : sp, ph = S2 ? sp & 3 : 0;
            for (int j = 0; j < phase_ntaps<S2, TWIN>(g, ph); ++j) {
              int tap, off_unused;
              phase_tap<S2, TWIN>(g, ph, j, tap, off_unused);
              ok = umma::mbar_wait(wempty(ws), wphase, abort_flag, wl);
              if (!ok) break;
              umma::mbar_expect_tx(wfull(ws), (uint32_t)kWSlot);
              if (g.drop_load && blockIdx.x == 0 && tile == (int)blockIdx.x && pair == 0 && sp == 0 && j == 0) {
                // self-test of the bounded waits: this tile never arrives
              } else if (TWIN) {
                // M rows [0,32) / [64,96) (D1 of channels 0..31 / 32..63): kernel tap (0, kw), or zeros (a box past
                // the end of the tensor) in the second three groups; rows [32,64) / [96,128) (D2 of the same
                // channels): tap (1, kw), then tap (2, kw)
                const int kx = j < 3 ? tap * g.Cin + slab * 64 : 9 * g.Cin;
                const int kx2 = ((j < 3 ? 3 : 6) + tap) * g.Cin + slab * 64;
                const uint32_t dst = w_base + ws * (uint32_t)kWSlot;
                umma::tma_load_2d(dst, &wmap64, wfull(ws), kx, 0);
                umma::tma_load_2d(dst + 32u * 128u, &wmap64, wfull(ws), kx2, 0);
                umma::tma_load_2d(dst + 64u * 128u, &wmap64, wfull(ws), kx, 32);
                umma::tma_load_2d(dst + 96u * 128u, &wmap64, wfull(ws), kx2, 32);
              } else if (dup) {   // the same 64 rows into both halves of the tile
                umma::tma_load_2d(w_base + ws * (uint32_t)kWSlot, &wmap64, wfull(ws), tap * g.Cin + slab * 64, 0);
                umma::tma_load_2d(w_base + ws * (uint32_t)kWSlot + 64u * 128u, &wmap64, wfull(ws), tap * g.Cin + slab * 64, 0);
              } else {
                umma::tma_load_2d(w_base + ws * (uint32_t)kWSlot, &wmap, wfull(ws), tap * g.Cin + slab * 64, n0);
              }
              if (++ws == (uint32_t)g.wring) { ws = 0; wphase ^= 1u; }
            }
          }
          // shortcut conv: its weight tiles follow the pair's main-conv tiles, one per slab of the shortcut input
          for (int rs = 0; rs < g.sc_slabs && ok; ++rs) {
            ok = umma::mbar_wait(wempty(ws), wphase, abort_flag, wl);
            if (!ok) break;
            umma::mbar_expect_tx(wfull(ws), (uint32_t)kWSlot);
            umma::tma_load_2d(w_base + ws * (uint32_t)kWSlot, &scwmap, wfull(ws), rs * 64, n0);
            if (++ws == (uint32_t)g.wring) { ws = 0; wphase ^= 1u; }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == R::kMma) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma::make_idesc_f16(128, 128 * g.tq, std::is_same<XT, __nv_bfloat16>::value);
      uint64_t hdesc0 = umma::make_sw128_kmajor_desc(h_base);
      hdesc0 = (hdesc0 & ~((uint64_t)0x3FFF << 32)) | ((uint64_t)(g.row_bytes >> 4) << 32);
      const uint64_t wdesc0 = umma::make_sw128_kmajor_desc(w_base);
      uint32_t slot = 0, phase = 0, ws = 0, wphase = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x, ++it) {
        for (int pair = 0; pair < g.npairs && ok; ++pair) {
          // Timestep pairs alternate between the two accumulators (columns 0..255 and 256..511). `use` counts
          // how often this accumulator has been filled so far: even pairs use the first one, odd pairs the second.
          const uint32_t acc = (uint32_t)(pair & 1);
          const uint32_t use = it * (uint32_t)((g.npairs + 1 - (int)acc) >> 1) + (uint32_t)(pair >> 1);
          // the epilogue warps must have drained this accumulator (its previous use) before it is overwritten
          ok = umma::mbar_wait(accempty(acc), (use & 1u) ^ 1u, abort_flag, wl);
          if (!ok) break;
          umma::tc_fence_after_sync();
          const uint32_t d = tmem_base + acc * 256u;
          for (int sp = 0; sp < g.kslabs * (S2 ? 4 : 1) && ok; ++sp) {
            const int ph = S2 ? sp & 3 : 0;
            ok = umma::mbar_wait(hfull(slot), phase, abort_flag, wl);
            if (!ok) break;
            for (int tap = 0; tap < phase_ntaps<S2, TWIN>(g, ph); ++tap) {
              // resident weights: slot = tap, complete after the first pass over the six slots
              if (!(TWIN && g.wres) || (it == 0 && pair == 0)) ok = umma::mbar_wait(wfull(ws), wphase, abort_flag, wl);
              if (!ok) break;
              umma::tc_fence_after_sync();
              int wtap_unused, off;
              phase_tap<S2, TWIN>(g, ph, tap, wtap_unused, off);
              const uint64_t xdesc = hdesc0 + (uint64_t)((slot * slot_bytes + (uint32_t)off * 128u) >> 4);
              const uint64_t wdesc = wdesc0 + (uint64_t)((ws * (uint32_t)kWSlot) >> 4);
#pragma unroll
              for (int k = 0; k < 4; ++k)   // A = weights (M = 128 channels), B = pixels (N = 128 per timestep)
                umma::mma_f16_ss(d, wdesc + (uint64_t)(2 * k), xdesc + (uint64_t)(2 * k), idesc,
                                 (sp > 0 || tap > 0 || k > 0) ? 1u : 0u);
              umma::mma_commit(wempty(ws));
              if (++ws == (uint32_t)g.wring) { ws = 0; wphase ^= 1u; }
            }
            if (ok) umma::mma_commit(hempty(slot));
            if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
          }
          // residual: accumulate I . R (centre tap of the residual's halo tile); with a shortcut conv the
          // weight tile of each slab of the shortcut input takes the identity's place
          const int n0 = (tile % g.n_tiles_n) * 128;
          const int n_res = g.sc_slabs ? g.sc_slabs : 2;
          for (int rs = 0; rs < n_res && g.has_res && ok; ++rs) {
            if (!g.sc_slabs && n0 + rs * 64 >= g.Cout) break;
            ok = umma::mbar_wait(hfull(slot), phase, abort_flag, wl);
            if (!ok) break;
            uint64_t adesc;
            if (g.sc_slabs) {
              ok = umma::mbar_wait(wfull(ws), wphase, abort_flag, wl);
              if (!ok) break;
              adesc = wdesc0 + (uint64_t)((ws * (uint32_t)kWSlot) >> 4);
            } else {
              adesc = umma::make_sw128_kmajor_desc(ident_base + ((rs == 0 && !dup && !TWIN) ? 64u * 128u : 0u));
            }
            umma::tc_fence_after_sync();
            const uint64_t xdesc = hdesc0 + (uint64_t)((slot * slot_bytes + (g.flat ? 0u : (uint32_t)(kPW + 1) * 128u)) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma::mma_f16_ss(d, adesc + (uint64_t)(2 * k), xdesc + (uint64_t)(2 * k), idesc, 1u);
            if (g.sc_slabs) {
              umma::mma_commit(wempty(ws));
              if (++ws == (uint32_t)g.wring) { ws = 0; wphase ^= 1u; }
            }
            umma::mma_commit(hempty(slot));
            if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
          }
          if (ok) umma::mma_commit(accfull(acc));
        }
      }
    }
    __syncwarp();
  } else if constexpr (TWIN) {
    // ------------------------------------------------- epilogue, twin mode (see PairGeom::twin)
    // Lane quarter q holds D1 (q even) or D2 (q odd) of channels 32 * (q / 2) .. + 31 and is read by four warps
    // (w, w + 4, w + 8, w + 12). The eight warps of a channel group each run the LIF for two tile rows:
    // part = 2 * (w / 4) + kind, rows 2 * part and 2 * part + 1 (part 7 holds rows 14, 15, which never exist).
    // A D1 warp needs D2 of the rows below its own, a D2 warp needs D1 of its own rows: partners (w, w ^ 1) pass
    // each other those 16 pixels per timestep through shared memory and meet at a barrier of their own. Whether
    // a wait on the accumulator gave up is agreed on by all sixteen warps together, so nobody is left behind at
    // a barrier.
    const int quarter = warp & 3, kind = quarter & 1;
    const int part = 2 * (warp >> 2) + kind, r_begin = 2 * part;
    const int ch = (quarter >> 1) * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t xchg = smem_base + (uint32_t)g.stage_off;
    const uint32_t out_row = xchg + (uint32_t)warp * kXchgWarp + (uint32_t)lane * 64u;        // what I pass on
    const uint32_t in_row = xchg + (uint32_t)(warp ^ 1) * kXchgWarp + (uint32_t)lane * 64u;   // what my partner passed
    const int bar_id = 4 + (warp >> 1);   // warps (0,1) (2,3) .. (14,15): barriers 4..11
    const uint32_t own_col = (uint32_t)((r_begin + kind) * 8);               // my half for my rows: D1[R] or D2[R + 1]
    const uint32_t send_col = (uint32_t)(((part ^ 1) * 2 + kind) * 8);       // my half for my partner's rows
    const bool has_rows = r_begin < kTileRows;   // false for part 7: it only passes its half on
    const long long frame_out = (long long)g.B * g.Ho * g.Wo * g.Cout;
    bool ok = true;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x, ++it) {
      int n0, w0, h0, b, wlo, hlo;
      decode(tile, n0, w0, h0, b, wlo, hlo);
      if (!g.own) { wlo = w0; hlo = h0; }
      const int row_first = h0 + r_begin;
      const bool c_ok = ch < g.Cout && has_rows;
      const float bias_c = (bias != nullptr && c_ok) ? DT<XT>::to_f(bias[ch]) : 0.f;
      PixMap pm;
      pm.Cout = g.Cout;
      pm.row_stride = g.Wo * g.Cout;
      pm.row0_off = ((long long)b * g.Ho + row_first) * pm.row_stride + (long long)w0 * g.Cout + ch;
      pm.rows_ok = 0;
      pm.cols_ok = 0;
#pragma unroll
      for (int r = 0; r < 2; ++r)
        if (c_ok && row_first + r < g.Ho && row_first + r >= hlo) pm.rows_ok |= 1 << r;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (w0 + j < g.Wo && w0 + j >= wlo) pm.cols_ok |= 1 << j;
      const bool full = __all_sync(0xffffffffu, pm.rows_ok == 3 && pm.cols_ok == 0xFF);
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.f;
      if (g.lif && v_init != nullptr) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (((pm.rows_ok >> (i >> 3)) & 1) && ((pm.cols_ok >> (i & 7)) & 1))
            v[i] = DT<VT>::to_f(v_init[pm.row0_off + (long long)(i >> 3) * pm.row_stride + (i & 7) * pm.Cout]);
      }
      for (int pair = 0; pair < g.npairs && ok; ++pair) {
        const uint32_t acc = (uint32_t)(pair & 1);
        const uint32_t use = it * (uint32_t)((g.npairs + 1 - (int)acc) >> 1) + (uint32_t)(pair >> 1);
        if (lane == 0) ok = umma::mbar_wait(accfull(acc), use & 1u, abort_flag, wl);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        {   // all epilogue warps agree: continue only if every one of them saw the accumulator arrive
          uint32_t all_ok;
          asm volatile(
              "{\n\t"
              ".reg .pred P, Q;\n\t"
              "setp.ne.b32 P, %1, 0;\n\t"
              "bar.red.and.pred Q, 3, %2, P;\n\t"
              "selp.b32 %0, 1, 0, Q;\n\t"
              "}\n"
              : "=r"(all_ok) : "r"((int)ok), "r"(32 * R::kEpi) : "memory");
          ok = all_ok != 0;
        }
        if (!ok) break;
        umma::tc_fence_after_sync();
        for (int q = 0; q < g.tq; ++q) {
          const uint32_t tcol = lane_base + acc * 256u + (uint32_t)(q * 128);
          {
            uint32_t a[16];
            umma::tmem_ld_x16(tcol + send_col, a);
            umma::tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(xchg_piece(out_row, lane, k)),
                           "r"(a[4 * k]), "r"(a[4 * k + 1]), "r"(a[4 * k + 2]), "r"(a[4 * k + 3]) : "memory");
          }
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");   // both partners have written timestep q
          if (has_rows) {   // warp-uniform
            ST *out = spikes + (long long)(pair * g.tq + q) * frame_out;
            const uint32_t taddr = tcol + own_col;
            if (!g.lif) {
              twin_step<XT, ST, kLifOff>(p, taddr, in_row, lane, bias_c, out, pm, v);
            } else if (p.mode == 1 && p.hard) {
              if (full && p.v_reset == 0.f && g.Cout == 64) twin_step_lean<ST>(p, taddr, in_row, lane, bias_c, out, pm, v);
              else twin_step<XT, ST, kLifFast>(p, taddr, in_row, lane, bias_c, out, pm, v);
            } else {
              twin_step<XT, ST, kLifAny>(p, taddr, in_row, lane, bias_c, out, pm, v);
            }
          }
          asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory");   // both have read: the buffers may be overwritten
        }
        // this accumulator may now be overwritten by later MMAs
        umma::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(accempty(acc));
      }
      if (ok && g.lif && v_out != nullptr) {
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (((pm.rows_ok >> (i >> 3)) & 1) && ((pm.cols_ok >> (i & 7)) & 1))
            v_out[pm.row0_off + (long long)(i >> 3) * pm.row_stride + (i & 7) * pm.Cout] = DT<VT>::from_f(v[i]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    // Pixel split: normally the two warps of a lane quarter take tile rows 0..7 / 8..15. In dup mode lanes
    // 64..127 repeat lanes 0..63, so the four warps that see the same 32 channels take 4 rows each.
    const int r_begin = dup ? ((quarter >> 1) * 2 + (warp >> 2)) * 4 : ((warp < 4) ? 0 : 8);
    const int my_rows = dup ? 4 : 8;
    constexpr int NV = DUP ? 32 : 64;   // membrane values a thread keeps
    const int ch_in_tile = dup ? (quarter & 1) * 32 + lane : quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(r_begin * 8);
    const long long frame_out = (long long)g.B * g.Ho * g.Wo * g.Cout;
    bool ok = true;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x, ++it) {
      int n0, w0, h0, b, wlo, hlo;
      decode(tile, n0, w0, h0, b, wlo, hlo);
      if (!g.own) { wlo = w0; hlo = h0; }              // duplicates write the same values: no need to mask them
      const int c = n0 + ch_in_tile;                   // output channel of this thread
      const int img = g.stack ? b + (r_begin >> 3) : b;   // two images per tile: row groups 8.. belong to image b + 1
      const int row_first = g.stack ? 0 : h0 + r_begin;   // image row of this thread's first row group
      const int row_limit = g.stack ? 8 : g.tile_rows - r_begin;   // row groups of this thread that can hold outputs
      const bool c_ok = c < g.Cout && img < g.B;
      // the two biases of a conv with a fused shortcut conv are widened first and added in fp32
      const float bias_c = ((bias != nullptr && c_ok) ? DT<XT>::to_f(bias[c]) : 0.f) +
                           ((bias2 != nullptr && c_ok) ? DT<XT>::to_f(bias2[c]) : 0.f);
      PixMap pm;
      pm.Cout = g.Cout;
      pm.row_stride = g.Wo * g.Cout;
      pm.row0_off = ((long long)img * g.Ho + row_first) * pm.row_stride + (long long)w0 * g.Cout + c;
      pm.rows_ok = 0;
      pm.cols_ok = 0;
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (c_ok && r < my_rows && r < row_limit && row_first + r < g.Ho && (g.stack || row_first + r >= hlo))
          pm.rows_ok |= 1 << r;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (w0 + j < g.Wo && w0 + j >= wlo) pm.cols_ok |= 1 << j;
      float v[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) v[i] = 0.f;
      if (g.lif && v_init != nullptr) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (((pm.rows_ok >> (i >> 3)) & 1) && ((pm.cols_ok >> (i & 7)) & 1))
            v[i] = DT<VT>::to_f(v_init[pm.row0_off + (long long)(i >> 3) * pm.row_stride + (i & 7) * pm.Cout]);
      }
      for (int pair = 0; pair < g.npairs && ok; ++pair) {
        const uint32_t acc = (uint32_t)(pair & 1);
        const uint32_t use = it * (uint32_t)((g.npairs + 1 - (int)acc) >> 1) + (uint32_t)(pair >> 1);
        if (lane == 0) ok = umma::mbar_wait(accfull(acc), use & 1u, abort_flag, wl);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        umma::tc_fence_after_sync();
        const long long toff = (long long)(pair * g.tq) * frame_out;
        const uint32_t taddr = lane_base + acc * 256u;
        ST *out = spikes + toff;
        const XT *rs = nullptr;   // the residual was already added by the tensor cores
        const int rows_valid = min(my_rows, row_limit);   // rows 14, 15 of a one-image tile never exist
        const int rows_want = (1 << rows_valid) - 1;
        const int nchunks = (rows_valid + 1) / 2;
        // warp-uniform choice: the TMEM loads inside are warp-collective
        const bool full = __all_sync(0xffffffffu, pm.rows_ok == rows_want && pm.cols_ok == 0xFF);
        const bool fast = g.lif && p.mode == 1 && p.hard && g.tq == 2 && full;
        const bool lean = fast && p.v_reset == 0.f;
        bool done = false;
        if constexpr (!DUP) {   // eight or six tile rows per thread
          if (lean && rows_valid >= 6) {
            if (rows_valid == 8) pair_epilogue_lean_any<ST, 8, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            else pair_epilogue_lean_any<ST, 6, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            done = true;
          } else if (fast && rows_valid >= 6) {
            if (rows_valid == 8) pair_epilogue_full<XT, ST, 8, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            else pair_epilogue_full<XT, ST, 6, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            done = true;
          }
        }
        if constexpr (DUP) {   // duplicated weight rows at stride 1: four or two tile rows per thread (strided convs
                               // with at most 64 outputs take the general body below)
          if (!done && lean && g.Cout == 64 && rows_valid <= 4) {
            if (rows_valid == 4) pair_epilogue_lean<ST, 4, 64, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            else pair_epilogue_lean<ST, 2, 64, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            done = true;
          } else if (!done && fast && rows_valid <= 4) {
            if (rows_valid == 4) pair_epilogue_full<XT, ST, 4, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            else pair_epilogue_full<XT, ST, 2, NV>(p, taddr, bias_c, out, frame_out, pm, v);
            done = true;
          }
        }
        if (done) {
        } else if (g.lif && p.mode == 1 && p.hard && g.tq == 2) {
          pair_epilogue<XT, ST, kLifFast, true, false, NV>(p, taddr, bias_c, rs, out, frame_out, pm, v, nchunks);
        } else if (g.lif) {
          if (g.tq == 2) pair_epilogue<XT, ST, kLifAny, true, false, NV>(p, taddr, bias_c, rs, out, frame_out, pm, v, nchunks);
          else pair_epilogue<XT, ST, kLifAny, false, false, NV>(p, taddr, bias_c, rs, out, frame_out, pm, v, nchunks);
        } else {
          if (g.tq == 2) pair_epilogue<XT, ST, kLifOff, true, false, NV>(p, taddr, bias_c, rs, out, frame_out, pm, v, nchunks);
          else pair_epilogue<XT, ST, kLifOff, false, false, NV>(p, taddr, bias_c, rs, out, frame_out, pm, v, nchunks);
        }
        // this accumulator may now be overwritten by the next tile's MMAs
        umma::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(accempty(acc));
      }
      if (ok && g.lif && v_out != nullptr) {
#pragma unroll
        for (int i = 0; i < NV; ++i)
          if (((pm.rows_ok >> (i >> 3)) & 1) && ((pm.cols_ok >> (i & 7)) & 1))
            v_out[pm.row0_off + (long long)(i >> 3) * pm.row_stride + (i & 7) * pm.Cout] = DT<VT>::from_f(v[i]);
      }
    }
  }

  umma::tc_fence_before_sync();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) atomicExch(&g_pair_status, 1);
  if (warp == R::kMma) {
    umma::tc_fence_after_sync();
    umma::tmem_dealloc(tmem_base, (uint32_t)g.tmem_cols);
  }
}

template <typename XT, typename ST, typename VT>
int launch(const ConvArgs &a, cudaStream_t stream) {
  PairGeom g;
  g.T = a.T;
  g.Tacc = (a.x_t_stride == 0) ? 1 : a.T;
  g.B = a.B; g.Cin = a.Cin; g.Cout = a.Cout; g.Ho = a.Ho; g.Wo = a.Wo;
  g.kslabs = (a.Cin + 63) / 64;
  g.ntaps = a.KH * a.KW;
  g.s2 = a.stride == 2 ? 1 : 0;
  g.tq = g.Tacc >= 2 ? 2 : 1;
  g.npairs = g.Tacc / g.tq;
  g.n_tiles_n = (a.Cout + 127) / 128;
  g.stack = (a.Ho <= 7 && a.Wo <= 8) ? 1 : 0;
  g.flat = (g.ntaps == 1 && !g.stack && a.Ho >= 16) ? 1 : 0;
  g.pw = g.flat ? 8 : kPW;
  g.row_bytes = g.pw * 128;
  g.halo_t = g.pw * kPH * 128;
  g.tile_rows = g.flat ? 16 : kTileRows;
  g.row_tiles = (a.Ho + g.tile_rows - 1) / g.tile_rows;
  g.w_strips = (a.Wo + 7) / 8;
  g.tmem_cols = g.npairs >= 2 ? 512 : (g.tq == 2 ? 256 : 128);
  g.lif = a.lif;
  g.sc_slabs = a.sc_x != nullptr ? a.sc_cin / 64 : 0;
  g.has_res = a.res != nullptr || g.sc_slabs > 0;
  const long long tiles = g.stack ? (long long)((a.B + 1) / 2) * g.n_tiles_n
                                  : (long long)a.B * g.row_tiles * g.w_strips * g.n_tiles_n;
  if (tiles > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "conv_lif: problem too large for the grid");
  g.total_tiles = (int)tiles;
  int dev = 0;
  const int sms = sm_count();
  if (cudaGetDevice(&dev) != cudaSuccess || sms < 1) return fail(SNNB_ERR_CUDA, "conv_lif: cannot query the SM count");
  const long long grid = tiles < sms ? tiles : sms;   // persistent: one CTA per SM walks the tiles
  const int es = 2;
  CUtensorMap xm, wm, xph[4];
  {
    // stride 1: one map of the frame. Stride 2: four phase views (row parity a, column parity b) with doubled
    // strides; pixel (u, v) of view (a, b) is x at (2u + a, 2v + b).
    const int s_ = g.s2 ? 2 : 1;
    const cuuint64_t frame_bytes = (cuuint64_t)a.B * a.H * a.W * a.Cin * es;
    for (int ph = 0; ph < (g.s2 ? 4 : 1); ++ph) {
      const int pa = ph >> 1, pb = ph & 1;
      cuuint64_t dims[5] = {(cuuint64_t)a.Cin, (cuuint64_t)((a.W - pb + s_ - 1) / s_), (cuuint64_t)((a.H - pa + s_ - 1) / s_),
                            (cuuint64_t)a.B, (cuuint64_t)g.Tacc};
      cuuint64_t strides[4] = {(cuuint64_t)s_ * a.Cin * es, (cuuint64_t)s_ * a.W * a.Cin * es, (cuuint64_t)a.H * a.W * a.Cin * es,
                               g.Tacc > 1 ? (cuuint64_t)a.x_t_stride * es : frame_bytes};
      cuuint32_t box[5] = {64, (cuuint32_t)g.pw, (cuuint32_t)(g.stack ? 9 : kPH), 1, 1};
      const char *base = static_cast<const char *>(a.x) + ((size_t)pa * a.W + pb) * a.Cin * es;
      const int rc = encode_tmap(&xph[ph], a.dtype, 5, base, dims, strides, box);
      if (rc != SNNB_OK) return rc;
    }
    xm = xph[0];
    if (!g.s2) xph[1] = xph[2] = xph[3] = xm;
  }
  {
    const cuuint64_t K = (cuuint64_t)g.ntaps * a.Cin;
    cuuint64_t dims[2] = {K, (cuuint64_t)a.Cout};
    cuuint64_t strides[1] = {K * es};
    cuuint32_t box[2] = {64, 128};
    const int rc = encode_tmap(&wm, a.dtype, 2, a.w, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  g.twin = (a.Cout <= 64 && g.ntaps == 9 && !g.s2 && !g.stack && g.sc_slabs == 0 && twin_enabled()) ? 1 : 0;
  g.dup = (a.Cout <= 64 && !g.twin) ? 1 : 0;
  g.stage_off = 0;
  g.own = (a.lif && a.v_init != nullptr && a.v_init == a.v_out) ? 1 : 0;
  g.wait_limit = 4000000000ll;
  g.drop_load = 0;
  consume_wait_selftest(&g.wait_limit, &g.drop_load);
  CUtensorMap wm64 = wm;
  if (g.dup || g.twin) {
    const cuuint64_t K = (cuuint64_t)g.ntaps * a.Cin;
    cuuint64_t dims[2] = {K, (cuuint64_t)a.Cout};
    cuuint64_t strides[1] = {K * es};
    cuuint32_t box[2] = {64, (cuuint32_t)(g.twin ? 32 : 64)};
    const int rc = encode_tmap(&wm64, a.dtype, 2, a.w, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  CUtensorMap rm = xm, scwm = wm;
  if (g.sc_slabs) {
    // the shortcut input seen through its stride: pixel (h, w) of the map is sc_x at (h * s, w * s)
    const cuuint64_t sC = (cuuint64_t)a.sc_cin, s_ = (cuuint64_t)a.sc_stride;
    cuuint64_t dims[5] = {sC, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.B, (cuuint64_t)a.T};
    cuuint64_t strides[4] = {s_ * sC * es, s_ * (cuuint64_t)a.sc_W * sC * es, (cuuint64_t)a.sc_H * a.sc_W * sC * es,
                             (cuuint64_t)a.sc_t_stride * es};
    cuuint32_t box[5] = {64, (cuuint32_t)g.pw, (cuuint32_t)(g.stack ? 9 : kPH), 1, 1};
    int rc = encode_tmap(&rm, a.dtype, 5, a.sc_x, dims, strides, box);
    if (rc != SNNB_OK) return rc;
    cuuint64_t wdims[2] = {sC, (cuuint64_t)a.Cout};
    cuuint64_t wstrides[1] = {sC * es};
    cuuint32_t wbox[2] = {64, 128};
    rc = encode_tmap(&scwm, a.dtype, 2, a.sc_w, wdims, wstrides, wbox);
    if (rc != SNNB_OK) return rc;
  } else if (g.has_res) {   // the residual has the output's shape: [T][B][Ho][Wo][Cout]
    cuuint64_t dims[5] = {(cuuint64_t)a.Cout, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.B, (cuuint64_t)a.T};
    cuuint64_t strides[4] = {(cuuint64_t)a.Cout * es, (cuuint64_t)a.Wo * a.Cout * es, (cuuint64_t)a.Ho * a.Wo * a.Cout * es,
                             (cuuint64_t)a.B * a.Ho * a.Wo * a.Cout * es};
    cuuint32_t box[5] = {64, (cuuint32_t)g.pw, (cuuint32_t)(g.stack ? 9 : kPH), 1, 1};
    const int rc = encode_tmap(&rm, a.dtype, 5, a.res, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  // [identity block] + weight ring + halo ring + room for the junk rows the last descriptor group reads past a slot
  g.ring = g.flat ? kPairRingMax : kPairRing;
  const bool ident = g.has_res && !g.sc_slabs;
  g.wring = ident ? kWRingP - 1 : kWRingP;
  size_t smem = (ident ? (size_t)kIdentBytes : 0) + (size_t)g.wring * kWSlot + (size_t)g.ring * g.tq * g.halo_t +
                4 * kRowBytes + 1024;
  g.wres = 0;
  if (g.twin) {   // a smaller identity block and weight ring make room for the exchange buffers
    g.wring = ident ? 3 : 4;
    // (the junk rows read past the last halo slot fall into the exchange buffers, which only the epilogue writes)
    g.stage_off = (ident ? kTwinIdentBytes : 0) + g.wring * kWSlot + g.ring * g.tq * g.halo_t;
    smem = (size_t)g.stage_off + kXchgBytes + 1024;
    static_assert(kTwinIdentBytes + 3 * kWSlot + kPairRing * 2 * kHaloT + kXchgBytes + 1024 <= 225 * 1024, "twin mode: shared memory");
    static_assert(4 * kWSlot + kPairRing * 2 * kHaloT + kXchgBytes + 1024 <= 225 * 1024, "twin mode: shared memory");
    if (!ident && g.kslabs == 1 && g.tq == 2 && wres_enabled()) {   // all six weight tiles stay resident
      g.wres = 1;
      g.wring = 6;
      g.ring = 2;
      g.stage_off = g.wring * kWSlot + g.ring * g.tq * g.halo_t;
      smem = (size_t)g.stage_off + kXchgBytes + 1024;
      static_assert(6 * kWSlot + 2 * 2 * kHaloT + kXchgBytes + 1024 <= 225 * 1024, "twin mode, resident weights: shared memory");
      static_assert(6 <= kWBarsP, "twin mode, resident weights: barriers");
    }
  }
  auto kern = g.s2 ? conv3x3_pair_kernel<XT, ST, VT, true, false, false>
              : g.twin ? conv3x3_pair_kernel<XT, ST, VT, false, true, false>
              : g.dup  ? conv3x3_pair_kernel<XT, ST, VT, false, false, true>
                       : conv3x3_pair_kernel<XT, ST, VT, false, false, false>;
  const int kidx = g.s2 ? 1 : (g.twin ? 2 : (g.dup ? 3 : 0));
  {
    // once per kernel instantiation and device: allow the largest dynamic shared-memory size any call may ask for
    static bool raised[4][64] = {};
    if (dev < 0 || dev >= 64 || !raised[kidx][dev]) {
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024);
      if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "conv_lif: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
      if (dev >= 0 && dev < 64) raised[kidx][dev] = true;
    }
  }
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(g.twin ? Roles<true>::kThreads : Roles<false>::kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, xm, wm, rm, wm64, scwm, xph[1], xph[2], xph[3],
                                              static_cast<const XT *>(a.b), static_cast<const XT *>(a.b2),
                                              static_cast<const VT *>(a.v_init), static_cast<ST *>(a.spikes),
                                              static_cast<VT *>(a.v_out), g, a.p);
    if (le != cudaSuccess) return fail(SNNB_ERR_CUDA, "conv3x3_pair: launch failed: %s", cudaGetErrorString(le));
  }
  return SNNB_OK;
}

// Reads and clears this translation unit's status word (set when a bounded wait gave up).
int pair_tu_status(int *out) {
  int h = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&h, g_pair_status, sizeof(int));
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_pair_status, &zero, sizeof(int));
  }
  *out = h;
  return SNNB_OK;
}

}  // namespace
}  // namespace snnb
