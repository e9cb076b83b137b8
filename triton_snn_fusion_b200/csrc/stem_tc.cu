// GEMM + LIF stage of the 7x7 / stride 2 stem conv (stem.cu re-lays the image first): a persistent
// tcgen05 kernel.
//
// In the re-laid image the window of output pixel (oh, ow) is 4 runs (block rows oh .. oh+3) of 64
// contiguous values, so the conv is a GEMM with K = 4 x 64 whose A rows are read through a tensor map
// with a 32-byte pixel stride. K is tiny and the layer writes T spike frames per convolved frame: the
// kernel is bound by its output stream, not by the tensor pipe. What matters is that stores never
// wait for anything else, hence:
//   * one CTA per SM walks the output tiles (128 pixels = a BW x BH box, all Cout channels);
//   * the whole packed weight (Cout x 512 bytes) is loaded once per CTA and stays in shared memory;
//   * the activation chunks of the coming tiles stream through a ring of 16 KB slots;
//   * accumulators rotate through several TMEM stages, so the MMAs of tile i+1, i+2 run while the
//     epilogue warps convert and store tile i;
//   * with 64 output channels a pixel's spikes are one 128-byte row (64 bytes for u8 spikes): each epilogue
//     warp writes the rows of its 32 pixels for one timestep into a swizzled shared-memory slot of its
//     own and a TMA store moves them out, with no synchronisation between warps. (A thread owns a
//     pixel, so direct stores put every lane of a store instruction on a different 128-byte line,
//     32 memory transactions per instruction.) Warps 0-3 and 4-7 work on alternate tiles.
// Warps 0-7: epilogue (two per TMEM lane quarter, splitting the channels); warp 8: TMA producer;
// warp 9: MMA issuer. Every mbarrier wait is bounded; on a timeout the CTA raises a status word,
// skips its remaining work, frees its tensor memory and exits.
#include <type_traits>

#include "conv.cuh"
#include "tc_epilogue.cuh"
#include "tmap.cuh"
#include "umma.cuh"

namespace snnb {

static __device__ int g_stem_status = 0;

namespace {

constexpr int kChunkBytes = 16384;   // 128 pixels x 128 bytes: one K chunk of a tile
constexpr int kMaxRing = 12;
constexpr int kMaxAcc = 4;
constexpr int kStage = 4;            // staged epilogue: 4 x 16 KB = two 4 KB slots of outgoing rows per epilogue warp
// Warp roles: epilogue warps first (groups of four, one group per tile in flight), then the producer, then the MMA
// issuer. Two groups: a third one (tried for the bit-packed form, which has the registers for it) made the layer
// 5 % slower, i.e. the epilogue warps are not what the tiles wait for.
template <typename ST> struct StemRoles {
  static constexpr int kEpi = 8;
  static constexpr int kGroups = kEpi / 4;
  static constexpr int kProd = kEpi, kMma = kEpi + 1;
  static constexpr int kThreads = 32 * (kEpi + 2);
};

struct StemGeom {
  int T, Tacc, B, Ho, Wo, Cout;
  int BW, BH, WB, HB;   // tile = BW x BH output pixels; WB x HB tiles per image
  int total_tiles;
  int ring;             // activation slots
  int nacc;             // accumulator stages in TMEM
  int stage_cols;       // TMEM columns per stage = Tacc * Cout
  int tmem_cols;
  int w_chunk_bytes;    // Cout * 128
  int staged;           // spikes leave through shared memory + TMA stores (Cout = 64, 16-bit spikes)
};

// Staged epilogue of one tile for one warp, which owns 32 pixel rows of the tile (its TMEM lane quarter)
// with all 64 channels: LIF over T with the 64 membrane potentials of a thread in registers, the
// accumulator re-read from tensor memory at every step (that is cheap; keeping 64 more values in
// registers is not). The spikes of a step go to a 4 KB slot owned by the warp (128-byte swizzle:
// 16-byte chunk j of row r sits at chunk j ^ (r & 7)), which lane 0 hands to TMA as one box. The warp
// synchronises with nobody else.
// One-byte spikes (ST = uint8_t) make 64-byte rows: 16 channels per 16-byte chunk, 64-byte swizzle
// (chunk j of row r sits at chunk j ^ ((r >> 1) & 3)), slots of 2 KB.
// spike as 0.0f / 1.0f (bit pattern 0 / 0x3F800000) -> bit `pos` of a word
__device__ __forceinline__ uint32_t spike_bit(float s, int pos) {
  const uint32_t u = __float_as_uint(s);
  return pos <= 23 ? ((u >> (23 - pos)) & (1u << pos)) : ((u << (pos - 23)) & (1u << pos));
}

// KIND 0: any LIF (run-time lif_step); 1: tau a power of two and hard reset; 2: additionally v_reset == 0, which the
// bit-packed path evaluates two channels at a time on the packed fp32 pipe (same roundings as lif_step: h = v +
// (y - v) * inv_tau in three steps, and h - s * h is exactly 0 or h for s in {0, 1}).
template <typename XT, typename ST, typename VT, int KIND>
__device__ __forceinline__ void staged_tile(const StemGeom &g, const LifParams &p, const CUtensorMap *smap,
                                            ST *__restrict__ spikes, uint32_t acc_addr, uint32_t accempty_bar, uint32_t slots, uint32_t &sslot,
                                            const float *bias_s, const VT *__restrict__ v_init, VT *__restrict__ v_out,
                                            int bx, int by, int b, long long pix, bool valid) {
  const int lane = threadIdx.x & 31;
  const bool alias = g.Tacc != g.T;
  const long long o0 = pix * 64;
  if constexpr (std::is_same<ST, uint64_t>::value && KIND == 2) {
    if (alias) {
      // Direct encoding with bit-packed spikes: the conv output is the same at every step, so each half of the
      // pixel's 64 channels is read from tensor memory ONCE (bias added once) and the T steps then run in
      // registers. The accumulator stage is released after the second half's read, before any LIF arithmetic.
      // Spikes are packed without shifts: 16 channels are collected as two fp32 sums of 4^k terms (even and odd
      // channels, exact below 2^16) by packed multiply-adds and converted to an integer once.
      uint32_t *dst32 = reinterpret_cast<uint32_t *>(spikes);
      const long long frame_px = (long long)g.B * g.Ho * g.Wo;
      const float2 it2 = make_float2(p.inv_tau, p.inv_tau), four2 = make_float2(4.f, 4.f);
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        float2 y[16], v[16];
        {
          uint32_t a[16], c[16];
          umma::tmem_ld_x16(acc_addr + (uint32_t)(hf * 32), a);
          umma::tmem_ld_x16(acc_addr + (uint32_t)(hf * 32 + 16), c);
          umma::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            y[i] = __fadd2_rn(make_float2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1])),
                              make_float2(bias_s[hf * 32 + 2 * i], bias_s[hf * 32 + 2 * i + 1]));
            y[8 + i] = __fadd2_rn(make_float2(__uint_as_float(c[2 * i]), __uint_as_float(c[2 * i + 1])),
                                  make_float2(bias_s[hf * 32 + 16 + 2 * i], bias_s[hf * 32 + 16 + 2 * i + 1]));
          }
        }
        if (hf == 1) {   // last read of this accumulator stage: the MMA warp may overwrite it
          umma::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) umma::mbar_arrive(accempty_bar);
        }
        if (v_init != nullptr && valid) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float tmp[16];
            load_pack_stream<VT, 16>(v_init + o0 + hf * 32 + q * 16, tmp);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[q * 8 + i] = make_float2(tmp[2 * i], tmp[2 * i + 1]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = make_float2(0.f, 0.f);
        }
        for (int t = 0; t < g.T; ++t) {
          uint32_t word = 0u;
#pragma unroll
          for (int grp = 0; grp < 2; ++grp) {
            float2 bits = make_float2(0.f, 0.f);   // .x: even channels of the group, .y: odd ones; channel pair k -> 4^k
#pragma unroll
            for (int k = 7; k >= 0; --k) {
              const int i = grp * 8 + k;
              const float2 d = __fadd2_rn(y[i], make_float2(-v[i].x, -v[i].y));
              const float2 h = __fadd2_rn(v[i], __fmul2_rn(d, it2));
              const float2 sp = make_float2(h.x >= p.v_th ? 1.f : 0.f, h.y >= p.v_th ? 1.f : 0.f);
              v[i] = __ffma2_rn(make_float2(-sp.x, -sp.y), h, h);
              bits = __ffma2_rn(bits, four2, sp);
            }
            word |= (uint32_t)__fmaf_rn(bits.y, 2.f, bits.x) << (grp * 16);
          }
          if (valid) dst32[((long long)t * frame_px + pix) * 2 + hf] = word;
        }
        if (valid && v_out != nullptr) {
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float tmp[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) { tmp[2 * i] = v[q * 8 + i].x; tmp[2 * i + 1] = v[q * 8 + i].y; }
            store_pack<VT, 16, false>(v_out + o0 + hf * 32 + q * 16, tmp);
          }
        }
      }
      return;
    }
  }
  float v[64];
  if (v_init != nullptr && valid) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float tmp[16];
      load_pack_stream<VT, 16>(v_init + o0 + q * 16, tmp);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[q * 16 + i] = tmp[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = 0.f;
  }
  if constexpr (std::is_same<ST, uint64_t>::value) {
    // Bit-packed spikes: a thread owns all 64 channels of its pixel, so the spikes of a step are one 64-bit word
    // (channel c in bit c) that the thread stores itself: the 32 lanes of a warp write consecutive pixels, 256
    // contiguous bytes per store instruction, and no shared-memory staging or TMA store is involved.
    ST *dst = spikes;
    const long long frame_px = (long long)g.B * g.Ho * g.Wo;
    for (int t = 0; t < g.T; ++t) {
      const uint32_t src = acc_addr + (uint32_t)((alias ? 0 : t) * 64);
      uint32_t w0 = 0u, w1 = 0u;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t a[16];
        umma::tmem_ld_x16(src + (uint32_t)(q * 16), a);
        umma::tmem_ld_wait();
        if constexpr (KIND == 2) {
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const int c = q * 16 + i;
            const float2 y = __fadd2_rn(make_float2(__uint_as_float(a[i]), __uint_as_float(a[i + 1])),
                                        make_float2(bias_s[c], bias_s[c + 1]));
            const float2 vv = make_float2(v[c], v[c + 1]);
            const float2 d = __fadd2_rn(y, make_float2(-vv.x, -vv.y));
            const float2 h = __fadd2_rn(vv, __fmul2_rn(d, make_float2(p.inv_tau, p.inv_tau)));
            const float2 sp = make_float2(h.x >= p.v_th ? 1.f : 0.f, h.y >= p.v_th ? 1.f : 0.f);
            const float2 vn = __ffma2_rn(make_float2(-sp.x, -sp.y), h, h);
            v[c] = vn.x;
            v[c + 1] = vn.y;
            if (c < 32) w0 |= spike_bit(sp.x, c & 31) | spike_bit(sp.y, (c + 1) & 31);
            else w1 |= spike_bit(sp.x, c & 31) | spike_bit(sp.y, (c + 1) & 31);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int c = q * 16 + i;
            const float y = __uint_as_float(a[i]) + bias_s[c];
            const bool sp = (KIND != 0 ? lif_step_t<1, true>(y, v[c], p) : lif_step(y, v[c], p)) != 0.f;
            if (c < 32) w0 |= (sp ? 1u : 0u) << (c & 31);
            else w1 |= (sp ? 1u : 0u) << (c & 31);
          }
        }
      }
      if (t == g.T - 1) {   // last read of this accumulator stage: the MMA warp may overwrite it
        umma::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(accempty_bar);
      }
      if (valid) dst[(long long)t * frame_px + pix] = (uint64_t)w0 | ((uint64_t)w1 << 32);
    }
    if (valid && v_out != nullptr) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float tmp[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) tmp[i] = v[q * 16 + i];
        store_pack<VT, 16, false>(v_out + o0 + q * 16, tmp);
      }
    }
    return;
  }
  for (int t = 0; t < g.T; ++t) {
    // the slot written now was handed to TMA two steps ago: that store must have read it out
    if (lane == 0) umma::bulk_wait_group_read<1>();
    __syncwarp();
    constexpr uint32_t kRow = 64u * (uint32_t)sizeof(ST);   // bytes of one pixel's 64 spikes
    const uint32_t row = slots + sslot * 4096u + (uint32_t)lane * kRow;
    const uint32_t src = acc_addr + (uint32_t)((alias ? 0 : t) * 64);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t a[16];
      umma::tmem_ld_x16(src + (uint32_t)(q * 16), a);
      umma::tmem_ld_wait();
      if constexpr (sizeof(ST) == 1) {
        Pack<uint8_t, 16> pk;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int c = q * 16 + i;
          const float y = __uint_as_float(a[i]) + bias_s[c];
          pk.v[i] = (uint8_t)((KIND != 0 ? lif_step_t<1, true>(y, v[c], p) : lif_step(y, v[c], p)) != 0.f);
        }
        const uint4 u = *reinterpret_cast<const uint4 *>(&pk);
        const uint32_t dst = row + ((uint32_t)(q ^ ((lane >> 1) & 3)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
      } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        Pack<XT, 8> pk;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = q * 16 + h * 8 + i;
          const float y = __uint_as_float(a[h * 8 + i]) + bias_s[c];
          pk.v[i] = DT<XT>::from_f(KIND != 0 ? lif_step_t<1, true>(y, v[c], p) : lif_step(y, v[c], p));
        }
        const uint4 u = *reinterpret_cast<const uint4 *>(&pk);
        const uint32_t dst = row + ((uint32_t)((q * 2 + h) ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
      }
      }
    }
    if (t == g.T - 1) {   // last read of this accumulator stage: the MMA warp may overwrite it
      umma::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(accempty_bar);
    }
    umma::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      umma::tma_store_4d(smap, slots + sslot * 4096u, 0, bx, by, t * g.B + b);
      umma::bulk_commit_group();
    }
    sslot ^= 1u;
  }
  if (valid && v_out != nullptr) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float tmp[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) tmp[i] = v[q * 16 + i];
      store_pack<VT, 16, false>(v_out + o0 + q * 16, tmp);
    }
  }
}

template <typename XT, typename ST, typename VT>
__global__ void __launch_bounds__(StemRoles<ST>::kThreads)
stem_gemm_lif_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                     const __grid_constant__ CUtensorMap smap, const XT *__restrict__ bias,
                     const VT *__restrict__ v_init, ST *__restrict__ spikes, VT *__restrict__ v_out,
                     const StemGeom g, const LifParams p) {
  using SR = StemRoles<ST>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * kMaxRing + 1 + 2 * kMaxAcc];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ float bias_s[128];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < 128) bias_s[threadIdx.x] = (bias != nullptr && (int)threadIdx.x < g.Cout) ? DT<XT>::to_f(bias[threadIdx.x]) : 0.f;
  const uint32_t smem_base = (umma::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t w_base = smem_base;                                   // 4 weight chunks, resident
  const uint32_t a_base = smem_base + 4u * (uint32_t)g.w_chunk_bytes;  // activation ring
  const uint32_t stage_base = a_base + (uint32_t)g.ring * (uint32_t)kChunkBytes;   // outgoing spike tiles (staged epilogue)
  const uint32_t bar_base = umma::smem_u32(bars);
  auto afull = [&](uint32_t s) { return bar_base + 8u * s; };
  auto aempty = [&](uint32_t s) { return bar_base + 8u * ((uint32_t)kMaxRing + s); };
  const uint32_t wfull = bar_base + 8u * (2u * kMaxRing);
  auto accfull = [&](uint32_t s) { return bar_base + 8u * (2u * kMaxRing + 1u + s); };
  auto accempty = [&](uint32_t s) { return bar_base + 8u * (2u * kMaxRing + 1u + kMaxAcc + s); };
  volatile int *abort_flag = &abort_s;

  auto decode = [&](int tile, int &w0, int &h0, int &b) {
    const int wb = tile % g.WB;
    const int m = tile / g.WB;
    w0 = wb * g.BW;
    h0 = (m % g.HB) * g.BH;
    b = m / g.HB;
  };

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < g.ring; ++s) { umma::mbar_init(afull(s), 1); umma::mbar_init(aempty(s), 1); }
    umma::mbar_init(wfull, 1);
    for (int s = 0; s < g.nacc; ++s) { umma::mbar_init(accfull(s), 1); umma::mbar_init(accempty(s), g.staged ? 4 : 8); }
    umma::fence_mbar_init();
  }
  if (warp == SR::kMma) {
    umma::tmem_alloc(umma::smem_u32(&tmem_base_s), (uint32_t)g.tmem_cols);
    umma::tmem_relinquish();
  }
  if (warp == SR::kProd && lane == 0) {
    umma::prefetch_tensormap(&xmap);
    umma::prefetch_tensormap(&wmap);
    if (g.staged) umma::prefetch_tensormap(&smap);
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  umma::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == SR::kProd) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      umma::mbar_expect_tx(wfull, 4u * (uint32_t)g.w_chunk_bytes);
      for (int i = 0; i < 4; ++i) umma::tma_load_2d(w_base + (uint32_t)(i * g.w_chunk_bytes), &wmap, wfull, i * 64, 0);
      uint32_t slot = 0, phase = 1;
      bool ok = true;
      for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x) {
        int w0, h0, b;
        decode(tile, w0, h0, b);
        for (int t = 0; t < g.Tacc && ok; ++t)
          for (int i = 0; i < 4; ++i) {   // block row h0 + i of the window = K chunk i
            ok = umma::mbar_wait(aempty(slot), phase, abort_flag);
            if (!ok) break;
            umma::mbar_expect_tx(afull(slot), (uint32_t)kChunkBytes);
            umma::tma_load_4d(a_base + slot * (uint32_t)kChunkBytes, &xmap, afull(slot), 0, w0, h0 + i, t * g.B + b);
            if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
          }
      }
    }
    __syncwarp();
  } else if (warp == SR::kMma) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma::make_idesc_f16(128, g.Cout, std::is_same<XT, __nv_bfloat16>::value);
      const uint64_t adesc0 = umma::make_sw128_kmajor_desc(a_base);
      const uint64_t wdesc0 = umma::make_sw128_kmajor_desc(w_base);
      uint32_t slot = 0, phase = 0, acc = 0, accphase = 0;
      bool ok = umma::mbar_wait(wfull, 0u, abort_flag);
      for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x) {
        // the epilogue warps must have read this stage (tile - nacc * gridDim.x) out of tensor memory
        ok = umma::mbar_wait(accempty(acc), accphase ^ 1u, abort_flag);
        if (!ok) break;
        umma::tc_fence_after_sync();
        for (int t = 0; t < g.Tacc && ok; ++t) {
          const uint32_t d = tmem_base + acc * (uint32_t)g.stage_cols + (uint32_t)(t * g.Cout);
          for (int i = 0; i < 4; ++i) {
            ok = umma::mbar_wait(afull(slot), phase, abort_flag);
            if (!ok) break;
            umma::tc_fence_after_sync();
            const uint64_t adesc = adesc0 + (uint64_t)((slot * (uint32_t)kChunkBytes) >> 4);
            const uint64_t wdesc = wdesc0 + (uint64_t)((uint32_t)(i * g.w_chunk_bytes) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma::mma_f16_ss(d, adesc + (uint64_t)(2 * k), wdesc + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
            umma::mma_commit(aempty(slot));
            if (++slot == (uint32_t)g.ring) { slot = 0; phase ^= 1u; }
          }
        }
        if (ok) umma::mma_commit(accfull(acc));
        if (++acc == (uint32_t)g.nacc) { acc = 0; accphase ^= 1u; }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;          // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    const int r = quarter * 32 + lane;     // row of the tile = output pixel owned by this thread
    const int ph = r / g.BW, pw = r - ph * g.BW;
    const int nch = g.Cout / 16, half = (nch + 1) / 2;
    const int c_begin = (warp < 4) ? 0 : half;
    const int c_end = (warp < 4) ? half : nch;
    const EpiGeom eg{g.T, g.Tacc, g.Cout, g.Cout, 0};
    const long long frame_out = (long long)g.B * g.Ho * g.Wo * g.Cout;
    bool ok = true;
    {
      if (g.staged) {
        // The groups of four warps take this CTA's tiles in turn (two groups: even / odd tiles); a warp converts
        // all 64 channels of its 32 pixels and sends them out by itself, so the epilogue has no block-wide
        // synchronisation.
        const int group = warp >> 2;
        const uint32_t slots = stage_base + (uint32_t)warp * 8192u;   // two 4 KB slots per warp
        uint32_t sslot = 0;
        // box of this warp inside the tile: 32 consecutive tile rows
        const int bx_off = (g.BW >= 32) ? (quarter * 32) % g.BW : 0;
        const int by_off = (g.BW >= 32) ? (quarter * 32) / g.BW : quarter * (32 / g.BW);
        int it = group;
        for (int tile = blockIdx.x + group * gridDim.x; tile < g.total_tiles && ok; tile += SR::kGroups * gridDim.x, it += SR::kGroups) {
          int w0, h0, b;
          decode(tile, w0, h0, b);
          const int wo = w0 + pw, ho = h0 + ph;
          const bool valid = wo < g.Wo && ho < g.Ho;
          const long long pix = ((long long)b * g.Ho + ho) * g.Wo + wo;
          const uint32_t acc = (uint32_t)(it % g.nacc), accphase = (uint32_t)((it / g.nacc) & 1);
          if (lane == 0) ok = umma::mbar_wait(accfull(acc), accphase, abort_flag);
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
          if (!ok) break;
          umma::tc_fence_after_sync();
          const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (uint32_t)g.stage_cols;
          if (p.mode == 1 && p.hard && p.v_reset == 0.f && std::is_same<ST, uint64_t>::value)
            staged_tile<XT, ST, VT, 2>(g, p, &smap, spikes, acc_addr, accempty(acc), slots, sslot, bias_s, v_init, v_out,
                                       w0 + bx_off, h0 + by_off, b, pix, valid);
          else if (p.mode == 1 && p.hard)
            staged_tile<XT, ST, VT, 1>(g, p, &smap, spikes, acc_addr, accempty(acc), slots, sslot, bias_s, v_init, v_out,
                                      w0 + bx_off, h0 + by_off, b, pix, valid);
          else
            staged_tile<XT, ST, VT, 0>(g, p, &smap, spikes, acc_addr, accempty(acc), slots, sslot, bias_s, v_init, v_out,
                                       w0 + bx_off, h0 + by_off, b, pix, valid);
        }
        // the shared-memory slots must outlive the TMA stores that read them
        if (lane == 0) umma::bulk_wait_group_read<0>();
        ok = false;   // done: skip the direct-store loop below
      }
    }
    uint32_t acc = 0, accphase = 0;
    for (int tile = blockIdx.x; tile < g.total_tiles && ok; tile += gridDim.x) {
      int w0, h0, b;
      decode(tile, w0, h0, b);
      const int wo = w0 + pw, ho = h0 + ph;
      const bool valid = wo < g.Wo && ho < g.Ho;
      const long long pix = ((long long)b * g.Ho + ho) * g.Wo + wo;
      if (lane == 0) ok = umma::mbar_wait(accfull(acc), accphase, abort_flag);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      if (!ok) break;
      umma::tc_fence_after_sync();
      const uint32_t acc_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (uint32_t)g.stage_cols;
      if constexpr (!std::is_same<ST, uint64_t>::value) {   // bit-packed spikes exist for the staged (64-channel) form only
        const EpiArgs<XT, ST, VT> ea{bias, nullptr, v_init, spikes, v_out, acc_addr,
                                     pix, frame_out, 0, c_begin, c_end, valid};
        epilogue_dispatch<XT, ST, VT>(ea, eg, 1, p);
      }
      // this stage may now be overwritten
      umma::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(accempty(acc));
      if (++acc == (uint32_t)g.nacc) { acc = 0; accphase ^= 1u; }
    }
  }

  // ------------------------------------------------------------------ teardown
  umma::tc_fence_before_sync();
  __syncthreads();
  if (abort_s && threadIdx.x == 0) atomicExch(&g_stem_status, 1);
  if (warp == SR::kMma) {
    umma::tc_fence_after_sync();
    umma::tmem_dealloc(tmem_base, (uint32_t)g.tmem_cols);
  }
}

// Tile box with BW * BH = 128 that covers the Ho x Wo map with the fewest wasted pixels (ties: the wider).
void choose_tile(int Ho, int Wo, int &BW, int &BH) {
  long long best = -1;
  BW = 128; BH = 1;
  for (int bw = 128; bw >= 1; bw /= 2) {
    const int bh = 128 / bw;
    const long long covered = (long long)((Wo + bw - 1) / bw) * bw * ((Ho + bh - 1) / bh) * bh;
    if (best < 0 || covered < best) { best = covered; BW = bw; BH = bh; }
  }
}

template <typename XT, typename ST, typename VT>
int launch(const StemGemmArgs &a, cudaStream_t stream) {
  StemGeom g;
  g.T = a.T; g.Tacc = a.frames; g.B = a.B; g.Ho = a.Ho; g.Wo = a.Wo; g.Cout = a.Cout;
  choose_tile(a.Ho, a.Wo, g.BW, g.BH);
  g.WB = (a.Wo + g.BW - 1) / g.BW;
  g.HB = (a.Ho + g.BH - 1) / g.BH;
  const long long tiles = (long long)a.B * g.WB * g.HB;
  if (tiles > 0x7fffffffLL) return fail(SNNB_ERR_INVALID, "stem7x7_lif: problem too large for the grid");
  g.total_tiles = (int)tiles;
  g.stage_cols = g.Tacc * a.Cout;
  g.nacc = 512 / g.stage_cols < kMaxAcc ? 512 / g.stage_cols : kMaxAcc;
  int cols = 32;
  while (cols < g.nacc * g.stage_cols) cols *= 2;
  g.tmem_cols = cols;
  g.w_chunk_bytes = a.Cout * 128;
  g.staged = a.Cout == 64 ? 1 : 0;   // a pixel's spikes are one 128-byte (16-bit) or 64-byte (u8) row
  // bit-packed spikes are stored by the threads themselves: no staging slots, more activation slots instead
  const bool staging = g.staged && !std::is_same<ST, uint64_t>::value;
  const int budget = 224 * 1024 - 1024 - 4 * g.w_chunk_bytes - (staging ? kStage * kChunkBytes : 0);
  g.ring = budget / kChunkBytes < kMaxRing ? budget / kChunkBytes : kMaxRing;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return fail(SNNB_ERR_CUDA, "stem7x7_lif: cannot query the SM count");
  const long long grid = tiles < sms ? tiles : sms;

  const int es = 2;
  CUtensorMap xm, wm;
  {  // windows of 64 values, one per output column, overlapping: the pixel stride is one 16-value block
    cuuint64_t dims[4] = {64, (cuuint64_t)a.Wo, (cuuint64_t)a.Hb, (cuuint64_t)a.frames * a.B};
    cuuint64_t strides[3] = {(cuuint64_t)16 * es, (cuuint64_t)a.Wb * 16 * es, (cuuint64_t)a.Hb * a.Wb * 16 * es};
    cuuint32_t box[4] = {64, (cuuint32_t)g.BW, (cuuint32_t)g.BH, 1};
    const int rc = encode_tmap(&xm, a.dtype, 4, a.s2d, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  {
    cuuint64_t dims[2] = {256, (cuuint64_t)a.Cout};
    cuuint64_t strides[1] = {(cuuint64_t)256 * es};
    cuuint32_t box[2] = {64, (cuuint32_t)a.Cout};
    const int rc = encode_tmap(&wm, a.dtype, 2, a.w_packed, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  CUtensorMap sm = xm;
  constexpr bool kBits = std::is_same<ST, uint64_t>::value;   // one 64-bit word per pixel, stored by the threads themselves
  if (kBits && !g.staged) return fail(SNNB_ERR_UNSUPPORTED, "stem7x7_lif: bit-packed spikes need Cout == 64");
  if (g.staged && !kBits) {  // spikes [T * B][Ho][Wo][64]: a tile of one step leaves as one box
    const cuuint64_t ss = sizeof(ST);
    cuuint64_t dims[4] = {64, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.T * a.B};
    cuuint64_t strides[3] = {(cuuint64_t)64 * ss, (cuuint64_t)a.Wo * 64 * ss, (cuuint64_t)a.Ho * a.Wo * 64 * ss};
    // a warp stores its 32 tile rows: part of one image row, or 32 / BW whole rows of the tile
    cuuint32_t box[4] = {64, (cuuint32_t)(g.BW >= 32 ? 32 : g.BW), (cuuint32_t)(g.BW >= 32 ? 1 : 32 / g.BW), 1};
    const int rc = sizeof(ST) == 1 ? encode_tmap(&sm, SNNB_U8, 4, a.spikes, dims, strides, box, 64)
                                   : encode_tmap(&sm, a.dtype, 4, a.spikes, dims, strides, box);
    if (rc != SNNB_OK) return rc;
  }
  const size_t smem = (size_t)4 * g.w_chunk_bytes + (size_t)g.ring * kChunkBytes + (staging ? (size_t)kStage * kChunkBytes : 0) + 1024;
  auto kern = stem_gemm_lif_kernel<XT, ST, VT>;
  const cudaError_t e = raise_smem_limit_once<stem_gemm_lif_kernel<XT, ST, VT>>(225 * 1024);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "stem7x7_lif: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
  kern<<<(unsigned)grid, StemRoles<ST>::kThreads, smem, stream>>>(xm, wm, sm, static_cast<const XT *>(a.b), static_cast<const VT *>(a.v_init),
                                                    static_cast<ST *>(a.spikes), static_cast<VT *>(a.v_out), g, a.p);
  SNNB_CHECK_LAUNCH("stem_gemm_lif");
  return SNNB_OK;
}

template <typename XT>
int dispatch(const StemGemmArgs &a, cudaStream_t stream) {
  const bool s_u8 = a.spike_dtype == SNNB_U8;
  const bool v_f32 = a.v_dtype == SNNB_F32;
  if (a.spike_dtype == SNNB_B1) return v_f32 ? launch<XT, uint64_t, float>(a, stream) : launch<XT, uint64_t, XT>(a, stream);
  if (s_u8 && v_f32) return launch<XT, uint8_t, float>(a, stream);
  if (s_u8) return launch<XT, uint8_t, XT>(a, stream);
  if (v_f32) return launch<XT, XT, float>(a, stream);
  return launch<XT, XT, XT>(a, stream);
}

}  // namespace

bool stem_gemm_supported(const StemGemmArgs &a) {
  if (a.dtype != SNNB_BF16 && a.dtype != SNNB_F16) return false;
  if (a.Cout % 32 != 0 || a.Cout > 128) return false;        // the two warps of a lane quarter split 16-channel groups evenly
  if (a.frames * a.Cout > 256) return false;                  // at least two accumulator stages
  if (!aligned16(a.s2d) || !aligned16(a.w_packed) || !aligned16(a.spikes) || !aligned16(a.v_out) ||
      (a.b && !aligned16(a.b)) || (a.v_init && !aligned16(a.v_init)))
    return false;
  return true;
}

int stem_gemm_lif(const StemGemmArgs &a, cudaStream_t stream) {
  return a.dtype == SNNB_BF16 ? dispatch<__nv_bfloat16>(a, stream) : dispatch<__half>(a, stream);
}

int stem_device_status(int *out) {
  int h = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&h, g_stem_status, sizeof(int));
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  if (h != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_stem_status, &zero, sizeof(int));
  }
  *out = h;
  return SNNB_OK;
}

}  // namespace snnb
