// Epilogue shared by the tcgen05 conv kernels: TMEM accumulators -> bias (+ residual) -> LIF over T
// with the membrane in registers -> spikes / membrane in global memory.
#pragma once

#include "common.cuh"
#include "umma.cuh"

namespace snnb {

// What the epilogue needs to know about the tile.
struct EpiGeom {
  int T;        // timesteps to emit
  int Tacc;     // accumulators in TMEM (1 when every step sees the same frame, else T)
  int BN;       // columns per accumulator
  int Cout;
  int has_res;
};

template <typename XT, typename ST, typename VT>
struct EpiArgs {
  const XT *bias;
  const XT *res;
  const VT *v_init;
  ST *spikes;
  VT *v_out;
  uint32_t lane_base;   // TMEM address of this thread's lane, column 0 of accumulator 0
  long long pix;        // flat output pixel index of this thread
  long long frame_out;  // elements per output frame
  int n0, c_begin, c_end;
  bool valid;
};

// Epilogue of one thread: for each of its 16-channel groups, walk the T accumulators in order with
// the membrane in registers. The TMEM load of step t+1 is in flight while step t is evaluated.
template <typename XT, typename ST, typename VT, int MODE, bool HARD, bool LIFON>
__device__ __forceinline__ void epilogue_cols(const EpiArgs<XT, ST, VT> &e, const EpiGeom &g, const LifParams &p) {
  const bool alias = (g.Tacc != g.T);
  for (int c = e.c_begin; c < e.c_end; ++c) {
    const int n = e.n0 + c * 16;
    if (n >= g.Cout) break;
    uint32_t nxt[16];
    umma::tmem_ld_x16(e.lane_base + (uint32_t)(c * 16), nxt);
    float bj[16];
    if (e.bias != nullptr) {
      load_pack<XT, 16>(e.bias + n, bj);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) bj[i] = 0.f;
    }
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
    const long long o0 = e.pix * g.Cout + n;
    if (LIFON && e.v_init != nullptr && e.valid) load_pack_stream<VT, 16>(e.v_init + o0, v);
    for (int t = 0; t < g.T; ++t) {
      float y[16];
      umma::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) y[i] = __uint_as_float(nxt[i]) + bj[i];
      if (t + 1 < g.T && !alias) umma::tmem_ld_x16(e.lane_base + (uint32_t)((t + 1) * g.BN + c * 16), nxt);
      if (e.valid) {
        const long long o = (long long)t * e.frame_out + o0;
        if (g.has_res) {
          float rr[16];
          load_pack<XT, 16>(e.res + o, rr);
#pragma unroll
          for (int i = 0; i < 16; ++i) y[i] += rr[i];
        }
        if constexpr (LIFON) {
          float s[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) s[i] = lif_step_t<MODE, HARD>(y[i], v[i], p);
          store_pack<ST, 16, false>(e.spikes + o, s);
        } else {
          store_pack<XT, 16, false>(reinterpret_cast<XT *>(e.spikes) + o, y);
        }
      }
    }
    if (LIFON && e.valid && e.v_out != nullptr) store_pack<VT, 16, false>(e.v_out + o0, v);
  }
  umma::tmem_ld_wait();
}

// Selects the compile-time LIF kind once per tile (charge mode x reset kind, or no LIF at all).
template <typename XT, typename ST, typename VT>
__device__ __forceinline__ void epilogue_dispatch(const EpiArgs<XT, ST, VT> &ea, const EpiGeom &eg, int lif,
                                                  const LifParams &p) {
  if (!lif) {
    epilogue_cols<XT, ST, VT, 0, true, false>(ea, eg, p);
    return;
  }
  switch (p.mode * 2 + p.hard) {
    case 0: epilogue_cols<XT, ST, VT, 0, false, true>(ea, eg, p); break;
    case 1: epilogue_cols<XT, ST, VT, 0, true, true>(ea, eg, p); break;
    case 2: epilogue_cols<XT, ST, VT, 1, false, true>(ea, eg, p); break;
    case 3: epilogue_cols<XT, ST, VT, 1, true, true>(ea, eg, p); break;
    case 4: epilogue_cols<XT, ST, VT, 2, false, true>(ea, eg, p); break;
    default: epilogue_cols<XT, ST, VT, 2, true, true>(ea, eg, p); break;
  }
}

}  // namespace snnb
