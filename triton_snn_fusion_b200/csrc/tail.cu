// LIF -> global average pool -> linear, summed over T, in ONE kernel.
//
// A thread-block cluster of 8 CTAs serves a group of S samples. Phase 1 (HBM-bound):
// each CTA scans its slice of the channels of every sample of the group over the T
// steps with the membrane in registers, writes the last membrane, and counts spikes
// per channel in shared memory. The counts are integers, so the shared-memory atomics
// that collect them are order-independent and the result is deterministic (the
// reference accumulates floats with global atomics). Phase 2: the CTAs exchange their
// count slices through distributed shared memory, then each CTA computes its slice of
// the classes for all S samples, one warp per class with a shuffle reduction:
//   out[n][k] = (sum_c w[k][c] * count[n][c]) / HW + T * b[k]
// which equals sum_t (W . mean_hw(spike_t) + b).
#include <cooperative_groups.h>


#include <type_traits>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace snnb {
namespace {

constexpr int CL = 8;     // CTAs per cluster
constexpr int NT = 256;
constexpr int SMAX = 8;   // samples per cluster (upper bound)

template <typename XT, typename VT, bool NHWC, int VEC>
__global__ void __launch_bounds__(NT)
lif_avgpool_linear_kernel(const XT *__restrict__ x, const VT *__restrict__ v_init,
                          const XT *__restrict__ fc_w, const XT *__restrict__ fc_b,
                          XT *__restrict__ out, VT *__restrict__ v_out,
                          int T, int N, int C, int HW, int K, int S, LifParams p) {
  extern __shared__ int cnt[];  // [S][C] spike counts summed over t and pixels
  cg::cluster_group cluster = cg::this_cluster();
  const int r = (int)cluster.block_rank();
  const int g = blockIdx.x / CL;
  const int n0 = g * S;
  const int ns = min(S, N - n0);
  const int tid = threadIdx.x;

  for (int i = tid; i < S * C; i += NT) cnt[i] = 0;
  __syncthreads();

  const int Cs = (C + CL - 1) / CL;
  int cs = r * Cs, ce = min(C, cs + Cs);
  if (VEC > 1) {  // keep slices vector-aligned
    const int Cv = ((C / VEC + CL - 1) / CL) * VEC;
    cs = min(C, r * Cv);
    ce = min(C, cs + Cv);
  }
  const int64_t frame = (int64_t)N * C * HW;

  for (int s = 0; s < ns; ++s) {
    const int n = n0 + s;
    if constexpr (NHWC) {
      // Two items (pixel x VEC channels) per trip with the loads of up to four timesteps of both issued
      // before the first use: the phase is a pure stream, so bytes in flight per thread set its speed.
      const int cvn = (ce - cs) / VEC;
      const int items = HW * cvn;
      for (int it0 = tid; it0 < items; it0 += 2 * NT) {
        int64_t e[2];
        int cc[2];
        bool on[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int it = it0 + u * NT;
          on[u] = it < items;
          const int itc = on[u] ? it : it0;
          const int pix = itc / cvn;
          cc[u] = cs + (itc % cvn) * VEC;
          e[u] = ((int64_t)n * HW + pix) * C + cc[u];
        }
        float v[2][VEC];
        int k[2][VEC];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (v_init != nullptr) load_pack_stream<VT, VEC>(v_init + e[u], v[u]);
          else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[u][i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < VEC; ++i) k[u][i] = 0;
        }
        for (int t0 = 0; t0 < T; t0 += 4) {
          float xv[2][4][VEC];
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (t0 + j < T) load_pack_stream<XT, VEC>(x + (int64_t)(t0 + j) * frame + e[u], xv[u][j]);
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (t0 + j < T) {
#pragma unroll
                for (int i = 0; i < VEC; ++i) k[u][i] += (int)lif_step(xv[u][j][i], v[u][i], p);
              }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
          if (on[u]) {
            store_pack<VT, VEC>(v_out + e[u], v[u]);
#pragma unroll
            for (int i = 0; i < VEC; ++i)
              if (k[u][i]) atomicAdd(&cnt[s * C + cc[u] + i], k[u][i]);
          }
      }
    } else {
      const int items = (ce - cs) * HW;
      const int64_t e0 = ((int64_t)n * C + cs) * HW;
      for (int it = tid; it < items; it += NT) {
        const int c = cs + it / HW;
        const int64_t e = e0 + it;
        float v = v_init != nullptr ? DT<VT>::to_f(v_init[e]) : 0.f;
        int k = 0;
        for (int t = 0; t < T; ++t) k += (int)lif_step(DT<XT>::to_f(x[(int64_t)t * frame + e]), v, p);
        v_out[e] = DT<VT>::from_f(v);
        if (k) atomicAdd(&cnt[s * C + c], k);
      }
    }
  }

  // ---- exchange the count slices through distributed shared memory
  cluster.sync();
  for (int q = 0; q < CL; ++q) {
    if (q == r) continue;
    int qs = q * Cs, qe = min(C, qs + Cs);
    if (VEC > 1) {
      const int Cv = ((C / VEC + CL - 1) / CL) * VEC;
      qs = min(C, q * Cv);
      qe = min(C, qs + Cv);
    }
    const int *peer = cluster.map_shared_rank(cnt, q);
    const int len = qe - qs;
    for (int i = tid; i < ns * len; i += NT) {
      const int s = i / len, c = qs + i % len;
      cnt[s * C + c] = peer[s * C + c];
    }
  }
  cluster.sync();  // nobody leaves (or overwrites) before every peer has read its slice

  // ---- linear: this CTA's classes for all samples of the group
  const int Ks = (K + CL - 1) / CL;
  const int ks = r * Ks, ke = min(K, ks + Ks);
  const int warp = tid / 32, lane = tid % 32;
  const float inv_hw = 1.0f / (float)HW;
  for (int k = ks + warp; k < ke; k += NT / 32) {
    float acc[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s) acc[s] = 0.f;
    const XT *wk = fc_w + (int64_t)k * C;
    if (VEC > 1 && C % 8 == 0 && (reinterpret_cast<uintptr_t>(fc_w) & 15u) == 0 && sizeof(XT) == 2) {
      for (int c = lane * 8; c < C; c += 32 * 8) {   // 16 bytes of weights per lane and trip
        float wv[8];
        load_pack<XT, 8>(wk + c, wv);
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < ns) {
            const int4 c0 = *reinterpret_cast<const int4 *>(&cnt[s * C + c]);
            const int4 c1 = *reinterpret_cast<const int4 *>(&cnt[s * C + c + 4]);
            float a = acc[s];
            a = fmaf(wv[0], (float)c0.x, a); a = fmaf(wv[1], (float)c0.y, a);
            a = fmaf(wv[2], (float)c0.z, a); a = fmaf(wv[3], (float)c0.w, a);
            a = fmaf(wv[4], (float)c1.x, a); a = fmaf(wv[5], (float)c1.y, a);
            a = fmaf(wv[6], (float)c1.z, a); a = fmaf(wv[7], (float)c1.w, a);
            acc[s] = a;
          }
      }
    } else {
      for (int c = lane; c < C; c += 32) {
        const float wv = DT<XT>::to_f(wk[c]);
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < ns) acc[s] = fmaf(wv, (float)cnt[s * C + c], acc[s]);
      }
    }
    const float bk = fc_b != nullptr ? DT<XT>::to_f(fc_b[k]) * (float)T : 0.f;
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      float a = acc[s];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (lane == 0 && s < ns) out[(int64_t)(n0 + s) * K + k] = DT<XT>::from_f(a * inv_hw + bk);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Streaming form for channels-last input whose channel count splits evenly over the cluster.
// Same plan (scan + integer counts, DSMEM exchange, warp-per-class mat-vec), laid out for bandwidth:
//   * scan: the (sample, pixel, channel-vector) items of the CTA's channel slice form ONE index space over all
//     samples of the group; a thread takes two items per trip and issues their 16-byte loads for up to four
//     timesteps (and the initial membranes) before the first use, i.e. up to 160 bytes in flight per thread,
//     with two blocks resident per SM;
//   * exchange: the peers' count slices are copied with 16-byte DSMEM loads;
//   * mat-vec: a warp works on four classes at a time, so every count read from shared memory feeds four
//     dot products, and its four 16-byte weight loads per trip are independent.
constexpr int NTF = 256;

// a 16-byte vector of XT as loaded (kept packed until it is used, which keeps 16 loads in flight cheap in registers)
template <typename XT, int VEC>
__device__ __forceinline__ void unpack16(const int4 &raw, float (&out)[VEC]) {
  static_assert(sizeof(XT) * VEC == 16, "one 16-byte vector");
  const XT *e = reinterpret_cast<const XT *>(&raw);
#pragma unroll
  for (int i = 0; i < VEC; ++i) out[i] = DT<XT>::to_f(e[i]);
}

template <typename XT, typename VT, int VEC>
__global__ void __launch_bounds__(NTF, 2)
lif_avgpool_linear_stream_kernel(const XT *__restrict__ x, const VT *v_init, const XT *__restrict__ fc_w,
                                 const XT *__restrict__ fc_b, XT *__restrict__ out, VT *v_out,
                                 int T, int N, int C, int HW, int K, int S, LifParams p) {
  extern __shared__ __align__(16) int cnt[];  // [S][C] spike counts summed over t and pixels
  cg::cluster_group cluster = cg::this_cluster();
  const int r = (int)cluster.block_rank();
  const int n0 = (blockIdx.x / CL) * S;
  const int ns = min(S, N - n0);
  const int tid = threadIdx.x;
  for (int i = tid; i < S * C; i += NTF) cnt[i] = 0;
  __syncthreads();

  const int Cs = C / CL;            // channels of this CTA, a multiple of VEC
  const int cvn = Cs / VEC;         // vectors per pixel; NTF % cvn == 0, so a thread keeps its channel vector
  const int cs = r * Cs;
  const int64_t frame = (int64_t)N * C * HW;
  const int items = ns * HW * cvn;
  const int cc = cs + (tid % cvn) * VEC;
  constexpr int IT = 2;   // items per thread and trip
  for (int it0 = tid; it0 < items; it0 += IT * NTF) {
    int64_t e[IT];
    int smp[IT];
    bool on[IT];
#pragma unroll
    for (int u = 0; u < IT; ++u) {
      const int it = it0 + u * NTF;
      on[u] = it < items;
      const int ps = (on[u] ? it : it0) / cvn;   // (sample, pixel) index
      smp[u] = ps / HW;
      e[u] = ((int64_t)(n0 + smp[u]) * HW + (ps - smp[u] * HW)) * C + cc;
    }
    float v[IT][VEC];
    int k[IT][VEC];
#pragma unroll
    for (int u = 0; u < IT; ++u) {
      if (v_init != nullptr) load_pack_stream<VT, VEC>(v_init + e[u], v[u]);
      else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[u][i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) k[u][i] = 0;
    }
    for (int t0 = 0; t0 < T; t0 += 4) {
      int4 raw[IT][4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int u = 0; u < IT; ++u)
          if (t0 + j < T) raw[u][j] = __ldcs(reinterpret_cast<const int4 *>(x + (int64_t)(t0 + j) * frame + e[u]));
#pragma unroll
      for (int u = 0; u < IT; ++u)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (t0 + j < T) {
            float xv[VEC];
            unpack16<XT, VEC>(raw[u][j], xv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) k[u][i] += (int)lif_step(xv[i], v[u][i], p);
          }
    }
#pragma unroll
    for (int u = 0; u < IT; ++u)
      if (on[u]) {
        store_pack<VT, VEC>(v_out + e[u], v[u]);
#pragma unroll
        for (int i = 0; i < VEC; ++i)
          if (k[u][i]) atomicAdd(&cnt[smp[u] * C + cc + i], k[u][i]);
      }
  }

  // ---- exchange the count slices through distributed shared memory, 16 bytes at a time
  cluster.sync();
  {
    const int q4 = Cs / 4;   // int4 per (peer, sample)
    for (int i = tid; i < (CL - 1) * ns * q4; i += NTF) {
      int q = i / (ns * q4);
      const int rem = i - q * (ns * q4);
      q += (q >= r) ? 1 : 0;                       // skip this CTA's own slice
      const int s = rem / q4, j = rem - s * q4;
      const int off = s * C + q * Cs + j * 4;
      const int *peer = cluster.map_shared_rank(cnt, q);
      *reinterpret_cast<int4 *>(&cnt[off]) = *reinterpret_cast<const int4 *>(&peer[off]);
    }
  }
  cluster.sync();  // nobody leaves (or overwrites) before every peer has read its slice

  // ---- linear: this CTA's classes for all samples of the group, four classes per warp and trip
  const int Ks = (K + CL - 1) / CL;
  const int ks = r * Ks, ke = min(K, ks + Ks);
  const int warp = tid / 32, lane = tid % 32;
  const float inv_hw = 1.0f / (float)HW;
  for (int k0 = ks + 4 * warp; k0 < ke; k0 += 4 * (NTF / 32)) {
    float acc[4][SMAX];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int s = 0; s < SMAX; ++s) acc[q][s] = 0.f;
    for (int c = lane * 8; c < C; c += 32 * 8) {
      float wv[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (k0 + q < ke) load_pack<XT, 8>(fc_w + (int64_t)(k0 + q) * C + c, wv[q]);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) wv[q][i] = 0.f;
        }
      }
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        if (s < ns) {
          const int4 c0 = *reinterpret_cast<const int4 *>(&cnt[s * C + c]);
          const int4 c1 = *reinterpret_cast<const int4 *>(&cnt[s * C + c + 4]);
          const float cf[8] = {(float)c0.x, (float)c0.y, (float)c0.z, (float)c0.w,
                               (float)c1.x, (float)c1.y, (float)c1.z, (float)c1.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float a = acc[q][s];
#pragma unroll
            for (int i = 0; i < 8; ++i) a = fmaf(wv[q][i], cf[i], a);
            acc[q][s] = a;
          }
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float bk = (fc_b != nullptr && k0 + q < ke) ? DT<XT>::to_f(fc_b[k0 + q]) * (float)T : 0.f;
#pragma unroll
      for (int s = 0; s < SMAX; ++s) {
        float a = acc[q][s];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0 && s < ns && k0 + q < ke) out[(int64_t)(n0 + s) * K + k0 + q] = DT<XT>::from_f(a * inv_hw + bk);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Second streaming form, 16-bit activations: register sums and a warp-level tensor-core mat-vec.
//   * scan: a thread keeps ONE (sample, pixel group, channel vector) and walks that sample's pixels (pixel pg,
//     pg + PG, ...), two pixels per trip with the 16-byte loads of up to four timesteps of both issued before
//     the first use; its spike counts stay in registers (packed fp32 adds) until it is done and then go to a
//     shared-memory row of its own, so there are no atomics and no index arithmetic per item. The rows of a
//     sample's pixel groups are added in a fixed order: the result is deterministic. tau a power of two with
//     hard reset to zero runs the packed-fp32 LIF (same operation order and rounding as lif_step). MODE 2 skips
//     the LIF and sums the inputs themselves (the network head: average pool + linear over spikes that exist
//     already).
//   * exchange: every CTA gathers the eight slices of sums through DSMEM and stores them as 16-bit floats.
//     Spike counts are at most T * HW: exact in bf16 up to 256 and in fp16 up to 2048. SPLIT stores a second
//     16-bit float with the rounding error of the first: exact for counts up to 2^16, and for sums of arbitrary
//     values a relative error of 2^-16 instead of 2^-8.
//   * linear: out[s][k] = sum_c sum[s][c] * w[k][c] as mma.sync m16n8k16 with the samples as the M rows
//     (rows 8..15 are zero) and eight classes as N. A thread's 16-byte load of w[k][c .. c + 7] and its
//     16-byte shared-memory read of sum[s][c .. c + 7] are the operands of two MMAs (the channel order
//     inside a K block is permuted the same way on both sides, which a dot product does not see).
template <typename XT> struct Mma16;
template <> struct Mma16<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};
template <> struct Mma16<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};

enum : int { kScanLif = 0, kScanLifFast = 1, kScanSum = 2 };

// Two LIF steps side by side; kScanLifFast: h = v + (y - v) * inv_tau as three separately rounded packed
// operations (what lif_step does one lane at a time), reset to zero as h - s * h.
template <int MODE>
__device__ __forceinline__ float2 scan_two(float2 y, float2 &v, const LifParams &p) {
  if constexpr (MODE == kScanSum) {
    return y;
  } else if constexpr (MODE == kScanLifFast) {
    const float2 d = __fadd2_rn(y, make_float2(-v.x, -v.y));
    const float2 h = __fadd2_rn(v, __fmul2_rn(d, make_float2(p.inv_tau, p.inv_tau)));
    const float2 s = make_float2(h.x >= p.v_th ? 1.f : 0.f, h.y >= p.v_th ? 1.f : 0.f);
    v = __ffma2_rn(make_float2(-s.x, -s.y), h, h);
    return s;
  } else {
    float2 s;
    s.x = lif_step(y.x, v.x, p);
    s.y = lif_step(y.y, v.y, p);
    return s;
  }
}

// out[n][k] = out_scale * sum_c w[k][c] * (sum over t and pixels of spikes or inputs)[n][c] + bias_mul * b[k]
template <typename XT, typename OT, int MODE, bool SPLIT>
__global__ void __launch_bounds__(NTF, 2)
pool_linear_mma_kernel(const XT *__restrict__ x, const XT *v_init, const XT *__restrict__ fc_w,
                       const XT *__restrict__ fc_b, OT *__restrict__ out, XT *v_out,
                       int T, int N, int C, int HW, int K, int S, float out_scale, float bias_mul, LifParams p) {
  constexpr int VEC = 8, NP = SPLIT ? 2 : 1;
  extern __shared__ __align__(16) float tail_smem_f[];
  cg::cluster_group cluster = cg::this_cluster();
  const int r = (int)cluster.block_rank();
  const int n0 = (blockIdx.x / CL) * S;
  const int ns = min(S, N - n0);
  const int tid = threadIdx.x;
  const int Cs = C / CL;            // channels of this CTA, a multiple of VEC
  const int cvn = Cs / VEC;         // vectors per pixel; NTF % cvn == 0
  const int slots = NTF / cvn;      // (sample, pixel group) pairs that run side by side
  const int PG = max(1, slots / ns);   // pixel groups per sample
  const int AP = C + 8;             // row pitch of the gathered sums in elements: rows 16 bytes apart in the banks
  float *part = tail_smem_f;                                   // [max(slots, S)][Cs] one row per (sample, pixel group)
  float *sums = part + max(slots, S) * Cs;                     // [S][Cs] this CTA's slice
  XT *amat = reinterpret_cast<XT *>(sums + S * Cs);            // [NP][S][AP] all slices as 16-bit floats

  // ---- scan
  {
    const int cv = tid % cvn;
    const int cc = r * Cs + cv * VEC;
    const int64_t frame = (int64_t)N * C * HW;
    for (int sp = tid / cvn; sp < ns * PG; sp += slots) {
      const int smp = sp / PG, pg = sp - smp * PG;
      const int64_t e0 = (int64_t)(n0 + smp) * HW * C + cc;
      float2 k2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) k2[i] = make_float2(0.f, 0.f);
      for (int p0 = pg; p0 < HW; p0 += 2 * PG) {
        const bool two = p0 + PG < HW;
        const int64_t e[2] = {e0 + (int64_t)p0 * C, e0 + (int64_t)(two ? p0 + PG : p0) * C};
        float2 v[2][4];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (MODE != kScanSum && v_init != nullptr) {
            float vv[VEC];
            load_pack_stream<XT, VEC>(v_init + e[u], vv);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[u][i] = make_float2(vv[2 * i], vv[2 * i + 1]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[u][i] = make_float2(0.f, 0.f);
          }
        }
        for (int t0 = 0; t0 < T; t0 += 4) {
          int4 raw[2][4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int u = 0; u < 2; ++u)
              if (t0 + j < T) raw[u][j] = __ldcs(reinterpret_cast<const int4 *>(x + (int64_t)(t0 + j) * frame + e[u]));
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (t0 + j < T && (u == 0 || two)) {
                float xv[VEC];
                unpack16<XT, VEC>(raw[u][j], xv);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  k2[i] = __fadd2_rn(k2[i], scan_two<MODE>(make_float2(xv[2 * i], xv[2 * i + 1]), v[u][i], p));
              }
        }
        if constexpr (MODE != kScanSum) {
#pragma unroll
          for (int u = 0; u < 2; ++u)
            if (u == 0 || two) {
              const float vv[VEC] = {v[u][0].x, v[u][0].y, v[u][1].x, v[u][1].y, v[u][2].x, v[u][2].y, v[u][3].x, v[u][3].y};
              store_pack<XT, VEC>(v_out + e[u], vv);
            }
        }
      }
      float4 *row = reinterpret_cast<float4 *>(part + sp * Cs + cv * VEC);
      row[0] = make_float4(k2[0].x, k2[0].y, k2[1].x, k2[1].y);
      row[1] = make_float4(k2[2].x, k2[2].y, k2[3].x, k2[3].y);
    }
  }
  __syncthreads();
  for (int i = tid; i < ns * Cs; i += NTF) {   // a sample's pixel groups, added in a fixed order
    const int smp = i / Cs, j = i - smp * Cs;
    float a = part[(smp * PG) * Cs + j];
    for (int pg = 1; pg < PG; ++pg) a += part[(smp * PG + pg) * Cs + j];
    sums[i] = a;
  }

  // ---- gather all slices through distributed shared memory, as 16-bit floats
  cluster.sync();
  {
    const int q4 = Cs / 4;  // float4 per (peer, sample)
    const float *peers[CL];
#pragma unroll
    for (int q = 0; q < CL; ++q) peers[q] = cluster.map_shared_rank(sums, q);
    for (int i = tid; i < ns * q4; i += NTF) {   // the eight remote loads of an item are in flight together
      const int smp = i / q4, j = i - smp * q4;
      float4 c4[CL];
#pragma unroll
      for (int q = 0; q < CL; ++q) c4[q] = *reinterpret_cast<const float4 *>(&peers[q][smp * Cs + j * 4]);
#pragma unroll
      for (int q = 0; q < CL; ++q) {
        const float cf[4] = {c4[q].x, c4[q].y, c4[q].z, c4[q].w};
        XT *dst = amat + smp * AP + q * Cs + j * 4;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const XT hi = DT<XT>::from_f(cf[u]);
          dst[u] = hi;
          if (SPLIT) dst[S * AP + u] = DT<XT>::from_f(cf[u] - DT<XT>::to_f(hi));
        }
      }
    }
    for (int part_i = 0; part_i < NP; ++part_i)   // unused sample rows
      for (int i = tid; i < (S - ns) * AP; i += NTF) amat[(part_i * S + ns) * AP + i] = DT<XT>::from_f(0.f);
  }
  cluster.sync();  // nobody leaves before every peer has read its slice; amat is complete

  // ---- linear on the tensor cores: a warp takes eight classes at a time
  {
    const int Ks = (K + CL - 1) / CL;
    const int ks = r * Ks, ke = min(K, ks + Ks);
    const int warp = tid / 32, lane = tid % 32;
    const int g = lane >> 2, t4 = lane & 3;
    const XT *arow = amat + (g < S ? g : 0) * AP;   // sample g (rows past S never reach the output)
    // two class tiles per trip: eight independent 16-byte weight loads in flight per thread
    for (int k0 = ks + 16 * warp; k0 < ke; k0 += 16 * (NTF / 32)) {
      const XT *wrow[2];
#pragma unroll
      for (int h = 0; h < 2; ++h)   // classes past the end repeat the last one and are not stored
        wrow[h] = fc_w + (int64_t)min(k0 + 8 * h + g, ke - 1) * C;
      float d[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int c0 = 0; c0 < C; c0 += 128) {
        int4 wv[2][4], av[4], al[4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + u * 32 < C) wv[h][u] = __ldg(reinterpret_cast<const int4 *>(wrow[h] + c0 + u * 32 + t4 * 8));
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * 32 < C) {
            av[u] = *reinterpret_cast<const int4 *>(arow + c0 + u * 32 + t4 * 8);
            if (SPLIT) al[u] = *reinterpret_cast<const int4 *>(arow + S * AP + c0 + u * 32 + t4 * 8);
          }
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (c0 + u * 32 < C) {
              if (SPLIT) {   // the small parts first
                Mma16<XT>::run(d[h], (uint32_t)al[u].x, (uint32_t)al[u].y, (uint32_t)wv[h][u].x, (uint32_t)wv[h][u].y);
                Mma16<XT>::run(d[h], (uint32_t)al[u].z, (uint32_t)al[u].w, (uint32_t)wv[h][u].z, (uint32_t)wv[h][u].w);
              }
              Mma16<XT>::run(d[h], (uint32_t)av[u].x, (uint32_t)av[u].y, (uint32_t)wv[h][u].x, (uint32_t)wv[h][u].y);
              Mma16<XT>::run(d[h], (uint32_t)av[u].z, (uint32_t)av[u].w, (uint32_t)wv[h][u].z, (uint32_t)wv[h][u].w);
            }
      }
      // d[h][0], d[h][1]: sample g, classes k0 + 8 * h + 2 * t4, + 1
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int k = k0 + 8 * h + 2 * t4 + j;
          if (g < ns && k < ke) {
            const float bk = fc_b != nullptr ? DT<XT>::to_f(fc_b[k]) * bias_mul : 0.f;
            out[(int64_t)(n0 + g) * K + k] = DT<OT>::from_f(d[h][j] * out_scale + bk);
          }
        }
    }
  }
}

// Whether the tensor-core form takes the shape (the stricter count limit for spike counts is the caller's).
inline bool pool_linear_mma_ok(const void *x, const void *w, int C) {
  const int Cs = C / CL;
  return aligned16(x) && aligned16(w) && C % (CL * 8) == 0 && C % 32 == 0 && NTF % (Cs / 8) == 0 && Cs / 8 <= NTF &&
         C <= 4096;
}

template <typename XT, typename OT, bool SPLIT>
int launch_mma(const void *x, const void *v_init, const void *w, const void *b, void *out, void *v_out,
               int T, int N, int C, int HW, int K, int mode, float out_scale, float bias_mul, const LifParams &p,
               cudaStream_t stream) {
  const int sms = sm_count() > 0 ? sm_count() : 128;
  // samples per cluster: the largest power of two (the scan's thread layout divides evenly, and every cluster
  // re-reads the weight matrix from L2, so few large groups beat many small ones) that still leaves about
  // 1.5 blocks per SM. Measured at 1024 -> 1000, 7x7, T = 4: batch 256 takes 0.042 ms with 8 samples per cluster,
  // 0.056 with 4, 0.061 with 7; batch 64 takes 0.020 ms with 2, 0.024 with 4, 0.029 with 1.
  int S = SMAX;
  while (S > 1 && (long long)N * CL / S < (3LL * sms) / 2) S >>= 1;
  const int Cs = C / CL, slots = NTF / (Cs / 8);
  const size_t smem = (size_t)((slots > S ? slots : S) + S) * Cs * sizeof(float) + (size_t)(SPLIT ? 2 : 1) * S * (C + 8) * sizeof(XT);
  const int groups = (N + S - 1) / S;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(groups * CL));
  cfg.blockDim = dim3(NTF);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto kern = mode == kScanSum ? pool_linear_mma_kernel<XT, OT, kScanSum, SPLIT>
                               : (mode == kScanLifFast ? pool_linear_mma_kernel<XT, OT, kScanLifFast, SPLIT>
                                                       : pool_linear_mma_kernel<XT, OT, kScanLif, SPLIT>);
  if (smem > 48 * 1024) {
    const cudaError_t ea = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ea != cudaSuccess) return fail(SNNB_ERR_CUDA, "pool_linear: cannot raise the shared-memory limit: %s", cudaGetErrorString(ea));
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<const XT *>(x), static_cast<const XT *>(v_init),
                                     static_cast<const XT *>(w), static_cast<const XT *>(b),
                                     static_cast<OT *>(out), static_cast<XT *>(v_out), T, N, C, HW, K, S, out_scale,
                                     bias_mul, p);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "pool_linear: launch failed: %s", cudaGetErrorString(e));
  return SNNB_OK;
}

template <typename XT, typename VT, bool NHWC, int VEC>
int launch(const void *x, const void *v_init, const void *w, const void *b, void *out, void *v_out,
           int T, int N, int C, int HW, int K, const LifParams &p, cudaStream_t stream) {
  const int sms = sm_count() > 0 ? sm_count() : 128;
  int S = (N * CL) / (2 * sms);   // samples per cluster: about two CTAs per SM in flight
  S = S < 1 ? 1 : (S > SMAX ? SMAX : S);
  while (S > 1 && (size_t)S * C * sizeof(int) > 48 * 1024) --S;
  const size_t smem = (size_t)S * C * sizeof(int);
  if (smem > 48 * 1024) return fail(SNNB_ERR_UNSUPPORTED, "lif_avgpool_linear: C=%d too large", C);
  const int groups = (N + S - 1) / S;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(groups * CL));
  cfg.blockDim = dim3(NT);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, lif_avgpool_linear_kernel<XT, VT, NHWC, VEC>,
                                     static_cast<const XT *>(x), static_cast<const VT *>(v_init),
                                     static_cast<const XT *>(w), static_cast<const XT *>(b),
                                     static_cast<XT *>(out), static_cast<VT *>(v_out), T, N, C, HW, K, S, p);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "lif_avgpool_linear: launch failed: %s", cudaGetErrorString(e));
  return SNNB_OK;
}

template <typename XT, typename VT, int VEC>
int launch_stream(const void *x, const void *v_init, const void *w, const void *b, void *out, void *v_out,
                  int T, int N, int C, int HW, int K, const LifParams &p, cudaStream_t stream) {
  const int sms = sm_count() > 0 ? sm_count() : 128;
  // samples per cluster: as many as keep about two CTAs per SM in flight (each cluster re-reads the weight
  // matrix from L2, so few large groups beat many small ones), within 48 KB of counts
  int S = (N * CL + 2 * sms - 1) / (2 * sms);
  S = S < 1 ? 1 : (S > SMAX ? SMAX : S);
  while (S > 1 && (size_t)S * C * sizeof(int) > 48 * 1024) --S;
  const size_t smem = (size_t)S * C * sizeof(int);
  const int groups = (N + S - 1) / S;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(groups * CL));
  cfg.blockDim = dim3(NTF);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, lif_avgpool_linear_stream_kernel<XT, VT, VEC>,
                                     static_cast<const XT *>(x), static_cast<const VT *>(v_init),
                                     static_cast<const XT *>(w), static_cast<const XT *>(b),
                                     static_cast<XT *>(out), static_cast<VT *>(v_out), T, N, C, HW, K, S, p);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "lif_avgpool_linear: launch failed: %s", cudaGetErrorString(e));
  return SNNB_OK;
}

template <typename XT, typename VT>
int pick(const void *x, const void *v_init, const void *w, const void *b, void *out, void *v_out,
         int T, int N, int C, int HW, int K, int layout, const LifParams &p, cudaStream_t stream) {
  if (layout == SNNB_NHWC) {
    const bool al = aligned16(x) && aligned16(v_out) && (v_init == nullptr || aligned16(v_init));
    {   // streaming form: the channels split evenly over the cluster into 16-byte vectors
      constexpr int V = 16 / (int)sizeof(XT);
      const int Cs = C / CL;
      if constexpr (sizeof(XT) == 2 && std::is_same<XT, VT>::value) {
        // 16-bit activations and membrane, counts exact as 16-bit floats: tensor-core mat-vec form
        const int max_count = std::is_same<XT, __nv_bfloat16>::value ? 256 : 2048;
        if (al && pool_linear_mma_ok(x, w, C) && (long long)T * HW <= 65536) {
          const int mode = (p.mode == 1 && p.hard && p.v_reset == 0.f) ? kScanLifFast : kScanLif;
          if ((long long)T * HW <= max_count)
            return launch_mma<XT, XT, false>(x, v_init, w, b, out, v_out, T, N, C, HW, K, mode, 1.0f / (float)HW, (float)T, p, stream);
          // larger counts: two 16-bit parts (an integer below 2^16 is the sum of two bf16 / fp16 values exactly)
          return launch_mma<XT, XT, true>(x, v_init, w, b, out, v_out, T, N, C, HW, K, mode, 1.0f / (float)HW, (float)T, p, stream);
        }
      }
      if (al && aligned16(w) && C % (CL * V) == 0 && C % 8 == 0 && NTF % (Cs / V) == 0 &&
          (size_t)C * sizeof(int) <= 48 * 1024 && (sizeof(VT) == sizeof(XT)))
        return launch_stream<XT, VT, V>(x, v_init, w, b, out, v_out, T, N, C, HW, K, p, stream);
    }
    if (al && sizeof(XT) == 2 && C % 8 == 0) return launch<XT, VT, true, 8>(x, v_init, w, b, out, v_out, T, N, C, HW, K, p, stream);
    const bool vec = (C % 4 == 0) && al;
    if (vec) return launch<XT, VT, true, 4>(x, v_init, w, b, out, v_out, T, N, C, HW, K, p, stream);
    return launch<XT, VT, true, 1>(x, v_init, w, b, out, v_out, T, N, C, HW, K, p, stream);
  }
  return launch<XT, VT, false, 1>(x, v_init, w, b, out, v_out, T, N, C, HW, K, p, stream);
}

}  // namespace

// Average pool + linear + mean over T of a channels-last bf16 sequence through the tensor-core form above (the
// sums of arbitrary inputs are kept as two bf16 parts). Returns SNNB_OK with *taken = false when the shape is not
// one it serves.
int head_pool_linear_bf16(const void *x, const void *w, const void *b, float *out, int T, int N, int C, int HW, int K,
                          cudaStream_t stream, bool *taken) {
  *taken = pool_linear_mma_ok(x, w, C);
  if (!*taken) return SNNB_OK;
  LifParams p = make_lif_params(1.f, 0.f, 2.f);   // unused by the summing scan
  return launch_mma<__nv_bfloat16, float, true>(x, nullptr, w, b, out, nullptr, T, N, C, HW, K, kScanSum,
                                               1.0f / ((float)T * (float)HW), 1.0f, p, stream);
}

}  // namespace snnb

extern "C" int snnb_lif_avgpool_linear(const void *x_seq, const void *v_init, const void *fc_w,
                                       const void *fc_b, void *out_sum, void *v_out,
                                       int T, int N, int C, int HW, int K, int layout,
                                       int dtype, int v_dtype,
                                       float v_th, float v_reset, float tau, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(x_seq && fc_w && out_sum && v_out, "lif_avgpool_linear: null pointer");
  SNNB_CHECK_ARG(T >= 1 && N >= 1 && C >= 1 && HW >= 1 && K >= 1, "lif_avgpool_linear: sizes must be positive");
  SNNB_CHECK_ARG(layout == SNNB_NCHW || layout == SNNB_NHWC, "lif_avgpool_linear: bad layout %d", layout);
  SNNB_CHECK_ARG(is_act_dtype(dtype), "lif_avgpool_linear: unsupported dtype %d", dtype);
  SNNB_CHECK_ARG(v_dtype == dtype || v_dtype == SNNB_F32, "lif_avgpool_linear: v dtype must be the x dtype or f32");
  SNNB_CHECK_ARG(tau != 0.0f, "lif_avgpool_linear: unsupported_tau: tau must be nonzero");
  const LifParams p = make_lif_params(v_th, v_reset, tau);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool v_f32 = v_dtype == SNNB_F32;
#define SNNB_ARGS x_seq, v_init, fc_w, fc_b, out_sum, v_out, T, N, C, HW, K, layout, p, s
  switch (dtype) {
    case SNNB_F32: return pick<float, float>(SNNB_ARGS);
    case SNNB_BF16: return v_f32 ? pick<__nv_bfloat16, float>(SNNB_ARGS) : pick<__nv_bfloat16, __nv_bfloat16>(SNNB_ARGS);
    default: return v_f32 ? pick<__half, float>(SNNB_ARGS) : pick<__half, __half>(SNNB_ARGS);
  }
#undef SNNB_ARGS
}
