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
