// Shared device/host helpers: dtype traits, 128-bit vector access, the LIF
// update, error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/snnb200.h"

namespace snnb {

// ---------------------------------------------------------------- errors ----
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define SNNB_CHECK_ARG(cond, ...)                               \
  do {                                                          \
    if (!(cond)) return ::snnb::fail(SNNB_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define SNNB_CHECK_LAUNCH(name)                                                         \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess)                                                             \
      return ::snnb::fail(SNNB_ERR_CUDA, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
  } while (0)

// Whether kernels that support it are launched with programmatic dependent launch (on unless the environment
// variable SNNB_PDL is set to 0).
bool pdl_enabled();
// tail.cu: average pool + linear + mean over T on the tensor cores (bf16, channels-last); see its definition
int head_pool_linear_bf16(const void *x, const void *w, const void *b, float *out, int T, int N, int C, int HW, int K,
                          cudaStream_t stream, bool *taken);
// Whether 3x3 / stride 1 convs with at most 64 output channels use the two-kernel-rows-per-MMA form of the
// timestep-pair kernel (default; SNNB_TWIN=0 in the environment selects the form that duplicates the weight rows).
bool twin_enabled();
// experiment switch: SNNB_WRES=0 keeps the weight ring in the twin form
bool wres_enabled();

// Number of SMs of the current device (queried once per device; 0 if the query fails).
int sm_count();

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int dtype_size(int dt) { return dt == SNNB_F32 ? 4 : (dt == SNNB_U8 ? 1 : 2); }
inline bool is_act_dtype(int dt) { return dt == SNNB_F32 || dt == SNNB_BF16 || dt == SNNB_F16; }

// Raises the dynamic shared-memory limit of kernel `Kern` to `bytes` once per device (the kernel is a template
// argument, so every kernel has its own flags).
template <auto Kern>
inline cudaError_t raise_smem_limit_once(int bytes) {
  static bool done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
  return e;
}

// ---------------------------------------------------------------- dtypes ----
template <typename T> struct DT;
template <> struct DT<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct DT<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct DT<__half> {
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct DT<uint8_t> {
  static __device__ __forceinline__ float to_f(uint8_t v) { return (float)v; }
  static __device__ __forceinline__ uint8_t from_f(float v) { return (uint8_t)(v != 0.f); }
};

// N consecutive elements of type T moved with the widest access that N*sizeof(T)
// allows (16 / 8 / 4 / 2 / 1 bytes). `p` must be aligned to that width.
template <typename T, int N> struct alignas(sizeof(T) * N >= 16 ? 16 : sizeof(T) * N) Pack {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ void load_pack_stream(const T *p, float (&out)[N]) {
  // streaming (evict-first) load: the data is read exactly once
  constexpr int BYTES = sizeof(T) * N;
  Pack<T, N> pk;
  if constexpr (BYTES % 16 == 0) {
    int4 *dst = reinterpret_cast<int4 *>(&pk);
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) dst[i] = __ldcs(reinterpret_cast<const int4 *>(p) + i);
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<int2 *>(&pk) = __ldcs(reinterpret_cast<const int2 *>(p));
  } else if constexpr (BYTES == 4) {
    *reinterpret_cast<int *>(&pk) = __ldcs(reinterpret_cast<const int *>(p));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) pk.v[i] = __ldcs(p + i);
  }
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = DT<T>::to_f(pk.v[i]);
}

template <typename T, int N>
__device__ __forceinline__ void load_pack(const T *p, float (&out)[N]) {
  constexpr int BYTES = sizeof(T) * N;
  Pack<T, N> pk;
  if constexpr (BYTES % 16 == 0) {
    int4 *dst = reinterpret_cast<int4 *>(&pk);
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) dst[i] = __ldg(reinterpret_cast<const int4 *>(p) + i);
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<int2 *>(&pk) = __ldg(reinterpret_cast<const int2 *>(p));
  } else if constexpr (BYTES == 4) {
    *reinterpret_cast<int *>(&pk) = __ldg(reinterpret_cast<const int *>(p));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) pk.v[i] = p[i];
  }
#pragma unroll
  for (int i = 0; i < N; ++i) out[i] = DT<T>::to_f(pk.v[i]);
}

template <typename T, int N, bool STREAM = true>
__device__ __forceinline__ void store_pack(T *p, const float (&in)[N]) {
  constexpr int BYTES = sizeof(T) * N;
  Pack<T, N> pk;
#pragma unroll
  for (int i = 0; i < N; ++i) pk.v[i] = DT<T>::from_f(in[i]);
  if constexpr (BYTES % 16 == 0) {
    const int4 *src = reinterpret_cast<const int4 *>(&pk);
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      if constexpr (STREAM) __stcs(reinterpret_cast<int4 *>(p) + i, src[i]);
      else reinterpret_cast<int4 *>(p)[i] = src[i];
    }
  } else if constexpr (BYTES == 8) {
    if constexpr (STREAM) __stcs(reinterpret_cast<int2 *>(p), *reinterpret_cast<const int2 *>(&pk));
    else *reinterpret_cast<int2 *>(p) = *reinterpret_cast<const int2 *>(&pk);
  } else if constexpr (BYTES == 4) {
    if constexpr (STREAM) __stcs(reinterpret_cast<int *>(p), *reinterpret_cast<const int *>(&pk));
    else *reinterpret_cast<int *>(p) = *reinterpret_cast<const int *>(&pk);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) p[i] = pk.v[i];
  }
}

// ------------------------------------------------------------------- LIF ----
// Runtime LIF constants, prepared once on the host.
struct LifParams {
  float v_th;
  float v_reset;   // used when hard != 0
  float tau;
  float inv_tau;   // exact reciprocal when tau is a power of two
  int mode;        // 0: h = v + x (tau <= 1); 1: h = v + (x - v) * inv_tau (tau a power of two,
                   // bit-identical to the division); 2: h = v + (x - v) / tau (IEEE division)
  int hard;        // 1: hard reset to v_reset; 0: soft reset (v_reset < 0 in the reference's API)
};

LifParams make_lif_params(float v_th, float v_reset, float tau);

// One LIF step in fp32 with the reference's operation order
// (runtime/snn_custom_ops.py:393-408). Explicit round-to-nearest intrinsics keep
// the compiler from contracting the multiply-add into an FMA, which would change
// the last bit of h and therefore flip spikes that sit exactly on the threshold.
__device__ __forceinline__ float lif_step(float x, float &v, const LifParams &p) {
  float h;
  if (p.mode == 0) {
    h = __fadd_rn(v, x);
  } else if (p.mode == 1) {
    h = __fadd_rn(v, __fmul_rn(__fsub_rn(x, v), p.inv_tau));
  } else {
    h = __fadd_rn(v, __fdiv_rn(__fsub_rn(x, v), p.tau));
  }
  const bool s = h >= p.v_th;
  if (p.hard) v = s ? p.v_reset : h;
  else v = s ? __fsub_rn(h, p.v_th) : h;
  return s ? 1.0f : 0.0f;
}

// The same update with the charge mode and the reset kind fixed at compile time, for loops
// that cannot afford the per-element branches (bit-identical to lif_step).
template <int MODE, bool HARD>
__device__ __forceinline__ float lif_step_t(float x, float &v, const LifParams &p) {
  float h;
  if constexpr (MODE == 0) h = __fadd_rn(v, x);
  else if constexpr (MODE == 1) h = __fadd_rn(v, __fmul_rn(__fsub_rn(x, v), p.inv_tau));
  else h = __fadd_rn(v, __fdiv_rn(__fsub_rn(x, v), p.tau));
  const bool s = h >= p.v_th;
  if constexpr (HARD) v = s ? p.v_reset : h;
  else v = s ? __fsub_rn(h, p.v_th) : h;
  return s ? 1.0f : 0.0f;
}

}  // namespace snnb
