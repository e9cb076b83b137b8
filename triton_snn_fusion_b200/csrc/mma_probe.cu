// Diagnostic: how long one tcgen05.mma (kind::f16, fp32 accumulate, K = 16, both operands from shared memory)
// takes for a given M x N, alone on the GPU or on every SM at once. The conv kernels' tile layout (weights as
// M = 128, two timesteps x 128 pixels as N = 256) rests on these figures.
//
// One CTA per SM (or a single CTA): 512 tensor-memory columns, a zero-filled 128 x 64 A tile and an N x 64 B tile
// in shared memory (K-major, 128-byte swizzle; zeros, so the layout of the values does not matter). One thread
// issues `reps` batches of four MMAs (one 64-wide K slab, like a tap of the conv kernels) into the same
// accumulator, commits them to an mbarrier and waits for it with the usual bounded wait; the elapsed SM cycles
// divided by 4 * reps are written out per CTA, together with the nanoseconds of the global timer over the same
// span: cycles / nanoseconds is the SM clock the block really ran at, which drops under the board's power cap when
// the operands are not zeros (`random_fill`). With thousands of MMAs behind one commit the figure is the
// issue-to-completion throughput of the tensor pipe for that shape, not the latency of a single instruction.
#include "common.cuh"
#include "umma.cuh"

namespace snnb {
namespace {

__global__ void __launch_bounds__(128)
mma_probe_kernel(int M, int N, int reps, int random_fill, int commit_every, int nslots, long long *cycles, long long *nanos, int *status) {
  extern __shared__ uint8_t probe_smem[];
  __shared__ __align__(8) uint64_t bar, side_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  const uint32_t base = (umma::smem_u32(probe_smem) + 1023u) & ~1023u;
  // `nslots` operand tile pairs of 48 KB (A 16 KB, B 32 KB); batch r reads pair r % nslots
  const uint32_t a_base = base, b_base = base + 128u * 128u;
  constexpr uint32_t kPairBytes = 128u * 128u + 256u * 128u;
  uint4 *z = reinterpret_cast<uint4 *>(probe_smem + (base - umma::smem_u32(probe_smem)));
  for (int i = threadIdx.x; i < nslots * (int)(kPairBytes / 16); i += blockDim.x) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (random_fill) {   // bf16 values in (-2, 2) with random mantissas: operands that toggle the datapath
      uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u + 12345u;
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        h ^= h << 13; h ^= h >> 17; h ^= h << 5;
        w[j] = (h & 0x807F807Fu) | 0x3F003F00u | ((h >> 7) & 0x00800080u);
      }
      v = make_uint4(w[0], w[1], w[2], w[3]);
    }
    z[i] = v;
  }
  if (threadIdx.x == 0) {
    abort_s = 0;
    umma::mbar_init(umma::smem_u32(&bar), 1);
    umma::mbar_init(umma::smem_u32(&side_bar), (1u << 20) - 1u);   // never completes: a target for the extra commits
    umma::fence_mbar_init();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the zeros are read by the MMA unit
  if (threadIdx.x < 32) {
    umma::tmem_alloc(umma::smem_u32(&tmem_base_s), 512u);
    umma::tmem_relinquish();
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  umma::tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  if (threadIdx.x == 0) {
    const uint32_t idesc = umma::make_idesc_f16(M, N, true);
    const uint64_t adesc = umma::make_sw128_kmajor_desc(a_base), bdesc = umma::make_sw128_kmajor_desc(b_base);
    long long n0, n1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n0));
    const long long t0 = clock64();
    int sl = 0;
    for (int r = 0; r < reps; ++r) {
      const uint64_t so = (uint64_t)((uint32_t)sl * kPairBytes >> 4);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        umma::mma_f16_ss(tmem_base, adesc + so + (uint64_t)(2 * k), bdesc + so + (uint64_t)(2 * k), idesc, (r > 0 || k > 0) ? 1u : 0u);
      if (++sl == nslots) sl = 0;
      // the conv kernels commit after every K slab (to release its weight slot); what does that cost?
      if (commit_every > 0 && (r + 1) % commit_every == 0) umma::mma_commit(umma::smem_u32(&side_bar));
    }
    umma::mma_commit(umma::smem_u32(&bar));
    const bool ok = umma::mbar_wait(umma::smem_u32(&bar), 0u, &abort_s);
    const long long t1 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n1));
    cycles[blockIdx.x] = ok ? (t1 - t0) : -1;
    if (nanos != nullptr) nanos[blockIdx.x] = n1 - n0;
    if (!ok) atomicExch(status, 1);
  }
  umma::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) {
    umma::tc_fence_after_sync();
    umma::tmem_dealloc(tmem_base, 512u);
  }
}

}  // namespace
}  // namespace snnb

extern "C" int snnb_probe_mma_cycles(int M, int N, int reps, int ctas, int random_fill, int commit_every, int nslots,
                                     long long *cycles_out, long long *nanos_out, int *status_out, void *stream) {
  using namespace snnb;
  SNNB_CHECK_ARG(cycles_out != nullptr && status_out != nullptr, "probe_mma_cycles: null pointer");
  SNNB_CHECK_ARG(M == 64 || M == 128, "probe_mma_cycles: M must be 64 or 128");
  SNNB_CHECK_ARG(N >= 16 && N <= 256 && N % 16 == 0, "probe_mma_cycles: N must be a multiple of 16 in [16, 256]");
  SNNB_CHECK_ARG(reps >= 1 && reps <= (1 << 20) && ctas >= 1 && ctas <= 1024, "probe_mma_cycles: reps in [1, 2^20], ctas in [1, 1024]");
  SNNB_CHECK_ARG(nslots >= 1 && nslots <= 4, "probe_mma_cycles: nslots in [1, 4]");
  const size_t smem = (size_t)nslots * (128 * 128 + 256 * 128) + 1024;
  const cudaError_t e = raise_smem_limit_once<mma_probe_kernel>(200 * 1024);
  if (e != cudaSuccess) return fail(SNNB_ERR_CUDA, "probe_mma_cycles: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
  mma_probe_kernel<<<(unsigned)ctas, 128, smem, static_cast<cudaStream_t>(stream)>>>(M, N, reps, random_fill, commit_every, nslots, cycles_out, nanos_out, status_out);
  SNNB_CHECK_LAUNCH("mma_probe");
  return SNNB_OK;
}
