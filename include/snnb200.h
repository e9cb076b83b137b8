/*
 * snnb200 — C ABI of the B200 (sm_100a) fused temporal SNN kernels.
 *
 * Every entry point replaces one Triton launcher (and the backend function in
 * front of it) of pengjh0111/triton-snn-fusion; the reference item is cited
 * above each declaration as <file>:<lines> inside that project.
 *
 * Conventions shared by all entry points
 *   - plain device pointers, sizes and scalars; no torch types;
 *   - the caller owns every buffer; nothing is allocated and nothing is
 *     synchronised, so calls are re-entrant and may be issued on any stream
 *     (`stream` is a cudaStream_t passed as void*; NULL = the legacy default
 *     stream). The only state the library keeps between calls: the diagnostic
 *     status words read by snnb_device_status(), per-device constants it
 *     queries once (SM count, kernel attributes), and the scratch array and
 *     address cache of snnb_stem7x7_lif_static (see there);
 *   - v_init and v_out may be the very same buffer (the membrane is then
 *     updated in place, like the reference's in/out membrane buffer,
 *     kernels/benchmark_conv_lif_temporal_general.py:422-455): every kernel
 *     reads and writes each membrane value from one thread only. Two different
 *     buffers that overlap are rejected (SNNB_ERR_INVALID). No other pair of
 *     arguments may overlap;
 *   - return value: SNNB_OK or an SNNB_ERR_* code; the text of the last error
 *     on the calling thread is returned by snnb_last_error();
 *   - activations are dense channels-last ("NHWC") unless a layout argument
 *     says otherwise: a frame is [B][H][W][C] with C innermost, a sequence is
 *     T such frames `x_t_stride` elements apart;
 *   - LIF update (reference runtime/snn_custom_ops.py:384-409), all in fp32
 *     without FMA contraction:
 *         h = (tau <= 1) ? v + x : v + (x - v) / tau
 *         s = (h >= v_th)
 *         v = (v_reset >= 0) ? (s ? v_reset : h)      hard reset
 *                            : h - s * v_th           soft reset
 *     `v_init == NULL` means a zero initial membrane (the reference's 0-dim
 *     tensor convention, runtime/snn_custom_ops.py:378-381);
 *   - dtypes are snnb_dtype values. `spike_dtype` may be the activation dtype
 *     (drop-in: 0.0 / 1.0) or SNNB_U8 (0 / 1 bytes). `v_dtype` is the dtype of
 *     both v_init and v_out: the activation dtype (drop-in) or SNNB_F32.
 */
#ifndef SNNB200_H_
#define SNNB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SNNB_OK 0
#define SNNB_ERR_INVALID 1     /* bad argument (null pointer, size, alignment) */
#define SNNB_ERR_UNSUPPORTED 2 /* valid request this build has no kernel for   */
#define SNNB_ERR_CUDA 3        /* a CUDA runtime / driver call failed          */

/* SNNB_B1: spikes packed one bit each along the channel axis: the spikes of channels 32k .. 32k+31 of a pixel
 * are one little-endian 32-bit word (channel c in bit c % 32 of word c / 32), C % 32 == 0. Written by
 * snnb_stem7x7_lif (Cout == 64) and read by snnb_maxpool3x3s2_bits. */
typedef enum snnb_dtype { SNNB_F32 = 0, SNNB_BF16 = 1, SNNB_F16 = 2, SNNB_U8 = 3, SNNB_B1 = 4 } snnb_dtype;
typedef enum snnb_layout { SNNB_NCHW = 0, SNNB_NHWC = 1 } snnb_layout;

/* Which conv / linear implementation to use. AUTO picks a tcgen05 kernel when
 * the shape qualifies (16-bit activations, Cin a multiple of 64, see
 * snnb_conv_lif) and the CUDA-core path otherwise. TCGEN05 insists on a tensor-core
 * kernel (error if none applies). Among the tensor-core kernels, 3x3 / stride 1 /
 * padding 1 convs prefer the timestep-pair kernel (T = 1 or even; weights as the M
 * operand, 256 pixels as N), then the shared-memory halo kernel; TCGEN05_HALO skips
 * the first, TCGEN05_TAPS forces the general one-load-per-tap kernel (for comparison). */
typedef enum snnb_path {
  SNNB_PATH_AUTO = 0, SNNB_PATH_SIMT = 1, SNNB_PATH_TCGEN05 = 2, SNNB_PATH_TCGEN05_TAPS = 3,
  SNNB_PATH_TCGEN05_HALO = 4
} snnb_path;

/* Library version (major*10000 + minor*100 + patch). */
int snnb_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char *snnb_last_error(void);

/* Reads and clears the device-side status word that the tcgen05 kernels set
 * when one of their bounded mbarrier waits gives up. Synchronises the device.
 * 0 = no kernel reported a problem. Diagnostic only; never called on the hot
 * path. */
int snnb_device_status(int *status_out);

/*
 * Self-test of those bounded waits (no counterpart in the reference, whose Triton kernels do not wait on
 * barriers of their own). Arms the NEXT snnb_conv_lif / snnb_linear_lif / snnb_conv3x3_shortcut_lif call
 * that runs on the timestep-pair kernel: its waits give up after `limit_cycles` SM cycles (1e3 .. 4e9) instead
 * of about two seconds, and its first thread block announces one weight tile that it never loads. That block's
 * waits therefore run out: it records the fact in the status word, releases its tensor memory and returns,
 * while the other blocks finish normally. Nothing traps, faults or hangs; the armed call returns SNNB_OK, its
 * output is incomplete, and snnb_device_status() then reports a non-zero status once. The call after it runs
 * normally again.
 */
int snnb_selftest_arm_wait_timeout(long long limit_cycles);

/*
 * Diagnostic (no counterpart in the reference): SM cycles that `ctas` thread blocks, one per SM, each need for
 * 4 * reps tcgen05.mma instructions of shape M x N x 16 (bf16, fp32 accumulate, operands in shared memory, one
 * accumulator), from the first issue to the completion of the last. cycles_out[ctas] (device memory) receives one
 * figure per block, -1 where the bounded wait for completion gave up, in which case *status_out (device memory,
 * zeroed by the caller) is set to 1; nanos_out[ctas] (device memory, may be NULL) the global-timer nanoseconds of the
 * same span. random_fill != 0 fills the operand tiles with random bf16 values instead of zeros; commit_every = c > 0
 * adds a tcgen05.commit after every c-th batch of four instructions (as the conv kernels do per K slab); batch r reads
 * operand tile pair r % nslots (1 to 4 pairs of 48 KB in shared memory). M is 64 or 128, N a
 * multiple of 16 up to 256, reps at most 2^20 (the wait for completion gives up after about two seconds).
 */
int snnb_probe_mma_cycles(int M, int N, int reps, int ctas, int random_fill, int commit_every, int nslots,
                          long long *cycles_out, long long *nanos_out, int *status_out, void *stream);

/*
 * Standalone temporal LIF scan.
 * Replaces run_triton_fused_temporal_lif_state
 * (runtime/triton_temporal_lif_backend.py:57-117) and
 * _fused_temporal_lif_state_kernel / run_fused_temporal_lif_state_kernel
 * (kernels/generated_temporal_lif_kernel.py:53-154).
 *   x_seq  [T][n]  activation dtype     spikes [T][n] spike_dtype
 *   v_init [n] or NULL, v_out [n]       v_dtype
 * Any T >= 1 (the reference only takes 1,2,4,8,16). Spikes are bit-exact
 * against the fp32 reference loop.
 */
int snnb_lif_scan(const void *x_seq, const void *v_init, void *spikes, void *v_out,
                  int T, int64_t n, int x_dtype, int spike_dtype, int v_dtype,
                  float v_th, float v_reset, float tau, void *stream);

/*
 * LIF -> global average pool -> linear tail, summed over T, one kernel.
 * Replaces run_triton_fused_temporal_lif_avgpool_linear
 * (runtime/triton_temporal_lif_avgpool_linear_backend.py:58-108) and the two
 * kernels + launcher of kernels/generated_temporal_lif_avgpool_linear_kernel.py:8-209.
 *   x_seq [T][N][C][HW] (SNNB_NCHW) or [T][N][HW][C] (SNNB_NHWC), dtype
 *   fc_w [K][C], fc_b [K] or NULL, dtype
 *   out_sum [N][K] dtype   = sum_t ( W * mean_hw(spike_t) + b )
 *   v_init / v_out as x_seq[0], v_dtype
 */
int snnb_lif_avgpool_linear(const void *x_seq, const void *v_init, const void *fc_w,
                            const void *fc_b, void *out_sum, void *v_out,
                            int T, int N, int C, int HW, int K, int layout,
                            int dtype, int v_dtype,
                            float v_th, float v_reset, float tau, void *stream);

/*
 * 3x3 depthwise conv (BN folded into w, b) + optional residual + LIF over T.
 * Replaces the depthwise kernels emitted by
 * kernels/benchmark_conv_lif_temporal_general.py:713-817 and the backend
 * run_triton_fused_temporal_depthwise_conv_lif_state
 * (runtime/triton_convlif_backend.py:473-510, :513-598).
 *   x_seq [T][B][H][W][C] (frames x_t_stride elements apart; 0 = one frame
 *   reused for every step), w [C][3][3] (the torch [C,1,3,3] tensor), b [C],
 *   residual NULL or [T][B][Ho][Wo][C], spikes [T][B][Ho][Wo][C],
 *   v_init/v_out [B][Ho][Wo][C]; stride 1 or 2, padding 1.
 */
int snnb_dwconv3x3_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                       const void *residual, const void *v_init, void *spikes, void *v_out,
                       int T, int B, int C, int H, int W, int stride,
                       int dtype, int spike_dtype, int v_dtype,
                       float v_th, float v_reset, float tau, void *stream);

/*
 * Dense conv (groups = 1, BN folded into w, b) + optional residual + LIF over T.
 * Replaces the regular / pointwise / residual kernels emitted by
 * kernels/benchmark_conv_lif_temporal_general.py:561-710 (+ :685-703 residual),
 * their launchers (:971-1323) and the backends
 * run_triton_fused_temporal_conv_lif_state / _pointwise_ / _conv_add_ /
 * _packed_out (runtime/triton_convlif_backend.py:393-817).
 *   x_seq [T][B][H][W][Cin], frames x_t_stride elements apart (0 = the same
 *   frame at every step: the conv is evaluated once and only the LIF runs T
 *   times), w [Cout][KH][KW][Cin] (the torch weight in channels_last memory
 *   format), b [Cout], residual NULL or [T][B][Ho][Wo][Cout],
 *   spikes [T][B][Ho][Wo][Cout], v_init/v_out [B][Ho][Wo][Cout]. v_out may be NULL: the
 *   membrane after step T is then not written (a forward pass through a whole network needs
 *   only the spikes; the reference's op always returns it).
 * `lif` = 0 turns the LIF off: `spikes` then receives conv + bias (+ residual)
 * in the activation dtype for every t and v_init / v_out are ignored (used for
 * the BN-folded shortcut convs that feed a residual input).
 * path: the tensor-core kernels need dtype bf16/f16, Cin % 64 == 0, Cout % 16 == 0,
 * stride 1 or 2, kernel at most 11x11 and T accumulators that fit the 512 TMEM
 * columns (T <= 32); anything else runs on SNNB_PATH_SIMT.
 */
int snnb_conv_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                  const void *residual, const void *v_init, void *spikes, void *v_out,
                  int T, int B, int Cin, int H, int W, int Cout, int KH, int KW,
                  int stride, int pad, int lif,
                  int dtype, int spike_dtype, int v_dtype,
                  float v_th, float v_reset, float tau, int path, void *stream);

/*
 * Diagnostic: the name of the kernel snnb_conv_lif would run for a call of this shape ("conv3x3_pair",
 * "conv3x3_halo", "conv_lif_tc", "conv3x3_smallcin" or "conv_lif_simt"), assuming 16-byte aligned dense buffers.
 * one_frame != 0: the same input frame at every step (x_t_stride == 0). Launches nothing. The reference reports
 * its kernel choice through kernel_key / kernel_temporal_config of its result objects
 * (runtime/triton_convlif_backend.py:7-15); this is the C-level counterpart.
 */
int snnb_conv_lif_which(int T, int B, int Cin, int H, int W, int Cout, int KH, int KW, int stride, int pad,
                        int lif, int dtype, int one_frame, int has_residual, int path, char *name, int name_len);

/*
 * 3x3 / stride 1 / padding 1 conv + a 1x1 shortcut conv with stride sc_stride over a second input,
 * summed before the LIF: the second conv of a ResNet block whose shortcut is a strided 1x1 conv + BN.
 * The reference runs the shortcut conv as its own op and feeds it to the residual input of
 * run_triton_fused_temporal_conv_add_lif_state (runtime/triton_convlif_backend.py:689-817); here the
 * shortcut is accumulated on the tensor cores as extra K slabs of the same GEMM, so its output is
 * never written. No counterpart in the reference.
 *   x_seq [T][B][H][W][Cin], w [Cout][3][3][Cin], b [Cout] bias of the main conv (or NULL),
 *   sc_x [T][B][sc_H][sc_W][sc_cin] (frames sc_t_stride elements apart), sc_w [Cout][sc_cin], sc_b [Cout] bias
 *   of the shortcut conv (or NULL); the two biases are widened to fp32 before they are added;
 *   output pixel (h, w) adds sc_w . sc_x[h * sc_stride][w * sc_stride]; (sc_H - 1) / sc_stride + 1 == H.
 *   spikes [T][B][H][W][Cout], v_init / v_out [B][H][W][Cout] (either may be NULL).
 * Tensor-core only (bf16 / f16, Cin % 64 == 0, sc_cin % 64 == 0, Cout > 64, T = 1 or even); other calls
 * return SNNB_ERR_UNSUPPORTED and the caller uses the two-op sequence.
 */
int snnb_conv3x3_shortcut_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                              const void *sc_x, int64_t sc_t_stride, const void *sc_w, const void *sc_b,
                              int sc_cin, int sc_H, int sc_W, int sc_stride,
                              const void *v_init, void *spikes, void *v_out,
                              int T, int B, int Cin, int H, int W, int Cout,
                              int dtype, int spike_dtype, int v_dtype,
                              float v_th, float v_reset, float tau, void *stream);

/*
 * 7x7 / stride 2 / padding 3 stem conv with 3 input channels (+ folded BN) + LIF over T on the
 * tensor cores. Same reference items as snnb_conv_lif (kernel key k7_s2_p3,
 * kernels/benchmark_conv_lif_temporal_general.py:561-710, runtime/triton_convlif_backend.py:393-430);
 * snnb_conv_lif runs this shape on CUDA cores, this entry is the fast path for 16-bit data.
 *   x_seq [T][B][H][W][3] (x_t_stride elements apart; 0 = one frame for every step, convolved once;
 *   4-byte aligned with an even stride: it is read in 32-bit words), H and W even; w_packed [Cout][4][4][16] produced once by snnb_stem7x7_pack_weight from the
 *   [Cout][7][7][3] channels-last weight; spikes [T][B][H/2][W/2][Cout]; v_init/v_out [B][H/2][W/2][Cout]
 *   (v_out may be NULL, as for snnb_conv_lif). With Cout == 64 spike_dtype may also be SNNB_B1 (bit-packed,
 *   [T][B][H/2][W/2] 64-bit words).
 *   scratch: snnb_stem7x7_scratch_bytes(frames, H, W) bytes of device memory, 16-byte aligned, where
 *   frames = B if x_t_stride == 0 else T*B. It holds the input re-laid as 2x2-pixel blocks with a
 *   zero border; its contents are overwritten by every call.
 */
int64_t snnb_stem7x7_scratch_bytes(int frames, int H, int W);
int snnb_stem7x7_pack_weight(const void *w, void *w_packed, int Cout, int dtype, void *stream);
int snnb_stem7x7_lif(const void *x_seq, int64_t x_t_stride, const void *w_packed, const void *b,
                     const void *v_init, void *spikes, void *v_out, void *scratch, int64_t scratch_bytes,
                     int T, int B, int H, int W, int Cout, int dtype, int spike_dtype, int v_dtype,
                     float v_th, float v_reset, float tau, void *stream);

/*
 * snnb_stem7x7_lif without caller-provided scratch. No counterpart in the reference.
 *
 * For callers that cannot obtain device memory of their own at call time: a plugin slot of a
 * host runtime that owns the whole device pool and passes a plugin nothing but its input and
 * output buffers, or a serving loop that has frozen its memory plan and must not touch the
 * driver allocator (cudaMalloc may block on the whole device). This entry neither allocates nor
 * frees anything and calls no allocating library routine; the re-laid input goes into an array
 * that is part of the library image (16 MiB, snnb_stem7x7_static_scratch_bytes()) and therefore
 * occupies that much memory on every GPU the library is loaded on until the process exits.
 *
 *   - Limit: snnb_stem7x7_scratch_bytes(frames, H, W) must not exceed the array, where
 *     frames = B if x_t_stride == 0 else T*B (e.g. up to 39 frames of 224x224). Larger calls are
 *     rejected with SNNB_ERR_UNSUPPORTED and a message naming both sizes; nothing is launched.
 *   - The first call on each device looks the array's device address up (one runtime query with
 *     that device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array and it keeps whatever the previous call left. No
 *     part of it has to be cleared by the caller: each call rewrites every byte it later reads,
 *     zero border included. Two calls that may overlap in time on the GPU (different streams
 *     without an ordering between them) race on it; order them, or use snnb_stem7x7_lif.
 * Arguments and results are those of snnb_stem7x7_lif.
 */
int64_t snnb_stem7x7_static_scratch_bytes(void);
int snnb_stem7x7_lif_static(const void *x_seq, int64_t x_t_stride, const void *w_packed, const void *b,
                            const void *v_init, void *spikes, void *v_out,
                            int T, int B, int H, int W, int Cout, int dtype, int spike_dtype, int v_dtype,
                            float v_th, float v_reset, float tau, void *stream);

/*
 * Temporal linear + LIF.
 * Replaces run_triton_fused_temporal_linear_lif_state{,_packed,_packed_out}
 * (runtime/triton_temporal_linear_lif_backend.py:74-274) and
 * _fused_temporal_linear_lif_state_kernel + launcher
 * (kernels/generated_temporal_linear_lif_kernel.py:91-363).
 *   x_seq [T][M][K] (x_t_stride elements apart), w [N][K], b [N] or NULL,
 *   spikes [T][M][N], v_init/v_out [M][N].
 * The tcgen05 path needs dtype bf16/f16 and K % 64 == 0, N % 16 == 0.
 */
int snnb_linear_lif(const void *x_seq, int64_t x_t_stride, const void *w, const void *b,
                    const void *v_init, void *spikes, void *v_out,
                    int T, int M, int K, int N,
                    int dtype, int spike_dtype, int v_dtype,
                    float v_th, float v_reset, float tau, int path, void *stream);

/*
 * Stateless neighbours of the fused ops inside a spiking ResNet, so that a
 * whole network runs on this library's channels-last layout. In the reference
 * these stay ordinary aten ops applied to flatten(0,1) of the spike stack
 * (compiler/fx_spatial_batching.py:799-879).
 */
/* NCHW <-> NHWC of `frames` frames [C][HW] <-> [HW][C]. */
int snnb_nchw_to_nhwc(const void *src, void *dst, int64_t frames, int C, int HW, int dtype, void *stream);
int snnb_nhwc_to_nchw(const void *src, void *dst, int64_t frames, int C, int HW, int dtype, void *stream);
/* max_pool2d(kernel 3, stride 2, padding 1) over `frames` NHWC frames. */
int snnb_maxpool3x3s2(const void *x, void *y, int64_t frames, int H, int W, int C, int dtype, void *stream);

/*
 * The same pooling for spikes stored as one byte each (spike_dtype = SNNB_U8 of the fused entry
 * points): x [frames][H][W][C] uint8 (0 / 1) -> y [frames][Ho][Wo][C] in out_dtype. C % 16 == 0.
 * Reading one byte per spike halves the traffic of the widest activation of a ResNet (the stem
 * output). No counterpart in the reference, whose spikes always have the activation dtype.
 */
int snnb_maxpool3x3s2_u8(const void *x, void *y, int64_t frames, int H, int W, int C, int out_dtype,
                         void *stream);
/*
 * The same pooling for bit-packed spikes (SNNB_B1): x [frames][H][W][C / 32] 32-bit words -> y
 * [frames][Ho][Wo][C] in out_dtype (0.0 / 1.0). The max over a window of 0 / 1 values is the OR of the words, so a
 * pooled pixel costs nine word loads per 32 channels. With the stem writing SNNB_B1 the widest activation of a
 * ResNet crosses HBM at one bit per spike. C % 64 == 0. No counterpart in the reference.
 */
int snnb_maxpool3x3s2_bits(const void *x, void *y, int64_t frames, int H, int W, int C, int out_dtype,
                           void *stream);
/* out[n][k] = (1/T) sum_t ( fc_w . mean_hw x[t][n] + fc_b ), x NHWC [T][N][HW][C], out fp32. */
int snnb_avgpool_linear_mean(const void *x_seq, const void *fc_w, const void *fc_b, float *out,
                             int T, int N, int C, int HW, int K, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SNNB200_H_ */
