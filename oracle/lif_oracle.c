/*
 * CPU oracle for the temporal LIF scan in plain C — TEST INFRASTRUCTURE ONLY.
 *
 * Restates, element by element and in fp32 with no FMA contraction (build with
 * -ffp-contract=off), the loop of pengjh0111/triton-snn-fusion's
 * fused_temporal_lif_state_torch (runtime/snn_custom_ops.py:521-536) around
 * lif_forward_state_torch (runtime/snn_custom_ops.py:384-409). It is pinned
 * against the reference's own functions through the golden vectors under
 * tests/golden/. Only the tests, the smoke check and the benchmark's CPU
 * baseline may call it; the shipped library never does.
 */
#include <stdint.h>
#include <stddef.h>

/* x_seq [T][n], v_init [n] or NULL (zero state), spikes [T][n] (0.0f / 1.0f), v_out [n]. */
void lif_scan_f32(const float *x_seq, const float *v_init, float *spikes, float *v_out,
                  int T, int64_t n, float v_th, float v_reset, float tau) {
  const int plain_sum = tau <= 1.0f;
  const int soft = v_reset < 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    float v = v_init ? v_init[i] : 0.0f;
    for (int t = 0; t < T; ++t) {
      const float x = x_seq[(int64_t)t * n + i];
      float h;
      if (plain_sum) {
        h = v + x;
      } else {
        const float d = x - v;
        const float q = d / tau;
        h = v + q;
      }
      const float s = (h >= v_th) ? 1.0f : 0.0f;
      if (soft) {
        const float drop = s * v_th;
        v = h - drop;
      } else {
        v = (s != 0.0f) ? v_reset : h;
      }
      spikes[(int64_t)t * n + i] = s;
    }
    v_out[i] = v;
  }
}

/* Number of positions where two spike arrays differ (checker helper). */
int64_t count_mismatch_f32(const float *a, const float *b, int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) bad += (a[i] != b[i]);
  return bad;
}
