// Error reporting and host-side LIF parameter preparation.
#include "common.cuh"

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace snnb {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

const char *last_error() { return g_err; }

bool pdl_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("SNNB_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

bool twin_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("SNNB_TWIN");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

bool wres_enabled() {
  static const bool on = [] {
    const char *e = std::getenv("SNNB_WRES");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

int sm_count() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) return 0;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

LifParams make_lif_params(float v_th, float v_reset, float tau) {
  LifParams p;
  p.v_th = v_th;
  p.tau = tau;
  p.inv_tau = 1.0f;
  p.hard = v_reset >= 0.0f ? 1 : 0;
  p.v_reset = v_reset;
  if (tau <= 1.0f) {
    p.mode = 0;
  } else {
    int e = 0;
    const float m = std::frexp(tau, &e);
    if (m == 0.5f) {  // tau is a power of two: x * (1/tau) == x / tau bit for bit (no subnormal inputs lost
      p.mode = 1;     // that the division would keep: both round the same exact quotient)
      p.inv_tau = 1.0f / tau;
    } else {
      p.mode = 2;
    }
  }
  return p;
}

}  // namespace snnb

extern "C" {
int snnb_version(void) { return 100; }
const char *snnb_last_error(void) { return snnb::last_error(); }
}
