// Temporary: entry points not implemented yet.
#include "common.cuh"
#define STUB(name, ...) extern "C" int name(__VA_ARGS__) { return snnb::fail(SNNB_ERR_UNSUPPORTED, #name ": not implemented"); }
STUB(snnb_device_status, int *)
STUB(snnb_lif_avgpool_linear, const void *, const void *, const void *, const void *, void *, void *, int, int, int, int, int, int, int, int, float, float, float, void *)
STUB(snnb_dwconv3x3_lif, const void *, int64_t, const void *, const void *, const void *, const void *, void *, void *, int, int, int, int, int, int, int, int, int, float, float, float, void *)
STUB(snnb_conv_lif, const void *, int64_t, const void *, const void *, const void *, const void *, void *, void *, int, int, int, int, int, int, int, int, int, int, int, int, int, int, float, float, float, int, void *)
STUB(snnb_linear_lif, const void *, int64_t, const void *, const void *, const void *, void *, void *, int, int, int, int, int, int, int, float, float, float, int, void *)
STUB(snnb_nchw_to_nhwc, const void *, void *, int64_t, int, int, int, void *)
STUB(snnb_nhwc_to_nchw, const void *, void *, int64_t, int, int, int, void *)
STUB(snnb_maxpool3x3s2, const void *, void *, int64_t, int, int, int, int, void *)
STUB(snnb_avgpool_linear_mean, const void *, const void *, const void *, float *, int, int, int, int, int, int, void *)
