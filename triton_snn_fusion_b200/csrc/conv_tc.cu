// placeholder until the tcgen05 kernel lands
#include "conv.cuh"
namespace snnb {
bool conv_lif_tc_supported(const ConvArgs &, const char **why) { *why = "not built"; return false; }
int conv_lif_tc(const ConvArgs &, cudaStream_t) { return fail(SNNB_ERR_UNSUPPORTED, "tcgen05 path not built"); }
}
extern "C" int snnb_device_status(int *out) { if (out) *out = 0; return SNNB_OK; }
