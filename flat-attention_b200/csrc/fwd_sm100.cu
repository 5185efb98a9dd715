#include "common.h"
namespace flat {
bool forward_sm100_supported(const FwdParams &) { return false; }
uint64_t forward_sm100_workspace_bytes(const FwdParams &) { return 0; }
int launch_forward_sm100(flat_ctx *ctx, const FwdParams &) { return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "not built"); }
}
