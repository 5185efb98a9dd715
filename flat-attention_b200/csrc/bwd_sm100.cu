#include "common.h"
namespace flat {
bool backward_sm100_supported(const BwdParams &) { return false; }
uint64_t backward_sm100_workspace_bytes(const BwdParams &) { return 0; }
int launch_backward_sm100(flat_ctx *ctx, const BwdParams &) { return fail(ctx, FLAT_ERR_UNSUPPORTED_SHAPE, "not built"); }
}
