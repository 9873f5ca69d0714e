// placeholder
#include "common.cuh"
namespace ahpc {
bool fa_tc_supported(const FaLaunch&, const char** why) { if (why) *why = "not built"; return false; }
ahpc_status launch_fa_tc(const FaLaunch&) { return fail(AHPC_UNSUPPORTED_OPERATION, "not built"); }
}
