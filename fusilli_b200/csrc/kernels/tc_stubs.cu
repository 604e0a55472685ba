// placeholder while the tensor-core kernels are brought up
#include "../common.h"
namespace fb {
bool sdpa_tc_eligible(const Plan &, const Step &) { return false; }
fb_status launch_sdpa_tc(const ExecContext &, const Step &) { return fail(FB_INTERNAL_ERROR, "sdpa tc not built"); }
}
