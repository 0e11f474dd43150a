// Placeholders while the tcgen05 kernels are brought up one by one.
#include "tm_core.h"
namespace tmc {
#ifndef TM_HAVE_GEMM_TC
bool gemm_tc_eligible(const GemmProblem&, std::string* why) { if (why) *why = "not built"; return false; }
std::string launch_gemm_tc(const GemmProblem&, const LaunchCtx&) { return "not built"; }
#endif
#ifndef TM_HAVE_ATTN_FWD_TC
bool attn_fwd_tc_eligible(const AttnProblem&, std::string* why) { if (why) *why = "not built"; return false; }
std::string launch_attn_fwd_tc(const AttnProblem&, const LaunchCtx&) { return "not built"; }
#endif
#ifndef TM_HAVE_ATTN_BWD_TC
bool attn_bwd_tc_eligible(const AttnProblem&, std::string* why) { if (why) *why = "not built"; return false; }
std::string launch_attn_bwd_dq_tc(const AttnProblem&, const LaunchCtx&) { return "not built"; }
std::string launch_attn_bwd_dkdv_tc(const AttnProblem&, const LaunchCtx&) { return "not built"; }
#endif
}
