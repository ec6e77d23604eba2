// Persistent form of the backward tensor-core kernel for head_dim 32 with factor operands (plain and masked logits):
// the short-sequence shapes, where a CTA that handles one work item spends more time starting and draining than
// on its tiles.
#include "fb_bwd_p_sm100.cuh"

namespace fb {

template <typename T, int MODE>
static int dispatch_rank_p(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  switch (plan.RP) {
    case 16: return plan.nq == 2 ? launch_bwd_p<T, 32, 16, 2, MODE>(p, plan, st)
                                  : launch_bwd_p<T, 32, 16, 1, MODE>(p, plan, st);
    case 32: return plan.nq == 2 ? launch_bwd_p<T, 32, 32, 2, MODE>(p, plan, st)
                                  : launch_bwd_p<T, 32, 32, 1, MODE>(p, plan, st);
    case 64: return plan.nq == 2 ? launch_bwd_p<T, 32, 64, 2, MODE>(p, plan, st)
                                  : launch_bwd_p<T, 32, 64, 1, MODE>(p, plan, st);
  }
  return FB_ENOTBUILT;
}

template <typename T>
static int dispatch_bwd_p(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  if (p->alibi_slopes) return FB_ENOTBUILT;
  if (p->mask_kind != FB_MASK_NONE) return dispatch_rank_p<T, BWD_MASK>(p, plan, st);
  return dispatch_rank_p<T, BWD_PLAIN>(p, plan, st);
}

int dispatch_bwd_d32p(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  return p->dtype == FB_DTYPE_F16 ? dispatch_bwd_p<__half>(p, plan, st) : dispatch_bwd_p<__nv_bfloat16>(p, plan, st);
}

}  // namespace fb
