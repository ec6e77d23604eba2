// Backward tensor-core kernels for head_dim 32 (every packed rank that fits, both 16-bit types).
#include "fb_bwd_t_sm100.cuh"

namespace fb {

template <typename T, int MODE>
static int dispatch_rank(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  switch (plan.RP) {
    case 0:  // no factor operands: the key-major kernel, unless the caller asks for the query-major one
      return (p->flags & FB_FLAG_BWD_QUERY_MAJOR) ? launch_bwd_t<T, 32, 0, 1, MODE>(p, plan, st)
                                                  : launch_bwd_t_t<T, 32, MODE>(p, plan, st);
    case 16: return plan.nq == 2 ? launch_bwd_t<T, 32, 16, 2, MODE>(p, plan, st)
                                  : launch_bwd_t<T, 32, 16, 1, MODE>(p, plan, st);
    case 32: return plan.nq == 2 ? launch_bwd_t<T, 32, 32, 2, MODE>(p, plan, st)
                                  : launch_bwd_t<T, 32, 32, 1, MODE>(p, plan, st);
    case 64: return plan.nq == 2 ? launch_bwd_t<T, 32, 64, 2, MODE>(p, plan, st)
                                  : launch_bwd_t<T, 32, 64, 1, MODE>(p, plan, st);
  }
  return FB_ENOTBUILT;
}

template <typename T>
static int dispatch_bwd_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  if (p->alibi_slopes) return dispatch_rank<T, BWD_ALIBI>(p, plan, st);
  if (p->mask_kind != FB_MASK_NONE) return dispatch_rank<T, BWD_MASK>(p, plan, st);
  return dispatch_rank<T, BWD_PLAIN>(p, plan, st);
}

int dispatch_bwd_d32(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  return p->dtype == FB_DTYPE_F16 ? dispatch_bwd_t<__half>(p, plan, st) : dispatch_bwd_t<__nv_bfloat16>(p, plan, st);
}

}  // namespace fb
