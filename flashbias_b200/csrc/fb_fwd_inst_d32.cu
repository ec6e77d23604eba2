// Forward tensor-core kernels for head_dim 32 (every packed rank, both 16-bit types).
#include "fb_fwd_sm100.cuh"

namespace fb {

FB_FWD_DISPATCH_BODY(32)

int dispatch_fwd_d32(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  return p->dtype == FB_DTYPE_F16 ? dispatch_fwd_t<__half>(p, plan, st) : dispatch_fwd_t<__nv_bfloat16>(p, plan, st);
}

}  // namespace fb
