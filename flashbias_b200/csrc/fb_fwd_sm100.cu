// Forward tensor-core path, host side: which problems the tcgen05/TMA kernels take, and the dispatch to the
// per-head_dim translation units that hold the kernel instantiations.
#include "fb_fwd_sm100.cuh"

namespace fb {

static bool o_store_ok(const fb_params* p) {
  if (reinterpret_cast<uintptr_t>(p->o) & 15) return false;
  for (int i = 0; i < 3; ++i)
    if (p->o_stride[i] & 7) return false;
  return true;
}

bool fwd_cfg_fits(int D, int RP, int nq) {
#define FB_FIT(DD, RR) \
  if (D == DD && RP == RR) return nq == 2 ? FwdCfg<DD, RR, 2>::FITS : FwdCfg<DD, RR, 1>::FITS;
  FB_FIT(32, 0) FB_FIT(32, 16) FB_FIT(32, 32) FB_FIT(32, 64) FB_FIT(32, 128)
  FB_FIT(64, 0) FB_FIT(64, 16) FB_FIT(64, 32) FB_FIT(64, 64) FB_FIT(64, 128)
  FB_FIT(128, 0) FB_FIT(128, 16) FB_FIT(128, 32) FB_FIT(128, 64) FB_FIT(128, 128)
#undef FB_FIT
  return false;
}

bool fwd_sm100_supported(const fb_params* p, PackPlan* plan) {
  if (p->flags & FB_FLAG_FORCE_GENERAL) return false;
  if (p->alibi_slopes && p->mask_kind != FB_MASK_NONE) return false;  // both at once: shape-generic kernels
  if (!(p->D == 32 || p->D == 64 || p->D == 128)) return false;
  if (!(p->softmax_scale > 0.f) || !isfinite(p->softmax_scale)) return false;
  if (!tma_compatible(p->q, p->q_stride[2], p->q_stride[1], p->q_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->k, p->k_stride[2], p->k_stride[1], p->k_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->v, p->v_stride[2], p->v_stride[1], p->v_stride[0], p->H, p->B)) return false;
  if (!o_store_ok(p)) return false;
  if ((int64_t)p->B * p->H * ((p->Sq + 127) / 128) > 0x7fffffffLL) return false;
  if (!plan_pack(p, plan)) return false;
  return fwd_cfg_fits(p->D, plan->RP, plan->nq);  // shared or tensor memory of an SM exceeded: generic kernels
}

int launch_fwd_sm100(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  switch (p->D) {
    case 32: return dispatch_fwd_d32(p, plan, st);
    case 64: return dispatch_fwd_d64(p, plan, st);
    case 128: return dispatch_fwd_d128(p, plan, st);
  }
  return FB_ENOTBUILT;
}

}  // namespace fb
