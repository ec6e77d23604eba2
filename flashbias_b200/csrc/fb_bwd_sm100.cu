// Backward tensor-core path, host side: which problems the tcgen05/TMA kernels take, workspace size, and the
// dispatch to the per-head_dim translation units that hold the kernel instantiations.
#include "fb_bwd_sm100.cuh"

namespace fb {

static bool rows_16b_ok(const void* ptr, const int64_t* st) {
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
  for (int i = 0; i < 3; ++i)
    if (st[i] & 7) return false;
  return true;
}

// the variants launch_bwd_sm100 can dispatch to, and whether their tiles fit one SM
bool bwd_cfg_fits(int D, int RP, int nq) {
#define FB_FIT(DD, RR) \
  if (D == DD && RP == RR) return nq == 2 ? BwdCfg<DD, RR, 2>::FITS : BwdCfg<DD, RR, 1>::FITS;
  FB_FIT(32, 0) FB_FIT(32, 16) FB_FIT(32, 32) FB_FIT(32, 64)
  FB_FIT(64, 0) FB_FIT(64, 16) FB_FIT(64, 32)
#undef FB_FIT
  return false;
}

bool bwd_sm100_supported(const fb_params* p, PackPlan* plan) {
  if (p->flags & FB_FLAG_FORCE_GENERAL) return false;
  if (p->alibi_slopes && p->mask_kind != FB_MASK_NONE) return false;  // both at once: shape-generic kernels
  if (!(p->D == 32 || p->D == 64)) return false;
  if (!(p->softmax_scale > 0.f) || !isfinite(p->softmax_scale)) return false;
  if (!plan_pack(p, plan, true)) return false;
  if (!bwd_cfg_fits(p->D, plan->RP, plan->nq)) return false;  // shared or tensor memory of an SM exceeded
  if (!tma_compatible(p->q, p->q_stride[2], p->q_stride[1], p->q_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->k, p->k_stride[2], p->k_stride[1], p->k_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->v, p->v_stride[2], p->v_stride[1], p->v_stride[0], p->H, p->B)) return false;
  if (p->dout && !tma_compatible(p->dout, p->dout_stride[2], p->dout_stride[1], p->dout_stride[0], p->H, p->B))
    return false;
  if (p->dq && !rows_16b_ok(p->dq, p->dq_stride)) return false;
  if (p->dk && !rows_16b_ok(p->dk, p->dk_stride)) return false;
  if (p->dv && !rows_16b_ok(p->dv, p->dv_stride)) return false;
  if ((int64_t)p->B * p->H * ((p->Sk + 127) / 128) > 0x7fffffffLL) return false;
  return true;
}

size_t bwd_sm100_workspace(const fb_params* p, const PackPlan& plan) { return bwd_layout(p, plan).total; }

// Whether the persistent form of the query-major kernel is the better one: few query tiles per work item (a CTA
// that handles one item then spends more time starting and draining than on its tiles) and more items than SMs.
static bool bwd_prefers_persistent(const fb_params* p) {
  int dev = 0;
  cudaGetDevice(&dev);
  const int sms = device_sm_count(dev);
  const int nq = (p->Sq + 127) / 128, nk = (p->Sk + 127) / 128;
  const int tiles_per_item = p->causal ? (nq + 1) / 2 : nq;  // mean, under causal masking
  return sms > 0 && tiles_per_item <= 8 && (int64_t)nk * p->B * p->H >= 2 * (int64_t)sms;
}

int launch_bwd_sm100(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  // (the persistent form writes dK and dV with tile stores: their layout must be one a tensor map can describe)
  if (p->D == 32 && plan.RP > 0 && !p->alibi_slopes && !(p->flags & FB_FLAG_BWD_ONE_ITEM) &&
      ((p->flags & FB_FLAG_BWD_PERSISTENT) || bwd_prefers_persistent(p)) &&
      tma_compatible(p->dk, p->dk_stride[2], p->dk_stride[1], p->dk_stride[0], p->H, p->B) &&
      tma_compatible(p->dv, p->dv_stride[2], p->dv_stride[1], p->dv_stride[0], p->H, p->B))
    return dispatch_bwd_d32p(p, plan, st);
  return p->D == 32 ? dispatch_bwd_d32(p, plan, st) : p->D == 64 ? dispatch_bwd_d64(p, plan, st) : FB_ENOTBUILT;
}

}  // namespace fb
