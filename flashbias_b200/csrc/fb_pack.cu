// Packing of the low-rank bias factors into tensor-core operand columns.
//
// The tensor-core kernels accumulate  S' = q.k + qp.kp  in one fp32 accumulator and apply the
// softmax scale afterwards, so the q-side factor is divided by the scale first.  To keep the
// unscaled bias term exact to fp32 level, q_bias/scale is split into `nsplit` 16-bit terms
// (x = hi + mid + lo, each the rounding of the running remainder) stored side by side, and the
// k-side factor is repeated under each term.  Columns beyond nsplit*R are zero.
#include <math.h>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

static int pad_pow2_16(int x) {
  int r = 16;
  while (r < x) r <<= 1;
  return r;
}

bool plan_pack(const fb_params* p, PackPlan* plan, int min_rp) {
  plan->Bq = p->q_bias_stride[0] == 0 ? 1 : p->B;
  plan->Hq = p->q_bias_stride[1] == 0 ? 1 : p->H;
  plan->Bk = p->k_bias_stride[0] == 0 ? 1 : p->B;
  plan->Hk = p->k_bias_stride[1] == 0 ? 1 : p->H;
  if (p->R <= 0) {
    plan->nsplit = 1;
    plan->RP = 0;
    plan->q_bytes = plan->k_bytes = 0;
    return true;
  }
  int e;
  const bool pow2 = frexpf(p->softmax_scale, &e) == 0.5f;
  if (pow2) {
    plan->nsplit = 1;
  } else {
    plan->nsplit = pad_pow2_16(3 * p->R) == pad_pow2_16(2 * p->R) ? 3 : 2;
  }
  // at least two column groups: the centred k-side copy used by the backward holds a (hi, lo) pair
  plan->RP = pad_pow2_16((plan->nsplit < 2 ? 2 : plan->nsplit) * p->R);
  if (plan->RP < min_rp) plan->RP = min_rp;
  if (plan->RP > 64) return false;
  plan->q_bytes = round256((size_t)plan->Bq * plan->Hq * p->Sq * plan->RP * 2);
  plan->k_bytes = round256((size_t)plan->Bk * plan->Hk * p->Sk * plan->RP * 2);
  return true;
}

template <typename T>
__global__ void __launch_bounds__(256) pack_factor_kernel(const T* __restrict__ src, int64_t sb, int64_t sh, int64_t ss,
                                                          int Bx, int Hx, int S, int R, int RP, int nsplit,
                                                          float mult, int split, T* __restrict__ dst,
                                                          T* __restrict__ dst_centered, int* status) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // (b, h, s)
  const int64_t total = (int64_t)Bx * Hx * S;
  if (idx >= total) return;
  const int s = (int)(idx % S);
  const int h = (int)((idx / S) % Hx);
  const int b = (int)(idx / ((int64_t)S * Hx));
  const T* in = src + b * sb + h * sh + s * ss;
  T* out = dst + idx * RP;
  for (int c = nsplit * R; c < RP; ++c) out[c] = from_f32<T>(0.f);
  if (dst_centered) {
    // k-side factor minus the factor of the middle key of its group of 32 keys: small-magnitude copy used
    // for dq_bias = dS.k_bias (the removed constant is re-applied in fp32 through the row sum of dS)
    int s0 = (s & ~31) + 16;
    if (s0 > S - 1) s0 = S - 1;
    const T* in0 = src + b * sb + h * sh + (int64_t)s0 * ss;
    T* outc = dst_centered + idx * RP;
    for (int c = 2 * R; c < RP; ++c) outc[c] = from_f32<T>(0.f);
    for (int c = 0; c < R; ++c) {  // two-term split: columns [0,R) hi, [R,2R) lo
      const float x = to_f32(in[c]) - to_f32(in0[c]);
      const T hi = from_f32<T>(x);
      outc[c] = hi;
      outc[R + c] = from_f32<T>(x - to_f32(hi));
    }
  }
  for (int r = 0; r < R; ++r) {
    const T raw = in[r];
    if (!split) {
      for (int t = 0; t < nsplit; ++t) out[t * R + r] = raw;
    } else {
      float rem = to_f32(raw) * mult;
      for (int t = 0; t < nsplit; ++t) {
        const T term = from_f32<T>(rem);
        const float tf = to_f32(term);
        if (t == 0 && !isfinite(tf) && isfinite(to_f32(raw)) && status) atomicExch(status, FB_DEV_FACTOR_OVERFLOW);
        out[t * R + r] = term;
        rem -= tf;
      }
    }
  }
}

template <typename T>
static int launch_pack_t(const fb_params* p, const PackPlan& plan, void* qpack, void* kpack, void* kcenter,
                         cudaStream_t st) {
  const float inv_scale = (float)(1.0 / (double)p->softmax_scale);
  const int64_t nq = (int64_t)plan.Bq * plan.Hq * p->Sq, nk = (int64_t)plan.Bk * plan.Hk * p->Sk;
  pack_factor_kernel<T><<<(unsigned)((nq + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const T*>(p->q_bias), p->q_bias_stride[0], p->q_bias_stride[1], p->q_bias_stride[2], plan.Bq,
      plan.Hq, p->Sq, p->R, plan.RP, plan.nsplit, inv_scale, 1, reinterpret_cast<T*>(qpack), nullptr, p->status);
  pack_factor_kernel<T><<<(unsigned)((nk + 255) / 256), 256, 0, st>>>(
      reinterpret_cast<const T*>(p->k_bias), p->k_bias_stride[0], p->k_bias_stride[1], p->k_bias_stride[2], plan.Bk,
      plan.Hk, p->Sk, p->R, plan.RP, plan.nsplit, 1.f, 0, reinterpret_cast<T*>(kpack), reinterpret_cast<T*>(kcenter),
      p->status);
  note_launch(2);
  return (int)cudaGetLastError();
}

int launch_pack(const fb_params* p, const PackPlan& plan, void* qpack, void* kpack, void* kcenter, cudaStream_t st) {
  if (plan.RP == 0) return 0;
  return p->dtype == FB_DTYPE_F16 ? launch_pack_t<__half>(p, plan, qpack, kpack, kcenter, st)
                                  : launch_pack_t<__nv_bfloat16>(p, plan, qpack, kpack, kcenter, st);
}

}  // namespace fb
