// Operand preparation for the tensor-core kernels.
//
// The kernels accumulate all logit terms in ONE fp32 accumulator,  S = qs.k + qb.kb,  where the softmax
// scale has to live inside an operand:
//   * scale an exact power of two: qs = q (the caller's tensor, untouched) and qb = q_bias / scale,
//     which is exact in the 16-bit type; the exponent argument is S * scale * log2(e);
//   * otherwise: qs = q * scale, stored as a (hi, lo) pair of 16-bit terms (contraction 2*head_dim),
//     and qb = q_bias as given, so that the products of the bias factors stay exact and un-scaled --
//     terms as large as an ALiBi position cancel inside one MMA instead of being rounded first.
// The backward keeps its key tile resident and streams the query tiles, so it puts the split on the key side
// instead: S = q.(k*scale), with k*scale as a (hi, lo) pair.
// Factors are zero-padded to RP columns (16/32/64; the forward also takes 128).  The backward also gets a centred k-side copy
// (k_bias minus the k_bias of the middle key of its group of 32 keys, as a (hi, lo) pair).
#include <math.h>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

static int pad_pow2_16(int x) {
  int r = 16;
  while (r < x) r <<= 1;
  return r;
}

bool plan_pack(const fb_params* p, PackPlan* plan, bool for_bwd) {
  plan->Bq = p->q_bias_stride[0] == 0 ? 1 : p->B;
  plan->Hq = p->q_bias_stride[1] == 0 ? 1 : p->H;
  plan->Bk = p->k_bias_stride[0] == 0 ? 1 : p->B;
  plan->Hk = p->k_bias_stride[1] == 0 ? 1 : p->H;
  int e;
  bool pow2 = frexpf(p->softmax_scale, &e) == 0.5f;
  // fp16 factors divided by a scale below one could leave the range of the type: take the split form instead
  if (pow2 && p->dtype == FB_DTYPE_F16 && p->softmax_scale != 1.f && p->R > 0) pow2 = false;
  // without factor operands nothing shares the accumulator with q.k: the scale lives in the exponent multiplier
  if (p->R <= 0) pow2 = true;
  plan->nq = pow2 ? 1 : 2;
  plan->qb_mult = (pow2 && p->R > 0) ? (float)(1.0 / (double)p->softmax_scale) : 1.f;
  // forward: scaled-query copy; backward: scaled-key copy
  plan->qs_bytes = pow2 ? 0 : round256((size_t)p->B * p->H * (for_bwd ? p->Sk : p->Sq) * 2 * p->D * 2);
  plan->RC = 0;
  plan->kc_bytes = 0;
  if (p->R <= 0) {
    plan->RP = 0;
    plan->q_bytes = plan->k_bytes = 0;
    return true;
  }
  // the centred k-side copy of the backward holds a (hi, lo) pair: twice the rank
  plan->RP = pad_pow2_16(for_bwd ? 2 * p->R : p->R);
  // backward at head_dim 32: factor tiles as wide as the Q/K tiles, so that [Q | Qb] and [K | Kc] are read as one
  // MMA operand each (one product instead of two per 16 query rows / keys)
  if (for_bwd && p->D == 32 && plan->RP < 32) plan->RP = 32;
  if (plan->RP > (for_bwd ? 64 : 128)) return false;
  plan->q_bytes = round256((size_t)plan->Bq * plan->Hq * p->Sq * plan->RP * 2);
  plan->k_bytes = round256((size_t)plan->Bk * plan->Hk * p->Sk * plan->RP * 2);
  if (for_bwd) {
    // beside a head_dim-32 K tile the centred copy is 32 columns wide: [K | Kc] then reads as one MMA operand
    plan->RC = (p->D == 32 && plan->RP < 32) ? 32 : plan->RP;
    plan->kc_bytes = round256((size_t)plan->Bk * plan->Hk * p->Sk * plan->RC * 2);
  }
  return true;
}

// One factor: (Bx, Hx, S, R) with strides -> packed rows (and the centred copy for the k side of the backward).
template <typename T>
struct FactorJob {
  const T* src;
  int64_t sb, sh, ss;
  int Bx, Hx, S;
  float mult;
  T* dst;
  T* dst_centered;
};
// One tensor scaled and split: (B, H, S, D) with strides -> (B, H, S, 2D) = [hi | lo] of x * scale.
template <typename T>
struct ScaledJob {
  const T* src;
  int64_t sb, sh, ss;
  int S;
  T* dst;  // nullptr: no such job
};

// One thread per (b, h, s) row; the packed row is built 8 columns (one 16-byte store) at a time.
template <typename T>
__device__ __forceinline__ void pack_factor_row(const FactorJob<T>& j, int64_t idx, int R, int RP, int RC, int* status) {
  const T* __restrict__ src = j.src;
  const int64_t sb = j.sb, sh = j.sh, ss = j.ss;
  const int Hx = j.Hx, S = j.S;
  const float mult = j.mult;
  T* __restrict__ dst = j.dst;
  T* __restrict__ dst_centered = j.dst_centered;
  const int64_t total = (int64_t)j.Bx * Hx * S;
  if (idx >= total) return;
  const int s = (int)(idx % S);
  const int h = (int)((idx / S) % Hx);
  const int b = (int)(idx / ((int64_t)S * Hx));
  const T* in = src + b * sb + h * sh + s * ss;
  bool overflow = false;
  for (int c0 = 0; c0 < RP; c0 += 8) {
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    T* y = reinterpret_cast<T*>(&w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int c = c0 + i;
      if (c < R) {
        const float x = to_f32(in[c]);
        y[i] = from_f32<T>(x * mult);  // mult is 1 or a power of two: exact unless it overflows
        overflow |= !isfinite(to_f32(y[i])) && isfinite(x);
      }
    }
    *reinterpret_cast<uint4*>(dst + idx * RP + c0) = w;
  }
  if (overflow && status) atomicExch(status, FB_DEV_FACTOR_OVERFLOW);
  if (dst_centered) {
    // k-side factor minus the factor of the middle key of its group of 32 keys: small-magnitude copy used
    // for dq_bias = dS.k_bias (the removed constant is re-applied in fp32 through the row sum of dS);
    // two-term split: columns [0,R) hi, [RC/2, RC/2 + R) lo, zero elsewhere
    int s0 = (s & ~31) + 16;
    if (s0 > S - 1) s0 = S - 1;
    const T* in0 = src + b * sb + h * sh + (int64_t)s0 * ss;
    for (int c0 = 0; c0 < RC; c0 += 8) {
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      T* y = reinterpret_cast<T*>(&w);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i;
        const bool lo = c >= RC / 2;
        const int cc = lo ? c - RC / 2 : c;
        if (cc < R) {
          const float x = to_f32(in[cc]) - to_f32(in0[cc]);
          const T hi = from_f32<T>(x);
          y[i] = lo ? from_f32<T>(x - to_f32(hi)) : hi;
        }
      }
      *reinterpret_cast<uint4*>(dst_centered + idx * RC + c0) = w;
    }
  }
}

// qs[b][h][s][0:D] = T(x * scale), qs[b][h][s][D:2D] = T(x * scale - hi): the scaled query (or key) as two 16-bit
// terms.
// One thread converts 8 consecutive elements (16-byte load, two 16-byte stores).
template <typename T>
__device__ __forceinline__ void pack_scaled_chunk(const ScaledJob<T>& j, int64_t idx, int B, int H, int D, float scale) {
  const T* __restrict__ q = j.src;
  const int64_t sb = j.sb, sh = j.sh, ss = j.ss;
  const int S = j.S;
  T* __restrict__ qs = j.dst;
  const int d8 = D / 8;  // idx = (b, h, s, d/8)
  const int64_t total = (int64_t)B * H * S * d8;
  if (idx >= total) return;
  const int c = (int)(idx % d8);
  const int s = (int)((idx / d8) % S);
  const int h = (int)((idx / ((int64_t)d8 * S)) % H);
  const int b = (int)(idx / ((int64_t)d8 * S * H));
  const uint4 raw = *reinterpret_cast<const uint4*>(q + b * sb + h * sh + s * ss + c * 8);
  const T* x = reinterpret_cast<const T*>(&raw);
  uint4 hi4, lo4;
  T* hi = reinterpret_cast<T*>(&hi4);
  T* lo = reinterpret_cast<T*>(&lo4);
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float v = to_f32(x[e]) * scale;
    hi[e] = from_f32<T>(v);
    lo[e] = from_f32<T>(v - to_f32(hi[e]));
  }
  T* row = qs + (((int64_t)b * H + h) * S + s) * (2 * D);
  *reinterpret_cast<uint4*>(row + c * 8) = hi4;
  *reinterpret_cast<uint4*>(row + D + c * 8) = lo4;
}

// All operand preparation of one call in one launch: blocks [0, nbq) pack the q-side factor, [nbq, nbq + nbk) the
// k-side factor (and its centred copy), the rest split the scaled query (forward) or key (backward).
template <typename T>
__global__ void __launch_bounds__(256) pack_operands_kernel(FactorJob<T> fq, FactorJob<T> fk, ScaledJob<T> sc,
                                                            unsigned nbq, unsigned nbk, int B, int H, int D, int R,
                                                            int RP, int RC, float scale, int* status) {
  const unsigned blk = blockIdx.x;
  if (blk < nbq) {
    pack_factor_row<T>(fq, (int64_t)blk * 256 + threadIdx.x, R, RP, RC, status);
  } else if (blk < nbq + nbk) {
    pack_factor_row<T>(fk, (int64_t)(blk - nbq) * 256 + threadIdx.x, R, RP, RC, status);
  } else {
    pack_scaled_chunk<T>(sc, (int64_t)(blk - nbq - nbk) * 256 + threadIdx.x, B, H, D, scale);
  }
}

template <typename T>
static int launch_pack_operands_t(const fb_params* p, const PackPlan& plan, void* qpack, void* kpack, void* kcenter,
                                  bool scaled_is_key, void* scaled, cudaStream_t st) {
  FactorJob<T> fq{}, fk{};
  ScaledJob<T> sc{};
  unsigned nbq = 0, nbk = 0, nbs = 0;
  if (plan.RP) {
    fq = {reinterpret_cast<const T*>(p->q_bias), p->q_bias_stride[0], p->q_bias_stride[1], p->q_bias_stride[2],
          plan.Bq, plan.Hq, p->Sq, plan.qb_mult, reinterpret_cast<T*>(qpack), nullptr};
    fk = {reinterpret_cast<const T*>(p->k_bias), p->k_bias_stride[0], p->k_bias_stride[1], p->k_bias_stride[2],
          plan.Bk, plan.Hk, p->Sk, 1.f, reinterpret_cast<T*>(kpack), reinterpret_cast<T*>(kcenter)};
    nbq = (unsigned)(((int64_t)plan.Bq * plan.Hq * p->Sq + 255) / 256);
    nbk = (unsigned)(((int64_t)plan.Bk * plan.Hk * p->Sk + 255) / 256);
  }
  if (plan.nq == 2) {
    const int S = scaled_is_key ? p->Sk : p->Sq;
    const int64_t* stv = scaled_is_key ? p->k_stride : p->q_stride;
    sc = {reinterpret_cast<const T*>(scaled_is_key ? p->k : p->q), stv[0], stv[1], stv[2], S,
          reinterpret_cast<T*>(scaled)};
    nbs = (unsigned)(((int64_t)p->B * p->H * S * (p->D / 8) + 255) / 256);
  }
  if (nbq + nbk + nbs == 0) return 0;
  pack_operands_kernel<T><<<nbq + nbk + nbs, 256, 0, st>>>(fq, fk, sc, nbq, nbk, p->B, p->H, p->D, p->R, plan.RP,
                                                           plan.RC, p->softmax_scale, p->status);
  note_launch();
  return (int)cudaGetLastError();
}

int launch_pack_operands(const fb_params* p, const PackPlan& plan, void* qpack, void* kpack, void* kcenter,
                         bool scaled_is_key, void* scaled, cudaStream_t st) {
  return p->dtype == FB_DTYPE_F16
             ? launch_pack_operands_t<__half>(p, plan, qpack, kpack, kcenter, scaled_is_key, scaled, st)
             : launch_pack_operands_t<__nv_bfloat16>(p, plan, qpack, kpack, kcenter, scaled_is_key, scaled, st);
}

}  // namespace fb
