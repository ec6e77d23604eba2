// Shape-generic CUDA-core kernels: any head_dim <= 128, any rank <= 256, any strides, additive
// masks.  They serve the argument combinations the tensor-core kernels do not take and double as
// an on-device cross-check of them.  One warp owns one query row (forward, dQ) or one key row
// (dK/dV); the partner rows are visited 32 at a time, one per lane.
#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

constexpr int kWarps = 4;
constexpr int kMaxD = 128;
constexpr int kMaxR = 256;

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

__device__ __forceinline__ float load_mask(const fb_params& p, int b, int h, int row, int col) {
  if (p.mask_kind == FB_MASK_NONE) return 0.f;
  if (p.mask_batch_period > 0) b %= p.mask_batch_period;
  const int64_t off = b * p.mask_stride[0] + h * p.mask_stride[1] +
                      (p.mask_kind == FB_MASK_MATRIX ? row * p.mask_stride[2] : 0) + col;
  if (p.mask_dtype == FB_DTYPE_F32) return reinterpret_cast<const float*>(p.mask)[off];
  if (p.mask_dtype == FB_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(p.mask)[off]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.mask)[off]);
}

template <typename T>
__device__ __forceinline__ const T* row_ptr(const void* base, const int64_t* st, int b, int h, int row) {
  return reinterpret_cast<const T*>(base) + b * st[0] + h * st[1] + row * st[2];
}

// logit of (query row in shared memory, key row j in global memory)
template <typename T>
__device__ __forceinline__ float logit(const fb_params& p, const float* sq, const float* sqb, int b, int h, int i,
                                       int j) {
  const T* kr = row_ptr<T>(p.k, p.k_stride, b, h, j);
  float acc = 0.f;
  for (int d = 0; d < p.D; ++d) acc += sq[d] * to_f32(kr[d]);
  acc *= p.softmax_scale;
  if (p.R > 0) {
    const T* kb = row_ptr<T>(p.k_bias, p.k_bias_stride, b, h, j);
    float bb = 0.f;
    for (int r = 0; r < p.R; ++r) bb += sqb[r] * to_f32(kb[r]);
    acc += bb;
  }
  if (p.alibi_slopes) acc += p.alibi_slopes[h] * (float)(j - i);
  return acc + load_mask(p, b, h, i, j);
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) fwd_general_kernel(const fb_params p) {
  __shared__ float s_q[kWarps][kMaxD];
  __shared__ float s_qb[kWarps][kMaxR];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t gw = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t total = (int64_t)p.B * p.H * p.Sq;
  if (gw >= total) return;
  const int i = (int)(gw % p.Sq);
  const int bh = (int)(gw / p.Sq);
  const int b = bh / p.H, h = bh % p.H;
  const T* qr = row_ptr<T>(p.q, p.q_stride, b, h, i);
  for (int d = lane; d < p.D; d += 32) s_q[warp][d] = to_f32(qr[d]);
  if (p.R > 0) {
    const T* qb = row_ptr<T>(p.q_bias, p.q_bias_stride, b, h, i);
    for (int r = lane; r < p.R; r += 32) s_qb[warp][r] = to_f32(qb[r]);
  }
  __syncwarp();
  float m = -INFINITY, l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  const int jend = p.causal ? min(p.Sk, i + 1) : p.Sk;
  for (int j0 = 0; j0 < jend; j0 += 32) {
    const int j = j0 + lane;
    float s = j < jend ? logit<T>(p, s_q[warp], s_qb[warp], b, h, i, j) : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float pj = __expf(s - m_new);  // exp(-inf) = 0
    const float alpha = __expf(m - m_new);
    l = l * alpha + warp_sum(pj);
    m = m_new;
    const int cnt = min(32, jend - j0);
#pragma unroll
    for (int t = 0; t < 4; ++t) o[t] *= alpha;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pp = __shfl_sync(0xffffffffu, pj, jj);
      const T* vr = row_ptr<T>(p.v, p.v_stride, b, h, j0 + jj);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < p.D) o[t] += pp * to_f32(vr[d]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  T* orow = reinterpret_cast<T*>(p.o) + b * p.o_stride[0] + h * p.o_stride[1] + (int64_t)i * p.o_stride[2];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int d = lane + 32 * t;
    if (d < p.D) orow[d] = from_f32<T>(o[t] * inv);
  }
  if (lane == 0) p.lse[(int64_t)bh * p.lse_stride_bh + i] = l > 0.f ? m + logf(l) : -INFINITY;
}

// delta[bh, i] = sum_d o[i, d] * dout[i, d]
template <typename T>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const fb_params p) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // (b, i, h), h fastest
  const int64_t total = (int64_t)p.B * p.Sq * p.H;
  if (idx >= total) return;
  const int h = (int)(idx % p.H);
  const int i = (int)((idx / p.H) % p.Sq);
  const int b = (int)(idx / ((int64_t)p.H * p.Sq));
  const T* orow = row_ptr<T>(p.o, p.o_stride, b, h, i);
  const T* drow = row_ptr<T>(p.dout, p.dout_stride, b, h, i);
  float acc = 0.f;
  const bool vec = (p.D % 8 == 0) && ((reinterpret_cast<uintptr_t>(orow) | reinterpret_cast<uintptr_t>(drow)) & 15) == 0;
  if (vec) {
    for (int d = 0; d < p.D; d += 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(orow + d);
      const uint4 c = *reinterpret_cast<const uint4*>(drow + d);
      const T* pa = reinterpret_cast<const T*>(&a);
      const T* pc = reinterpret_cast<const T*>(&c);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += to_f32(pa[e]) * to_f32(pc[e]);
    }
  } else {
    for (int d = 0; d < p.D; ++d) acc += to_f32(orow[d]) * to_f32(drow[d]);
  }
  p.delta[((int64_t)b * p.H + h) * p.lse_stride_bh + i] = acc;
}

// fp32 accumulators of the factor gradients live in the workspace, un-expanded (broadcast dims of
// size 1), contiguous (Bx, S, Hx, R).
struct FactorAcc {
  float* dqb;
  float* dkb;
  int Bq, Hq, Bk, Hk;
};
__host__ __device__ inline FactorAcc factor_acc(const fb_params& p) {
  FactorAcc a;
  a.Bq = p.q_bias_stride[0] == 0 ? 1 : p.B;
  a.Hq = p.q_bias_stride[1] == 0 ? 1 : p.H;
  a.Bk = p.k_bias_stride[0] == 0 ? 1 : p.B;
  a.Hk = p.k_bias_stride[1] == 0 ? 1 : p.H;
  a.dqb = reinterpret_cast<float*>(p.workspace);
  a.dkb = a.dqb + ((((size_t)a.Bq * p.Sq * a.Hq * p.R) + 63) & ~size_t(63));
  return a;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) bwd_dq_general_kernel(const fb_params p) {
  __shared__ float s_q[kWarps][kMaxD];
  __shared__ float s_do[kWarps][kMaxD];
  __shared__ float s_qb[kWarps][kMaxR];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t gw = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t total = (int64_t)p.B * p.H * p.Sq;
  if (gw >= total) return;
  const int i = (int)(gw % p.Sq);
  const int bh = (int)(gw / p.Sq);
  const int b = bh / p.H, h = bh % p.H;
  const T* qr = row_ptr<T>(p.q, p.q_stride, b, h, i);
  const T* dr = row_ptr<T>(p.dout, p.dout_stride, b, h, i);
  for (int d = lane; d < p.D; d += 32) {
    s_q[warp][d] = to_f32(qr[d]);
    s_do[warp][d] = to_f32(dr[d]);
  }
  if (p.R > 0) {
    const T* qb = row_ptr<T>(p.q_bias, p.q_bias_stride, b, h, i);
    for (int r = lane; r < p.R; r += 32) s_qb[warp][r] = to_f32(qb[r]);
  }
  __syncwarp();
  const float lse = p.lse[(int64_t)bh * p.lse_stride_bh + i];
  const float delta = p.delta[(int64_t)bh * p.lse_stride_bh + i];
  float dq[4] = {0.f, 0.f, 0.f, 0.f}, dqb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int jend = p.causal ? min(p.Sk, i + 1) : p.Sk;
  for (int j0 = 0; j0 < jend && lse != -INFINITY; j0 += 32) {
    const int j = j0 + lane;
    float ds = 0.f;
    if (j < jend) {
      const float s = logit<T>(p, s_q[warp], s_qb[warp], b, h, i, j);
      const float pj = __expf(s - lse);
      const T* vr = row_ptr<T>(p.v, p.v_stride, b, h, j);
      float dp = 0.f;
      for (int d = 0; d < p.D; ++d) dp += s_do[warp][d] * to_f32(vr[d]);
      ds = pj * (dp - delta);
    }
    const int cnt = min(32, jend - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float g = __shfl_sync(0xffffffffu, ds, jj);
      const T* kr = row_ptr<T>(p.k, p.k_stride, b, h, j0 + jj);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < p.D) dq[t] += g * to_f32(kr[d]);
      }
      if (p.R > 0) {
        const T* kb = row_ptr<T>(p.k_bias, p.k_bias_stride, b, h, j0 + jj);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int r = lane + 32 * t;
          if (r < p.R) dqb[t] += g * to_f32(kb[r]);
        }
      }
    }
  }
  T* dqrow = reinterpret_cast<T*>(p.dq) + b * p.dq_stride[0] + h * p.dq_stride[1] + (int64_t)i * p.dq_stride[2];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int d = lane + 32 * t;
    if (d < p.D) dqrow[d] = from_f32<T>(dq[t] * p.softmax_scale);
  }
  if (p.R > 0) {
    const FactorAcc fa = factor_acc(p);
    const int bb = fa.Bq == 1 ? 0 : b, hh = fa.Hq == 1 ? 0 : h;
    float* dst = fa.dqb + (((int64_t)bb * p.Sq + i) * fa.Hq + hh) * p.R;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int r = lane + 32 * t;
      if (r < p.R) atomicAdd(dst + r, dqb[t]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32) bwd_dkv_general_kernel(const fb_params p) {
  __shared__ float s_k[kWarps][kMaxD];
  __shared__ float s_v[kWarps][kMaxD];
  __shared__ float s_kb[kWarps][kMaxR];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t gw = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t total = (int64_t)p.B * p.H * p.Sk;
  if (gw >= total) return;
  const int j = (int)(gw % p.Sk);
  const int bh = (int)(gw / p.Sk);
  const int b = bh / p.H, h = bh % p.H;
  const T* kr = row_ptr<T>(p.k, p.k_stride, b, h, j);
  const T* vr = row_ptr<T>(p.v, p.v_stride, b, h, j);
  for (int d = lane; d < p.D; d += 32) {
    s_k[warp][d] = to_f32(kr[d]);
    s_v[warp][d] = to_f32(vr[d]);
  }
  if (p.R > 0) {
    const T* kb = row_ptr<T>(p.k_bias, p.k_bias_stride, b, h, j);
    for (int r = lane; r < p.R; r += 32) s_kb[warp][r] = to_f32(kb[r]);
  }
  __syncwarp();
  float dk[4] = {0.f, 0.f, 0.f, 0.f}, dv[4] = {0.f, 0.f, 0.f, 0.f};
  float dkb[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int ibeg = p.causal ? (j / 32) * 32 : 0;
  for (int i0 = ibeg; i0 < p.Sq; i0 += 32) {
    const int i = i0 + lane;
    float pj = 0.f, ds = 0.f;
    if (i < p.Sq && (!p.causal || j <= i)) {
      const float lse = p.lse[(int64_t)bh * p.lse_stride_bh + i];
      if (lse != -INFINITY) {
        const T* qr = row_ptr<T>(p.q, p.q_stride, b, h, i);
        const T* dr = row_ptr<T>(p.dout, p.dout_stride, b, h, i);
        float s = 0.f, dp = 0.f;
        for (int d = 0; d < p.D; ++d) {
          s += to_f32(qr[d]) * s_k[warp][d];
          dp += to_f32(dr[d]) * s_v[warp][d];
        }
        s *= p.softmax_scale;
        if (p.R > 0) {
          const T* qb = row_ptr<T>(p.q_bias, p.q_bias_stride, b, h, i);
          float bb = 0.f;
          for (int r = 0; r < p.R; ++r) bb += to_f32(qb[r]) * s_kb[warp][r];
          s += bb;
        }
        if (p.alibi_slopes) s += p.alibi_slopes[h] * (float)(j - i);
        s += load_mask(p, b, h, i, j);
        pj = __expf(s - lse);
        ds = pj * (dp - p.delta[(int64_t)bh * p.lse_stride_bh + i]);
      }
    }
    const int cnt = min(32, p.Sq - i0);
    for (int ii = 0; ii < cnt; ++ii) {
      const float pp = __shfl_sync(0xffffffffu, pj, ii);
      const float g = __shfl_sync(0xffffffffu, ds, ii);
      if (pp == 0.f && g == 0.f) continue;
      const T* qr = row_ptr<T>(p.q, p.q_stride, b, h, i0 + ii);
      const T* dr = row_ptr<T>(p.dout, p.dout_stride, b, h, i0 + ii);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int d = lane + 32 * t;
        if (d < p.D) {
          dv[t] += pp * to_f32(dr[d]);
          dk[t] += g * to_f32(qr[d]);
        }
      }
      if (p.R > 0) {
        const T* qb = row_ptr<T>(p.q_bias, p.q_bias_stride, b, h, i0 + ii);
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const int r = lane + 32 * t;
          if (r < p.R) dkb[t] += g * to_f32(qb[r]);
        }
      }
    }
  }
  T* dkrow = reinterpret_cast<T*>(p.dk) + b * p.dk_stride[0] + h * p.dk_stride[1] + (int64_t)j * p.dk_stride[2];
  T* dvrow = reinterpret_cast<T*>(p.dv) + b * p.dv_stride[0] + h * p.dv_stride[1] + (int64_t)j * p.dv_stride[2];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int d = lane + 32 * t;
    if (d < p.D) {
      dkrow[d] = from_f32<T>(dk[t] * p.softmax_scale);
      dvrow[d] = from_f32<T>(dv[t]);
    }
  }
  if (p.R > 0) {
    const FactorAcc fa = factor_acc(p);
    const int bb = fa.Bk == 1 ? 0 : b, hh = fa.Hk == 1 ? 0 : h;
    float* dst = fa.dkb + (((int64_t)bb * p.Sk + j) * fa.Hk + hh) * p.R;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int r = lane + 32 * t;
      if (r < p.R) atomicAdd(dst + r, dkb[t]);
    }
  }
}

// fp32 accumulator -> 16-bit gradient tensor with the factor's own strides.  The accumulator is addressed
// (b, h, s, r) through element strides (ab, ah, as, ar): (Bx, S, Hx, R), or -- `tiled` -- head-major in tiles of
// 128 rows stored rank-major, [r][row in tile] (the tensor-core backward stages its tiles that way: consecutive
// rows are consecutive floats, which keeps the threads' shared-memory stores free of bank conflicts); `slots`
// copies at distance `slot_stride` are summed.
template <typename T>
struct FactorStoreJob {
  const float* acc;
  int64_t ab, ah, as;
  int tiled, slots;
  int64_t slot_stride;
  T* out;
  int Bx, S, Hx;
  int64_t sb, sh, ss;
};

// One launch for both factors: blocks [0, nbq) store dq_bias, the rest dk_bias.
template <typename T>
__global__ void __launch_bounds__(256) factor_grad_store_kernel(FactorStoreJob<T> jq, FactorStoreJob<T> jk, unsigned nbq,
                                                                int R) {
  const bool is_q = blockIdx.x < nbq;
  const FactorStoreJob<T>& j = is_q ? jq : jk;
  const int64_t idx = (int64_t)(is_q ? blockIdx.x : blockIdx.x - nbq) * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)j.Bx * j.S * j.Hx * R;
  if (idx >= total) return;
  const int r = (int)(idx % R);
  const int h = (int)((idx / R) % j.Hx);
  const int s = (int)((idx / ((int64_t)R * j.Hx)) % j.S);
  const int b = (int)(idx / ((int64_t)R * j.Hx * j.S));
  const float* src = j.tiled ? j.acc + b * j.ab + h * j.ah + (int64_t)(s / 128) * (128 * R) + r * 128 + (s % 128)
                             : j.acc + b * j.ab + h * j.ah + s * j.as + r;
  float v = 0.f;
  for (int e = 0; e < j.slots; ++e) v += src[e * j.slot_stride];
  j.out[b * j.sb + h * j.sh + s * j.ss + r] = from_f32<T>(v);
}

size_t bwd_general_workspace(const fb_params* p) {
  if (p->R <= 0) return 0;
  const FactorAcc fa = factor_acc(*p);
  const size_t nq = (((size_t)fa.Bq * p->Sq * fa.Hq * p->R) + 63) & ~size_t(63);
  const size_t nk = (((size_t)fa.Bk * p->Sk * fa.Hk * p->R) + 63) & ~size_t(63);
  return round256((nq + nk) * sizeof(float));
}

template <typename T>
static FactorStoreJob<T> factor_store_job(const float* acc, FactorAccLayout l, T* out, int Bx, int S, int Hx, int R,
                                          const int64_t* stride) {
  if (l.rows > 0)  // (slots, Bx, Hx, rows, R)
    return {acc, Hx * l.rows * R, l.rows * R, R, 1, l.slots, l.slot_stride, out, Bx, S, Hx, stride[0], stride[1], stride[2]};
  // (Bx, S, Hx, R)
  return {acc, (int64_t)S * Hx * R, R, (int64_t)Hx * R, 0, 1, 0, out, Bx, S, Hx, stride[0], stride[1], stride[2]};
}

template <typename T>
static int launch_store_factor_grads(const fb_params* p, float* dqb, float* dkb, cudaStream_t st,
                                     FactorAccLayout ql, FactorAccLayout kl) {
  const FactorAcc fa = factor_acc(*p);
  const FactorStoreJob<T> jq = factor_store_job<T>(dqb, ql, reinterpret_cast<T*>(p->dq_bias), fa.Bq, p->Sq, fa.Hq, p->R,
                                                   p->dq_bias_stride);
  const FactorStoreJob<T> jk = factor_store_job<T>(dkb, kl, reinterpret_cast<T*>(p->dk_bias), fa.Bk, p->Sk, fa.Hk, p->R,
                                                   p->dk_bias_stride);
  const unsigned nbq = (unsigned)(((int64_t)fa.Bq * p->Sq * fa.Hq * p->R + 255) / 256);
  const unsigned nbk = (unsigned)(((int64_t)fa.Bk * p->Sk * fa.Hk * p->R + 255) / 256);
  factor_grad_store_kernel<T><<<nbq + nbk, 256, 0, st>>>(jq, jk, nbq, p->R);
  note_launch();
  return (int)cudaGetLastError();
}

// Round the fp32 factor-gradient accumulators into dq_bias / dk_bias.
int store_factor_grads_from(const fb_params* p, float* dqb, float* dkb, cudaStream_t st, FactorAccLayout q_layout,
                            FactorAccLayout k_layout) {
  return p->dtype == FB_DTYPE_F16 ? launch_store_factor_grads<__half>(p, dqb, dkb, st, q_layout, k_layout)
                                  : launch_store_factor_grads<__nv_bfloat16>(p, dqb, dkb, st, q_layout, k_layout);
}

int launch_fwd_general(const fb_params* p, cudaStream_t st) {
  const int64_t rows = (int64_t)p->B * p->H * p->Sq;
  const unsigned blocks = (unsigned)((rows + kWarps - 1) / kWarps);
  prof_before(KC_FWD_MAIN, st);
  if (p->dtype == FB_DTYPE_F16)
    fwd_general_kernel<__half><<<blocks, kWarps * 32, 0, st>>>(*p);
  else
    fwd_general_kernel<__nv_bfloat16><<<blocks, kWarps * 32, 0, st>>>(*p);
  prof_after(KC_FWD_MAIN, st);
  note_launch();
  return (int)cudaGetLastError();
}

int launch_bwd_preprocess(const fb_params* p, cudaStream_t st) {
  const int64_t rows = (int64_t)p->B * p->H * p->Sq;
  const unsigned blocks = (unsigned)((rows + 255) / 256);
  prof_before(KC_BWD_PREPROCESS, st);
  if (p->dtype == FB_DTYPE_F16)
    bwd_preprocess_kernel<__half><<<blocks, 256, 0, st>>>(*p);
  else
    bwd_preprocess_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(*p);
  prof_after(KC_BWD_PREPROCESS, st);
  note_launch();
  return (int)cudaGetLastError();
}

int launch_bwd_general(const fb_params* p, cudaStream_t st) {
  if (p->R > 0) {
    cudaError_t e = cudaMemsetAsync(p->workspace, 0, bwd_general_workspace(p), st);
    if (e != cudaSuccess) return (int)e;
  }
  const unsigned bq = (unsigned)(((int64_t)p->B * p->H * p->Sq + kWarps - 1) / kWarps);
  const unsigned bk = (unsigned)(((int64_t)p->B * p->H * p->Sk + kWarps - 1) / kWarps);
  prof_before(KC_BWD_MAIN, st);
  if (p->dtype == FB_DTYPE_F16) {
    bwd_dq_general_kernel<__half><<<bq, kWarps * 32, 0, st>>>(*p);
    bwd_dkv_general_kernel<__half><<<bk, kWarps * 32, 0, st>>>(*p);
  } else {
    bwd_dq_general_kernel<__nv_bfloat16><<<bq, kWarps * 32, 0, st>>>(*p);
    bwd_dkv_general_kernel<__nv_bfloat16><<<bk, kWarps * 32, 0, st>>>(*p);
  }
  prof_after(KC_BWD_MAIN, st);
  note_launch(2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  if (p->R <= 0) return 0;
  const FactorAcc fa = factor_acc(*p);
  return store_factor_grads_from(p, fa.dqb, fa.dkb, st);
}

}  // namespace fb
