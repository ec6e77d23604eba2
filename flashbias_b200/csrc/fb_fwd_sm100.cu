// Forward FlashBias attention for sm_100a: TMA-staged operand tiles, tcgen05 MMAs accumulating in
// tensor memory, warp-specialised roles.
//
// One CTA owns one tile of 128 query rows of one (batch, head) and walks the key/value tiles:
//   warp 4      TMA producer: barrier set-up and the first loads before the CTA-wide sync; Q (or the (hi, lo)
//               split of q*scale) | packed q_bias once, then K|packed k_bias and V tiles through rings of up
//               to four shared-memory stages.
//   warp 5      MMA issuer (one thread): S = [Q|Qb].[K|Kb]^T into TMEM, bias products first.
//   warp 6      MMA issuer (one thread, another warp scheduler): O += P.V with P read from TMEM.
//   warps 0-3   softmax: one thread per query row (= one TMEM lane).  Pass 1 reads S and takes the
//               row maximum; pass 2 reads S again, exponentiates, accumulates the row sum and writes P
//               (16-bit pairs) to TMEM.  S is released as soon as its last chunk is in registers, so the
//               next key tile's logits are computed under the remaining exponentials.  O is rescaled in
//               TMEM only when the running maximum has grown by more than 2^8 ("lazy rescale"), which is
//               exact because the row sum carries the same reference maximum.
// All logit terms share one accumulator: S' = qs.k + qb.k_bias, with qs = q and qb = q_bias/scale when the
// scale is a power of two (p = exp2((S' - m) * scale * log2 e)), else qs = (hi, lo) of q*scale and qb = q_bias.
// Two CTAs share an SM (256 TMEM columns each) so one CTA's softmax overlaps the other's MMAs.
#include <type_traits>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

struct FwdArgs {
  int B, H, Sq, Sk, nq_tiles, causal;
  int hq_bcast, bq_bcast, hk_bcast, bk_bcast;  // 1 = the packed factor has extent 1 on that dim
  float scale, scale_log2;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride_bh;
  int* status;
};

template <int D, int RP, int NQ>
struct FwdCfg {
  // (K stages, V stages, CTAs per SM) chosen so that the tiles fit the shared memory of the SM
  static constexpr int MINB = (D == 128) ? 1 : 2;
  // as many K|Kb and V stages (up to 4) as fit beside Q in the shared memory of one of MINB co-resident CTAs:
  // the TMA producer runs that many key tiles ahead, which is what hides the L2/HBM latency of the loads
  static constexpr int BUDGET = (MINB == 2 ? 110 : 220) * 1024 - 2048;
  static constexpr int PER_STAGE = 2 * tile_bytes(D) + (RP ? tile_bytes(RP ? RP : 16) : 0);
  static constexpr int FIT = (BUDGET - NQ * tile_bytes(D) - (RP ? tile_bytes(RP ? RP : 16) : 0)) / PER_STAGE;
  static constexpr int KST = FIT >= 4 ? 4 : (FIT >= 2 ? FIT : 2);
  static constexpr int VST = KST;
  static constexpr int Q_BYTES = tile_bytes(D);
  static constexpr int QB_BYTES = RP ? tile_bytes(RP ? RP : 16) : 0;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_QB = OFF_Q + NQ * Q_BYTES;  // NQ query terms (q, or hi and lo of q*scale), then Qb
  static constexpr int OFF_K = OFF_QB + QB_BYTES;
  static constexpr int OFF_KB = OFF_K + KST * Q_BYTES;
  static constexpr int OFF_V = OFF_KB + KST * QB_BYTES;
  static constexpr int OFF_BAR = OFF_V + VST * Q_BYTES;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;  // barriers + alignment slack
  // tensor memory: S fp32 [0,128), P 16-bit pairs [128,192), O fp32 [192, 192+D)
  static constexpr int T_S = 0, T_P = 128, T_O = 192;
  static constexpr int TMEM_COLS = (T_O + D <= 256) ? 256 : 512;
};

template <int C>
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int row0, int h, int b,
                                            int col0 = 0) {
  constexpr int SWB = swizzle_bytes(C);
  constexpr int NB = C * 2 / SWB;
#pragma unroll
  for (int blk = 0; blk < NB; ++blk) tma_load_4d(dst + blk * 128 * SWB, m, bar, col0 + blk * (SWB / 2), row0, h, b);
}

// Development aid, compiled only with -DFB_TRACE: CTA 0 records clock64() at phase boundaries, 16 slots per key tile.
#ifdef FB_TRACE
__device__ long long g_fwd_trace[64 * 16];
#define FB_TRACE_MARK(j, slot) \
  do { if (blockIdx.x == 0 && (j) < 64) g_fwd_trace[(j) * 16 + (slot)] = clock64(); } while (0)
#else
#define FB_TRACE_MARK(j, slot) do { } while (0)
#endif

template <typename T, int D, int RP, int NQ>
__global__ void __launch_bounds__(224, FwdCfg<D, RP, NQ>::MINB)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQb,
                 const __grid_constant__ CUtensorMap tmKb, const FwdArgs a) {
  using Cfg = FwdCfg<D, RP, NQ>;
  constexpr int KST = Cfg::KST, VST = Cfg::VST;
  constexpr int RPX = RP ? RP : 16;  // keeps templates well-formed when there is no bias
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Cfg::OFF_Q, sQb = sbase + Cfg::OFF_QB, sK = sbase + Cfg::OFF_K,
                 sKb = sbase + Cfg::OFF_KB, sV = sbase + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  // barrier slots
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0, s_full = bar0 + 8, p_ready = bar0 + 16, pv_done = bar0 + 24, s_read = bar0 + 176;
  const uint32_t k_full = bar0 + 32, k_free = bar0 + 64, v_full = bar0 + 96, v_free = bar0 + 128;  // 4 slots each
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 160);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 168);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = a.B * a.H;
  int qt, bh;
  if (a.causal) {  // heaviest (last) query tiles first
    qt = a.nq_tiles - 1 - (int)(blockIdx.x / BH);
    bh = (int)(blockIdx.x % BH);
  } else {
    qt = (int)(blockIdx.x % a.nq_tiles);
    bh = (int)(blockIdx.x / a.nq_tiles);
  }
  const int b = bh / a.H, h = bh % a.H;
  const int q0 = qt * 128;
  const int kv_end = a.causal ? min(a.Sk, q0 + 128) : a.Sk;
  const int n_kv = (kv_end + 127) / 128;

  // producer thread only: the K|Kb and V tiles of key tile j
  const int hk = a.hk_bcast ? 0 : h, bk = a.bk_bcast ? 0 : b;
  auto load_kv = [&](int j) {
    const int ks = j % KST, vs = j % VST;
    mbar_expect_tx(k_full + 8 * ks, Cfg::Q_BYTES + Cfg::QB_BYTES);
    tma_tile_4d<D>(sK + ks * Cfg::Q_BYTES, &tmK, k_full + 8 * ks, j * 128, h, b);
    if (RP) tma_tile_4d<RPX>(sKb + ks * Cfg::QB_BYTES, &tmKb, k_full + 8 * ks, j * 128, hk, bk);
    mbar_expect_tx(v_full + 8 * vs, Cfg::Q_BYTES);
    tma_tile_4d<D>(sV + vs * Cfg::Q_BYTES, &tmV, v_full + 8 * vs, j * 128, h, b);
  };
  if (warp == 4) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(q_full, 1);
      mbar_init(s_full, 1);
      mbar_init(p_ready, 4);  // one arrival per softmax warp
      mbar_init(s_read, 4);   // likewise: the logits of the tile are in registers
      mbar_init(pv_done, 1);
      for (int i = 0; i < 4; ++i) {
        mbar_init(k_full + 8 * i, 1);
        mbar_init(k_free + 8 * i, 1);
        mbar_init(v_full + 8 * i, 1);
        mbar_init(v_free + 8 * i, 1);
      }
      mbar_fence_init();
      // the first loads start before the rest of the CTA has finished its set-up
      const int hq = a.hq_bcast ? 0 : h, bq = a.bq_bcast ? 0 : b;
      mbar_expect_tx(q_full, NQ * Cfg::Q_BYTES + Cfg::QB_BYTES);
#pragma unroll
      for (int t = 0; t < NQ; ++t) tma_tile_4d<D>(sQ + t * Cfg::Q_BYTES, &tmQ, q_full, q0, h, b, t * D);
      if (RP) tma_tile_4d<RPX>(sQb, &tmQb, q_full, q0, hq, bq);
      for (int j = 0; j < KST && j < n_kv; ++j) load_kv(j);
    }
  } else if (warp == 5) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem + Cfg::T_S, tP = tmem + Cfg::T_P, tO = tmem + Cfg::T_O;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = KST; j < n_kv; ++j) {
        mbar_wait(k_free + 8 * (j % KST), ((j / KST) - 1) & 1, abort_flag, a.status);
        mbar_wait(v_free + 8 * (j % VST), ((j / VST) - 1) & 1, abort_flag, a.status);
        load_kv(j);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer: S = [Q|Qb].[K|Kb]^T
    if (lane == 0) {
      constexpr uint32_t idS = instr_desc(kBf16, false, false, 128, 128);
      // descriptor views built once; each MMA only adds a constant to the start-address field
      const DescBase dQ = kmajor_base<D>(sQ), dQb = kmajor_base<RPX>(sQb), dK = kmajor_base<D>(sK),
                     dKb = kmajor_base<RPX>(sKb);
      auto issue_S = [&](int j) {
        const int ks = j % KST;
        mbar_wait(k_full + 8 * ks, (j / KST) & 1, abort_flag, a.status);
        tc_fence_after_sync();
        const uint32_t ko = ks * Cfg::Q_BYTES, kbo = ks * Cfg::QB_BYTES;
        // The bias products go first, into the empty accumulator: factor terms as large as a sequence
        // position then only meet each other (and cancel exactly), instead of forcing the small q.k sum to be
        // aligned to their magnitude inside the tensor core's adder.
        if (RP) {
#pragma unroll
          for (int s = 0; s < RPX / 16; ++s)
            umma_ss(tS, desc_at(dQb, kmajor_step<RPX>(s)), desc_at(dKb, kbo + kmajor_step<RPX>(s)), idS, s > 0);
        }
#pragma unroll
        for (int t = 0; t < NQ; ++t) {  // query terms share the K tile
#pragma unroll
          for (int s = 0; s < D / 16; ++s)
            umma_ss(tS, desc_at(dQ, t * Cfg::Q_BYTES + kmajor_step<D>(s)), desc_at(dK, ko + kmajor_step<D>(s)), idS,
                    (RP || t > 0 || s > 0) ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(k_free + 8 * ks);
      };
      mbar_wait(q_full, 0, abort_flag, a.status);
      for (int j = 0; j < n_kv; ++j) {
        if (j > 0) {  // the softmax warps hold the logits of the previous key tile in registers
          mbar_wait(s_read, (j - 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
        }
        FB_TRACE_MARK(j, 8);
        issue_S(j);
        FB_TRACE_MARK(j, 9);
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ MMA issuer: O += P.V
    // A second issuing thread on another warp scheduler: S of the next key tile and P.V of this one are
    // issued concurrently (an issuing thread only gets a slot when the softmax warps of its scheduler stall).
    if (lane == 0) {
      constexpr uint32_t idO = instr_desc(kBf16, false, true, 128, D);
      const DescBase dV = mnmajor_base<D>(sV);
      for (int j = 0; j < n_kv; ++j) {
        const int vs = j % VST;
        mbar_wait(v_full + 8 * vs, (j / VST) & 1, abort_flag, a.status);
        mbar_wait(p_ready, j & 1, abort_flag, a.status);
        tc_fence_after_sync();
        FB_TRACE_MARK(j, 10);
        const uint32_t vo = vs * Cfg::Q_BYTES;
#pragma unroll
        for (int s = 0; s < 8; ++s)
          umma_ts(tO, tP + s * 8, desc_at(dV, vo + mnmajor_step<D>(s)), idO, (j > 0 || s > 0) ? 1u : 0u);
        umma_commit(pv_done);
        umma_commit(v_free + 8 * vs);
        FB_TRACE_MARK(j, 11);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int row = warp * 32 + lane;
    const int grow = q0 + row;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const float sl2 = a.scale_log2;
    float m_used = -INFINITY, l = 0.f;
    uint32_t ra[32], rb[32];  // two register buffers: the TMEM load of one chunk overlaps the math of the other
    for (int j = 0; j < n_kv; ++j) {
      const int k0 = j * 128;
      if (threadIdx.x == 0) FB_TRACE_MARK(j, 0);
      mbar_wait(s_full, j & 1, abort_flag, a.status);
      tc_fence_after_sync();
      if (threadIdx.x == 0) FB_TRACE_MARK(j, 1);
      const bool need_mask = (a.causal && k0 + 127 > q0) || (k0 + 128 > a.Sk);
      const uint32_t tSl = tS + lane_off;
      // ---- pass 1: row maximum (four independent chains)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto chunk_max = [&](const uint32_t (&r)[32], int c) {
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0 + c * 32 + i;
            const bool dead = col >= a.Sk || (a.causal && col > grow);
            mx4[i & 3] = fmaxf(mx4[i & 3], dead ? -INFINITY : __uint_as_float(r[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(r[i]));
        }
      };
      tmem_ld32(tSl, ra);
      tmem_wait_ld(ra);
      tmem_ld32(tSl + 32, rb);
      chunk_max(ra, 0);
      tmem_wait_ld(rb);
      tmem_ld32(tSl + 64, ra);
      chunk_max(rb, 1);
      tmem_wait_ld(ra);
      tmem_ld32(tSl + 96, rb);
      chunk_max(ra, 2);
      tmem_wait_ld(rb);
      tmem_ld32(tSl, ra);  // first chunk of pass 2
      chunk_max(rb, 3);
      const float m_new = fmaxf(m_used, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
      if (threadIdx.x == 0) FB_TRACE_MARK(j, 2);
      if (j > 0) {
        mbar_wait(pv_done, (j - 1) & 1, abort_flag, a.status);  // P buffer free, O stable
        tc_fence_after_sync();
        if (threadIdx.x == 0) FB_TRACE_MARK(j, 3);
        const bool grow_needed = (m_new - m_used) * sl2 > 8.f;
        if (__any_sync(0xffffffffu, grow_needed)) {
          const float alpha = m_new == -INFINITY ? 1.f : fast_exp2((m_used - m_new) * sl2);
          l *= alpha;
          m_used = m_new;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            tmem_ld32(tO + lane_off + c * 32, rb);
            tmem_wait_ld(rb);
#pragma unroll
            for (int i = 0; i < 32; ++i) rb[i] = __float_as_uint(__uint_as_float(rb[i]) * alpha);
            tmem_st32(tO + lane_off + c * 32, rb);
          }
          tmem_wait_st();
        }
      } else {
        m_used = m_new;
      }
      // ---- pass 2: p = exp2(s*sl2 - m*sl2), row sum, P -> shared memory
      const float msc = m_used == -INFINITY ? 0.f : m_used * sl2;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      auto chunk_exp = [&](uint32_t (&r)[32], int c) {
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = k0 + c * 32 + i;
            const bool dead = col >= a.Sk || (a.causal && col > grow);
            const float p = dead ? 0.f : fast_exp2(fmaf(__uint_as_float(r[i]), sl2, -msc));
            l4[i & 3] += p;
            r[i] = __float_as_uint(p);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p = fast_exp2(fmaf(__uint_as_float(r[i]), sl2, -msc));
            l4[i & 3] += p;
            r[i] = __float_as_uint(p);
          }
        }
        // P goes back to tensor memory as the A operand of O += P.V: 32 keys = 16 packed words
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = Pack2<T>::pack(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        tmem_st16(tP + lane_off + c * 16, w);
      };
      tmem_wait_ld(ra);
      tmem_ld32(tSl + 32, rb);
      chunk_exp(ra, 0);
      tmem_wait_ld(rb);
      tmem_ld32(tSl + 64, ra);
      chunk_exp(rb, 1);
      tmem_wait_ld(ra);
      tmem_ld32(tSl + 96, rb);
      // the last chunk is awaited before the arithmetic of the third: S is then entirely in registers and the
      // tensor core starts on the next key tile half a pass earlier
      tmem_wait_ld(rb);
      tc_fence_before_sync();
      if (threadIdx.x == 0) FB_TRACE_MARK(j, 4);
      mbar_arrive_warp(s_read);
      chunk_exp(ra, 2);
      chunk_exp(rb, 3);
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tmem_wait_st();
      tc_fence_before_sync();
      if (threadIdx.x == 0) FB_TRACE_MARK(j, 5);
      mbar_arrive_warp(p_ready);
    }
    // ---- epilogue: O / l -> global, lse
    mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, a.status);
    tc_fence_after_sync();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* orow = reinterpret_cast<T*>(a.o) + b * a.o_stride[0] + h * a.o_stride[1] + (int64_t)grow * a.o_stride[2];
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + lane_off + c * 32, r);
      tmem_wait_ld(r);
      if (grow < a.Sq) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = Pack2<T>::pack(__uint_as_float(r[g * 8 + 0]) * inv, __uint_as_float(r[g * 8 + 1]) * inv);
          w.y = Pack2<T>::pack(__uint_as_float(r[g * 8 + 2]) * inv, __uint_as_float(r[g * 8 + 3]) * inv);
          w.z = Pack2<T>::pack(__uint_as_float(r[g * 8 + 4]) * inv, __uint_as_float(r[g * 8 + 5]) * inv);
          w.w = Pack2<T>::pack(__uint_as_float(r[g * 8 + 6]) * inv, __uint_as_float(r[g * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = w;
        }
      }
    }
    if (grow < a.Sq) {
      a.lse[(int64_t)bh * a.lse_stride_bh + grow] = l > 0.f ? m_used * a.scale + logf(l) : -INFINITY;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tmem_dealloc(tmem, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
#ifdef FB_TRACE
}  // namespace fb
extern "C" int fb_debug_trace_fwd(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, fb::g_fwd_trace, sizeof(long long) * (n < 1024 ? n : 1024));
}
namespace fb {
#endif
static bool o_store_ok(const fb_params* p) {
  if (reinterpret_cast<uintptr_t>(p->o) & 15) return false;
  for (int i = 0; i < 3; ++i)
    if (p->o_stride[i] & 7) return false;
  return true;
}

bool fwd_sm100_supported(const fb_params* p, PackPlan* plan) {
  if (p->flags & FB_FLAG_FORCE_GENERAL) return false;
  if (p->mask_kind != FB_MASK_NONE) return false;
  if (!(p->D == 32 || p->D == 64 || p->D == 128)) return false;
  if (!(p->softmax_scale > 0.f) || !isfinite(p->softmax_scale)) return false;
  if (!tma_compatible(p->q, p->q_stride[2], p->q_stride[1], p->q_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->k, p->k_stride[2], p->k_stride[1], p->k_stride[0], p->H, p->B)) return false;
  if (!tma_compatible(p->v, p->v_stride[2], p->v_stride[1], p->v_stride[0], p->H, p->B)) return false;
  if (!o_store_ok(p)) return false;
  if ((int64_t)p->B * p->H * ((p->Sq + 127) / 128) > 0x7fffffffLL) return false;
  return plan_pack(p, plan);
}

template <typename T, int D, int RP, int NQ>
static int launch_fwd_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  using Cfg = FwdCfg<D, RP, NQ>;
  int rc;
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  void* qpack = ws;
  void* kpack = ws + plan.q_bytes;
  void* qs = ws + plan.q_bytes + plan.k_bytes;
  if ((rc = launch_pack_operands(p, plan, qpack, kpack, nullptr, false, qs, st))) return rc;
  CUtensorMap tQ, tK, tV, tQb, tKb;
  constexpr int BOXD = D > 64 ? 64 : D;
  if (NQ == 2) {
    // query operand = (hi, lo) of q*scale, laid out (B, H, Sq, 2D) in the workspace
    if ((rc = make_tmap_4d(&tQ, qs, 2 * D, p->Sq, p->H, p->B, 2 * D, (int64_t)2 * D * p->Sq,
                           (int64_t)2 * D * p->Sq * p->H, BOXD, 128)))
      return rc;
  } else if ((rc = make_tmap_4d(&tQ, p->q, D, p->Sq, p->H, p->B, p->q_stride[2], p->q_stride[1], p->q_stride[0], BOXD,
                                128))) {
    return rc;
  }
  if ((rc = make_tmap_4d(&tK, p->k, D, p->Sk, p->H, p->B, p->k_stride[2], p->k_stride[1], p->k_stride[0], BOXD, 128)))
    return rc;
  if ((rc = make_tmap_4d(&tV, p->v, D, p->Sk, p->H, p->B, p->v_stride[2], p->v_stride[1], p->v_stride[0], BOXD, 128)))
    return rc;
  if (RP) {
    if ((rc = make_tmap_4d(&tQb, qpack, RP, p->Sq, plan.Hq, plan.Bq, RP, (int64_t)RP * p->Sq,
                           (int64_t)RP * p->Sq * plan.Hq, RP, 128)))
      return rc;
    if ((rc = make_tmap_4d(&tKb, kpack, RP, p->Sk, plan.Hk, plan.Bk, RP, (int64_t)RP * p->Sk,
                           (int64_t)RP * p->Sk * plan.Hk, RP, 128)))
      return rc;
  } else {
    tQb = tQ;
    tKb = tK;
  }
  FwdArgs a;
  a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
  a.nq_tiles = (p->Sq + 127) / 128;
  a.causal = p->causal;
  a.hq_bcast = plan.Hq == 1; a.bq_bcast = plan.Bq == 1; a.hk_bcast = plan.Hk == 1; a.bk_bcast = plan.Bk == 1;
  // logits = a.scale * S: the scale is already inside the query operand when it is split
  a.scale = NQ == 2 ? 1.f : p->softmax_scale;
  a.scale_log2 = a.scale * 1.4426950408889634f;
  a.o = p->o;
  for (int i = 0; i < 3; ++i) a.o_stride[i] = p->o_stride[i];
  a.lse = p->lse;
  a.lse_stride_bh = p->lse_stride_bh;
  a.status = p->status;
  auto kern = fwd_sm100_kernel<T, D, RP, NQ>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_done[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_done[dev & 63] = true;
  }
  const unsigned grid = (unsigned)((int64_t)a.nq_tiles * p->B * p->H);
  prof_before(KC_FWD_MAIN, st);
  kern<<<grid, 224, Cfg::SMEM, st>>>(tQ, tK, tV, tQb, tKb, a);
  prof_after(KC_FWD_MAIN, st);
  note_launch();
  return (int)cudaGetLastError();
}

template <typename T>
static int dispatch_fwd(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
#define FB_CASE(DD, RR)                                                              \
  if (p->D == DD && plan.RP == RR)                                                   \
    return plan.nq == 2 ? launch_fwd_t<T, DD, RR, 2>(p, plan, st) : launch_fwd_t<T, DD, RR, 1>(p, plan, st);
  FB_CASE(32, 0) FB_CASE(32, 16) FB_CASE(32, 32) FB_CASE(32, 64)
  FB_CASE(64, 0) FB_CASE(64, 16) FB_CASE(64, 32) FB_CASE(64, 64)
  FB_CASE(128, 0) FB_CASE(128, 16) FB_CASE(128, 32) FB_CASE(128, 64)
#undef FB_CASE
  return FB_ENOTBUILT;
}

int launch_fwd_sm100(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  return p->dtype == FB_DTYPE_F16 ? dispatch_fwd<__half>(p, plan, st) : dispatch_fwd<__nv_bfloat16>(p, plan, st);
}

}  // namespace fb
