// Forward FlashBias attention for sm_100a: TMA-staged operand tiles, tcgen05 MMAs accumulating in
// tensor memory, warp-specialised roles.  (Kernel and launcher templates; the instantiations are spread
// over several translation units so that they compile in parallel.)
//
// The kernel is persistent: the grid is one CTA per resident slot of the GPU, and a CTA walks work items (a tile of
// 128 query rows of one (batch, head)) with a stride of the grid size, heaviest first under causal masking.  The
// operand rings, the barrier phases and the tensor-memory allocation carry over from item to item, so the loads of
// the next item (Q as soon as this item's last logit product has completed, K/V as ring slots free) run under the
// softmax and the P.V products of this one, and the per-CTA set-up is paid once per SM slot instead of once per
// query tile -- which is what a short sequence (Swin windows: two key tiles per item) needs.
// For one item the CTA walks the key/value tiles:
//   warp 4      TMA producer: Q (or the (hi, lo) split of q*scale) | packed q_bias once per item, then K|packed k_bias
//               and V tiles through rings of shared-memory stages.
//   warp 5      MMA issuer (one thread): S = [Q|Qb].[K|Kb]^T into TMEM, bias products first.
//   warp 6      MMA issuer (one thread, another warp scheduler): O += P.V with P read from TMEM.
//   warp 7      idle (completes the second warpgroup, which hands most of its registers to the first).
//   warps 0-3   softmax: one thread per query row (= one TMEM lane).  The thread takes all 128 logits of
//               its row into registers with one round of TMEM loads and releases S at once, so the tensor
//               core computes the next key tile's logits under this tile's exponentials.  Row maximum,
//               exponentials, row sum and the 16-bit P (written back to TMEM as the A operand of P.V) are
//               all computed from those registers: S is read from tensor memory exactly once.
//               O is rescaled in TMEM only when the running maximum has grown by more than 2^8 ("lazy
//               rescale"), which is exact because the row sum carries the same reference maximum.
// All logit terms share one accumulator: S' = qs.k + qb.k_bias, with qs = q and qb = q_bias/scale when the
// scale is a power of two (p = exp2((S' - m) * scale * log2 e)), else qs = (hi, lo) of q*scale and qb = q_bias.
// An additive mask tensor is added in registers (row-contiguous loads, one mask row per thread); the fused
// ALiBi producer adds slope * (col - row) with one FMA per logit and needs no factor operands at all.
// Two CTAs share an SM when their tiles fit (256 TMEM columns each) so one CTA's softmax overlaps the
// other's MMAs and loads.
#pragma once

#include <mutex>
#include <type_traits>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

struct FwdArgs {
  int B, H, Sq, Sk, nq_tiles, causal;
  int total_items;  // query tiles x batch x heads: the CTAs walk them with a stride of the grid size
  int hq_bcast, bq_bcast, hk_bcast, bk_bcast;  // 1 = the packed factor has extent 1 on that dim
  float scale, scale_log2;
  void* o;
  int64_t o_stride[3];
  float* lse;
  int64_t lse_stride_bh;
  int* status;
  const void* mask;  // additive mask, (batch, head, row) element strides; row stride 0 for a (1, Sk) mask
  int64_t mask_stride[3];
  int mask_kind, mask_dtype, mask_batch_period;
  const float* alibi_slopes;
};

template <int D, int RP, int NQ>
struct FwdCfg {
  static constexpr int RPX = RP ? RP : 16;  // keeps templates well-formed when there is no bias
  static constexpr int Q_BYTES = tile_bytes(D);
  static constexpr int QB_BYTES = RP ? tile_bytes(RPX) : 0;
  static constexpr int TAIL = 256 + 1024;  // barriers + alignment slack
  static constexpr int K_STAGE = Q_BYTES + QB_BYTES, V_STAGE = Q_BYTES;
  static constexpr int smem_for(int kst, int vst) {
    return NQ * Q_BYTES + QB_BYTES + kst * K_STAGE + vst * V_STAGE + TAIL;
  }
  // tensor memory: S fp32 [0,128), P 16-bit pairs [128,192), O fp32 [192, 192+D)
  static constexpr int T_S = 0, T_P = 128, T_O = 192;
  static constexpr int TMEM_COLS = (T_O + D <= 256) ? 256 : 512;
  // Two CTAs per SM (each CTA reserves 1 KB of the 228 KB) when two stages of each ring fit; else one.
  static constexpr int LIM2 = 113 * 1024, LIM1 = 227 * 1024;
  static constexpr bool TWO = TMEM_COLS == 256 && smem_for(2, 2) <= LIM2;
  static constexpr int LIM = TWO ? LIM2 : LIM1;
  static constexpr int MINB = TWO ? 2 : 1;
  // as many K|Kb and V stages (up to 4) as fit: the TMA producer runs that many key tiles ahead, which is
  // what hides the L2/HBM latency of the loads
  static constexpr int KST = smem_for(4, 4) <= LIM ? 4 : smem_for(3, 3) <= LIM ? 3 : smem_for(2, 2) <= LIM ? 2
                             : smem_for(2, 1) <= LIM ? 2 : 1;
  static constexpr int VST = smem_for(KST, KST) <= LIM ? KST : 1;
  static constexpr int SMEM = smem_for(KST, VST);
  static constexpr bool FITS = SMEM <= LIM;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_QB = OFF_Q + NQ * Q_BYTES;  // NQ query terms (q, or hi and lo of q*scale), then Qb
  static constexpr int OFF_K = OFF_QB + QB_BYTES;
  static constexpr int OFF_KB = OFF_K + KST * Q_BYTES;
  static constexpr int OFF_V = OFF_KB + KST * QB_BYTES;
  static constexpr int OFF_BAR = OFF_V + VST * Q_BYTES;
};

template <int C>
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int row0, int h, int b,
                                            int col0 = 0) {
  constexpr int SWB = swizzle_bytes(C);
  constexpr int NB = C * 2 / SWB;
#pragma unroll
  for (int blk = 0; blk < NB; ++blk) tma_load_4d(dst + blk * 128 * SWB, m, bar, col0 + blk * (SWB / 2), row0, h, b);
}

enum { FWD_PLAIN = 0, FWD_MASK = 1, FWD_ALIBI = 2 };

template <typename T, int D, int RP, int NQ, bool ALIBI>
__global__ void __launch_bounds__(256, FwdCfg<D, RP, NQ>::MINB)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQb,
                 const __grid_constant__ CUtensorMap tmKb, const FwdArgs a) {
  using Cfg = FwdCfg<D, RP, NQ>;
  constexpr int KST = Cfg::KST, VST = Cfg::VST;
  constexpr int RPX = Cfg::RPX;
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
  const uint32_t q_free = bar0 + 184;  // every logit product of an item has completed: Q may be overwritten
  struct Item {
    int bh, b, h, q0, n_kv;
  };
  // The w-th work item of this CTA.  Items are ordered heaviest first (causal); the CTAs take them in snake order
  // (0..G-1, then G-1..0, ...), which evens out the sums of a decreasing sequence much better than a plain stride.
  auto item_index = [&](int w) {
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    return w * G + ((w & 1) ? G - 1 - c : c);
  };
  auto item_of = [&](int idx) {
    Item it;
    int qt;
    if (a.causal) {  // heaviest (last) query tiles first
      qt = a.nq_tiles - 1 - idx / BH;
      it.bh = idx % BH;
    } else {
      qt = idx % a.nq_tiles;
      it.bh = idx / a.nq_tiles;
    }
    it.b = it.bh / a.H;
    it.h = it.bh % a.H;
    it.q0 = qt * 128;
    const int kv_end = a.causal ? min(a.Sk, it.q0 + 128) : a.Sk;
    it.n_kv = (kv_end + 127) / 128;
    return it;
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
      mbar_init(q_free, 1);
      mbar_fence_init();
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

  if (warp >= 4) {
    // With two CTAs per SM the kernel is compiled for 128 registers per thread; the producer / issuer
    // warpgroup keeps 48 and the softmax warpgroup, which holds a whole row of logits, takes 208.
    if constexpr (Cfg::MINB == 2) setmaxnreg_dec<48>();
    if (warp == 4) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        int kc = 0, vc = 0, n = 0;  // K and V tiles loaded so far (ring positions), items started
        for (int w = 0, idx; (idx = item_index(w)) < a.total_items; ++w, ++n) {
          const Item it = item_of(idx);
          const int hq = a.hq_bcast ? 0 : it.h, bq = a.bq_bcast ? 0 : it.b;
          const int hk = a.hk_bcast ? 0 : it.h, bk = a.bk_bcast ? 0 : it.b;
          if (n > 0) mbar_wait(q_free, (n - 1) & 1, abort_flag, a.status);
          mbar_expect_tx(q_full, NQ * Cfg::Q_BYTES + Cfg::QB_BYTES);
#pragma unroll
          for (int t = 0; t < NQ; ++t) tma_tile_4d<D>(sQ + t * Cfg::Q_BYTES, &tmQ, q_full, it.q0, it.h, it.b, t * D);
          if (RP) tma_tile_4d<RPX>(sQb, &tmQb, q_full, it.q0, hq, bq);
          for (int j = 0; j < it.n_kv; ++j, ++kc, ++vc) {
            const int ks = kc % KST, vs = vc % VST;
            if (kc >= KST) mbar_wait(k_free + 8 * ks, ((kc / KST) - 1) & 1, abort_flag, a.status);
            mbar_expect_tx(k_full + 8 * ks, Cfg::Q_BYTES + Cfg::QB_BYTES);
            tma_tile_4d<D>(sK + ks * Cfg::Q_BYTES, &tmK, k_full + 8 * ks, j * 128, it.h, it.b);
            if (RP) tma_tile_4d<RPX>(sKb + ks * Cfg::QB_BYTES, &tmKb, k_full + 8 * ks, j * 128, hk, bk);
            if (vc >= VST) mbar_wait(v_free + 8 * vs, ((vc / VST) - 1) & 1, abort_flag, a.status);
            mbar_expect_tx(v_full + 8 * vs, Cfg::Q_BYTES);
            tma_tile_4d<D>(sV + vs * Cfg::Q_BYTES, &tmV, v_full + 8 * vs, j * 128, it.h, it.b);
          }
        }
      }
    } else if (warp == 5) {
      // ------------------------------------------------------------------ MMA issuer: S = [Q|Qb].[K|Kb]^T
      if (lane == 0) {
        constexpr uint32_t idS = instr_desc(kBf16, false, false, 128, 128);
        // descriptor views built once; each MMA only adds a constant to the start-address field
        const DescBase dQ = kmajor_base<D>(sQ), dQb = kmajor_base<RPX>(sQb), dK = kmajor_base<D>(sK),
                       dKb = kmajor_base<RPX>(sKb);
        int t = 0, n = 0;  // key tiles and items issued so far
        for (int w = 0, idx; (idx = item_index(w)) < a.total_items; ++w, ++n) {
          const Item it = item_of(idx);
          mbar_wait(q_full, n & 1, abort_flag, a.status);
          for (int j = 0; j < it.n_kv; ++j, ++t) {
            if (t > 0) {  // the softmax warps hold the logits of the previous key tile in registers
              mbar_wait(s_read, (t - 1) & 1, abort_flag, a.status);
              tc_fence_after_sync();
            }
            const int ks = t % KST;
            mbar_wait(k_full + 8 * ks, (t / KST) & 1, abort_flag, a.status);
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
            for (int q = 0; q < NQ; ++q) {  // query terms share the K tile
#pragma unroll
              for (int s = 0; s < D / 16; ++s)
                umma_ss(tS, desc_at(dQ, q * Cfg::Q_BYTES + kmajor_step<D>(s)), desc_at(dK, ko + kmajor_step<D>(s)),
                        idS, (RP || q > 0 || s > 0) ? 1u : 0u);
            }
            umma_commit(s_full);
            umma_commit(k_free + 8 * ks);
          }
          umma_commit(q_free);  // Q | Qb of this item are no longer read
        }
      }
    } else if (warp == 6) {
      // ------------------------------------------------------------------ MMA issuer: O += P.V
      // A second issuing thread on another warp scheduler: S of the next key tile and P.V of this one are
      // issued concurrently (an issuing thread only gets a slot when the softmax warps of its scheduler stall).
      if (lane == 0) {
        constexpr uint32_t idO = instr_desc(kBf16, false, true, 128, D);
        const DescBase dV = mnmajor_base<D>(sV);
        int t = 0;
        for (int w = 0, idx; (idx = item_index(w)) < a.total_items; ++w) {
          const Item it = item_of(idx);
          for (int j = 0; j < it.n_kv; ++j, ++t) {
            const int vs = t % VST;
            mbar_wait(v_full + 8 * vs, (t / VST) & 1, abort_flag, a.status);
            mbar_wait(p_ready, t & 1, abort_flag, a.status);
            tc_fence_after_sync();
            const uint32_t vo = vs * Cfg::Q_BYTES;
#pragma unroll
            for (int s = 0; s < 8; ++s)
              umma_ts(tO, tP + s * 8, desc_at(dV, vo + mnmajor_step<D>(s)), idO, (j > 0 || s > 0) ? 1u : 0u);
            umma_commit(pv_done);
            umma_commit(v_free + 8 * vs);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    if constexpr (Cfg::MINB == 2) setmaxnreg_inc<208>();
    constexpr float kLog2e = 1.4426950408889634f;
    const int row = warp * 32 + lane;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const float sl2 = a.scale_log2;
    // state of the current work item
    int q0 = 0, grow = 0;
    float m_used = -INFINITY, l = 0.f;  // running reference maximum and row sum, in units of log2 (logit * log2 e)
    float slope2 = 0.f;                 // ALiBi slope of this head, times log2 e
    const char* mrow = nullptr;         // additive mask: this thread's row
    int msize = 4;
    bool mvec = false;
    int t = 0;  // key tiles processed so far by this CTA (barrier phases run across work items)
    uint32_t s[4][32];  // the thread's row of the logit tile

    // One key tile.  MODE: how the logits are completed (plain / + mask tensor / + ALiBi term);
    // DEAD: the tile has columns beyond Sk or above the causal diagonal.
    auto tile = [&](int j, auto mode_c, auto dead_c) {
      constexpr int MODE = decltype(mode_c)::value;
      constexpr bool DEAD = decltype(dead_c)::value;
      const int k0 = j * 128;
      // ---- logits from tensor memory (the load of one 32-column chunk overlaps the arithmetic of the previous
      // one), completed (log2 units for MODE != PLAIN), and the row maximum, four chains
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      const float abase = slope2 * (float)(k0 - grow);
      const uint64_t sl2p = f2(sl2, sl2);
      const uint32_t tSl = tS + lane_off;
      auto complete = [&](int c) {
        float mv[32];
        if (MODE == FWD_MASK) {
          const int n = min(32, a.Sk - (k0 + c * 32));
          const char* p = mrow + (int64_t)(k0 + c * 32) * msize;
          const bool vec = mvec && n == 32;
          if (a.mask_dtype == FB_DTYPE_F32) load_mask_chunk(reinterpret_cast<const float*>(p), n, vec, mv);
          else if (a.mask_dtype == FB_DTYPE_F16) load_mask_chunk(reinterpret_cast<const __half*>(p), n, vec, mv);
          else load_mask_chunk(reinterpret_cast<const __nv_bfloat16*>(p), n, vec, mv);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float v0 = __uint_as_float(s[c][i]), v1 = __uint_as_float(s[c][i + 1]);
          if (MODE == FWD_MASK) f2_unpack(f2_fma(f2(v0, v1), sl2p, f2(mv[i], mv[i + 1])), v0, v1);
          if (MODE == FWD_ALIBI)
            f2_unpack(f2_fma(f2(v0, v1), sl2p,
                             f2(fmaf((float)(c * 32 + i), slope2, abase), fmaf((float)(c * 32 + i + 1), slope2, abase))),
                      v0, v1);
          if (DEAD) {
            const int col = k0 + c * 32 + i;
            if (col >= a.Sk || (a.causal && col > grow)) v0 = -INFINITY;
            if (col + 1 >= a.Sk || (a.causal && col + 1 > grow)) v1 = -INFINITY;
          }
          if (MODE != FWD_PLAIN || DEAD) {
            s[c][i] = __float_as_uint(v0);
            s[c][i + 1] = __float_as_uint(v1);
          }
          mx4[(i >> 1) & 3] = fmax3(mx4[(i >> 1) & 3], v0, v1);
        }
      };
      tmem_ld32(tSl, s[0]);
      tmem_wait_ld(s[0]);
      tmem_ld32(tSl + 32, s[1]);
      complete(0);
      tmem_wait_ld(s[1]);
      tmem_ld32(tSl + 64, s[2]);
      complete(1);
      tmem_wait_ld(s[2]);
      tmem_ld32(tSl + 96, s[3]);
      complete(2);
      tmem_wait_ld(s[3]);
      // S is entirely in registers: the tensor core may start on the next key tile
      tc_fence_before_sync();
      mbar_arrive_warp(s_read);
      complete(3);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      if (MODE == FWD_PLAIN) mx *= sl2;  // sl2 > 0
      const float m_new = fmaxf(m_used, mx);
      if (j > 0) {
        mbar_wait(pv_done, (t - 1) & 1, abort_flag, a.status);  // P buffer free, O stable
        tc_fence_after_sync();
        const bool grow_needed = m_new - m_used > 8.f;
        if (__any_sync(0xffffffffu, grow_needed)) {
          const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_used - m_new);
          l *= alpha;
          m_used = m_new;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + lane_off + c * 32, r);
            tmem_wait_ld(r);
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + lane_off + c * 32, r);
          }
          tmem_wait_st();
        }
      } else {
        m_used = m_new;
      }
      // ---- p = exp2(logit2 - m), row sum, P -> tensor memory (the A operand of O += P.V)
      const float msub = m_used == -INFINITY ? 0.f : m_used;
      uint64_t l2a = f2(0.f, 0.f), l2b = f2(0.f, 0.f);
      const uint64_t nm = f2(-msub, -msub);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t w[16];  // 32 keys = 16 packed words
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint64_t v = f2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
          float a0, a1;
          f2_unpack(MODE == FWD_PLAIN ? f2_fma(v, sl2p, nm) : f2_add(v, nm), a0, a1);
          const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
          if (i & 2) l2b = f2_add(l2b, f2(p0, p1)); else l2a = f2_add(l2a, f2(p0, p1));
          w[i / 2] = Pack2<T>::pack(p0, p1);
        }
        tmem_st16(tP + lane_off + c * 16, w);
      }
      {
        float x0, x1, x2, x3;
        f2_unpack(l2a, x0, x1);
        f2_unpack(l2b, x2, x3);
        l += (x0 + x1) + (x2 + x3);
      }
    };

    for (int w = 0, idx; (idx = item_index(w)) < a.total_items; ++w) {
    const Item item = item_of(idx);
    const int b = item.b, h = item.h, bh = item.bh, n_kv = item.n_kv;
    q0 = item.q0;
    grow = q0 + row;
    m_used = -INFINITY;
    l = 0.f;
    if (ALIBI) slope2 = __ldg(a.alibi_slopes + h) * kLog2e;
    if (!ALIBI && a.mask_kind != FB_MASK_NONE) {
      msize = a.mask_dtype == FB_DTYPE_F32 ? 4 : 2;
      const int mb = a.mask_batch_period > 0 ? b % a.mask_batch_period : b;
      const int64_t off = mb * a.mask_stride[0] + h * a.mask_stride[1] +
                          (int64_t)min(grow, a.Sq - 1) * a.mask_stride[2];
      mrow = reinterpret_cast<const char*>(a.mask) + off * msize;
      mvec = (reinterpret_cast<uintptr_t>(mrow) & 15) == 0;
    }
    for (int j = 0; j < n_kv; ++j, ++t) {
      const int k0 = j * 128;
      mbar_wait(s_full, t & 1, abort_flag, a.status);
      tc_fence_after_sync();
      const bool dead = (a.causal && k0 + 127 > q0) || (k0 + 128 > a.Sk);
      if constexpr (ALIBI) {
        if (dead) tile(j, std::integral_constant<int, FWD_ALIBI>{}, std::true_type{});
        else tile(j, std::integral_constant<int, FWD_ALIBI>{}, std::false_type{});
      } else if (mrow) {
        if (dead) tile(j, std::integral_constant<int, FWD_MASK>{}, std::true_type{});
        else tile(j, std::integral_constant<int, FWD_MASK>{}, std::false_type{});
      } else {
        if (dead) tile(j, std::integral_constant<int, FWD_PLAIN>{}, std::true_type{});
        else tile(j, std::integral_constant<int, FWD_PLAIN>{}, std::false_type{});
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(p_ready);
    }
    // ---- epilogue: O / l -> global, lse
    mbar_wait(pv_done, (t - 1) & 1, abort_flag, a.status);
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
      // natural-log lse of the logits: (m + log2 l) * ln 2
      a.lse[(int64_t)bh * a.lse_stride_bh + grow] =
          l > 0.f ? (m_used + fast_log2(l)) * 0.6931471805599453f : -INFINITY;
    }
    // the reads of O above are complete before the next item's first P.V product (issued after this warp's next
    // arrival on p_ready) overwrites the accumulator
    tc_fence_before_sync();
    }  // work items
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
template <typename T, int D, int RP, int NQ, bool ALIBI>
int launch_fwd_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  using Cfg = FwdCfg<D, RP, NQ>;
  if constexpr (!Cfg::FITS) {
    return FB_ENOTBUILT;
  } else {
    int rc;
    uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
    void* qpack = ws;
    void* kpack = ws + plan.q_bytes;
    void* qs = ws + plan.q_bytes + plan.k_bytes;
    CUtensorMap tQ, tK, tV, tQb, tKb;
    constexpr int BOXD = D > 64 ? 64 : D;
    constexpr int BOXR = RP > 64 ? 64 : (RP ? RP : 16);
    if (NQ == 2) {
      // query operand = (hi, lo) of q*scale, laid out (B, H, Sq, 2D) in the workspace
      if ((rc = make_tmap_4d(&tQ, qs, 2 * D, p->Sq, p->H, p->B, 2 * D, (int64_t)2 * D * p->Sq,
                             (int64_t)2 * D * p->Sq * p->H, BOXD, 128)))
        return rc;
    } else if ((rc = make_tmap_4d(&tQ, p->q, D, p->Sq, p->H, p->B, p->q_stride[2], p->q_stride[1], p->q_stride[0],
                                  BOXD, 128))) {
      return rc;
    }
    if ((rc = make_tmap_4d(&tK, p->k, D, p->Sk, p->H, p->B, p->k_stride[2], p->k_stride[1], p->k_stride[0], BOXD,
                           128)))
      return rc;
    if ((rc = make_tmap_4d(&tV, p->v, D, p->Sk, p->H, p->B, p->v_stride[2], p->v_stride[1], p->v_stride[0], BOXD,
                           128)))
      return rc;
    if (RP) {
      if ((rc = make_tmap_4d(&tQb, qpack, RP, p->Sq, plan.Hq, plan.Bq, RP, (int64_t)RP * p->Sq,
                             (int64_t)RP * p->Sq * plan.Hq, BOXR, 128)))
        return rc;
      if ((rc = make_tmap_4d(&tKb, kpack, RP, p->Sk, plan.Hk, plan.Bk, RP, (int64_t)RP * p->Sk,
                             (int64_t)RP * p->Sk * plan.Hk, BOXR, 128)))
        return rc;
    } else {
      tQb = tQ;
      tKb = tK;
    }
    FwdArgs a;
    a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
    a.nq_tiles = (p->Sq + 127) / 128;
    a.total_items = (int)((int64_t)a.nq_tiles * p->B * p->H);
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
    a.mask = p->mask;
    for (int i = 0; i < 3; ++i) a.mask_stride[i] = p->mask_stride[i];
    if (p->mask_kind == FB_MASK_VECTOR) a.mask_stride[2] = 0;
    a.mask_kind = p->mask_kind;
    a.mask_dtype = p->mask_dtype;
    a.mask_batch_period = p->mask_batch_period;
    a.alibi_slopes = p->alibi_slopes;
    // (the tensor maps above are encoded first: the host then has the main kernel's launch ready while the operand
    // preparation runs)
    if ((rc = launch_pack_operands(p, plan, qpack, kpack, nullptr, false, qs, st))) return rc;
    auto kern = fwd_sm100_kernel<T, D, RP, NQ, ALIBI>;
    // per kernel instantiation and device: raise the dynamic shared-memory limit once
    static std::mutex mu;
    static int sm_count[64] = {};  // 0: not set up on that device yet
    int dev = 0;
    cudaGetDevice(&dev);
    {
      std::lock_guard<std::mutex> lk(mu);
      if (!sm_count[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        int n = 0;
        e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || n <= 0) return e != cudaSuccess ? (int)e : FB_ENOTBUILT;
        sm_count[dev & 63] = n;
      }
    }
    // persistent: one CTA per resident slot (or fewer, if there are fewer work items)
    const int slots = sm_count[dev & 63] * Cfg::MINB;
    const unsigned grid = (unsigned)(a.total_items < slots ? a.total_items : slots);
    prof_before(KC_FWD_MAIN, st);
    kern<<<grid, 256, Cfg::SMEM, st>>>(tQ, tK, tV, tQb, tKb, a);
    prof_after(KC_FWD_MAIN, st);
    note_launch();
    return (int)cudaGetLastError();
  }
}

// whether the variant for (head_dim, packed rank, query terms) exists and fits one SM
bool fwd_cfg_fits(int D, int RP, int nq);

// dispatch over the packed rank for one head_dim (one translation unit per head_dim)
int dispatch_fwd_d32(const fb_params* p, const PackPlan& plan, cudaStream_t st);
int dispatch_fwd_d64(const fb_params* p, const PackPlan& plan, cudaStream_t st);
int dispatch_fwd_d128(const fb_params* p, const PackPlan& plan, cudaStream_t st);

#define FB_FWD_DISPATCH_BODY(DD)                                                                            \
  template <typename T>                                                                                     \
  static int dispatch_fwd_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {                    \
    if (p->alibi_slopes) return launch_fwd_t<T, DD, 0, 1, true>(p, plan, st);                               \
    switch (plan.RP) {                                                                                      \
      case 0: return launch_fwd_t<T, DD, 0, 1, false>(p, plan, st);                                         \
      case 16: return plan.nq == 2 ? launch_fwd_t<T, DD, 16, 2, false>(p, plan, st)                         \
                                   : launch_fwd_t<T, DD, 16, 1, false>(p, plan, st);                        \
      case 32: return plan.nq == 2 ? launch_fwd_t<T, DD, 32, 2, false>(p, plan, st)                         \
                                   : launch_fwd_t<T, DD, 32, 1, false>(p, plan, st);                        \
      case 64: return plan.nq == 2 ? launch_fwd_t<T, DD, 64, 2, false>(p, plan, st)                         \
                                   : launch_fwd_t<T, DD, 64, 1, false>(p, plan, st);                        \
      case 128: return plan.nq == 2 ? launch_fwd_t<T, DD, 128, 2, false>(p, plan, st)                       \
                                    : launch_fwd_t<T, DD, 128, 1, false>(p, plan, st);                      \
    }                                                                                                       \
    return FB_ENOTBUILT;                                                                                    \
  }

}  // namespace fb
