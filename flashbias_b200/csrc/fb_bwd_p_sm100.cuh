// Backward FlashBias attention for sm_100a, persistent form of the query-major kernel.
//
// Same decomposition, roles, shared-memory and tensor-memory layout as bwd_sm100_kernel: a work item is a tile of
// 128 keys of one (batch, head) with the query tiles that see it.  Here one CTA per SM walks a sequence of items:
// the query-tile ring, the barrier phases, the P/dS buffers and the dQ accumulators run on counters that carry over
// from item to item, so the loads of the next item's first query tiles are in flight while the last tiles of this
// item are computed, and the allocation of tensor memory, the barrier set-up and the CTA launch happen once.
// Between items the resident key tiles are reloaded in two groups, each as soon as its last reader has completed
// (the S|dP operands one query tile before the item ends), the dV / dK accumulators are handed over through one
// more barrier (acc_free), and dV, dK and dk_bias leave as staged tiles through the copy engine.
//
// Short sequences are what this form is for (windowed attention: two query tiles per item), where the set-up
// and drain of a CTA cost more than its tiles; with many query tiles per item the one-item-per-CTA kernel, whose
// item coordinates are launch constants, runs the tile loop faster and is the one used.
#pragma once

#include "fb_bwd_sm100.cuh"

namespace fb {

// n / d for 0 <= n < 2^31 with (m, s) from fast_div_magic(d): one multiply-high, one add, one shift
__device__ __forceinline__ int fast_div(int n, const uint32_t (&ms)[2]) {
  return (int)((__umulhi((uint32_t)n, ms[0]) + (uint32_t)n) >> ms[1]);
}
inline void fast_div_magic(int d, uint32_t (&ms)[2]) {
  uint32_t s = 0;
  while ((1u << s) < (uint32_t)d) ++s;  // ceil(log2 d)
  ms[0] = (uint32_t)((((uint64_t)1 << 32) * (((uint64_t)1 << s) - (uint64_t)d)) / (uint64_t)d + 1);
  ms[1] = s;
}

// one work item of the backward: a tile of 128 keys of one (batch, head) and the query tiles that see it
struct BwdItem {
  int kt, bh, b, h, k0, i_begin, n_it;
  bool valid;
};


// arguments of the persistent form beyond BwdArgs
struct BwdPArgs {
  int total_items;   // (key tile, batch, head) work items = nk_tiles * B * H
  int active_items;  // the first so many have query tiles to visit (all of them unless causal with Sq < Sk)
  uint32_t div_bh[2], div_nk[2], div_h[2];  // (multiplier, shift) of the divisions by B*H, nk_tiles and H
};

template <typename T, int D, int RP, int NQ, int MODE>
__global__ void __launch_bounds__(512, 1)
bwd_p_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmQb, const __grid_constant__ CUtensorMap tmKb,
                 const __grid_constant__ CUtensorMap tmKc, const __grid_constant__ CUtensorMap tmKs,
                 const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                 const BwdArgs a, const BwdPArgs pa) {
  using Cfg = BwdCfg<D, RP, NQ>;
  constexpr int RPX = Cfg::RPX;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase + Cfg::OFF_K, sKs = sbase + Cfg::OFF_KS, sKb = sbase + Cfg::OFF_KB,
                 sKc = sbase + Cfg::OFF_KC, sV = sbase + Cfg::OFF_V, sStage = sbase + Cfg::OFF_STAGE,
                 sP = sbase + Cfg::OFF_P, sDS = sbase + Cfg::OFF_DS, sStg = sbase + Cfg::OFF_STG,
                 sStgB = sStg + 128 * D * 4;
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  const uint32_t kva_full = bar0, kvb_full = bar0 + 8, dp_full = bar0 + 16, sdp_read = bar0 + 24,
                 dq_full = bar0 + 32 /*2*/, qdo_full = bar0 + 48 /*3*/, qdo_free = bar0 + 72 /*3*/,
                 all_done = bar0 + 112, pds_free = bar0 + 120, pds_ready = bar0 + 136 /*2*/,
                 dq_drained = bar0 + 152 /*2*/, acc_free = bar0 + 168, sdp_done = bar0 + 176;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 104);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = a.B * a.H;
  // Persistent CTA: work item w of this CTA is item w * gridDim.x + (position of the CTA in row w), the rows
  // alternating in direction (snake order) so that the CTAs that got the heavier items of one row get the lighter
  // ones of the next.  Under causal masking key tile 0 sees the most query tiles: heaviest items first.
  // Every role walks the same item sequence; barrier phases, ring stages and buffer indices run on counters that
  // carry over from item to item (n: items with work so far, T: query tiles so far).
  auto get_item = [&](int w, int limit) {
    BwdItem x;
    const int G = (int)gridDim.x, c = (int)blockIdx.x;
    const int idx = w * G + ((w & 1) ? G - 1 - c : c);
    x.valid = idx < limit;
    if (a.causal) {
      x.kt = fast_div(idx, pa.div_bh);
      x.bh = idx - x.kt * BH;
    } else {
      x.bh = fast_div(idx, pa.div_nk);
      x.kt = idx - x.bh * a.nk_tiles;
    }
    x.b = fast_div(x.bh, pa.div_h);
    x.h = x.bh - x.b * a.H;
    x.k0 = x.kt * 128;
    x.i_begin = a.causal ? x.kt : 0;    // first query tile with a row >= k0
    x.n_it = a.nq_tiles - x.i_begin;    // <= 0 for the items past active_items (causal with Sq < Sk)
    return x;
  };
  // Items without query tiles (key tiles that no query sees) come last in the order above: every role but the
  // compute warps, which zero those keys' gradients, stops at active_items.
  auto next_active = [&](int& w) { return get_item(w, pa.active_items); };

  // producer thread only: one stage of the query-tile ring (tl: running tile count of this CTA)
  auto load_tile = [&](const BwdItem& x, int it, uint32_t tl) {
    const int st = (int)(tl % Cfg::NSTAGE);
    const uint32_t base = sStage + st * Cfg::STAGE_BYTES;
    const int hq = a.hq_bcast ? 0 : x.h, bq = a.bq_bcast ? 0 : x.b;
    mbar_expect_tx(qdo_full + 8 * st, Cfg::STAGE_BYTES);
    const int q0 = (x.i_begin + it) * 128;
    tma_tile_bwd<D>(base, &tmQ, qdo_full + 8 * st, q0, x.h, x.b);
    if (RP) tma_tile_bwd<RPX>(base + Cfg::OFF_QB, &tmQb, qdo_full + 8 * st, q0, hq, bq);
    tma_tile_bwd<D>(base + Cfg::OFF_DO, &tmDO, qdo_full + 8 * st, q0, x.h, x.b);
  };
  // The resident tiles of an item's key block, in two groups by reader.  Group A -- (hi, lo) of k*scale, Kb, V --
  // is read by the S and dP products only: the thread that issues them reloads it for the next item as soon as the
  // last S|dP of this item has completed, one query tile before the item ends, so that the tensor core computes
  // the next item's first S and dP under this item's last tile of arithmetic.  Group B -- K, Kc -- is read by
  // the dQ | dQb products (K also by S when the scale is not split): the producer reloads it after the last dQ.
  constexpr uint32_t KVA_BYTES = (NQ == 2 ? 2 * Cfg::D_BYTES : 0) + Cfg::R_BYTES + Cfg::D_BYTES;
  constexpr uint32_t KVB_BYTES = Cfg::D_BYTES + Cfg::RC_BYTES;
  static_assert(KVA_BYTES + KVB_BYTES == (uint32_t)Cfg::KV_BYTES, "resident tiles");
  auto load_kva = [&](const BwdItem& x) {
    const int hk = a.hk_bcast ? 0 : x.h, bk = a.bk_bcast ? 0 : x.b;
    mbar_expect_tx(kva_full, KVA_BYTES);
    if (NQ == 2) {
      tma_tile_bwd<D>(sKs, &tmKs, kva_full, x.k0, x.h, x.b);
      tma_tile_bwd<D>(sKs + Cfg::D_BYTES, &tmKs, kva_full, x.k0, x.h, x.b, D);
    }
    if (RP) tma_tile_bwd<RPX>(sKb, &tmKb, kva_full, x.k0, hk, bk);
    tma_tile_bwd<D>(sV, &tmV, kva_full, x.k0, x.h, x.b);
  };
  auto load_kvb = [&](const BwdItem& x) {
    const int hk = a.hk_bcast ? 0 : x.h, bk = a.bk_bcast ? 0 : x.b;
    mbar_expect_tx(kvb_full, KVB_BYTES);
    tma_tile_bwd<D>(sK, &tmK, kvb_full, x.k0, x.h, x.b);
    if (RP) tma_tile_bwd<Cfg::RCX>(sKc, &tmKc, kvb_full, x.k0, hk, bk);
  };
  // cursor of the ring loads (producer thread): runs NSTAGE tiles ahead of the products, across item boundaries
  int lw = 0, lit = 0;
  uint32_t TL = 0;
  BwdItem lx;
  lx.valid = false;
  auto load_next = [&]() {
    load_tile(lx, lit, TL);
    ++TL;
    if (++lit == lx.n_it) {
      lit = 0;
      ++lw;
      lx = next_active(lw);
    }
  };

  if (warp == 12) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(kva_full, 1);
      mbar_init(kvb_full, 1);
      mbar_init(sdp_done, 1);  // the last S|dP products of an item have completed
      mbar_init(dp_full, 1);
      mbar_init(sdp_read, 8);  // every compute warp has S and dP of the tile in registers
      mbar_init(all_done, 4);  // one commit per issuing thread, per item
      mbar_init(acc_free, 8);  // the compute warps have read the dV / dK | dKb accumulators of an item
      for (int i = 0; i < 2; ++i)  // the dV, dK, dQ (and dKb) chains have read P and dS of a query tile (per buffer pair)
        mbar_init(pds_free + 8 * i, Cfg::SEP_DKB ? 4 : 3);
      for (int i = 0; i < 3; ++i) {
        mbar_init(qdo_full + 8 * i, 1);
        mbar_init(qdo_free + 8 * i, 3);  // S|dP, dV and dK chains read a stage
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(dq_full + 8 * i, 1);
        mbar_init(dq_drained + 8 * i, 4);  // the drain warps
        mbar_init(pds_ready + 8 * i, 8);   // the compute warps; alternating by query tile, as the issuers wait at
                                           // different times
      }
      mbar_fence_init();
      // the first loads start before the rest of the CTA has finished its set-up
      lx = next_active(lw);
      if (lx.valid) {
        load_kva(lx);
        load_kvb(lx);
        for (int i = 0; i < Cfg::NSTAGE && lx.valid; ++i) load_next();
      }
    }
  } else if (warp == 13) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // 512 threads start with 128 registers each; the two compute warpgroups hold a whole tile of S and dP in
  // registers and take 192, the drain warpgroup and the producer/issuer warpgroup keep 64.  Each warpgroup
  // changes its budget at the head of its own branch.
  if (warp >= 12) {
  setmaxnreg_dec<64>();
  if (warp == 12) {
    // ------------------------------------------------------------------ TMA producer, dQ | dQb chain
    if (lane == 0) {
      // The same thread issues the dQ | dQb products: they become due when a query tile's P/dS are written,
      // the next load when the other chains have finished with that tile's stage -- in this order, every tile.
      constexpr uint32_t idQD = instr_desc(kBf16, false, true, 128, D);             // dQ: A K-major, B MN-major
      constexpr uint32_t idQM = instr_desc(kBf16, false, true, 128, D + Cfg::RCX);  // dQ|dQb merged
      constexpr uint32_t idQC = instr_desc(kBf16, false, true, 128, Cfg::RCX);      // dQb alone
      const DescBase kDS = kmajor_base<128>(sDS), mK = mnmajor_base<D>(sK), mKc = mnmajor_base<Cfg::RCX>(sKc);
      // [K | Kc]: 32-column blocks of 64-byte-swizzled rows, the second block at the distance between the tiles
      const uint64_t dKKc = smem_desc(sK, Cfg::OFF_KC - Cfg::OFF_K, 8 * 64, 64);
      const DescBase mKKc{(uint32_t)dKKc, (uint32_t)(dKKc >> 32)};
      auto issue_dQ = [&](uint32_t it) {  // it: running tile count
        const int qb = (int)(it % Cfg::NDQ);  // dQ|dQb accumulator of this tile
        const uint32_t tq = tmem + qb * Cfg::DQ_STRIDE;
        const uint32_t pb = (it % Cfg::NBUF) * Cfg::PDS_STRIDE;  // P/dS buffer pair of this tile
        mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
        if (it >= (uint32_t)Cfg::NDQ)  // the drain warpgroup has read the tile that used this accumulator last
          mbar_wait(dq_drained + 8 * qb, (it / Cfg::NDQ - 1) & 1, abort_flag, a.status);
        tc_fence_after_sync();
#pragma unroll
        for (int s = 0; s < 8; ++s) {  // contraction over the 128 keys
          if (Cfg::MERGE_Q) {
            umma_ss(tq + Cfg::T_DQ, desc_at(kDS, pb + kmajor_step<128>(s)), desc_at(mKKc, mnmajor_step<D>(s)),
                    idQM, s > 0);
          } else {
            umma_ss(tq + Cfg::T_DQ, desc_at(kDS, pb + kmajor_step<128>(s)), desc_at(mK, mnmajor_step<D>(s)),
                    idQD, s > 0);
            if (RP)
              umma_ss(tq + Cfg::T_DQB, desc_at(kDS, pb + kmajor_step<128>(s)),
                      desc_at(mKc, mnmajor_step<Cfg::RCX>(s)), idQC, s > 0);
          }
        }
        umma_commit(dq_full + 8 * qb);
        umma_commit(pds_free + 8 * (it % Cfg::NBUF));  // this chain no longer reads dS of the tile
      };
      uint32_t tn = 0;
      int n = 0;
#pragma unroll 1
      for (int w = 0;; ++w) {
        const BwdItem x = next_active(w);
        if (!x.valid) break;
        mbar_wait(kvb_full, n & 1, abort_flag, a.status);
#pragma unroll 1
        for (int it = 0; it < x.n_it; ++it, ++tn) {
          issue_dQ(tn);
          if (lx.valid) {  // the S|dP, dV and dK chains have finished reading the stage of tile tn: tile tn + NSTAGE
            mbar_wait(qdo_free + 8 * (tn % Cfg::NSTAGE), (tn / Cfg::NSTAGE) & 1, abort_flag, a.status);
            load_next();
          }
        }
        umma_commit(all_done);
        const BwdItem nx = get_item(w + 1, pa.active_items);
        if (nx.valid) {  // K and Kc are free once the dQ | dQb products of the item's last tile have completed
          const uint32_t tl = tn - 1;
          mbar_wait(dq_full + 8 * (tl % Cfg::NDQ), (tl / Cfg::NDQ) & 1, abort_flag, a.status);
          load_kvb(nx);
        }
        ++n;
      }
    }
  } else if (warp >= 13) {
    // ------------------------------------------------------------------ MMA issuers
    // One elected thread per warp, each warp on its own warp scheduler (the producer warp issues the fourth
    // chain, dQ | dQb).  A thread that issues tcgen05.mma competes with the compute warps of its scheduler, so
    // one thread alone cannot feed the tensor core; the chains are independent (different accumulators) and
    // run concurrently:
    //   warp 13  S and dP of query tile i, as soon as tile i-1 is in registers
    //   warp 13  also dKb when it is a separate accumulator      warp 14  dV
    //   warp 15  dK (or dK | dKb merged)
    // Every accumulator is only ever touched by one thread, which keeps its MMAs ordered.
    if (lane == 0) {
      const int role = warp - 13;
      constexpr uint32_t idS = instr_desc(kBf16, false, false, 128, 128);  // S, dP: both operands K-major
      constexpr uint32_t idTD = instr_desc(kBf16, true, true, 128, D);     // dV, dK: A^T (MN-major), B MN-major
      constexpr uint32_t idTR = instr_desc(kBf16, true, true, 128, RPX);   // dKb
      constexpr uint32_t idKM = instr_desc(kBf16, true, true, 128, 64);    // dK | dKb merged
      uint32_t tn = 0;  // running tile count
      int n = 0;       // items with work so far
      if (role == 0) {
        // descriptor views built once (stage 0); each MMA adds a constant to the address field
        const DescBase kQ = kmajor_base<D>(sStage), kDO = kmajor_base<D>(sStage + Cfg::OFF_DO),
                       kQb = kmajor_base<RPX>(sStage + Cfg::OFF_QB), kK = kmajor_base<D>(NQ == 2 ? sKs : sK),
                       kKb = kmajor_base<RPX>(sKb), kV = kmajor_base<D>(sV);
        // dKb, when it is an accumulator of its own (no merged [Q | Qb] operand), is issued by this thread as
        // well: between S|dP of query tile i and of tile i+1 it would otherwise idle, and the dV thread, which
        // releases the stage of the tile, gets shorter
        const DescBase mQbT = mnmajor_base<RPX>(sStage + Cfg::OFF_QB), mDST = mnmajor_base<128>(sDS);
        auto issue_dKb = [&](int it, uint32_t t) {  // it: tile of the item, t: running tile count
          const int st = (int)(t % Cfg::NSTAGE);
          const uint32_t so = st * Cfg::STAGE_BYTES;
          mbar_wait(pds_ready + 8 * (t & 1), (t >> 1) & 1, abort_flag, a.status);
          if (it == 0 && n > 0)  // the compute warps have read the previous item's accumulator
            mbar_wait(acc_free, (n - 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma_ss(tmem + Cfg::T_DKB, desc_at(mDST, (t % Cfg::NBUF) * Cfg::PDS_STRIDE + mnmajor_step<128>(s)),
                    desc_at(mQbT, so + mnmajor_step<RPX>(s)), idTR, (it > 0 || s > 0) ? 1u : 0u);
          umma_commit(qdo_free + 8 * st);  // S|dP and dKb of the tile: this thread is done with its stage
          umma_commit(pds_free + 8 * (t % Cfg::NBUF));
        };
#pragma unroll 1
        for (int w = 0;; ++w) {
          const BwdItem x = next_active(w);
          if (!x.valid) break;
          mbar_wait(kva_full, n & 1, abort_flag, a.status);
          if (NQ != 2) mbar_wait(kvb_full, n & 1, abort_flag, a.status);  // S reads K itself
          tc_fence_after_sync();
#pragma unroll 1
          for (int it = 0; it < x.n_it; ++it, ++tn) {
            const int st = (int)(tn % Cfg::NSTAGE);
            const uint32_t so = st * Cfg::STAGE_BYTES;
            if (tn > 0) {  // the compute warps hold S and dP of the previous tile in registers
              mbar_wait(sdp_read, (tn - 1) & 1, abort_flag, a.status);
              tc_fence_after_sync();
            }
            mbar_wait(qdo_full + 8 * st, (tn / Cfg::NSTAGE) & 1, abort_flag, a.status);
            tc_fence_after_sync();
            // bias products first, into the empty accumulator (large factor terms cancel among themselves)
            if (RP) {
#pragma unroll
              for (int s = 0; s < RPX / 16; ++s)
                umma_ss(tmem + Cfg::T_S, desc_at(kQb, so + kmajor_step<RPX>(s)), desc_at(kKb, kmajor_step<RPX>(s)),
                        idS, s > 0);
            }
#pragma unroll
            for (int t = 0; t < NQ; ++t) {  // key terms (k, or hi and lo of k*scale) share the Q tile
#pragma unroll
              for (int s = 0; s < D / 16; ++s)
                umma_ss(tmem + Cfg::T_S, desc_at(kQ, so + kmajor_step<D>(s)),
                        desc_at(kK, t * Cfg::D_BYTES + kmajor_step<D>(s)), idS, (RP || t > 0 || s > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int s = 0; s < D / 16; ++s)
              umma_ss(tmem + Cfg::T_DP, desc_at(kDO, so + kmajor_step<D>(s)), desc_at(kV, kmajor_step<D>(s)), idS,
                      s > 0);
            umma_commit(dp_full);
            if (it + 1 == x.n_it) umma_commit(sdp_done);
            if (Cfg::SEP_DKB) {
              if (it > 0) issue_dKb(it - 1, tn - 1);
            } else {
              umma_commit(qdo_free + 8 * st);
            }
          }
          {
            const BwdItem nx = get_item(w + 1, pa.active_items);
            if (nx.valid) {  // group A of the next item, while the compute warps are on this item's last tile
              mbar_wait(sdp_done, n & 1, abort_flag, a.status);
              load_kva(nx);
            }
          }
          if (Cfg::SEP_DKB) issue_dKb(x.n_it - 1, tn - 1);
          umma_commit(all_done);  // every MMA of this thread for the item
          ++n;
        }
      } else {
        const DescBase mQ = mnmajor_base<D>(sStage), mDO = mnmajor_base<D>(sStage + Cfg::OFF_DO),
                       mP = mnmajor_base<128>(sP), mDS = mnmajor_base<128>(sDS);
        // [Q | Qb]: 32-column blocks of 64-byte-swizzled rows, the second block at the distance between the tiles
        const uint64_t dQQb = smem_desc(sStage, Cfg::OFF_QB, 8 * 64, 64);
        const DescBase mQQb{(uint32_t)dQQb, (uint32_t)(dQQb >> 32)};
#pragma unroll 1
        for (int w = 0;; ++w) {
          const BwdItem x = next_active(w);
          if (!x.valid) break;
#pragma unroll 1
          for (int it = 0; it < x.n_it; ++it, ++tn) {
            const int st = (int)(tn % Cfg::NSTAGE);
            const uint32_t so = st * Cfg::STAGE_BYTES;
            const uint32_t acc0 = it > 0 ? 1u : 0u;
            const uint32_t pb = (tn % Cfg::NBUF) * Cfg::PDS_STRIDE;  // P/dS buffer pair of this tile
            mbar_wait(qdo_full + 8 * st, (tn / Cfg::NSTAGE) & 1, abort_flag, a.status);
            mbar_wait(pds_ready + 8 * (tn & 1), (tn >> 1) & 1, abort_flag, a.status);
            if (it == 0 && n > 0)  // the compute warps have read the previous item's accumulators
              mbar_wait(acc_free, (n - 1) & 1, abort_flag, a.status);
            tc_fence_after_sync();
            if (role == 1) {
#pragma unroll
              for (int s = 0; s < 8; ++s)  // contraction over the 128 query rows
                umma_ss(tmem + Cfg::T_DV, desc_at(mP, pb + mnmajor_step<128>(s)),
                        desc_at(mDO, so + mnmajor_step<D>(s)), idTD, (acc0 | (s > 0)) ? 1u : 0u);
            } else {
#pragma unroll
              for (int s = 0; s < 8; ++s) {
                if (Cfg::MERGE_K)
                  umma_ss(tmem + Cfg::T_DK, desc_at(mDS, pb + mnmajor_step<128>(s)),
                          desc_at(mQQb, so + mnmajor_step<D>(s)), idKM, (acc0 | (s > 0)) ? 1u : 0u);
                else
                  umma_ss(tmem + Cfg::T_DK, desc_at(mDS, pb + mnmajor_step<128>(s)),
                          desc_at(mQ, so + mnmajor_step<D>(s)), idTD, (acc0 | (s > 0)) ? 1u : 0u);
              }
            }
            umma_commit(qdo_free + 8 * st);
            umma_commit(pds_free + 8 * (tn % Cfg::NBUF));  // this chain no longer reads P / dS of the tile
          }
          umma_commit(all_done);  // every MMA of this thread for the item
          ++n;
        }
      }
    }
  }
  } else if (warp >= 8) {
    setmaxnreg_dec<64>();
    // ------------------------------------------------------------------ drain warpgroup
    // dQ | dQb of each query tile from TMEM into the fp32 accumulators in global memory, off the critical path
    // of the warps that compute P and dS.  One thread per query row.
    {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
      float* s_kbc = reinterpret_cast<float*>(smem + Cfg::OFF_KBC);
      // k_bias of the four keys the centred copy refers to (one per 32-key group), as fp32, laid out [column][key
      // group]: one entry per thread, fetched one item ahead so that the load is not waited for at the item's head
      float kbc_next = 0.f;
      auto fetch_kbc = [&](const BwdItem& y) {
        const int i = (int)threadIdx.x - 256;
        const int c = i >> 2, g = i & 3;
        kbc_next = 0.f;
        if (i < 2 * Cfg::RCX && c < a.R) {
          const T* kb_bh = a.k_bias_t<T>() + (a.bk_bcast ? 0 : y.b) * a.kb_stride[0] + (a.hk_bcast ? 0 : y.h) * a.kb_stride[1];
          kbc_next = to_f32(kb_bh[(int64_t)min(y.k0 + 32 * g + 16, a.Sk - 1) * a.kb_stride[2] + c]);
        }
      };
      if (RP) {
        int w0 = 0;
        const BwdItem first = next_active(w0);
        if (first.valid) fetch_kbc(first);
      }
      uint32_t tn = 0;  // running tile count
#pragma unroll 1
      for (int w = 0;; ++w) {
      const BwdItem x = next_active(w);
      if (!x.valid) break;
      const int b = x.b, h = x.h, bh = x.bh, i_begin = x.i_begin;
      if (RP) {
        // written and read by this warpgroup only: every tile of the previous item has been drained when it gets here
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if ((int)threadIdx.x - 256 < 2 * Cfg::RCX) s_kbc[threadIdx.x - 256] = kbc_next;
        asm volatile("bar.sync 3, 128;" ::: "memory");
        const BwdItem nx = get_item(w + 1, pa.active_items);
        if (nx.valid) fetch_kbc(nx);
      }
#pragma unroll 1
      for (int it = 0; it < x.n_it; ++it, ++tn) {
        const int grow = (i_begin + it) * 128 + row;
        const int qb = (int)(tn % Cfg::NDQ);
        const uint32_t tq = tmem + qb * Cfg::DQ_STRIDE + lane_off;
        mbar_wait(dq_full + 8 * qb, (tn / Cfg::NDQ) & 1, abort_flag, a.status);
        tc_fence_after_sync();
        if (!Cfg::STAGED) {
          // no staging tile: reduce straight from registers (one row per thread)
          float* dst = a.dq_acc + (((int64_t)b * a.Sq + grow) * a.H + h) * D;
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tq + Cfg::T_DQ + c0, r);
            tmem_wait_ld(r);
            if (grow < a.Sq) {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                red_add_v4(dst + c0 + g * 4, __uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]),
                           __uint_as_float(r[g * 4 + 2]), __uint_as_float(r[g * 4 + 3]));
            }
          }
        } else {
          // dQ tile: TMEM -> registers -> shared-memory staging -> ONE bulk reduction into the fp32 accumulator.
          // Per-thread vector reductions (32 per row) crowd the load/store unit that the compute warps need for
          // their P/dS stores; the bulk form is executed by the copy engine.  The first columns are fetched into
          // registers while the copy engine may still be reading the previous tile from the staging tile; the
          // thread that issued that reduction then waits for its shared-memory reads and the warpgroup syncs.
          uint32_t r0[16], r1[16];
          tmem_ld16(tq + Cfg::T_DQ, r0);
          tmem_ld16(tq + Cfg::T_DQ + 16, r1);
          if (warp == 8 && lane == 0) bulk_wait_group_read0();
          __syncwarp();
          asm volatile("bar.sync 3, 128;" ::: "memory");  // the drain warpgroup only
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            if (c0 > 0) {
              tmem_ld16(tq + Cfg::T_DQ + c0, r0);
              tmem_ld16(tq + Cfg::T_DQ + c0 + 16, r1);
            }
            tmem_wait_ld(r0);
            tmem_wait_ld(r1);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              st_shared_v4(sStg + dq_stage_off(row, c0 / 4 + g), r0[g * 4], r0[g * 4 + 1], r0[g * 4 + 2],
                           r0[g * 4 + 3]);
              st_shared_v4(sStg + dq_stage_off(row, c0 / 4 + 4 + g), r1[g * 4], r1[g * 4 + 1], r1[g * 4 + 2],
                           r1[g * 4 + 3]);
            }
          }
        }
        if (RP) {
          const float* s_rowsum = reinterpret_cast<const float*>(smem + Cfg::OFF_ROWSUM) + (tn & 3) * 512;
          const int bq = a.bq_bcast ? 0 : b, hq = a.hq_bcast ? 0 : h;
          // accumulator laid out (Bq, Hq, query tiles, R, 128 rows): a tile is contiguous
          float* tileb = a.dqb_acc + (bh % a.dqb_slots) * a.dqb_slot_stride +
                         (((int64_t)bq * a.Hq + hq) * a.nq_tiles + (i_begin + it)) * (128 * a.R);
          float* stgb = reinterpret_cast<float*>(smem + Cfg::OFF_STG + 128 * D * 4) + row;
          drain_dq_bias<Cfg>(tq + Cfg::T_DQB, s_rowsum, sbase + Cfg::OFF_KBC, stgb, tileb, row, grow < a.Sq, a.R);
        }
        tc_fence_before_sync();
        mbar_arrive_warp(dq_drained + 8 * qb);  // every tensor-memory read of the tile is done
        if (Cfg::STAGED) {
          fence_proxy_async_smem();  // the staged tiles become visible to the copy engine
          asm volatile("bar.sync 3, 128;" ::: "memory");
          if (warp == 8 && lane == 0) {
            bulk_reduce_add_f32(a.dq_acc + ((int64_t)bh * a.nq_tiles + (i_begin + it)) * (128 * D), sStg,
                                  128 * D * 4);
            if (RP) {
              const int bq = a.bq_bcast ? 0 : b, hq = a.hq_bcast ? 0 : h;
              bulk_reduce_add_f32(
                  a.dqb_acc + (bh % a.dqb_slots) * a.dqb_slot_stride +
                      (((int64_t)bq * a.Hq + hq) * a.nq_tiles + (i_begin + it)) * (128 * a.R),
                  sStgB,
                  128 * a.R * 4);
            }
            bulk_commit_group();
          }
        }
      }
      }
      // the staging tile must outlive the last reduction's reads; its global side completes with the kernel
      if (Cfg::STAGED && warp == 8 && lane == 0) bulk_wait_group_read0();
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups (warps 0-7)
    setmaxnreg_inc<192>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = a.scale_log2;
    constexpr int DH = D / 2;  // dV / dK columns per warpgroup in the epilogue
    uint32_t tn = 0;  // running tile count
    int n = 0;        // items with work so far
    // Row statistics of a query tile.  Raw loads only: the values are consumed one tile later, so the global-memory
    // latency hides under the current tile's math instead of stalling the thread (volatile: the compiler must not
    // sink the loads to their use).
    auto load_stats = [&](int bh_, int g, bool ok, float& lse_raw, float& dlt) {
      lse_raw = INFINITY;
      dlt = 0.f;
      if (ok && g < a.Sq) {
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(lse_raw) : "l"(a.lse + (int64_t)bh_ * a.lse_stride_bh + g));
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(dlt) : "l"(a.delta + (int64_t)bh_ * a.lse_stride_bh + g));
      }
    };
    float lse_raw = INFINITY, dlt = 0.f;
    bool staged_out = false;  // an item's epilogue tiles may still be being read from the P tile
#pragma unroll 1
    for (int w = 0;; ++w) {
    const BwdItem x = get_item(w, pa.total_items);
    if (!x.valid) break;
    const int b = x.b, h = x.h, bh = x.bh, kt = x.kt, k0 = x.k0, i_begin = x.i_begin, n_it = x.n_it;
    if (n_it <= 0) {
      // causal with Sq < Sk: these keys are seen by no query; their gradients are zero
      const int krow = k0 + row;
      if (krow < a.Sk) {
        T* dvrow = reinterpret_cast<T*>(a.dv) + b * a.dv_stride[0] + h * a.dv_stride[1] + (int64_t)krow * a.dv_stride[2];
        T* dkrow = reinterpret_cast<T*>(a.dk) + b * a.dk_stride[0] + h * a.dk_stride[1] + (int64_t)krow * a.dk_stride[2];
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int c0 = wg * (D / 2); c0 < wg * (D / 2) + D / 2; c0 += 8) {
          *reinterpret_cast<uint4*>(dvrow + c0) = z;
          *reinterpret_cast<uint4*>(dkrow + c0) = z;
        }
      }
      continue;
    }

    if (n == 0) load_stats(bh, i_begin * 128 + row, true, lse_raw, dlt);  // later items: fetched in the previous item's last tile
    float slope2 = 0.f;  // ALiBi slope of this head, times log2 e
    if (MODE == BWD_ALIBI) slope2 = __ldg(a.alibi_slopes + h) * kLog2e;
    const char* mrow = nullptr;  // additive mask of this (batch, head), row 0
    int msize = 4;
    if (MODE == BWD_MASK) {
      msize = a.mask_dtype == FB_DTYPE_F32 ? 4 : 2;
      const int mb = a.mask_batch_period > 0 ? b % a.mask_batch_period : b;
      mrow = reinterpret_cast<const char*>(a.mask) + (mb * a.mask_stride[0] + h * a.mask_stride[1]) * msize;
    }
    // The thread's 64 columns of S and of dP live in registers, as two chunks of 32.  Chunk 0 of a tile is fetched
    // from tensor memory under the P/dS stores of the previous tile; once chunk 1 has followed at the
    // head of the tile, S and dP are released and the tensor core computes the next tile's under this tile's math.
    uint32_t rs0[32], rd0[32], rs1[32], rd1[32];
    const uint32_t tSl = tmem + Cfg::T_S + lane_off + wg * 64, tDl = tmem + Cfg::T_DP + lane_off + wg * 64;
    mbar_wait(dp_full, tn & 1, abort_flag, a.status);  // committed after the S and the dP products: covers both
    tc_fence_after_sync();
    tmem_ld32(tSl, rs0);
    tmem_ld32(tDl, rd0);
#pragma unroll 1
    for (int it = 0; it < n_it; ++it, ++tn) {
      const int q0 = (i_begin + it) * 128;
      const int grow = q0 + row;
      // a row that saw no key has lse = -inf: make its probabilities exactly zero
      const float lse2_cur = lse_raw == -INFINITY ? INFINITY : lse_raw * kLog2e, dlt_cur = dlt;
      const bool need_mask = (a.causal && k0 + 127 > q0) || (k0 + 128 > a.Sk);
      float ds_sum0 = 0.f, ds_sum1 = 0.f;  // fp32 row sums of dS over this thread's two 32-column groups
      tmem_ld32(tSl + 32, rs1);
      tmem_ld32(tDl + 32, rd1);
      tmem_wait_ld(rs0);
      tmem_wait_ld(rd0);
      tmem_wait_ld(rs1);
      tmem_wait_ld(rd1);
      tc_fence_before_sync();
      mbar_arrive_warp(sdp_read);
      // P and dS of the tile stay in registers as packed 16-bit pairs (16 words per 32-column chunk each) until
      // both chunks are done: the shared-memory tiles are still being read by the products of the previous tile.
      // MODE: how the logits are completed (plain / + mask tensor / + ALiBi term).
      auto chunk = [&](uint32_t (&rs)[32], uint32_t (&rd)[32], uint32_t (&pk)[16], uint32_t (&dk)[16], int c) {
        const int col0 = wg * 64 + c * 32;
        const uint64_t sl2p = f2(sl2, sl2), nlse = f2(-lse2_cur, -lse2_cur), ndlt = f2(-dlt_cur, -dlt_cur);
        uint64_t sum2 = f2(0.f, 0.f);
        float mv[32];
        if (MODE == BWD_MASK) {
          const int n = min(32, a.Sk - (k0 + col0));
          const char* p = mrow + ((int64_t)min(grow, a.Sq - 1) * a.mask_stride[2] + k0 + col0) * msize;
          const bool vec = (reinterpret_cast<uintptr_t>(p) & 15) == 0 && n == 32;
          if (n <= 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i) mv[i] = 0.f;
          } else if (a.mask_dtype == FB_DTYPE_F32) load_mask_chunk(reinterpret_cast<const float*>(p), n, vec, mv);
          else if (a.mask_dtype == FB_DTYPE_F16) load_mask_chunk(reinterpret_cast<const __half*>(p), n, vec, mv);
          else load_mask_chunk(reinterpret_cast<const __nv_bfloat16*>(p), n, vec, mv);
        }
        const float abase = slope2 * (float)(k0 + col0 - grow) - lse2_cur;  // ALiBi term of column col0, minus lse
        // the masked and the unmasked tile get separate straight-line loops: a per-element test of need_mask
        // becomes a branch per element and the 32 elements then run one after the other
        auto elems = [&](auto masked) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t sp = f2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1]));
            uint64_t arg;
            if (MODE == BWD_PLAIN) arg = f2_fma(sp, sl2p, nlse);
            if (MODE == BWD_MASK) arg = f2_fma(sp, sl2p, f2_add(f2(mv[i], mv[i + 1]), nlse));
            if (MODE == BWD_ALIBI)
              arg = f2_fma(sp, sl2p, f2(fmaf((float)i, slope2, abase), fmaf((float)(i + 1), slope2, abase)));
            float a0, a1;
            f2_unpack(arg, a0, a1);
            float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
            if (decltype(masked)::value) {
              const int col = k0 + col0 + i;
              if (col >= a.Sk || (a.causal && col > grow)) p0 = 0.f;
              if (col + 1 >= a.Sk || (a.causal && col + 1 > grow)) p1 = 0.f;
            }
            const uint64_t ds = f2_mul(f2(p0, p1), f2_add(f2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1])), ndlt));
            if (RP) sum2 = f2_add(sum2, ds);
            float d0, d1;
            f2_unpack(ds, d0, d1);
            pk[i / 2] = Pack2<T>::pack(p0, p1);
            dk[i / 2] = Pack2<T>::pack(d0, d1);
          }
        };
        if (need_mask) elems(std::true_type{}); else elems(std::false_type{});
        float x0, x1;
        f2_unpack(sum2, x0, x1);
        return x0 + x1;
      };
      uint32_t pk0[16], pk1[16], dk0[16], dk1[16];
      ds_sum0 = chunk(rs0, rd0, pk0, dk0, 0);
      // next tile's statistics (the next item's first tile after the last one): the loads complete under this math
      if (it + 1 < n_it) {
        load_stats(bh, (i_begin + it + 1) * 128 + row, true, lse_raw, dlt);
      } else {
        const BwdItem nx = get_item(w + 1, pa.active_items);
        load_stats(nx.bh, nx.i_begin * 128 + row, nx.valid, lse_raw, dlt);
      }
      ds_sum1 = chunk(rs1, rd1, pk1, dk1, 1);
      // Chunk 0 of the next tile is fetched under the stores below if its S and dP are already there (they were
      // issued when this tile was released).  If not -- a 2-stage ring delivers the next tile late -- the stores
      // must not wait for it: they release this tile's products, which in turn free the stage.
      bool prefetched = false;
      if (it + 1 < n_it) {
        prefetched = __all_sync(0xffffffffu, mbar_test_wait(dp_full, (tn + 1) & 1));
        if (prefetched) {
          tc_fence_after_sync();
          tmem_ld32(tSl, rs0);
          tmem_ld32(tDl, rd0);
        }
      }
      // the dV, dK and dQ products of the query tile that used this buffer pair last have read P and dS
      if (tn >= (uint32_t)Cfg::NBUF)
        mbar_wait(pds_free + 8 * (tn % Cfg::NBUF), (tn / Cfg::NBUF - 1) & 1, abort_flag, a.status);
      if (it == 0 && staged_out) {  // the previous item's epilogue tiles have left the P tile
        if (threadIdx.x == 0) bulk_wait_group_read0();
        __syncwarp();
        asm volatile("bar.sync 5, 256;" ::: "memory");
      }
      const uint32_t pb = (tn % Cfg::NBUF) * Cfg::PDS_STRIDE;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint32_t o0 = pb + tile_chunk_offset<128>(row, wg * 64 + g * 8),
                       o1 = pb + tile_chunk_offset<128>(row, wg * 64 + 32 + g * 8);
        st_shared_v4(sP + o0, pk0[g * 4], pk0[g * 4 + 1], pk0[g * 4 + 2], pk0[g * 4 + 3]);
        st_shared_v4(sDS + o0, dk0[g * 4], dk0[g * 4 + 1], dk0[g * 4 + 2], dk0[g * 4 + 3]);
        st_shared_v4(sP + o1, pk1[g * 4], pk1[g * 4 + 1], pk1[g * 4 + 2], pk1[g * 4 + 3]);
        st_shared_v4(sDS + o1, dk1[g * 4], dk1[g * 4 + 1], dk1[g * 4 + 2], dk1[g * 4 + 3]);
      }
      if (RP) {
        // four buffers: the drain warpgroup may lag up to three query tiles behind
        float* s_rowsum = reinterpret_cast<float*>(smem + Cfg::OFF_ROWSUM) + (tn & 3) * 512;
        s_rowsum[(2 * wg) * 128 + row] = ds_sum0;
        s_rowsum[(2 * wg + 1) * 128 + row] = ds_sum1;
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(pds_ready + 8 * (tn & 1));
      if (it + 1 < n_it && !prefetched) {
        mbar_wait(dp_full, (tn + 1) & 1, abort_flag, a.status);
        tc_fence_after_sync();
        tmem_ld32(tSl, rs0);
        tmem_ld32(tDl, rd0);
      }
    }
    // the dV and dK|dKb accumulators are final once every MMA of the CTA has completed
    mbar_wait(all_done, n & 1, abort_flag, a.status);
    tc_fence_after_sync();

    // ---- epilogue: dV, dK (x scale), dKb.  The tiles are staged in the (now idle) P tile -- dV, dK as the 16-bit
    // [128][D] tiles a TMA store takes, dk_bias rank-major as fp32 -- and leave through the copy engine: one tile
    // store each for dV and dK (whole rows; per-thread stores would touch 32 lines per instruction) and one bulk
    // reduction for dk_bias (other (batch, head) pairs add to the same rows when the factor is shared).
    static_assert(2 * Cfg::D_BYTES + 128 * (RPX / 2) * 4 <= Cfg::TILE128 || !RP, "epilogue staging");
    {
#pragma unroll 1
      for (int c0 = wg * DH; c0 < wg * DH + DH; c0 += 16) {
        uint32_t rv[16], rk[16];
        tmem_ld16(tmem + Cfg::T_DV + lane_off + c0, rv);
        tmem_ld16(tmem + Cfg::T_DK + lane_off + c0, rk);
        tmem_wait_ld(rv);
        tmem_wait_ld(rk);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t off = tile_chunk_offset<D>(row, c0 + g * 8);
          st_shared_v4(sP + off, Pack2<T>::pack(__uint_as_float(rv[g * 8 + 0]), __uint_as_float(rv[g * 8 + 1])),
                       Pack2<T>::pack(__uint_as_float(rv[g * 8 + 2]), __uint_as_float(rv[g * 8 + 3])),
                       Pack2<T>::pack(__uint_as_float(rv[g * 8 + 4]), __uint_as_float(rv[g * 8 + 5])),
                       Pack2<T>::pack(__uint_as_float(rv[g * 8 + 6]), __uint_as_float(rv[g * 8 + 7])));
          st_shared_v4(sP + Cfg::D_BYTES + off,
                       Pack2<T>::pack(__uint_as_float(rk[g * 8 + 0]) * a.dk_scale, __uint_as_float(rk[g * 8 + 1]) * a.dk_scale),
                       Pack2<T>::pack(__uint_as_float(rk[g * 8 + 2]) * a.dk_scale, __uint_as_float(rk[g * 8 + 3]) * a.dk_scale),
                       Pack2<T>::pack(__uint_as_float(rk[g * 8 + 4]) * a.dk_scale, __uint_as_float(rk[g * 8 + 5]) * a.dk_scale),
                       Pack2<T>::pack(__uint_as_float(rk[g * 8 + 6]) * a.dk_scale, __uint_as_float(rk[g * 8 + 7]) * a.dk_scale));
        }
      }
    }
    if (RP && wg == 0) {
      float* stg = reinterpret_cast<float*>(smem + Cfg::OFF_P + 2 * Cfg::D_BYTES) + row;
      const int used = a.R;
#pragma unroll 1
      for (int c0 = 0; c0 < RPX && c0 < used; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem + Cfg::T_DKB + lane_off + c0, r);
        tmem_wait_ld(r);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (c0 + i < used) stg[(c0 + i) * 128] = __uint_as_float(r[i]) * a.dkb_scale;
      }
    }
    // the accumulators may be overwritten by the next item's products
    tc_fence_before_sync();
    mbar_arrive_warp(acc_free);
    fence_proxy_async_smem();  // the staged tiles become visible to the copy engine
    asm volatile("bar.sync 5, 256;" ::: "memory");  // both compute warpgroups
    if (threadIdx.x == 0) {
      tma_store_4d(&tmDV, sP, 0, k0, h, b);
      tma_store_4d(&tmDK, sP + Cfg::D_BYTES, 0, k0, h, b);
      if (RP) {
        const int bk = a.bk_bcast ? 0 : b, hk = a.hk_bcast ? 0 : h;
        bulk_reduce_add_f32(a.dkb_acc + (bh % a.dkb_slots) * a.dkb_slot_stride +
                                (((int64_t)bk * a.Hk + hk) * a.nk_tiles + kt) * (128 * a.R),
                            sP + 2 * Cfg::D_BYTES, 128 * a.R * 4);
      }
      bulk_commit_group();
      // (the reads of the staged tiles are awaited before the next stores into the P tile, or at the end)
    }
    staged_out = true;
    ++n;
    }
    // the staged tiles must outlive the copy engine's reads; the global side completes with the kernel
    if (staged_out && threadIdx.x == 0) bulk_wait_group_read0();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 13) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}


template <typename T, int D, int RP, int NQ, int MODE>
int launch_bwd_p(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  using Cfg = BwdCfg<D, RP, NQ>;
  if constexpr (!Cfg::FITS) {
    return FB_ENOTBUILT;
  } else {
    int rc;
    cudaError_t e;
    BwdLaunch L;
    if ((rc = bwd_prepare<T, D, RP, NQ>(p, plan, st, L))) return rc;
    const BwdArgs& a = L.a;
    BwdPArgs pa;
    pa.total_items = (int)((int64_t)a.nk_tiles * p->B * p->H);
    pa.active_items = (p->causal && a.nq_tiles < a.nk_tiles ? a.nq_tiles : a.nk_tiles) * p->B * p->H;
    fast_div_magic(p->B * p->H, pa.div_bh);
    fast_div_magic(a.nk_tiles, pa.div_nk);
    fast_div_magic(p->H, pa.div_h);
    CUtensorMap tDK, tDV;  // dK and dV leave through tile stores
    if ((rc = make_tmap_4d(&tDK, p->dk, D, p->Sk, p->H, p->B, p->dk_stride[2], p->dk_stride[1], p->dk_stride[0], D, 128)))
      return rc;
    if ((rc = make_tmap_4d(&tDV, p->dv, D, p->Sk, p->H, p->B, p->dv_stride[2], p->dv_stride[1], p->dv_stride[0], D, 128)))
      return rc;
    auto kern = bwd_p_sm100_kernel<T, D, RP, NQ, MODE>;
    // per kernel instantiation and device: raise the dynamic shared-memory limit once
    static std::mutex mu;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    {
      std::lock_guard<std::mutex> lk(mu);
      if (!attr_done[dev & 63]) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        if (e != cudaSuccess) return (int)e;
        attr_done[dev & 63] = true;
      }
    }
    const int sms = device_sm_count(dev);
    if (sms <= 0) return FB_ENOTBUILT;
    // one CTA per SM (or fewer, if there are fewer work items)
    const unsigned grid = (unsigned)(pa.total_items < sms ? pa.total_items : sms);
    prof_before(KC_BWD_MAIN, st);
    kern<<<grid, 512, Cfg::SMEM, st>>>(L.tQ, L.tK, L.tV, L.tDO, L.tQb, L.tKb, L.tKc, L.tKs, tDK, tDV, a, pa);
    prof_after(KC_BWD_MAIN, st);
    note_launch();
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
    return bwd_finish<T, D, RP, NQ>(p, L, st);
  }
}

}  // namespace fb
