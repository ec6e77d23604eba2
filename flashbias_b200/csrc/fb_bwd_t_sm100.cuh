// Backward FlashBias attention for sm_100a, key-major ("transposed") form, for problems without factor operands
// (no bias, an additive mask tensor, or the fused ALiBi producer) at head_dim 32.
//
// At head_dim 32 the backward is bound by shared-memory bandwidth (128 bytes per clock feed both the tensor
// core's operand fetches and the threads' stores): in the query-major kernel of fb_bwd_sm100.cuh every query
// tile moves 64 KB of P / dS stores and ~150 KB of operand fetches.  Here the logits are computed transposed,
//     S^T = K.Q^T        dP^T = V.dO^T          (lane = key, column = query)
// so that P^T and dS^T are already the A operands of
//     dV += P^T.dO       dK += dS^T.Q
// and stay in TENSOR MEMORY (written by the threads with tcgen05.st, read by the MMA without any shared-memory
// fetch); only dS^T also goes to shared memory, as the (transposed) A operand of dQ = dS.K.  That removes the P
// stores and the A-operand fetches of two of the three product chains: ~120 KB per query tile instead of ~216 KB.
// The row statistics (lse, delta) belong to the columns now, where a thread cannot hold them in a register.  They are
// folded into the accumulators by the tensor core instead: one more 16-wide contraction step adds
// -lse_i * log2(e) / (scale * log2 e) to every element of column i of S^T and -delta_i to column i of dP^T (each
// value as three 16-bit terms, so nothing is lost), and the per-element arithmetic shrinks to
//     P^T = exp2(c * S^T')      dS^T = P^T * dP^T'.
//
// One CTA (512 threads) per tile of 128 keys of one (batch, head); K and V resident in shared memory, dV and dK
// accumulators resident in tensor memory (no atomics), loop over the query tiles that see those keys:
//   warps 0-7   two compute warpgroups, thread = key (TMEM lane), each warpgroup half of the query columns
//   warps 8-11  drain warpgroup: dQ tile from TMEM through a staging tile into the fp32 accumulator in global
//               memory with one bulk reduction per query tile (thread = query row)
//   warp 12     TMA producer (Q, dO tiles through a 3-stage ring) and issuer of the dQ chain
//   warps 13-15 MMA issuers: S^T and dP^T; dV; dK
#pragma once

#include "fb_bwd_sm100.cuh"

namespace fb {

template <int D>
struct BwdTCfg {
  static constexpr int D_BYTES = tile_bytes(D);
  static constexpr int AUX_BYTES = tile_bytes(16);  // [128][16] tiles of the extra contraction step
  // resident: K, V and the two constant key-side tiles of the extra step (ones in columns 0-2 / 3-5)
  static constexpr int OFF_K = 0, OFF_V = D_BYTES, OFF_ES = 2 * D_BYTES, OFF_ED = OFF_ES + AUX_BYTES;
  static constexpr int KV_BYTES = 2 * D_BYTES;  // bytes that arrive by TMA
  // one stage: Q, dO (TMA) and the query-side tile of the extra step (written by threads)
  static constexpr int OFF_DO = D_BYTES, OFF_AUX = 2 * D_BYTES, TMA_STAGE_BYTES = 2 * D_BYTES;
  static constexpr int STAGE_BYTES = TMA_STAGE_BYTES + AUX_BYTES;
  static constexpr int NSTAGE = 3;
  static constexpr int OFF_STAGE = OFF_ED + AUX_BYTES;
  static constexpr int TILE128 = tile_bytes(128);
  static constexpr int OFF_DS = OFF_STAGE + NSTAGE * STAGE_BYTES;  // dS^T tile, [128 keys][128 queries]
  static constexpr int OFF_STG = OFF_DS + TILE128;                 // fp32 dQ staging tile
  static constexpr int OFF_BAR = OFF_STG + 128 * D * 4;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;
  // tensor memory: S^T fp32 [0,128), dP^T fp32 [128,256), P^T 16-bit pairs [256,320), dS^T pairs [320,384),
  // dV [384, 384+D), dK, then two dQ accumulators
  static constexpr int T_ST = 0, T_DPT = 128, T_PT = 256, T_DST = 320, T_DV = 384, T_DK = T_DV + D, T_DQ = T_DK + D;
  static constexpr int NDQ = (T_DQ + 2 * D <= 512) ? 2 : 1;
  static constexpr bool FITS = SMEM <= 227 * 1024 && T_DQ + D <= 512;
};

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(512, 1)
bwd_t_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const BwdArgs a) {
  using Cfg = BwdTCfg<D>;
  constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase + Cfg::OFF_K, sV = sbase + Cfg::OFF_V, sStage = sbase + Cfg::OFF_STAGE,
                 sDS = sbase + Cfg::OFF_DS, sStg = sbase + Cfg::OFF_STG, sES = sbase + Cfg::OFF_ES, sED = sbase + Cfg::OFF_ED;
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  const uint32_t kv_full = bar0, dp_full = bar0 + 16, sdp_read = bar0 + 24,
                 dq_full = bar0 + 32 /*2*/, qdo_full = bar0 + 48 /*3*/, qdo_free = bar0 + 72 /*3*/,
                 all_done = bar0 + 112, pds_free = bar0 + 120, pds_ready = bar0 + 136 /*2*/,
                 dq_drained = bar0 + 152 /*2*/, aux_ready = bar0 + 168 /*3*/;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::OFF_BAR + 104);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int BH = a.B * a.H;
  int kt, bh;
  if (a.causal) {  // key tile 0 sees the most query tiles: heaviest first
    kt = (int)(blockIdx.x / BH);
    bh = (int)(blockIdx.x % BH);
  } else {
    kt = (int)(blockIdx.x % a.nk_tiles);
    bh = (int)(blockIdx.x / a.nk_tiles);
  }
  const int b = bh / a.H, h = bh % a.H;
  const int k0 = kt * 128;
  const int i_begin = a.causal ? kt : 0;  // first query tile with a row >= k0
  const int n_it = a.nq_tiles - i_begin;  // may be <= 0 when Sq < Sk under causal masking

  // producer thread only: one stage of the query-tile ring
  auto load_tile = [&](int it) {
    const int st = it % Cfg::NSTAGE;
    const uint32_t base = sStage + st * Cfg::STAGE_BYTES;
    mbar_expect_tx(qdo_full + 8 * st, Cfg::TMA_STAGE_BYTES);
    const int q0 = (i_begin + it) * 128;
    tma_tile_bwd<D>(base, &tmQ, qdo_full + 8 * st, q0, h, b);
    tma_tile_bwd<D>(base + Cfg::OFF_DO, &tmDO, qdo_full + 8 * st, q0, h, b);
  };

  if (warp == 12) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(kv_full, 1);
      mbar_init(dp_full, 1);
      mbar_init(sdp_read, 8);   // every compute warp has S^T and dP^T of the tile in registers
      mbar_init(all_done, 4);   // one commit per issuing thread
      mbar_init(pds_free, 3);   // the dV, dK and dQ chains have read P^T and dS^T of a query tile
      for (int i = 0; i < 3; ++i) {
        mbar_init(qdo_full + 8 * i, 1);
        mbar_init(qdo_free + 8 * i, 3);  // S^T|dP^T, dV and dK chains read a stage
        mbar_init(aux_ready + 8 * i, 4);  // the first compute warpgroup has written the stage's statistics tile
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(dq_full + 8 * i, 1);
        mbar_init(dq_drained + 8 * i, 4);  // the drain warps
        mbar_init(pds_ready + 8 * i, 8);   // the compute warps; alternating by query tile
      }
      mbar_fence_init();
      if (n_it > 0) {
        mbar_expect_tx(kv_full, Cfg::KV_BYTES);
        tma_tile_bwd<D>(sK, &tmK, kv_full, k0, h, b);
        tma_tile_bwd<D>(sV, &tmV, kv_full, k0, h, b);
        for (int it = 0; it < Cfg::NSTAGE && it < n_it; ++it) load_tile(it);
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

  if (warp >= 12) {
    setmaxnreg_dec<64>();
    if (lane == 0 && n_it > 0) {
      // B operands read transposed (MN-major: rows are the contraction index), A of dQ likewise
      constexpr uint32_t idS = instr_desc(kBf16, false, false, 128, 128);  // S^T, dP^T: both operands K-major
      constexpr uint32_t idTS = instr_desc(kBf16, false, true, 128, D);    // dV, dK: A in TMEM, B MN-major
      constexpr uint32_t idQ = instr_desc(kBf16, true, true, 128, D);      // dQ: A = dS (transposed tile), B = K
      mbar_wait(kv_full, 0, abort_flag, a.status);
      tc_fence_after_sync();
      if (warp == 12) {
        // ------------------------------------------------------------------ TMA producer, dQ chain
        const DescBase mDS = mnmajor_base<128>(sDS), mK = mnmajor_base<D>(sK);
#pragma unroll 1
        for (int it = 0; it < n_it; ++it) {
          const int qb = it % Cfg::NDQ;
          mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
          if (it >= Cfg::NDQ)  // the drain warpgroup has read the tile that used this accumulator last
            mbar_wait(dq_drained + 8 * qb, (it / Cfg::NDQ - 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int s = 0; s < 8; ++s)  // contraction over the 128 keys
            umma_ss(tmem + Cfg::T_DQ + qb * D, desc_at(mDS, mnmajor_step<128>(s)), desc_at(mK, mnmajor_step<D>(s)),
                    idQ, s > 0);
          umma_commit(dq_full + 8 * qb);
          umma_commit(pds_free);
          if (it + Cfg::NSTAGE < n_it) {  // the S^T|dP^T, dV and dK chains have finished reading the stage of tile it
            mbar_wait(qdo_free + 8 * (it % Cfg::NSTAGE), (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
            load_tile(it + Cfg::NSTAGE);
          }
        }
      } else if (warp == 13) {
        // ------------------------------------------------------------------ S^T = K.Q^T, dP^T = V.dO^T
        const DescBase kK = kmajor_base<D>(sK), kV = kmajor_base<D>(sV), kQ = kmajor_base<D>(sStage),
                       kDO = kmajor_base<D>(sStage + Cfg::OFF_DO), kES = kmajor_base<16>(sES),
                       kED = kmajor_base<16>(sED), kAux = kmajor_base<16>(sStage + Cfg::OFF_AUX);
#pragma unroll 1
        for (int it = 0; it < n_it; ++it) {
          const int st = it % Cfg::NSTAGE;
          const uint32_t so = st * Cfg::STAGE_BYTES;
          if (it > 0) {  // the compute warps hold S^T and dP^T of the previous tile in registers
            mbar_wait(sdp_read, (it - 1) & 1, abort_flag, a.status);
            tc_fence_after_sync();
          }
          mbar_wait(qdo_full + 8 * st, (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          mbar_wait(aux_ready + 8 * st, (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int s = 0; s < D / 16; ++s)
            umma_ss(tmem + Cfg::T_ST, desc_at(kK, kmajor_step<D>(s)), desc_at(kQ, so + kmajor_step<D>(s)), idS, s > 0);
          umma_ss(tmem + Cfg::T_ST, desc_at(kES, 0), desc_at(kAux, so), idS, 1u);  // + (-lse2_i / c) per column
#pragma unroll
          for (int s = 0; s < D / 16; ++s)
            umma_ss(tmem + Cfg::T_DPT, desc_at(kV, kmajor_step<D>(s)), desc_at(kDO, so + kmajor_step<D>(s)), idS,
                    s > 0);
          umma_ss(tmem + Cfg::T_DPT, desc_at(kED, 0), desc_at(kAux, so), idS, 1u);  // + (-delta_i) per column
          umma_commit(dp_full);
          umma_commit(qdo_free + 8 * st);
        }
      } else {
        // ------------------------------------------------------------------ dV += P^T.dO (14), dK += dS^T.Q (15)
        const DescBase mB = mnmajor_base<D>(warp == 14 ? sStage + Cfg::OFF_DO : sStage);
        const uint32_t tA = tmem + (warp == 14 ? Cfg::T_PT : Cfg::T_DST);
        const uint32_t tD = tmem + (warp == 14 ? Cfg::T_DV : Cfg::T_DK);
#pragma unroll 1
        for (int it = 0; it < n_it; ++it) {
          const int st = it % Cfg::NSTAGE;
          const uint32_t so = st * Cfg::STAGE_BYTES;
          mbar_wait(qdo_full + 8 * st, (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int s = 0; s < 8; ++s)  // contraction over the 128 query rows; A: 8 TMEM columns per 16 rows
            umma_ts(tD, tA + s * 8, desc_at(mB, so + mnmajor_step<D>(s)), idTS, (it > 0 || s > 0) ? 1u : 0u);
          umma_commit(qdo_free + 8 * st);
          umma_commit(pds_free);
        }
      }
      umma_commit(all_done);  // every MMA of this thread
    }
  } else if (warp >= 8) {
    setmaxnreg_dec<64>();
    // ------------------------------------------------------------------ drain warpgroup (thread = query row)
    if (n_it > 0) {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int qb = it % Cfg::NDQ;
        const uint32_t tq = tmem + Cfg::T_DQ + qb * D + lane_off;
        mbar_wait(dq_full + 8 * qb, (it / Cfg::NDQ) & 1, abort_flag, a.status);
        tc_fence_after_sync();
        // The first columns are fetched into registers while the copy engine may still be reading the previous
        // tile from the staging tile; the thread that issued that reduction then waits for its shared-memory
        // reads and the warpgroup syncs.
        uint32_t r0[16], r1[16];
        tmem_ld16(tq, r0);
        tmem_ld16(tq + 16, r1);
        if (warp == 8 && lane == 0) bulk_wait_group_read0();
        __syncwarp();
        asm volatile("bar.sync 3, 128;" ::: "memory");  // the drain warpgroup only
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          if (c0 > 0) {
            tmem_ld16(tq + c0, r0);
            tmem_ld16(tq + c0 + 16, r1);
          }
          tmem_wait_ld(r0);
          tmem_wait_ld(r1);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            st_shared_v4(sStg + dq_stage_off(row, c0 / 4 + g), r0[g * 4], r0[g * 4 + 1], r0[g * 4 + 2], r0[g * 4 + 3]);
            st_shared_v4(sStg + dq_stage_off(row, c0 / 4 + 4 + g), r1[g * 4], r1[g * 4 + 1], r1[g * 4 + 2],
                         r1[g * 4 + 3]);
          }
        }
        tc_fence_before_sync();
        mbar_arrive_warp(dq_drained + 8 * qb);  // every tensor-memory read of the tile is done
        fence_proxy_async_smem();               // the staged tile becomes visible to the copy engine
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (warp == 8 && lane == 0) {
          bulk_reduce_add_f32(a.dq_acc + ((int64_t)bh * a.nq_tiles + (i_begin + it)) * (128 * D), sStg, 128 * D * 4);
          bulk_commit_group();
        }
      }
      // the staging tile must outlive the last reduction's reads; its global side completes with the kernel
      if (warp == 8 && lane == 0) bulk_wait_group_read0();
    }
  } else if (n_it > 0) {
    // ------------------------------------------------------------------ compute warpgroups (warps 0-7)
    setmaxnreg_inc<192>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;  // key of this thread within the tile
    const int key = k0 + row;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = a.scale_log2;
    constexpr int DH = D / 2;  // dV / dK columns per warpgroup in the epilogue
    float slope2 = 0.f, akey = 0.f;  // ALiBi: slope * log2 e, and the key's share of the bias
    if (MODE == BWD_ALIBI) {
      slope2 = __ldg(a.alibi_slopes + h) * kLog2e;
      akey = slope2 * (float)key;
    }
    const char* mcol = nullptr;  // additive mask: this thread's key column of query row 0
    int msize = 4;
    if (MODE == BWD_MASK) {
      msize = a.mask_dtype == FB_DTYPE_F32 ? 4 : 2;
      const int mb = a.mask_batch_period > 0 ? b % a.mask_batch_period : b;
      mcol = reinterpret_cast<const char*>(a.mask) +
             (mb * a.mask_stride[0] + h * a.mask_stride[1] + min(key, a.Sk - 1)) * msize;
    }
    // Row statistics of query tile `it`: threads 0..127 each fetch one query row (raw loads; consumed one tile later,
    // so the latency hides under the arithmetic in between) ...
    auto load_row_stats = [&](int it, float& lse_raw, float& dlt) {
      const int g = (i_begin + it) * 128 + (int)threadIdx.x;
      lse_raw = -INFINITY;  // rows beyond Sq and rows that saw no key: probabilities exactly zero
      dlt = 0.f;
      if (threadIdx.x < 128 && it < n_it && g < a.Sq) {
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(lse_raw) : "l"(a.lse + (int64_t)bh * a.lse_stride_bh + g));
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(dlt) : "l"(a.delta + (int64_t)bh * a.lse_stride_bh + g));
      }
    };
    // ... and write that row of the stage's statistics tile: columns 0-2 hold x = -lse2_i / (32 c) as three 16-bit
    // terms (the key-side tile has 32 in those columns: 32 x is added to column i of S^T, and c S^T' = c S^T - lse2_i),
    // columns 3-5 hold -delta_i likewise (key-side tile: 1).  With the ALiBi producer the query's share of the bias,
    // -slope2 * i, rides along with -lse2_i.  -inf is replaced by the most negative finite value of the type.
    auto split3 = [](float x, T& hi, T& mid, T& lo) {
      hi = from_f32<T>(x);
      const float r1 = x - to_f32(hi);
      mid = from_f32<T>(r1);
      lo = from_f32<T>(r1 - to_f32(mid));
    };
    auto store_row_stats = [&](int it, float lse_raw, float dlt) {
      if (threadIdx.x < 128) {
        const int g = (i_begin + it) * 128 + (int)threadIdx.x;
        const float kMostNeg = kBf16 ? -1e30f : -6e4f;
        float x = kMostNeg;
        if (lse_raw != -INFINITY) {
          float nl = -lse_raw * kLog2e;
          if (MODE == BWD_ALIBI) nl -= slope2 * (float)g;
          x = fmaxf(nl / (32.f * sl2), kMostNeg);
        }
        uint4 w = make_uint4(0u, 0u, 0u, 0u);
        T* e = reinterpret_cast<T*>(&w);
        split3(x, e[0], e[1], e[2]);
        split3(-dlt, e[3], e[4], e[5]);
        const uint32_t base = sStage + (it % Cfg::NSTAGE) * Cfg::STAGE_BYTES + Cfg::OFF_AUX;
        st_shared_v4(base + tile_chunk_offset<16>((int)threadIdx.x, 0), w.x, w.y, w.z, w.w);
        st_shared_v4(base + tile_chunk_offset<16>((int)threadIdx.x, 8), 0u, 0u, 0u, 0u);
      }
      if (wg == 0) {
        fence_proxy_async_smem();
        mbar_arrive_warp(aux_ready + 8 * (it % Cfg::NSTAGE));
      }
    };

    if (threadIdx.x < 128) {  // the constant key-side tiles of the extra contraction step
      uint4 ws = make_uint4(0u, 0u, 0u, 0u), wd = make_uint4(0u, 0u, 0u, 0u);
      T* es = reinterpret_cast<T*>(&ws);
      T* ed = reinterpret_cast<T*>(&wd);
      for (int i = 0; i < 3; ++i) {
        es[i] = from_f32<T>(32.f);
        ed[3 + i] = from_f32<T>(1.f);
      }
      st_shared_v4(sES + tile_chunk_offset<16>((int)threadIdx.x, 0), ws.x, ws.y, ws.z, ws.w);
      st_shared_v4(sES + tile_chunk_offset<16>((int)threadIdx.x, 8), 0u, 0u, 0u, 0u);
      st_shared_v4(sED + tile_chunk_offset<16>((int)threadIdx.x, 0), wd.x, wd.y, wd.z, wd.w);
      st_shared_v4(sED + tile_chunk_offset<16>((int)threadIdx.x, 8), 0u, 0u, 0u, 0u);
    }
    float lse_raw, dlt;
    load_row_stats(0, lse_raw, dlt);
    store_row_stats(0, lse_raw, dlt);
    load_row_stats(1, lse_raw, dlt);
    uint32_t rs0[32], rd0[32], rs1[32], rd1[32];
    const uint32_t tSl = tmem + Cfg::T_ST + lane_off + wg * 64, tDl = tmem + Cfg::T_DPT + lane_off + wg * 64;
    mbar_wait(dp_full, 0, abort_flag, a.status);  // committed after the S^T and the dP^T products: covers both
    tc_fence_after_sync();
    tmem_ld32(tSl, rs0);
    tmem_ld32(tDl, rd0);
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
      const int q0 = (i_begin + it) * 128;
      const bool need_mask = (a.causal && k0 + 127 > q0) || (k0 + 128 > a.Sk);
      // the next tile's statistics tile (its stage was last read two tiles ago); the S^T|dP^T products of that tile
      // wait for it
      if (it + 1 < n_it) store_row_stats(it + 1, lse_raw, dlt);
      load_row_stats(it + 2, lse_raw, dlt);
      tmem_ld32(tSl + 32, rs1);
      tmem_ld32(tDl + 32, rd1);
      tmem_wait_ld(rs0);
      tmem_wait_ld(rd0);
      tmem_wait_ld(rs1);
      tmem_wait_ld(rd1);
      tc_fence_before_sync();
      mbar_arrive_warp(sdp_read);
      // P^T and dS^T of the tile stay in registers as packed 16-bit pairs until both chunks are done: the tensor
      // memory and shared-memory tiles are still being read by the products of the previous tile
      auto chunk = [&](uint32_t (&rs)[32], uint32_t (&rd)[32], uint32_t (&pk)[16], uint32_t (&dk)[16], int c) {
        const int col0 = wg * 64 + c * 32;  // first query column of the chunk
        const uint64_t sl2p = f2(sl2, sl2), akp = f2(akey, akey);
        float mv[32];
        if (MODE == BWD_MASK) {
          // one element per query row; the 32 lanes of a warp read 32 consecutive keys of that row
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int q = min(q0 + col0 + i, a.Sq - 1);
            const char* p = mcol + (int64_t)q * a.mask_stride[2] * msize;
            mv[i] = (a.mask_dtype == FB_DTYPE_F32   ? __ldg(reinterpret_cast<const float*>(p))
                     : a.mask_dtype == FB_DTYPE_F16 ? __half2float(__ldg(reinterpret_cast<const __half*>(p)))
                                                    : __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(p)))) *
                    kLog2e;
          }
        }
        auto elems = [&](auto masked) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t sp = f2(__uint_as_float(rs[i]), __uint_as_float(rs[i + 1]));
            float a0, a1;
            f2_unpack(MODE == BWD_ALIBI  ? f2_fma(sp, sl2p, akp)
                      : MODE == BWD_MASK ? f2_fma(sp, sl2p, f2(mv[i], mv[i + 1]))
                                         : f2_mul(sp, sl2p),
                      a0, a1);
            float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
            if (decltype(masked)::value) {
              const int q = q0 + col0 + i;
              if (key >= a.Sk || (a.causal && key > q)) p0 = 0.f;
              if (key >= a.Sk || (a.causal && key > q + 1)) p1 = 0.f;
            }
            const uint64_t ds = f2_mul(f2(p0, p1), f2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1])));
            float d0, d1;
            f2_unpack(ds, d0, d1);
            pk[i / 2] = Pack2<T>::pack(p0, p1);
            dk[i / 2] = Pack2<T>::pack(d0, d1);
          }
        };
        if (need_mask) elems(std::true_type{}); else elems(std::false_type{});
      };
      uint32_t pk0[16], pk1[16], dk0[16], dk1[16];
      chunk(rs0, rd0, pk0, dk0, 0);
      chunk(rs1, rd1, pk1, dk1, 1);
      // Chunk 0 of the next tile is fetched under the stores below if its S^T and dP^T are already there.
      bool prefetched = false;
      if (it + 1 < n_it) {
        prefetched = __all_sync(0xffffffffu, mbar_test_wait(dp_full, (it + 1) & 1));
        if (prefetched) {
          tc_fence_after_sync();
          tmem_ld32(tSl, rs0);
          tmem_ld32(tDl, rd0);
        }
      }
      // the dV, dK and dQ products of the previous query tile have read P^T and dS^T
      if (it >= 1) mbar_wait(pds_free, (it - 1) & 1, abort_flag, a.status);
      tc_fence_after_sync();
      // P^T and dS^T into tensor memory (A operands of dV and dK) ...
      tmem_st16(tmem + Cfg::T_PT + lane_off + wg * 32, pk0);
      tmem_st16(tmem + Cfg::T_PT + lane_off + wg * 32 + 16, pk1);
      tmem_st16(tmem + Cfg::T_DST + lane_off + wg * 32, dk0);
      tmem_st16(tmem + Cfg::T_DST + lane_off + wg * 32 + 16, dk1);
      // ... and dS^T into shared memory as well (A operand of dQ, read transposed)
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        st_shared_v4(sDS + tile_chunk_offset<128>(row, wg * 64 + g * 8), dk0[g * 4], dk0[g * 4 + 1], dk0[g * 4 + 2],
                     dk0[g * 4 + 3]);
        st_shared_v4(sDS + tile_chunk_offset<128>(row, wg * 64 + 32 + g * 8), dk1[g * 4], dk1[g * 4 + 1],
                     dk1[g * 4 + 2], dk1[g * 4 + 3]);
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive_warp(pds_ready + 8 * (it & 1));
      if (it + 1 < n_it && !prefetched) {
        mbar_wait(dp_full, (it + 1) & 1, abort_flag, a.status);
        tc_fence_after_sync();
        tmem_ld32(tSl, rs0);
        tmem_ld32(tDl, rd0);
      }
    }
    // the dV and dK accumulators are final once every MMA of the CTA has completed
    mbar_wait(all_done, 0, abort_flag, a.status);
    tc_fence_after_sync();

    // ---- epilogue: dV, dK (x scale); thread = key row, each warpgroup half of the columns
    {
      T* dvrow = reinterpret_cast<T*>(a.dv) + b * a.dv_stride[0] + h * a.dv_stride[1] + (int64_t)key * a.dv_stride[2];
      T* dkrow = reinterpret_cast<T*>(a.dk) + b * a.dk_stride[0] + h * a.dk_stride[1] + (int64_t)key * a.dk_stride[2];
#pragma unroll 1
      for (int c0 = wg * DH; c0 < wg * DH + DH; c0 += 16) {
        uint32_t rv[16], rk[16];
        tmem_ld16(tmem + Cfg::T_DV + lane_off + c0, rv);
        tmem_ld16(tmem + Cfg::T_DK + lane_off + c0, rk);
        tmem_wait_ld(rv);
        tmem_wait_ld(rk);
        if (key < a.Sk) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            uint4 wv, wk;
            wv.x = Pack2<T>::pack(__uint_as_float(rv[g * 8 + 0]), __uint_as_float(rv[g * 8 + 1]));
            wv.y = Pack2<T>::pack(__uint_as_float(rv[g * 8 + 2]), __uint_as_float(rv[g * 8 + 3]));
            wv.z = Pack2<T>::pack(__uint_as_float(rv[g * 8 + 4]), __uint_as_float(rv[g * 8 + 5]));
            wv.w = Pack2<T>::pack(__uint_as_float(rv[g * 8 + 6]), __uint_as_float(rv[g * 8 + 7]));
            wk.x = Pack2<T>::pack(__uint_as_float(rk[g * 8 + 0]) * a.dk_scale, __uint_as_float(rk[g * 8 + 1]) * a.dk_scale);
            wk.y = Pack2<T>::pack(__uint_as_float(rk[g * 8 + 2]) * a.dk_scale, __uint_as_float(rk[g * 8 + 3]) * a.dk_scale);
            wk.z = Pack2<T>::pack(__uint_as_float(rk[g * 8 + 4]) * a.dk_scale, __uint_as_float(rk[g * 8 + 5]) * a.dk_scale);
            wk.w = Pack2<T>::pack(__uint_as_float(rk[g * 8 + 6]) * a.dk_scale, __uint_as_float(rk[g * 8 + 7]) * a.dk_scale);
            *reinterpret_cast<uint4*>(dvrow + c0 + g * 8) = wv;
            *reinterpret_cast<uint4*>(dkrow + c0 + g * 8) = wk;
          }
        }
      }
    }
  } else {
    // causal with Sq < Sk: these keys are seen by no query; their gradients are zero
    const int wg = warp >> 2;
    const int krow = k0 + (warp & 3) * 32 + lane;
    if (krow < a.Sk) {
      T* dvrow = reinterpret_cast<T*>(a.dv) + b * a.dv_stride[0] + h * a.dv_stride[1] + (int64_t)krow * a.dv_stride[2];
      T* dkrow = reinterpret_cast<T*>(a.dk) + b * a.dk_stride[0] + h * a.dk_stride[1] + (int64_t)krow * a.dk_stride[2];
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int c0 = wg * (D / 2); c0 < wg * (D / 2) + D / 2; c0 += 8) {
        *reinterpret_cast<uint4*>(dvrow + c0) = z;
        *reinterpret_cast<uint4*>(dkrow + c0) = z;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 13) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <typename T, int D, int MODE>
int launch_bwd_t_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  using Cfg = BwdTCfg<D>;
  static_assert(Cfg::FITS, "key-major backward: tiles exceed one SM");
  int rc;
  const BwdWs w = bwd_layout(p, plan);
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  cudaError_t e = cudaMemsetAsync(ws + w.off_dq, 0, w.zero_bytes, st);
  if (e != cudaSuccess) return (int)e;
  CUtensorMap tQ, tK, tV, tDO;
  if ((rc = make_tmap_4d(&tQ, p->q, D, p->Sq, p->H, p->B, p->q_stride[2], p->q_stride[1], p->q_stride[0], D, 128)))
    return rc;
  if ((rc = make_tmap_4d(&tK, p->k, D, p->Sk, p->H, p->B, p->k_stride[2], p->k_stride[1], p->k_stride[0], D, 128)))
    return rc;
  if ((rc = make_tmap_4d(&tV, p->v, D, p->Sk, p->H, p->B, p->v_stride[2], p->v_stride[1], p->v_stride[0], D, 128)))
    return rc;
  if ((rc = make_tmap_4d(&tDO, p->dout, D, p->Sq, p->H, p->B, p->dout_stride[2], p->dout_stride[1],
                         p->dout_stride[0], D, 128)))
    return rc;
  BwdArgs a = {};
  a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
  a.nq_tiles = (p->Sq + 127) / 128;
  a.nk_tiles = (p->Sk + 127) / 128;
  a.causal = p->causal;
  a.R = 0;
  a.dk_scale = p->softmax_scale;  // dK accumulates dS^T.q
  a.scale_log2 = p->softmax_scale * 1.4426950408889634f;
  a.lse = p->lse;
  a.delta = p->delta;
  a.lse_stride_bh = p->lse_stride_bh;
  a.dq_acc = reinterpret_cast<float*>(ws + w.off_dq);
  a.dk = p->dk;
  a.dv = p->dv;
  for (int i = 0; i < 3; ++i) {
    a.dk_stride[i] = p->dk_stride[i];
    a.dv_stride[i] = p->dv_stride[i];
  }
  a.status = p->status;
  a.mask = p->mask;
  for (int i = 0; i < 3; ++i) a.mask_stride[i] = p->mask_stride[i];
  if (p->mask_kind == FB_MASK_VECTOR) a.mask_stride[2] = 0;
  a.mask_kind = p->mask_kind;
  a.mask_dtype = p->mask_dtype;
  a.mask_batch_period = p->mask_batch_period;
  a.alibi_slopes = p->alibi_slopes;
  auto kern = bwd_t_sm100_kernel<T, D, MODE>;
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
  const unsigned grid = (unsigned)((int64_t)a.nk_tiles * p->B * p->H);
  prof_before(KC_BWD_MAIN, st);
  kern<<<grid, 512, Cfg::SMEM, st>>>(tQ, tK, tV, tDO, a);
  prof_after(KC_BWD_MAIN, st);
  note_launch();
  if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  const int64_t n8 = ((int64_t)p->B * p->Sq * p->H * D) / 8;
  dq_store_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(
      a.dq_acc, reinterpret_cast<T*>(p->dq), p->B, p->Sq, p->H, D, p->dq_stride[0], p->dq_stride[1], p->dq_stride[2],
      p->softmax_scale, 1);
  note_launch();
  return (int)cudaGetLastError();
}

}  // namespace fb
