// Backward FlashBias attention for sm_100a.  (Kernel and launcher templates; the instantiations are spread over
// one translation unit per head_dim so that they compile in parallel.)
//
// One CTA (512 threads) owns one tile of 128 keys of one (batch, head): K (and the (hi, lo) split of k*scale
// when the scale is not a power of two), the packed k_bias tiles and V stay resident in shared memory, the
// dK|dk_bias and dV accumulators stay resident in tensor memory (no atomics on them), and the CTA walks the
// query tiles that see those keys:
//   warp 12     TMA producer: resident tiles once, then Q|Qb|dO tiles through a 2- or 3-stage ring; the same
//               thread issues the dQ | dQb MMAs.
//   warps 13-15 MMA issuers (one thread each, every warp on its own warp scheduler), per query tile:
//                 13: S  = [Q|Qb].[K|Kb]^T      dP = dO.V^T                     (TMEM, fresh)
//                     (and dKb += dS^T.Qb when it is not merged into the dK product)
//                 14: dV += P^T.dO              15: dK|dKb += dS^T.[Q|Qb]       (TMEM, accumulated)
//                 12: dQ|dQb = dS.[K|Kc]                                        (TMEM, fresh, two accumulators)
//   warps 0-7   two compute warpgroups, each thread owns one query row (TMEM lane) and half of the key
//               columns: S and dP go to registers (fetched under the previous tile's stores, which releases
//               them for the next tile's MMAs at the head of the tile),
//               P = exp2(S*c - lse*log2e), dS = P*(dP - delta), both rounded to 16 bits and, once the previous
//               tile's products have released them, written to shared memory as operand tiles.
//   warps 8-11  drain warpgroup: the dQ|dQb tile goes from TMEM through a shared-memory staging tile into fp32
//               accumulators in global memory with one bulk reduction each.
// dQ is the only quantity that crosses CTAs (every key tile contributes to every query row), hence
// the fp32 accumulators; a final pass scales and rounds them.  P and dS are read by the tensor core
// both "as stored" and transposed, which is only a different shared-memory descriptor.
#pragma once

#include <mutex>
#include <type_traits>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

struct BwdArgs {
  int B, H, Sq, Sk, nq_tiles, nk_tiles, causal, R;
  int hq_bcast, bq_bcast, hk_bcast, bk_bcast;
  int Hq, Hk;  // head extents of the un-expanded factors
  float dk_scale;    // applied to dK on store
  float dkb_scale;   // applied to dk_bias on store
  float scale_log2;  // logits * log2(e) = S * scale_log2
  const float* lse;
  const float* delta;
  int64_t lse_stride_bh;
  float* dq_acc;   // (B, Sq, H, D) fp32
  float* dqb_acc;  // (slots, Bq, Hq, nq_tiles * 128, R) fp32
  int dqb_slots;   // copies of the dq_bias accumulator; (batch, head) pairs that share a factor use different ones
  int64_t dqb_slot_stride;  // floats per copy
  float* dkb_acc;  // (slots, Bk, Hk, nk_tiles * 128, R) fp32
  int dkb_slots;
  int64_t dkb_slot_stride;
  void* dk;
  void* dv;
  int64_t dk_stride[3], dv_stride[3];
  const void* k_bias;  // original (unpacked) k-side factor and its (batch, head, row) strides
  int64_t kb_stride[3];
  int* status;
  const void* mask;  // additive mask, (batch, head, row) element strides; row stride 0 for a (1, Sk) mask
  int64_t mask_stride[3];
  int mask_kind, mask_dtype, mask_batch_period;
  const float* alibi_slopes;
  template <typename T>
  __device__ __forceinline__ const T* k_bias_t() const { return reinterpret_cast<const T*>(k_bias); }
};

template <int D, int RP, int NQ>
struct BwdCfg {
  static constexpr int RPX = RP ? RP : 16;
  static constexpr int D_BYTES = tile_bytes(D);
  static constexpr int R_BYTES = RP ? tile_bytes(RPX) : 0;
  // centred k-side factor tile: as wide as a head_dim-32 tile, so that [K | Kc] reads as one MMA operand
  static constexpr int RC = RP ? ((D == 32 && RP < 32) ? 32 : RP) : 0;
  static constexpr int RCX = RC ? RC : 16;
  static constexpr int RC_BYTES = RC ? tile_bytes(RCX) : 0;
  // one stage of the query-tile ring: Q, Qb, dO
  static constexpr int OFF_QB = D_BYTES;
  static constexpr int OFF_DO = OFF_QB + R_BYTES;
  static constexpr int STAGE_BYTES = OFF_DO + D_BYTES;
  static constexpr int TILE128 = tile_bytes(128);  // one P or dS tile
  // Operands that share the A tile are read as ONE MN-major B operand of two 32-column blocks (head_dim 32:
  // 64-byte-swizzled tiles at a constant distance), which saves the repeated shared-memory fetch of A:
  //   dK chain:  dS^T . [Q | Qb]   (when Qb is 32 columns wide)        dQ chain:  dS . [K | Kc]
  static constexpr bool MERGE_K = (D == 32 && RP == 32);
  static constexpr bool MERGE_Q = (D == 32 && RC == 32);
  static constexpr bool SEP_DKB = RP && !MERGE_K;  // dKb is an accumulator (and an MMA chain) of its own
  // resident tiles of the key block: K, (hi, lo) of k*scale when the scale is not a power of two, Kb, Kc, V
  static constexpr int OFF_K = 0;
  static constexpr int OFF_KS = OFF_K + D_BYTES;
  static constexpr int OFF_KB = OFF_KS + (NQ == 2 ? 2 * D_BYTES : 0);
  static constexpr int OFF_KC = OFF_KB + R_BYTES;  // centred k_bias tile (dq_bias only)
  static constexpr int OFF_V = OFF_KC + RC_BYTES;
  static constexpr int KV_BYTES = OFF_V + D_BYTES;
  static constexpr int OFF_STAGE = KV_BYTES;
  static constexpr int TAIL_BYTES = 256 + 8192 + 4 * RCX * 4 + 1024;  // barriers, row sums, centre keys, alignment
  // P and dS buffers: the compute warps keep the 16-bit P and dS of a query tile in registers until the tile's
  // arithmetic is done and only then store them.  With one buffer pair (NBUF = 1) they first wait for the products
  // of the previous tile to release it.  Where shared memory allows (head_dim 32 without factor tiles) there are
  // two pairs, used alternately, and the stores of a tile never wait for the products of the previous one.
  // STAGED: a staging tile from which the fp32 dQ tile is reduced into global memory in bulk
  // (and a [128][rank] tile for dq_bias, rank <= RC / 2)
  static constexpr int STG_WANT = 128 * D * 4 + 256 * RC;
  static constexpr int NBUF =
      (KV_BYTES + 4 * TILE128 + TAIL_BYTES + 2 * STAGE_BYTES + STG_WANT <= 227 * 1024) ? 2 : 1;
  static constexpr int PDS_STRIDE = 2 * TILE128;  // bytes between the buffer pairs
  static constexpr int BASE_BYTES = KV_BYTES + NBUF * PDS_STRIDE + TAIL_BYTES;
  static constexpr bool STAGED = BASE_BYTES + 2 * STAGE_BYTES + STG_WANT <= 227 * 1024;
  static constexpr int STG_BYTES = STAGED ? STG_WANT : 0;
  static constexpr int FIXED_BYTES = BASE_BYTES + STG_BYTES;
  // as many stages of the query-tile ring as fit (2 or 3): a load takes longer than the products that free a stage
  static constexpr int NSTAGE = (FIXED_BYTES + 3 * STAGE_BYTES <= 227 * 1024) ? 3 : 2;
  static constexpr int OFF_P = OFF_STAGE + NSTAGE * STAGE_BYTES;
  static constexpr int OFF_DS = OFF_P + TILE128;
  static constexpr int OFF_STG = OFF_P + NBUF * PDS_STRIDE;
  static constexpr int OFF_BAR = OFF_STG + STG_BYTES;
  static constexpr int OFF_ROWSUM = OFF_BAR + 256;   // 4 x 4 x 128 floats: dS row sums per 32-key group
  static constexpr int OFF_KBC = OFF_ROWSUM + 8192;  // 4 x RCX floats: k_bias of the 4 centre keys
  static constexpr int SMEM = FIXED_BYTES + NSTAGE * STAGE_BYTES;
  // tensor-memory columns
  static constexpr int DK_COLS = MERGE_K ? 64 : D;  // dKb sits behind dK when the operands are merged
  static constexpr int T_S = 0, T_DP = 128, T_DV = 256, T_DK = T_DV + D;
  static constexpr int T_DKB = MERGE_K ? T_DK + 32 : T_DK + DK_COLS;
  static constexpr int T_DQ = T_DK + DK_COLS + (MERGE_K ? 0 : RP);
  static constexpr int T_DQB = T_DQ + D, T_END = T_DQB + RC;
  // a second dQ|dQb accumulator when tensor memory has room: the dQ MMAs of query tile i+1 then do not wait
  // for the drain of tile i
  static constexpr int NDQ = (T_END + D + RC <= 512) ? 2 : 1;
  static constexpr int DQ_STRIDE = T_END - T_DQ;  // columns between the two accumulators
  // otherwise the variant is not built (shape-generic kernels take the problem)
  static constexpr bool FITS = SMEM <= 227 * 1024 && T_END <= 512;
};

template <int C>
__device__ __forceinline__ void tma_tile_bwd(uint32_t dst, const CUtensorMap* m, uint32_t bar, int row0, int h,
                                             int b, int col0 = 0) {
  constexpr int SWB = swizzle_bytes(C);
  constexpr int NB = C * 2 / SWB;
#pragma unroll
  for (int blk = 0; blk < NB; ++blk) tma_load_4d(dst + blk * 128 * SWB, m, bar, col0 + blk * (SWB / 2), row0, h, b);
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Bulk asynchronous reduction shared -> global (fp32 add), executed by the copy engine instead of the
// load/store unit.  Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_reduce_add_f32(float* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(src_smem),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the shared-memory source of every committed group has been read
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Byte offset of 16-byte chunk `ch` of row `r` in a staged [128][D] fp32 dQ tile: 128-byte lines, chunks XOR-swizzled
// by row so that one row per thread writes without bank conflicts.  The fp32 dQ accumulator in global memory keeps
// this arrangement per (batch, head, query tile) when the tile is reduced in bulk.
__host__ __device__ __forceinline__ int dq_stage_off(int r, int ch) {
  return (ch >> 3) * (128 * 128) + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
}

// dq_bias of one query tile, one thread per query row: dq_bias = dS . k_bias, evaluated per group of 32 keys as
// dS16 . (k_bias - c) + c * rowsum_fp32(dS) with c the k_bias of the group's middle key (rows of dS sum to ~0, so
// rounding dS to 16 bits against a large, slowly varying factor -- ALiBi positions -- would otherwise dominate the
// result).  The accumulator holds dS16 . hi(k_bias - c) in columns [0, R) and dS16 . lo(k_bias - c) in columns
// [RCX/2, RCX/2 + R); s_kbc holds c as [column][key group] (4 floats per column, one vector load).
// The result goes rank-major ([R][128 rows]) into the staging tile (STAGED) or straight into the accumulator in
// global memory: consecutive threads then write consecutive floats.
template <typename Cfg>
__device__ __forceinline__ void drain_dq_bias(uint32_t tq_dqb, const float* s_rowsum, uint32_t s_kbc, float* stgb,
                                              float* tileb, int row, bool row_ok, int R) {
  constexpr int HALF = Cfg::RCX / 2;
  constexpr int W = HALF >= 16 ? 16 : 8;
  float rsum[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) rsum[g] = s_rowsum[g * 128 + row];
#pragma unroll 1
  for (int c0 = 0; c0 < HALF && c0 < R; c0 += W) {
    uint32_t rh[W], rl[W];
    tmem_ld(tq_dqb + c0, rh);
    tmem_ld(tq_dqb + HALF + c0, rl);
    tmem_wait_ld(rh);
    tmem_wait_ld(rl);
#pragma unroll
    for (int i = 0; i < W; ++i) {
      const int c = c0 + i;
      if (c < R) {
        const float4 kc = ld_shared_v4f(s_kbc + c * 16);
        float v = __uint_as_float(rh[i]) + __uint_as_float(rl[i]);
        v = fmaf(kc.x, rsum[0], v);
        v = fmaf(kc.y, rsum[1], v);
        v = fmaf(kc.z, rsum[2], v);
        v = fmaf(kc.w, rsum[3], v);
        if (Cfg::STAGED) stgb[c * 128] = v;
        else if (row_ok) atomicAdd(tileb + c * 128 + row, v);
      }
    }
  }
}

enum { BWD_PLAIN = 0, BWD_MASK = 1, BWD_ALIBI = 2 };

// MODE: how the logits are completed -- as computed (BWD_PLAIN), plus an additive mask tensor (BWD_MASK), plus the
// fused ALiBi term (BWD_ALIBI).  A kernel parameter rather than a run-time branch: the mask path needs 32 more
// registers per thread in the P/dS loop, which would otherwise spill in every variant.
template <typename T, int D, int RP, int NQ, int MODE>
__global__ void __launch_bounds__(512, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                 const __grid_constant__ CUtensorMap tmQb, const __grid_constant__ CUtensorMap tmKb,
                 const __grid_constant__ CUtensorMap tmKc, const __grid_constant__ CUtensorMap tmKs,
                 const BwdArgs a) {
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
  const uint32_t kv_full = bar0, dp_full = bar0 + 16, sdp_read = bar0 + 24,
                 dq_full = bar0 + 32 /*2*/, qdo_full = bar0 + 48 /*3*/, qdo_free = bar0 + 72 /*3*/,
                 all_done = bar0 + 112, pds_free = bar0 + 120, pds_ready = bar0 + 136 /*2*/,
                 dq_drained = bar0 + 152 /*2*/;
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
  const int hq = a.hq_bcast ? 0 : h, bq = a.bq_bcast ? 0 : b;
  auto load_tile = [&](int it) {
    const int st = it % Cfg::NSTAGE;
    const uint32_t base = sStage + st * Cfg::STAGE_BYTES;
    mbar_expect_tx(qdo_full + 8 * st, Cfg::STAGE_BYTES);
    const int q0 = (i_begin + it) * 128;
    tma_tile_bwd<D>(base, &tmQ, qdo_full + 8 * st, q0, h, b);
    if (RP) tma_tile_bwd<RPX>(base + Cfg::OFF_QB, &tmQb, qdo_full + 8 * st, q0, hq, bq);
    tma_tile_bwd<D>(base + Cfg::OFF_DO, &tmDO, qdo_full + 8 * st, q0, h, b);
  };

  if (warp == 12) {
    if (lane == 0) {
      *abort_flag = 0;
      mbar_init(kv_full, 1);
      mbar_init(dp_full, 1);
      mbar_init(sdp_read, 8);  // every compute warp has S and dP of the tile in registers
      mbar_init(all_done, 4);  // one commit per issuing thread
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
      if (n_it > 0) {
        // the first loads start before the rest of the CTA has finished its set-up
        const int hk = a.hk_bcast ? 0 : h, bk = a.bk_bcast ? 0 : b;
        mbar_expect_tx(kv_full, Cfg::KV_BYTES);
        tma_tile_bwd<D>(sK, &tmK, kv_full, k0, h, b);
        if (NQ == 2) {
          tma_tile_bwd<D>(sKs, &tmKs, kv_full, k0, h, b);
          tma_tile_bwd<D>(sKs + Cfg::D_BYTES, &tmKs, kv_full, k0, h, b, D);
        }
        if (RP) tma_tile_bwd<RPX>(sKb, &tmKb, kv_full, k0, hk, bk);
        tma_tile_bwd<D>(sV, &tmV, kv_full, k0, h, b);
        load_tile(0);
        if (RP) tma_tile_bwd<Cfg::RCX>(sKc, &tmKc, kv_full, k0, hk, bk);
        for (int it = 1; it < Cfg::NSTAGE && it < n_it; ++it) load_tile(it);
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
    if (lane == 0 && n_it > 0) {
      // The same thread issues the dQ | dQb products: they become due when a query tile's P/dS are written,
      // the next load when the other chains have finished with that tile's stage -- in this order, every tile.
      constexpr uint32_t idQD = instr_desc(kBf16, false, true, 128, D);             // dQ: A K-major, B MN-major
      constexpr uint32_t idQM = instr_desc(kBf16, false, true, 128, D + Cfg::RCX);  // dQ|dQb merged
      constexpr uint32_t idQC = instr_desc(kBf16, false, true, 128, Cfg::RCX);      // dQb alone
      const DescBase kDS = kmajor_base<128>(sDS), mK = mnmajor_base<D>(sK), mKc = mnmajor_base<Cfg::RCX>(sKc);
      // [K | Kc]: 32-column blocks of 64-byte-swizzled rows, the second block at the distance between the tiles
      const uint64_t dKKc = smem_desc(sK, Cfg::OFF_KC - Cfg::OFF_K, 8 * 64, 64);
      const DescBase mKKc{(uint32_t)dKKc, (uint32_t)(dKKc >> 32)};
      mbar_wait(kv_full, 0, abort_flag, a.status);
      auto issue_dQ = [&](int it) {
        const int qb = it % Cfg::NDQ;  // dQ|dQb accumulator of this tile
        const uint32_t tq = tmem + qb * Cfg::DQ_STRIDE;
        const uint32_t pb = (it % Cfg::NBUF) * Cfg::PDS_STRIDE;  // P/dS buffer pair of this tile
        mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
        if (it >= Cfg::NDQ)  // the drain warpgroup has read the tile that used this accumulator last
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
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        issue_dQ(it);
        if (it + Cfg::NSTAGE < n_it) {  // the S|dP, dV and dK chains have finished reading the stage of tile it
          mbar_wait(qdo_free + 8 * (it % Cfg::NSTAGE), (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          load_tile(it + Cfg::NSTAGE);
        }
      }
      umma_commit(all_done);
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
    if (lane == 0 && n_it > 0) {
      const int role = warp - 13;
      constexpr uint32_t idS = instr_desc(kBf16, false, false, 128, 128);  // S, dP: both operands K-major
      constexpr uint32_t idTD = instr_desc(kBf16, true, true, 128, D);     // dV, dK: A^T (MN-major), B MN-major
      constexpr uint32_t idTR = instr_desc(kBf16, true, true, 128, RPX);   // dKb
      constexpr uint32_t idKM = instr_desc(kBf16, true, true, 128, 64);    // dK | dKb merged
      mbar_wait(kv_full, 0, abort_flag, a.status);
      tc_fence_after_sync();
      if (role == 0) {
        // descriptor views built once (stage 0); each MMA adds a constant to the address field
        const DescBase kQ = kmajor_base<D>(sStage), kDO = kmajor_base<D>(sStage + Cfg::OFF_DO),
                       kQb = kmajor_base<RPX>(sStage + Cfg::OFF_QB), kK = kmajor_base<D>(NQ == 2 ? sKs : sK),
                       kKb = kmajor_base<RPX>(sKb), kV = kmajor_base<D>(sV);
        // dKb, when it is an accumulator of its own (no merged [Q | Qb] operand), is issued by this thread as
        // well: between S|dP of query tile i and of tile i+1 it would otherwise idle, and the dV thread, which
        // releases the stage of the tile, gets shorter
        const DescBase mQbT = mnmajor_base<RPX>(sStage + Cfg::OFF_QB), mDST = mnmajor_base<128>(sDS);
        auto issue_dKb = [&](int it) {
          const int st = it % Cfg::NSTAGE;
          const uint32_t so = st * Cfg::STAGE_BYTES;
          mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
#pragma unroll
          for (int s = 0; s < 8; ++s)
            umma_ss(tmem + Cfg::T_DKB, desc_at(mDST, (it % Cfg::NBUF) * Cfg::PDS_STRIDE + mnmajor_step<128>(s)),
                    desc_at(mQbT, so + mnmajor_step<RPX>(s)), idTR, (it > 0 || s > 0) ? 1u : 0u);
          umma_commit(qdo_free + 8 * st);  // S|dP and dKb of the tile: this thread is done with its stage
          umma_commit(pds_free + 8 * (it % Cfg::NBUF));
        };
#pragma unroll 1
        for (int it = 0; it < n_it; ++it) {
          const int st = it % Cfg::NSTAGE;
          const uint32_t so = st * Cfg::STAGE_BYTES;
          if (it > 0) {  // the compute warps hold S and dP of the previous tile in registers
            mbar_wait(sdp_read, (it - 1) & 1, abort_flag, a.status);
            tc_fence_after_sync();
          }
          mbar_wait(qdo_full + 8 * st, (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          tc_fence_after_sync();
          // bias products first, into the empty accumulator (large factor terms cancel among themselves)
          if (RP) {
#pragma unroll
            for (int s = 0; s < RPX / 16; ++s)
              umma_ss(tmem + Cfg::T_S, desc_at(kQb, so + kmajor_step<RPX>(s)), desc_at(kKb, kmajor_step<RPX>(s)), idS,
                      s > 0);
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
          if (Cfg::SEP_DKB) {
            if (it > 0) issue_dKb(it - 1);
          } else {
            umma_commit(qdo_free + 8 * st);
          }
        }
        if (Cfg::SEP_DKB) issue_dKb(n_it - 1);
      } else {
        const DescBase mQ = mnmajor_base<D>(sStage), mDO = mnmajor_base<D>(sStage + Cfg::OFF_DO),
                       mP = mnmajor_base<128>(sP), mDS = mnmajor_base<128>(sDS);
        // [Q | Qb]: 32-column blocks of 64-byte-swizzled rows, the second block at the distance between the tiles
        const uint64_t dQQb = smem_desc(sStage, Cfg::OFF_QB, 8 * 64, 64);
        const DescBase mQQb{(uint32_t)dQQb, (uint32_t)(dQQb >> 32)};
#pragma unroll 1
        for (int it = 0; it < n_it; ++it) {
          const int st = it % Cfg::NSTAGE;
          const uint32_t so = st * Cfg::STAGE_BYTES;
          const uint32_t acc0 = it > 0 ? 1u : 0u;
          const uint32_t pb = (it % Cfg::NBUF) * Cfg::PDS_STRIDE;  // P/dS buffer pair of this tile
          mbar_wait(qdo_full + 8 * st, (it / Cfg::NSTAGE) & 1, abort_flag, a.status);
          mbar_wait(pds_ready + 8 * (it & 1), (it >> 1) & 1, abort_flag, a.status);
          tc_fence_after_sync();
          if (role == 1) {
#pragma unroll
            for (int s = 0; s < 8; ++s)  // contraction over the 128 query rows
              umma_ss(tmem + Cfg::T_DV, desc_at(mP, pb + mnmajor_step<128>(s)), desc_at(mDO, so + mnmajor_step<D>(s)), idTD,
                      (acc0 | (s > 0)) ? 1u : 0u);
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
          umma_commit(pds_free + 8 * (it % Cfg::NBUF));  // this chain no longer reads P / dS of the tile
        }
      }
      umma_commit(all_done);  // every MMA of this thread
    }
  }
  } else if (warp >= 8) {
    setmaxnreg_dec<64>();
    // ------------------------------------------------------------------ drain warpgroup
    // dQ | dQb of each query tile from TMEM into the fp32 accumulators in global memory, off the critical path
    // of the warps that compute P and dS.  One thread per query row.
    if (n_it > 0) {
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
#pragma unroll 1
      for (int it = 0; it < n_it; ++it) {
        const int grow = (i_begin + it) * 128 + row;
        const int qb = it % Cfg::NDQ;
        const uint32_t tq = tmem + qb * Cfg::DQ_STRIDE + lane_off;
        mbar_wait(dq_full + 8 * qb, (it / Cfg::NDQ) & 1, abort_flag, a.status);
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
          const float* s_rowsum = reinterpret_cast<const float*>(smem + Cfg::OFF_ROWSUM) + (it & 3) * 512;
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
      // the staging tile must outlive the last reduction's reads; its global side completes with the kernel
      if (Cfg::STAGED && warp == 8 && lane == 0) bulk_wait_group_read0();
    }
  } else if (n_it > 0) {
    // ------------------------------------------------------------------ compute warpgroups (warps 0-7)
    setmaxnreg_inc<192>();
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = a.scale_log2;
    constexpr int DH = D / 2;  // dV / dK columns per warpgroup in the epilogue
    float* s_kbc = reinterpret_cast<float*>(smem + Cfg::OFF_KBC);
    if (RP) {
      // k_bias of the four keys the centred copy refers to (one per 32-key group), as fp32; read by the drain
      // warpgroup, which is ordered after this through the first pds_ready -> dq_full chain
      const T* kb_bh = a.k_bias_t<T>() + (a.bk_bcast ? 0 : b) * a.kb_stride[0] + (a.hk_bcast ? 0 : h) * a.kb_stride[1];
      for (int i = threadIdx.x; i < 2 * Cfg::RCX; i += 256) {  // [column][key group]
        const int c = i >> 2, g = i & 3;
        s_kbc[i] = c < a.R ? to_f32(kb_bh[(int64_t)min(k0 + 32 * g + 16, a.Sk - 1) * a.kb_stride[2] + c]) : 0.f;
      }
    }

    // Raw loads only: the values are consumed one iteration later, so the global-memory latency
    // hides under the current tile's math instead of stalling the thread here.
    auto load_row_stats = [&](int it, float& lse_raw, float& dlt) {
      const int g = (i_begin + it) * 128 + row;
      lse_raw = INFINITY;
      dlt = 0.f;
      if (it < n_it && g < a.Sq) {
        // volatile: the compiler must not sink the loads to their use one tile later
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(lse_raw) : "l"(a.lse + (int64_t)bh * a.lse_stride_bh + g));
        asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(dlt) : "l"(a.delta + (int64_t)bh * a.lse_stride_bh + g));
      }
    };

    float lse_raw, dlt;
    load_row_stats(0, lse_raw, dlt);
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
    mbar_wait(dp_full, 0, abort_flag, a.status);  // committed after the S and the dP products: covers both
    tc_fence_after_sync();
    tmem_ld32(tSl, rs0);
    tmem_ld32(tDl, rd0);
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
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
      load_row_stats(it + 1, lse_raw, dlt);  // next tile's statistics: the loads complete under this tile's math
      ds_sum1 = chunk(rs1, rd1, pk1, dk1, 1);
      // Chunk 0 of the next tile is fetched under the stores below if its S and dP are already there (they were
      // issued when this tile was released).  If not -- a 2-stage ring delivers the next tile late -- the stores
      // must not wait for it: they release this tile's products, which in turn free the stage.
      bool prefetched = false;
      if (it + 1 < n_it) {
        prefetched = __all_sync(0xffffffffu, mbar_test_wait(dp_full, (it + 1) & 1));
        if (prefetched) {
          tc_fence_after_sync();
          tmem_ld32(tSl, rs0);
          tmem_ld32(tDl, rd0);
        }
      }
      // the dV, dK and dQ products of the query tile that used this buffer pair last have read P and dS
      if (it >= Cfg::NBUF)
        mbar_wait(pds_free + 8 * (it % Cfg::NBUF), (it / Cfg::NBUF - 1) & 1, abort_flag, a.status);
      const uint32_t pb = (it % Cfg::NBUF) * Cfg::PDS_STRIDE;
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
        float* s_rowsum = reinterpret_cast<float*>(smem + Cfg::OFF_ROWSUM) + (it & 3) * 512;
        s_rowsum[(2 * wg) * 128 + row] = ds_sum0;
        s_rowsum[(2 * wg + 1) * 128 + row] = ds_sum1;
      }
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
    // the dV and dK|dKb accumulators are final once every MMA of the CTA has completed
    mbar_wait(all_done, 0, abort_flag, a.status);
    tc_fence_after_sync();

    // ---- epilogue: dV, dK (x scale), dKb
    const int krow = k0 + row;
    {
      T* dvrow = reinterpret_cast<T*>(a.dv) + b * a.dv_stride[0] + h * a.dv_stride[1] + (int64_t)krow * a.dv_stride[2];
      T* dkrow = reinterpret_cast<T*>(a.dk) + b * a.dk_stride[0] + h * a.dk_stride[1] + (int64_t)krow * a.dk_stride[2];
#pragma unroll 1
      for (int c0 = wg * DH; c0 < wg * DH + DH; c0 += 16) {
        uint32_t rv[16], rk[16];
        tmem_ld16(tmem + Cfg::T_DV + lane_off + c0, rv);
        tmem_ld16(tmem + Cfg::T_DK + lane_off + c0, rk);
        tmem_wait_ld(rv);
        tmem_wait_ld(rk);
        if (krow < a.Sk) {
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
    if (RP && wg == 0) {
      // dk_bias tile of this CTA: staged rank-major, [R][128], in the (now idle) P tile, one bulk reduction into the accumulator
      // (other (batch, head) pairs add to the same rows when the factor is shared)
      const int bk = a.bk_bcast ? 0 : b, hk = a.hk_bcast ? 0 : h;
      float* stg = reinterpret_cast<float*>(smem + Cfg::OFF_P) + row;
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
      fence_proxy_async_smem();
      asm volatile("bar.sync 4, 128;" ::: "memory");  // warpgroup 0 only
      if (threadIdx.x == 0) {
        bulk_reduce_add_f32(a.dkb_acc + (bh % a.dkb_slots) * a.dkb_slot_stride +
                                (((int64_t)bk * a.Hk + hk) * a.nk_tiles + kt) * (128 * a.R),
                            sP, 128 * a.R * 4);
        bulk_commit_group();
        bulk_wait_group_read0();  // shared memory must stay until it is read; the global side completes with the kernel
      }
    }
  } else {
    // causal with Sq < Sk: these keys are seen by no query; their gradients are zero
    const int wg = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
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
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 13) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

// dq = T(scale * acc).  acc is fp32, laid out (B, Sq, H, D), or -- `tiled` -- per (batch, head, query tile) as the
// staged [128][D] tile of dq_stage_off.
template <typename T>
__global__ void __launch_bounds__(256) dq_store_kernel(const float* __restrict__ acc, T* __restrict__ dq, int B, int Sq,
                                                       int H, int D, int64_t sb, int64_t sh, int64_t ss, float scale,
                                                       int tiled) {
  const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;  // 8 consecutive d
  const int64_t total = (int64_t)B * Sq * H * D;
  if (idx >= total) return;
  const int d = (int)(idx % D);
  const int h = (int)((idx / D) % H);
  const int s = (int)((idx / ((int64_t)D * H)) % Sq);
  const int b = (int)(idx / ((int64_t)D * H * Sq));
  float4 x, y;
  if (tiled) {
    const int nq_tiles = (Sq + 127) / 128;
    const char* tile = reinterpret_cast<const char*>(acc + (((int64_t)b * H + h) * nq_tiles + s / 128) * (128 * D));
    x = *reinterpret_cast<const float4*>(tile + dq_stage_off(s % 128, d / 4));
    y = *reinterpret_cast<const float4*>(tile + dq_stage_off(s % 128, d / 4 + 1));
  } else {
    x = *reinterpret_cast<const float4*>(acc + idx);
    y = *reinterpret_cast<const float4*>(acc + idx + 4);
  }
  uint4 w;
  w.x = Pack2<T>::pack(x.x * scale, x.y * scale);
  w.y = Pack2<T>::pack(x.z * scale, x.w * scale);
  w.z = Pack2<T>::pack(y.x * scale, y.y * scale);
  w.w = Pack2<T>::pack(y.z * scale, y.w * scale);
  *reinterpret_cast<uint4*>(dq + b * sb + h * sh + s * ss + d) = w;
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
struct BwdWs {
  size_t off_qpack, off_kpack, off_kcenter, off_qs, off_dq, off_dqb, off_dkb, total, zero_bytes;
  int dqb_slots, dkb_slots;
  size_t dqb_slot_bytes, dkb_slot_bytes;
};
inline BwdWs bwd_layout(const fb_params* p, const PackPlan& plan) {
  BwdWs w;
  w.off_qpack = 0;
  w.off_kpack = plan.q_bytes;
  w.off_kcenter = w.off_kpack + plan.k_bytes;
  w.off_qs = w.off_kcenter + plan.kc_bytes;
  w.off_dq = w.off_qs + plan.qs_bytes;
  // query rows padded to whole tiles: the bulk reductions of the backward write whole [128][D] tiles
  const size_t dq = round256((size_t)p->B * ((p->Sq + 127) / 128) * 128 * p->H * p->D * 4);
  // (Bq, Hq, query rows padded to whole tiles, R): a query tile's rows are contiguous for the bulk reduction.
  // When the factor is shared by several (batch, head) pairs they would all add into the same addresses; up to
  // 64 copies spread them, the final store sums the copies.
  const int64_t sharing = (int64_t)(p->B / plan.Bq) * (p->H / plan.Hq);
  w.dqb_slots = p->R ? (int)(sharing < 64 ? sharing : 64) : 1;
  w.dqb_slot_bytes = p->R ? round256((size_t)plan.Bq * plan.Hq * ((p->Sq + 127) / 128) * 128 * p->R * 4) : 0;
  const size_t dqb = w.dqb_slot_bytes * w.dqb_slots;
  const int64_t ksharing = (int64_t)(p->B / plan.Bk) * (p->H / plan.Hk);
  w.dkb_slots = p->R ? (int)(ksharing < 64 ? ksharing : 64) : 1;
  w.dkb_slot_bytes = p->R ? round256((size_t)plan.Bk * plan.Hk * ((p->Sk + 127) / 128) * 128 * p->R * 4) : 0;
  const size_t dkb = w.dkb_slot_bytes * w.dkb_slots;
  w.off_dqb = w.off_dq + dq;
  w.off_dkb = w.off_dqb + dqb;
  w.total = w.off_dkb + dkb;
  w.zero_bytes = dq + dqb + dkb;
  return w;
}

// everything a launch of a backward main kernel needs: tensor maps and arguments
struct BwdLaunch {
  CUtensorMap tQ, tK, tV, tDO, tQb, tKb, tKc, tKs;
  BwdArgs a;
};

// Host work before the main kernel: packs the factor operands, zeroes the fp32 accumulators, encodes the tensor
// maps and fills the kernel arguments.
template <typename T, int D, int RP, int NQ>
int bwd_prepare(const fb_params* p, const PackPlan& plan, cudaStream_t st, BwdLaunch& L) {
  using Cfg = BwdCfg<D, RP, NQ>;
  int rc;
  const BwdWs w = bwd_layout(p, plan);
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  void* qpack = ws + w.off_qpack;
  void* kpack = ws + w.off_kpack;
  void* kcenter = ws + w.off_kcenter;
  CUtensorMap &tQ = L.tQ, &tK = L.tK, &tV = L.tV, &tDO = L.tDO, &tQb = L.tQb, &tKb = L.tKb, &tKc = L.tKc, &tKs = L.tKs;
  if ((rc = make_tmap_4d(&tQ, p->q, D, p->Sq, p->H, p->B, p->q_stride[2], p->q_stride[1], p->q_stride[0], D, 128)))
    return rc;
  if (NQ == 2) {
    // key operand of S = (hi, lo) of k*scale, laid out (B, H, Sk, 2D) in the workspace
    void* ks = ws + w.off_qs;
    if ((rc = make_tmap_4d(&tKs, ks, 2 * D, p->Sk, p->H, p->B, 2 * D, (int64_t)2 * D * p->Sk,
                           (int64_t)2 * D * p->Sk * p->H, D, 128)))
      return rc;
  }
  if ((rc = make_tmap_4d(&tK, p->k, D, p->Sk, p->H, p->B, p->k_stride[2], p->k_stride[1], p->k_stride[0], D, 128)))
    return rc;
  if (NQ != 2) tKs = tK;
  if ((rc = make_tmap_4d(&tV, p->v, D, p->Sk, p->H, p->B, p->v_stride[2], p->v_stride[1], p->v_stride[0], D, 128)))
    return rc;
  if ((rc = make_tmap_4d(&tDO, p->dout, D, p->Sq, p->H, p->B, p->dout_stride[2], p->dout_stride[1],
                         p->dout_stride[0], D, 128)))
    return rc;
  if (RP) {
    if ((rc = make_tmap_4d(&tQb, qpack, RP, p->Sq, plan.Hq, plan.Bq, RP, (int64_t)RP * p->Sq,
                           (int64_t)RP * p->Sq * plan.Hq, RP, 128)))
      return rc;
    if ((rc = make_tmap_4d(&tKb, kpack, RP, p->Sk, plan.Hk, plan.Bk, RP, (int64_t)RP * p->Sk,
                           (int64_t)RP * p->Sk * plan.Hk, RP, 128)))
      return rc;
    constexpr int RC = Cfg::RCX;
    if ((rc = make_tmap_4d(&tKc, kcenter, RC, p->Sk, plan.Hk, plan.Bk, RC, (int64_t)RC * p->Sk,
                           (int64_t)RC * p->Sk * plan.Hk, RC, 128)))
      return rc;
  } else {
    tQb = tQ;
    tKb = tK;
    tKc = tK;
  }
  BwdArgs& a = L.a;
  a.B = p->B; a.H = p->H; a.Sq = p->Sq; a.Sk = p->Sk;
  a.nq_tiles = (p->Sq + 127) / 128;
  a.nk_tiles = (p->Sk + 127) / 128;
  a.causal = p->causal;
  a.R = p->R;
  a.hq_bcast = plan.Hq == 1; a.bq_bcast = plan.Bq == 1; a.hk_bcast = plan.Hk == 1; a.bk_bcast = plan.Bk == 1;
  a.Hq = plan.Hq; a.Hk = plan.Hk;
  // with a split key operand the scale is already inside S
  a.dk_scale = p->softmax_scale;                     // dK accumulates dS^T.q
  a.dkb_scale = NQ == 2 ? 1.f : p->softmax_scale;    // the packed q-side factor carries 1/scale when nq == 1
  a.scale_log2 = (NQ == 2 ? 1.f : p->softmax_scale) * 1.4426950408889634f;
  a.lse = p->lse;
  a.delta = p->delta;
  a.lse_stride_bh = p->lse_stride_bh;
  a.dq_acc = reinterpret_cast<float*>(ws + w.off_dq);
  a.dqb_acc = reinterpret_cast<float*>(ws + w.off_dqb);
  a.dqb_slots = w.dqb_slots;
  a.dqb_slot_stride = (int64_t)(w.dqb_slot_bytes / 4);
  a.dkb_acc = reinterpret_cast<float*>(ws + w.off_dkb);
  a.dkb_slots = w.dkb_slots;
  a.dkb_slot_stride = (int64_t)(w.dkb_slot_bytes / 4);
  a.dk = p->dk;
  a.dv = p->dv;
  for (int i = 0; i < 3; ++i) {
    a.dk_stride[i] = p->dk_stride[i];
    a.dv_stride[i] = p->dv_stride[i];
  }
  a.k_bias = p->k_bias;
  for (int i = 0; i < 3; ++i) a.kb_stride[i] = p->k_bias_stride[i];
  a.status = p->status;
  a.mask = p->mask;
  for (int i = 0; i < 3; ++i) a.mask_stride[i] = p->mask_stride[i];
  if (p->mask_kind == FB_MASK_VECTOR) a.mask_stride[2] = 0;
  a.mask_kind = p->mask_kind;
  a.mask_dtype = p->mask_dtype;
  a.mask_batch_period = p->mask_batch_period;
  a.alibi_slopes = p->alibi_slopes;
  // launches last: the tensor maps and arguments above are ready when the main kernel's turn comes
  if ((rc = launch_pack_operands(p, plan, qpack, kpack, kcenter, true, ws + w.off_qs, st))) return rc;
  cudaError_t e = cudaMemsetAsync(ws + w.off_dq, 0, w.zero_bytes, st);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

// Host work after the main kernel: dq and the factor gradients leave their fp32 accumulators.
template <typename T, int D, int RP, int NQ>
int bwd_finish(const fb_params* p, const BwdLaunch& L, cudaStream_t st) {
  using Cfg = BwdCfg<D, RP, NQ>;
  const BwdArgs& a = L.a;
  cudaError_t e;
  const int64_t n8 = ((int64_t)p->B * p->Sq * p->H * D) / 8;
  dq_store_kernel<T><<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(
      a.dq_acc, reinterpret_cast<T*>(p->dq), p->B, p->Sq, p->H, D, p->dq_stride[0], p->dq_stride[1], p->dq_stride[2],
      p->softmax_scale, Cfg::STAGED ? 1 : 0);
  note_launch();
  if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  if (p->R > 0)
    return store_factor_grads_from(p, a.dqb_acc, a.dkb_acc, st,
                                   {(int64_t)a.nq_tiles * 128, a.dqb_slots, a.dqb_slot_stride},
                                   {(int64_t)a.nk_tiles * 128, a.dkb_slots, a.dkb_slot_stride});
  return 0;
}

template <typename T, int D, int RP, int NQ, int MODE>
int launch_bwd_t(const fb_params* p, const PackPlan& plan, cudaStream_t st) {
  using Cfg = BwdCfg<D, RP, NQ>;
  if constexpr (!Cfg::FITS) {
    return FB_ENOTBUILT;
  } else {
  int rc;
  cudaError_t e;
  BwdLaunch L;
  if ((rc = bwd_prepare<T, D, RP, NQ>(p, plan, st, L))) return rc;
  const BwdArgs& a = L.a;
  auto kern = bwd_sm100_kernel<T, D, RP, NQ, MODE>;
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
  const unsigned grid = (unsigned)((int64_t)a.nk_tiles * p->B * p->H);
  prof_before(KC_BWD_MAIN, st);
  kern<<<grid, 512, Cfg::SMEM, st>>>(L.tQ, L.tK, L.tV, L.tDO, L.tQb, L.tKb, L.tKc, L.tKs, a);
  prof_after(KC_BWD_MAIN, st);
  note_launch();
  if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
  return bwd_finish<T, D, RP, NQ>(p, L, st);
  }
}

bool bwd_cfg_fits(int D, int RP, int nq);
int dispatch_bwd_d32(const fb_params* p, const PackPlan& plan, cudaStream_t st);
int dispatch_bwd_d64(const fb_params* p, const PackPlan& plan, cudaStream_t st);
// persistent form (head_dim 32 with factor operands, plain or masked logits)
int dispatch_bwd_d32p(const fb_params* p, const PackPlan& plan, cudaStream_t st);

}  // namespace fb
