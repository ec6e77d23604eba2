// Descriptor self-check: one 128 x N x K product per operand-layout flavour the attention kernels
// rely on (K-major and MN-major operands, 32/64/128-byte swizzle, TMA-written and thread-written
// tiles, accumulation of two operand pairs into one accumulator).  The test-suite compares the
// result with a host matmul; a wrong descriptor shows up as a wrong number, not as a fault.
#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

struct SelfCase {
  int mode;  // 0: A,B K-major via TMA (+ optional second pair of width c2) -> D = A B^T          (N = 128)
             // 1: A K-major written by threads, B MN-major via TMA          -> D = A B            (N = c)
             // 2: A MN-major written by threads, B MN-major via TMA         -> D = A^T B          (N = c)
             // 3: A written to tensor memory by threads, B MN-major via TMA -> D = A B            (N = c)
  int c;
  int c2;
};

static const SelfCase kCases[] = {
    {0, 16, 0}, {0, 32, 0}, {0, 64, 0}, {0, 128, 0}, {0, 32, 16}, {0, 64, 16}, {0, 64, 32}, {0, 128, 64},
    {1, 16, 0}, {1, 32, 0}, {1, 64, 0}, {1, 128, 0},
    {2, 16, 0}, {2, 32, 0}, {2, 64, 0}, {2, 128, 0},
    {3, 32, 0}, {3, 64, 0}, {3, 128, 0},
};
static const int kNumCases = sizeof(kCases) / sizeof(kCases[0]);

template <int C>
__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* m, uint32_t bar, int col0) {
  constexpr int SWB = swizzle_bytes(C);
  constexpr int NB = C * 2 / SWB;
#pragma unroll
  for (int b = 0; b < NB; ++b) tma_load_4d(dst + b * 128 * SWB, m, bar, col0 + b * (SWB / 2), 0, 0, 0);
}

template <int MODE, int C, int C2>
__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmA2,
                                                       const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmB2,
                                                       const uint16_t* __restrict__ a_glob, float* __restrict__ d_out,
                                                       int bf16, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                  // 32 KB
  uint8_t* sB = smem + 32768;          // 32 KB
  uint8_t* sA2 = smem + 65536;         // 16 KB
  uint8_t* sB2 = smem + 65536 + 16384; // 16 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 98304);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 98304 + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 98304 + 72);
  constexpr int N = MODE == 0 ? 128 : C;

  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t bar_tma = smem_u32(&bars[0]), bar_mma = smem_u32(&bars[1]);
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  if (MODE == 1 || MODE == 2) {
    // thread t writes row t of the 128 x 128 A tile, 16-byte chunks, in the swizzled layout
    const uint4* src = reinterpret_cast<const uint4*>(a_glob + (size_t)tid * 128);
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      *reinterpret_cast<uint4*>(sA + tile_chunk_offset<128>(tid, ch * 8)) = src[ch];
    }
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  if (MODE == 3) {
    // thread t stores row t of A (128 16-bit values = 64 words) into tensor-memory columns [128, 192)
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a_glob + (size_t)tid * 128);
    for (int c0 = 0; c0 < 64; c0 += 16) {
      uint32_t r[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = src[c0 + i];
      tmem_st16(tmem + ((uint32_t)(warp * 32) << 16) + 128 + c0, r);
    }
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
  }

  if (tid == 0) {
    uint32_t bytes = tile_bytes(C) + (MODE == 0 ? tile_bytes(C) : 0) + (C2 ? 2 * tile_bytes(C2 ? C2 : 16) : 0);
    mbar_expect_tx(bar_tma, bytes);
    if (MODE == 0) tma_tile<C>(smem_u32(sA), &tmA, bar_tma, 0);
    tma_tile<C>(smem_u32(sB), &tmB, bar_tma, 0);
    if (C2) {
      tma_tile<(C2 ? C2 : 16)>(smem_u32(sA2), &tmA2, bar_tma, C);
      tma_tile<(C2 ? C2 : 16)>(smem_u32(sB2), &tmB2, bar_tma, C);
    }
    mbar_wait(bar_tma, 0, abort_flag, status);
    tc_fence_after_sync();
    if (MODE == 0) {
      const uint32_t id = instr_desc(bf16 != 0, false, false, 128, 128);
      for (int ks = 0; ks < C / 16; ++ks)
        umma_ss(tmem, desc_kmajor<C>(smem_u32(sA), ks * 16), desc_kmajor<C>(smem_u32(sB), ks * 16), id, ks > 0);
      if (C2) {
        for (int ks = 0; ks < C2 / 16; ++ks)
          umma_ss(tmem, desc_kmajor<(C2 ? C2 : 16)>(smem_u32(sA2), ks * 16),
                  desc_kmajor<(C2 ? C2 : 16)>(smem_u32(sB2), ks * 16), id, 1);
      }
    } else if (MODE == 1) {
      const uint32_t id = instr_desc(bf16 != 0, false, true, 128, N);
      for (int ks = 0; ks < 8; ++ks)
        umma_ss(tmem, desc_kmajor<128>(smem_u32(sA), ks * 16), desc_mnmajor<C>(smem_u32(sB), ks * 16), id, ks > 0);
    } else if (MODE == 2) {
      const uint32_t id = instr_desc(bf16 != 0, true, true, 128, N);
      for (int ks = 0; ks < 8; ++ks)
        umma_ss(tmem, desc_mnmajor<128>(smem_u32(sA), ks * 16), desc_mnmajor<C>(smem_u32(sB), ks * 16), id, ks > 0);
    } else {
      const uint32_t id = instr_desc(bf16 != 0, false, true, 128, N);
      for (int ks = 0; ks < 8; ++ks)
        umma_ts(tmem, tmem + 128 + ks * 8, desc_mnmajor<C>(smem_u32(sB), ks * 16), id, ks > 0);
    }
    umma_commit(bar_mma);
  }
  __syncwarp();
  mbar_wait(bar_mma, 0, abort_flag, status);
  tc_fence_after_sync();
  const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
  for (int c0 = 0; c0 < N; c0 += 16) {
    uint32_t r[16];
    tmem_ld16(taddr + c0, r);
    tmem_wait_ld(r);
#pragma unroll
    for (int i = 0; i < 16; ++i) d_out[(size_t)tid * N + c0 + i] = __uint_as_float(r[i]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

template <int MODE, int C, int C2>
static int run_case(int bf16, const void* a, const void* b, float* d_out, int* status, cudaStream_t st) {
  CUtensorMap tA, tA2, tB, tB2;
  const int acols = MODE == 0 ? C + C2 : 128;
  const int bcols = MODE == 0 ? C + C2 : C;
  int rc;
  constexpr int BOXC = C > 64 ? 64 : C;
  constexpr int BOXC2 = C2 == 0 ? 16 : (C2 > 64 ? 64 : C2);
  if ((rc = make_tmap_4d(&tA, a, acols, 128, 1, 1, acols, 0, 0, MODE == 0 ? BOXC : 64, 128))) return rc;
  if ((rc = make_tmap_4d(&tB, b, bcols, 128, 1, 1, bcols, 0, 0, BOXC, 128))) return rc;
  if ((rc = make_tmap_4d(&tA2, a, acols, 128, 1, 1, acols, 0, 0, BOXC2, 128))) return rc;
  if ((rc = make_tmap_4d(&tB2, b, bcols, 128, 1, 1, bcols, 0, 0, BOXC2, 128))) return rc;
  auto kern = selftest_kernel<MODE, C, C2>;
  const int smem = 98304 + 128 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  kern<<<1, 128, smem, st>>>(tA, tA2, tB, tB2, reinterpret_cast<const uint16_t*>(a), d_out, bf16, status);
  note_launch();
  return (int)cudaGetLastError();
}

}  // namespace fb

extern "C" int fb_selftest_count(void) { return fb::kNumCases; }

extern "C" int fb_selftest_info(int case_id, int32_t* a_rows, int32_t* a_cols, int32_t* b_rows, int32_t* b_cols,
                                int32_t* n, int32_t* a_transposed, int32_t* b_transposed) {
  if (case_id < 0 || case_id >= fb::kNumCases) return FB_EINVAL_SHAPE;
  const fb::SelfCase& c = fb::kCases[case_id];
  *a_rows = 128;
  *b_rows = 128;
  if (c.mode == 0) {  // D = A B^T over K = c + c2
    *a_cols = c.c + c.c2; *b_cols = c.c + c.c2; *n = 128; *a_transposed = 0; *b_transposed = 1;
  } else {            // D = A B (mode 1) or A^T B (mode 2), K = 128, N = c
    *a_cols = 128; *b_cols = c.c; *n = c.c; *a_transposed = c.mode == 2; *b_transposed = 0;
  }
  return 0;
}

extern "C" int fb_selftest_run(int case_id, int32_t dtype, const void* a, const void* b, float* d_out,
                               int32_t* status, void* cuda_stream) {
  using namespace fb;
  if (case_id < 0 || case_id >= kNumCases) return FB_EINVAL_SHAPE;
  if (!a || !b || !d_out) return FB_EINVAL_NULL;
  if (dtype != FB_DTYPE_F16 && dtype != FB_DTYPE_BF16) return FB_EINVAL_DTYPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  const int bf = dtype == FB_DTYPE_BF16;
  switch (case_id) {
    case 0: return run_case<0, 16, 0>(bf, a, b, d_out, status, st);
    case 1: return run_case<0, 32, 0>(bf, a, b, d_out, status, st);
    case 2: return run_case<0, 64, 0>(bf, a, b, d_out, status, st);
    case 3: return run_case<0, 128, 0>(bf, a, b, d_out, status, st);
    case 4: return run_case<0, 32, 16>(bf, a, b, d_out, status, st);
    case 5: return run_case<0, 64, 16>(bf, a, b, d_out, status, st);
    case 6: return run_case<0, 64, 32>(bf, a, b, d_out, status, st);
    case 7: return run_case<0, 128, 64>(bf, a, b, d_out, status, st);
    case 8: return run_case<1, 16, 0>(bf, a, b, d_out, status, st);
    case 9: return run_case<1, 32, 0>(bf, a, b, d_out, status, st);
    case 10: return run_case<1, 64, 0>(bf, a, b, d_out, status, st);
    case 11: return run_case<1, 128, 0>(bf, a, b, d_out, status, st);
    case 12: return run_case<2, 16, 0>(bf, a, b, d_out, status, st);
    case 13: return run_case<2, 32, 0>(bf, a, b, d_out, status, st);
    case 14: return run_case<2, 64, 0>(bf, a, b, d_out, status, st);
    case 15: return run_case<2, 128, 0>(bf, a, b, d_out, status, st);
    case 16: return run_case<3, 32, 0>(bf, a, b, d_out, status, st);
    case 17: return run_case<3, 64, 0>(bf, a, b, d_out, status, st);
    case 18: return run_case<3, 128, 0>(bf, a, b, d_out, status, st);
  }
  return FB_EINVAL_SHAPE;
}
