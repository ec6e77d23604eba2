// Device-side building blocks for the sm_100a FlashBias kernels: mbarrier, TMA (bulk tensor
// copies), tcgen05 (tensor-memory MMA) wrappers and the shared-memory / instruction descriptors
// they consume.  Everything here is inline PTX; there is no library dependency.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flashbias_b200.h"

namespace fb {

// Kernels whose bounded waits expire store FB_DEV_WAIT_TIMEOUT (flashbias_b200.h) in the caller's status word:
// never a trap, never an endless spin.
constexpr uint32_t kSpinLimit = 1u << 22;  // try_wait polls before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One arrival per warp: every lane has finished (and fenced) its own work, the warp converges, lane 0
// arrives.  The barrier is initialised with the number of participating warps, so a phase costs a handful
// of shared-memory atomics instead of one per thread.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking test of a phase (no suspension).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory: once any wait of the CTA has expired every
// later wait returns at once, so a broken pipeline drains in bounded time.  Returns false on expiry.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  if (status) atomicExch(status, FB_DEV_WAIT_TIMEOUT);
  return false;
}

// ---------------------------------------------------------------------------------------------
// Fences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA: tiled bulk tensor load, global -> shared, completion on an mbarrier.  Every CTA loads its own copy.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tile store shared -> global (the mirror of tma_load_4d); rows past the tensor's extent are clipped.  Completion
// is tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tensor memory (TMEM) management
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory operand tiles are always [128 rows][C columns] of a 16-bit type, stored the way a
// TMA box of (min(C,64) columns x 128 rows) with the matching swizzle writes them: `nblk` column
// blocks, each 128 rows of SWB = min(2C,128) bytes, 16-byte chunks XOR-swizzled within each
// 8-row group.  The same bytes can be read by the tensor core
//   * K-major  : rows are the M/N index, columns the contraction index, or
//   * MN-major : columns are the M/N index, rows the contraction index.
constexpr __host__ __device__ int swizzle_bytes(int cols) { return cols * 2 >= 128 ? 128 : cols * 2; }
constexpr __host__ __device__ int tile_bytes(int cols) { return 128 * cols * 2; }

// sm_100 shared-memory matrix descriptor: start address [0,14), leading byte offset [16,30),
// stride byte offset [32,46) (all in 16-byte units), version 1 at [46,48), layout type at [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, int swb) {
  const uint64_t layout = swb == 128 ? 2ull : swb == 64 ? 4ull : swb == 32 ? 6ull : 0ull;
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (layout << 61);
}

// K-major view, contraction columns [col0, col0+16) of a [128][C] tile at `base`.
template <int C>
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int col0) {
  constexpr int SWB = swizzle_bytes(C);
  const int byte0 = col0 * 2;
  const uint32_t addr = base + (byte0 / SWB) * (128 * SWB) + (byte0 % SWB);
  return smem_desc(addr, 16, 8 * SWB, SWB);
}

// MN-major view, contraction rows [row0, row0+16) of a [128][C] tile at `base`; the M/N extent
// starts at column `col0` (a multiple of the swizzle atom width, SWB/2 columns).
template <int C>
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int row0, int col0 = 0) {
  constexpr int SWB = swizzle_bytes(C);
  const uint32_t addr = base + ((col0 * 2) / SWB) * (128 * SWB) + row0 * SWB;
  return smem_desc(addr, 128 * SWB, 8 * SWB, SWB);
}

// Descriptors whose base address is only known at run time: everything but the start-address field is
// fixed per (tile width, major), so a view is built once and each MMA adds a compile-time byte offset.
struct DescBase {
  uint32_t lo, hi;
};
template <int C>
__device__ __forceinline__ DescBase kmajor_base(uint32_t base) {
  const uint64_t d = desc_kmajor<C>(base, 0);
  return DescBase{(uint32_t)d, (uint32_t)(d >> 32)};
}
template <int C>
__device__ __forceinline__ DescBase mnmajor_base(uint32_t base) {
  const uint64_t d = desc_mnmajor<C>(base, 0, 0);
  return DescBase{(uint32_t)d, (uint32_t)(d >> 32)};
}
// byte offset of K-step s (16 contraction elements) inside a [128][C] tile
template <int C>
__host__ __device__ constexpr uint32_t kmajor_step(int s) {
  return ((s * 32) / swizzle_bytes(C)) * (128 * swizzle_bytes(C)) + (s * 32) % swizzle_bytes(C);
}
template <int C>
__host__ __device__ constexpr uint32_t mnmajor_step(int s) {
  return s * 16 * swizzle_bytes(C);
}
__device__ __forceinline__ uint64_t desc_at(DescBase d, uint32_t byte_off) {
  return ((uint64_t)d.hi << 32) | (uint64_t)(d.lo + (byte_off >> 4));
}

// Instruction descriptor for tcgen05.mma.kind::f16: fp32 accumulate, A/B of the same 16-bit type.
// c_format F32 at [4,6); a/b format (0 f16, 1 bf16) at [7,10)/[10,13); a/b major (1 = MN) at 15/16;
// N>>3 at [17,23); M>>4 at [24,29).
__host__ __device__ constexpr uint32_t instr_desc(bool bf16, bool a_mn, bool b_mn, int M, int N) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn ? 1u : 0u) << 15) |
         ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A is K-major in tensor memory: lane = row, each 32-bit column holds two
// consecutive 16-bit contraction elements (16 elements = 8 columns per MMA).  Issued by ONE thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Make an mbarrier track completion of all MMAs issued so far by this thread.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers.  Shape 32x32b: thread t of the warp owns TMEM lane (32*(warp%4) + t) and
// receives N consecutive 32-bit columns.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[8]) { tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The loaded registers are operands of the wait, so no use of them can be scheduled ahead of it.
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]) :: "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Per-warpgroup register budget (all four warps of the warpgroup execute it): warps that only move data or issue
// MMAs hand registers to the warps that do the arithmetic.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// 16-byte store to a shared-memory address (32-bit shared-window address, no generic-address translation)
__device__ __forceinline__ float4 ld_shared_v4f(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Small math / conversion helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed fp32 pairs (sm_100 executes add/mul/fma on two fp32 values with one instruction): the softmax and
// P/dS loops are bound by instruction issue, not by the FMA pipe, so halving their FMA-pipe instructions pays.
__device__ __forceinline__ uint64_t f2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// max of three values in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <typename T> struct Pack2;
template <> struct Pack2<__half> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct Pack2<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }

// 256-bit load through the read-only path (32-byte aligned address): one request covers a whole 32-byte sector.
__device__ __forceinline__ void ldg_nc_v8(const void* p, uint32_t (&w)[8]) {
  asm("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(p));
}

// 32 consecutive mask values of one row as fp32 (times log2 e).  `p` points at the first of them; `n` of them
// exist (the rest read as 0); `vec` says that p is 16-byte aligned and n == 32.
template <typename MT>
__device__ __forceinline__ void load_mask_chunk(const MT* __restrict__ p, int n, bool vec, float (&mv)[32]) {
  constexpr float kLog2e = 1.4426950408889634f;
  if (vec && (reinterpret_cast<uintptr_t>(p) & 31) == 0) {
    // Every thread reads its own row, so a load instruction of the warp touches 32 different lines whatever its
    // width: 256-bit loads halve the number of instructions (and of line requests) of the 128-bit form.
    constexpr int PER = 32 / (int)sizeof(MT);
#pragma unroll
    for (int g = 0; g < 32 / PER; ++g) {
      uint32_t w[8];
      ldg_nc_v8(reinterpret_cast<const char*>(p) + 32 * g, w);
      const MT* e = reinterpret_cast<const MT*>(w);
#pragma unroll
      for (int i = 0; i < PER; ++i) mv[g * PER + i] = to_f32(e[i]) * kLog2e;
    }
  } else if (vec) {
    constexpr int PER = 16 / (int)sizeof(MT);
#pragma unroll
    for (int g = 0; g < 32 / PER; ++g) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(p) + g);
      const MT* e = reinterpret_cast<const MT*>(&w);
#pragma unroll
      for (int i = 0; i < PER; ++i) mv[g * PER + i] = to_f32(e[i]) * kLog2e;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) mv[i] = i < n ? to_f32(p[i]) * kLog2e : 0.f;
  }
}

// Byte offset of the 16-byte chunk holding columns [col, col+8) of `row` inside a [128][C] tile
// (the layout described above); `col` is a multiple of 8.
template <int C>
__device__ __forceinline__ uint32_t tile_chunk_offset(int row, int col) {
  constexpr int SWB = swizzle_bytes(C);
  constexpr int CHUNKS = SWB / 16;  // chunks per row of one block
  const int byte0 = col * 2;
  const int blk = byte0 / SWB;
  const int chunk = (byte0 % SWB) >> 4;
  // 128B swizzle XORs the chunk index with row%8; 64B with (row/2)%4; 32B with (row/4)%2.
  const int x = SWB == 128 ? (row & 7) : SWB == 64 ? ((row >> 1) & 3) : SWB == 32 ? ((row >> 2) & 1) : 0;
  return blk * (128 * SWB) + row * SWB + (((chunk ^ x) & (CHUNKS - 1)) << 4);
}

}  // namespace fb
