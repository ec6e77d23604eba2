// Host-side declarations shared by the translation units of libflashbias_b200.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "flashbias_b200.h"

namespace fb {

// ---- tensor maps (fb_tmap.cu) ---------------------------------------------------------------
// Tiled tensor map over a 16-bit tensor addressed (col, row, head, batch); strides in elements.
// Box = (box_cols x box_rows x 1 x 1), swizzle chosen from box_cols (32/64/128 bytes).
// Returns 0 or a negative FB_E* / positive cudaError_t.
int make_tmap_4d(CUtensorMap* out, const void* ptr, int cols, int64_t rows, int64_t heads, int64_t batch,
                 int64_t stride_row, int64_t stride_head, int64_t stride_batch, int box_cols, int box_rows);
// True if a (ptr, strides) tensor can be described by make_tmap_4d.
bool tma_compatible(const void* ptr, int64_t stride_row, int64_t stride_head, int64_t stride_batch, int64_t heads,
                    int64_t batch);

// ---- operand preparation (fb_pack.cu) ------------------------------------------------------------
// The tensor-core kernels contract over [scaled query terms | packed rank] in one fp32 accumulator.
//   nq == 1 (softmax_scale an exact power of two): the query operand is the caller's q, the q-side factor is
//           q_bias / scale (exact), logits = scale * S.
//   nq == 2: the query operand is q*scale as a (hi, lo) pair of 16-bit terms, laid out (B, H, Sq, 2D); factors
//           are used as given, logits = S.  (The backward splits k*scale instead: its key tile is the resident
//           one.)
// Packed factors: (Bb, Hb, S, RP) contiguous, Bb/Hb = 1 on broadcast dims, zero-padded to RP columns.
struct PackPlan {
  int nq;          // 1 or 2 query terms
  float qb_mult;   // multiplier applied to q_bias when packing (1/scale when nq == 1)
  int RP;          // packed factor width: 0 (no bias), 16, 32 or 64
  int RC;          // width of the centred k-side copy of the backward (>= RP; 32 beside a head_dim-32 K tile)
  int Bq, Hq, Bk, Hk;
  size_t q_bytes, k_bytes, kc_bytes, qs_bytes;  // packed q factor, packed k factor, centred k factor, scaled-query
                                               // copy (each rounded to 256)
};
// false if the rank does not fit the tensor path; for_bwd reserves room for the centred (hi, lo) k-side copy
bool plan_pack(const fb_params* p, PackPlan* plan, bool for_bwd = false);
// One launch prepares every operand of a call: packed q/k factors, kcenter (optional, rows of plan.RC columns:
// k_bias minus the k_bias of the middle key of each group of 32 keys) and, when plan.nq == 2, the (hi, lo) split
// of q*scale (forward) or k*scale (backward; scaled_is_key), laid out (B, H, S, 2D).
int launch_pack_operands(const fb_params* p, const PackPlan& plan, void* qpack, void* kpack, void* kcenter,
                         bool scaled_is_key, void* scaled, cudaStream_t st);

// ---- kernels ------------------------------------------------------------------------------------
int launch_fwd_general(const fb_params* p, cudaStream_t st);
int launch_bwd_preprocess(const fb_params* p, cudaStream_t st);
int launch_bwd_general(const fb_params* p, cudaStream_t st);
size_t bwd_general_workspace(const fb_params* p);

bool fwd_sm100_supported(const fb_params* p, PackPlan* plan);
int launch_fwd_sm100(const fb_params* p, const PackPlan& plan, cudaStream_t st);

bool bwd_sm100_supported(const fb_params* p, PackPlan* plan);
size_t bwd_sm100_workspace(const fb_params* p, const PackPlan& plan);
int launch_bwd_sm100(const fb_params* p, const PackPlan& plan, cudaStream_t st);

inline size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

// fp32 factor-gradient accumulators.  Default shape: the un-expanded (Bx, S, Hx, R).  The tensor-core backward
// uses `slots` copies (summed by the final store) of a head-major (Bx, Hx, rows, R) array with rows padded to
// whole 128-row tiles, so that a tile's rows are contiguous for a bulk reduction.
struct FactorAccLayout {
  int64_t rows;         // 0: default shape
  int slots;            // copies to sum
  int64_t slot_stride;  // floats between copies
};
int store_factor_grads_from(const fb_params* p, float* dqb, float* dkb, cudaStream_t st,
                            FactorAccLayout q_layout = {0, 1, 0}, FactorAccLayout k_layout = {0, 1, 0});

// ---- instrumentation (fb_api.cu) ----------------------------------------------------------------
// Every kernel launch of the library is counted; while profiling is armed for a kernel class, a pair
// of CUDA events is recorded around each launch of that class on the launching stream.
enum KernelClass { KC_OTHER = 0, KC_FWD_MAIN = 1, KC_BWD_MAIN = 2, KC_BWD_PREPROCESS = 3 };
void note_launch(int n = 1);
// number of SMs of a device (cached per device); 0 if the query fails
int device_sm_count(int dev);
void prof_before(int kernel_class, cudaStream_t st);
void prof_after(int kernel_class, cudaStream_t st);

}  // namespace fb
