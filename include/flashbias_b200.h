/*
 * flashbias_b200 -- C ABI of the B200 (sm_100a) FlashBias attention path.
 *
 * o = softmax(softmax_scale * q k^T + q_bias k_bias^T [+ mask] [causal]) v, forward and backward.
 *
 * This is the boundary a binding of the reference's operator would call: plain pointers, sizes
 * and strides, no framework types.  Every entry point is stream-ordered, allocates nothing on the
 * device, never synchronises the device, and returns 0 on success, a negative FB_E* code for a
 * rejected argument, or a positive cudaError_t.  All pointers are device pointers unless stated.
 *
 * Reference interface replaced (paths inside the reference project):
 *   fb_fwd             <- _flash_attn_forward + _fwd_kernel      flash_bias/flash_bias_triton.py:1100-1194, 75-355
 *   fb_bwd_preprocess  <- _bwd_preprocess_do_o_dot               flash_bias/flash_bias_triton.py:358-400, 1234-1251
 *   fb_bwd             <- _flash_attn_backward + _bwd_kernel     flash_bias/flash_bias_triton.py:1197-1342, 905-1097
 * The Python operator FlashBiasFunc (flash_bias/flash_bias_triton.py:1345-1405) sits on top of these.
 */
#ifndef FLASHBIAS_B200_H_
#define FLASHBIAS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FB_VERSION 2

/* element types */
#define FB_DTYPE_F16 0
#define FB_DTYPE_BF16 1
#define FB_DTYPE_F32 2 /* mask only */

/* additive mask kinds: last two dims (1, Sk) = vector, (Sq, Sk) = matrix
 * (flash_bias/flash_bias_triton.py:1120-1127) */
#define FB_MASK_NONE 0
#define FB_MASK_VECTOR 1
#define FB_MASK_MATRIX 2

/* flags */
#define FB_FLAG_FORCE_GENERAL 1 /* use the shape-generic CUDA-core kernels even where the tensor-core path applies */
#define FB_FLAG_BWD_QUERY_MAJOR 2 /* backward without factor operands at head_dim 32: use the query-major tensor-core
                                     kernel instead of the key-major one (cross-checks; same results up to rounding) */
#define FB_FLAG_BWD_ONE_ITEM 4   /* backward with factor operands at head_dim 32: one work item (128 keys of a (batch,
                                     head)) per CTA, whatever the shape */
#define FB_FLAG_BWD_PERSISTENT 8 /* ... one persistent CTA per SM walking the work items, whatever the shape (by
                                     default: chosen when a work item has few query tiles) */

/* error codes (negative); positive return values are cudaError_t */
#define FB_OK 0
#define FB_EINVAL_NULL -1      /* a required pointer is null */
#define FB_EINVAL_SHAPE -2     /* a dimension is out of range (head_dim must be 1..128, rank 0..256, sizes > 0) */
#define FB_EINVAL_DTYPE -3     /* dtype / mask_dtype not supported */
#define FB_EINVAL_STRIDE -4    /* a stride is negative or a last dimension is not contiguous */
#define FB_EINVAL_MASK -5      /* mask_kind inconsistent with the mask pointer */
#define FB_EINVAL_WORKSPACE -6 /* workspace missing or smaller than fb_*_workspace_bytes() */
#define FB_EINVAL_BIAS -7      /* exactly one of q_bias / k_bias given, or rank mismatch */
#define FB_EINVAL_LSE -8       /* lse_stride_bh smaller than Sq */
#define FB_ENOTBUILT -9        /* the library was built without the requested kernel */
#define FB_EDEVICE -10         /* a kernel reported a device-side error through the status word */
#define FB_EINVAL_SIZE -11     /* the problem needs more scratch than a fixed-capacity entry point holds */

/*
 * One problem description, shared by forward and backward.
 *
 * Tensors are addressed as ptr[b*stride[0] + h*stride[1] + row*stride[2] + col] in ELEMENTS; the
 * last dimension is contiguous.  q, o, dout, dq: (B, Sq, H, D).  k, v, dk, dv: (B, Sk, H, D).
 * q_bias, dq_bias: (B|1, Sq, H|1, R); k_bias, dk_bias: (B|1, Sk, H|1, R); a stride of 0 in the batch
 * and/or head slot marks a broadcast dimension, and gradients of a broadcast factor are summed over it.
 * mask: (B|1, H|1, 1|Sq, Sk) with strides (batch, head, row); added to the logits after the bias.
 * lse / delta: fp32, (B*H, lse_stride_bh) with lse_stride_bh >= Sq (the reference rounds Sq up to 128).
 */
typedef struct fb_params {
  int32_t B, H, Sq, Sk, D, R;
  int32_t dtype;      /* FB_DTYPE_F16 | FB_DTYPE_BF16: q,k,v,o,factors and all gradients */
  int32_t causal;     /* top-left aligned: row >= col is visible */
  int32_t mask_kind;  /* FB_MASK_* */
  int32_t mask_dtype; /* FB_DTYPE_F16 | FB_DTYPE_BF16 | FB_DTYPE_F32 */
  int32_t flags;      /* FB_FLAG_* */
  float softmax_scale; /* applied to q.k only; the bias term is not scaled */

  const void *q, *k, *v, *q_bias, *k_bias, *mask;
  int64_t q_stride[3], k_stride[3], v_stride[3], q_bias_stride[3], k_bias_stride[3], mask_stride[3];

  void *o;
  int64_t o_stride[3];
  float *lse; /* forward: written; backward: read */
  int64_t lse_stride_bh;

  /* backward only */
  const void *dout;
  int64_t dout_stride[3];
  float *delta; /* rowsum(o * dout): written by fb_bwd_preprocess, read by fb_bwd; layout as lse */
  void *dq, *dk, *dv, *dq_bias, *dk_bias;
  int64_t dq_stride[3], dk_stride[3], dv_stride[3], dq_bias_stride[3], dk_bias_stride[3];

  void *workspace; /* scratch of at least fb_{fwd,bwd}_workspace_bytes(); 256-byte aligned */
  size_t workspace_bytes;
  int32_t *status; /* optional int32 the device can write (device memory or mapped pinned host memory), zeroed by
                      the caller; kernels store a non-zero FB_DEV_* code there on a device-side error */

  /*
   * Fused bias producer (optional).  alibi_slopes: fp32, one slope per head (H values).  When given, the bias
   * slope[h] * (col - row) is generated inside the kernels from the row and column indices instead of being read
   * as factors: it is the bias of the rank-2 factors q_bias[i] = [-m i, 1], k_bias[j] = [1, m j]
   * (1_Language_Model/attention_with_alibi_bias.py:8-15, 47-52) evaluated in fp32, without the rounding of the
   * positions to 16 bits.  q_bias / k_bias must then be null and R = 0; the slopes are constants (the reference
   * registers them as a buffer), so the backward returns dq, dk, dv only.
   */
  const float *alibi_slopes;

  /*
   * mask_batch_period > 0: the mask holds that many batch entries and batch entry b reads entry b % period.
   * Swin-V2 repeats its (nW, N, N) shift mask B/nW times along the batch (2_Vision_Transformer/
   * swin_transformer_v2.py:189-192); with the period the nW masks are read in place and stay in L2.
   */
  int32_t mask_batch_period;
} fb_params;

/* values of *status */
#define FB_DEV_OK 0
#define FB_DEV_WAIT_TIMEOUT 1    /* a bounded wait inside a kernel expired; the results of that call are invalid */
#define FB_DEV_FACTOR_OVERFLOW 2 /* a pre-scaled bias factor left the range of the 16-bit type */

int fb_version(void);
size_t fb_params_size(void); /* sizeof(fb_params) as compiled, for bindings to check their mirror of the struct */
const char *fb_strerror(int code);

/* 1 if the tcgen05/TMA kernels handle this problem, 0 if the shape-generic kernels do, <0 on invalid arguments */
int fb_fwd_uses_tensor_path(const fb_params *p);
int fb_bwd_uses_tensor_path(const fb_params *p);

size_t fb_fwd_workspace_bytes(const fb_params *p);
int fb_fwd(const fb_params *p, void *cuda_stream);

size_t fb_bwd_workspace_bytes(const fb_params *p);
int fb_bwd_preprocess(const fb_params *p, void *cuda_stream);
int fb_bwd(const fb_params *p, void *cuda_stream);

/*
 * Reads a status word after the work queued on `cuda_stream` has completed (copies it to the host and
 * synchronises that stream): FB_OK if it is zero, FB_EDEVICE otherwise; *value (optional) receives the word.
 * No counterpart in the reference, whose kernels have no device-side error path.  A caller that keeps the
 * word in mapped pinned host memory can simply read it instead.
 */
int fb_read_status(const int32_t *status, int32_t *value, void *cuda_stream);
const char *fb_status_string(int32_t value);

/*
 * Caller-side glue in one pass: y = T(normalize?(x) * head_scale[h]) with x and y addressed as
 * ptr[b*stride[0] + h*stride[1] + row*stride[2] + col] (ELEMENT strides, contiguous rows of D in {8, 16, 32,
 * 64, 128} elements that start on 16-byte boundaries).  x: fp32, fp16 or bf16; y: fp16 or bf16.  normalize != 0
 * divides every row by max(|row|_2, eps) first (torch.nn.functional.normalize); head_scale is optional (H
 * fp32 values).  Replaces the .permute(0, 2, 1, 3).contiguous().half() copies -- and, for Swin-V2, the
 * F.normalize(q) * logit_scale product -- that the reference's call sites run before flash_bias_func
 * (2_Vision_Transformer/swin_transformer_v2.py:194-199, 4_AlphaFold3/protenix/openfold_local/model/
 * primitives.py:636-640, flash_bias/benchmark.py:316-317): the result may keep the caller's (B, H, S, D) layout,
 * because fb_fwd / fb_bwd take the same strides.
 */
int fb_prepare_rows(const void *x, int32_t x_dtype, const int64_t *x_stride, void *y, int32_t y_dtype,
                    const int64_t *y_stride, int32_t B, int32_t H, int32_t S, int32_t D, int32_t normalize,
                    const float *head_scale, float eps, void *cuda_stream);

/*
 * fb_fwd for callers that cannot allocate device memory.  This entry point has no counterpart in the
 * reference, whose launcher allocates its scratch with torch.
 *
 * Who needs it: hosts that call the library from a hook which receives only input and output buffers
 * and must not call cudaMalloc there -- for example the enqueue step of an inference-runtime plugin or a
 * custom-op ABI without a workspace argument.  A device allocation inside such a call would synchronise
 * the device and can fail under memory pressure in the middle of a step.
 *
 * Same arguments and results as fb_fwd; p->workspace and p->workspace_bytes are ignored.  The scratch
 * (packed bias factors) lives in a fixed array of FB_NOALLOC_SCRATCH_BYTES inside the library, held by
 * every GPU that loads the library until the process exits.  A problem whose fb_fwd_workspace_bytes()
 * exceeds that capacity is rejected with FB_EINVAL_SIZE before anything is launched.  No cudaMalloc,
 * cudaFree or other allocating call is made.
 *
 * The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with
 * that device current), and the first call of each kernel variant on a device raises that kernel's
 * shared-memory limit (and, under lazy module loading, loads its code); make one warm-up call per device
 * and problem kind outside any stream capture and outside the hook that forbids allocation.  All
 * calls on a device share the one array, which keeps the previous call's contents: every byte a call
 * reads it has written itself first, so nothing needs clearing, but two calls that overlap on the GPU
 * (different streams) race on it -- keep them on one stream or order them with events.
 */
#define FB_NOALLOC_SCRATCH_BYTES (32u << 20)
size_t fb_fwd_noalloc_capacity(void);
int fb_fwd_noalloc(const fb_params *p, void *cuda_stream);

/*
 * Instrumentation (no counterpart in the reference).  fb_launch_count: kernels launched by this
 * library in this process so far.  fb_prof_begin(kernel_class) arms per-launch CUDA-event timing of one
 * kernel class (1 forward main kernel, 2 backward main kernel, 3 backward pre-pass) on the launching
 * stream; fb_prof_end synchronises those events and returns the summed device time and launch count.
 */
long long fb_launch_count(void);
int fb_prof_begin(int kernel_class);
int fb_prof_end(float *total_ms, int *launches);

/*
 * Descriptor self-check of the tensor-core building blocks: runs one 128 x N x K product through
 * TMA + tcgen05 for the operand layout `case_id` and writes the fp32 result (128 x N, row-major) to
 * d_out.  a and b are 16-bit device matrices of the shape the case documents (see fb_selftest_info).
 * No counterpart in the reference; used by the test-suite.
 */
int fb_selftest_count(void);
int fb_selftest_info(int case_id, int32_t *a_rows, int32_t *a_cols, int32_t *b_rows, int32_t *b_cols, int32_t *n,
                     int32_t *a_transposed, int32_t *b_transposed);
int fb_selftest_run(int case_id, int32_t dtype, const void *a, const void *b, float *d_out, int32_t *status,
                    void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHBIAS_B200_H_ */
