// Caller-side glue fused into one pass: cast to the 16-bit run type, optional L2 normalisation of every row
// and optional per-head scale.  Input and output are addressed through (batch, head, row) element strides, so
// a (B, H, S, D) tensor is read where it lies and the result can keep that layout: the attention kernels take
// the same strides, which removes the permute + contiguous + cast copies of the reference's call sites
// (2_Vision_Transformer/swin_transformer_v2.py:194-199, 4_AlphaFold3/protenix/openfold_local/model/
// primitives.py:636-640).  HBM-bound: every element is read once and written once.
#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

struct PrepArgs {
  const void* x;
  void* y;
  int64_t xs[3], ys[3];  // (batch, head, row) element strides
  int B, H, S, D;
  int normalize;
  const float* head_scale;  // optional, H values
  float eps;
};

// D / 8 threads per row (a power of two up to 16), 8 consecutive elements per thread.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) prepare_rows_kernel(const PrepArgs a) {
  const int tpr = a.D / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t rowi = gid / tpr;
  const int part = (int)(gid % tpr);
  const int64_t total = (int64_t)a.B * a.H * a.S;
  const bool live = rowi < total;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int b = 0, h = 0, s = 0;
  if (live) {
    s = (int)(rowi % a.S);
    h = (int)((rowi / a.S) % a.H);
    b = (int)(rowi / ((int64_t)a.S * a.H));
    const TI* src = reinterpret_cast<const TI*>(a.x) + b * a.xs[0] + h * a.xs[1] + s * a.xs[2] + part * 8;
    if (sizeof(TI) == 4) {
      const float4 p0 = *reinterpret_cast<const float4*>(src), p1 = *reinterpret_cast<const float4*>(src + 4);
      v[0] = p0.x; v[1] = p0.y; v[2] = p0.z; v[3] = p0.w; v[4] = p1.x; v[5] = p1.y; v[6] = p1.z; v[7] = p1.w;
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const TI* e = reinterpret_cast<const TI*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = to_f32(e[i]);
    }
  }
  float mult = 1.f;
  if (a.normalize) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    for (int o = tpr >> 1; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    mult = 1.f / fmaxf(sqrtf(ss), a.eps);  // x / max(|x|, eps), as torch.nn.functional.normalize
  }
  if (live) {
    if (a.head_scale) mult *= a.head_scale[h];
    uint4 w;
    w.x = Pack2<TO>::pack(v[0] * mult, v[1] * mult);
    w.y = Pack2<TO>::pack(v[2] * mult, v[3] * mult);
    w.z = Pack2<TO>::pack(v[4] * mult, v[5] * mult);
    w.w = Pack2<TO>::pack(v[6] * mult, v[7] * mult);
    TO* dst = reinterpret_cast<TO*>(a.y) + b * a.ys[0] + h * a.ys[1] + s * a.ys[2] + part * 8;
    *reinterpret_cast<uint4*>(dst) = w;
  }
}

template <typename TO>
static int launch_prepare_t(const PrepArgs& a, int in_dtype, cudaStream_t st) {
  const int64_t threads = (int64_t)a.B * a.H * a.S * (a.D / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  if (in_dtype == FB_DTYPE_F32) prepare_rows_kernel<float, TO><<<blocks, 256, 0, st>>>(a);
  else if (in_dtype == FB_DTYPE_F16) prepare_rows_kernel<__half, TO><<<blocks, 256, 0, st>>>(a);
  else prepare_rows_kernel<__nv_bfloat16, TO><<<blocks, 256, 0, st>>>(a);
  note_launch();
  return (int)cudaGetLastError();
}

}  // namespace fb

extern "C" int fb_prepare_rows(const void* x, int32_t x_dtype, const int64_t* x_stride, void* y, int32_t y_dtype,
                               const int64_t* y_stride, int32_t B, int32_t H, int32_t S, int32_t D,
                               int32_t normalize, const float* head_scale, float eps, void* cuda_stream) {
  using namespace fb;
  if (!x || !y || !x_stride || !y_stride) return FB_EINVAL_NULL;
  if (B <= 0 || H <= 0 || S <= 0) return FB_EINVAL_SHAPE;
  if (!(D == 8 || D == 16 || D == 32 || D == 64 || D == 128)) return FB_EINVAL_SHAPE;
  if (x_dtype != FB_DTYPE_F32 && x_dtype != FB_DTYPE_F16 && x_dtype != FB_DTYPE_BF16) return FB_EINVAL_DTYPE;
  if (y_dtype != FB_DTYPE_F16 && y_dtype != FB_DTYPE_BF16) return FB_EINVAL_DTYPE;
  const int in_vec = x_dtype == FB_DTYPE_F32 ? 4 : 8;  // elements per 16-byte load
  PrepArgs a;
  a.x = x; a.y = y;
  for (int i = 0; i < 3; ++i) {
    if (x_stride[i] < 0 || y_stride[i] < 0) return FB_EINVAL_STRIDE;
    if ((x_stride[i] % in_vec) || (y_stride[i] % 8)) return FB_EINVAL_STRIDE;  // rows start on 16-byte boundaries
    a.xs[i] = x_stride[i];
    a.ys[i] = y_stride[i];
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return FB_EINVAL_STRIDE;
  a.B = B; a.H = H; a.S = S; a.D = D;
  a.normalize = normalize;
  a.head_scale = head_scale;
  a.eps = eps;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  return y_dtype == FB_DTYPE_F16 ? launch_prepare_t<__half>(a, x_dtype, st)
                                 : launch_prepare_t<__nv_bfloat16>(a, x_dtype, st);
}
