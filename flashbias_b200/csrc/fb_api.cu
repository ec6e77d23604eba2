// C ABI of libflashbias_b200: argument validation, kernel selection, workspace sizing.
#include <math.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "fb_internal.h"

namespace fb {

// strides are (batch, head, row) in elements; 0 marks a broadcast batch/head dimension
static int check_strides(const int64_t* s, bool /*may_broadcast*/) {
  for (int i = 0; i < 3; ++i) {
    if (s[i] < 0) return FB_EINVAL_STRIDE;
  }
  return 0;
}

static int validate_common(const fb_params* p) {
  if (!p) return FB_EINVAL_NULL;
  if (p->B <= 0 || p->H <= 0 || p->Sq <= 0 || p->Sk <= 0) return FB_EINVAL_SHAPE;
  if (p->D <= 0 || p->D > 128) return FB_EINVAL_SHAPE;  // reference: head dimensions up to 128
  if (p->R < 0 || p->R > 256) return FB_EINVAL_SHAPE;
  if (p->dtype != FB_DTYPE_F16 && p->dtype != FB_DTYPE_BF16) return FB_EINVAL_DTYPE;
  if (!p->q || !p->k || !p->v || !p->o || !p->lse) return FB_EINVAL_NULL;
  if (p->lse_stride_bh < p->Sq) return FB_EINVAL_LSE;
  int rc;
  if ((rc = check_strides(p->q_stride, false))) return rc;
  if ((rc = check_strides(p->k_stride, false))) return rc;
  if ((rc = check_strides(p->v_stride, false))) return rc;
  if ((rc = check_strides(p->o_stride, false))) return rc;
  if (p->R > 0) {
    if (!p->q_bias || !p->k_bias) return FB_EINVAL_BIAS;
    if ((rc = check_strides(p->q_bias_stride, true))) return rc;
    if ((rc = check_strides(p->k_bias_stride, true))) return rc;
  } else if (p->q_bias || p->k_bias) {
    return FB_EINVAL_BIAS;
  }
  if (p->alibi_slopes && p->R > 0) return FB_EINVAL_BIAS;  // the producer replaces the factors
  if (p->mask_kind != FB_MASK_NONE) {
    if (p->mask_kind != FB_MASK_VECTOR && p->mask_kind != FB_MASK_MATRIX) return FB_EINVAL_MASK;
    if (!p->mask) return FB_EINVAL_MASK;
    if (p->mask_dtype != FB_DTYPE_F16 && p->mask_dtype != FB_DTYPE_BF16 && p->mask_dtype != FB_DTYPE_F32)
      return FB_EINVAL_DTYPE;
    for (int i = 0; i < 3; ++i)
      if (p->mask_stride[i] < 0) return FB_EINVAL_STRIDE;
    if (p->mask_batch_period < 0) return FB_EINVAL_MASK;
  } else if (p->mask) {
    return FB_EINVAL_MASK;
  }
  return 0;
}

static int validate_bwd(const fb_params* p) {
  int rc = validate_common(p);
  if (rc) return rc;
  if (!p->dout || !p->delta || !p->dq || !p->dk || !p->dv) return FB_EINVAL_NULL;
  if ((rc = check_strides(p->dout_stride, false))) return rc;
  if ((rc = check_strides(p->dq_stride, false))) return rc;
  if ((rc = check_strides(p->dk_stride, false))) return rc;
  if ((rc = check_strides(p->dv_stride, false))) return rc;
  if (p->R > 0) {
    if (!p->dq_bias || !p->dk_bias) return FB_EINVAL_NULL;
    if ((rc = check_strides(p->dq_bias_stride, true))) return rc;
    if ((rc = check_strides(p->dk_bias_stride, true))) return rc;
  }
  return 0;
}

static int check_workspace(const fb_params* p, size_t need) {
  if (need == 0) return 0;
  if (!p->workspace || p->workspace_bytes < need) return FB_EINVAL_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(p->workspace) & 255) return FB_EINVAL_WORKSPACE;
  return 0;
}

static std::atomic<long long> g_launches{0};
static std::mutex g_prof_mu;
static int g_prof_class = 0;
static std::vector<std::pair<cudaEvent_t, cudaEvent_t>> g_prof_events;
static cudaEvent_t g_prof_open = nullptr;

void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int device_sm_count(int dev) {
  static std::mutex mu;
  static int cached[64] = {};
  std::lock_guard<std::mutex> lk(mu);
  int& n = cached[dev & 63];
  if (!n) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
  }
  return n;
}

void prof_before(int kernel_class, cudaStream_t st) {
  if (!g_prof_class) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof_class != kernel_class) return;
  cudaEvent_t a = nullptr;
  if (cudaEventCreate(&a) != cudaSuccess) return;
  cudaEventRecord(a, st);
  g_prof_open = a;
}

void prof_after(int kernel_class, cudaStream_t st) {
  if (!g_prof_class) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof_class != kernel_class || !g_prof_open) return;
  cudaEvent_t b = nullptr;
  if (cudaEventCreate(&b) != cudaSuccess) return;
  cudaEventRecord(b, st);
  g_prof_events.emplace_back(g_prof_open, b);
  g_prof_open = nullptr;
}

}  // namespace fb

using namespace fb;

extern "C" long long fb_launch_count(void) { return g_launches.load(); }

extern "C" int fb_prof_begin(int kernel_class) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (kernel_class < 1 || kernel_class > 3) return FB_EINVAL_SHAPE;
  g_prof_class = kernel_class;
  return 0;
}

extern "C" int fb_prof_end(float* total_ms, int* launches) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  float sum = 0.f;
  int n = 0;
  for (auto& ev : g_prof_events) {
    float ms = 0.f;
    if (cudaEventSynchronize(ev.second) == cudaSuccess && cudaEventElapsedTime(&ms, ev.first, ev.second) == cudaSuccess) {
      sum += ms;
      ++n;
    }
    cudaEventDestroy(ev.first);
    cudaEventDestroy(ev.second);
  }
  g_prof_events.clear();
  g_prof_class = 0;
  if (total_ms) *total_ms = sum;
  if (launches) *launches = n;
  return 0;
}

extern "C" int fb_version(void) { return FB_VERSION; }
extern "C" size_t fb_params_size(void) { return sizeof(fb_params); }

extern "C" const char* fb_strerror(int code) {
  switch (code) {
    case FB_OK: return "ok";
    case FB_EINVAL_NULL: return "a required pointer is null";
    case FB_EINVAL_SHAPE: return "dimension out of range (head_dim 1..128, rank 0..256, sizes > 0)";
    case FB_EINVAL_DTYPE: return "only fp16 and bf16 tensors are supported (mask: fp16, bf16 or fp32)";
    case FB_EINVAL_STRIDE: return "negative stride or non-contiguous last dimension";
    case FB_EINVAL_MASK: return "mask pointer and mask_kind disagree";
    case FB_EINVAL_WORKSPACE: return "workspace missing, misaligned or too small";
    case FB_EINVAL_BIAS: return "q_bias and k_bias must be given together with rank > 0 (and not with alibi_slopes)";
    case FB_EINVAL_LSE: return "lse_stride_bh is smaller than Sq";
    case FB_ENOTBUILT: return "kernel variant not available in this build";
    case FB_EDEVICE: return "a kernel reported a device-side error";
    case FB_EINVAL_SIZE: return "problem needs more scratch than the fixed-capacity entry point holds";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown flashbias error";
  }
}

extern "C" const char* fb_status_string(int32_t value) {
  switch (value) {
    case FB_DEV_OK: return "ok";
    case FB_DEV_WAIT_TIMEOUT: return "a bounded wait inside a kernel expired; the results of that call are invalid";
    case FB_DEV_FACTOR_OVERFLOW: return "a pre-scaled bias factor left the range of the 16-bit type";
    default: return "unknown device status";
  }
}

extern "C" int fb_read_status(const int32_t* status, int32_t* value, void* cuda_stream) {
  if (!status) return FB_EINVAL_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  int32_t host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, status, sizeof(host), cudaMemcpyDefault, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return (int)e;
  if (value) *value = host;
  return host == FB_DEV_OK ? FB_OK : FB_EDEVICE;
}

extern "C" int fb_fwd_uses_tensor_path(const fb_params* p) {
  int rc = validate_common(p);
  if (rc) return rc;
  PackPlan plan;
  return fwd_sm100_supported(p, &plan) ? 1 : 0;
}

extern "C" int fb_bwd_uses_tensor_path(const fb_params* p) {
  int rc = validate_common(p);
  if (rc) return rc;
  PackPlan plan;
  return bwd_sm100_supported(p, &plan) ? 1 : 0;
}

extern "C" size_t fb_fwd_workspace_bytes(const fb_params* p) {
  if (validate_common(p)) return 0;
  PackPlan plan;
  if (fwd_sm100_supported(p, &plan)) return plan.q_bytes + plan.k_bytes + plan.qs_bytes;
  return 0;
}

extern "C" int fb_fwd(const fb_params* p, void* cuda_stream) {
  int rc = validate_common(p);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  PackPlan plan;
  if (fwd_sm100_supported(p, &plan)) {
    if ((rc = check_workspace(p, plan.q_bytes + plan.k_bytes + plan.qs_bytes))) return rc;
    return launch_fwd_sm100(p, plan, st);
  }
  return launch_fwd_general(p, st);
}

extern "C" size_t fb_bwd_workspace_bytes(const fb_params* p) {
  if (validate_common(p)) return 0;
  PackPlan plan;
  if (bwd_sm100_supported(p, &plan)) return bwd_sm100_workspace(p, plan);
  return bwd_general_workspace(p);
}

extern "C" int fb_bwd_preprocess(const fb_params* p, void* cuda_stream) {
  int rc = validate_bwd(p);
  if (rc) return rc;
  return launch_bwd_preprocess(p, reinterpret_cast<cudaStream_t>(cuda_stream));
}

extern "C" int fb_bwd(const fb_params* p, void* cuda_stream) {
  int rc = validate_bwd(p);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(cuda_stream);
  PackPlan plan;
  if (bwd_sm100_supported(p, &plan)) {
    if ((rc = check_workspace(p, bwd_sm100_workspace(p, plan)))) return rc;
    return launch_bwd_sm100(p, plan, st);
  }
  if ((rc = check_workspace(p, bwd_general_workspace(p)))) return rc;
  return launch_bwd_general(p, st);
}
