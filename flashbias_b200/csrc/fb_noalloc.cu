// Forward entry point for callers that cannot allocate device memory.
//
// fb_fwd needs scratch for the packed bias factors and expects the caller to provide it.  Some hosts
// of this library cannot do that: an operator hook of an inference runtime or a custom-op ABI that
// hands the plugin nothing but its input and output buffers, and forbids cudaMalloc inside the call
// because an allocation synchronises the whole device and can fail half-way through a step.  For those
// callers the scratch lives in a fixed array inside the library image.
#include <mutex>

#include "fb_internal.h"

namespace fb {

// Every GPU that loads the library holds this array until the process exits.
static __device__ __align__(256) unsigned char g_fwd_scratch[FB_NOALLOC_SCRATCH_BYTES];

// In host code `g_fwd_scratch` is only a handle for the runtime, not a device address.  The address
// is looked up once per device, with that device current, and cached.
static void* g_scratch_ptr[64] = {};
static std::mutex g_scratch_mu;

static int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return FB_EINVAL_SHAPE;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_fwd_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace fb

extern "C" size_t fb_fwd_noalloc_capacity(void) { return FB_NOALLOC_SCRATCH_BYTES; }

extern "C" int fb_fwd_noalloc(const fb_params* p, void* cuda_stream) {
  using namespace fb;
  if (!p) return FB_EINVAL_NULL;
  const size_t need = fb_fwd_workspace_bytes(p);  // 0 for invalid arguments: fb_fwd reports those below
  if (need > FB_NOALLOC_SCRATCH_BYTES) return FB_EINVAL_SIZE;
  fb_params q = *p;
  q.workspace = nullptr;
  q.workspace_bytes = 0;
  if (need > 0) {
    void* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    q.workspace = scratch;
    q.workspace_bytes = FB_NOALLOC_SCRATCH_BYTES;
  }
  return fb_fwd(&q, cuda_stream);
}
