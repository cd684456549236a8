// wsvd_latent_decode_static: the decode op for hosts that cannot hand the library a
// workspace buffer.
//
// Some integrations run the op from a context where device allocation is off the table:
// a serving engine that has already given every free byte of HBM to its KV-cache pool, a
// plugin called from inside a region where cudaMalloc would serialise the device or break
// the engine's own allocator accounting, or a plain C host that owns no allocator at all.
// For those callers the split-KV scratch (partials, log-sum-exp, and the cos/sin position
// table when none is passed) lives in a fixed array inside this library instead of a
// caller-provided workspace.  The price is a hard size limit and no concurrency: see the
// declaration in include/wsvd_b200.h.
#include <mutex>

#include "common.cuh"

namespace {

// One array per GPU that loads the library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[WSVD_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// In host code `g_static_scratch` is only a handle; the address the kernels need comes from
// cudaGetSymbolAddress, asked once per device with that device current.
cudaError_t scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" int wsvd_latent_decode_static(const WsvdLatentDecodeParams* p, void* stream) {
  // the same argument checks, in the same order, as the workspace entry point: an invalid
  // block is reported as such whatever its batch size
  const int st = wsvd::validate_decode_params(p);
  if (st != WSVD_OK) return st;
  if (p->batch == 0) return WSVD_OK;
  const size_t need = wsvd_latent_decode_workspace_bytes(p);
  if (need > (size_t)WSVD_STATIC_SCRATCH_BYTES) return WSVD_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) return wsvd::record_cuda_error(e);
  // Nothing in the scratch has to start at zero: every partial slot the merge reads is
  // written by stage 1 of the same call, and the position table is rebuilt when used.
  // (The cached address stays valid for the life of the device's primary context; a host
  // that calls cudaDeviceReset must not use this entry point afterwards.)
  return wsvd_latent_decode(p, scratch, (size_t)WSVD_STATIC_SCRATCH_BYTES, stream);
}
