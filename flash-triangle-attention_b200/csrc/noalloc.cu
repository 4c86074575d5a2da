// fta_backward_noalloc: the backward pass for callers that cannot hand over a workspace.
//
// Some hosts of this library have no way to allocate device memory at the point where they
// call it: code running inside a framework's memory-planning phase, plugins whose interface
// only passes input and output buffers, or real-time loops that forbid cudaMalloc. For them
// the scratch memory of the backward pass (the float32 dQ accumulator, the partial dBias
// planes, the key-major bias copy) lives in a fixed array inside the library image.
//
// The array is `kNoAllocMaxBytes` long and exists once per GPU that loads the library, until
// the process exits. In host code its name is only a handle, not a device address, so the
// address is fetched with cudaGetSymbolAddress (once per device, with that device current)
// and that pointer is what the kernels receive.
#include "../../include/fta.h"

#include "fta_kernels.h"

#include <cuda_runtime.h>
#include <mutex>

namespace {

constexpr size_t kNoAllocMaxBytes = 64ull << 20;  // 64 MiB per GPU

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocMaxBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mu;

// Device address of the scratch array on the current device; looked up on first use.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fta::record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return fta::record_cuda_error(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return fta::record_cuda_error(e);
    if (!p) return fta::record_cuda_error(cudaErrorInvalidSymbol);
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return FTA_OK;
}

}  // namespace

extern "C" {

size_t fta_noalloc_max_bytes(void) { return kNoAllocMaxBytes; }

int fta_backward_noalloc(const FtaProblem* prob, const FtaTensor5* q, const FtaTensor5* k, const FtaTensor5* v,
                         const FtaTensor4* bias, const FtaTensor5* dout, const float* lse, const float* delta,
                         float sm_scale, const FtaTensor5* dq, const FtaTensor5* dk, const FtaTensor5* dv,
                         float* dbias_f32, void* dbias_cast, int32_t* status, void* stream) {
  if (!prob) return FTA_ERR_NULL;
  const size_t need = fta_bwd_workspace_bytes(prob);
  if (need == 0) {
    // let the regular entry point name the problem with the shape / dtype / head dimension
    return fta_backward(prob, q, k, v, bias, dout, lse, delta, sm_scale, dq, dk, dv, dbias_f32, dbias_cast,
                        reinterpret_cast<void*>(256), 0, status, stream);
  }
  if (need > kNoAllocMaxBytes) return FTA_ERR_TOO_LARGE;  // problem needs more scratch than the fixed array
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FTA_OK) return rc;
  // fta_backward zeroes the dQ accumulator and overwrites every other part of the scratch it
  // reads, so whatever the previous call left in the array does not matter.
  return fta_backward(prob, q, k, v, bias, dout, lse, delta, sm_scale, dq, dk, dv, dbias_f32, dbias_cast, scratch,
                      kNoAllocMaxBytes, status, stream);
}

}  // extern "C"
