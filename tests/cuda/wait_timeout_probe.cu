// Test-only kernel (never part of libfta.so): exercises the bounded mbarrier wait of the product
// kernels (csrc/tc05.cuh: mbar_wait / mbar_wait_warp) when nobody arrives. The wait is given a
// limit of a few milliseconds; it must run out, record 0x1000 | site in the status word, raise
// the CTA's abort flag, let every role reach the tear-down (tensor memory freed) and return - no
// trap, no hang - so that the context stays usable for the next launch.
//
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC -I <csrc> ...
#include <cuda_runtime.h>
#include <stdint.h>

#include "tc05.cuh"

using namespace fta;

__global__ void __launch_bounds__(64) wait_probe_kernel(int* status, int arrive, unsigned long long limit_ns,
                                                        unsigned long long* waited_ns) {
  __shared__ uint64_t bar_storage;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  const WaitCtx w{smem_u32(&abort_flag), status, limit_ns};
  if (warp == 0) {
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait_warp(bar, 0, w, 0x7);  // site id 7
    if (threadIdx.x == 0) *waited_ns = ok ? 0ull : global_timer_ns() - t0;
  } else if (threadIdx.x == 32 && arrive) {
    mbar_arrive(bar);  // the healthy case: the producer role does its part
  }
  // tear-down, as in the product kernels
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 32);
}

extern "C" int wait_probe_launch(int* status, int arrive, unsigned long long limit_ns, unsigned long long* waited_ns,
                                 void* stream) {
  wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, arrive, limit_ns, waited_ns);
  return static_cast<int>(cudaGetLastError());
}
