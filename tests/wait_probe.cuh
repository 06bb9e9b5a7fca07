#pragma once
// Test-only kernel for the bounded-wait path of the attention kernels (not part of the product).
//
// One warp waits, through the same mbar_wait the attention kernels use, on an mbarrier that nothing
// ever arrives on.  No copy, no MMA and no tensor memory is in flight, so when the wait gives up the
// kernel simply returns: the test then reads the sticky status word the wait left behind, checks that
// a later launch returns at entry, and that clearing the status re-arms the library.  The wait's
// cycle budget is cut to about a millisecond for this translation unit.
#define FRAY_WAIT_LIMIT_CYCLES 2000000LL
#include "flash_attn/host_sm100.cuh"
#include "flash_attn/sm100_ptx.cuh"

namespace fray_test {

static constexpr unsigned int kProbeSite = 0x7E1;   // site code the probe's wait reports
static constexpr int kProbeExtra = 42;

// out[0]: 1 = the wait ran out and the kernel returned normally, 2 = the status was already raised and the
// kernel returned at entry (as every attention kernel does), 3 = the barrier flipped (cannot happen).
__global__ void wait_probe_kernel(int* out) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = (*reinterpret_cast<volatile int*>(&fray::sm100::fray_attn_status[0]) != 0) ? 2u : 0u;
    fray::sm100::mbar_init(&bar, 1);
    fray::sm100::fence_barrier_init();
  }
  __syncthreads();
  if (abort_flag != 0) {
    if (threadIdx.x == 0) out[0] = 2;
    return;
  }
  if (threadIdx.x < 32) fray::sm100::mbar_wait(&bar, 0, &abort_flag, kProbeSite, kProbeExtra);
  __syncthreads();
  if (threadIdx.x == 0) out[0] = abort_flag == 1u ? 1 : 3;
}

inline void launch_wait_probe(int* out, cudaStream_t stream, int& rc) {
  wait_probe_kernel<<<1, 64, 0, stream>>>(out);
  rc = cudaGetLastError() == cudaSuccess ? 0 : 8;
}

}  // namespace fray_test
