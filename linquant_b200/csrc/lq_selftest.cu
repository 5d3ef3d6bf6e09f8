// Self-test of the bounded waits the tcgen05 kernels rely on. Nothing here is on the product path: the entry exists so
// that a test suite can watch a wait run out -- status word raised, tensor memory released, kernel returned -- without
// faulting or hanging the GPU. The mbarrier is initialised with one expected arrival and nothing ever arrives on it
// (no TMA copy and no MMA is issued, so nothing is in flight when the wait gives up).
#include "lq_tc.cuh"

namespace lq {

__global__ void __launch_bounds__(128) selftest_wait_timeout_kernel(int* status, int* trace, int hold_tmem) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t s_tbase;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t bar_u32 = smem_u32(&bar);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(bar_u32));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (hold_tmem && warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tbase)), "r"(32u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  bool ok = true;
  if (tid == 0) {
    trace[0] = 1;
    ok = mbar_wait_bounded(bar_u32, 0);  // the same helper, with the same poll limit, as the product kernels
    if (!ok) trace[1] = 2;
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (!ok && tid == 0 && status != nullptr) atomicExch(status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (hold_tmem && warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(s_tbase), "r"(32u) : "memory");
    if (tid == 32) trace[2] = 3;
  }
  if (tid == 0) trace[3] = 4;
}

}  // namespace lq

extern "C" int lq_selftest_wait_timeout(int* status, int* trace, int hold_tmem, lq_stream stream) {
  if (!status || !trace) return lq::fail(LQ_ERR_NULL, "selftest_wait_timeout: status and trace are required");
  lq::selftest_wait_timeout_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, trace, hold_tmem);
  return lq::check_launch("selftest_wait_timeout_kernel");
}
