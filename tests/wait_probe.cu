// Test-only library (NOT part of libpalimpsa_b200.so): runs the bounded mbarrier wait of the product kernels
// (tc::mbar_wait, palimpsa_b200/csrc/tc_common.cuh) to its give-up path on purpose, the way the tensor-core
// kernels would meet it: one small CTA allocates TMEM, waits on an mbarrier with a poll limit given by the
// caller, records a status code, frees its TMEM and returns.  With `arrive` = 0 nobody ever arrives at the
// barrier, so the wait runs out by construction after `limit` polls (nothing hangs and nothing faults); with
// `arrive` = 1 one thread arrives first and the wait succeeds.
#include "../palimpsa_b200/csrc/tc_common.cuh"

namespace {

__global__ void __launch_bounds__(32) wait_probe_kernel(int arrive, unsigned limit, int* status) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ unsigned tmem_slot;
    using namespace palimpsa;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar);
        tc::mbar_init_fence();
    }
    tc::tmem_alloc(&tmem_slot, 32);
    tc::fence_before_sync();
    __syncwarp();
    tc::fence_after_sync();
    const unsigned tmem = tmem_slot;
    if (arrive && threadIdx.x == 0)
        asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(tc::smem_u32(&bar)) : "memory");
    __syncwarp();
    const bool ok = tc::mbar_wait(&bar, 0, limit);
    if (threadIdx.x == 0) *status = ok ? 0 : 7;     // 7: the probe's own code for "the wait gave up"
    __syncwarp();
    tc::fence_before_sync();
    tc::tmem_free(tmem, 32);
}

}  // namespace

// status_dev: one int in device memory.  Returns 0, or -1 if the launch was refused.
extern "C" int palimpsa_test_wait_probe(int arrive, unsigned limit, int* status_dev, void* cuda_stream) {
    wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(arrive, limit, status_dev);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
