// Stream-ordered signalling between the GPUs of one node through peer-mapped memory.
//
// The context-parallel mode passes one small boundary state from rank to rank (forward) and one state gradient
// back (backward).  With the ranks' exchange buffers mapped into each other's address space, the producing
// kernel stores its result straight into the next rank's buffer over NVLink, and two one-thread kernels order
// the hand-over on the stream: `peer_signal_kernel` publishes a sequence number after everything the stream did
// before it (system-scope fence + release store into the peer's flag), `peer_wait_kernel` holds the stream until
// the local flag has reached a sequence number (acquire loads).  No host round trip and no library call per hop.
// The wait is bounded by a wall-clock limit: when it runs out, the kernel records a status code, poisons the
// buffer it guards with a NaN and returns, so the stream never hangs on a peer that died.
// The reference has no counterpart (it has no multi-GPU code of its own).
#include "host.h"

namespace palimpsa {

__device__ int g_peer_status = 0;   // 0 ok; 7: a wait on a peer's signal ran out

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void peer_wait_kernel(const unsigned long long* flag, unsigned long long value, unsigned long long limit_ns,
                                 float* poison) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
        if (v >= value) return;
        if (global_ns() - t0 > limit_ns) break;
        __nanosleep(100);
    }
    atomicCAS(&g_peer_status, 0, 7);
    if (poison) *poison = __int_as_float(0x7fc00000);
}

__global__ void peer_signal_kernel(unsigned long long* flag, unsigned long long value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(value) : "memory");
}

int launch_peer_wait(const void* flag, unsigned long long value, unsigned timeout_ms, float* poison, cudaStream_t stream) {
    peer_wait_kernel<<<1, 1, 0, stream>>>(static_cast<const unsigned long long*>(flag), value,
                                          (unsigned long long)timeout_ms * 1000000ull, poison);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int launch_peer_signal(void* flag, unsigned long long value, cudaStream_t stream) {
    peer_signal_kernel<<<1, 1, 0, stream>>>(static_cast<unsigned long long*>(flag), value);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int peer_status() {
    int s = 0;
    if (cudaMemcpyFromSymbol(&s, g_peer_status, sizeof(int)) != cudaSuccess) return -1;
    if (s) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return s;
}

}  // namespace palimpsa
