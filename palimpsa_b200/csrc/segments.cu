// Boundary scans over the segments of a sequence (sm_100a): tiny HBM-bound element-wise kernels.
//
// Forward: the state recurrence is linear in (M, J = I - Ip) with one scalar decay per head, so the
// state at the start of segment g+1 is  decay_g * S_g + sum_g  where sum_g is the end state of
// segment g started from zero.  Backward: the gradient w.r.t. a segment's end state obeys
// carry_{g-1} = rloc_g + decay_g * carry_g  with rloc_g the start-state gradient obtained from a
// zero end-state gradient.  One thread walks the G segments of one float4 of state.
// The reference has no counterpart (it never splits a sequence).
#include "common.cuh"
#include "host.h"

namespace palimpsa {

__device__ __forceinline__ float4 f4_axpy(float a, float4 x, float4 y) {
    return make_float4(fmaf(a, x.x, y.x), fmaf(a, x.y, y.y), fmaf(a, x.z, y.z), fmaf(a, x.w, y.w));
}

__global__ void combine_fwd_kernel(const palimpsa_problem p, const palimpsa_segments sg, const float* __restrict__ in_M,
                                   const float* __restrict__ in_J, float* __restrict__ out_M,
                                   float* __restrict__ out_J, int KP, long long total4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int K4 = KP / 4, G = sg.num_segments;
    const int c4 = (int)(i % K4);
    const long long row = i / K4;  // (n*H + h)*V + v
    const int v = (int)(row % p.V);
    const long long nh = row / p.V;
    const int h = (int)(nh % p.H);
    const long long n = nh / p.H;
    const float ip = p.Ip[h];
    float4 M = make_float4(0.f, 0.f, 0.f, 0.f), J = M;
    if (in_M) {
        M = reinterpret_cast<const float4*>(in_M)[i];
        J = reinterpret_cast<const float4*>(in_J)[i];
    } else if (p.init_mu) {
        const long long e = row * p.K + 4 * c4;
        float mu[4] = {0.f, 0.f, 0.f, 0.f}, pr[4] = {ip, ip, ip, ip};
        for (int c = 0; c < 4; ++c)
            if (4 * c4 + c < p.K) {
                mu[c] = p.init_mu[e + c];
                pr[c] = p.init_I[e + c];
            }
        M = make_float4(mu[0] * pr[0], mu[1] * pr[1], mu[2] * pr[2], mu[3] * pr[3]);
        J = make_float4(pr[0] - ip, pr[1] - ip, pr[2] - ip, pr[3] - ip);
    }
    for (int g = 0; g < G; ++g) {
        const long long e = ((((n * G + g) * p.H + h) * p.V + v) * (long long)KP) / 4 + c4;
        reinterpret_cast<float4*>(sg.start_M)[e] = M;
        reinterpret_cast<float4*>(sg.start_I)[e] = make_float4(J.x + ip, J.y + ip, J.z + ip, J.w + ip);
        const float d = sg.decay[(n * G + g) * p.H + h];
        M = f4_axpy(d, M, reinterpret_cast<const float4*>(sg.sum_M)[e]);
        J = f4_axpy(d, J, reinterpret_cast<const float4*>(sg.sum_J)[e]);
    }
    if (out_M) {
        reinterpret_cast<float4*>(out_M)[i] = M;
        reinterpret_cast<float4*>(out_J)[i] = J;
    }
}

__global__ void combine_bwd_kernel(const palimpsa_problem p, const palimpsa_segments sg, const float* __restrict__ in_M,
                                   const float* __restrict__ in_I, float* __restrict__ out_M,
                                   float* __restrict__ out_I, int KP, long long total4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int K4 = KP / 4, G = sg.num_segments;
    const int c4 = (int)(i % K4);
    const long long row = i / K4;
    const int v = (int)(row % p.V);
    const long long nh = row / p.V;
    const int h = (int)(nh % p.H);
    const long long n = nh / p.H;
    float4 CM = make_float4(0.f, 0.f, 0.f, 0.f), CI = CM;
    if (in_M) {
        CM = reinterpret_cast<const float4*>(in_M)[i];
        CI = reinterpret_cast<const float4*>(in_I)[i];
    }
    for (int g = G - 1; g >= 0; --g) {
        const long long e = ((((n * G + g) * p.H + h) * p.V + v) * (long long)KP) / 4 + c4;
        reinterpret_cast<float4*>(sg.carry_M)[e] = CM;
        reinterpret_cast<float4*>(sg.carry_I)[e] = CI;
        const float d = sg.decay[(n * G + g) * p.H + h];
        CM = f4_axpy(d, CM, reinterpret_cast<const float4*>(sg.rloc_M)[e]);
        CI = f4_axpy(d, CI, reinterpret_cast<const float4*>(sg.rloc_I)[e]);
    }
    if (out_M) {
        reinterpret_cast<float4*>(out_M)[i] = CM;
        reinterpret_cast<float4*>(out_I)[i] = CI;
    }
}

// What a rank in the middle of a context-parallel chain adds to a state that passes through it, computed BEFORE
// the state arrives: forward, the end state of its segments from a zero start; backward, the start-state gradient
// from a zero end-state gradient.  No other output (the segments' own start states / carries need the true value).
__global__ void relay_total_kernel(const palimpsa_problem p, const palimpsa_segments sg, int backward,
                                   float* __restrict__ tot_A, float* __restrict__ tot_B, int KP, long long total4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int K4 = KP / 4, G = sg.num_segments;
    const int c4 = (int)(i % K4);
    const long long row = i / K4;
    const int v = (int)(row % p.V);
    const long long nh = row / p.V;
    const int h = (int)(nh % p.H);
    const long long n = nh / p.H;
    const float* srcA = backward ? sg.rloc_M : sg.sum_M;
    const float* srcB = backward ? sg.rloc_I : sg.sum_J;
    float4 A = make_float4(0.f, 0.f, 0.f, 0.f), B = A;
    for (int s = 0; s < G; ++s) {
        const int g = backward ? G - 1 - s : s;
        const long long e = ((((n * G + g) * p.H + h) * p.V + v) * (long long)KP) / 4 + c4;
        const float d = sg.decay[(n * G + g) * p.H + h];
        A = f4_axpy(d, A, reinterpret_cast<const float4*>(srcA)[e]);
        B = f4_axpy(d, B, reinterpret_cast<const float4*>(srcB)[e]);
    }
    reinterpret_cast<float4*>(tot_A)[i] = A;
    reinterpret_cast<float4*>(tot_B)[i] = B;
}

// The hop itself: out = (product of the rank's segment decays) * in + total.  3 state-sized streams; the output
// usually lies in the next rank's memory (peer-mapped pointer, plain stores over NVLink).
__global__ void relay_kernel(const palimpsa_problem p, const palimpsa_segments sg, const float* __restrict__ in_A,
                             const float* __restrict__ in_B, const float* __restrict__ tot_A,
                             const float* __restrict__ tot_B, float* __restrict__ out_A, float* __restrict__ out_B,
                             int KP, long long total4) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int G = sg.num_segments;
    const long long nh = i / (KP / 4) / p.V;
    const int h = (int)(nh % p.H);
    const long long n = nh / p.H;
    float P = 1.f;
    for (int g = 0; g < G; ++g) P *= sg.decay[(n * G + g) * p.H + h];
    reinterpret_cast<float4*>(out_A)[i] =
        f4_axpy(P, reinterpret_cast<const float4*>(in_A)[i], reinterpret_cast<const float4*>(tot_A)[i]);
    reinterpret_cast<float4*>(out_B)[i] =
        f4_axpy(P, reinterpret_cast<const float4*>(in_B)[i], reinterpret_cast<const float4*>(tot_B)[i]);
}

int launch_relay_total(const palimpsa_problem& p, const palimpsa_segments& segs, int backward, float* tot_A,
                       float* tot_B, cudaStream_t stream) {
    const int KP = palimpsa_padded_k(p.K);
    const long long total4 = (long long)p.num_seqs * p.H * p.V * (KP / 4);
    if (total4 == 0) return PALIMPSA_OK;
    relay_total_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(p, segs, backward, tot_A, tot_B, KP, total4);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int launch_relay(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_A, const float* in_B,
                 const float* tot_A, const float* tot_B, float* out_A, float* out_B, cudaStream_t stream) {
    const int KP = palimpsa_padded_k(p.K);
    const long long total4 = (long long)p.num_seqs * p.H * p.V * (KP / 4);
    if (total4 == 0) return PALIMPSA_OK;
    relay_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(p, segs, in_A, in_B, tot_A, tot_B, out_A, out_B,
                                                                      KP, total4);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int launch_combine_fwd(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_M, const float* in_J,
                       float* out_M, float* out_J, cudaStream_t stream) {
    const int KP = palimpsa_padded_k(p.K);
    const long long total4 = (long long)p.num_seqs * p.H * p.V * (KP / 4);
    if (total4 == 0) return PALIMPSA_OK;
    combine_fwd_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(p, segs, in_M, in_J, out_M, out_J, KP,
                                                                            total4);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int launch_combine_bwd(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_M, const float* in_I,
                       float* out_M, float* out_I, cudaStream_t stream) {
    const int KP = palimpsa_padded_k(p.K);
    const long long total4 = (long long)p.num_seqs * p.H * p.V * (KP / 4);
    if (total4 == 0) return PALIMPSA_OK;
    combine_bwd_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, stream>>>(p, segs, in_M, in_I, out_M, out_I, KP,
                                                                            total4);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

}  // namespace palimpsa
