// Single-token decode step of the Palimpsa operator (sm_100a): HBM-bound.
//
// Every sequence-head owns a (mu, I) state of V x K float32 pairs that must be read and written once
// per generated token (2 x 2 x V x K x 4 bytes; 262 144 B at V = K = 128), against ~1 KB of token
// inputs.  The kernel is therefore laid out for memory throughput only: a lane owns one float4 column
// group of a state row, so a warp reads and writes whole 512-byte rows; each warp issues the loads of
// RB rows (2 x RB 16-byte loads per lane) before it touches any of them, to keep enough bytes in
// flight; the update runs in place.  Outputs are reduced over the lanes of a row with one batched
// (transposed) butterfly per RB rows.
//
// Replaces the reference's use of fused_palimpsa_recurrent_fwd_kernel with T = 1 and a cached state
// (fused_recurrent_palimpsa.py:24-154 called from palimpsa/layers/palimpsa.py:317-331), including the
// seven separate float32 casts it makes per step (fused_recurrent_palimpsa.py:226-236).
#include "common.cuh"
#include "host.h"

namespace palimpsa {

struct DecArgs {
    palimpsa_problem p;
    void* o;
    void* o_var;
    float* final_mu;
    float* final_I;
};

template <int DT>
__device__ __forceinline__ float4 ldg4(const void* base, long long idx) {  // idx: element index, multiple of 4
    if (DT == PALIMPSA_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(base) + idx);
    float2 a, b;
    if (DT == PALIMPSA_BF16) {
        a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    } else {
        a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
    }
    return make_float4(a.x, a.y, b.x, b.y);
}

// KL lanes cover one state row (KL * 4 = padded d_k); a warp handles 32/KL rows side by side and RB such
// row sets per pass.
template <int KL, int RB, bool UNC, int DT>
__global__ void __launch_bounds__(128) decode_kernel(const DecArgs a) {
    constexpr int RG = 32 / KL, ROWS_PER_WARP = RG * RB, NRED = RB * (UNC ? 2 : 1);
    const palimpsa_problem& p = a.p;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int kl = lane % KL, rg = lane / KL;
    const int nh = blockIdx.y, h = nh % p.H;
    const int K = p.K, V = p.V;
    const int kc = 4 * kl;
    const bool kin = kc < K;
    const int rbase = (blockIdx.x * 4 + w) * ROWS_PER_WARP + rg;  // rows rbase + i*RG, i < RB

    // ---- state rows first: everything else hides behind these loads ----------------------------------
    const long long sbase = (long long)nh * V * K + kc;
    float4 mu[RB], pr[RB];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        const int row = rbase + i * RG;
        if (kin && row < V) {
            mu[i] = __ldcs(reinterpret_cast<const float4*>(p.init_mu + sbase + (long long)row * K));
            pr[i] = __ldcs(reinterpret_cast<const float4*>(p.init_I + sbase + (long long)row * K));
        } else {
            mu[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            pr[i] = make_float4(1.f, 1.f, 1.f, 1.f);
        }
    }
    // ---- token inputs ------------------------------------------------------------------------------------
    float4 k4 = make_float4(0.f, 0.f, 0.f, 0.f), q4 = k4;
    if (kin) {
        k4 = ldg4<DT>(p.k, (long long)nh * K + kc);
        q4 = ldg4<DT>(p.q, (long long)nh * K + kc);
    }
    const float sc = p.scale;
    q4 = make_float4(q4.x * sc, q4.y * sc, q4.z * sc, q4.w * sc);
    const float4 kk4 = make_float4(k4.x * k4.x, k4.y * k4.y, k4.z * k4.z, k4.w * k4.w);
    const float f = expf(-p.gt[nh] * p.g[h]);
    const float c = (1.f - f) * p.Ip[h];
    float red[NRED];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        const int row = rbase + i * RG;
        float vv = 0.f, bb = 0.f;
        if (row < V) {
            vv = ld1<DT>(p.v, (long long)nh * V + row);
            bb = ld1<DT>(p.b, (long long)nh * V + row);
        }
        float y = 0.f, yv = 0.f;
        auto upd = [&](float& m, float& pi, float kx, float kkx, float qx) {
            const float fi = f * pi;
            const float mm = fmaf(m, fi, vv * kx);          // f * (mu*I) + v k
            const float in = fi + fmaf(bb, kkx, c);         // f * I + (1-f) Ip + b k^2
            float r = rcp_approx(in);
            r = fmaf(r, fmaf(-in, r, 1.f), r);              // one Newton step: the stored mean keeps full precision
            m = mm * r;
            pi = in;
            y = fmaf(m, qx, y);
            if (UNC) yv = fmaf(r, qx * qx, yv);
        };
        upd(mu[i].x, pr[i].x, k4.x, kk4.x, q4.x);
        upd(mu[i].y, pr[i].y, k4.y, kk4.y, q4.y);
        upd(mu[i].z, pr[i].z, k4.z, kk4.z, q4.z);
        upd(mu[i].w, pr[i].w, k4.w, kk4.w, q4.w);
        if (kin && row < V) {
            __stcs(reinterpret_cast<float4*>(a.final_mu + sbase + (long long)row * K), mu[i]);
            __stcs(reinterpret_cast<float4*>(a.final_I + sbase + (long long)row * K), pr[i]);
        }
        red[i * (UNC ? 2 : 1)] = y;
        // o_var = scale * sum q^2 / I with q already scaled once: divide one scale back out
        if (UNC) red[i * 2 + 1] = (sc != 0.f) ? yv / sc : 0.f;
    }
    xreduce<NRED, KL>(red, lane);
    constexpr int REM = NRED >= KL ? NRED / KL : 1;
    const int base = xreduce_index<NRED, KL>(lane);
    const bool owner = NRED >= KL ? true : (kl & (KL / (NRED < KL ? NRED : KL) - 1)) == 0;
    if (owner) {
#pragma unroll
        for (int j = 0; j < REM; ++j) {
            const int id = base + j;
            const int which = UNC ? (id & 1) : 0;
            const int i = UNC ? (id >> 1) : id;
            const int row = rbase + i * RG;
            if (row < V) st1(which ? a.o_var : a.o, (long long)nh * V + row, red[j], p.io_dtype);
        }
    }
}

template <int KL, int RB>
static int launch_decode_t(const DecArgs& a, cudaStream_t stream) {
    const palimpsa_problem& p = a.p;
    constexpr int ROWS_PER_CTA = 4 * (32 / KL) * RB;
    dim3 grid((p.V + ROWS_PER_CTA - 1) / ROWS_PER_CTA, p.num_seqs * p.H, 1);
    const bool unc = (p.flags & PALIMPSA_FLAG_UNCERTAINTY) != 0;
#define PALIMPSA_DEC_LAUNCH(U, D) decode_kernel<KL, RB, U, D><<<grid, 128, 0, stream>>>(a)
    if (p.io_dtype == PALIMPSA_BF16) {
        if (unc) PALIMPSA_DEC_LAUNCH(true, PALIMPSA_BF16); else PALIMPSA_DEC_LAUNCH(false, PALIMPSA_BF16);
    } else if (p.io_dtype == PALIMPSA_F32) {
        if (unc) PALIMPSA_DEC_LAUNCH(true, PALIMPSA_F32); else PALIMPSA_DEC_LAUNCH(false, PALIMPSA_F32);
    } else {
        if (unc) PALIMPSA_DEC_LAUNCH(true, PALIMPSA_F16); else PALIMPSA_DEC_LAUNCH(false, PALIMPSA_F16);
    }
#undef PALIMPSA_DEC_LAUNCH
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

// True if the dedicated decode kernel covers this call (else the general forward kernel runs it).
bool decode_supported(const palimpsa_fwd_params* prm) {
    const palimpsa_problem& p = prm->p;
    if (p.cu_seqlens || p.seq_len != 1 || !p.init_mu || !prm->final_mu || prm->ckpt_M) return false;
    if (p.K % 8 != 0 || p.K > 128) return false;
    const int KP = palimpsa_padded_k(p.K);
    if (KP != 16 && KP != 32 && KP != 64 && KP != 128) return false;
    auto al = [](const void* x, int m) { return (reinterpret_cast<uintptr_t>(x) & (m - 1)) == 0; };
    return al(p.q, 16) && al(p.k, 16) && al(p.init_mu, 16) && al(p.init_I, 16) && al(prm->final_mu, 16) &&
           al(prm->final_I, 16);
}

int launch_decode(const palimpsa_fwd_params* prm, cudaStream_t stream) {
    DecArgs a;
    a.p = prm->p;
    a.o = prm->o;
    a.o_var = prm->o_var;
    a.final_mu = prm->final_mu;
    a.final_I = prm->final_I;
    switch (palimpsa_padded_k(a.p.K)) {
        case 16: return launch_decode_t<4, 2>(a, stream);
        case 32: return launch_decode_t<8, 4>(a, stream);
        case 64: return launch_decode_t<16, 4>(a, stream);
        case 128: return launch_decode_t<32, 8>(a, stream);
        default: return PALIMPSA_E_DIM;
    }
}

}  // namespace palimpsa
