// Shared device helpers for the Palimpsa sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/palimpsa_b200.h"

namespace palimpsa {

// Tokens per staged block.  Equal to the checkpoint interval, so that every staged block of a
// sequence starts on a checkpoint.
constexpr int TB = PALIMPSA_CKPT_INTERVAL;

// ---------------------------------------------------------------------------------------------
// Packed FP32 arithmetic: sm_100 executes two FP32 lanes per instruction on 64-bit register
// pairs (fma.rn.f32x2 and friends), halving the issue slots of the element-wise recurrence.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 dup2(float x) { return make_float2(x, x); }

// One MUFU op, relative error <= 2^-23.
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float2 rcp2(float2 x) { return make_float2(rcp_approx(x.x), rcp_approx(x.y)); }

// ---------------------------------------------------------------------------------------------
// Asynchronous global->shared copies (LDGSTS).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
    unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------
// io dtype handling.  DT is PALIMPSA_F32 / BF16 / F16.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int dtype_size(int dt) { return dt == PALIMPSA_F32 ? 4 : 2; }

// Four consecutive values, group index idx4, from a 16-byte aligned buffer (shared or global).
template <int DT>
__device__ __forceinline__ float4 ld4(const void* base, int idx4) {
    if (DT == PALIMPSA_F32) {
        return reinterpret_cast<const float4*>(base)[idx4];
    } else {
        uint2 u = reinterpret_cast<const uint2*>(base)[idx4];
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
}

// One value from global memory, any alignment.
template <int DT>
__device__ __forceinline__ float ld1(const void* base, long long idx) {
    if (DT == PALIMPSA_F32) return reinterpret_cast<const float*>(base)[idx];
    if (DT == PALIMPSA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    return __half2float(reinterpret_cast<const __half*>(base)[idx]);
}

// Four values starting at element idx, each read only if its index is below limit (else 0).
template <int DT>
__device__ __forceinline__ float4 ld4_guarded(const void* base, long long idx, long long limit) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (idx + 0 < limit) r.x = ld1<DT>(base, idx + 0);
    if (idx + 1 < limit) r.y = ld1<DT>(base, idx + 1);
    if (idx + 2 < limit) r.z = ld1<DT>(base, idx + 2);
    if (idx + 3 < limit) r.w = ld1<DT>(base, idx + 3);
    return r;
}

__device__ __forceinline__ void st1(void* base, long long idx, float x, int dt) {
    if (dt == PALIMPSA_F32)
        reinterpret_cast<float*>(base)[idx] = x;
    else if (dt == PALIMPSA_BF16)
        reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x);
    else
        reinterpret_cast<__half*>(base)[idx] = __float2half_rn(x);
}

__host__ __device__ __forceinline__ int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Token range of sequence n.
__device__ __forceinline__ void seq_range(const palimpsa_problem& p, int n, int& bos, int& len) {
    if (p.cu_seqlens) {
        bos = p.cu_seqlens[n];
        len = p.cu_seqlens[n + 1] - bos;
    } else {
        bos = n * p.seq_len;
        len = p.seq_len;
    }
    if (len < 0) len = 0;
}

// First checkpoint slot of sequence n.
__device__ __forceinline__ long long seq_first_slot(const palimpsa_problem& p, int n) {
    if (p.chunk_offsets) return p.chunk_offsets[n];
    return (long long)n * ((p.seq_len + TB - 1) / TB);
}

// Store four values as duplicated pairs {x,x,y,y},{z,z,w,w} (operands of packed FP32 instructions).
__device__ __forceinline__ void st_dup4(float4* dst, int i, float4 x) {
    dst[2 * i] = make_float4(x.x, x.x, x.y, x.y);
    dst[2 * i + 1] = make_float4(x.z, x.z, x.w, x.w);
}


// How the threads of a CTA split the 16-byte chunks of a [tokens][chunks] tile among themselves: thread ->
// (first token, chunk), then every `step` tokens.  Computed once per kernel, so that the per-block copy loops
// carry no integer division.  `step` = 0: the thread count is not a multiple of the chunk count (generic loop).
struct ChunkSplit {
    int t0, c, step;
};
__device__ __forceinline__ ChunkSplit chunk_split(int chunks, int nthr, int tid) {
    ChunkSplit s{0, 0, 0};
    if (chunks > 0 && chunks <= nthr && nthr % chunks == 0) {
        s.t0 = tid / chunks;
        s.c = tid - s.t0 * chunks;
        s.step = nthr / chunks;
    }
    return s;
}

// Sum N per-lane values over the L lanes that differ from this one in the low log2(L) bits
// (L = 2^s <= 32).  "Transposed" butterfly: each step exchanges half of the remaining values, so it
// costs N-1 (+ a few) shuffles instead of N*log2(L).  On return x[i], i < max(1, N/L), holds the sum of
// value xreduce_index<N, L>(lane) + i.
template <int N, int L>
__device__ __forceinline__ void xreduce(float (&x)[N], int lane) {
    int n = N;
#pragma unroll
    for (int off = L / 2; off >= 1; off >>= 1) {
        if (n > 1) {
            const int half = n / 2;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < N / 2; ++i) {
                if (i < half) {
                    const float keep = up ? x[i + half] : x[i];
                    const float send = up ? x[i] : x[i + half];
                    x[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            n = half;
        } else {
            x[0] += __shfl_xor_sync(0xffffffffu, x[0], off);
        }
    }
}
template <int N, int L>
__device__ __forceinline__ int xreduce_index(int lane) {
    int idx = 0, n = N;
#pragma unroll
    for (int off = L / 2; off >= 1; off >>= 1) {
        if (n > 1) {
            n /= 2;
            if (lane & off) idx += n;
        }
    }
    return idx;
}

}  // namespace palimpsa
