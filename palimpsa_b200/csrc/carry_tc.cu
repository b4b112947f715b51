// Carried-gradient terms of a segmented backward on the tensor cores (tcgen05 + TMEM), bf16 io.
//
// When a sequence is cut into segments, every segment's backward first runs with a ZERO gradient at its
// end state; the true end-state gradient R = (R_M, R_I) (from the later segments, or from the next rank)
// then adds terms that are linear in R (a_t = prod_{s>t} f_s to the segment's end):
//     dv_t += a_t (R_M k_t)            db_t += a_t (R_I k_t^2)
//     dk_t += a_t (R_M^T v_t + 2 k_t * (R_I^T b_t))
//     df_t += a_t c_t ,  c_{t+1} = f_t c_t + <R_M^T v_t, k_t> + <R_I^T b_t, k_t^2>,  c_first = <R_M, M_start> + <R_I, J_start>
//     sum(GI_t) += a_t sum(R_I)        (enters dIp)
// i.e. four [tokens x 128]*[128 x 128] products per segment plus per-token scalar work.  One CTA per
// (sequence, head, segment) keeps R (bf16, both orientations) resident in shared memory as UMMA B
// operands and walks the segment in 128-token tiles.  The token rows of k, v and b are A operands exactly as they
// lie in global memory (token-major, contraction dimension contiguous = K-major), so where the head dimensions
// allow it (d_k, d_v multiples of 64) they arrive by TMA: cp.async.bulk.tensor 2-D tiles of 128 tokens x 64
// elements with the 128-byte swizzle, completion on an mbarrier (complete_tx), descriptors in the matching
// swizzled layout; only k^2 is produced in registers (each thread squares its own token row into the unswizzled
// core-matrix layout).  Other shapes copy all four row sets by hand.  One thread issues the
// tcgen05.mma's into four TMEM accumulators, and every thread reads back the TMEM lane of its token and
// applies the result (read-modify-write of dv, db; dk / df / dIp terms into the extra partial slot the
// finishing kernels sum).  All waits are bounded.  The reference has no counterpart: it never splits a
// sequence; the algebra is the linear part of its backward (chunk_palimpsa_forgetting_scalar.py:380-430).
#include "host.h"
#include "tc_common.cuh"

namespace palimpsa {

constexpr int CT = 128;                    // tokens per tile = UMMA M
constexpr int C_LBO = 128;                 // bytes between K-direction core matrices
constexpr int C_SBO = 16 * 128 + 16;       // bytes between 8-row groups (K extent <= 128; padded against bank conflicts)
constexpr int C_OPER = 16 * C_SBO;         // one 128-row operand
constexpr int C_BOX = 128 * 128;           // one TMA box: 128 token rows x 64 bf16 (128 bytes), swizzled
constexpr int C_A0 = 2 * C_BOX;            // A0: up to two boxes side by side (contraction extent <= 128)
constexpr int C_A1 = (C_OPER + 1023) / 1024 * 1024;   // A1: by hand (k^2, unswizzled) or by TMA (b rows)
constexpr int C_MAXTILES = 1024;           // segment length limit: 131 072 tokens

__device__ int g_carry_status = 0;         // 0 ok; 3 / 4: the bounded wait after phase 1 / phase 2 gave up

struct CarryArgs {
    palimpsa_problem p;
    int seg_len;
    const float *carry_M, *carry_I;        // [N,G,H,V,KP]
    const float *ckpt_M, *ckpt_I;          // forward checkpoints: start state of the segment
    void *dv, *db;                         // read-modify-write, bf16
    float *dk_x, *df_x, *dip_x;            // extra partial slot: [rows][KP], [rows], [rows]
    int KP, VP;
};

struct CarryMaps {                         // tensor maps over this GPU's k, v, b: rows = tokens, row = H * d elements
    CUtensorMap k, v, b;
};

__device__ __forceinline__ unsigned char* core_addr(unsigned char* base, int row, int chunk) {
    return base + (row >> 3) * C_SBO + chunk * 128 + (row & 7) * 16;
}

template <bool TMA>
__global__ void __launch_bounds__(128) carry_tc_kernel(const CarryArgs a, const __grid_constant__ CarryMaps maps) {
    extern __shared__ __align__(128) unsigned char sm_raw[];
    // the TMA destinations want 1024-byte alignment (swizzle atom): round the dynamic base up
    unsigned char* sm = sm_raw + ((1024u - (tc::smem_u32(sm_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ __align__(8) unsigned long long tbar;   // completion of the TMA tile loads
    __shared__ unsigned tmem_slot;
    __shared__ float tail_s[C_MAXTILES];
    __shared__ float lf_s[CT];
    __shared__ float red_s[8];
    __shared__ float2 wtot_s[4];
    __shared__ float cnext_s;
    const palimpsa_problem& p = a.p;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    const int g = blockIdx.y, G = gridDim.y;
    const int KP = a.KP, VP = a.VP, K = p.K, V = p.V, H = p.H;
    int bos, len;
    seq_range(p, n, bos, len);
    const int s0 = min(len, g * a.seg_len), s1 = min(len, s0 + a.seg_len);
    if (s1 <= s0) return;
    const int ntiles = (s1 - s0 + CT - 1) / CT;
    const float gh = p.g[h], iph = p.Ip[h];
    const long long seg_row = (((long long)n * G + g) * H + h) * V;
    const bool has_init = p.init_mu != nullptr || (p.flags & PALIMPSA_FLAG_EXPLICIT_INIT);
    unsigned char* A0 = sm;                    // 1024-byte aligned: TMA destination (k rows, then v rows)
    unsigned char* A1 = sm + C_A0;             // 1024-byte aligned: k^2 by hand, then b rows by TMA
    unsigned char* B_RM = sm + C_A0 + C_A1;    // rows v, K = k      (for X = K R_M^T)
    unsigned char* B_RI = B_RM + C_OPER;
    unsigned char* B_RMt = B_RM + 2 * C_OPER;  // rows k, K = v      (for U = V R_M)
    unsigned char* B_RIt = B_RM + 3 * C_OPER;

    if (tid == 0) {
        tc::mbar_init(&bars[0]);
        tc::mbar_init(&bars[1]);
        tc::mbar_init(&tbar);
        tc::mbar_init_fence();
        if (TMA) {
            tc::tma_prefetch_map(&maps.k);
            tc::tma_prefetch_map(&maps.v);
            tc::tma_prefetch_map(&maps.b);
        }
    }
    if (w == 0) tc::tmem_alloc(&tmem_slot, 512);
    // ---- B operands: R in bf16, both orientations; zero everything first (padding rows / columns) ----
    for (int i = tid; i < (C_A0 + C_A1 + 4 * C_OPER) / 16; i += 128) reinterpret_cast<uint4*>(sm)[i] = make_uint4(0, 0, 0, 0);
    tc::fence_async_smem();   // these plain stores are ordered before the TMA writes into the same buffers
    __syncthreads();
    float c0 = 0.f, sri = 0.f;
    {
        const long long slot = seq_first_slot(p, n) + s0 / TB;
        const float* cM = a.carry_M + seg_row * KP;
        const float* cI = a.carry_I + seg_row * KP;
        const float* sM = a.ckpt_M + ((slot * H + h) * (long long)V) * KP;
        const float* sI = a.ckpt_I + ((slot * H + h) * (long long)V) * KP;
        const int C8 = KP / 8;
        for (int i = tid; i < V * C8; i += 128) {
            const int v = i / C8, c = i - v * C8;
            float rm[8], ri[8];
#pragma unroll
            for (int j = 0; j < 8; j += 4) {
                const float4 x = *reinterpret_cast<const float4*>(cM + (long long)v * KP + 8 * c + j);
                const float4 y = *reinterpret_cast<const float4*>(cI + (long long)v * KP + 8 * c + j);
                const float4 m = *reinterpret_cast<const float4*>(sM + (long long)v * KP + 8 * c + j);
                const float4 q = *reinterpret_cast<const float4*>(sI + (long long)v * KP + 8 * c + j);
                rm[j] = x.x, rm[j + 1] = x.y, rm[j + 2] = x.z, rm[j + 3] = x.w;
                ri[j] = y.x, ri[j + 1] = y.y, ri[j + 2] = y.z, ri[j + 3] = y.w;
                c0 += x.x * m.x + x.y * m.y + x.z * m.z + x.w * m.w;
                c0 += y.x * (q.x - iph) + y.y * (q.y - iph) + y.z * (q.z - iph) + y.w * (q.w - iph);
                sri += y.x + y.y + y.z + y.w;
            }
            *reinterpret_cast<uint4*>(core_addr(B_RM, v, c)) =
                make_uint4(tc::pack_bf16(rm[0], rm[1]), tc::pack_bf16(rm[2], rm[3]), tc::pack_bf16(rm[4], rm[5]),
                           tc::pack_bf16(rm[6], rm[7]));
            *reinterpret_cast<uint4*>(core_addr(B_RI, v, c)) =
                make_uint4(tc::pack_bf16(ri[0], ri[1]), tc::pack_bf16(ri[2], ri[3]), tc::pack_bf16(ri[4], ri[5]),
                           tc::pack_bf16(ri[6], ri[7]));
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // transposed copies: row k = 8c + j, K index v
                const int kr = 8 * c + j;
                *reinterpret_cast<__nv_bfloat16*>(core_addr(B_RMt, kr, v >> 3) + (v & 7) * 2) = __float2bfloat16_rn(rm[j]);
                *reinterpret_cast<__nv_bfloat16*>(core_addr(B_RIt, kr, v >> 3) + (v & 7) * 2) = __float2bfloat16_rn(ri[j]);
            }
        }
    }
    // block sums of c0 and sum(R_I)
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        c0 += __shfl_xor_sync(0xffffffffu, c0, off);
        sri += __shfl_xor_sync(0xffffffffu, sri, off);
    }
    if (lane == 0) {
        red_s[w] = c0;
        red_s[4 + w] = sri;
    }
    // ---- log-decay of every tile, then the sum over the tiles after each one ----
    for (int j = 0; j < ntiles; ++j) {
        const int t = s0 + j * CT + tid;
        float lf = t < s1 ? -p.gt[((long long)bos + t) * H + h] * gh : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) lf += __shfl_xor_sync(0xffffffffu, lf, off);
        if (lane == 0) lf_s[w] = lf;
        __syncthreads();
        if (tid == 0) tail_s[j] = lf_s[0] + lf_s[1] + lf_s[2] + lf_s[3];
        __syncthreads();
    }
    if (tid == 0) {
        float run = 0.f;
        for (int j = ntiles - 1; j >= 0; --j) {
            const float x = tail_s[j];
            tail_s[j] = run;
            run += x;
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const unsigned tmem = tmem_slot;
    float c_run = red_s[0] + red_s[1] + red_s[2] + red_s[3];
    const float SRI = red_s[4] + red_s[5] + red_s[6] + red_s[7];
    const unsigned idesc_v = tc::idesc_bf16(VP), idesc_k = tc::idesc_bf16(KP);
    const unsigned lane_base = (unsigned)(32 * w) << 16;
    int status = 0;
    unsigned tpar = 0;                     // thread 0: parity of the next completion of tbar
    const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);
    const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
    const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(p.b);
    __nv_bfloat16* odv = reinterpret_cast<__nv_bfloat16*>(a.dv);
    __nv_bfloat16* odb = reinterpret_cast<__nv_bfloat16*>(a.db);
    for (int j = 0; j < ntiles; ++j) {
        const int t0 = s0 + j * CT;
        const int nt = min(CT, s1 - t0);
        const bool live = tid < nt;
        const long long row = ((long long)bos + t0 + tid) * H + h;     // this thread's (token, head) row
        const unsigned par = (unsigned)(j & 1);
        // ---- per-token scalars: f_t and a_t = exp(sum of log f over the later tokens of the segment) ----
        const float lf = live ? -p.gt[row] * gh : 0.f;
        lf_s[tid] = lf;
        __syncthreads();
        float sfx = tail_s[j];
        for (int s = tid + 1; s < nt; ++s) sfx += lf_s[s];
        const float f_t = __expf(lf);
        const float a_t = live ? __expf(sfx) : 0.f;

        // ---- phase 1 operands: A0 = k rows (TMA, or copied by hand), A1 = k*k rows (each thread squares its own row) ----
        if (TMA && tid == 0 && status == 0) {
            tc::mbar_expect_tx(&tbar, (unsigned)(KP / 64) * C_BOX);
            for (int i = 0; i < KP / 64; ++i)
                tc::tma_load_2d(A0 + i * C_BOX, &maps.k, h * K + 64 * i, (int)(bos + t0), &tbar);
        }
        for (int c = 0; c < KP / 8; ++c) {
            uint4 x = make_uint4(0, 0, 0, 0);
            if (live && 8 * c < K) x = *reinterpret_cast<const uint4*>(gk + row * K + 8 * c);
            if (!TMA) *reinterpret_cast<uint4*>(core_addr(A0, tid, c)) = x;
            const unsigned u[4] = {x.x, x.y, x.z, x.w};
            unsigned sq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 fx = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[i]));
                sq[i] = tc::pack_bf16(fx.x * fx.x, fx.y * fx.y);
            }
            *reinterpret_cast<uint4*>(core_addr(A1, tid, c)) = make_uint4(sq[0], sq[1], sq[2], sq[3]);
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (tid == 0 && status == 0) {
            tc::fence_after_sync();
            if (TMA) {
                if (!tc::mbar_wait(&tbar, tpar)) status = 3;
                tpar ^= 1;
            }
        }
        if (tid == 0 && status == 0) {
            const unsigned a0 = tc::smem_u32(A0), a1 = tc::smem_u32(A1), brm = tc::smem_u32(B_RM), bri = tc::smem_u32(B_RI);
            for (int kk = 0; kk < KP / 16; ++kk) {
                // a swizzled box holds 4 steps of K = 16 (32 bytes each); the next box is C_BOX further
                const unsigned long long dA0 = TMA ? tc::desc_sw128(a0 + (kk >> 2) * C_BOX + (kk & 3) * 32)
                                                   : tc::desc(a0 + kk * 256, C_LBO, C_SBO);
                tc::mma(tmem + 0, dA0, tc::desc(brm + kk * 256, C_LBO, C_SBO), idesc_v, kk > 0);
                tc::mma(tmem + 128, tc::desc(a1 + kk * 256, C_LBO, C_SBO), tc::desc(bri + kk * 256, C_LBO, C_SBO), idesc_v, kk > 0);
            }
            tc::commit(&bars[0]);
        }
        if (status == 0 && !tc::mbar_wait(&bars[0], par)) status = 3;
        tc::fence_after_sync();
        // ---- phase 2 operands: A0 = v rows, A1 = b rows (the phase-1 MMAs have finished reading A0/A1) ----
        if (TMA) {
            if (tid == 0 && status == 0) {
                tc::mbar_expect_tx(&tbar, 2u * (unsigned)(VP / 64) * C_BOX);
                for (int i = 0; i < VP / 64; ++i) {
                    tc::tma_load_2d(A0 + i * C_BOX, &maps.v, h * V + 64 * i, (int)(bos + t0), &tbar);
                    tc::tma_load_2d(A1 + i * C_BOX, &maps.b, h * V + 64 * i, (int)(bos + t0), &tbar);
                }
            }
        } else {
            for (int c = 0; c < VP / 8; ++c) {
                uint4 x = make_uint4(0, 0, 0, 0), y = x;
                if (live && 8 * c < V) {
                    x = *reinterpret_cast<const uint4*>(gv + row * V + 8 * c);
                    y = *reinterpret_cast<const uint4*>(gb + row * V + 8 * c);
                }
                *reinterpret_cast<uint4*>(core_addr(A0, tid, c)) = x;
                *reinterpret_cast<uint4*>(core_addr(A1, tid, c)) = y;
            }
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (tid == 0 && status == 0) {
            tc::fence_after_sync();
            if (TMA) {
                if (!tc::mbar_wait(&tbar, tpar)) status = 4;
                tpar ^= 1;
            }
        }
        if (tid == 0 && status == 0) {
            const unsigned a0 = tc::smem_u32(A0), a1 = tc::smem_u32(A1), brm = tc::smem_u32(B_RMt), bri = tc::smem_u32(B_RIt);
            for (int kk = 0; kk < VP / 16; ++kk) {
                const unsigned so = (kk >> 2) * C_BOX + (kk & 3) * 32;
                const unsigned long long dA0 = TMA ? tc::desc_sw128(a0 + so) : tc::desc(a0 + kk * 256, C_LBO, C_SBO);
                const unsigned long long dA1 = TMA ? tc::desc_sw128(a1 + so) : tc::desc(a1 + kk * 256, C_LBO, C_SBO);
                tc::mma(tmem + 256, dA0, tc::desc(brm + kk * 256, C_LBO, C_SBO), idesc_k, kk > 0);
                tc::mma(tmem + 384, dA1, tc::desc(bri + kk * 256, C_LBO, C_SBO), idesc_k, kk > 0);
            }
            tc::commit(&bars[1]);
        }
        // ---- epilogue of phase 1 (runs while the phase-2 MMAs execute): dv += a X, db += a Y ----
        if (status == 0) {
            for (int c0 = 0; c0 < VP; c0 += 32) {
                float x[32], y[32];
                tc::tmem_ld32(tmem + lane_base + 0 + c0, x);
                tc::tmem_ld32(tmem + lane_base + 128 + c0, y);
                if (live) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int col = c0 + 8 * q;
                        if (col < V) {
                            uint4 dvv = *reinterpret_cast<const uint4*>(odv + row * V + col);
                            uint4 dbv = *reinterpret_cast<const uint4*>(odb + row * V + col);
                            unsigned* pv = reinterpret_cast<unsigned*>(&dvv);
                            unsigned* pb = reinterpret_cast<unsigned*>(&dbv);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float2 fv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pv[i]));
                                float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pb[i]));
                                fv.x = fmaf(a_t, x[8 * q + 2 * i], fv.x);
                                fv.y = fmaf(a_t, x[8 * q + 2 * i + 1], fv.y);
                                fb.x = fmaf(a_t, y[8 * q + 2 * i], fb.x);
                                fb.y = fmaf(a_t, y[8 * q + 2 * i + 1], fb.y);
                                pv[i] = tc::pack_bf16(fv.x, fv.y);
                                pb[i] = tc::pack_bf16(fb.x, fb.y);
                            }
                            *reinterpret_cast<uint4*>(odv + row * V + col) = dvv;
                            *reinterpret_cast<uint4*>(odb + row * V + col) = dbv;
                        }
                    }
                }
            }
        }
        if (status == 0 && !tc::mbar_wait(&bars[1], par)) status = 4;
        tc::fence_after_sync();
        // ---- epilogue of phase 2: dk terms into the extra slot, and w_t = <U,k> + <W,k*k> ----
        float w_t = 0.f;
        if (status == 0) {
            for (int c0 = 0; c0 < KP; c0 += 32) {
                float u[32], wv[32];
                tc::tmem_ld32(tmem + lane_base + 256 + c0, u);
                tc::tmem_ld32(tmem + lane_base + 384 + c0, wv);
                if (live) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int col = c0 + 8 * q;
                        if (col >= KP) continue;   // padded d_k = 48: columns past the accumulator hold nothing
                        uint4 kx = make_uint4(0, 0, 0, 0);
                        if (col < K) kx = *reinterpret_cast<const uint4*>(gk + row * K + col);
                        const unsigned* pk = reinterpret_cast<const unsigned*>(&kx);
                        float o[8];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 kf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[i]));
                            const float u0 = u[8 * q + 2 * i], u1 = u[8 * q + 2 * i + 1];
                            const float w0 = wv[8 * q + 2 * i], w1 = wv[8 * q + 2 * i + 1];
                            w_t += u0 * kf.x + w0 * kf.x * kf.x + u1 * kf.y + w1 * kf.y * kf.y;
                            o[2 * i] = a_t * (u0 + 2.f * kf.x * w0);
                            o[2 * i + 1] = a_t * (u1 + 2.f * kf.y * w1);
                        }
                        float4* dst = reinterpret_cast<float4*>(a.dk_x + row * KP + col);
                        dst[0] = make_float4(o[0], o[1], o[2], o[3]);
                        dst[1] = make_float4(o[4], o[5], o[6], o[7]);
                    }
                }
            }
        }
        // ---- c_t = value of the recursion c_{t+1} = f_t c_t + w_t BEFORE token t: scan of affine maps ----
        float F = live ? f_t : 1.f, Wc = live ? w_t : 0.f;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float Fo = __shfl_up_sync(0xffffffffu, F, off), Wo = __shfl_up_sync(0xffffffffu, Wc, off);
            if (lane >= off) {
                Wc = fmaf(F, Wo, Wc);
                F = F * Fo;
            }
        }
        if (lane == 31) wtot_s[w] = make_float2(F, Wc);
        const float Fp = __shfl_up_sync(0xffffffffu, F, 1), Wp = __shfl_up_sync(0xffffffffu, Wc, 1);
        __syncthreads();
        float c_ws = c_run;                               // value at the first token of this warp
        for (int x = 0; x < w; ++x) c_ws = fmaf(wtot_s[x].x, c_ws, wtot_s[x].y);
        const float c_t = lane == 0 ? c_ws : fmaf(Fp, c_ws, Wp);
        if (tid == 127) cnext_s = fmaf(F, c_ws, Wc);
        if (live) {
            a.df_x[row] = status == 0 ? a_t * c_t : __int_as_float(0x7fc00000);  // a wait ran out: mark dgt / dg invalid
            float dip = (1.f - f_t) * a_t * SRI;
            if (t0 + tid == 0 && !has_init) dip += f_t * a_t * SRI;
            a.dip_x[row] = dip;
        }
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();
        c_run = cnext_s;
    }
    tc::fence_before_sync();
    __syncthreads();
    if (status != 0 && tid == 0) atomicCAS(&g_carry_status, 0, status);
    if (w == 0) tc::tmem_free(tmem, 512);
}

bool carry_tc_supported(const palimpsa_problem& p) {
    const int KP = palimpsa_padded_k(p.K);
    auto al = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    return p.io_dtype == PALIMPSA_BF16 && !(p.flags & PALIMPSA_FLAG_UNCERTAINTY) && p.V <= 128 && p.V % 8 == 0 &&
           p.K % 8 == 0 && KP >= 32 && KP <= 128 && KP % 16 == 0 && al(p.k) && al(p.v) && al(p.b);
}

int launch_carry_tc(const palimpsa_bwd_params* prm, const palimpsa_segments& sg, cudaStream_t stream) {
    const palimpsa_problem& p = prm->p;
    const BwdWorkspace ws = bwd_workspace_layout(p);
    if (!ws.tiles) return PALIMPSA_E_DIM;
    if ((sg.seg_len + CT - 1) / CT > C_MAXTILES) return PALIMPSA_E_LIMIT;
    char* base = reinterpret_cast<char*>(prm->workspace);
    const size_t rows = (size_t)p.total_tokens * p.H;
    CarryArgs a;
    a.p = p;
    a.seg_len = sg.seg_len;
    a.carry_M = sg.carry_M;
    a.carry_I = sg.carry_I;
    a.ckpt_M = prm->ckpt_M;
    a.ckpt_I = prm->ckpt_I;
    a.dv = prm->dv;
    a.db = prm->db;
    a.KP = ws.KP;
    a.VP = (p.V + 31) / 32 * 32;
    a.dk_x = reinterpret_cast<float*>(base + ws.dk_part) + (size_t)ws.tiles * rows * ws.KP;
    a.df_x = reinterpret_cast<float*>(base + ws.df_part) + (size_t)ws.tiles * rows;
    a.dip_x = reinterpret_cast<float*>(base + ws.dip_part) + (size_t)ws.tiles * rows;
    const int smem = C_A0 + C_A1 + 4 * C_OPER + 1024;   // + slack to round the base up to 1024 bytes
    dim3 grid(p.num_seqs * p.H, sg.num_segments, 1);
    // The k, v, b rows go in by TMA when a row of a head is whole 128-byte boxes (d_k, d_v multiples of 64) and the
    // driver accepts the tensor maps (base 16-byte aligned, row pitch a multiple of 16 bytes: both hold here).
    CarryMaps maps{};
    const bool tma = p.K % 64 == 0 && p.V % 64 == 0 && p.total_tokens > 0 &&
                     make_tensor_map_bf16_rows(&maps.k, p.k, (unsigned long long)p.total_tokens, (unsigned long long)p.H * p.K, CT) &&
                     make_tensor_map_bf16_rows(&maps.v, p.v, (unsigned long long)p.total_tokens, (unsigned long long)p.H * p.V, CT) &&
                     make_tensor_map_bf16_rows(&maps.b, p.b, (unsigned long long)p.total_tokens, (unsigned long long)p.H * p.V, CT);
    if (tma) {
        if (cudaFuncSetAttribute(carry_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return PALIMPSA_E_LAUNCH;
        carry_tc_kernel<true><<<grid, 128, smem, stream>>>(a, maps);
    } else {
        if (cudaFuncSetAttribute(carry_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return PALIMPSA_E_LAUNCH;
        carry_tc_kernel<false><<<grid, 128, smem, stream>>>(a, maps);
    }
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int carry_tc_status() {
    int s = 0;
    if (cudaMemcpyFromSymbol(&s, g_carry_status, sizeof(int)) != cudaSuccess) return -1;
    if (s) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_carry_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return s;
}

}  // namespace palimpsa
