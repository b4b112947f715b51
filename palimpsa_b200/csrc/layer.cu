// Element-wise work of the layer around the Palimpsa operator (sm_100a): one pass over HBM per side.
//
// Prologue: what palimpsa/layers/palimpsa.py:266-281 does in about ten PyTorch passes (repeat of q/k over
// value heads, softplus(dt + bias), L2-normalise q and k, bs = sigmoid, v = x*bs, b = sigmoid*softplus*bs).
// Epilogue: D-residual and (gated) RMS norm of :337-343.
// One warp owns one (token, head) row; lanes cover the row in 4-element chunks (8- or 16-byte accesses),
// row reductions are xor-shuffles.  These kernels are HBM-bound: every input element is read once
// (second passes over a row hit L1) and every output element written once.  Parameter gradients are
// per-row partials in a workspace, summed by small ordered-reduction kernels (reproducible, no atomics).
#include "common.cuh"
#include "host.h"

namespace palimpsa {

namespace {

constexpr float NORM_EPS = 1e-12f;  // F.normalize's default eps

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    return x;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
// torch's softplus (beta = 1, threshold = 20)
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float softplus_grad(float x) { return x > 20.f ? 1.f : sigmoidf_(x); }
template <int DT>
__device__ __forceinline__ float round_io(float x) {
    if (DT == PALIMPSA_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    if (DT == PALIMPSA_F16) return __half2float(__float2half_rn(x));
    return x;
}

// A row of n elements starting at element `off` of `base`; chunk c covers elements 4c .. 4c+3.
// `vec`: n % 4 == 0 and the buffer is aligned for 4-element accesses.
template <int DT>
struct RowIn {
    const void* base;
    long long off;
    int n;
    bool vec;
    __device__ __forceinline__ float4 ld(int c) const {
        if (vec) return ld4<DT>(reinterpret_cast<const char*>(base) + off * (DT == PALIMPSA_F32 ? 4 : 2), c);
        return ld4_guarded<DT>(base, off + 4 * c, off + n);
    }
};
template <int DT>
struct RowOut {
    void* base;
    long long off;
    int n;
    bool vec;
    __device__ __forceinline__ void st(int c, float4 v) const {
        if (vec) {
            char* rowp = reinterpret_cast<char*>(base) + off * (DT == PALIMPSA_F32 ? 4 : 2);
            if (DT == PALIMPSA_F32) {
                reinterpret_cast<float4*>(rowp)[c] = v;
            } else if (DT == PALIMPSA_BF16) {
                __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&a);
                u.y = *reinterpret_cast<unsigned*>(&b);
                reinterpret_cast<uint2*>(rowp)[c] = u;
            } else {
                __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
                uint2 u;
                u.x = *reinterpret_cast<unsigned*>(&a);
                u.y = *reinterpret_cast<unsigned*>(&b);
                reinterpret_cast<uint2*>(rowp)[c] = u;
            }
        } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (4 * c + i < n) st1(base, off + 4 * c + i, e[i], DT);
        }
    }
};
__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }

constexpr int MAXKC = 2;  // chunks of 4 per lane over d_k <= 256

// ---- prologue, forward: one warp per (token, head) ---------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) layer_prologue_fwd_kernel(const palimpsa_layer_prologue a, long long rows,
                                                                 bool veck, bool vecv) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int K = a.K, V = a.V, H = a.H, rep = a.H / a.Hq;
    const int kc = (K + 3) / 4, vc = (V + 3) / 4;
    for (long long row = warp0; row < rows; row += nwarps) {
        const long long tok = row / H;
        const int h = (int)(row - tok * H);
        const long long roff = (tok * a.Hq + h / rep) * K;
        const RowIn<DT> qi{a.q_raw, roff, K, veck}, ki{a.k_raw, roff, K, veck};
        const RowOut<DT> qo{a.q, row * K, K, veck}, ko{a.k, row * K, K, veck};
        float4 qv[MAXKC], kv[MAXKC];
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int i = 0; i < MAXKC; ++i) {
            const int c = lane + 32 * i;
            qv[i] = kv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < kc) {
                qv[i] = qi.ld(c);
                kv[i] = ki.ld(c);
                sq += dot4(qv[i], qv[i]);
                sk += dot4(kv[i], kv[i]);
            }
        }
        const float rq = 1.f / fmaxf(sqrtf(warp_sum(sq)), NORM_EPS);
        const float rk = 1.f / fmaxf(sqrtf(warp_sum(sk)), NORM_EPS);
#pragma unroll
        for (int i = 0; i < MAXKC; ++i) {
            const int c = lane + 32 * i;
            if (c < kc) {
                qo.st(c, scale4(qv[i], rq));
                ko.st(c, scale4(kv[i], rk));
            }
        }
        const float bs = round_io<DT>(sigmoidf_(ld1<DT>(a.bs_raw, row)));
        const float spb = softplusf_(a.b_scale[h]) * bs;
        if (lane == 0) a.gt[row] = softplusf_(ld1<DT>(a.dt_raw, row) + a.dt_bias[h]);
        const RowIn<DT> xi{a.x, row * V, V, vecv}, bi{a.b_raw, row * V, V, vecv};
        const RowOut<DT> vo{a.v, row * V, V, vecv}, bo{a.b, row * V, V, vecv};
        for (int c = lane; c < vc; c += 32) {
            const float4 xv = xi.ld(c), br = bi.ld(c);
            vo.st(c, scale4(xv, bs));
            bo.st(c, make_float4(sigmoidf_(br.x) * spb, sigmoidf_(br.y) * spb, sigmoidf_(br.z) * spb,
                                 sigmoidf_(br.w) * spb));
        }
    }
}

// ---- prologue, backward: one warp per (token, q/k head); it loops over the value heads that share it ----
// y = x / n, n = max(|x|, eps):  dx = (G - y <y, G>) / n  (G = sum of the gradients of the repeated heads;
// with the norm clamped, n is a constant and dx = G / eps).
template <int DT>
__global__ void __launch_bounds__(256) layer_prologue_bwd_kernel(const palimpsa_layer_prologue a, long long qrows,
                                                                 bool veck, bool vecv, float* w_dtb, float* w_bsc) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int K = a.K, V = a.V, H = a.H, rep = a.H / a.Hq;
    const int kc = (K + 3) / 4, vc = (V + 3) / 4;
    for (long long qrow = warp0; qrow < qrows; qrow += nwarps) {
        const long long tok = qrow / a.Hq;
        const int hq = (int)(qrow - tok * a.Hq);
        const RowIn<DT> qi{a.q_raw, qrow * K, K, veck}, ki{a.k_raw, qrow * K, K, veck};
        float4 qv[MAXKC], kv[MAXKC], gq[MAXKC], gk[MAXKC];
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int i = 0; i < MAXKC; ++i) {
            const int c = lane + 32 * i;
            qv[i] = kv[i] = gq[i] = gk[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < kc) {
                qv[i] = qi.ld(c);
                kv[i] = ki.ld(c);
                sq += dot4(qv[i], qv[i]);
                sk += dot4(kv[i], kv[i]);
            }
        }
        const float nq = sqrtf(warp_sum(sq)), nk = sqrtf(warp_sum(sk));
        const float rq = 1.f / fmaxf(nq, NORM_EPS), rk = 1.f / fmaxf(nk, NORM_EPS);
        for (int r = 0; r < rep; ++r) {
            const long long row = tok * H + hq * rep + r;
            const RowIn<DT> dqi{a.dq, row * K, K, veck}, dki{a.dk, row * K, K, veck};
#pragma unroll
            for (int i = 0; i < MAXKC; ++i) {
                const int c = lane + 32 * i;
                if (c < kc) {
                    const float4 x = dqi.ld(c), y = dki.ld(c);
                    gq[i] = make_float4(gq[i].x + x.x, gq[i].y + x.y, gq[i].z + x.z, gq[i].w + x.w);
                    gk[i] = make_float4(gk[i].x + y.x, gk[i].y + y.y, gk[i].z + y.z, gk[i].w + y.w);
                }
            }
        }
        float dq_ = 0.f, dk_ = 0.f;
#pragma unroll
        for (int i = 0; i < MAXKC; ++i) {
            dq_ += dot4(qv[i], gq[i]);
            dk_ += dot4(kv[i], gk[i]);
        }
        // <y, G> * (1/n) with y = x/n: coefficient of x in the projection term
        const float cq = nq > NORM_EPS ? warp_sum(dq_) * rq * rq : 0.f;
        const float ck = nk > NORM_EPS ? warp_sum(dk_) * rk * rk : 0.f;
        const RowOut<DT> qo{a.dq_raw, qrow * K, K, veck}, ko{a.dk_raw, qrow * K, K, veck};
#pragma unroll
        for (int i = 0; i < MAXKC; ++i) {
            const int c = lane + 32 * i;
            if (c < kc) {
                qo.st(c, make_float4((gq[i].x - qv[i].x * cq) * rq, (gq[i].y - qv[i].y * cq) * rq,
                                     (gq[i].z - qv[i].z * cq) * rq, (gq[i].w - qv[i].w * cq) * rq));
                ko.st(c, make_float4((gk[i].x - kv[i].x * ck) * rk, (gk[i].y - kv[i].y * ck) * rk,
                                     (gk[i].z - kv[i].z * ck) * rk, (gk[i].w - kv[i].w * ck) * rk));
            }
        }
        // value-head rows of this (token, q/k head)
        for (int r = 0; r < rep; ++r) {
            const int h = hq * rep + r;
            const long long row = tok * H + h;
            const float bsf = sigmoidf_(ld1<DT>(a.bs_raw, row));
            const float bs = round_io<DT>(bsf);
            const float bsc = a.b_scale[h];
            const float sp = softplusf_(bsc);
            const RowIn<DT> xi{a.x, row * V, V, vecv}, bi{a.b_raw, row * V, V, vecv};
            const RowIn<DT> dvi{a.dv, row * V, V, vecv}, dbi{a.db, row * V, V, vecv};
            const RowOut<DT> dxo{a.dx, row * V, V, vecv}, dbo{a.db_raw, row * V, V, vecv};
            float acc_bs = 0.f, acc_sc = 0.f;
            for (int c = lane; c < vc; c += 32) {
                const float4 xv = xi.ld(c), br = bi.ld(c), dv = dvi.ld(c), db = dbi.ld(c);
                const float4 sg = make_float4(sigmoidf_(br.x), sigmoidf_(br.y), sigmoidf_(br.z), sigmoidf_(br.w));
                dxo.st(c, scale4(dv, bs));
                const float w = sp * bs;
                dbo.st(c, make_float4(db.x * w * sg.x * (1.f - sg.x), db.y * w * sg.y * (1.f - sg.y),
                                      db.z * w * sg.z * (1.f - sg.z), db.w * w * sg.w * (1.f - sg.w)));
                acc_bs += dot4(dv, xv) + sp * dot4(db, sg);
                acc_sc += dot4(db, sg);
            }
            acc_bs = warp_sum(acc_bs);
            acc_sc = warp_sum(acc_sc);
            if (lane == 0) {
                st1(a.dbs_raw, row, acc_bs * bsf * (1.f - bsf), DT);
                w_bsc[row] = acc_sc * bs * softplus_grad(bsc);
                const float ddt = a.dgt[row] * softplus_grad(ld1<DT>(a.dt_raw, row) + a.dt_bias[h]);
                st1(a.ddt_raw, row, ddt, DT);
                w_dtb[row] = ddt;
            }
        }
    }
}

// out[h] = sum over tokens of w[token*H + h], in a fixed order (one CTA per head).
__global__ void __launch_bounds__(256) layer_sum_heads_kernel(const float* __restrict__ w, float* __restrict__ out,
                                                              long long tokens, int H) {
    __shared__ float red[256];
    const int h = blockIdx.x;
    float s = 0.f;
    for (long long t = threadIdx.x; t < tokens; t += 256) s += w[t * H + h];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int off = 128; off >= 1; off >>= 1) {
        if ((int)threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[h] = red[0];
}

// ---- epilogue, forward: one warp per (token, head) ------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256) layer_epilogue_fwd_kernel(const palimpsa_layer_epilogue a, long long rows,
                                                                 bool vecv) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int V = a.V, H = a.H, vc = (V + 3) / 4;
    const bool res = a.flags & PALIMPSA_LAYER_RESIDUAL, gated = a.flags & PALIMPSA_LAYER_GATE;
    for (long long row = warp0; row < rows; row += nwarps) {
        const int h = (int)(row % H);
        const float d = res ? a.D[h] : 0.f;
        const RowIn<DT> oi{a.o, row * V, V, vecv}, xi{a.x, row * V, V, vecv}, gi{a.gate, row * V, V, vecv};
        const RowOut<DT> yo{a.y, row * V, V, vecv};
        float ss = 0.f;
        for (int c = lane; c < vc; c += 32) {
            float4 z = oi.ld(c);
            if (res) {
                const float4 xv = xi.ld(c);
                z = make_float4(z.x + xv.x * d, z.y + xv.y * d, z.z + xv.z * d, z.w + xv.w * d);
            }
            ss += dot4(z, z);
        }
        const float rstd = 1.f / sqrtf(warp_sum(ss) / (float)V + a.eps);
        for (int c = lane; c < vc; c += 32) {  // second pass: the row is in L1
            float4 z = oi.ld(c);
            if (res) {
                const float4 xv = xi.ld(c);
                z = make_float4(z.x + xv.x * d, z.y + xv.y * d, z.z + xv.z * d, z.w + xv.w * d);
            }
            const float4 w = ld4_guarded<PALIMPSA_F32>(a.weight, 4 * c, V);
            float4 y = make_float4(z.x * rstd * w.x, z.y * rstd * w.y, z.z * rstd * w.z, z.w * rstd * w.w);
            if (gated) {
                const float4 g = gi.ld(c);
                y = make_float4(y.x * g.x * sigmoidf_(g.x), y.y * g.y * sigmoidf_(g.y), y.z * g.z * sigmoidf_(g.z),
                                y.w * g.w * sigmoidf_(g.w));
            }
            yo.st(c, y);
        }
    }
}

// ---- epilogue, backward: persistent CTAs, one warp per row; NC = chunks of 4 per lane (V <= 128*NC) -------
//   xh = z r,  yn = xh w,  y = yn g s(g):   dg = dy yn (s + g s (1-s)),  dyn = dy g s(g)  (or dy without gate)
//   dw += dyn xh,  dxh = dyn w,  dz = r (dxh - xh mean(dxh xh)),  d_o = dz,  dx = dz D,  dD += <dz, x>
template <int DT, int NC>
__global__ void __launch_bounds__(256) layer_epilogue_bwd_kernel(const palimpsa_layer_epilogue a, long long rows,
                                                                 bool vecv, float* w_dD, float* w_dw) {
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const long long warp0 = (long long)blockIdx.x * 8 + wid;
    const long long nwarps = (long long)gridDim.x * 8;
    const int V = a.V, H = a.H, vc = (V + 3) / 4;
    const bool res = a.flags & PALIMPSA_LAYER_RESIDUAL, gated = a.flags & PALIMPSA_LAYER_GATE;
    float4 dw[NC], wv[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) {
        dw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        wv[i] = ld4_guarded<PALIMPSA_F32>(a.weight, 4 * (lane + 32 * i), V);
    }
    for (long long row = warp0; row < rows; row += nwarps) {
        const int h = (int)(row % H);
        const float d = res ? a.D[h] : 0.f;
        const RowIn<DT> oi{a.o, row * V, V, vecv}, xi{a.x, row * V, V, vecv}, gi{a.gate, row * V, V, vecv};
        const RowIn<DT> dyi{a.dy, row * V, V, vecv};
        float4 z[NC], xv[NC];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            const int c = lane + 32 * i;
            z[i] = xv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < vc) {
                z[i] = oi.ld(c);
                if (res) {
                    xv[i] = xi.ld(c);
                    z[i] = make_float4(z[i].x + xv[i].x * d, z[i].y + xv[i].y * d, z[i].z + xv[i].z * d,
                                       z[i].w + xv[i].w * d);
                }
                ss += dot4(z[i], z[i]);
            }
        }
        const float rstd = 1.f / sqrtf(warp_sum(ss) / (float)V + a.eps);
        float4 dxh[NC];
        float c1 = 0.f;
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            const int c = lane + 32 * i;
            dxh[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < vc) {
                const float4 xh = scale4(z[i], rstd);
                float4 dyn = dyi.ld(c);
                if (gated) {
                    const float4 g = gi.ld(c);
                    const float4 s = make_float4(sigmoidf_(g.x), sigmoidf_(g.y), sigmoidf_(g.z), sigmoidf_(g.w));
                    const RowOut<DT> dgo{a.dgate, row * V, V, vecv};
                    dgo.st(c, make_float4(dyn.x * xh.x * wv[i].x * (s.x + g.x * s.x * (1.f - s.x)),
                                          dyn.y * xh.y * wv[i].y * (s.y + g.y * s.y * (1.f - s.y)),
                                          dyn.z * xh.z * wv[i].z * (s.z + g.z * s.z * (1.f - s.z)),
                                          dyn.w * xh.w * wv[i].w * (s.w + g.w * s.w * (1.f - s.w))));
                    dyn = make_float4(dyn.x * g.x * s.x, dyn.y * g.y * s.y, dyn.z * g.z * s.z, dyn.w * g.w * s.w);
                }
                dw[i] = make_float4(dw[i].x + dyn.x * xh.x, dw[i].y + dyn.y * xh.y, dw[i].z + dyn.z * xh.z,
                                    dw[i].w + dyn.w * xh.w);
                dxh[i] = make_float4(dyn.x * wv[i].x, dyn.y * wv[i].y, dyn.z * wv[i].z, dyn.w * wv[i].w);
                c1 += dot4(dxh[i], xh);
                z[i] = xh;  // keep the normalised row for the last pass
            }
        }
        c1 = warp_sum(c1) / (float)V;
        float dd = 0.f;
        const RowOut<DT> doo{a.d_o, row * V, V, vecv}, dxo{a.dx, row * V, V, vecv};
#pragma unroll
        for (int i = 0; i < NC; ++i) {
            const int c = lane + 32 * i;
            if (c < vc) {
                const float4 dz = make_float4(rstd * (dxh[i].x - z[i].x * c1), rstd * (dxh[i].y - z[i].y * c1),
                                              rstd * (dxh[i].z - z[i].z * c1), rstd * (dxh[i].w - z[i].w * c1));
                doo.st(c, dz);
                if (res) {
                    dxo.st(c, scale4(dz, d));
                    dd += dot4(dz, xv[i]);
                }
            }
        }
        if (res) {
            dd = warp_sum(dd);
            if (lane == 0) w_dD[row] = dd;
        }
    }
    // this CTA's share of dweight: sum its 8 warps, one partial row per CTA
#pragma unroll
    for (int i = 0; i < NC; ++i) {
        __syncthreads();
        red[wid][lane] = dw[i];
        __syncthreads();
        if (wid == 0) {
            float4 s = red[0][lane];
            for (int x = 1; x < 8; ++x) {
                const float4 t = red[x][lane];
                s = make_float4(s.x + t.x, s.y + t.y, s.z + t.z, s.w + t.w);
            }
            const int c = lane + 32 * i;
            const float e[4] = {s.x, s.y, s.z, s.w};
            for (int j = 0; j < 4; ++j)
                if (4 * c + j < V) w_dw[(long long)blockIdx.x * V + 4 * c + j] = e[j];
        }
    }
}

// out[v] = sum over partial rows of w[r*V + v], in row order (one thread per column).
__global__ void layer_sum_cols_kernel(const float* __restrict__ w, float* __restrict__ out, int nrows, int V) {
    const int v = blockIdx.x * blockDim.x + threadIdx.x;
    if (v >= V) return;
    float s = 0.f;
    for (int r = 0; r < nrows; ++r) s += w[(long long)r * V + v];
    out[v] = s;
}

}  // namespace

// -------------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------------
namespace {

constexpr int LAYER_MAX_V = 1024;
constexpr int DW_CTAS = 148 * 4;  // partial rows of dweight (persistent CTAs of the epilogue backward)

bool aligned_for(const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dt == PALIMPSA_F32 ? 15 : 7)) == 0; }
unsigned row_blocks(long long rows, int cap) {
    long long b = (rows + 7) / 8;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}
size_t ws_bytes(long long tokens, int H, int V) {
    const size_t rows = (size_t)tokens * H;
    const size_t a = 2 * rows, b = rows + (size_t)DW_CTAS * V;
    return ((a > b ? a : b) * 4 + 255) / 256 * 256;
}
int check_dims(int io_dtype, int H, int V, long long tokens) {
    if (io_dtype != PALIMPSA_F32 && io_dtype != PALIMPSA_BF16 && io_dtype != PALIMPSA_F16) return PALIMPSA_E_DTYPE;
    if (H <= 0 || V <= 0 || tokens < 0) return PALIMPSA_E_SHAPE;
    if (V > LAYER_MAX_V) return PALIMPSA_E_DIM;
    return PALIMPSA_OK;
}
int check_pro(const palimpsa_layer_prologue* a, bool bwd) {
    if (!a) return PALIMPSA_E_NULL;
    if (a->struct_size != sizeof(palimpsa_layer_prologue)) return PALIMPSA_E_VERSION;
    if (int rc = check_dims(a->io_dtype, a->H, a->V, a->tokens)) return rc;
    if (a->K <= 0 || a->Hq <= 0 || a->H % a->Hq) return PALIMPSA_E_SHAPE;
    if (a->K > PALIMPSA_MAX_K) return PALIMPSA_E_DIM;
    if (!a->q_raw || !a->k_raw || !a->x || !a->b_raw || !a->dt_raw || !a->bs_raw || !a->dt_bias || !a->b_scale)
        return PALIMPSA_E_NULL;
    if (!bwd) return (a->q && a->k && a->v && a->b && a->gt) ? PALIMPSA_OK : PALIMPSA_E_NULL;
    if (!a->dq || !a->dk || !a->dv || !a->db || !a->dgt || !a->dq_raw || !a->dk_raw || !a->dx || !a->db_raw ||
        !a->ddt_raw || !a->dbs_raw || !a->d_dt_bias || !a->d_b_scale)
        return PALIMPSA_E_NULL;
    if (!a->workspace || a->workspace_bytes < ws_bytes(a->tokens, a->H, a->V) ||
        (reinterpret_cast<uintptr_t>(a->workspace) & 255))
        return PALIMPSA_E_WORKSPACE;
    return PALIMPSA_OK;
}
int check_epi(const palimpsa_layer_epilogue* a, bool bwd) {
    if (!a) return PALIMPSA_E_NULL;
    if (a->struct_size != sizeof(palimpsa_layer_epilogue)) return PALIMPSA_E_VERSION;
    if (int rc = check_dims(a->io_dtype, a->H, a->V, a->tokens)) return rc;
    const bool res = a->flags & PALIMPSA_LAYER_RESIDUAL, gated = a->flags & PALIMPSA_LAYER_GATE;
    if (!a->o || !a->weight || (res && (!a->x || !a->D)) || (gated && !a->gate)) return PALIMPSA_E_NULL;
    if (!bwd) return a->y ? PALIMPSA_OK : PALIMPSA_E_NULL;
    if (!a->dy || !a->d_o || !a->dweight || (res && (!a->dx || !a->dD)) || (gated && !a->dgate)) return PALIMPSA_E_NULL;
    if (!a->workspace || a->workspace_bytes < ws_bytes(a->tokens, a->H, a->V) ||
        (reinterpret_cast<uintptr_t>(a->workspace) & 255))
        return PALIMPSA_E_WORKSPACE;
    return PALIMPSA_OK;
}
int launched() { return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH; }

#define PALIMPSA_BY_DTYPE(dt, CALL)                                   \
    do {                                                              \
        if ((dt) == PALIMPSA_BF16) { CALL(PALIMPSA_BF16); }           \
        else if ((dt) == PALIMPSA_F16) { CALL(PALIMPSA_F16); }        \
        else { CALL(PALIMPSA_F32); }                                  \
    } while (0)

}  // namespace
}  // namespace palimpsa

using namespace palimpsa;

extern "C" {

size_t palimpsa_layer_workspace_bytes(int64_t tokens, int32_t H, int32_t V) {
    if (tokens < 0 || H <= 0 || V <= 0) return 0;
    return ws_bytes(tokens, H, V);
}

int palimpsa_layer_prologue_fwd(const palimpsa_layer_prologue* a, void* cuda_stream) {
    if (int rc = check_pro(a, false)) return rc;
    const long long rows = a->tokens * a->H;
    if (rows == 0) return PALIMPSA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int dt = a->io_dtype;
    const bool veck = a->K % 4 == 0 && aligned_for(a->q_raw, dt) && aligned_for(a->k_raw, dt) && aligned_for(a->q, dt) &&
                      aligned_for(a->k, dt);
    const bool vecv = a->V % 4 == 0 && aligned_for(a->x, dt) && aligned_for(a->b_raw, dt) && aligned_for(a->v, dt) &&
                      aligned_for(a->b, dt);
#define CALL(D) layer_prologue_fwd_kernel<D><<<row_blocks(rows, 148 * 8), 256, 0, st>>>(*a, rows, veck, vecv)
    PALIMPSA_BY_DTYPE(dt, CALL);
#undef CALL
    return launched();
}

int palimpsa_layer_prologue_bwd(const palimpsa_layer_prologue* a, void* cuda_stream) {
    if (int rc = check_pro(a, true)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const long long rows = a->tokens * a->H, qrows = a->tokens * a->Hq;
    float* w_dtb = reinterpret_cast<float*>(a->workspace);
    float* w_bsc = w_dtb + rows;
    if (rows > 0) {
        const int dt = a->io_dtype;
        const bool veck = a->K % 4 == 0 && aligned_for(a->q_raw, dt) && aligned_for(a->k_raw, dt) &&
                          aligned_for(a->dq, dt) && aligned_for(a->dk, dt) && aligned_for(a->dq_raw, dt) &&
                          aligned_for(a->dk_raw, dt);
        const bool vecv = a->V % 4 == 0 && aligned_for(a->x, dt) && aligned_for(a->b_raw, dt) && aligned_for(a->dv, dt) &&
                          aligned_for(a->db, dt) && aligned_for(a->dx, dt) && aligned_for(a->db_raw, dt);
#define CALL(D) \
    layer_prologue_bwd_kernel<D><<<row_blocks(qrows, 148 * 8), 256, 0, st>>>(*a, qrows, veck, vecv, w_dtb, w_bsc)
        PALIMPSA_BY_DTYPE(dt, CALL);
#undef CALL
        if (int rc = launched()) return rc;
    }
    layer_sum_heads_kernel<<<a->H, 256, 0, st>>>(w_dtb, a->d_dt_bias, a->tokens, a->H);
    layer_sum_heads_kernel<<<a->H, 256, 0, st>>>(w_bsc, a->d_b_scale, a->tokens, a->H);
    return launched();
}

int palimpsa_layer_epilogue_fwd(const palimpsa_layer_epilogue* a, void* cuda_stream) {
    if (int rc = check_epi(a, false)) return rc;
    const long long rows = a->tokens * a->H;
    if (rows == 0) return PALIMPSA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int dt = a->io_dtype;
    const bool vecv = a->V % 4 == 0 && aligned_for(a->o, dt) && aligned_for(a->y, dt) &&
                      (!(a->flags & PALIMPSA_LAYER_RESIDUAL) || aligned_for(a->x, dt)) &&
                      (!(a->flags & PALIMPSA_LAYER_GATE) || aligned_for(a->gate, dt));
#define CALL(D) layer_epilogue_fwd_kernel<D><<<row_blocks(rows, 148 * 8), 256, 0, st>>>(*a, rows, vecv)
    PALIMPSA_BY_DTYPE(dt, CALL);
#undef CALL
    return launched();
}

int palimpsa_layer_epilogue_bwd(const palimpsa_layer_epilogue* a, void* cuda_stream) {
    if (int rc = check_epi(a, true)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const long long rows = a->tokens * a->H;
    const bool res = a->flags & PALIMPSA_LAYER_RESIDUAL, gated = a->flags & PALIMPSA_LAYER_GATE;
    float* w_dD = reinterpret_cast<float*>(a->workspace);
    float* w_dw = w_dD + rows;
    const unsigned nb = row_blocks(rows, DW_CTAS);
    if (rows > 0) {
        const int dt = a->io_dtype;
        const bool vecv = a->V % 4 == 0 && aligned_for(a->o, dt) && aligned_for(a->dy, dt) && aligned_for(a->d_o, dt) &&
                          (!res || (aligned_for(a->x, dt) && aligned_for(a->dx, dt))) &&
                          (!gated || (aligned_for(a->gate, dt) && aligned_for(a->dgate, dt)));
        const int nc = (a->V + 127) / 128;
#define CALL(D)                                                                                          \
    do {                                                                                                 \
        if (nc <= 1) layer_epilogue_bwd_kernel<D, 1><<<nb, 256, 0, st>>>(*a, rows, vecv, w_dD, w_dw);     \
        else if (nc <= 2) layer_epilogue_bwd_kernel<D, 2><<<nb, 256, 0, st>>>(*a, rows, vecv, w_dD, w_dw); \
        else if (nc <= 4) layer_epilogue_bwd_kernel<D, 4><<<nb, 256, 0, st>>>(*a, rows, vecv, w_dD, w_dw); \
        else layer_epilogue_bwd_kernel<D, 8><<<nb, 256, 0, st>>>(*a, rows, vecv, w_dD, w_dw);             \
    } while (0)
        PALIMPSA_BY_DTYPE(dt, CALL);
#undef CALL
        if (int rc = launched()) return rc;
    }
    if (res) layer_sum_heads_kernel<<<a->H, 256, 0, st>>>(w_dD, a->dD, a->tokens, a->H);
    layer_sum_cols_kernel<<<(a->V + 127) / 128, 128, 0, st>>>(w_dw, a->dweight, rows > 0 ? (int)nb : 0, a->V);
    return launched();
}

}  // extern "C"
