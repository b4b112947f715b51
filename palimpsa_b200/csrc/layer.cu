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

// F.normalize clamps the norm at eps = 1e-12; in squares: 1/max(sqrt(s), eps) = rsqrt(max(s, eps^2))
constexpr float NORM_EPS2 = 1e-24f;

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
    return x;
}
// exp and reciprocal as single MUFU ops (relative error about 2^-21 together): the kernels evaluate one
// sigmoid per element and would otherwise be bound by instruction issue, not by HBM
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_approx(1.f + __expf(-x)); }
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
// VEC: n % 4 == 0 and the buffer is aligned for 4-element accesses (8 or 16 bytes per lane).
template <int DT, bool VEC>
struct RowIn {
    const char* rowp;
    const void* base;
    long long off;
    int n;
    __device__ __forceinline__ RowIn(const void* b, long long o, int n_)
        : rowp(reinterpret_cast<const char*>(b) + o * (DT == PALIMPSA_F32 ? 4 : 2)), base(b), off(o), n(n_) {}
    __device__ __forceinline__ float4 ld(int c) const {
        if (VEC) return ld4<DT>(rowp, c);
        return ld4_guarded<DT>(base, off + 4 * c, off + n);
    }
};
template <int DT, bool VEC>
struct RowOut {
    char* rowp;
    void* base;
    long long off;
    int n;
    __device__ __forceinline__ RowOut(void* b, long long o, int n_)
        : rowp(reinterpret_cast<char*>(b) + o * (DT == PALIMPSA_F32 ? 4 : 2)), base(b), off(o), n(n_) {}
    __device__ __forceinline__ void st(int c, float4 v) const {
        if (VEC) {
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

__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 mul4(float4 a, float4 b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
__device__ __forceinline__ float4 fma4(float4 a, float s, float4 c) {
    return make_float4(a.x * s + c.x, a.y * s + c.y, a.z * s + c.z, a.w * s + c.w);
}
__device__ __forceinline__ float4 sigmoid4(float4 a) {
    return make_float4(sigmoidf_(a.x), sigmoidf_(a.y), sigmoidf_(a.z), sigmoidf_(a.w));
}

// Resident CTAs to compile for: the narrow shapes (one chunk per lane) want many warps in flight, the wide ones
// need their registers for the row itself.
constexpr int min_ctas(int chunks, int narrow) { return chunks == 1 ? narrow : (chunks == 2 ? 2 : 1); }

// Every kernel below gives one warp R (token, head) rows per iteration and issues ALL global loads of those
// rows before the first use.  NCK / NCV = 4-element chunks per lane over d_k / d_v (compile-time, so the rows
// live in registers); R = 2 only for the narrowest shapes.  Per-row scalars that need the accurate
// exp/log (softplus) are not computed by whole warps: the per-head ones go through a table in shared memory,
// the per-row ones through a thread-per-row loop at the start of the kernel.

// ---- prologue, forward ---------------------------------------------------------------------------------
template <int DT, int NCK, int NCV, int R, bool VECK, bool VECV>
__global__ void __launch_bounds__(256, min_ctas(NCK * NCV, 4)) layer_prologue_fwd_kernel(const palimpsa_layer_prologue a, int rows) {
    extern __shared__ float head_tab[];  // [H] softplus(b_scale)
    const int lane = threadIdx.x & 31;
    const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    const int K = a.K, V = a.V, H = a.H, rep = a.H / a.Hq;
    const int kc = (K + 3) / 4, vc = (V + 3) / 4;
    for (int h = threadIdx.x; h < H; h += blockDim.x) head_tab[h] = softplusf_(a.b_scale[h]);
    // gt = softplus(dt_raw + dt_bias): one thread per row
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x)
        a.gt[i] = softplusf_(ld1<DT>(a.dt_raw, i) + a.dt_bias[i % H]);
    __syncthreads();
    for (long long base = (long long)warp0 * R; base < rows; base += (long long)nwarps * R) {
        float4 qv[R][NCK], kv[R][NCK], xv[R][NCV], br[R][NCV];
        float bsr[R];
        int hh[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            const int tok = row / H;
            hh[r] = row - tok * H;
            const long long roff = ((long long)tok * a.Hq + (rep == 1 ? hh[r] : hh[r] / rep)) * K;
            const RowIn<DT, VECK> qi(a.q_raw, roff, K), ki(a.k_raw, roff, K);
            const RowIn<DT, VECV> xi(a.x, (long long)row * V, V), bi(a.b_raw, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NCK; ++i) {
                const int c = lane + 32 * i;
                const bool on = ok && c < kc;
                qv[r][i] = on ? qi.ld(c) : zero4();
                kv[r][i] = on ? ki.ld(c) : zero4();
            }
#pragma unroll
            for (int i = 0; i < NCV; ++i) {
                const int c = lane + 32 * i;
                const bool on = ok && c < vc;
                xv[r][i] = on ? xi.ld(c) : zero4();
                br[r][i] = on ? bi.ld(c) : zero4();
            }
            bsr[r] = ok ? ld1<DT>(a.bs_raw, row) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int i = 0; i < NCK; ++i) {
                sq += dot4(qv[r][i], qv[r][i]);
                sk += dot4(kv[r][i], kv[r][i]);
            }
            const float rq = rsqrtf(fmaxf(warp_sum(sq), NORM_EPS2));
            const float rk = rsqrtf(fmaxf(warp_sum(sk), NORM_EPS2));
            const RowOut<DT, VECK> qo(a.q, (long long)row * K, K), ko(a.k, (long long)row * K, K);
#pragma unroll
            for (int i = 0; i < NCK; ++i) {
                const int c = lane + 32 * i;
                if (ok && c < kc) {
                    qo.st(c, scale4(qv[r][i], rq));
                    ko.st(c, scale4(kv[r][i], rk));
                }
            }
            const float bs = round_io<DT>(sigmoidf_(bsr[r]));
            const float spb = head_tab[ok ? hh[r] : 0] * bs;
            const RowOut<DT, VECV> vo(a.v, (long long)row * V, V), bo(a.b, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NCV; ++i) {
                const int c = lane + 32 * i;
                if (ok && c < vc) {
                    vo.st(c, scale4(xv[r][i], bs));
                    bo.st(c, scale4(sigmoid4(br[r][i]), spb));
                }
            }
        }
    }
}

// ---- prologue, backward: one warp per (token, q/k head); it loops over the value heads that share it ----
// y = x / n, n = max(|x|, eps):  dx = (G - y <y, G>) / n  (G = sum of the gradients of the repeated heads;
// with the norm clamped, n is a constant and dx = G / eps).
template <int DT, int NCK, int NCV, bool VECK, bool VECV>
__global__ void __launch_bounds__(256, min_ctas(NCK * NCV, 4)) layer_prologue_bwd_kernel(const palimpsa_layer_prologue a, int qrows,
                                                                    float* w_dtb, float* w_bsc) {
    extern __shared__ float head_tab[];  // [2][H]: softplus(b_scale), its derivative
    const int lane = threadIdx.x & 31;
    const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    const int K = a.K, V = a.V, H = a.H, rep = a.H / a.Hq;
    const int kc = (K + 3) / 4, vc = (V + 3) / 4;
    const int rows = qrows * rep;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        head_tab[h] = softplusf_(a.b_scale[h]);
        head_tab[H + h] = softplus_grad(a.b_scale[h]);
    }
    // d dt_raw = dgt * softplus'(dt_raw + dt_bias): one thread per row
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += gridDim.x * blockDim.x) {
        const float x = ld1<DT>(a.dt_raw, i) + a.dt_bias[i % H];
        const float ddt = a.dgt[i] * (x > 20.f ? 1.f : 1.f / (1.f + expf(-x)));
        st1(a.ddt_raw, i, ddt, DT);
        w_dtb[i] = ddt;
    }
    __syncthreads();
    for (int qrow = warp0; qrow < qrows; qrow += nwarps) {
        const int tok = qrow / a.Hq;
        const int hq = qrow - tok * a.Hq;
        const RowIn<DT, VECK> qi(a.q_raw, (long long)qrow * K, K), ki(a.k_raw, (long long)qrow * K, K);
        float4 qv[NCK], kv[NCK], gq[NCK], gk[NCK];
#pragma unroll
        for (int i = 0; i < NCK; ++i) {
            const int c = lane + 32 * i;
            qv[i] = c < kc ? qi.ld(c) : zero4();
            kv[i] = c < kc ? ki.ld(c) : zero4();
            gq[i] = gk[i] = zero4();
        }
        for (int r = 0; r < rep; ++r) {
            const int h = hq * rep + r;
            const long long row = (long long)tok * H + h;
            // every load of this value-head row first
            const RowIn<DT, VECK> dqi(a.dq, row * K, K), dki(a.dk, row * K, K);
            const RowIn<DT, VECV> xi(a.x, row * V, V), bi(a.b_raw, row * V, V);
            const RowIn<DT, VECV> dvi(a.dv, row * V, V), dbi(a.db, row * V, V);
            float4 xv[NCV], br[NCV], dv[NCV], db[NCV];
#pragma unroll
            for (int i = 0; i < NCK; ++i) {
                const int c = lane + 32 * i;
                if (c < kc) {
                    gq[i] = add4(gq[i], dqi.ld(c));
                    gk[i] = add4(gk[i], dki.ld(c));
                }
            }
#pragma unroll
            for (int i = 0; i < NCV; ++i) {
                const int c = lane + 32 * i;
                const bool on = c < vc;
                xv[i] = on ? xi.ld(c) : zero4();
                br[i] = on ? bi.ld(c) : zero4();
                dv[i] = on ? dvi.ld(c) : zero4();
                db[i] = on ? dbi.ld(c) : zero4();
            }
            const float bsf = sigmoidf_(ld1<DT>(a.bs_raw, row));
            const float bs = round_io<DT>(bsf);
            const float sp = head_tab[h];
            const RowOut<DT, VECV> dxo(a.dx, row * V, V), dbo(a.db_raw, row * V, V);
            float acc_bs = 0.f, acc_sc = 0.f;
            const float w = sp * bs;
#pragma unroll
            for (int i = 0; i < NCV; ++i) {
                const int c = lane + 32 * i;
                if (c < vc) {
                    const float4 sg = sigmoid4(br[i]);
                    dxo.st(c, scale4(dv[i], bs));
                    dbo.st(c, make_float4(db[i].x * w * sg.x * (1.f - sg.x), db[i].y * w * sg.y * (1.f - sg.y),
                                          db[i].z * w * sg.z * (1.f - sg.z), db[i].w * w * sg.w * (1.f - sg.w)));
                    const float dsg = dot4(db[i], sg);
                    acc_bs += dot4(dv[i], xv[i]) + sp * dsg;
                    acc_sc += dsg;
                }
            }
            acc_bs = warp_sum(acc_bs);
            acc_sc = warp_sum(acc_sc);
            if (lane == 0) {
                st1(a.dbs_raw, row, acc_bs * bsf * (1.f - bsf), DT);
                w_bsc[row] = acc_sc * bs * head_tab[H + h];
            }
        }
        float sq = 0.f, sk = 0.f, dq_ = 0.f, dk_ = 0.f;
#pragma unroll
        for (int i = 0; i < NCK; ++i) {
            sq += dot4(qv[i], qv[i]);
            sk += dot4(kv[i], kv[i]);
            dq_ += dot4(qv[i], gq[i]);
            dk_ += dot4(kv[i], gk[i]);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float rq = rsqrtf(fmaxf(sq, NORM_EPS2)), rk = rsqrtf(fmaxf(sk, NORM_EPS2));
        // <y, G> / n with y = x / n: the coefficient of x in the projection term (0 while the norm is clamped)
        dq_ = warp_sum(dq_);
        dk_ = warp_sum(dk_);
        const float cq = sq > NORM_EPS2 ? dq_ * rq * rq : 0.f;
        const float ck = sk > NORM_EPS2 ? dk_ * rk * rk : 0.f;
        const RowOut<DT, VECK> qo(a.dq_raw, (long long)qrow * K, K), ko(a.dk_raw, (long long)qrow * K, K);
#pragma unroll
        for (int i = 0; i < NCK; ++i) {
            const int c = lane + 32 * i;
            if (c < kc) {
                qo.st(c, scale4(fma4(qv[i], -cq, gq[i]), rq));
                ko.st(c, scale4(fma4(kv[i], -ck, gk[i]), rk));
            }
        }
    }
}

// out[h] = sum over tokens of w[token*H + h] in a fixed order, for up to two arrays at once (blockIdx.y picks
// the array): one CTA of 1024 threads per head; every thread sums a strided subsequence with 8 loads in
// flight, then a tree over the CTA.
__device__ __forceinline__ void sum_heads_body(const float* __restrict__ w, float* __restrict__ out, long long tokens,
                                               int H, int h, float* red) {
    float s = 0.f;
    long long t = threadIdx.x;
    for (; t + 7 * 1024 < tokens; t += 8 * 1024) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = w[(t + i * 1024) * H + h];
#pragma unroll
        for (int i = 0; i < 8; ++i) s += v[i];
    }
    for (; t < tokens; t += 1024) s += w[t * H + h];
    red[threadIdx.x] = s;
    __syncthreads();
    for (int off = 512; off >= 1; off >>= 1) {
        if ((int)threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[h] = red[0];
}
__global__ void __launch_bounds__(1024) layer_sum_heads_kernel(const float* __restrict__ w0, float* __restrict__ out0,
                                                               const float* __restrict__ w1, float* __restrict__ out1,
                                                               long long tokens, int H) {
    __shared__ float red[1024];
    sum_heads_body(blockIdx.y ? w1 : w0, blockIdx.y ? out1 : out0, tokens, H, blockIdx.x, red);
}

// ---- epilogue, forward -----------------------------------------------------------------------------------
template <int DT, int NC, int R, bool VEC>
__global__ void __launch_bounds__(256, min_ctas(NC, 4)) layer_epilogue_fwd_kernel(const palimpsa_layer_epilogue a, int rows) {
    const int lane = threadIdx.x & 31;
    const int warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * (blockDim.x >> 5);
    const int V = a.V, H = a.H, vc = (V + 3) / 4;
    const bool res = a.flags & PALIMPSA_LAYER_RESIDUAL, gated = a.flags & PALIMPSA_LAYER_GATE;
    float4 wv[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) wv[i] = ld4_guarded<PALIMPSA_F32>(a.weight, 4 * (lane + 32 * i), V);
    for (long long base = (long long)warp0 * R; base < rows; base += (long long)nwarps * R) {
        float4 z[R][NC], xv[R][NC], g[R][NC];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            const RowIn<DT, VEC> oi(a.o, (long long)row * V, V), xi(a.x, (long long)row * V, V);
            const RowIn<DT, VEC> gi(a.gate, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = lane + 32 * i;
                const bool on = ok && c < vc;
                z[r][i] = on ? oi.ld(c) : zero4();
                xv[r][i] = (on && res) ? xi.ld(c) : zero4();
                g[r][i] = (on && gated) ? gi.ld(c) : zero4();
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            const float d = (res && ok) ? a.D[row % H] : 0.f;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                z[r][i] = fma4(xv[r][i], d, z[r][i]);
                ss += dot4(z[r][i], z[r][i]);
            }
            const float rstd = rsqrtf(warp_sum(ss) / (float)V + a.eps);
            const RowOut<DT, VEC> yo(a.y, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = lane + 32 * i;
                if (ok && c < vc) {
                    float4 y = mul4(scale4(z[r][i], rstd), wv[i]);
                    if (gated) y = mul4(y, mul4(g[r][i], sigmoid4(g[r][i])));
                    yo.st(c, y);
                }
            }
        }
    }
}

// ---- epilogue, backward: persistent CTAs (each also accumulates its share of dweight) ------------------------
//   xh = z r,  yn = xh w,  y = yn g s(g):   dg = dy yn (s + g s (1-s)),  dyn = dy g s(g)  (or dy without gate)
//   dw += dyn xh,  dxh = dyn w,  dz = r (dxh - xh mean(dxh xh)),  d_o = dz,  dx = dz D,  dD += <dz, x>
template <int DT, int NC, int R, bool VEC>
__global__ void __launch_bounds__(256, min_ctas(NC, 4)) layer_epilogue_bwd_kernel(const palimpsa_layer_epilogue a, int rows,
                                                                    float* w_dD, float* w_dw) {
    __shared__ float4 red[8][32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int warp0 = blockIdx.x * 8 + wid;
    const int nwarps = gridDim.x * 8;
    const int V = a.V, H = a.H, vc = (V + 3) / 4;
    const bool res = a.flags & PALIMPSA_LAYER_RESIDUAL, gated = a.flags & PALIMPSA_LAYER_GATE;
    float4 dw[NC], wv[NC];
#pragma unroll
    for (int i = 0; i < NC; ++i) {
        dw[i] = zero4();
        wv[i] = ld4_guarded<PALIMPSA_F32>(a.weight, 4 * (lane + 32 * i), V);
    }
    for (long long base = (long long)warp0 * R; base < rows; base += (long long)nwarps * R) {
        float4 z[R][NC], xv[R][NC], g[R][NC], dy[R][NC];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            const RowIn<DT, VEC> oi(a.o, (long long)row * V, V), xi(a.x, (long long)row * V, V);
            const RowIn<DT, VEC> gi(a.gate, (long long)row * V, V), dyi(a.dy, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = lane + 32 * i;
                const bool on = ok && c < vc;
                z[r][i] = on ? oi.ld(c) : zero4();
                dy[r][i] = on ? dyi.ld(c) : zero4();
                xv[r][i] = (on && res) ? xi.ld(c) : zero4();
                g[r][i] = (on && gated) ? gi.ld(c) : zero4();
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int row = (int)base + r;
            const bool ok = row < rows;
            const float d = (res && ok) ? a.D[row % H] : 0.f;
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                z[r][i] = fma4(xv[r][i], d, z[r][i]);
                ss += dot4(z[r][i], z[r][i]);
            }
            const float rstd = rsqrtf(warp_sum(ss) / (float)V + a.eps);
            const RowOut<DT, VEC> dgo(a.dgate, (long long)row * V, V);
            float c1 = 0.f;
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = lane + 32 * i;
                const float4 xh = scale4(z[r][i], rstd);
                float4 dyn = dy[r][i];
                if (gated) {
                    const float4 gg = g[r][i], s = sigmoid4(gg);
                    if (ok && c < vc)
                        dgo.st(c, make_float4(dyn.x * xh.x * wv[i].x * (s.x + gg.x * s.x * (1.f - s.x)),
                                              dyn.y * xh.y * wv[i].y * (s.y + gg.y * s.y * (1.f - s.y)),
                                              dyn.z * xh.z * wv[i].z * (s.z + gg.z * s.z * (1.f - s.z)),
                                              dyn.w * xh.w * wv[i].w * (s.w + gg.w * s.w * (1.f - s.w))));
                    dyn = mul4(dyn, mul4(gg, s));
                }
                dw[i] = add4(dw[i], mul4(dyn, xh));
                dy[r][i] = mul4(dyn, wv[i]);  // dxh
                c1 += dot4(dy[r][i], xh);
                z[r][i] = xh;
            }
            c1 = warp_sum(c1) / (float)V;
            float dd = 0.f;
            const RowOut<DT, VEC> doo(a.d_o, (long long)row * V, V), dxo(a.dx, (long long)row * V, V);
#pragma unroll
            for (int i = 0; i < NC; ++i) {
                const int c = lane + 32 * i;
                if (ok && c < vc) {
                    const float4 dz = scale4(fma4(z[r][i], -c1, dy[r][i]), rstd);
                    doo.st(c, dz);
                    if (res) {
                        dxo.st(c, scale4(dz, d));
                        dd += dot4(dz, xv[r][i]);
                    }
                }
            }
            if (res) {
                dd = warp_sum(dd);
                if (ok && lane == 0) w_dD[row] = dd;
            }
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
            for (int x = 1; x < 8; ++x) s = add4(s, red[x][lane]);
            const int c = lane + 32 * i;
            const float e[4] = {s.x, s.y, s.z, s.w};
            for (int j = 0; j < 4; ++j)
                if (4 * c + j < V) w_dw[(long long)blockIdx.x * V + 4 * c + j] = e[j];
        }
    }
}

// out[v] = sum over partial rows of w[r*V + v] in a fixed order: a CTA covers 32 columns with 32 row slices
// (every thread sums rows slice, slice+32, ... with 8 loads in flight), then the slices are summed in order.
__device__ __forceinline__ void sum_cols_body(const float* __restrict__ w, float* __restrict__ out, int nrows, int V,
                                              int cblock, float* red) {
    const int cx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const int v = cblock * 32 + cx;
    float s = 0.f;
    if (v < V) {
        int r = sl;
        for (; r + 7 * 32 < nrows; r += 8 * 32) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = w[(long long)(r + 32 * i) * V + v];
#pragma unroll
            for (int i = 0; i < 8; ++i) s += x[i];
        }
        for (; r < nrows; r += 32) s += w[(long long)r * V + v];
    }
    red[sl * 32 + cx] = s;
    __syncthreads();
    if (sl == 0 && v < V) {
        float t = 0.f;
        for (int i = 0; i < 32; ++i) t += red[i * 32 + cx];
        out[v] = t;
    }
}
// The epilogue backward's two parameter reductions in one launch: CTAs [0, nh) sum dD per head (nh = H, or 0
// without the residual), the others sum 32 columns of dweight each.
__global__ void __launch_bounds__(1024) layer_epilogue_reduce_kernel(const float* __restrict__ w_dD,
                                                                     float* __restrict__ dD, long long tokens, int H,
                                                                     int nh, const float* __restrict__ w_dw,
                                                                     float* __restrict__ dweight, int nrows, int V) {
    __shared__ float red[1024];
    if ((int)blockIdx.x < nh)
        sum_heads_body(w_dD, dD, tokens, H, blockIdx.x, red);
    else
        sum_cols_body(w_dw, dweight, nrows, V, blockIdx.x - nh, red);
}

}  // namespace

// -------------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------------
namespace {

constexpr int LAYER_MAX_V = 1024;
constexpr int DW_CTAS = 1024;  // capacity for the partial rows of dweight (one per persistent CTA of the epilogue backward)

bool aligned_for(const void* p, int dt) { return (reinterpret_cast<uintptr_t>(p) & (dt == PALIMPSA_F32 ? 15 : 7)) == 0; }
int sm_count() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        return v;
    }();
    return n;
}
// CTAs of 8 warps for `warps` warp-rows: at most `waves` full waves of the kernel's resident CTAs (the
// kernels loop over the rest), so that no partial wave trails behind.
template <class Kern>
unsigned row_blocks(Kern kern, long long warps, size_t smem, int waves, int cap = 1 << 30) {
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, 256, smem) != cudaSuccess || occ < 1) occ = 1;
    long long full = (long long)sm_count() * occ * waves;
    if (full > cap) full = cap;
    const long long b = (warps + 7) / 8;
    return (unsigned)(b < 1 ? 1 : (b > full ? full : b));
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
    if (tokens * H > 0x7fffffffLL) return PALIMPSA_E_LIMIT;  // rows are indexed with 32-bit integers
    return PALIMPSA_OK;
}
int check_pro(const palimpsa_layer_prologue* a, bool bwd) {
    if (!a) return PALIMPSA_E_NULL;
    if (a->struct_size != sizeof(palimpsa_layer_prologue)) return PALIMPSA_E_VERSION;
    if (int rc = check_dims(a->io_dtype, a->H, a->V, a->tokens)) return rc;
    if (a->K <= 0 || a->Hq <= 0 || a->H % a->Hq) return PALIMPSA_E_SHAPE;
    if (a->K > PALIMPSA_MAX_K) return PALIMPSA_E_DIM;
    if (a->H > 4096) return PALIMPSA_E_LIMIT;  // per-head table in shared memory
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

// ---- dispatch on (dtype, chunks per lane, vector path) -----------------------------------------------------
template <int DT, int NCK, int NCV>
void pro_fwd_launch(const palimpsa_layer_prologue& a, int rows, bool veck, bool vecv, cudaStream_t st) {
    constexpr int R = (NCK == 1 && NCV == 1) ? 2 : 1;
    const size_t sm = (size_t)a.H * sizeof(float);
    const long long warps = (rows + R - 1) / R;
    if (veck && vecv) {
        auto kern = layer_prologue_fwd_kernel<DT, NCK, NCV, R, true, true>;
        kern<<<row_blocks(kern, warps, sm, 2), 256, sm, st>>>(a, rows);
    } else {
        auto kern = layer_prologue_fwd_kernel<DT, NCK, NCV, R, false, false>;
        kern<<<row_blocks(kern, warps, sm, 2), 256, sm, st>>>(a, rows);
    }
}
template <int DT, int NCK, int NCV>
void pro_bwd_launch(const palimpsa_layer_prologue& a, int qrows, bool veck, bool vecv, float* w0, float* w1,
                    cudaStream_t st) {
    const size_t sm = 2 * (size_t)a.H * sizeof(float);
    if (veck && vecv) {
        auto kern = layer_prologue_bwd_kernel<DT, NCK, NCV, true, true>;
        kern<<<row_blocks(kern, qrows, sm, 2), 256, sm, st>>>(a, qrows, w0, w1);
    } else {
        auto kern = layer_prologue_bwd_kernel<DT, NCK, NCV, false, false>;
        kern<<<row_blocks(kern, qrows, sm, 2), 256, sm, st>>>(a, qrows, w0, w1);
    }
}
template <int DT, int NC>
void epi_fwd_launch(const palimpsa_layer_epilogue& a, int rows, bool vecv, cudaStream_t st) {
    constexpr int R = NC == 1 ? 2 : 1;
    const long long warps = (rows + R - 1) / R;
    if (vecv) {
        auto kern = layer_epilogue_fwd_kernel<DT, NC, R, true>;
        kern<<<row_blocks(kern, warps, 0, 2), 256, 0, st>>>(a, rows);
    } else {
        auto kern = layer_epilogue_fwd_kernel<DT, NC, R, false>;
        kern<<<row_blocks(kern, warps, 0, 2), 256, 0, st>>>(a, rows);
    }
}
// returns the number of CTAs launched = partial rows of dweight written (one resident wave, at most DW_CTAS)
template <int DT, int NC>
unsigned epi_bwd_launch(const palimpsa_layer_epilogue& a, int rows, bool vecv, float* w0, float* w1, cudaStream_t st) {
    constexpr int R = NC == 1 ? 2 : 1;
    const long long warps = (rows + R - 1) / R;
    unsigned nb;
    if (vecv) {
        auto kern = layer_epilogue_bwd_kernel<DT, NC, R, true>;
        nb = row_blocks(kern, warps, 0, 1, DW_CTAS);
        kern<<<nb, 256, 0, st>>>(a, rows, w0, w1);
    } else {
        auto kern = layer_epilogue_bwd_kernel<DT, NC, R, false>;
        nb = row_blocks(kern, warps, 0, 1, DW_CTAS);
        kern<<<nb, 256, 0, st>>>(a, rows, w0, w1);
    }
    return nb;
}

#define PALIMPSA_BY_DTYPE(dt, CALL)                                   \
    do {                                                              \
        if ((dt) == PALIMPSA_BF16) { CALL(PALIMPSA_BF16); }           \
        else if ((dt) == PALIMPSA_F16) { CALL(PALIMPSA_F16); }        \
        else { CALL(PALIMPSA_F32); }                                  \
    } while (0)
// chunks of 4 per lane: 1, 2, 4 or 8 (d_v <= 128, 256, 512, 1024); d_k: 1 or 2
#define PALIMPSA_BY_NCV(ncv, CALL)            \
    do {                                      \
        if ((ncv) <= 1) { CALL(1); }          \
        else if ((ncv) <= 2) { CALL(2); }     \
        else if ((ncv) <= 4) { CALL(4); }     \
        else { CALL(8); }                     \
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
    const int rows = (int)(a->tokens * a->H);
    if (rows == 0) return PALIMPSA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int dt = a->io_dtype;
    const bool veck = a->K % 4 == 0 && aligned_for(a->q_raw, dt) && aligned_for(a->k_raw, dt) && aligned_for(a->q, dt) &&
                      aligned_for(a->k, dt);
    const bool vecv = a->V % 4 == 0 && aligned_for(a->x, dt) && aligned_for(a->b_raw, dt) && aligned_for(a->v, dt) &&
                      aligned_for(a->b, dt);
    const int nck = (a->K + 127) / 128, ncv = (a->V + 127) / 128;
#define CALL_V(NV)                                                                         \
    do {                                                                                   \
        if (nck <= 1) pro_fwd_launch<DTX, 1, NV>(*a, rows, veck, vecv, st);                \
        else pro_fwd_launch<DTX, 2, NV>(*a, rows, veck, vecv, st);                         \
    } while (0)
#define CALL_D(D)                      \
    do {                               \
        constexpr int DTX = D;         \
        PALIMPSA_BY_NCV(ncv, CALL_V);  \
    } while (0)
    PALIMPSA_BY_DTYPE(dt, CALL_D);
#undef CALL_D
#undef CALL_V
    return launched();
}

int palimpsa_layer_prologue_bwd(const palimpsa_layer_prologue* a, void* cuda_stream) {
    if (int rc = check_pro(a, true)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int rows = (int)(a->tokens * a->H), qrows = (int)(a->tokens * a->Hq);
    float* w_dtb = reinterpret_cast<float*>(a->workspace);
    float* w_bsc = w_dtb + rows;
    if (rows > 0) {
        const int dt = a->io_dtype;
        const bool veck = a->K % 4 == 0 && aligned_for(a->q_raw, dt) && aligned_for(a->k_raw, dt) &&
                          aligned_for(a->dq, dt) && aligned_for(a->dk, dt) && aligned_for(a->dq_raw, dt) &&
                          aligned_for(a->dk_raw, dt);
        const bool vecv = a->V % 4 == 0 && aligned_for(a->x, dt) && aligned_for(a->b_raw, dt) && aligned_for(a->dv, dt) &&
                          aligned_for(a->db, dt) && aligned_for(a->dx, dt) && aligned_for(a->db_raw, dt);
        const int nck = (a->K + 127) / 128, ncv = (a->V + 127) / 128;
#define CALL_V(NV)                                                                                \
    do {                                                                                          \
        if (nck <= 1) pro_bwd_launch<DTX, 1, NV>(*a, qrows, veck, vecv, w_dtb, w_bsc, st);        \
        else pro_bwd_launch<DTX, 2, NV>(*a, qrows, veck, vecv, w_dtb, w_bsc, st);                 \
    } while (0)
#define CALL_D(D)                      \
    do {                               \
        constexpr int DTX = D;         \
        PALIMPSA_BY_NCV(ncv, CALL_V);  \
    } while (0)
        PALIMPSA_BY_DTYPE(dt, CALL_D);
#undef CALL_D
#undef CALL_V
        if (int rc = launched()) return rc;
    }
    layer_sum_heads_kernel<<<dim3(a->H, 2), 1024, 0, st>>>(w_dtb, a->d_dt_bias, w_bsc, a->d_b_scale, a->tokens, a->H);
    return launched();
}

int palimpsa_layer_epilogue_fwd(const palimpsa_layer_epilogue* a, void* cuda_stream) {
    if (int rc = check_epi(a, false)) return rc;
    const int rows = (int)(a->tokens * a->H);
    if (rows == 0) return PALIMPSA_OK;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int dt = a->io_dtype;
    const bool vecv = a->V % 4 == 0 && aligned_for(a->o, dt) && aligned_for(a->y, dt) &&
                      (!(a->flags & PALIMPSA_LAYER_RESIDUAL) || aligned_for(a->x, dt)) &&
                      (!(a->flags & PALIMPSA_LAYER_GATE) || aligned_for(a->gate, dt));
    const int nc = (a->V + 127) / 128;
#define CALL_V(NV) epi_fwd_launch<DTX, NV>(*a, rows, vecv, st)
#define CALL_D(D)                     \
    do {                              \
        constexpr int DTX = D;        \
        PALIMPSA_BY_NCV(nc, CALL_V);  \
    } while (0)
    PALIMPSA_BY_DTYPE(dt, CALL_D);
#undef CALL_D
#undef CALL_V
    return launched();
}

int palimpsa_layer_epilogue_bwd(const palimpsa_layer_epilogue* a, void* cuda_stream) {
    if (int rc = check_epi(a, true)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    const int rows = (int)(a->tokens * a->H);
    const bool res = a->flags & PALIMPSA_LAYER_RESIDUAL, gated = a->flags & PALIMPSA_LAYER_GATE;
    float* w_dD = reinterpret_cast<float*>(a->workspace);
    float* w_dw = w_dD + rows;
    const int nc = (a->V + 127) / 128;
    unsigned nb = 0;
    if (rows > 0) {
        const int dt = a->io_dtype;
        const bool vecv = a->V % 4 == 0 && aligned_for(a->o, dt) && aligned_for(a->dy, dt) && aligned_for(a->d_o, dt) &&
                          (!res || (aligned_for(a->x, dt) && aligned_for(a->dx, dt))) &&
                          (!gated || (aligned_for(a->gate, dt) && aligned_for(a->dgate, dt)));
#define CALL_V(NV) nb = epi_bwd_launch<DTX, NV>(*a, rows, vecv, w_dD, w_dw, st)
#define CALL_D(D)                     \
    do {                              \
        constexpr int DTX = D;        \
        PALIMPSA_BY_NCV(nc, CALL_V);  \
    } while (0)
        PALIMPSA_BY_DTYPE(dt, CALL_D);
#undef CALL_D
#undef CALL_V
        if (int rc = launched()) return rc;
    }
    const int nh = res ? a->H : 0;
    layer_epilogue_reduce_kernel<<<nh + (a->V + 31) / 32, 1024, 0, st>>>(w_dD, a->dD, a->tokens, a->H, nh, w_dw,
                                                                          a->dweight, (int)nb, a->V);
    return launched();
}

}  // extern "C"
