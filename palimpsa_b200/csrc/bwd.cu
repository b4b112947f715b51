// Backward kernels of the Palimpsa operator (sm_100a).
//
// Main kernel: one CTA owns TV state rows x all KP columns of one (sequence, head) and walks the
// sequence's 16-token blocks from the last to the first.  Per block it
//   1. takes the block's start state (M, I) from the checkpoint the forward saved (prefetched into
//      shared memory one block ahead with cp.async, together with the block's raw inputs),
//   2. sweeps forward once, parking the state at the start of each 4-token group (thread-private
//      slots in shared memory),
//   3. per group, last first: recomputes the 4 per-token states into registers, then walks the
//      tokens in reverse, carrying the state gradients (GM, -GI) in registers:
//          h    = dy*q_s / I            GM = f_next*GM + h          -GI = f_next*(-GI) + h*mu (+var)
//          dq  += dy*mu   dk += GM*v + 2k*GI*b   dv += GM*k   db += GI*k^2
//          df   = <GM, M_prev> + <GI, I_prev - Ip>
//      (the algebra of chunk_palimpsa_bwd_kernel, chunk_palimpsa_forgetting_scalar.py:343-434,
//      with the previous state carried forward instead of rebuilt by a division, :409-410).
// Reductions: over d_k (dv, db) by xor-shuffles inside the lanes of a row; over d_v (dq, dk) first
// in registers across a thread's rows, then across the CTA's row groups through shared memory, and
// across the CTAs of different row tiles through fp32 partial buffers in the workspace, which the
// finishing kernel sums in a fixed order (bitwise reproducible; no atomics).  The CTA-wide barriers of
// the shared-memory step are mbarriers split into arrive / wait halves (bounded waits), so that the
// warps of the single resident CTA do not alternate in lockstep between FP32 work and reductions.
// One CTA per SM: 11 or 12 warps at d_k = 128 (22- or 24-row tiles, whichever pads d_v less).
//
// Finishing kernels: (1) per (token, head) row: sum the row tiles, cast dq/dk, form
// dgt = -g f df and the per-row terms of dg and dIp; (2) per head: ordered sum over rows.
#include <mutex>

#include "host.h"
#include "tc_common.cuh"

namespace palimpsa {

constexpr int GR = 4;  // tokens per register-resident group

// 0 ok; 5 / 6: a bounded wait on the split-phase barriers of the backward's group reduction gave up
__device__ int g_bwd_status = 0;

__device__ __forceinline__ void mbar_init_n(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tc::smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}" ::"r"(tc::smem_u32(bar)) : "memory");
}

struct BwdArgs {
    palimpsa_problem p;
    const void* d_o;
    const void* d_o_var;
    const float* ckpt_M;
    const float* ckpt_I;
    float *dq_part, *dk_part, *df_part, *dip_part;
    void *dv, *db;
    int aligned;
    int kbuf;        // shared-memory buffers for the per-group d_k-indexed partials: 2 where they fit, else 1
    int rows_total;  // tokens * H
    // segments (gridDim.z of them per sequence; seg_len tokens each, a multiple of 16; 0 = whole sequence)
    int seg_len;
    const float* carry_M;  // [N,G,H,V,KP] dL/d(end state of the segment), (M, I) form, or NULL (zero)
    const float* carry_I;
    float* rloc_M;         // [N,G,H,V,KP] dL/d(start state of the segment), or NULL
    float* rloc_I;
};

struct BwdSmem {
    int ks, qs, qqs, vs2, bs2, dys2, dyvs2, fc2, fn2, dvs, dbs, wred, slots, ckb, kred;
    int ck_stage;  // bytes of one (M, I) checkpoint stage
    int raw, rq, rk, rv, rb, rdo, rdov, rgt;
    int total;
};

// Columns per token of the raw d_v-indexed staging tiles: the row tile widened to 16-byte boundaries of the
// global rows on both sides (a tile of 22 rows does not start on one).
__host__ __device__ constexpr int bwd_staged_cols(int TV) { return (TV + 7) / 8 * 8 + 8; }

// Shared-memory plan of one backward CTA (KP padded d_k, TV state rows, NE state elements per thread,
// WV row groups).  Operand tiles v, b, dy are stored with every value duplicated ({x, x}) so that a
// 64-bit load yields the register pair the packed FP32 instructions want.
__host__ __device__ inline BwdSmem bwd_smem_layout(int KP, int TV, int NE, int nthr, int WV, int es, bool unc,
                                                  int kbuf) {
    BwdSmem s;
    int off = 0;
    auto take = [&](int bytes) {
        int o = off;
        off += round_up(bytes, 16);
        return o;
    };
    s.ks = take(TB * KP * 4);
    s.qs = take(TB * KP * 4);
    s.qqs = unc ? take(TB * KP * 4) : 0;
    s.vs2 = take(TB * TV * 8);
    s.bs2 = take(TB * TV * 8);
    s.dys2 = take(TB * TV * 8);
    s.dyvs2 = unc ? take(TB * TV * 8) : 0;
    s.fc2 = take(TB * 16);
    s.fn2 = take(TB * 8);
    s.dvs = take(TB * TV * 4);
    s.dbs = take(TB * TV * 4);
    s.wred = take((nthr / 32) * TB * 2 * 4);
    s.slots = take(2 * 2 * NE * nthr * 4);
    s.ck_stage = 2 * TV * KP * 4;
    s.ckb = take(2 * s.ck_stage);
    s.kred = take(kbuf * GR * WV * 2 * KP * 4);  // kbuf = 2 group buffers where they fit (host's choice), else 1
    s.raw = off;
    int r = 0;
    auto rtake = [&](int bytes) {
        int o = r;
        r += round_up(bytes, 16);
        return o;
    };
    const int TVS = bwd_staged_cols(TV);
    s.rq = rtake(TB * KP * es);
    s.rk = rtake(TB * KP * es);
    s.rv = rtake(TB * TVS * es);
    s.rb = rtake(TB * TVS * es);
    s.rdo = rtake(TB * TVS * es);
    s.rdov = unc ? rtake(TB * TVS * es) : 0;
    s.rgt = rtake((TB + 1) * 4);
    s.total = off + r;
    return s;
}

// Asynchronous copy of one block's checkpoint rows (M, I) into checkpoint stage `stage_idx`.
__device__ __forceinline__ void bwd_issue_ckpt(const BwdArgs& a, unsigned char* sm, const BwdSmem& L, int stage_idx,
                                               int KP, int TV, long long slot, int h, int v0, int tvw) {
    const palimpsa_problem& p = a.p;
    const int nthr = blockDim.x, tid = threadIdx.x;
    unsigned char* ck = sm + L.ckb + stage_idx * L.ck_stage;
    const int cr = KP / 4;
    const long long base = ((slot * p.H + h) * (long long)p.V + v0) * KP;
    for (int i = tid; i < tvw * cr; i += nthr) {
        cp_async16(ck + i * 16, a.ckpt_M + base + (long long)i * 4);
        cp_async16(ck + TV * KP * 4 + i * 16, a.ckpt_I + base + (long long)i * 4);
    }
}

// Asynchronous copy of one block's raw inputs (aligned path only).
__device__ __forceinline__ void bwd_issue_raw(const BwdArgs& a, unsigned char* sm, const BwdSmem& L, int es, int KP,
                                              int TV, long long tok0, int nt, int nt_ext, int h, int v0, int tvw) {
    const palimpsa_problem& p = a.p;
    const int nthr = blockDim.x, tid = threadIdx.x;
    unsigned char* stage = sm + L.raw;
    const int cq = p.K * es / 16;
    const char* gq = reinterpret_cast<const char*>(p.q);
    const char* gk = reinterpret_cast<const char*>(p.k);
    for (int i = tid; i < nt * cq; i += nthr) {
        int t = i / cq, c = i - t * cq;
        long long src = ((tok0 + t) * p.H + h) * (long long)p.K * es + c * 16;
        int dst = t * KP * es + c * 16;
        cp_async16(stage + L.rq + dst, gq + src);
        cp_async16(stage + L.rk + dst, gk + src);
    }
    // the aligned superset [va, va + span) of the tile's columns [v0, v0 + tvw); d_v*es is a multiple of 16 on
    // this path, so the superset stays inside the row
    const int ea = 16 / es, va = v0 / ea * ea, span = (v0 - va + tvw + ea - 1) / ea * ea;
    const int cv = span * es / 16, TVS = bwd_staged_cols(TV);
    const char* gv = reinterpret_cast<const char*>(p.v);
    const char* gb = reinterpret_cast<const char*>(p.b);
    const char* gdo = reinterpret_cast<const char*>(a.d_o);
    const char* gdov = reinterpret_cast<const char*>(a.d_o_var);
    for (int i = tid; i < nt * cv; i += nthr) {
        int t = i / cv, c = i - t * cv;
        long long src = (((tok0 + t) * p.H + h) * (long long)p.V + va) * es + c * 16;
        int dst = t * TVS * es + c * 16;
        cp_async16(stage + L.rv + dst, gv + src);
        cp_async16(stage + L.rb + dst, gb + src);
        cp_async16(stage + L.rdo + dst, gdo + src);
        if (gdov) cp_async16(stage + L.rdov + dst, gdov + src);
    }
    for (int i = tid; i < nt_ext; i += nthr) cp_async4(stage + L.rgt + i * 4, p.gt + (tok0 + i) * p.H + h);
}

// Two consecutive staged values starting at the even element index e (shared memory).
template <int DT>
__device__ __forceinline__ float2 ld2s(const unsigned char* base, int e) {
    if (DT == PALIMPSA_F32) return *reinterpret_cast<const float2*>(base + (size_t)e * 4);
    if (DT == PALIMPSA_BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(base + (size_t)e * 2));
    return __half22float2(*reinterpret_cast<const __half2*>(base + (size_t)e * 2));
}

template <int DT, bool ALIGNED, bool UNC>
__device__ __forceinline__ void bwd_convert(const BwdArgs& a, unsigned char* sm, const BwdSmem& L, int KP, int TV,
                                            long long tok0, int nt, int nt_ext, int h, int v0, float gh, float iph,
                                            bool carry_block) {
    const palimpsa_problem& p = a.p;
    const int nthr = blockDim.x, tid = threadIdx.x;
    const int K4 = KP / 4, V4 = TV / 4;
    const unsigned char* stage = sm + L.raw;
    float4* qs = reinterpret_cast<float4*>(sm + L.qs);
    float4* ks = reinterpret_cast<float4*>(sm + L.ks);
    float4* qqs = reinterpret_cast<float4*>(sm + L.qqs);
    const float sc = p.scale;
    for (int i = tid; i < TB * K4; i += nthr) {
        int t = i / K4, c4 = i - t * K4;
        float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), kv = qv;
        if (t < nt && c4 * 4 < p.K) {
            if (ALIGNED) {
                qv = ld4<DT>(stage + L.rq, i);
                kv = ld4<DT>(stage + L.rk, i);
            } else {
                long long row = ((tok0 + t) * p.H + h) * (long long)p.K;
                qv = ld4_guarded<DT>(p.q, row + c4 * 4, row + p.K);
                kv = ld4_guarded<DT>(p.k, row + c4 * 4, row + p.K);
            }
        }
        qs[i] = make_float4(qv.x * sc, qv.y * sc, qv.z * sc, qv.w * sc);
        ks[i] = kv;
        if (UNC) qqs[i] = make_float4(sc * qv.x * qv.x, sc * qv.y * qv.y, sc * qv.z * qv.z, sc * qv.w * qv.w);
    }
    float4* vs = reinterpret_cast<float4*>(sm + L.vs2);
    float4* bs = reinterpret_cast<float4*>(sm + L.bs2);
    float4* dys = reinterpret_cast<float4*>(sm + L.dys2);
    float4* dyvs = reinterpret_cast<float4*>(sm + L.dyvs2);
    const int TVS = bwd_staged_cols(TV);
    const int voff = ALIGNED ? v0 % (16 / dtype_size(DT)) : 0;  // tile start inside the staged superset
    if ((TV | voff) & 3) {
        // tile width or offset not a multiple of 4 (both are even): two values at a time
        const int V2 = TV / 2;
        for (int i = tid; i < TB * V2; i += nthr) {
            const int t = i / V2, c2 = i - t * V2;
            float2 vv = make_float2(0.f, 0.f), bv = vv, dv = vv, dvv = vv;
            if (t < nt && v0 + c2 * 2 < p.V) {
                if (ALIGNED) {
                    const int e = t * TVS + voff + 2 * c2;
                    vv = ld2s<DT>(stage + L.rv, e);
                    bv = ld2s<DT>(stage + L.rb, e);
                    dv = ld2s<DT>(stage + L.rdo, e);
                    if (UNC) dvv = ld2s<DT>(stage + L.rdov, e);
                } else {
                    const long long row = ((tok0 + t) * p.H + h) * (long long)p.V, e = row + v0 + c2 * 2;
                    const bool two = e + 1 < row + p.V;
                    vv = make_float2(ld1<DT>(p.v, e), two ? ld1<DT>(p.v, e + 1) : 0.f);
                    bv = make_float2(ld1<DT>(p.b, e), two ? ld1<DT>(p.b, e + 1) : 0.f);
                    dv = make_float2(ld1<DT>(a.d_o, e), two ? ld1<DT>(a.d_o, e + 1) : 0.f);
                    if (UNC) dvv = make_float2(ld1<DT>(a.d_o_var, e), two ? ld1<DT>(a.d_o_var, e + 1) : 0.f);
                }
            }
            vs[i] = make_float4(vv.x, vv.x, vv.y, vv.y);
            bs[i] = make_float4(bv.x, bv.x, bv.y, bv.y);
            dys[i] = make_float4(dv.x, dv.x, dv.y, dv.y);
            if (UNC) dyvs[i] = make_float4(dvv.x, dvv.x, dvv.y, dvv.y);
        }
    } else
    for (int i = tid; i < TB * V4; i += nthr) {
        int t = i / V4, c4 = i - t * V4;
        float4 vv = make_float4(0.f, 0.f, 0.f, 0.f), bv = vv, dv = vv, dvv = vv;
        if (t < nt && v0 + c4 * 4 < p.V) {
            if (ALIGNED) {
                const int g4 = (t * TVS + voff) / 4 + c4;  // TVS, voff multiples of 4 here
                vv = ld4<DT>(stage + L.rv, g4);
                bv = ld4<DT>(stage + L.rb, g4);
                dv = ld4<DT>(stage + L.rdo, g4);
                if (UNC) dvv = ld4<DT>(stage + L.rdov, g4);
            } else {
                long long row = ((tok0 + t) * p.H + h) * (long long)p.V;
                vv = ld4_guarded<DT>(p.v, row + v0 + c4 * 4, row + p.V);
                bv = ld4_guarded<DT>(p.b, row + v0 + c4 * 4, row + p.V);
                dv = ld4_guarded<DT>(a.d_o, row + v0 + c4 * 4, row + p.V);
                if (UNC) dvv = ld4_guarded<DT>(a.d_o_var, row + v0 + c4 * 4, row + p.V);
            }
        }
        st_dup4(vs, i, vv);
        st_dup4(bs, i, bv);
        st_dup4(dys, i, dv);
        if (UNC) st_dup4(dyvs, i, dvv);
    }
    // per token: {f, f, c, c} with c = (1-f)*Ip, and {fn, fn}: f of the NEXT token of the sequence (0 past its end)
    float4* fc2 = reinterpret_cast<float4*>(sm + L.fc2);
    float2* fn2 = reinterpret_cast<float2*>(sm + L.fn2);
    for (int i = tid; i < TB; i += nthr) {
        float g0 = 0.f, g1 = 0.f;
        const bool has0 = i < nt, has1 = i + 1 < nt_ext;
        if (ALIGNED) {
            const float* rg = reinterpret_cast<const float*>(stage + L.rgt);
            if (has0) g0 = rg[i];
            if (has1) g1 = rg[i + 1];
        } else {
            if (has0) g0 = p.gt[(tok0 + i) * p.H + h];
            if (has1) g1 = p.gt[(tok0 + i + 1) * p.H + h];
        }
        const float f = expf(-g0 * gh);
        float fn = has1 ? expf(-g1 * gh) : 0.f;
        // Last block of a segment whose end-state gradient is supplied: that gradient is already expressed
        // at the boundary, so the last real token (and any identity padding after it) passes it on undecayed.
        if (carry_block && i >= nt - 1) fn = 1.f;
        const float c = (1.f - f) * iph;
        fc2[i] = make_float4(f, f, c, c);
        fn2[i] = make_float2(fn, fn);
    }
}

template <int RV, int NP>
struct State {
    float2 M[RV][NP], I[RV][NP];
};

template <int RK, int KG, int RV, int W, bool UNC, bool CO>
__global__ void __launch_bounds__(32 * W) bwd_kernel(const BwdArgs a) {
    constexpr int KP = RK * KG, VG = 32 / KG, NP = RK / 2, NE = RV * RK, KP2 = KP / 2;
    constexpr int TV = W * VG * RV, WV = W * VG, NTHR = 32 * W;
    constexpr int NG = TB / GR;       // groups per block
    constexpr int NR1 = GR * RV * 2;  // per-group d_v-indexed partials of a thread: (token, row, dv|db)
    constexpr int NR2 = GR * 2;       // per-group per-token scalars: (token, df|sum GI)
    extern __shared__ __align__(16) unsigned char sm[];
    const palimpsa_problem& p = a.p;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int kg = lane % KG, vg = lane / KG, wv = w * VG + vg;
    const int row0 = wv * RV;
    const int ny = blockIdx.y / p.H, h = blockIdx.y - ny * p.H;
    const int n = p.seq_order ? p.seq_order[ny] : ny;  // blocks start in grid order: a packed batch lists its longest sequences first
    const int tile = blockIdx.x;
    const int v0 = tile * TV;
    const int tvw = min(TV, p.V - v0);
    const int es = dtype_size(p.io_dtype);
    const int KBUF = a.kbuf;  // shared-memory buffers for the d_k-indexed partials of a token group (1 or 2)
    const BwdSmem L = bwd_smem_layout(KP, TV, NE, NTHR, WV, es, UNC, KBUF);
    int bos, len;
    seq_range(p, n, bos, len);
    // this CTA's segment of the sequence: tokens [s0, s1), blocks [blk0, blk1)
    const int g = blockIdx.z, G = gridDim.z;
    const int s0 = a.seg_len > 0 ? min(len, g * a.seg_len) : 0;
    const int s1 = a.seg_len > 0 ? min(len, s0 + a.seg_len) : len;
    const long long seg_base = (((long long)n * G + g) * p.H + h) * p.V;  // row index into [N,G,H,V,KP] buffers
    if (s1 <= s0) {  // empty segment: the end-state gradient is the start-state gradient
        if (a.rloc_M) {
            for (int i = tid; i < tvw * (KP / 4); i += NTHR) {
                const long long e = (seg_base + v0) * KP + (long long)i * 4;
                float4 cm = make_float4(0.f, 0.f, 0.f, 0.f), ci = cm;
                if (!CO && a.carry_M) {
                    cm = *reinterpret_cast<const float4*>(a.carry_M + e);
                    ci = *reinterpret_cast<const float4*>(a.carry_I + e);
                }
                *reinterpret_cast<float4*>(a.rloc_M + e) = cm;
                *reinterpret_cast<float4*>(a.rloc_I + e) = ci;
            }
        }
        return;
    }
    const float gh = p.g[h], iph = p.Ip[h];
    const int V = p.V;
    const long long slot0 = seq_first_slot(p, n);
    const int blk0 = s0 / TB, blk1 = (s1 + TB - 1) / TB;
    const int nblk = blk1 - blk0;
    const bool has_carry = !CO && a.carry_M != nullptr;
    const bool has_init = p.init_mu != nullptr || (p.flags & PALIMPSA_FLAG_EXPLICIT_INIT);

    // The CTA-wide barriers of the per-group reduction over d_v are split into arrive / wait halves
    // (mbarriers, one arrival per warp).  A: a warp that has written its partials of a group goes on with its
    // own shuffle reductions before it waits for the others' partials.  B (single buffer only): a warp that
    // has read the buffer goes on with the next group's recompute before it waits for the others to finish
    // reading; with two buffers the next group writes the other one and A alone orders everything.  The warps
    // of the CTA then drift apart by up to a group and stop hitting the FP32 pipe and the reduction phases
    // all at the same time.  Waits are bounded; a wait that gives up is recorded.
    constexpr bool SPLIT_A = !CO;
    const bool SPLIT_B = KBUF == 1 && !CO;
    __shared__ __align__(8) unsigned long long gbar[2];
    unsigned ph_a = 0, ph_b = 0;
    int wait_fail = 0;
    if (SPLIT_A) {
        if (tid == 0) {
            mbar_init_n(&gbar[0], W);
            mbar_init_n(&gbar[1], W);
            tc::mbar_init_fence();
        }
        __syncthreads();
        if (SPLIT_B && lane == 0) mbar_arrive(&gbar[1]);  // nobody reads before the first group: B starts complete
    }

    // this thread's d_k columns are RK*kg .. RK*kg+RK-1: pair q covers columns RK*kg + 2q, +1
    const float2* ks2 = reinterpret_cast<const float2*>(sm + L.ks) + NP * kg;
    const float2* qs2 = reinterpret_cast<const float2*>(sm + L.qs) + NP * kg;
    const float2* qqs2 = reinterpret_cast<const float2*>(sm + L.qqs) + NP * kg;
    const float2* vs2 = reinterpret_cast<const float2*>(sm + L.vs2) + row0;
    const float2* bs2 = reinterpret_cast<const float2*>(sm + L.bs2) + row0;
    const float2* dys2 = reinterpret_cast<const float2*>(sm + L.dys2) + row0;
    const float2* dyvs2 = reinterpret_cast<const float2*>(sm + L.dyvs2) + row0;
    const float4* fc2 = reinterpret_cast<const float4*>(sm + L.fc2);
    const float2* fn2 = reinterpret_cast<const float2*>(sm + L.fn2);
    float* dvs = reinterpret_cast<float*>(sm + L.dvs);
    float* dbs = reinterpret_cast<float*>(sm + L.dbs);
    float* wred = reinterpret_cast<float*>(sm + L.wred);
    float4* slots4 = reinterpret_cast<float4*>(sm + L.slots) + tid;
    float2* kred2 = reinterpret_cast<float2*>(sm + L.kred);

    // running state gradients: GM = dL/dM_t, nGI = -dL/dI_t of the earliest token processed so far
    float2 GM[RV][NP], nGI[RV][NP];
#pragma unroll
    for (int r = 0; r < RV; ++r)
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            GM[r][q] = nGI[r][q] = make_float2(0.f, 0.f);
            if (has_carry && row0 + r < tvw) {
                const long long e = (seg_base + v0 + row0 + r) * KP + RK * kg + 2 * q;
                const float2 cm = *reinterpret_cast<const float2*>(a.carry_M + e);
                const float2 ci = *reinterpret_cast<const float2*>(a.carry_I + e);
                GM[r][q] = cm;
                nGI[r][q] = make_float2(-ci.x, -ci.y);
            }
        }

    auto load_ck = [&](State<RV, NP>& s, int stage_idx) {
        const float* ckM = reinterpret_cast<const float*>(sm + L.ckb + stage_idx * L.ck_stage);
        const float* ckI = ckM + TV * KP;
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            const bool ok = row0 + r < tvw;
#pragma unroll
            for (int q = 0; q < NP; ++q) {
                const int e = (row0 + r) * KP + RK * kg + 2 * q;
                s.M[r][q] = ok ? *reinterpret_cast<const float2*>(ckM + e) : make_float2(0.f, 0.f);
                s.I[r][q] = ok ? *reinterpret_cast<const float2*>(ckI + e) : make_float2(1.f, 1.f);
            }
        }
    };
    auto load_slot = [&](State<RV, NP>& s, int slot) {
        const float4* sl = slots4 + slot * (NE / 2) * NTHR;
#pragma unroll
        for (int r = 0; r < RV; ++r)
#pragma unroll
            for (int q = 0; q < NP; ++q) {
                const float4 x = sl[(r * NP + q) * NTHR];
                s.M[r][q] = make_float2(x.x, x.y);
                s.I[r][q] = make_float2(x.z, x.w);
            }
    };
    auto store_slot = [&](const State<RV, NP>& s, int slot) {
        float4* sl = slots4 + slot * (NE / 2) * NTHR;
#pragma unroll
        for (int r = 0; r < RV; ++r)
#pragma unroll
            for (int q = 0; q < NP; ++q)
                sl[(r * NP + q) * NTHR] = make_float4(s.M[r][q].x, s.M[r][q].y, s.I[r][q].x, s.I[r][q].y);
    };
    // operand loads: two adjacent 8-byte pairs come in as one 16-byte load where the tiling allows it
    auto ld_cols = [&](const float2* base, int tl, float2 (&dst)[NP]) {
        if constexpr (NP % 2 == 0) {
#pragma unroll
            for (int q = 0; q < NP; q += 2) {
                const float4 x = *reinterpret_cast<const float4*>(base + tl * KP2 + q);
                dst[q] = make_float2(x.x, x.y);
                dst[q + 1] = make_float2(x.z, x.w);
            }
        } else {
#pragma unroll
            for (int q = 0; q < NP; ++q) dst[q] = base[tl * KP2 + q];
        }
    };
    auto ld_rows = [&](const float2* base, int tl, float2 (&dst)[RV]) {
        if constexpr (RV % 2 == 0) {
#pragma unroll
            for (int r = 0; r < RV; r += 2) {
                const float4 x = *reinterpret_cast<const float4*>(base + tl * TV + r);
                dst[r] = make_float2(x.x, x.y);
                dst[r + 1] = make_float2(x.z, x.w);
            }
        } else {
#pragma unroll
            for (int r = 0; r < RV; ++r) dst[r] = base[tl * TV + r];
        }
    };
    // one forward step of the recurrence on token tl of the staged block
    auto fstep = [&](State<RV, NP>& s, int tl) {
        const float4 fv = fc2[tl];
        const float2 ff = make_float2(fv.x, fv.y), cc = make_float2(fv.z, fv.w);
        float2 vr[RV], br[RV], kpv[NP];
        ld_rows(vs2, tl, vr);
        ld_rows(bs2, tl, br);
        ld_cols(ks2, tl, kpv);
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            const float2 kp = kpv[q];
            const float2 kk = fmul2(kp, kp);
#pragma unroll
            for (int r = 0; r < RV; ++r) {
                s.M[r][q] = ffma2(ff, s.M[r][q], fmul2(vr[r], kp));
                s.I[r][q] = ffma2(ff, s.I[r][q], ffma2(br[r], kk, cc));
            }
        }
    };

    {
        const int c = blk1 - 1;
        const int nt = min(TB, len - c * TB);
        bwd_issue_ckpt(a, sm, L, 0, KP, TV, slot0 + c, h, v0, tvw);
        if (a.aligned) bwd_issue_raw(a, sm, L, es, KP, TV, (long long)bos + c * TB, nt, nt, h, v0, tvw);
        cp_async_commit();
    }

    for (int it = 0; it < nblk; ++it) {
        const int c = blk1 - 1 - it;
        const bool cblk = has_carry && it == 0;
        const int t0 = c * TB;
        const int nt = min(TB, len - t0);
        const int nt_ext = min(TB + 1, len - t0);
        const long long tok0 = (long long)bos + t0;
        const int st = it & 1;
        cp_async_wait<0>();
        __syncthreads();
        if (a.aligned) {
            if (p.io_dtype == PALIMPSA_BF16)
                bwd_convert<PALIMPSA_BF16, true, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
            else if (p.io_dtype == PALIMPSA_F32)
                bwd_convert<PALIMPSA_F32, true, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
            else
                bwd_convert<PALIMPSA_F16, true, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
        } else {
            if (p.io_dtype == PALIMPSA_BF16)
                bwd_convert<PALIMPSA_BF16, false, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
            else if (p.io_dtype == PALIMPSA_F32)
                bwd_convert<PALIMPSA_F32, false, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
            else
                bwd_convert<PALIMPSA_F16, false, UNC>(a, sm, L, KP, TV, tok0, nt, nt_ext, h, v0, gh, iph, cblk);
        }
        __syncthreads();
        // the raw stage is free again: fetch the next (earlier) block while this one is processed
        if (c > blk0) {
            const int t0n = t0 - TB;
            bwd_issue_ckpt(a, sm, L, st ^ 1, KP, TV, slot0 + c - 1, h, v0, tvw);
            if (a.aligned)
                bwd_issue_raw(a, sm, L, es, KP, TV, (long long)bos + t0n, TB, min(TB + 1, len - t0n), h, v0, tvw);
            cp_async_commit();
        }

        // Tokens past the end of the sequence (last block only) were staged as identity steps (f = 1,
        // all other operands 0): they leave the state and every gradient untouched, so the block is
        // always processed as NG full groups with no per-token conditionals.
        // ---- forward sweep: park the start states of groups 1 .. NG-2, keep the last group's in registers
        State<RV, NP> P[GR + 1];
        load_ck(P[0], st);
#pragma unroll 1
        for (int g = 0; g < NG - 1; ++g) {
#pragma unroll
            for (int j = 0; j < GR; ++j) fstep(P[0], g * GR + j);
            if (g < NG - 2) store_slot(P[0], g);
        }

#pragma unroll 1
        for (int gi = NG - 1; gi >= 0; --gi) {
            if (gi == 0)
                load_ck(P[0], st);
            else if (gi < NG - 1)
                load_slot(P[0], gi - 1);
#pragma unroll
            for (int j = 0; j < GR; ++j) {
                P[j + 1] = P[j];
                fstep(P[j + 1], gi * GR + j);
            }
            float red1[NR1], red2[NR2];
            // ---- reverse walk over the group ----------------------------------------------------
#pragma unroll
            for (int j = GR - 1; j >= 0; --j) {
                const int tl = gi * GR + j;
                const float2 fn = fn2[tl];
                float2 dqs[NP], Ak[NP], Bk[NP], Uk[NP];
                float2 Sa[RV], Sb[RV], Sc[RV];  // one accumulator per row: shorter dependent chains
#pragma unroll
                for (int r = 0; r < RV; ++r) Sa[r] = Sb[r] = Sc[r] = make_float2(0.f, 0.f);
#pragma unroll
                for (int q = 0; q < NP; ++q) dqs[q] = Ak[q] = Bk[q] = Uk[q] = make_float2(0.f, 0.f);
                float2 kp[NP], kk[NP], qp[NP], qq[NP];
                ld_cols(ks2, tl, kp);
                ld_cols(qs2, tl, qp);
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    kk[q] = fmul2(kp[q], kp[q]);
                    qq[q] = make_float2(0.f, 0.f);
                }
                if (UNC) ld_cols(qqs2, tl, qq);
                float2 vvr[RV], bvr[RV], dyr[RV], dyvr[RV];
                ld_rows(vs2, tl, vvr);
                ld_rows(bs2, tl, bvr);
                ld_rows(dys2, tl, dyr);
#pragma unroll
                for (int r = 0; r < RV; ++r) dyvr[r] = make_float2(0.f, 0.f);
                if (UNC) ld_rows(dyvs2, tl, dyvr);
#pragma unroll
                for (int r = 0; r < RV; ++r) {
                    const float2 vv = vvr[r];
                    const float2 bv = bvr[r];
                    const float2 dy = dyr[r];
                    const float2 dyv = dyvr[r];
                    float2 dva = make_float2(0.f, 0.f), dba = dva;
#pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        const float2 Mt = P[j + 1].M[r][q], It = P[j + 1].I[r][q];
                        const float2 rr = rcp2(It);
                        const float2 mu = fmul2(Mt, rr);
                        const float2 hh = fmul2(fmul2(dy, qp[q]), rr);
                        GM[r][q] = ffma2(fn, GM[r][q], hh);
                        float2 hm = fmul2(hh, mu);
                        if (UNC) hm = ffma2(fmul2(dyv, qq[q]), fmul2(rr, rr), hm);
                        nGI[r][q] = ffma2(fn, nGI[r][q], hm);
                        if (!CO) {
                            dqs[q] = ffma2(dy, mu, dqs[q]);
                            if (UNC) Uk[q] = ffma2(dyv, rr, Uk[q]);
                            Ak[q] = ffma2(GM[r][q], vv, Ak[q]);
                            Bk[q] = ffma2(nGI[r][q], bv, Bk[q]);
                            dva = ffma2(GM[r][q], kp[q], dva);
                            dba = ffma2(nGI[r][q], kk[q], dba);
                            Sa[r] = ffma2(GM[r][q], P[j].M[r][q], Sa[r]);
                            Sb[r] = ffma2(nGI[r][q], P[j].I[r][q], Sb[r]);
                            Sc[r] = fadd2(Sc[r], nGI[r][q]);
                        }
                    }
                    red1[(j * RV + r) * 2 + 0] = dva.x + dva.y;
                    red1[(j * RV + r) * 2 + 1] = -(dba.x + dba.y);
                }
                // this row group's share of dq and dk for the token -> shared memory
                if (SPLIT_B && j == GR - 1) {  // first write of the group: the previous group's readers must be done
                    if (!wait_fail && !tc::mbar_wait(&gbar[1], ph_b)) wait_fail = 6;  // after one failure: no more waiting
                    ph_b ^= 1;
                }
                if (!CO) {
                    float2* dst = kred2 + (gi & (KBUF - 1)) * (GR * WV * 2 * KP2) + ((j * WV + wv) * 2) * KP2 + NP * kg;
                    const float2 sc2 = dup2(p.scale), m2 = dup2(-2.f);
#pragma unroll
                    for (int q = 0; q < NP; ++q) {
                        float2 dqv = fmul2(sc2, dqs[q]);
                        if (UNC) dqv = ffma2(fmul2(dup2(2.f), qp[q]), Uk[q], dqv);
                        dst[q] = dqv;
                        dst[KP2 + q] = ffma2(fmul2(m2, kp[q]), Bk[q], Ak[q]);
                    }
                }
                float2 sa = Sa[0], sb = Sb[0], scv = Sc[0];
#pragma unroll
                for (int r = 1; r < RV; ++r) {
                    sa = fadd2(sa, Sa[r]);
                    sb = fadd2(sb, Sb[r]);
                    scv = fadd2(scv, Sc[r]);
                }
                const float sc_ = scv.x + scv.y;
                red2[j * 2 + 0] = (sa.x + sa.y) - (sb.x + sb.y) + iph * sc_;
                red2[j * 2 + 1] = -sc_;
            }
            if (CO) continue;  // carry-only pass: nothing but the state gradients is wanted
            __syncwarp();
            if (lane == 0) mbar_arrive(&gbar[0]);  // this warp's partials of the group are written
            // d_v-indexed sums over the KG lanes of a row; per-token scalars over the whole warp
            xreduce<NR1, KG>(red1, lane);
            {
                constexpr int REM = NR1 >= KG ? NR1 / KG : 1;
                const int base = xreduce_index<NR1, KG>(lane);
                const bool owner = NR1 >= KG ? true : (kg & (KG / (NR1 < KG ? NR1 : KG) - 1)) == 0;
                if (owner) {
#pragma unroll
                    for (int i = 0; i < REM; ++i) {
                        const int id = base + i;
                        const int j = id / (RV * 2), r = (id / 2) % RV, which = id & 1;
                        (which ? dbs : dvs)[(gi * GR + j) * TV + row0 + r] = red1[i];
                    }
                }
            }
            xreduce<NR2, 32>(red2, lane);
            if ((lane & (32 / NR2 - 1)) == 0) {
                const int id = xreduce_index<NR2, 32>(lane);
                wred[(w * TB + gi * GR + (id >> 1)) * 2 + (id & 1)] = red2[0];
            }
            if (!wait_fail && !tc::mbar_wait(&gbar[0], ph_a)) wait_fail = 5;
            ph_a ^= 1;
            // ---- sum the row groups' shares; emit this row tile's dq / dk partials ----------------------
            const int ng = min(GR, nt - gi * GR);  // tokens of the group that exist (<= 0 past the sequence end)
            for (int i = tid; i < ng * KP2; i += NTHR) {
                const int j = i / KP2, pi = i - j * KP2;
                const float2* src = kred2 + (gi & (KBUF - 1)) * (GR * WV * 2 * KP2) + (j * WV * 2) * KP2 + pi;
                float2 s0 = make_float2(0.f, 0.f), s1 = s0;
#pragma unroll
                for (int x = 0; x < WV; ++x) {
                    s0 = fadd2(s0, src[(x * 2) * KP2]);
                    s1 = fadd2(s1, src[(x * 2 + 1) * KP2]);
                }
                const size_t e = (((size_t)tile * a.rows_total + (size_t)(tok0 + gi * GR + j) * p.H + h) * KP2) + pi;
                reinterpret_cast<float2*>(a.dq_part)[e] = s0;
                reinterpret_cast<float2*>(a.dk_part)[e] = s1;
            }
            // with two buffers no second barrier is needed: the next group writes the other buffer, and the
            // barrier after ITS reverse walk orders this group's reads before the buffer is reused
            if (SPLIT_B) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&gbar[1]);  // this warp has read the buffer
            }
        }
        if (!CO) __syncthreads();  // dvs / dbs / wred of the whole block are complete

        // ---- block epilogue: dv, db rows and the per-token scalars -----------------------------------
        if (CO) continue;
        for (int i = tid; i < nt * TV; i += NTHR) {
            const int t = i / TV, r = i - t * TV;
            if (r < tvw) {
                const long long e = ((tok0 + t) * p.H + h) * (long long)V + v0 + r;
                st1(a.dv, e, dvs[i], p.io_dtype);
                st1(a.db, e, dbs[i], p.io_dtype);
            }
        }
        if (tid < nt) {
            float df = 0.f, s2 = 0.f;
#pragma unroll
            for (int x = 0; x < W; ++x) {
                df += wred[(x * TB + tid) * 2 + 0];
                s2 += wred[(x * TB + tid) * 2 + 1];
            }
            const float f = fc2[tid].x;
            float dip = (1.f - f) * s2;
            if (t0 + tid == 0 && !has_init) dip += f * s2;  // I_0 = Ip: the start-state gradient reaches Ip
            const size_t e = (size_t)tile * a.rows_total + (size_t)(tok0 + tid) * p.H + h;
            a.df_part[e] = df;
            a.dip_part[e] = dip;
        }
        // the next iteration's first barrier orders these reads before the buffers are reused
    }

    if (SPLIT_A && wait_fail) {
        // a barrier wait ran out: record it and mark this CTA's results as invalid (NaN in the decay-gradient
        // partial of its first token, which the finishing kernels carry into dgt and dg)
        atomicCAS(&g_bwd_status, 0, wait_fail);
        if (tid == 0)
            a.df_part[(size_t)tile * a.rows_total + (size_t)((long long)bos + s0) * p.H + h] = __int_as_float(0x7fc00000);
    }

    // ---- gradient w.r.t. the segment's start state: decay the first token's totals once more ----------
    if (a.rloc_M) {
        const float f0 = fc2[0].x;  // f of the segment's first token (operands of the last processed block)
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            if (row0 + r < tvw) {
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    const long long e = (seg_base + v0 + row0 + r) * KP + RK * kg + 2 * q;
                    *reinterpret_cast<float2*>(a.rloc_M + e) = make_float2(f0 * GM[r][q].x, f0 * GM[r][q].y);
                    *reinterpret_cast<float2*>(a.rloc_I + e) = make_float2(-f0 * nGI[r][q].x, -f0 * nGI[r][q].y);
                }
            }
        }
    }
}

// ---- finishing kernel 1: one warp per (token, head) row ------------------------------------------------
__device__ __forceinline__ void st2(void* base, long long idx, float2 x, int dt) {  // idx even, base 8-byte aligned
    if (dt == PALIMPSA_F32)
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(base) + idx) = x;
    else if (dt == PALIMPSA_BF16)
        *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(base) + idx) = __floats2bfloat162_rn(x.x, x.y);
    else
        *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(base) + idx) = __floats2half2_rn(x.x, x.y);
}

__global__ void __launch_bounds__(256) bwd_finish_rows(const palimpsa_problem p, const float* __restrict__ dq_part,
                                                       const float* __restrict__ dk_part,
                                                       const float* __restrict__ df_part,
                                                       const float* __restrict__ dip_part, void* dq, void* dk,
                                                       float* dgt, float* w_dg, float* w_dip, int tiles, int tiles_k,
                                                       int KP, long long rows, int pairs_ok) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int h = (int)(row % p.H);
    // per-token scalars: lane t fetches tile t's partial (tiles beyond 32 go round), summed by a fixed butterfly
    float df = 0.f, dip = 0.f;
    for (int t = lane; t < tiles_k; t += 32) {
        df += df_part[(size_t)t * rows + row];
        dip += dip_part[(size_t)t * rows + row];
    }
    const float gtv = p.gt[row], gh = p.g[h];
    // a lane owns four consecutive columns: one 16-byte load per tile partial, all tiles' loads independent
    const int KP4 = KP / 4;
    for (int c4 = lane; c4 < KP4; c4 += 32) {
        float4 sq = make_float4(0.f, 0.f, 0.f, 0.f), sk = sq;
        const float4* pq = reinterpret_cast<const float4*>(dq_part) + (size_t)row * KP4 + c4;
        const float4* pk = reinterpret_cast<const float4*>(dk_part) + (size_t)row * KP4 + c4;
        const size_t step = (size_t)rows * KP4;
#pragma unroll 6
        for (int t = 0; t < tiles; ++t) {
            const float4 x = pq[t * step], y = pk[t * step];
            sq.x += x.x, sq.y += x.y, sq.z += x.z, sq.w += x.w;
            sk.x += y.x, sk.y += y.y, sk.z += y.z, sk.w += y.w;
        }
        if (tiles_k > tiles) {  // dk has one slot more than dq: the carried-gradient terms
            const float4 y = pk[tiles * step];
            sk.x += y.x, sk.y += y.y, sk.z += y.z, sk.w += y.w;
        }
        const int kc = 4 * c4;
        if (pairs_ok) {          // K even, dq/dk 8-byte aligned: paired stores
            if (kc < p.K) {
                st2(dq, row * p.K + kc, make_float2(sq.x, sq.y), p.io_dtype);
                st2(dk, row * p.K + kc, make_float2(sk.x, sk.y), p.io_dtype);
            }
            if (kc + 2 < p.K) {
                st2(dq, row * p.K + kc + 2, make_float2(sq.z, sq.w), p.io_dtype);
                st2(dk, row * p.K + kc + 2, make_float2(sk.z, sk.w), p.io_dtype);
            }
        } else {
            const float q4[4] = {sq.x, sq.y, sq.z, sq.w}, k4[4] = {sk.x, sk.y, sk.z, sk.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (kc + i < p.K) {
                    st1(dq, row * p.K + kc + i, q4[i], p.io_dtype);
                    st1(dk, row * p.K + kc + i, k4[i], p.io_dtype);
                }
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        df += __shfl_xor_sync(0xffffffffu, df, off);
        dip += __shfl_xor_sync(0xffffffffu, dip, off);
    }
    if (lane == 0) {
        const float f = expf(-gtv * gh);
        dgt[row] = -gh * f * df;
        w_dg[row] = -gtv * f * df;
        w_dip[row] = dip;
    }
}

// ---- finishing kernel 2: one CTA per head, ordered sum over all rows -----------------------------------
__global__ void __launch_bounds__(256) bwd_finish_heads(const float* __restrict__ w_dg, const float* __restrict__ w_dip,
                                                       float* dg, float* dIp, long long tokens, int H) {
    __shared__ float s0[256], s1[256];
    const int h = blockIdx.x, tid = threadIdx.x;
    float a0 = 0.f, a1 = 0.f;
    for (long long t = tid; t < tokens; t += 256) {
        a0 += w_dg[t * H + h];
        a1 += w_dip[t * H + h];
    }
    s0[tid] = a0;
    s1[tid] = a1;
    __syncthreads();
    for (int s = 128; s >= 1; s >>= 1) {
        if (tid < s) {
            s0[tid] += s0[tid + s];
            s1[tid] += s1[tid + s];
        }
        __syncthreads();
    }
    if (tid == 0) {
        dg[h] = s0[0];
        dIp[h] = s1[0];
    }
}

// -------------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------------
struct BwdShape {
    int RK, KG, RV;
};
static BwdShape bwd_shape(int KP) {
    switch (KP) {
        case 16: return {2, 8, 2};
        case 32: return {4, 8, 2};
        case 48: return {6, 8, 2};
        case 64: return {4, 16, 2};
        case 96: return {6, 16, 2};
        case 128: return {4, 32, 2};
        case 192: return {6, 32, 2};
        case 256: return {8, 32, 1};
        default: return {0, 0, 0};
    }
}
// Warps per CTA: 8 when d_v is long enough to use them and the shared-memory layout fits, else 4.
struct BwdConfig {
    BwdShape s;
    int W, TV, smem, kbuf;
};
static BwdConfig bwd_config(const palimpsa_problem& p) {
    BwdConfig c{};
    c.s = bwd_shape(palimpsa_padded_k(p.K));
    if (!c.s.RK) return c;
    const int VG = 32 / c.s.KG, rpw = VG * c.s.RV, KP = c.s.RK * c.s.KG;
    const bool unc = (p.flags & PALIMPSA_FLAG_UNCERTAINTY) != 0;
    const int es = dtype_size(p.io_dtype);
    int W = (rpw == 1 || p.V > 4 * rpw) ? 8 : 4;
    // d_k = 128: 11 or 12 warps (22 / 24 rows) per CTA hide latency better than 8; of the two, the one that
    // pads d_v with fewer idle rows (d_v = 128: 6 tiles of 22 rows = 132 instead of 144)
    if (KP == 128 && rpw == 2 && p.V >= 48) {
        const int pad11 = (p.V + 21) / 22 * 22, pad12 = (p.V + 23) / 24 * 24;
        W = pad11 < pad12 ? 11 : 12;
    }
    // d_k = 48 (8 rows per warp): 6 warps = 48 rows where that pads d_v with fewer idle rows than 64 (d_v = 48, 96, 144)
    if (KP == 48 && rpw == 8 && W == 8 && (p.V + 47) / 48 * 48 < (p.V + 63) / 64 * 64) W = 6;
    for (;;) {
        c.W = W;
        c.TV = W * rpw;
        c.kbuf = 2;
        c.smem = bwd_smem_layout(KP, c.TV, c.s.RV * c.s.RK, 32 * W, W * VG, es, unc, 2).total;
        if (c.smem > 227 * 1024) {
            c.kbuf = 1;
            c.smem = bwd_smem_layout(KP, c.TV, c.s.RV * c.s.RK, 32 * W, W * VG, es, unc, 1).total;
        }
        if (c.smem <= 227 * 1024 || W == 4 || rpw == 1 || W >= 11) break;  // 6 and 8 fall back to 4
        W = 4;
    }
    return c;
}

int bwd_tile_rows(const palimpsa_problem& p) {
    const BwdConfig c = bwd_config(p);
    return (c.s.RK && c.smem <= 227 * 1024) ? c.TV : 0;
}

BwdWorkspace bwd_workspace_layout(const palimpsa_problem& p) {
    BwdWorkspace ws{};
    ws.KP = palimpsa_padded_k(p.K);
    const int TV = bwd_tile_rows(p);
    if (!TV) return ws;
    ws.tiles = (p.V + TV - 1) / TV;
    const size_t rows = (size_t)p.total_tokens * p.H;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += (bytes + 255) / 256 * 256;
        return o;
    };
    ws.dq_part = take((size_t)ws.tiles * rows * ws.KP * 4);
    // one slot more than there are row tiles: the carried-gradient terms of a segmented backward go there
    ws.dk_part = take((size_t)(ws.tiles + 1) * rows * ws.KP * 4);
    ws.df_part = take((size_t)(ws.tiles + 1) * rows * 4);
    ws.dip_part = take((size_t)(ws.tiles + 1) * rows * 4);
    ws.w_dg = take(rows * 4);
    ws.w_dip = take(rows * 4);
    ws.total = off;
    return ws;
}

template <int RK, int KG, int RV, int W>
static int launch_bwd_w(const BwdArgs& a, int tiles, int num_seg, bool carry_only, cudaStream_t stream) {
    constexpr int VG = 32 / KG, TV = W * VG * RV;
    const palimpsa_problem& p = a.p;
    const bool unc = (p.flags & PALIMPSA_FLAG_UNCERTAINTY) != 0;
    const BwdSmem L = bwd_smem_layout(RK * KG, TV, RV * RK, 32 * W, W * VG, dtype_size(p.io_dtype), unc, a.kbuf);
    if (L.total > 227 * 1024) return PALIMPSA_E_DIM;
    dim3 grid(tiles, p.num_seqs * p.H, num_seg);
    dim3 block(32 * W, 1, 1);
#define PALIMPSA_BWD_LAUNCH(U, C)                                                                                 \
    do {                                                                                                          \
        if (cudaFuncSetAttribute(bwd_kernel<RK, KG, RV, W, U, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 L.total) != cudaSuccess)                                                         \
            return PALIMPSA_E_LAUNCH;                                                                             \
        bwd_kernel<RK, KG, RV, W, U, C><<<grid, block, L.total, stream>>>(a);                                     \
    } while (0)
    if (carry_only) {
        if (unc) PALIMPSA_BWD_LAUNCH(true, true); else PALIMPSA_BWD_LAUNCH(false, true);
    } else {
        if (unc) PALIMPSA_BWD_LAUNCH(true, false); else PALIMPSA_BWD_LAUNCH(false, false);
    }
#undef PALIMPSA_BWD_LAUNCH
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

template <int RK, int KG, int RV>
static int launch_bwd_t(const BwdArgs& args, int tiles, int num_seg, bool carry_only, cudaStream_t stream) {
    const BwdConfig cfg = bwd_config(args.p);
    BwdArgs a = args;
    a.kbuf = cfg.kbuf;
    if (cfg.W == 8) return launch_bwd_w<RK, KG, RV, 8>(a, tiles, num_seg, carry_only, stream);
    if constexpr (RK == 6 && KG == 8 && RV == 2)
        if (cfg.W == 6) return launch_bwd_w<RK, KG, RV, 6>(a, tiles, num_seg, carry_only, stream);
    if constexpr (RK == 4 && KG == 32 && RV == 2) {
        if (cfg.W == 12) return launch_bwd_w<RK, KG, RV, 12>(a, tiles, num_seg, carry_only, stream);
        if (cfg.W == 11) return launch_bwd_w<RK, KG, RV, 11>(a, tiles, num_seg, carry_only, stream);
    }
    if constexpr (RV > 1) return launch_bwd_w<RK, KG, RV, 4>(a, tiles, num_seg, carry_only, stream);
    return PALIMPSA_E_DIM;
}

int bwd_wait_status() {
    int s = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&s, g_bwd_status, sizeof(int)) != cudaSuccess) return -1;
    if (s) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_bwd_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return s;
}

static bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

int launch_bwd(const palimpsa_bwd_params* prm, const palimpsa_segments* segs, bool carry_only, cudaStream_t stream,
               int stages) {
    const palimpsa_problem& p = prm->p;
    const BwdWorkspace ws = bwd_workspace_layout(p);
    if (!ws.tiles) return PALIMPSA_E_DIM;
    char* base = reinterpret_cast<char*>(prm->workspace);
    BwdArgs a{};
    a.p = p;
    int num_seg = 1;
    if (segs) {
        num_seg = segs->num_segments;
        a.seg_len = segs->seg_len;
        a.carry_M = carry_only ? nullptr : segs->carry_M;
        a.carry_I = carry_only ? nullptr : segs->carry_I;
        a.rloc_M = segs->rloc_M;
        a.rloc_I = segs->rloc_I;
    }
    if (carry_only) stages = 1;
    a.d_o = prm->d_o;
    a.d_o_var = (p.flags & PALIMPSA_FLAG_UNCERTAINTY) ? prm->d_o_var : nullptr;
    a.ckpt_M = prm->ckpt_M;
    a.ckpt_I = prm->ckpt_I;
    a.dq_part = reinterpret_cast<float*>(base + ws.dq_part);
    a.dk_part = reinterpret_cast<float*>(base + ws.dk_part);
    a.df_part = reinterpret_cast<float*>(base + ws.df_part);
    a.dip_part = reinterpret_cast<float*>(base + ws.dip_part);
    a.dv = prm->dv;
    a.db = prm->db;
    a.rows_total = p.total_tokens * p.H;
    const int es = dtype_size(p.io_dtype);
    a.aligned = ((p.K * es) % 16 == 0) && ((p.V * es) % 16 == 0) && aligned16(p.q) && aligned16(p.k) &&
                aligned16(p.v) && aligned16(p.b) && aligned16(prm->d_o) &&
                (a.d_o_var == nullptr || aligned16(a.d_o_var)) && ((reinterpret_cast<uintptr_t>(p.gt) & 3) == 0);
    int rc = PALIMPSA_OK;
    if (stages & 1) switch (ws.KP) {
        case 16: rc = launch_bwd_t<2, 8, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 32: rc = launch_bwd_t<4, 8, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 48: rc = launch_bwd_t<6, 8, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 64: rc = launch_bwd_t<4, 16, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 96: rc = launch_bwd_t<6, 16, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 128: rc = launch_bwd_t<4, 32, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 192: rc = launch_bwd_t<6, 32, 2>(a, ws.tiles, num_seg, carry_only, stream); break;
        case 256: rc = launch_bwd_t<8, 32, 1>(a, ws.tiles, num_seg, carry_only, stream); break;
        default: return PALIMPSA_E_DIM;
    }
    if (rc != PALIMPSA_OK) return rc;
    if (!(stages & 2)) return PALIMPSA_OK;
    const long long rows = a.rows_total;
    if (rows > 0) {
        const int wpb = 8;
        bwd_finish_rows<<<(unsigned)((rows + wpb - 1) / wpb), 32 * wpb, 0, stream>>>(
            p, a.dq_part, a.dk_part, a.df_part, a.dip_part, prm->dq, prm->dk, prm->dgt,
            reinterpret_cast<float*>(base + ws.w_dg), reinterpret_cast<float*>(base + ws.w_dip), ws.tiles,
            ws.tiles + ((stages & 4) ? 1 : 0), ws.KP, rows,
            (p.K % 2 == 0 && ((reinterpret_cast<uintptr_t>(prm->dq) | reinterpret_cast<uintptr_t>(prm->dk)) & 7) == 0) ? 1 : 0);
        if (cudaGetLastError() != cudaSuccess) return PALIMPSA_E_LAUNCH;
    }
    bwd_finish_heads<<<p.H, 256, 0, stream>>>(reinterpret_cast<float*>(base + ws.w_dg),
                                              reinterpret_cast<float*>(base + ws.w_dip), prm->dg, prm->dIp,
                                              p.total_tokens, p.H);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

// ---- backward with library-owned scratch -----------------------------------------------------------
// For callers that cannot allocate device memory themselves: the partial-sum scratch of the backward
// lives in this fixed array instead of a caller-provided workspace.  Every device on which the library's
// backward code gets loaded (primary context) carries the array from then until the process exits.  Host code may not use the array's name as an address; the
// device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_static_scratch[PALIMPSA_STATIC_SCRATCH_BYTES];

int launch_bwd_static(const palimpsa_bwd_params* prm, cudaStream_t stream) {
    constexpr int MAX_DEV = 64;
    static void* addr[MAX_DEV] = {};
    static std::mutex mu;
    const BwdWorkspace ws = bwd_workspace_layout(prm->p);
    if (!ws.tiles) return PALIMPSA_E_DIM;
    if (ws.total > (size_t)PALIMPSA_STATIC_SCRATCH_BYTES) return PALIMPSA_E_LIMIT;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return PALIMPSA_E_LAUNCH;
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!addr[dev]) {
            void* sym = nullptr;
            // may be the call that loads this module on the device (lazy loading): the array is reserved now,
            // and a device without 64 MiB to spare fails here
            if (cudaGetSymbolAddress(&sym, g_static_scratch) != cudaSuccess || !sym) {
                (void)cudaGetLastError();
                return PALIMPSA_E_SYMBOL;
            }
            addr[dev] = sym;
        }
        ptr = addr[dev];
    }
    palimpsa_bwd_params local = *prm;
    local.workspace = ptr;
    local.workspace_bytes = PALIMPSA_STATIC_SCRATCH_BYTES;
    return launch_bwd(&local, nullptr, false, stream, 3);
}

}  // namespace palimpsa
