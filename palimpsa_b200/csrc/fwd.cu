// Forward kernel of the Palimpsa operator (sm_100a).
//
// One CTA owns a tile of TV state rows (d_v) x all KP state columns (padded d_k) of one
// (sequence, head[, segment]) and walks its tokens in order with the (M, I) state pair held in
// registers for the whole walk.  Work per state element and token: 6 packed-FP32 lane ops and one
// MUFU reciprocal -- the kernel is bound by the MUFU pipe, not by HBM.
//
//   thread layout   lane = vg*KG + kg.  A thread owns RV rows x RK columns; the KG lanes of a row
//                   group own interleaved float4 column groups (column = 4*(j*KG+kg)+i), so that
//                   shared-memory operand reads and global state accesses of a warp are contiguous.
//                   Tile shapes are template parameters: every index in the hot loop is a constant.
//   staging         blocks of 16 tokens: cp.async (16 B) into a raw double buffer one block ahead,
//                   then one cooperative pass converts to fp32 operands (q*scale, k; v, b as
//                   duplicated pairs; {f, f, c, c} with f = exp(-gt*g), c = (1-f)*Ip) shared by every
//                   thread of the CTA.  k*k is formed in registers.
//   reduction       o[v] = sum_k: in-thread over RK, then one transposed butterfly per 4 tokens over
//                   the KG lanes of the row group.
//   checkpoints     optional (M, I) store at the start of every 16-token block (for backward).
//   segments        gridDim.z segments per sequence, each started from a given (M, I); the SUM
//                   variant computes only the zero-start end state and decay of every segment.
//
// It serves the chunked op and the fused-recurrent op: what the reference does with
// chunk_palimpsa_fwd_kernel (chunk_palimpsa_forgetting_scalar.py:66-218) and
// fused_palimpsa_recurrent_fwd_kernel (fused_recurrent_palimpsa.py:24-154).
#include "common.cuh"
#include "host.h"

namespace palimpsa {

struct FwdArgs {
    palimpsa_problem p;
    void* o;
    void* o_var;
    float* final_mu;
    float* final_I;
    float* ckpt_M;
    float* ckpt_I;
    int aligned;  // 1: every io row is 16-byte aligned and a multiple of 16 bytes
    // segments (gridDim.z of them per sequence; seg_len tokens each, a multiple of 16)
    int seg_len;
    const float* start_M;  // [N,G,H,V,KP] (M, I) at the start of every segment, or NULL
    const float* start_I;
    float* sum_M;          // summary mode: [N,G,H,V,KP] end state of the segment started from zero, (M, J) form
    float* sum_J;
    float* decay;          // summary mode: [N,G,H] product of f over the segment
};

struct FwdSmem {
    int qs, ks, qqs, vs, bs, fc, ys, yvs;  // fp32 operand / result buffers (byte offsets)
    int raw;                                    // two raw stages follow each other from here
    int rq, rk, rv, rb, rgt, raw_stage;         // offsets inside a stage, stage size
    int total;
};

__host__ __device__ inline FwdSmem fwd_smem_layout(int KP, int TV, int es, bool unc) {
    FwdSmem s;
    int off = 0;
    auto take = [&](int bytes) {
        int o = off;
        off += round_up(bytes, 16);
        return o;
    };
    s.qs = take(TB * KP * 4);
    s.ks = take(TB * KP * 4);
    s.qqs = unc ? take(TB * KP * 4) : 0;
    s.vs = take(TB * TV * 8);   // every value stored twice: {v, v}
    s.bs = take(TB * TV * 8);
    s.fc = take(TB * 16);       // {f, f, c, c}
    s.ys = take(TB * TV * 4);
    s.yvs = unc ? take(TB * TV * 4) : 0;
    s.raw = off;
    int r = 0;
    auto rtake = [&](int bytes) {
        int o = r;
        r += round_up(bytes, 16);
        return o;
    };
    s.rq = rtake(TB * KP * es);
    s.rk = rtake(TB * KP * es);
    s.rv = rtake(TB * TV * es);
    s.rb = rtake(TB * TV * es);
    s.rgt = rtake(TB * 4);
    s.raw_stage = r;
    s.total = off + 2 * r;
    return s;
}

// Issue the asynchronous copies of one block of nt tokens (aligned fast path only).
__device__ __forceinline__ void fwd_issue(const FwdArgs& a, unsigned char* stage, const FwdSmem& L, int es, int KP,
                                          int TV, long long tok0, int nt, int h, int v0, int tvw, const ChunkSplit& sq,
                                          const ChunkSplit& sv) {
    const palimpsa_problem& p = a.p;
    const int nthr = blockDim.x, tid = threadIdx.x;
    const int cq = p.K * es / 16;
    const char* gq = reinterpret_cast<const char*>(p.q);
    const char* gk = reinterpret_cast<const char*>(p.k);
    if (sq.step > 0) {
        for (int t = sq.t0; t < nt; t += sq.step) {
            long long src = ((tok0 + t) * p.H + h) * (long long)p.K * es + sq.c * 16;
            int dst = t * KP * es + sq.c * 16;
            cp_async16(stage + L.rq + dst, gq + src);
            cp_async16(stage + L.rk + dst, gk + src);
        }
    } else {
        for (int i = tid; i < nt * cq; i += nthr) {
            int t = i / cq, c = i - t * cq;
            long long src = ((tok0 + t) * p.H + h) * (long long)p.K * es + c * 16;
            int dst = t * KP * es + c * 16;
            cp_async16(stage + L.rq + dst, gq + src);
            cp_async16(stage + L.rk + dst, gk + src);
        }
    }
    const int cv = tvw * es / 16;
    const char* gv = reinterpret_cast<const char*>(p.v);
    const char* gb = reinterpret_cast<const char*>(p.b);
    if (sv.step > 0) {
        for (int t = sv.t0; t < nt; t += sv.step) {
            long long src = (((tok0 + t) * p.H + h) * (long long)p.V + v0) * es + sv.c * 16;
            int dst = t * TV * es + sv.c * 16;
            cp_async16(stage + L.rv + dst, gv + src);
            cp_async16(stage + L.rb + dst, gb + src);
        }
    } else {
        for (int i = tid; i < nt * cv; i += nthr) {
            int t = i / cv, c = i - t * cv;
            long long src = (((tok0 + t) * p.H + h) * (long long)p.V + v0) * es + c * 16;
            int dst = t * TV * es + c * 16;
            cp_async16(stage + L.rv + dst, gv + src);
            cp_async16(stage + L.rb + dst, gb + src);
        }
    }
    for (int i = tid; i < nt; i += nthr) cp_async4(stage + L.rgt + i * 4, p.gt + (tok0 + i) * p.H + h);
}

// Convert one block to fp32 operands.  ALIGNED: read the raw stage; otherwise read global memory
// element by element (any K, V, alignment).
template <int DT, bool ALIGNED, bool UNC>
__device__ __forceinline__ void fwd_convert(const FwdArgs& a, unsigned char* sm, const unsigned char* stage,
                                            const FwdSmem& L, int KP, int TV, long long tok0, int nt, int h, int v0,
                                            float gh, float iph) {
    const palimpsa_problem& p = a.p;
    const int nthr = blockDim.x, tid = threadIdx.x;
    const int K4 = KP / 4, V4 = TV / 4;
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
    float4* vs = reinterpret_cast<float4*>(sm + L.vs);
    float4* bs = reinterpret_cast<float4*>(sm + L.bs);
    for (int i = tid; i < TB * V4; i += nthr) {
        int t = i / V4, c4 = i - t * V4;
        float4 vv = make_float4(0.f, 0.f, 0.f, 0.f), bv = vv;
        if (t < nt && v0 + c4 * 4 < p.V) {
            if (ALIGNED) {
                vv = ld4<DT>(stage + L.rv, i);
                bv = ld4<DT>(stage + L.rb, i);
            } else {
                long long row = ((tok0 + t) * p.H + h) * (long long)p.V;
                vv = ld4_guarded<DT>(p.v, row + v0 + c4 * 4, row + p.V);
                bv = ld4_guarded<DT>(p.b, row + v0 + c4 * 4, row + p.V);
            }
        }
        st_dup4(vs, i, vv);
        st_dup4(bs, i, bv);
    }
    float4* fc = reinterpret_cast<float4*>(sm + L.fc);
    for (int i = tid; i < TB; i += nthr) {
        float gtv = 0.f;
        if (i < nt) gtv = ALIGNED ? reinterpret_cast<const float*>(stage + L.rgt)[i] : p.gt[(tok0 + i) * p.H + h];
        float f = expf(-gtv * gh);
        const float c = (1.f - f) * iph;
        fc[i] = make_float4(f, f, c, c);
    }
}

// The recurrence over G consecutive tokens (no bounds checks: the caller only passes full groups),
// followed by one batched reduction of the G*RV (x2 with uncertainty) output partials over the KG lanes
// of the row group.  Kept free of conditionals on purpose: the state arrays M, I are updated in place.
template <int RK, int KG, int RV, int TV, bool UNC, bool SUM, int G>
__device__ __forceinline__ void fwd_group(float2 (&M)[RV][RK / 4][2], float2 (&I)[RV][RK / 4][2], const float4* ks4,
                                          const float4* qs4, const float4* qqs4, const float2* vs2, const float2* bs2,
                                          const float4* fc, float* ys, float* yvs, int tg, int kg, int row0, int lane) {
    constexpr int KP = RK * KG, J4 = RK / 4, NRED = G * RV * (UNC ? 2 : 1);
    float red[NRED];
#pragma unroll
    for (int jt = 0; jt < G; ++jt) {
        const int t = tg + jt;
        const float4 fcv = fc[t];
        const float2 ff = make_float2(fcv.x, fcv.y), cc = make_float2(fcv.z, fcv.w);
        float2 vr[RV], br[RV], acc[RV], accv[RV];
        if constexpr (RV % 2 == 0) {  // two adjacent duplicated pairs come in as one 16-byte load (row0 and TV are even)
#pragma unroll
            for (int r = 0; r < RV; r += 2) {
                const float4 v4 = *reinterpret_cast<const float4*>(vs2 + t * TV + r);
                const float4 b4 = *reinterpret_cast<const float4*>(bs2 + t * TV + r);
                vr[r] = make_float2(v4.x, v4.y);
                vr[r + 1] = make_float2(v4.z, v4.w);
                br[r] = make_float2(b4.x, b4.y);
                br[r + 1] = make_float2(b4.z, b4.w);
            }
        } else {
#pragma unroll
            for (int r = 0; r < RV; ++r) {
                vr[r] = vs2[t * TV + r];
                br[r] = bs2[t * TV + r];
            }
        }
#pragma unroll
        for (int r = 0; r < RV; ++r) acc[r] = accv[r] = make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < J4; ++j) {
            const int idx = t * (KP / 4) + j * KG + kg;
            const float4 k4 = ks4[idx], q4 = qs4[idx];
            float4 qq4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (UNC) qq4 = qqs4[idx];
            const float2 kp[2] = {make_float2(k4.x, k4.y), make_float2(k4.z, k4.w)};
            const float2 kkp[2] = {fmul2(kp[0], kp[0]), fmul2(kp[1], kp[1])};
            const float2 qp[2] = {make_float2(q4.x, q4.y), make_float2(q4.z, q4.w)};
            const float2 qqp[2] = {make_float2(qq4.x, qq4.y), make_float2(qq4.z, qq4.w)};
#pragma unroll
            for (int r = 0; r < RV; ++r) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    M[r][j][e] = ffma2(ff, M[r][j][e], fmul2(vr[r], kp[e]));
                    if (SUM) {  // J = f*J + b k^2: no prior term, no output
                        I[r][j][e] = ffma2(ff, I[r][j][e], fmul2(br[r], kkp[e]));
                    } else {
                        I[r][j][e] = ffma2(ff, I[r][j][e], ffma2(br[r], kkp[e], cc));
                        const float2 rr = rcp2(I[r][j][e]);
                        acc[r] = ffma2(fmul2(M[r][j][e], rr), qp[e], acc[r]);
                        if (UNC) accv[r] = ffma2(rr, qqp[e], accv[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            red[(jt * RV + r) * (UNC ? 2 : 1)] = acc[r].x + acc[r].y;
            if (UNC) red[(jt * RV + r) * 2 + 1] = accv[r].x + accv[r].y;
        }
    }
    if (SUM) return;
    xreduce<NRED, KG>(red, lane);
    constexpr int REM = NRED >= KG ? NRED / KG : 1;
    const int base = xreduce_index<NRED, KG>(lane);
    const bool owner = NRED >= KG ? true : (kg & (KG / (NRED < KG ? NRED : KG) - 1)) == 0;
    if (owner) {
#pragma unroll
        for (int i = 0; i < REM; ++i) {
            const int id = base + i;
            const int which = UNC ? (id & 1) : 0;
            const int jr = UNC ? (id >> 1) : id;
            const int jt = jr / RV, r = jr % RV;
            (which ? yvs : ys)[(tg + jt) * TV + row0 + r] = red[i];
        }
    }
}

// The d_k = 128 tiling (16 state elements per thread, 16 lanes per row) reduces 8 tokens' outputs in one butterfly
// and is held to 128 registers (4 CTAs of 4 warps per SM): 1.57 -> 1.49 ms on the 170M shape.  The other tilings
// keep batches of 4 and the compiler's own register count (8 there costs them spills).
template <int RK, int KG, int RV, bool UNC>
constexpr bool fwd_small_tile = RK * RV <= 16 && KG == 16 && !UNC;

template <int RK, int KG, int RV, int W, bool UNC, bool SUM>
__global__ void __launch_bounds__(32 * W, fwd_small_tile<RK, KG, RV, UNC> ? 4 : 1) fwd_kernel(const FwdArgs a) {
    constexpr int KP = RK * KG, VG = 32 / KG, J4 = RK / 4, TV = W * VG * RV, NTHR = 32 * W;
    constexpr int GF = fwd_small_tile<RK, KG, RV, UNC> ? 8 : 4;  // tokens whose outputs are reduced together
    extern __shared__ __align__(16) unsigned char sm[];
    const palimpsa_problem& p = a.p;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int kg = lane % KG, vg = lane / KG;
    const int row0 = (w * VG + vg) * RV;
    const int ny = blockIdx.y / p.H, h = blockIdx.y - ny * p.H;
    const int n = p.seq_order ? p.seq_order[ny] : ny;  // blocks start in grid order: a packed batch lists its longest sequences first
    const int v0 = blockIdx.x * TV;
    const int tvw = min(TV, p.V - v0);
    const int es = dtype_size(p.io_dtype);
    const FwdSmem L = fwd_smem_layout(KP, TV, es, UNC);
    int bos, len;
    seq_range(p, n, bos, len);
    const float gh = p.g[h], iph = p.Ip[h];
    const int K = p.K, V = p.V;
    const bool vecK = (K % 4) == 0;
    // this CTA's segment of the sequence: tokens [s0, s1)
    const int g = blockIdx.z, G = gridDim.z;
    const int s0 = a.seg_len > 0 ? min(len, g * a.seg_len) : 0;
    const int s1 = a.seg_len > 0 ? min(len, s0 + a.seg_len) : len;
    const long long seg_base = (((long long)n * G + g) * p.H + h) * V;  // row index into [N,G,H,V,KP] buffers

    // ---- state registers ------------------------------------------------------------------
    float2 M[RV][J4][2], I[RV][J4][2];
    const long long st_base = ((long long)n * p.H + h) * V;
#pragma unroll
    for (int r = 0; r < RV; ++r) {
        const int vrow = v0 + row0 + r;
#pragma unroll
        for (int j = 0; j < J4; ++j) {
            const int kc = 4 * (j * KG + kg);
            float4 m4 = make_float4(0.f, 0.f, 0.f, 0.f);
            float4 i4 = make_float4(1.f, 1.f, 1.f, 1.f);
            if (SUM) {
                i4 = m4;  // summaries start from M = 0, J = 0
            } else if (a.start_M) {
                if (vrow < V) {
                    const long long e = (seg_base + vrow) * KP + kc;
                    m4 = *reinterpret_cast<const float4*>(a.start_M + e);
                    i4 = *reinterpret_cast<const float4*>(a.start_I + e);
                }
            } else if (vrow < V && kc < K) {
                if (p.init_mu) {
                    const long long e = (st_base + vrow) * K + kc;
                    float4 mu4;
                    if (vecK) {
                        mu4 = *reinterpret_cast<const float4*>(p.init_mu + e);
                        i4 = *reinterpret_cast<const float4*>(p.init_I + e);
                    } else {
                        const long long lim = (st_base + vrow + 1) * K;
                        mu4 = ld4_guarded<PALIMPSA_F32>(p.init_mu, e, lim);
                        i4 = ld4_guarded<PALIMPSA_F32>(p.init_I, e, lim);
                        if (kc + 1 >= K) i4.y = 1.f;
                        if (kc + 2 >= K) i4.z = 1.f;
                        if (kc + 3 >= K) i4.w = 1.f;
                    }
                    m4 = make_float4(mu4.x * i4.x, mu4.y * i4.y, mu4.z * i4.z, mu4.w * i4.w);
                } else {
                    i4 = make_float4(iph, iph, iph, iph);
                }
            }
            M[r][j][0] = make_float2(m4.x, m4.y);
            M[r][j][1] = make_float2(m4.z, m4.w);
            I[r][j][0] = make_float2(i4.x, i4.y);
            I[r][j][1] = make_float2(i4.z, i4.w);
        }
    }

    const int blk0 = s0 / TB, nblk = s1 > s0 ? (s1 + TB - 1) / TB : blk0;  // blocks [blk0, nblk) of the sequence
    const long long slot0 = seq_first_slot(p, n);
    float Pdecay = 1.f;
    const float4* qs4 = reinterpret_cast<const float4*>(sm + L.qs);
    const float4* ks4 = reinterpret_cast<const float4*>(sm + L.ks);
    const float4* qqs4 = reinterpret_cast<const float4*>(sm + L.qqs);
    const float2* vs2 = reinterpret_cast<const float2*>(sm + L.vs) + row0;
    const float2* bs2 = reinterpret_cast<const float2*>(sm + L.bs) + row0;
    const float4* fc = reinterpret_cast<const float4*>(sm + L.fc);
    float* ys = reinterpret_cast<float*>(sm + L.ys);
    float* yvs = reinterpret_cast<float*>(sm + L.yvs);
    unsigned char* raw = sm + L.raw;

    const ChunkSplit sq = chunk_split(K * es / 16, NTHR, tid), sv = chunk_split(tvw * es / 16, NTHR, tid);
    if (a.aligned && nblk > blk0) {
        fwd_issue(a, raw + (blk0 & 1) * L.raw_stage, L, es, KP, TV, (long long)bos + blk0 * TB, min(TB, s1 - blk0 * TB),
                  h, v0, tvw, sq, sv);
        cp_async_commit();
    }

    for (int blk = blk0; blk < nblk; ++blk) {
        const int t0 = blk * TB;
        const int nt = min(TB, s1 - t0);
        const long long tok0 = (long long)bos + t0;
        unsigned char* stage = raw + (blk & 1) * L.raw_stage;
        if (a.aligned) {
            if (blk + 1 < nblk) {
                fwd_issue(a, raw + ((blk + 1) & 1) * L.raw_stage, L, es, KP, TV, tok0 + TB, min(TB, s1 - t0 - TB), h,
                          v0, tvw, sq, sv);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
        }
        __syncthreads();
        if (a.aligned) {
            if (p.io_dtype == PALIMPSA_BF16)
                fwd_convert<PALIMPSA_BF16, true, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
            else if (p.io_dtype == PALIMPSA_F32)
                fwd_convert<PALIMPSA_F32, true, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
            else
                fwd_convert<PALIMPSA_F16, true, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
        } else {
            if (p.io_dtype == PALIMPSA_BF16)
                fwd_convert<PALIMPSA_BF16, false, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
            else if (p.io_dtype == PALIMPSA_F32)
                fwd_convert<PALIMPSA_F32, false, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
            else
                fwd_convert<PALIMPSA_F16, false, UNC>(a, sm, stage, L, KP, TV, tok0, nt, h, v0, gh, iph);
        }
        __syncthreads();

        if (SUM && tid == 0)
            for (int t = 0; t < nt; ++t) Pdecay *= fc[t].x;
        // ---- checkpoint: state before the first token of this block ---------------------------
        if (!SUM && a.ckpt_M) {
            const long long cbase = ((slot0 + blk) * p.H + h) * V;
#pragma unroll
            for (int r = 0; r < RV; ++r) {
                const int vrow = v0 + row0 + r;
                if (vrow < V) {
#pragma unroll
                    for (int j = 0; j < J4; ++j) {
                        const long long e = (cbase + vrow) * KP + 4 * (j * KG + kg);
                        *reinterpret_cast<float4*>(a.ckpt_M + e) =
                            make_float4(M[r][j][0].x, M[r][j][0].y, M[r][j][1].x, M[r][j][1].y);
                        *reinterpret_cast<float4*>(a.ckpt_I + e) =
                            make_float4(I[r][j][0].x, I[r][j][0].y, I[r][j][1].x, I[r][j][1].y);
                    }
                }
            }
        }

        // ---- the recurrence: full groups of GF tokens, then the remaining tokens one by one --------
        int tg = 0;
#pragma unroll 1
        for (; tg + GF <= nt; tg += GF)
            fwd_group<RK, KG, RV, TV, UNC, SUM, GF>(M, I, ks4, qs4, qqs4, vs2, bs2, fc, ys, yvs, tg, kg, row0, lane);
#pragma unroll 1
        for (; tg < nt; ++tg)
            fwd_group<RK, KG, RV, TV, UNC, SUM, 1>(M, I, ks4, qs4, qqs4, vs2, bs2, fc, ys, yvs, tg, kg, row0, lane);
        __syncthreads();

        // ---- write the block's outputs -----------------------------------------------------------
        if (!SUM)
        for (int i = tid; i < nt * TV; i += NTHR) {
            const int t = i / TV, r = i - t * TV;
            if (r < tvw) {
                const long long e = ((tok0 + t) * p.H + h) * (long long)V + v0 + r;
                st1(a.o, e, ys[i], p.io_dtype);
                if (UNC) st1(a.o_var, e, yvs[i], p.io_dtype);
            }
        }
    }

    if (SUM) {  // segment summary: end state from a zero start, and the segment's total decay
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            const int vrow = v0 + row0 + r;
            if (vrow < V) {
#pragma unroll
                for (int j = 0; j < J4; ++j) {
                    const long long e = (seg_base + vrow) * KP + 4 * (j * KG + kg);
                    *reinterpret_cast<float4*>(a.sum_M + e) =
                        make_float4(M[r][j][0].x, M[r][j][0].y, M[r][j][1].x, M[r][j][1].y);
                    *reinterpret_cast<float4*>(a.sum_J + e) =
                        make_float4(I[r][j][0].x, I[r][j][0].y, I[r][j][1].x, I[r][j][1].y);
                }
            }
        }
        if (tid == 0 && blockIdx.x == 0) a.decay[((long long)n * G + g) * p.H + h] = Pdecay;
        return;
    }
    // ---- final state in the API's (mu, I) form: written by the segment that holds the last token -----
    if (a.final_mu && s1 == len && (s0 < len || g == 0)) {
#pragma unroll
        for (int r = 0; r < RV; ++r) {
            const int vrow = v0 + row0 + r;
#pragma unroll
            for (int j = 0; j < J4; ++j) {
                const int kc = 4 * (j * KG + kg);
                if (vrow < V && kc < K) {
                    const float4 i4 = make_float4(I[r][j][0].x, I[r][j][0].y, I[r][j][1].x, I[r][j][1].y);
                    const float4 mu4 = make_float4(M[r][j][0].x / i4.x, M[r][j][0].y / i4.y, M[r][j][1].x / i4.z,
                                                   M[r][j][1].y / i4.w);
                    const long long e = (st_base + vrow) * K + kc;
                    if (vecK) {
                        *reinterpret_cast<float4*>(a.final_mu + e) = mu4;
                        *reinterpret_cast<float4*>(a.final_I + e) = i4;
                    } else {
                        const float mus[4] = {mu4.x, mu4.y, mu4.z, mu4.w};
                        const float is[4] = {i4.x, i4.y, i4.z, i4.w};
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (kc + c < K) {
                                a.final_mu[e + c] = mus[c];
                                a.final_I[e + c] = is[c];
                            }
                    }
                }
            }
        }
    }
}

// -------------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------------
template <int RK, int KG, int RV, int W>
static int launch_fwd_w(const FwdArgs& a, int num_seg, bool summary, cudaStream_t stream) {
    constexpr int VG = 32 / KG, TV = W * VG * RV;
    const palimpsa_problem& p = a.p;
    const bool unc = !summary && (p.flags & PALIMPSA_FLAG_UNCERTAINTY) != 0;
    const FwdSmem L = fwd_smem_layout(RK * KG, TV, dtype_size(p.io_dtype), unc);
    dim3 grid((p.V + TV - 1) / TV, p.num_seqs * p.H, num_seg);
    dim3 block(32 * W, 1, 1);
    cudaError_t e;
    if (summary) {
        e = cudaFuncSetAttribute(fwd_kernel<RK, KG, RV, W, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 L.total);
        if (e != cudaSuccess) return PALIMPSA_E_LAUNCH;
        fwd_kernel<RK, KG, RV, W, false, true><<<grid, block, L.total, stream>>>(a);
    } else if (unc) {
        e = cudaFuncSetAttribute(fwd_kernel<RK, KG, RV, W, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 L.total);
        if (e != cudaSuccess) return PALIMPSA_E_LAUNCH;
        fwd_kernel<RK, KG, RV, W, true, false><<<grid, block, L.total, stream>>>(a);
    } else {
        e = cudaFuncSetAttribute(fwd_kernel<RK, KG, RV, W, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 L.total);
        if (e != cudaSuccess) return PALIMPSA_E_LAUNCH;
        fwd_kernel<RK, KG, RV, W, false, false><<<grid, block, L.total, stream>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

// Warps per CTA: WMAX, or fewer when d_v is short (the row tile stays a multiple of 8 rows).
template <int RK, int KG, int RV, int WMAX>
static int fwd_warps(int V) {
    constexpr int RPW = (32 / KG) * RV;
    // d_k = 48 (16 rows per warp): 3 warps = 48 rows where that pads d_v with fewer idle rows than 64 (d_v = 48, 96, 144)
    if constexpr (RK == 12 && KG == 4 && RV == 2 && WMAX == 4)
        if (V > 32 && (V + 47) / 48 * 48 < (V + 63) / 64 * 64) return 3;
    if constexpr (WMAX >= 4 && (RPW * (WMAX / 4)) % 8 == 0)
        if (V <= RPW * (WMAX / 4)) return WMAX / 4;
    if constexpr (WMAX >= 2 && (RPW * (WMAX / 2)) % 8 == 0)
        if (V <= RPW * (WMAX / 2)) return WMAX / 2;
    return WMAX;
}

template <int RK, int KG, int RV, int WMAX>
static int launch_fwd_t(const FwdArgs& a, int num_seg, bool summary, cudaStream_t stream) {
    const int W = fwd_warps<RK, KG, RV, WMAX>(a.p.V);
    if constexpr (RK == 12 && KG == 4 && RV == 2 && WMAX == 4)
        if (W == 3) return launch_fwd_w<RK, KG, RV, 3>(a, num_seg, summary, stream);
    if constexpr (WMAX >= 4)
        if (W == WMAX / 4) return launch_fwd_w<RK, KG, RV, WMAX / 4>(a, num_seg, summary, stream);
    if constexpr (WMAX >= 2)
        if (W == WMAX / 2) return launch_fwd_w<RK, KG, RV, WMAX / 2>(a, num_seg, summary, stream);
    return launch_fwd_w<RK, KG, RV, WMAX>(a, num_seg, summary, stream);
}

// The thread tilings, one per padded d_k: X(RK, KG, RV, WMAX).
#define PALIMPSA_FWD_TILINGS(X)                                                                                \
    switch (KP) {                                                                                              \
        case 16: X(8, 2, 2, 2);                                                                                \
        case 32: X(8, 4, 2, 4);                                                                                \
        case 48: X(12, 4, 2, 4);                                                                               \
        case 64: X(16, 4, 2, 2);                                                                               \
        case 96: X(12, 8, 2, 4);                                                                               \
        case 128: X(8, 16, 2, 4);                                                                              \
        case 192: X(12, 16, 2, 4);                                                                             \
        case 256: X(16, 16, 2, 4);                                                                             \
        default: break;                                                                                        \
    }

int fwd_tile_rows(int K, int V) {
    const int KP = palimpsa_padded_k(K);
#define PALIMPSA_X(RK, KG, RV, WMAX) return fwd_warps<RK, KG, RV, WMAX>(V) * (32 / KG) * RV
    PALIMPSA_FWD_TILINGS(PALIMPSA_X)
#undef PALIMPSA_X
    return 0;
}

static bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; }

int launch_fwd(const palimpsa_fwd_params* prm, const palimpsa_segments* segs, bool summary, cudaStream_t stream) {
    FwdArgs a{};
    a.p = prm->p;
    a.o = prm->o;
    a.o_var = prm->o_var;
    a.final_mu = prm->final_mu;
    a.final_I = prm->final_I;
    a.ckpt_M = prm->ckpt_M;
    a.ckpt_I = prm->ckpt_I;
    int num_seg = 1;
    if (segs) {
        num_seg = segs->num_segments;
        a.seg_len = segs->seg_len;
        if (summary) {
            a.sum_M = segs->sum_M;
            a.sum_J = segs->sum_J;
            a.decay = segs->decay;
        } else {
            a.start_M = segs->start_M;
            a.start_I = segs->start_I;
        }
    }
    const palimpsa_problem& p = a.p;
    const int es = dtype_size(p.io_dtype);
    a.aligned = ((p.K * es) % 16 == 0) && ((p.V * es) % 16 == 0) && aligned16(p.q) && aligned16(p.k) &&
                aligned16(p.v) && aligned16(p.b) && ((reinterpret_cast<uintptr_t>(p.gt) & 3) == 0);
    const int KP = palimpsa_padded_k(p.K);
#define PALIMPSA_X(RK, KG, RV, WMAX) return launch_fwd_t<RK, KG, RV, WMAX>(a, num_seg, summary, stream)
    PALIMPSA_FWD_TILINGS(PALIMPSA_X)
#undef PALIMPSA_X
    return PALIMPSA_E_DIM;
}

}  // namespace palimpsa
