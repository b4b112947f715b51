// Segment summaries on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 inputs.
//
// The one GEMM-shaped piece of the operator: the end state of a segment started from zero,
//     S_M[v,k] = sum_t a_t v_t[v] k_t[k]        S_J[v,k] = sum_t a_t b_t[v] k_t[k]^2,
// a_t = prod_{s>t} f_s, i.e. two [V x T]*[T x K] products with T the segment's tokens (what the
// reference's forward does element by element when it closes a chunk,
// chunk_palimpsa_forgetting_scalar.py:209-212).  One CTA per (sequence, head, segment):
//   * the 128 threads turn 64-token blocks (walked from the segment's end, so that a_t is a running
//     product) into bf16 UMMA operands in shared memory -- a_t*v, a_t*b, k, k*k, transposed to the
//     K-major core-matrix layout (no swizzle; the row-group stride is padded by 16 bytes so that the
//     transposing stores spread over the banks);
//   * one thread issues tcgen05.mma (M = 128, N = padded d_k, K = 16, kind::f16, fp32 accumulate) into
//     two TMEM accumulators (S_M: columns 0..N-1, S_J: columns 128..128+N-1) and commits to an
//     mbarrier per operand stage; two stages, so operand production overlaps the tensor pipe;
//   * at the end every warp reads its 32 TMEM lanes back (tcgen05.ld) and writes fp32 rows.
// No TMA: every operand is transformed in registers on its way (scaled, squared, transposed), so a
// bulk copy into the MMA layout is not possible; global loads are plain 16-byte coalesced loads.
// Every wait is bounded; on a timeout the CTA records a status code, frees its TMEM and returns.
#include "common.cuh"
#include "host.h"

namespace palimpsa {

constexpr int TCK = 64;                        // tokens per operand block (4 MMAs of K = 16)
constexpr int TC_ROWS = 128;                   // UMMA M
constexpr int TC_SBO = (TCK / 8) * 128 + 16;   // bytes between 8-row groups of an operand (padded)
constexpr int TC_LBO = 128;                    // bytes between the K-direction core matrices
constexpr int TC_OPER = (TC_ROWS / 8) * TC_SBO;  // bytes of one operand tile
constexpr int TC_STAGE = 4 * TC_OPER;          // A_M, A_J, B_M, B_J
constexpr unsigned TC_SPIN = 1u << 24;

__device__ int g_tc_status = 0;  // 0 ok; otherwise the first bounded wait that gave up (1: stage, 2: final)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long umma_desc(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);               // start address
    d |= (unsigned long long)(TC_LBO >> 4) << 16;                   // leading (K-direction) byte offset
    d |= (unsigned long long)(TC_SBO >> 4) << 32;                   // stride (row-group) byte offset
    d |= 1ull << 46;                                                // descriptor version (sm_100)
    return d;                                                       // layout type 0: no swizzle
}

__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (unsigned i = 0; i < TC_SPIN; ++i) {
        unsigned ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 x = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&x);
}

struct TcArgs {
    palimpsa_problem p;
    int seg_len;
    float *sum_M, *sum_J, *decay;
    int KP;
};

__global__ void __launch_bounds__(128) summary_tc_kernel(const TcArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ unsigned tmem_base_s;
    __shared__ float a_s[TCK];
    __shared__ float lf_s[TCK];
    const palimpsa_problem& p = a.p;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int n = blockIdx.x / p.H, h = blockIdx.x - n * p.H;
    const int g = blockIdx.y, G = gridDim.y;
    const int KP = a.KP, K = p.K, V = p.V;
    int bos, len;
    seq_range(p, n, bos, len);
    const int s0 = min(len, g * a.seg_len), s1 = min(len, s0 + a.seg_len);
    const float gh = p.g[h];
    const long long seg_base = (((long long)n * G + g) * p.H + h) * V;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bars[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (w == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(256)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = tmem_base_s;
    // instruction descriptor: D fp32, A/B bf16, both K-major, N = KP, M = 128
    const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(KP >> 3) << 17) | ((unsigned)(TC_ROWS >> 4) << 24);

    const int nblk = (s1 - s0 + TCK - 1) / TCK;
    float logtail = 0.f;  // sum of log f over the tokens after the current block
    int status = 0;
    const int c = lane & 15, tpl = lane >> 4;
    const __nv_bfloat16* gv = reinterpret_cast<const __nv_bfloat16*>(p.v);
    const __nv_bfloat16* gb = reinterpret_cast<const __nv_bfloat16*>(p.b);
    const __nv_bfloat16* gk = reinterpret_cast<const __nv_bfloat16*>(p.k);

    for (int i = 0; i < nblk; ++i) {
        const int blk = nblk - 1 - i;                  // walk from the segment's end
        const int t0 = s0 + blk * TCK;
        const int nt = min(TCK, s1 - t0);
        const int st = i & 1, use = i >> 1;
        unsigned char* stage = sm + st * TC_STAGE;
        // ---- decay weights of the block: a_t = exp(logtail + sum_{s>t in block} log f_s) ----
        if (tid < TCK) lf_s[tid] = tid < nt ? -p.gt[((long long)bos + t0 + tid) * p.H + h] * gh : 0.f;
        __syncthreads();
        if (tid < TCK) {
            float sfx = 0.f;
            for (int s = tid + 1; s < nt; ++s) sfx += lf_s[s];
            a_s[tid] = tid < nt ? __expf(logtail + sfx) : 0.f;
        }
        float blocksum = 0.f;
        for (int s = 0; s < nt; ++s) blocksum += lf_s[s];
        // ---- the stage must be free: the MMAs that read it two blocks ago have completed ----
        if (use > 0 && status == 0) {
            if (!mbar_wait(smem_u32(&bars[st]), (use - 1) & 1)) status = 1;
        }
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // ---- operands: thread (c, tp) handles 8 consecutive rows (chunk c) of a token pair ----
#pragma unroll 1
        for (int it = 0; it < 4; ++it) {
            const int tp = (it * 4 + w) * 2 + tpl;     // token pair 0..31
            const int ta = 2 * tp, tb = ta + 1;
            const float aa = a_s[ta], ab = a_s[tb];
            const long long rowa = ((long long)bos + t0 + ta) * p.H + h, rowb = rowa + p.H;
            const unsigned off = (unsigned)c * TC_SBO + (unsigned)(ta >> 3) * TC_LBO + (unsigned)(ta & 7) * 2;
            auto emit = [&](const __nv_bfloat16* src, int dim, int oper, float wa, float wb, bool square, int oper2) {
                uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
                if (8 * c < dim) {
                    if (ta < nt) xa = *reinterpret_cast<const uint4*>(src + rowa * dim + 8 * c);
                    if (tb < nt) xb = *reinterpret_cast<const uint4*>(src + rowb * dim + 8 * c);
                }
                const unsigned ua[4] = {xa.x, xa.y, xa.z, xa.w}, ub[4] = {xb.x, xb.y, xb.z, xb.w};
                unsigned char* dst = stage + oper * TC_OPER + off;
                unsigned char* dst2 = stage + oper2 * TC_OPER + off;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ua[j]));
                    const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub[j]));
                    *reinterpret_cast<unsigned*>(dst + (2 * j) * 16) = pack_bf16(fa.x * wa, fb.x * wb);
                    *reinterpret_cast<unsigned*>(dst + (2 * j + 1) * 16) = pack_bf16(fa.y * wa, fb.y * wb);
                    if (square) {
                        *reinterpret_cast<unsigned*>(dst2 + (2 * j) * 16) = pack_bf16(fa.x * fa.x, fb.x * fb.x);
                        *reinterpret_cast<unsigned*>(dst2 + (2 * j + 1) * 16) = pack_bf16(fa.y * fa.y, fb.y * fb.y);
                    }
                }
            };
            emit(gv, V, 0, aa, ab, false, 0);   // A_M = a * v
            emit(gb, V, 1, aa, ab, false, 1);   // A_J = a * b
            emit(gk, K, 2, 1.f, 1.f, true, 3);  // B_M = k, B_J = k*k
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && status == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned sbase = smem_u32(stage);
#pragma unroll
            for (int kk = 0; kk < TCK / 16; ++kk) {
                const unsigned acc = (i > 0 || kk > 0) ? 1u : 0u;
                const unsigned long long dAM = umma_desc(sbase + 0 * TC_OPER + kk * 2 * TC_LBO);
                const unsigned long long dAJ = umma_desc(sbase + 1 * TC_OPER + kk * 2 * TC_LBO);
                const unsigned long long dBM = umma_desc(sbase + 2 * TC_OPER + kk * 2 * TC_LBO);
                const unsigned long long dBJ = umma_desc(sbase + 3 * TC_OPER + kk * 2 * TC_LBO);
                asm volatile(
                    "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem),
                    "l"(dAM), "l"(dBM), "r"(idesc), "r"(acc)
                    : "memory");
                asm volatile(
                    "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem + 128u),
                    "l"(dAJ), "l"(dBJ), "r"(idesc), "r"(acc)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&bars[st]))
                         : "memory");
        }
        logtail += blocksum;
    }
    // ---- wait for the last use of both stages ----
    if (status == 0) {
        for (int st = 0; st < 2; ++st) {
            const int uses = (nblk + 1 - st) / 2;      // blocks that used this stage
            if (uses > 0 && !mbar_wait(smem_u32(&bars[st]), (uses - 1) & 1)) status = 2;
        }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // ---- accumulators -> global: warp w owns TMEM lanes (= state rows) 32w .. 32w+31 ----
    const int row = 32 * w + lane;
    if (status == 0) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            float* dstp = (which ? a.sum_J : a.sum_M);
#pragma unroll 1
            for (int c0 = 0; c0 < KP; c0 += 32) {
                unsigned r[32];
                if (nblk > 0) {
                    const unsigned taddr = tmem + ((unsigned)(32 * w) << 16) + (unsigned)(which * 128 + c0);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
                        "%26,%27,%28,%29,%30,%31}, [%32];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                        : "r"(taddr)
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0u;   // empty segment: zero summary
                }
                if (row < V) {
                    float4* o4 = reinterpret_cast<float4*>(dstp + (seg_base + row) * KP + c0);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        o4[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
            }
        }
        if (tid == 0) a.decay[((long long)n * G + g) * p.H + h] = __expf(logtail);
    } else if (tid == 0) {
        atomicCAS(&g_tc_status, 0, status);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (w == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
}

bool summary_tc_supported(const palimpsa_problem& p) {
    const int KP = palimpsa_padded_k(p.K);
    auto al = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    return p.io_dtype == PALIMPSA_BF16 && p.V <= TC_ROWS && p.V % 8 == 0 && p.K % 8 == 0 && KP >= 32 && KP <= 128 &&
           KP % 32 == 0 && al(p.k) && al(p.v) && al(p.b);
}

int launch_summary_tc(const palimpsa_problem& p, const palimpsa_segments& sg, cudaStream_t stream) {
    TcArgs a;
    a.p = p;
    a.seg_len = sg.seg_len;
    a.sum_M = sg.sum_M;
    a.sum_J = sg.sum_J;
    a.decay = sg.decay;
    a.KP = palimpsa_padded_k(p.K);
    const int smem = 2 * TC_STAGE;
    if (cudaFuncSetAttribute(summary_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return PALIMPSA_E_LAUNCH;
    dim3 grid(p.num_seqs * p.H, sg.num_segments, 1);
    summary_tc_kernel<<<grid, 128, smem, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int summary_tc_status() {
    int s = 0;
    if (cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return s;
}

}  // namespace palimpsa
