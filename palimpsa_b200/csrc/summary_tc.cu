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
// TMA feeds the one operand that is used exactly as it lies in global memory: k as the B operand of S_M.  Its
// tile (64 tokens x d_k) is token-major, i.e. MN-major for the MMA, and arrives as cp.async.bulk.tensor boxes of
// 64 tokens x 64 columns with the 128-byte swizzle (completion on an mbarrier per stage; d_k a multiple of 64).
// The other three operands are transformed in registers on their way (scaled by a_t, squared, transposed).
// Every wait is bounded; on a timeout the CTA records a status code, frees its TMEM and returns.
#include "host.h"
#include "tc_common.cuh"

namespace palimpsa {

constexpr int TCK = 64;                        // tokens per operand block (4 MMAs of K = 16)
constexpr int TC_ROWS = 128;                   // UMMA M
constexpr int TC_SBO = (TCK / 8) * 128 + 16;   // bytes between 8-row groups of an operand (padded)
constexpr int TC_LBO = 128;                    // bytes between the K-direction core matrices
constexpr int TC_OPER = (TC_ROWS / 8) * TC_SBO;  // bytes of one operand tile
constexpr int TC_KBOX = TCK * 128;             // one TMA box of k: 64 tokens x 64 columns (128 bytes), swizzled
constexpr int TC_TMA = 2 * TC_KBOX;            // d_k <= 128: two boxes
constexpr int TC_STAGE = TC_TMA + 4 * TC_OPER; // [k by TMA] A_M, A_J, B_M (k by hand), B_J; a multiple of 1024 bytes
static_assert(TC_STAGE % 1024 == 0, "stages must keep the 1024-byte alignment of the TMA boxes");

__device__ int g_tc_status = 0;  // 0 ok; otherwise the first bounded wait that gave up (1: stage, 2: final)

struct TcArgs {
    palimpsa_problem p;
    int seg_len;
    float *sum_M, *sum_J, *decay;
    int KP;
};

template <bool TMA>
__global__ void __launch_bounds__(128) summary_tc_kernel(const TcArgs a, const __grid_constant__ CUtensorMap kmap) {
    extern __shared__ __align__(128) unsigned char sm_raw[];
    unsigned char* sm = sm_raw + ((1024u - (tc::smem_u32(sm_raw) & 1023u)) & 1023u);   // TMA boxes: 1024-byte aligned
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ __align__(8) unsigned long long tbars[2];   // completion of each stage's TMA load
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
        tc::mbar_init(&bars[0]);
        tc::mbar_init(&bars[1]);
        tc::mbar_init(&tbars[0]);
        tc::mbar_init(&tbars[1]);
        tc::mbar_init_fence();
        if (TMA) tc::tma_prefetch_map(&kmap);
    }
    if (w == 0) tc::tmem_alloc(&tmem_base_s, 256);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const unsigned tmem = tmem_base_s;
    const unsigned idesc = tc::idesc_bf16(KP);  // D fp32, A/B bf16, both K-major, N = KP, M = 128

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
            if (!tc::mbar_wait(&bars[st], (use - 1) & 1)) status = 1;
        }
        __syncthreads();
        tc::fence_after_sync();
        if (TMA && tid == 0 && status == 0) {   // k tile of the block straight into the stage (rows past the segment's
            tc::mbar_expect_tx(&tbars[st], (unsigned)(KP / 64) * TC_KBOX);   // end meet zero rows of the A operands)
            for (int x = 0; x < KP / 64; ++x)
                tc::tma_load_2d(stage + x * TC_KBOX, &kmap, h * K + 64 * x, (int)(bos + t0), &tbars[st]);
        }
        unsigned char* opers = stage + TC_TMA;
        // ---- operands: thread (c, tp) handles 8 consecutive rows (chunk c) of a token pair ----
#pragma unroll 1
        for (int it = 0; it < 4; ++it) {
            const int tp = (it * 4 + w) * 2 + tpl;     // token pair 0..31
            const int ta = 2 * tp, tb = ta + 1;
            const float aa = a_s[ta], ab = a_s[tb];
            const long long rowa = ((long long)bos + t0 + ta) * p.H + h, rowb = rowa + p.H;
            const unsigned off = (unsigned)c * TC_SBO + (unsigned)(ta >> 3) * TC_LBO + (unsigned)(ta & 7) * 2;
            auto emit = [&](const __nv_bfloat16* src, int dim, int oper, float wa, float wb, bool square, int oper2,
                            bool first = true) {
                uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
                if (8 * c < dim) {
                    if (ta < nt) xa = *reinterpret_cast<const uint4*>(src + rowa * dim + 8 * c);
                    if (tb < nt) xb = *reinterpret_cast<const uint4*>(src + rowb * dim + 8 * c);
                }
                const unsigned ua[4] = {xa.x, xa.y, xa.z, xa.w}, ub[4] = {xb.x, xb.y, xb.z, xb.w};
                unsigned char* dst = opers + oper * TC_OPER + off;
                unsigned char* dst2 = opers + oper2 * TC_OPER + off;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ua[j]));
                    const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ub[j]));
                    if (first) {
                        *reinterpret_cast<unsigned*>(dst + (2 * j) * 16) = tc::pack_bf16(fa.x * wa, fb.x * wb);
                        *reinterpret_cast<unsigned*>(dst + (2 * j + 1) * 16) = tc::pack_bf16(fa.y * wa, fb.y * wb);
                    }
                    if (square) {
                        *reinterpret_cast<unsigned*>(dst2 + (2 * j) * 16) = tc::pack_bf16(fa.x * fa.x, fb.x * fb.x);
                        *reinterpret_cast<unsigned*>(dst2 + (2 * j + 1) * 16) = tc::pack_bf16(fa.y * fa.y, fb.y * fb.y);
                    }
                }
            };
            emit(gv, V, 0, aa, ab, false, 0);   // A_M = a * v
            emit(gb, V, 1, aa, ab, false, 1);   // A_J = a * b
            emit(gk, K, 2, 1.f, 1.f, true, 3, !TMA);  // B_J = k*k, and B_M = k unless TMA brings it
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (TMA && tid == 0 && status == 0 && !tc::mbar_wait(&tbars[st], use & 1)) status = 1;
        if (tid == 0 && status == 0) {
            tc::fence_after_sync();
            const unsigned sbase = tc::smem_u32(opers), kbase = tc::smem_u32(stage);
#pragma unroll
            for (int kk = 0; kk < TCK / 16; ++kk) {
                const bool acc = i > 0 || kk > 0;
                const unsigned ko = kk * 2 * TC_LBO;
                // k by TMA: MN-major boxes, a K = 16 step = 16 token rows = two 8-row groups of 1024 bytes
                const unsigned long long dBM = TMA ? tc::desc_mn_sw128(kbase + kk * 2048, TC_KBOX)
                                                   : tc::desc(sbase + 2 * TC_OPER + ko, TC_LBO, TC_SBO);
                tc::mma(tmem, tc::desc(sbase + 0 * TC_OPER + ko, TC_LBO, TC_SBO), dBM,
                        TMA ? (idesc | tc::IDESC_B_MN_MAJOR) : idesc, acc);                       // S_M += (a v)^T k
                tc::mma(tmem + 128u, tc::desc(sbase + 1 * TC_OPER + ko, TC_LBO, TC_SBO),
                        tc::desc(sbase + 3 * TC_OPER + ko, TC_LBO, TC_SBO), idesc, acc);          // S_J += (a b)^T k^2
            }
            tc::commit(&bars[st]);
        }
        logtail += blocksum;
    }
    // ---- wait for the last use of both stages ----
    if (status == 0) {
        for (int st = 0; st < 2; ++st) {
            const int uses = (nblk + 1 - st) / 2;      // blocks that used this stage
            if (uses > 0 && !tc::mbar_wait(&bars[st], (uses - 1) & 1)) status = 2;
        }
    }
    tc::fence_after_sync();
    // ---- accumulators -> global: warp w owns TMEM lanes (= state rows) 32w .. 32w+31 ----
    const int row = 32 * w + lane;
    if (status == 0) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            float* dstp = (which ? a.sum_J : a.sum_M);
#pragma unroll 1
            for (int c0 = 0; c0 < KP; c0 += 32) {
                float r[32];
                if (nblk > 0) {
                    tc::tmem_ld32(tmem + ((unsigned)(32 * w) << 16) + (unsigned)(which * 128 + c0), r);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = 0.f;   // empty segment: zero summary
                }
                if (row < V) {
                    float4* o4 = reinterpret_cast<float4*>(dstp + (seg_base + row) * KP + c0);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (c0 + 4 * j < KP)   // padded d_k = 48: the last read covers 16 columns past the accumulator
                            o4[j] = make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                }
            }
        }
        if (tid == 0) a.decay[((long long)n * G + g) * p.H + h] = __expf(logtail);
    } else if (tid == 0) {
        // a wait ran out: record it and make the failure visible in the data (a NaN decay poisons every state
        // and output that depends on this segment)
        atomicCAS(&g_tc_status, 0, status);
        a.decay[((long long)n * G + g) * p.H + h] = __int_as_float(0x7fc00000);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (w == 0) tc::tmem_free(tmem, 256);
}

bool summary_tc_supported(const palimpsa_problem& p) {
    const int KP = palimpsa_padded_k(p.K);
    auto al = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    return p.io_dtype == PALIMPSA_BF16 && p.V <= TC_ROWS && p.V % 8 == 0 && p.K % 8 == 0 && KP >= 32 && KP <= 128 &&
           KP % 16 == 0 && al(p.k) && al(p.v) && al(p.b);
}

int launch_summary_tc(const palimpsa_problem& p, const palimpsa_segments& sg, cudaStream_t stream) {
    TcArgs a;
    a.p = p;
    a.seg_len = sg.seg_len;
    a.sum_M = sg.sum_M;
    a.sum_J = sg.sum_J;
    a.decay = sg.decay;
    a.KP = palimpsa_padded_k(p.K);
    const int smem = 2 * TC_STAGE + 1024;   // + slack to round the base up to 1024 bytes
    dim3 grid(p.num_seqs * p.H, sg.num_segments, 1);
    CUtensorMap kmap{};
    const bool tma = p.K % 64 == 0 && p.total_tokens > 0 &&
                     make_tensor_map_bf16_rows(&kmap, p.k, (unsigned long long)p.total_tokens, (unsigned long long)p.H * p.K, TCK);
    if (tma) {
        if (cudaFuncSetAttribute(summary_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return PALIMPSA_E_LAUNCH;
        summary_tc_kernel<true><<<grid, 128, smem, stream>>>(a, kmap);
    } else {
        if (cudaFuncSetAttribute(summary_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return PALIMPSA_E_LAUNCH;
        summary_tc_kernel<false><<<grid, 128, smem, stream>>>(a, kmap);
    }
    return cudaGetLastError() == cudaSuccess ? PALIMPSA_OK : PALIMPSA_E_LAUNCH;
}

int summary_tc_status() {
    int s = 0;
    if (cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    if (s) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    }
    return s;
}

}  // namespace palimpsa
