// Small inline-PTX helpers for the tcgen05 / TMEM kernels (sm_100a): shared-memory matrix descriptors
// for the K-major, unswizzled core-matrix layout, MMA issue, commit, bounded mbarrier waits, TMEM
// allocation and read-back.
#pragma once

#include <cuda.h>   // CUtensorMap and its enums only: the driver is reached through cudaGetDriverEntryPoint, never linked

#include "common.cuh"

namespace palimpsa {
namespace tc {

constexpr unsigned SPIN_LIMIT = 1u << 24;  // polls before a wait gives up (the kernel then reports and returns)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

// K-major operand without swizzle: 8-row x 16-byte core matrices; `lbo` = bytes between the two core
// matrices an MMA of K = 16 consumes, `sbo` = bytes between consecutive 8-row groups.
__device__ __forceinline__ unsigned long long desc(unsigned addr, unsigned lbo, unsigned sbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)(lbo >> 4) << 16;
    d |= (unsigned long long)(sbo >> 4) << 32;
    d |= 1ull << 46;  // descriptor version of sm_100; layout type 0 = no swizzle
    return d;
}

// K-major operand in the 128-byte-swizzle layout that a TMA tile load with CU_TENSOR_MAP_SWIZZLE_128B writes:
// rows of 128 bytes (64 bf16 of the contraction dimension), 8-row groups 1024 bytes apart, the tile 1024-byte
// aligned.  A K = 16 step advances the start address by 32 bytes inside the row; the leading-dimension offset is
// not used by this layout (set to its neutral value).
__device__ __forceinline__ unsigned long long desc_sw128(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= 1ull << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;   // descriptor version of sm_100
    d |= 2ull << 61;   // layout type: 128-byte swizzle
    return d;
}

// MN-major operand (the NON-contraction dimension contiguous in shared memory) in the 128-byte-swizzle layout:
// what a TMA tile load of [contraction rows][64 elements of the M/N dimension] writes.  Rows (contraction index)
// are 128 bytes apart, 8-row groups 1024 bytes apart (stride offset); `lbo` = bytes between consecutive 64-element
// blocks of the M/N dimension (one TMA box).  A K = 16 step advances the start address by two 8-row groups.
__device__ __forceinline__ unsigned long long desc_mn_sw128(unsigned addr, unsigned lbo) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)(lbo >> 4) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}
constexpr unsigned IDESC_B_MN_MAJOR = 1u << 16;   // instruction-descriptor bit: operand B is MN-major

// Instruction descriptor of kind::f16 with bf16 A/B (both K-major), fp32 D, M = 128, N = n.
__device__ __forceinline__ unsigned idesc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
}

__device__ __forceinline__ void mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc, bool acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(acc ? 1u : 0u)
        : "memory");
}

__device__ __forceinline__ void commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// Wait until the phase with this parity has completed; false if it did not within `limit` polls.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned limit = SPIN_LIMIT) {
    const unsigned addr = smem_u32(bar);
    for (unsigned i = 0; i < limit; ++i) {
        unsigned ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// ---- TMA (cp.async.bulk.tensor): 2-D tile of THIS GPU's memory into shared memory, completion on an mbarrier.
// Every load has this one CTA as its only destination.  x is the coordinate along the contiguous dimension: x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<unsigned long long>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(map)) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One full warp allocates / frees `cols` TMEM columns (power of two >= 32); the base lands in *slot.
__device__ __forceinline__ void tmem_alloc(unsigned* slot, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(unsigned base, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane (warp w may only touch lanes 32w .. 32w+31).
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
        "%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 x = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&x);
}

}  // namespace tc

// Host side: a 2-D tensor map over a row-major bf16 matrix [rows][row_elems] of this GPU's memory, box of 64
// elements (128 bytes) x box_rows rows, 128-byte swizzle, zero fill outside.  Returns false if the driver entry
// point is unavailable or refuses the description (the caller then takes its non-TMA path).
inline bool make_tensor_map_bf16_rows(CUtensorMap* map, const void* base, unsigned long long rows,
                                      unsigned long long row_elems, unsigned box_rows) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<encode_fn>(fn);
    }();
    if (!encode || rows == 0) return false;
    const cuuint64_t dims[2] = {row_elems, rows};
    const cuuint64_t strides[1] = {row_elems * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace palimpsa
