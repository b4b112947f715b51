// extern "C" surface of libpalimpsa_b200.so: argument validation and dispatch.  No kernel lives
// here; see fwd.cu and bwd.cu.

#include "common.cuh"
#include "host.h"

using namespace palimpsa;

namespace {

int check_problem(const palimpsa_problem& p) {
    if (p.num_seqs <= 0 || p.H <= 0 || p.K <= 0 || p.V <= 0 || p.total_tokens < 0) return PALIMPSA_E_SHAPE;
    if (!p.cu_seqlens && (p.seq_len < 0 || (long long)p.seq_len * p.num_seqs != p.total_tokens))
        return PALIMPSA_E_SHAPE;
    if (p.K > PALIMPSA_MAX_K) return PALIMPSA_E_DIM;
    if (p.io_dtype != PALIMPSA_F32 && p.io_dtype != PALIMPSA_BF16 && p.io_dtype != PALIMPSA_F16)
        return PALIMPSA_E_DTYPE;
    if (!p.g || !p.Ip) return PALIMPSA_E_NULL;
    if (p.total_tokens > 0 && (!p.q || !p.k || !p.v || !p.b || !p.gt)) return PALIMPSA_E_NULL;
    if ((p.init_mu == nullptr) != (p.init_I == nullptr)) return PALIMPSA_E_NULL;
    if ((long long)p.total_tokens * p.H >= (1ll << 31)) return PALIMPSA_E_SHAPE;
    return PALIMPSA_OK;
}

bool misaligned16(const void* x) { return x && (reinterpret_cast<uintptr_t>(x) & 15); }

int check_fwd(const palimpsa_fwd_params* prm) {
    if (!prm) return PALIMPSA_E_NULL;
    if (prm->struct_size != sizeof(palimpsa_fwd_params)) return PALIMPSA_E_VERSION;
    int rc = check_problem(prm->p);
    if (rc) return rc;
    const palimpsa_problem& p = prm->p;
    if (p.total_tokens > 0 && !prm->o) return PALIMPSA_E_NULL;
    if ((p.flags & PALIMPSA_FLAG_UNCERTAINTY) && p.total_tokens > 0 && !prm->o_var) return PALIMPSA_E_NULL;
    if ((prm->final_mu == nullptr) != (prm->final_I == nullptr)) return PALIMPSA_E_NULL;
    if ((prm->ckpt_M == nullptr) != (prm->ckpt_I == nullptr)) return PALIMPSA_E_NULL;
    if (misaligned16(prm->ckpt_M) || misaligned16(prm->ckpt_I)) return PALIMPSA_E_ALIGN;
    if (p.K % 4 == 0 && (misaligned16(p.init_mu) || misaligned16(p.init_I) || misaligned16(prm->final_mu) ||
                         misaligned16(prm->final_I)))
        return PALIMPSA_E_ALIGN;
    return PALIMPSA_OK;
}

int check_bwd(const palimpsa_bwd_params* prm, bool caller_workspace = true, bool need_outputs = true) {
    if (!prm) return PALIMPSA_E_NULL;
    if (prm->struct_size != sizeof(palimpsa_bwd_params)) return PALIMPSA_E_VERSION;
    int rc = check_problem(prm->p);
    if (rc) return rc;
    const palimpsa_problem& p = prm->p;
    if (need_outputs && (!prm->dg || !prm->dIp)) return PALIMPSA_E_NULL;
    if (p.total_tokens > 0) {
        if (!prm->d_o || !prm->ckpt_M || !prm->ckpt_I) return PALIMPSA_E_NULL;
        if (need_outputs && (!prm->dq || !prm->dk || !prm->dv || !prm->db || !prm->dgt)) return PALIMPSA_E_NULL;
        if ((p.flags & PALIMPSA_FLAG_UNCERTAINTY) && !prm->d_o_var) return PALIMPSA_E_NULL;
    }
    if (misaligned16(prm->ckpt_M) || misaligned16(prm->ckpt_I)) return PALIMPSA_E_ALIGN;
    const size_t need = palimpsa_bwd_workspace_bytes(&p);
    if (need == 0) return PALIMPSA_E_DIM;
    if (!caller_workspace) return PALIMPSA_OK;
    if (!prm->workspace || prm->workspace_bytes < need) return PALIMPSA_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(prm->workspace) & 255) return PALIMPSA_E_WORKSPACE;
    return PALIMPSA_OK;
}

int check_segments(const palimpsa_problem& p, const palimpsa_segments* sg) {
    if (!sg) return PALIMPSA_E_NULL;
    if (sg->num_segments < 1 || sg->seg_len <= 0 || sg->seg_len % PALIMPSA_CKPT_INTERVAL) return PALIMPSA_E_SHAPE;
    if (!p.cu_seqlens && (long long)sg->num_segments * sg->seg_len < p.seq_len) return PALIMPSA_E_SHAPE;
    if (palimpsa_padded_k(p.K) == 0) return PALIMPSA_E_DIM;
    const void* ptrs[] = {sg->sum_M, sg->sum_J, sg->start_M, sg->start_I, sg->carry_M, sg->carry_I, sg->rloc_M, sg->rloc_I};
    for (const void* x : ptrs)
        if (misaligned16(x)) return PALIMPSA_E_ALIGN;
    return PALIMPSA_OK;
}

}  // namespace

extern "C" {

int palimpsa_abi_version(void) { return PALIMPSA_ABI_VERSION; }

const char* palimpsa_last_error_string(int code) {
    switch (code) {
        case PALIMPSA_OK: return "ok";
        case PALIMPSA_E_NULL: return "a required pointer is NULL (or only one of a pointer pair was given)";
        case PALIMPSA_E_SHAPE: return "a size is non-positive or inconsistent";
        case PALIMPSA_E_DIM: return "d_k above the supported maximum for this entry point";
        case PALIMPSA_E_DTYPE: return "unknown io dtype";
        case PALIMPSA_E_WORKSPACE: return "workspace missing, too small or not 256-byte aligned";
        case PALIMPSA_E_LAUNCH: return "the CUDA runtime refused a kernel launch";
        case PALIMPSA_E_ALIGN: return "a state or checkpoint pointer is not 16-byte aligned";
        case PALIMPSA_E_VERSION: return "struct_size does not match this library (header/library mismatch)";
        case PALIMPSA_E_LIMIT: return "problem exceeds a fixed capacity of this entry point";
        case PALIMPSA_E_SYMBOL: return "the library's own scratch array could not be located on the current device";
        default: return "unknown error code";
    }
}

int palimpsa_padded_k(int K) {
    static const int sizes[] = {16, 32, 48, 64, 96, 128, 192, 256};
    if (K <= 0) return 0;
    for (int s : sizes)
        if (K <= s) return s;
    return 0;
}

int palimpsa_bwd_tile_rows(int K, int V, int io_dtype, int uncertainty) {
    if (K <= 0 || V <= 0 || K > PALIMPSA_MAX_K) return 0;
    if (io_dtype != PALIMPSA_F32 && io_dtype != PALIMPSA_BF16 && io_dtype != PALIMPSA_F16) return 0;
    palimpsa_problem p{};
    p.K = K;
    p.V = V;
    p.io_dtype = io_dtype;
    p.flags = uncertainty ? PALIMPSA_FLAG_UNCERTAINTY : 0;
    return bwd_tile_rows(p);
}

int palimpsa_fwd_tile_rows(int K, int V) {
    if (K <= 0 || V <= 0 || K > PALIMPSA_MAX_K) return 0;
    return fwd_tile_rows(K, V);
}

long long palimpsa_ckpt_slots(const palimpsa_problem* p) {
    if (!p) return 0;
    return ((long long)p->total_tokens + TB - 1) / TB + p->num_seqs;
}

int palimpsa_chunk_fwd(const palimpsa_fwd_params* prm, void* cuda_stream) {
    int rc = check_fwd(prm);
    if (rc) return rc;
    return launch_fwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_recurrent_fwd(const palimpsa_fwd_params* prm, void* cuda_stream) {
    int rc = check_fwd(prm);
    if (rc) return rc;
    if (decode_supported(prm)) return launch_decode(prm, static_cast<cudaStream_t>(cuda_stream));
    return launch_fwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_decode_step(const palimpsa_fwd_params* prm, void* cuda_stream) {
    int rc = check_fwd(prm);
    if (rc) return rc;
    const palimpsa_problem& p = prm->p;
    if (p.cu_seqlens || p.seq_len != 1 || p.total_tokens != p.num_seqs) return PALIMPSA_E_SHAPE;
    if (!p.init_mu || !prm->final_mu) return PALIMPSA_E_NULL;
    if (prm->ckpt_M) return PALIMPSA_E_SHAPE;
    if (decode_supported(prm)) return launch_decode(prm, static_cast<cudaStream_t>(cuda_stream));
    return launch_fwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_segment_summary(const palimpsa_problem* p, const palimpsa_segments* sg, void* cuda_stream) {
    if (!p) return PALIMPSA_E_NULL;
    int rc = check_problem(*p);
    if (rc) return rc;
    rc = check_segments(*p, sg);
    if (rc) return rc;
    if (!sg->sum_M || !sg->sum_J || !sg->decay) return PALIMPSA_E_NULL;
    // The tensor-core kernel costs the same per token whatever the head size (128-row tiles); below about
    // 8192 state elements per head the element-wise summary pass is the faster one (measured on 48x48 .. 128x128).
    if (summary_tc_supported(*p) && (long long)palimpsa_padded_k(p->K) * p->V >= 8192)
        return launch_summary_tc(*p, *sg, static_cast<cudaStream_t>(cuda_stream));
    palimpsa_fwd_params prm{};
    prm.struct_size = sizeof(prm);
    prm.p = *p;
    return launch_fwd(&prm, sg, true, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_tensor_core_status(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    const int a = summary_tc_status(), b = carry_tc_status(), c = bwd_wait_status(), d = peer_status();  // each clears what it read
    return a ? a : (b ? b : (c ? c : d));
}

int palimpsa_peer_wait(const void* flag, unsigned long long value, unsigned int timeout_ms, float* poison, void* cuda_stream) {
    if (!flag) return PALIMPSA_E_NULL;
    if ((reinterpret_cast<uintptr_t>(flag) & 7) != 0) return PALIMPSA_E_ALIGN;
    return launch_peer_wait(flag, value, timeout_ms, poison, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_peer_signal(void* flag, unsigned long long value, void* cuda_stream) {
    if (!flag) return PALIMPSA_E_NULL;
    if ((reinterpret_cast<uintptr_t>(flag) & 7) != 0) return PALIMPSA_E_ALIGN;
    return launch_peer_signal(flag, value, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_carry_apply_supported(const palimpsa_problem* p) { return p && carry_tc_supported(*p) ? 1 : 0; }

int palimpsa_carry_apply(const palimpsa_bwd_params* prm, const palimpsa_segments* sg, void* cuda_stream) {
    int rc = check_bwd(prm);
    if (rc) return rc;
    rc = check_segments(prm->p, sg);
    if (rc) return rc;
    if (!sg->carry_M || !sg->carry_I) return PALIMPSA_E_NULL;
    if (!carry_tc_supported(prm->p)) return PALIMPSA_E_DTYPE;
    return launch_carry_tc(prm, *sg, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_cp_combine(const palimpsa_problem* p, const palimpsa_segments* sg, const float* in_M, const float* in_J,
                        float* out_M, float* out_J, void* cuda_stream) {
    if (!p) return PALIMPSA_E_NULL;
    int rc = check_problem(*p);
    if (rc) return rc;
    rc = check_segments(*p, sg);
    if (rc) return rc;
    if (!sg->sum_M || !sg->sum_J || !sg->decay || !sg->start_M || !sg->start_I) return PALIMPSA_E_NULL;
    if ((in_M == nullptr) != (in_J == nullptr) || (out_M == nullptr) != (out_J == nullptr)) return PALIMPSA_E_NULL;
    if (misaligned16(in_M) || misaligned16(in_J) || misaligned16(out_M) || misaligned16(out_J)) return PALIMPSA_E_ALIGN;
    return launch_combine_fwd(*p, *sg, in_M, in_J, out_M, out_J, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_cp_combine_bwd(const palimpsa_problem* p, const palimpsa_segments* sg, const float* in_M,
                            const float* in_I, float* out_M, float* out_I, void* cuda_stream) {
    if (!p) return PALIMPSA_E_NULL;
    int rc = check_problem(*p);
    if (rc) return rc;
    rc = check_segments(*p, sg);
    if (rc) return rc;
    if (!sg->decay || !sg->carry_M || !sg->carry_I || !sg->rloc_M || !sg->rloc_I) return PALIMPSA_E_NULL;
    if ((in_M == nullptr) != (in_I == nullptr) || (out_M == nullptr) != (out_I == nullptr)) return PALIMPSA_E_NULL;
    if (misaligned16(in_M) || misaligned16(in_I) || misaligned16(out_M) || misaligned16(out_I)) return PALIMPSA_E_ALIGN;
    return launch_combine_bwd(*p, *sg, in_M, in_I, out_M, out_I, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_cp_relay_prepare(const palimpsa_problem* p, const palimpsa_segments* sg, int backward, float* tot_A,
                              float* tot_B, void* cuda_stream) {
    if (!p || !tot_A || !tot_B) return PALIMPSA_E_NULL;
    int rc = check_problem(*p);
    if (rc) return rc;
    rc = check_segments(*p, sg);
    if (rc) return rc;
    if (!sg->decay || (backward ? (!sg->rloc_M || !sg->rloc_I) : (!sg->sum_M || !sg->sum_J))) return PALIMPSA_E_NULL;
    if (misaligned16(tot_A) || misaligned16(tot_B)) return PALIMPSA_E_ALIGN;
    return launch_relay_total(*p, *sg, backward ? 1 : 0, tot_A, tot_B, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_cp_relay(const palimpsa_problem* p, const palimpsa_segments* sg, const float* in_A, const float* in_B,
                      const float* tot_A, const float* tot_B, float* out_A, float* out_B, void* cuda_stream) {
    if (!p || !in_A || !in_B || !tot_A || !tot_B || !out_A || !out_B) return PALIMPSA_E_NULL;
    int rc = check_problem(*p);
    if (rc) return rc;
    rc = check_segments(*p, sg);
    if (rc) return rc;
    if (!sg->decay) return PALIMPSA_E_NULL;
    if (misaligned16(in_A) || misaligned16(in_B) || misaligned16(tot_A) || misaligned16(tot_B) || misaligned16(out_A) ||
        misaligned16(out_B))
        return PALIMPSA_E_ALIGN;
    return launch_relay(*p, *sg, in_A, in_B, tot_A, tot_B, out_A, out_B, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_chunk_fwd_segments(const palimpsa_fwd_params* prm, const palimpsa_segments* sg, void* cuda_stream) {
    int rc = check_fwd(prm);
    if (rc) return rc;
    rc = check_segments(prm->p, sg);
    if (rc) return rc;
    if (!sg->start_M || !sg->start_I) return PALIMPSA_E_NULL;
    return launch_fwd(prm, sg, false, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_chunk_bwd_segments(const palimpsa_bwd_params* prm, const palimpsa_segments* sg, int mode,
                                void* cuda_stream) {
    if (mode < 0 || mode > 3) return PALIMPSA_E_SHAPE;
    const bool carry_only = mode == 1;
    int rc = check_bwd(prm, !carry_only, !carry_only);
    if (rc) return rc;
    rc = check_segments(prm->p, sg);
    if (rc) return rc;
    if ((sg->carry_M == nullptr) != (sg->carry_I == nullptr) || (sg->rloc_M == nullptr) != (sg->rloc_I == nullptr))
        return PALIMPSA_E_NULL;
    if ((mode == 1 || mode == 2) && !sg->rloc_M) return PALIMPSA_E_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    if (mode == 2) {  // main kernel only, zero end-state gradients
        palimpsa_segments z = *sg;
        z.carry_M = z.carry_I = nullptr;
        return launch_bwd(prm, &z, false, st, 1);
    }
    if (mode == 3) return launch_bwd(prm, sg, false, st, 2 | 4);  // finishing kernels, extra slot included
    return launch_bwd(prm, sg, carry_only, st, 3);
}

size_t palimpsa_bwd_workspace_bytes(const palimpsa_problem* p) {
    if (!p || p->K <= 0 || p->V <= 0 || p->K > PALIMPSA_MAX_K) return 0;
    return bwd_workspace_layout(*p).total;
}

int palimpsa_chunk_bwd(const palimpsa_bwd_params* prm, void* cuda_stream) {
    int rc = check_bwd(prm);
    if (rc) return rc;
    return launch_bwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream), 3);
}

int palimpsa_chunk_bwd_stages(const palimpsa_bwd_params* prm, void* cuda_stream, int stages) {
    int rc = check_bwd(prm);
    if (rc) return rc;
    if (stages < 1 || stages > 3) return PALIMPSA_E_SHAPE;
    return launch_bwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream), stages);
}

int palimpsa_chunk_bwd_static(const palimpsa_bwd_params* prm, void* cuda_stream) {
    int rc = check_bwd(prm, false);
    if (rc) return rc;
    return launch_bwd_static(prm, static_cast<cudaStream_t>(cuda_stream));
}

int palimpsa_recurrent_bwd(const palimpsa_bwd_params* prm, void* cuda_stream) {
    int rc = check_bwd(prm);
    if (rc) return rc;
    return launch_bwd(prm, nullptr, false, static_cast<cudaStream_t>(cuda_stream), 3);
}

}  // extern "C"
