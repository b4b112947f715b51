// Host-side declarations shared by the translation units of libpalimpsa_b200.so.
#pragma once

#include <cuda_runtime.h>

#include "../../include/palimpsa_b200.h"

namespace palimpsa {

// Enqueue the forward kernel (fwd.cu).  Parameters are assumed validated.  With `segs` every sequence is
// cut into segs->num_segments segments that run as separate CTAs: `summary` = false starts each from
// segs->start_M/start_I; `summary` = true computes the zero-start end state and decay of every segment.
int launch_fwd(const palimpsa_fwd_params* prm, const palimpsa_segments* segs, bool summary, cudaStream_t stream);

// Single-token decode step (decode.cu): dedicated HBM-bound kernel, when it covers the call.
bool decode_supported(const palimpsa_fwd_params* prm);
int launch_decode(const palimpsa_fwd_params* prm, cudaStream_t stream);

// Backward (bwd.cu): main kernel (stages bit 0) + the two finishing kernels (bit 1); bit 2: the finishing
// kernels also sum the extra partial slot that carry_tc.cu fills.
int launch_bwd(const palimpsa_bwd_params* prm, const palimpsa_segments* segs, bool carry_only, cudaStream_t stream,
               int stages);

// Segment summaries on the tensor cores (summary_tc.cu): bf16 inputs, d_v <= 128, padded d_k in {32,48,64,96,128}.
bool summary_tc_supported(const palimpsa_problem& p);
int launch_summary_tc(const palimpsa_problem& p, const palimpsa_segments& segs, cudaStream_t stream);
int summary_tc_status();

// Carried-gradient terms of a segmented backward on the tensor cores (carry_tc.cu).
bool carry_tc_supported(const palimpsa_problem& p);
int launch_carry_tc(const palimpsa_bwd_params* prm, const palimpsa_segments& segs, cudaStream_t stream);
int carry_tc_status();
int bwd_wait_status();  // 0, or the code of a bounded barrier wait of the backward main kernel that gave up

// Boundary scans over segments (segments.cu).
int launch_combine_fwd(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_M, const float* in_J,
                       float* out_M, float* out_J, cudaStream_t stream);
int launch_combine_bwd(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_M, const float* in_I,
                       float* out_M, float* out_I, cudaStream_t stream);

// Stream-ordered flags in peer-mapped memory (peer.cu): a bounded wait until *flag >= value, and a release store.
int launch_peer_wait(const void* flag, unsigned long long value, unsigned timeout_ms, float* poison, cudaStream_t stream);
int launch_peer_signal(void* flag, unsigned long long value, cudaStream_t stream);
int peer_status();   // 0, or 7 when a wait ran out

// A context-parallel hop split in two (segments.cu): what this rank adds to a state passing through, computed
// before the state arrives, and out = decay_product * in + total when it does.
int launch_relay_total(const palimpsa_problem& p, const palimpsa_segments& segs, int backward, float* tot_A,
                       float* tot_B, cudaStream_t stream);
int launch_relay(const palimpsa_problem& p, const palimpsa_segments& segs, const float* in_A, const float* in_B,
                 const float* tot_A, const float* tot_B, float* out_A, float* out_B, cudaStream_t stream);

// Backward whose scratch is the library's own fixed device array (bwd.cu).
int launch_bwd_static(const palimpsa_bwd_params* prm, cudaStream_t stream);

// State rows (d_v) one forward CTA owns at these head dimensions (0: d_k unsupported).
int fwd_tile_rows(int K, int V);

// State rows (d_v) one backward CTA owns for this problem; the number of row tiles follows.
int bwd_tile_rows(const palimpsa_problem& p);

// Layout of the backward scratch memory (byte offsets from a 256-byte aligned base).
struct BwdWorkspace {
    size_t dq_part, dk_part;    // float [tiles][tokens*H][KP]   (dk, df, dip: tiles + 1 slots)
    size_t df_part, dip_part;   // float [tiles][tokens*H]
    size_t w_dg, w_dip;         // float [tokens*H]
    size_t total;
    int tiles, KP;
};
BwdWorkspace bwd_workspace_layout(const palimpsa_problem& p);

}  // namespace palimpsa
