/*
 * palimpsa_b200.h -- C ABI of libpalimpsa_b200.so
 *
 * Hand-written sm_100a CUDA implementation of the Palimpsa operator (Bayesian-metaplastic linear
 * attention): per sequence and head a mean/precision state pair (mu, I) of shape [V, K] is
 * updated token by token,
 *
 *     f_t = exp(-gt_t * g_h)
 *     M_t = f_t * M_{t-1} + v_t k_t^T                    (M = mu * I)
 *     I_t = f_t * I_{t-1} + (1 - f_t) * Ip_h + b_t (k_t*k_t)^T
 *     o_t = scale * (M_t / I_t) q_t          o_var_t = scale * (1 / I_t) (q_t*q_t)
 *
 * Every entry point takes a plain struct of device pointers and sizes plus a CUDA stream, enqueues
 * its kernels on that stream and returns at once: 0 on success, a negative PALIMPSA_E_* code
 * otherwise.  Nothing here allocates, frees or synchronises unless the comment on the function
 * says so; the caller owns every buffer.  There is no CPU path.
 *
 * Reference interfaces these replace (paths inside the Palimpsa repository):
 *   palimpsa/ops/palimpsa/chunk_palimpsa_forgetting_scalar.py   chunk_palimpsa, ChunkPalimpsa
 *   palimpsa/ops/palimpsa/fused_recurrent_palimpsa.py           fused_recurrent_palimpsa
 *
 * Tensor layouts (all contiguous, last dimension fastest):
 *   q, k        [tokens, H, K]   io dtype          v, b, o, o_var, do, do_var   [tokens, H, V]
 *   gt, dgt     [tokens, H]      float32           g, Ip, dg, dIp               [H] float32
 *   states      [N, H, V, K]     float32  (V-major, K contiguous: the reference's layout,
 *                                          chunk_palimpsa_forgetting_scalar.py:475-476)
 * "tokens" is the flattened (batch, time) axis.  With cu_seqlens == NULL sequence n owns tokens
 * [n*seq_len, (n+1)*seq_len); otherwise tokens [cu_seqlens[n], cu_seqlens[n+1]).
 */
#ifndef PALIMPSA_B200_H
#define PALIMPSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PALIMPSA_ABI_VERSION 11

/* io dtype of q, k, v, b, o, o_var, do, do_var, dq, dk, dv, db */
#define PALIMPSA_F32 0
#define PALIMPSA_BF16 1
#define PALIMPSA_F16 2

/* flags */
#define PALIMPSA_FLAG_UNCERTAINTY 1 /* o_var is produced (forward) / do_var is consumed (backward) */
#define PALIMPSA_FLAG_EXPLICIT_INIT 2 /* backward only: the forward ran from an explicit initial state
                                         (init_mu/init_I need not be passed again); changes dIp */

/* error codes */
#define PALIMPSA_OK 0
#define PALIMPSA_E_NULL (-1)        /* a required pointer is NULL */
#define PALIMPSA_E_SHAPE (-2)       /* a size is non-positive or inconsistent */
#define PALIMPSA_E_DIM (-3)         /* K or V above the supported maximum */
#define PALIMPSA_E_DTYPE (-4)       /* unknown io dtype */
#define PALIMPSA_E_WORKSPACE (-5)   /* workspace missing, too small or misaligned */
#define PALIMPSA_E_LAUNCH (-6)      /* the CUDA runtime refused a launch; see cudaGetLastError */
#define PALIMPSA_E_ALIGN (-7)       /* a state/workspace pointer is not 16-byte aligned */
#define PALIMPSA_E_VERSION (-8)     /* struct_size does not match this library */
#define PALIMPSA_E_LIMIT (-9)       /* problem exceeds a fixed capacity of the entry point */
#define PALIMPSA_E_SYMBOL (-10)     /* the library's own scratch array could not be located on this device */

#define PALIMPSA_MAX_K 256
#define PALIMPSA_CKPT_INTERVAL 16   /* tokens between saved (M, I) checkpoints */
#define PALIMPSA_STATIC_SCRATCH_BYTES (64u << 20) /* capacity of palimpsa_chunk_bwd_static */

/* Problem description shared by forward and backward. */
typedef struct palimpsa_problem {
    int32_t num_seqs;      /* N: batch size, or number of packed sequences                     */
    int32_t seq_len;       /* T per sequence when cu_seqlens == NULL (ignored otherwise)       */
    int32_t total_tokens;  /* rows of q/k/v/b/gt                                               */
    int32_t H, K, V;
    int32_t io_dtype;      /* PALIMPSA_F32 / BF16 / F16                                        */
    int32_t flags;
    float scale;           /* multiplies q (default of the Python wrappers: K^-0.5)            */
    int32_t reserved0;
    const void *q, *k, *v, *b;
    const float *gt, *g, *Ip;
    const int32_t *cu_seqlens;    /* [N+1] device, or NULL                                      */
    const int32_t *chunk_offsets; /* [N] device: first checkpoint slot of each sequence =
                                     exclusive cumsum of ceil(len/16); NULL => n*ceil(T/16)     */
    const float *init_mu, *init_I; /* [N,H,V,K] or both NULL (=> mu=0, I=Ip)                     */
    const int32_t *seq_order;     /* [N] device, or NULL: a permutation of 0..N-1 giving the order in
                                     which the forward and backward main kernels hand sequences to
                                     their CTAs (grid column i works on sequence seq_order[i]).  A
                                     scheduling hint only -- results do not depend on it; packed
                                     batches pass their sequences longest first, so that the long
                                     documents do not end up as the tail of the launch.  The reference
                                     has no counterpart (its programs take sequences in order,
                                     chunk_palimpsa_forgetting_scalar.py:119-126).                */
} palimpsa_problem;

/* Forward.  Replaces chunk_palimpsa_fwd_kernel (chunk_palimpsa_forgetting_scalar.py:66-218) and
 * fused_palimpsa_recurrent_fwd_kernel (fused_recurrent_palimpsa.py:24-154). */
typedef struct palimpsa_fwd_params {
    size_t struct_size;    /* sizeof(palimpsa_fwd_params), checked                              */
    palimpsa_problem p;
    void *o;               /* [tokens,H,V] io dtype                                             */
    void *o_var;           /* same, required iff PALIMPSA_FLAG_UNCERTAINTY                      */
    float *final_mu, *final_I; /* [N,H,V,K] or both NULL; may alias init_mu/init_I (in place)   */
    float *ckpt_M, *ckpt_I;    /* [slots,H,V,KP] float32 or both NULL.  One (M, I) pair per 16
                                  tokens of every sequence (state BEFORE the first token of the
                                  block); needed only by a later backward.  KP = padded K, see
                                  palimpsa_padded_k().  slots >= palimpsa_ckpt_slots().          */
} palimpsa_fwd_params;

/* Backward.  Replaces chunk_palimpsa_bwd_kernel (chunk_palimpsa_forgetting_scalar.py:239-434)
 * and the host-side reductions at :609-613; also serves the fused-recurrent op, whose backward
 * the reference leaves unimplemented (fused_recurrent_palimpsa.py:250-253). */
typedef struct palimpsa_bwd_params {
    size_t struct_size;
    palimpsa_problem p;
    const void *d_o;       /* [tokens,H,V] io dtype                                             */
    const void *d_o_var;   /* required iff PALIMPSA_FLAG_UNCERTAINTY                            */
    const float *ckpt_M, *ckpt_I; /* written by the forward                                     */
    void *dq, *dk, *dv, *db;      /* io dtype                                                   */
    float *dgt;            /* [tokens,H] float32                                                */
    float *dg, *dIp;       /* [H] float32 (summed over sequences and tokens)                    */
    void *workspace;       /* scratch, >= palimpsa_bwd_workspace_bytes(), 256-byte aligned       */
    size_t workspace_bytes;
} palimpsa_bwd_params;

/* Segments.  A sequence may be cut into G segments of seg_len tokens (a multiple of 16) that are
 * processed by different CTAs -- or by different GPUs (context parallelism), where each rank's
 * share of the sequence is its own problem and the boundary states travel between ranks.  The
 * recurrence is linear in (M, J = I - Ip) with a scalar decay per head, so segment g's start state
 * follows from the zero-start summaries of the segments before it:
 *     S_{g+1} = decay_g * S_g + sum_g.
 * The reference has no counterpart: it walks every sequence serially in one program
 * (chunk_palimpsa_forgetting_scalar.py:128-142) and has no context parallelism.
 * All buffers are float32, [N, G, H, V, KP] unless noted; those a call does not use may be NULL. */
typedef struct palimpsa_segments {
    int32_t num_segments;      /* G >= 1                                                        */
    int32_t seg_len;           /* tokens per segment, multiple of 16; G*seg_len >= longest seq   */
    float *sum_M, *sum_J;      /* end state of each segment when started from zero, (M, J) form  */
    float *decay;              /* [N, G, H] product of f over the segment                        */
    float *start_M, *start_I;  /* state at the start of each segment, (M, I) form                */
    float *carry_M, *carry_I;  /* backward: dL/d(end state of the segment), (M, I) form          */
    float *rloc_M, *rloc_I;    /* backward: dL/d(start state of the segment), (M, I) form        */
} palimpsa_segments;

/* Fills sum_M, sum_J and decay for every segment (no reciprocal, no output: the cheap pass).  bf16 problems with
 * d_v <= 128 and at least 8192 state elements per head (padded d_k x d_v) run as two GEMMs on the tensor cores
 * (tcgen05, k by TMA when d_k is a multiple of 64); everything else element by element on the CUDA cores. */
int palimpsa_segment_summary(const palimpsa_problem *p, const palimpsa_segments *segs, void *cuda_stream);

/* Diagnostic: 0 unless a bounded wait inside a kernel gave up on this device since the last call of this
 * function; then the code of the wait (1, 2: tensor-core summary kernel; 3, 4: tensor-core carried-gradient
 * kernel; 5, 6: barriers of the backward main kernel; 7: palimpsa_peer_wait).  Every in-kernel wait of this library is bounded: a
 * kernel that gives up records the code, releases what it holds and returns.  Its results are invalid, and it
 * marks them so that the failure cannot pass unnoticed: the summary kernel writes NaN into the segment's decay
 * (every later output becomes NaN), the other two write NaN into the decay-gradient partials (dgt of the
 * affected tokens and dg come out NaN).  Synchronises the device; reading clears the recorded code, so a
 * non-zero value belongs to the work enqueued since the previous call. */
int palimpsa_tensor_core_status(void);

/* Forward boundary scan: start_M/start_I of every segment from the summaries.  The state before
 * segment 0 is (in_M, in_J) [N,H,V,KP] in (M, J) form if given (a previous rank's end state), else
 * p->init_mu/init_I, else the prior (0, 0).  If out_M/out_J are given they receive the state after
 * the last segment, (M, J) form: what the next rank needs. */
int palimpsa_cp_combine(const palimpsa_problem *p, const palimpsa_segments *segs, const float *in_M,
                        const float *in_J, float *out_M, float *out_J, void *cuda_stream);

/* Backward boundary scan: carry_M/carry_I of every segment from the zero-carry start-state
 * gradients in rloc_M/rloc_I and decay:  carry_{g-1} = rloc_g + decay_g * carry_g.  (in_M, in_I)
 * [N,H,V,KP] is dL/d(end state of the last segment) (a later rank's out), or NULL for zero;
 * (out_M, out_I), if given, receive dL/d(start state of segment 0). */
int palimpsa_cp_combine_bwd(const palimpsa_problem *p, const palimpsa_segments *segs, const float *in_M,
                            const float *in_I, float *out_M, float *out_I, void *cuda_stream);

/* A rank in the middle of a context-parallel chain, split so that only three state-sized streams lie between the
 * arrival of a boundary state and its departure.  palimpsa_cp_relay_prepare, enqueued BEFORE the state arrives,
 * computes what the rank's own segments add to a state that passes through ([N,H,V,KP] pairs, float32): forward
 * (backward = 0) the end state of its segments from a zero start, out of sum_M/sum_J and decay; backward
 * (backward = 1) the start-state gradient from a zero end-state gradient, out of rloc_M/rloc_I and decay.
 * palimpsa_cp_relay then forms  out = (product of the segments' decays) * in + total.  The full boundary scan
 * (palimpsa_cp_combine[_bwd] with the same `in`) follows off the chain's critical path.  Same algebra as the scan
 * (the recurrence is linear in the state with a scalar decay per head); no counterpart in the reference. */
int palimpsa_cp_relay_prepare(const palimpsa_problem *p, const palimpsa_segments *segs, int backward, float *tot_A,
                              float *tot_B, void *cuda_stream);
int palimpsa_cp_relay(const palimpsa_problem *p, const palimpsa_segments *segs, const float *in_A, const float *in_B,
                      const float *tot_A, const float *tot_B, float *out_A, float *out_B, void *cuda_stream);

/* Hand-over of a boundary state between the GPUs of one node without a host round trip or a library call per hop.
 * The exchange buffers of the ranks are mapped into each other's address space (CUDA peer / symmetric memory: the
 * host arranges that); the producer hands palimpsa_cp_combine[_bwd] an out_M/out_J pointer INTO THE NEXT RANK'S
 * buffer, then enqueues palimpsa_peer_signal(flag in the next rank's memory, n): a system-scope fence and a
 * release store of the sequence number n, ordered after everything enqueued on the stream before it.  The consumer
 * enqueues palimpsa_peer_wait(its own flag, n, ...) before the kernels that read the buffer: the stream is held
 * until the flag has reached n (8-byte aligned unsigned 64-bit flags, sequence numbers only grow).  The wait
 * is bounded: after timeout_ms of wall-clock time it records code 7 for palimpsa_tensor_core_status(), writes a NaN
 * to *poison if given (the first element of the buffer it guards, so the failure shows in the results) and lets
 * the stream go on.  Plain loads and stores over NVLink; no multimem, no bulk copies.  Nothing in the reference
 * corresponds (torch.distributed send/recv of the same state is the other transport of
 * palimpsa_b200.parallel.cp_chunk_palimpsa). */
int palimpsa_peer_wait(const void *flag, unsigned long long value, unsigned int timeout_ms, float *poison,
                       void *cuda_stream);
int palimpsa_peer_signal(void *flag, unsigned long long value, void *cuda_stream);

/* palimpsa_chunk_fwd with every segment started from segs->start_M/start_I. */
int palimpsa_chunk_fwd_segments(const palimpsa_fwd_params *params, const palimpsa_segments *segs,
                                void *cuda_stream);

/* palimpsa_chunk_bwd per segment; `mode` selects the pass:
 *   0  full backward with segs->carry_M/carry_I (NULL = zero) as end-state gradients; rloc_M/rloc_I, if
 *      given, receive the start-state gradients;
 *   1  state gradients only, from a zero end-state gradient: writes rloc_M/rloc_I and nothing else
 *      (no workspace, no output buffers needed);
 *   2  main kernel only with zero end-state gradients: every zero-carry gradient term plus rloc_M/rloc_I;
 *      to be followed by palimpsa_cp_combine_bwd, palimpsa_carry_apply and mode 3;
 *   3  the finishing kernels, including the partial slot palimpsa_carry_apply fills. */
int palimpsa_chunk_bwd_segments(const palimpsa_bwd_params *params, const palimpsa_segments *segs,
                                int mode, void *cuda_stream);

/* Adds the terms that are linear in the end-state gradients segs->carry_M/carry_I to a backward that
 * ran with mode 2: dv, db are updated in place, the dk / dgt / dg / dIp terms go to a partial slot of
 * the workspace that mode 3 sums.  Four [tokens x d]*[d x d] products per segment on the tensor cores
 * (tcgen05, TMEM accumulators; the k, v, b token rows arrive by TMA when d_k and d_v are multiples of 64).
 * bf16 io without uncertainty output, d_v <= 128, padded d_k in
 * {32,48,64,96,128}: palimpsa_carry_apply_supported() tells; otherwise use modes 1 and 0. */
int palimpsa_carry_apply_supported(const palimpsa_problem *p);
int palimpsa_carry_apply(const palimpsa_bwd_params *params, const palimpsa_segments *segs, void *cuda_stream);

/* Version of this header the library was built from. */
int palimpsa_abi_version(void);

/* Human-readable text for a PALIMPSA_E_* code (static storage). */
const char *palimpsa_last_error_string(int code);

/* K rounded up to the kernels' tile width (16, 32, 48, 64, 96, 128, 192 or 256); 0 if K > 256. */
int palimpsa_padded_k(int K);

/* State rows (d_v) that one CTA of the forward kernel owns at head dimensions (K, V); 0 if d_k is not
 * supported.  A forward launch has ceil(V / rows) x num_seqs x H CTAs (times the segment count): hosts use it
 * to decide whether a problem fills the GPU or should be cut into segments.  No counterpart in the reference,
 * whose grid is fixed at (V/16) x N x H programs (chunk_palimpsa_forgetting_scalar.py:478). */
int palimpsa_fwd_tile_rows(int K, int V);

/* The same for the backward kernel, whose tile also depends on the element type (PALIMPSA_F32 / _BF16 / _F16) and on
 * whether the uncertainty output takes part (shared-memory budget): a backward launch has ceil(V / rows) x num_seqs x
 * H CTAs of up to 12 warps, usually one resident per SM, so hosts that plan a training step count waves with it.
 * 0 if the shape is not supported.  No counterpart in the reference (grid (V/16) x N x H,
 * chunk_palimpsa_forgetting_scalar.py:558). */
int palimpsa_bwd_tile_rows(int K, int V, int io_dtype, int uncertainty);

/* Upper bound on checkpoint slots for a problem: ceil(total_tokens/16) + num_seqs (varlen needs
 * no host synchronisation to size its buffers). */
long long palimpsa_ckpt_slots(const palimpsa_problem *p);

/* Chunked forward (training / prefill): the layers' mode 'chunk' (palimpsa/layers/palimpsa.py:309). */
int palimpsa_chunk_fwd(const palimpsa_fwd_params *params, void *cuda_stream);

/* Fused-recurrent forward: the layers' mode 'fused_recurrent' (palimpsa/layers/palimpsa.py:317).
 * Same kernels as the chunked forward; kept as its own symbol because the reference has two ops. */
int palimpsa_recurrent_fwd(const palimpsa_fwd_params *params, void *cuda_stream);

/* One decode step for every sequence of a state cache, in place: tokens == num_seqs, seq_len == 1,
 * final_mu/final_I may equal init_mu/init_I.  The state cache replaces the (final_mu, final_I)
 * tuple the layer stores in its Cache (palimpsa/layers/palimpsa.py:325-331). */
int palimpsa_decode_step(const palimpsa_fwd_params *params, void *cuda_stream);

/* Scratch bytes the backward needs for this problem. */
size_t palimpsa_bwd_workspace_bytes(const palimpsa_problem *p);

/* Backward of the chunked op (ChunkPalimpsa.backward, chunk_palimpsa_forgetting_scalar.py:522-620). */
int palimpsa_chunk_bwd(const palimpsa_bwd_params *params, void *cuda_stream);

/* The same backward split in two: stages bit 0 = main kernel (fills the workspace partials, dv, db),
 * bit 1 = finishing kernels (dq, dk, dgt, dg, dIp from the workspace).  Lets a caller time or
 * overlap the two; stages == 3 equals palimpsa_chunk_bwd.  No counterpart in the reference, whose
 * backward is one kernel plus torch reductions (chunk_palimpsa_forgetting_scalar.py:592-613). */
int palimpsa_chunk_bwd_stages(const palimpsa_bwd_params *params, void *cuda_stream, int stages);

/* Backward for callers that must not allocate device memory: plugin hosts whose memory pool is
 * fixed at start-up, real-time or interrupt-style service threads, and code running where
 * cudaMalloc is unavailable or would stall the device (it synchronises).  Identical to
 * palimpsa_chunk_bwd, except that params->workspace / workspace_bytes are ignored: the scratch is a
 * fixed PALIMPSA_STATIC_SCRATCH_BYTES (64 MiB) array inside the library, resident on every GPU that
 * loads the library for as long as the process lives.  The caller still passes every input and
 * output buffer.  It calls no cudaMalloc, cudaFree or any allocating routine.
 *   - Problems whose palimpsa_bwd_workspace_bytes() exceeds the capacity return PALIMPSA_E_LIMIT
 *     (at d_k = d_v = 128 the capacity covers about 9900 (token, head) rows: 6720 bytes per row).
 *   - The first call on each device looks up the array's device address (once per device, with that
 *     device current); make that first call outside any stream capture.  With the CUDA runtime's
 *     default lazy module loading the 64 MiB are only reserved when the library's backward code is first
 *     loaded on a device, which can be this very call: on a device whose memory is already handed out
 *     the look-up then fails and the call returns PALIMPSA_E_SYMBOL without launching anything.  Hosts
 *     with a fixed pool should therefore make one small call at start-up, before they carve up the
 *     device.  The address is cached per device ordinal: only the device's primary context (the one the
 *     CUDA runtime uses) is supported.
 *   - All calls share the one array, which keeps whatever the previous call left in it.  Nothing in
 *     it has to start at zero: each call's main kernel writes every byte its finishing kernels read.
 *     Two calls that overlap on the GPU (different streams, or threads) race on it; serialise them.
 * This entry point has no counterpart in the reference. */
int palimpsa_chunk_bwd_static(const palimpsa_bwd_params *params, void *cuda_stream);

/* Backward of the fused-recurrent op (absent in the reference: fused_recurrent_palimpsa.py:250-253). */
int palimpsa_recurrent_bwd(const palimpsa_bwd_params *params, void *cuda_stream);

/* ---- Layer-side element-wise work around the operator ---------------------------------------------
 * The reference's layer prepares the operator's inputs and post-processes its output with a dozen
 * separate PyTorch element-wise passes (palimpsa/layers/palimpsa.py:269-283 and :337-344).  These
 * entry points do each side in ONE pass over HBM.  Arithmetic is float32 with a single rounding to the
 * io dtype, except bs, which is rounded to the io dtype before use exactly as the layer does (:272).
 * All tensors are contiguous; `tokens` counts every token of the (packed) batch. */

/* Prologue (layers/palimpsa.py:269-281):
 *     gt = softplus(dt_raw + dt_bias[h])            q = q_raw / max(|q_raw|_2, 1e-12)   (same for k)
 *     bs = sigmoid(bs_raw)  (rounded to io dtype)    v = x * bs
 *     b  = sigmoid(b_raw) * softplus(b_scale[h]) * bs
 * q_raw / k_raw carry Hq <= H heads (H % Hq == 0); head h reads head h / (H/Hq) (the layer's repeat, :266). */
typedef struct palimpsa_layer_prologue {
    size_t struct_size;
    int32_t io_dtype;            /* PALIMPSA_F32 / BF16 / F16                                      */
    int32_t H, Hq, K, V;         /* K <= 256, V <= 1024                                             */
    int64_t tokens;
    const void *q_raw, *k_raw;   /* [tokens,Hq,K] io dtype                                          */
    const void *x, *b_raw;       /* [tokens,H,V]  io dtype                                          */
    const void *dt_raw, *bs_raw; /* [tokens,H]    io dtype                                          */
    const float *dt_bias, *b_scale; /* [H] float32                                                  */
    void *q, *k;                 /* out [tokens,H,K] io dtype                                       */
    void *v, *b;                 /* out [tokens,H,V] io dtype                                       */
    float *gt;                   /* out [tokens,H] float32                                          */
    /* backward only */
    const void *dq, *dk, *dv, *db; /* gradients w.r.t. the outputs above, io dtype                  */
    const float *dgt;            /* [tokens,H] float32                                              */
    void *dq_raw, *dk_raw;       /* out [tokens,Hq,K] io dtype                                      */
    void *dx, *db_raw;           /* out [tokens,H,V]  io dtype (dx: the v = x*bs branch only)       */
    void *ddt_raw, *dbs_raw;     /* out [tokens,H]    io dtype                                      */
    float *d_dt_bias, *d_b_scale;/* out [H] float32, summed over tokens in a fixed order            */
    void *workspace;             /* backward scratch, >= palimpsa_layer_workspace_bytes()           */
    size_t workspace_bytes;
} palimpsa_layer_prologue;

/* Epilogue (layers/palimpsa.py:337-343; the gated RMS norm is FusedRMSNormGated of the pinned
 * dependency flash-linear-attention 0.5.1, activation "swish"):
 *     z = o + x * D[h]   (PALIMPSA_LAYER_RESIDUAL)        r = 1 / sqrt(mean_v(z^2) + eps)
 *     y = z * r * weight[v] * gate * sigmoid(gate)        (PALIMPSA_LAYER_GATE; else y = z * r * weight[v]) */
#define PALIMPSA_LAYER_RESIDUAL 1u
#define PALIMPSA_LAYER_GATE 2u
typedef struct palimpsa_layer_epilogue {
    size_t struct_size;
    int32_t io_dtype;
    int32_t H, V;                /* V <= 1024                                                       */
    uint32_t flags;
    float eps;
    int64_t tokens;
    const void *o, *x, *gate;    /* [tokens,H,V] io dtype (x / gate may be NULL without their flag) */
    const float *D, *weight;     /* [H], [V] float32                                                */
    void *y;                     /* out [tokens,H,V] io dtype                                       */
    /* backward only */
    const void *dy;              /* [tokens,H,V] io dtype                                           */
    void *d_o, *dx, *dgate;      /* out [tokens,H,V] io dtype (dx: the residual branch only)        */
    float *dD, *dweight;         /* out [H], [V] float32, summed in a fixed order                   */
    void *workspace;
    size_t workspace_bytes;
} palimpsa_layer_epilogue;

/* Scratch either backward needs for `tokens` x H rows of width V (the larger of the two). */
size_t palimpsa_layer_workspace_bytes(int64_t tokens, int32_t H, int32_t V);
int palimpsa_layer_prologue_fwd(const palimpsa_layer_prologue *a, void *cuda_stream);
int palimpsa_layer_prologue_bwd(const palimpsa_layer_prologue *a, void *cuda_stream);
int palimpsa_layer_epilogue_fwd(const palimpsa_layer_epilogue *a, void *cuda_stream);
int palimpsa_layer_epilogue_bwd(const palimpsa_layer_epilogue *a, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* PALIMPSA_B200_H */
