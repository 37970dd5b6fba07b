/*
 * C ABI of libtpf_b200.so - B200 (sm_100a) kernels for the OpenFold3 pair-stack
 * operators: triangle attention and the triangle multiplicative update.
 *
 * Conventions
 *  - Every function returns 0 on success or a TPF_ERR_* code; the message for the
 *    last failure on the calling thread is tpf_last_error_string().
 *  - All pointers are device pointers unless stated otherwise.  Nothing here
 *    allocates device memory (except where a function says so) or synchronises;
 *    work is enqueued on `stream` (a cudaStream_t passed as void*).
 *  - bf16 tensors are 16-byte aligned, and so are the fp32 dbias output and every workspace
 *    (rows are written with 16-byte vector stores); other fp32 tensors are 4-byte aligned.
 *    A misaligned pointer is rejected with TPF_ERR_INVALID_ARGUMENT before anything is launched.
 *    Extents are int64_t.
 *  - Host threads may call concurrently and a process may use several GPUs: launch attributes,
 *    symbol addresses and the SM count are cached per device.
 *  - Kernels never spin forever: a wait that exceeds its time limit records a
 *    code that tpf_device_status() returns after the stream has been synchronised.
 *
 * Each entry point names the reference interface it stands in for
 * (paths are relative to the reference project's root).
 */
#ifndef TPF_B200_H_
#define TPF_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPF_OK 0
#define TPF_ERR_INVALID_ARGUMENT 1
#define TPF_ERR_UNSUPPORTED 2
#define TPF_ERR_CUDA 3
#define TPF_ERR_WORKSPACE 4
#define TPF_ERR_DEVICE_STATUS 5

/* Library identification ("tpf_b200 <version> sm_100a"). */
const char* tpf_version(void);

/* Message of the last error raised on this host thread (never NULL). */
const char* tpf_last_error_string(void);

/* Reads and clears the device status words of the current device (synchronous
 * small copies).  *status = 0 when every bounded wait completed.
 * Stands in for the reference's launch checks, which only call
 * cudaGetLastError (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_forward.cu:1957). */
int tpf_device_status(int* status);

/* Kernel launches issued through this library by the calling process so far (host counter). */
int64_t tpf_launch_count(void);

/* Self-test of the bounded wait every kernel uses: launches one 32-thread CTA that waits, with a
 * limit of about one millisecond, on a barrier nothing arrives on.  The wait gives up, the kernel
 * ends normally, and the next tpf_device_status() (after the stream is synchronised) reports 1
 * (wait timeout) and clears it.  `report` (device, 3 x uint32, may be NULL) receives the SM cycles
 * the first wait took, the cycles of a second wait in the same CTA (which must return at once) and
 * 1 once the kernel reached its end.  The reference has no bounded waits, hence no counterpart;
 * its kernels rely on cudaGetLastError alone
 * (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_forward.cu:1957). */
int tpf_selftest_bounded_wait(unsigned int* report, void* stream);

/* Batched bf16 GEMM  D[b][m][n] = sum_k A[b][m][k] * B[b][n][k], fp32 accumulate.
 * a_mn / b_mn = 0: operand stored [batch][mn][k] (k contiguous);
 *             = 1: operand stored [batch][k][mn] (m or n contiguous).
 * lda/ldb/ldd and the batch strides are in elements.  out_f32 selects fp32 or bf16 D.
 * k_per_split > 0 runs `batch` K-slices of ONE problem (D[b] holds slice b's partial sum).
 * Replaces torch.bmm in
 * openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:244-249, 357-362. */
int tpf_bmm_bf16(const void* A, int64_t lda, int64_t batch_stride_a, int a_mn,
                 const void* B, int64_t ldb, int64_t batch_stride_b, int b_mn,
                 void* D, int64_t ldd, int64_t batch_stride_d, int out_f32,
                 int64_t M, int64_t N, int64_t K, int64_t batch, int64_t k_per_split,
                 int swizzle_bytes, void* stream);

/* Triangle-attention forward.
 *   q,k,v   bf16, logical shape [B,O,H,N,D]; *_strides = element strides of (b,o,h,n); the last
 *           dimension is contiguous (covers both the head-major and the sequence-major storage
 *           order of the reference).  D in {16,32,64}.  Q is NOT pre-scaled; `scale` multiplies Q K^T.
 *   mask    fp32 additive [B,O,mask_pitch] (first N entries of each row are used; 0 keeps, -inf drops)
 *   bias    bf16 [bias_batch,H,N,bias_pitch], bias_batch = 1 (shared by all b) or B
 *   out     bf16 [B,O,N,H,D] contiguous;  lse fp32 [B,O,H,N] (natural log; -inf for a fully masked row)
 * Replaces turbopairformer_triangle_forward_out / _forward_shadow_out
 * (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_forward.cu:1826-2004). */
int tpf_attn_fwd(const void* q, const void* k, const void* v,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const float* mask, int64_t mask_pitch,
                 const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* out, float* lse,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, void* stream);

/* Bytes of device scratch tpf_attn_bwd needs for this shape (0 is possible). */
int64_t tpf_attn_bwd_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, int64_t bias_batch);

/* Triangle-attention backward: dq, dk, dv (bf16, contiguous [B,O,H,N,D]), dbias (fp32
 * [bias_batch,H,N,N], summed over the outer axis and over b when bias_batch == 1) and
 * delta (fp32 [B,O,H,N], rowsum(dO * O), caller-allocated scratch that is also an output).
 *   d_out, out   bf16 [B,O,N,H,D] contiguous (gradient of / the forward output)
 *   lse          fp32 [B,O,H,N] from tpf_attn_fwd
 *   workspace    at least tpf_attn_bwd_workspace_bytes(...) bytes, 256-byte aligned (may be NULL when 0)
 * Other arguments as in tpf_attn_fwd.  Deterministic: fixed summation orders, no atomics.
 * Replaces turbopairformer_triangle_delta_out + turbopairformer_triangle_sr_backward_out
 * (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_delta.cu:343-414,
 *  openfold3/core/kernels/turbopairformer/turbopairformer_triangle_dq_dbias.cu:2526-2648) and the
 * Python workspace planner in turbopairformer_triangle_dq_dbias.py:466-669. */
#define TPF_ATTN_BWD_STAGE_DELTA 1  /* delta = rowsum(dO * O) */
#define TPF_ATTN_BWD_STAGE_DQKV 2   /* dq, dk, dv (reads delta) */
#define TPF_ATTN_BWD_STAGE_DBIAS 4  /* dbias (reads delta) */
#define TPF_ATTN_BWD_STAGE_ALL 7

/* tpf_attn_bwd restricted to the stages in `stages` (bit mask above); used to time the
 * stages separately.  tpf_attn_bwd(...) is tpf_attn_bwd_stages(..., TPF_ATTN_BWD_STAGE_ALL). */
int tpf_attn_bwd_stages(const void* q, const void* k, const void* v, const void* d_out,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const void* out, const float* lse,
                 const float* mask, int64_t mask_pitch,
                 const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* dq, void* dk, void* dv, float* dbias, float* delta,
                 void* workspace, int64_t workspace_bytes,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, int stages, void* stream);

int tpf_attn_bwd(const void* q, const void* k, const void* v, const void* d_out,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const void* out, const float* lse,
                 const float* mask, int64_t mask_pitch,
                 const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* dq, void* dk, void* dv, float* dbias, float* delta,
                 void* workspace, int64_t workspace_bytes,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, void* stream);

/* Capacity in bytes of the scratch array built into the library (see tpf_attn_bwd_static_scratch). */
int64_t tpf_attn_bwd_static_scratch_capacity(void);

/* tpf_attn_bwd for callers that cannot allocate device memory (code between stream-capture
 * begin/end, plugin or real-time hosts that get their memory once at start-up, runtimes that
 * own the device heap): same inputs, outputs and results as tpf_attn_bwd, but the scratch is a
 * fixed 16 MiB array inside the library image instead of a caller workspace.  The call allocates
 * and frees nothing.  This entry point has no counterpart in the reference.
 *  - Shapes whose scratch need (tpf_attn_bwd_workspace_bytes) exceeds the capacity are rejected
 *    with TPF_ERR_WORKSPACE and a message; nothing is launched.
 *  - The first call on each device looks up the array's device address (a synchronous runtime
 *    query); make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps whatever the last call left there.
 *    Nothing in it needs clearing between calls, but two calls that overlap on the GPU
 *    (different streams, no ordering) race on it; order them.
 *  - Every GPU that loads the library keeps the 16 MiB until the process exits. */
int tpf_attn_bwd_static_scratch(const void* q, const void* k, const void* v, const void* d_out,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const void* out, const float* lse,
                 const float* mask, int64_t mask_pitch,
                 const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* dq, void* dk, void* dv, float* dbias, float* delta,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, void* stream);

/* Scratch sizes of the TriMul entry points (bytes; 256-byte aligned buffers). */
int64_t tpf_trimul_fwd_workspace_bytes(int64_t B, int64_t N, int64_t C);
int64_t tpf_trimul_bwd_workspace_bytes(int64_t B, int64_t N, int64_t C);

/* Triangle multiplicative update, forward.  direction: 0 = outgoing, 1 = incoming.
 *   z        bf16 [B,N,N,C] contiguous, C in {32,64,96,128}, N a multiple of 8
 *   mask     fp32 [B,N,N] (1 keeps, 0 drops)
 *   weights  fp32 masters: p_in [2C,C] = cat[a_p,b_p], g_in [2C,C] = cat[a_g,b_g],
 *            p_out [C,C] (linear_z), g_out [C,C] (linear_g); LayerNorm vectors fp32 [C]
 *   out      bf16 [B,N,N,C]
 *   saved state for the backward pass, all caller-allocated:
 *            zln, gate, xln bf16 [B*N*N,C]; a_cm, b_cm, x_cm bf16 [B*C,N*N] (channel-major);
 *            mean_in, rstd_in, mean_out, rstd_out fp32 [B*N*N]
 * Replaces trimul_in_fwd + torch.bmm + trimul_out_fwd
 * (openfold3/core/kernels/turbopairformer/turbopairformer_trimul_cuda.cu:1049-1166, 1472-1530;
 *  openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:184-292). */
int tpf_trimul_fwd(const void* z, const float* mask,
                   const float* p_in, const float* g_in, const float* p_out, const float* g_out,
                   const float* norm_in_w, const float* norm_in_b, const float* norm_out_w, const float* norm_out_b,
                   int direction, int64_t B, int64_t N, int64_t C,
                   void* out, void* zln, float* mean_in, float* rstd_in, void* a_cm, void* b_cm, void* gate,
                   void* x_cm, void* xln, float* mean_out, float* rstd_out,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* Triangle multiplicative update, backward.  Inputs: d_out bf16 [B,N,N,C], the forward's inputs and
 * saved state.  Outputs: d_z bf16 [B,N,N,C]; fp32 weight gradients d_p_in [2C,C], d_g_in [2C,C],
 * d_p_out [C,C], d_g_out [C,C]; fp32 LayerNorm gradients [C] each.  Weight gradients are split-K
 * sums folded in ascending order (no atomics).
 * Replaces sig_mul_bwd_out, transpose_ln_bwd, trimul_gate_split_bwd, ln_bwd_dx, ln_bwd_dgb,
 * trimul_wgrad_fixed_fold and the cuBLAS calls between them
 * (openfold3/core/kernels/turbopairformer/turbopairformer_trimul_cuda.cu:1789-2171;
 *  openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:295-392). */
int tpf_trimul_bwd(const void* d_out, const void* z, const float* mask,
                   const float* p_in, const float* g_in, const float* p_out, const float* g_out,
                   const float* norm_in_w, const float* norm_out_w,
                   int direction, int64_t B, int64_t N, int64_t C,
                   const void* out, const void* zln, const float* mean_in, const float* rstd_in,
                   const void* a_cm, const void* b_cm, const void* gate, const void* x_cm, const void* xln,
                   const float* mean_out, const float* rstd_out,
                   void* d_z, float* d_p_in, float* d_g_in, float* d_p_out, float* d_g_out,
                   float* d_norm_in_w, float* d_norm_in_b, float* d_norm_out_w, float* d_norm_out_b,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* Stage-wise TriMul for row-sharded (axially parallel) execution.  `rows_per_batch` is the number of
 * pair rows each batch entry holds on this rank (N_local * N; 0 means N * N; a multiple of 64) and
 * replaces N*N in every [B*N*N, C] / [B*C, N*N] extent above.  `stages` selects
 *   forward : 1 = LayerNorm + projections + gating (z -> zln, a_cm, b_cm, gate, statistics)
 *             2 = k-contraction (whole pair tensors only; sharded callers run tpf_bmm_bf16 on their
 *                 channel shard between two all-to-alls instead)
 *             4 = output LayerNorm + projection + gate (x_cm, gate -> out, xln, statistics)
 *   backward: 1 = output gate / projection / LayerNorm backward (-> dx_cm, d_p_out, d_norm_out_*)
 *             2 = contraction backward (dx_cm, a_cm, b_cm -> da_cm, db_cm)
 *             4 = projection / input LayerNorm backward (da_cm, db_cm -> d_z, d_p_in, d_g_in, d_g_out, d_norm_in_*)
 * Backward stages 1 and 4 communicate through `workspace`: pass the same buffer to both calls
 * (size: tpf_trimul_bwd_stages_workspace_bytes).  dx_cm / da_cm / db_cm, when not NULL, are used
 * instead of the workspace's own buffers so the caller can exchange them between ranks.
 * The reference has no sharded TriMul; these follow the stage split of
 * openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:225-263, 327-392. */
int64_t tpf_trimul_bwd_stages_workspace_bytes(int64_t B, int64_t rows_per_batch, int64_t C);
int tpf_trimul_fwd_stages(const void* z, const float* mask,
                   const float* p_in, const float* g_in, const float* p_out, const float* g_out,
                   const float* norm_in_w, const float* norm_in_b, const float* norm_out_w, const float* norm_out_b,
                   int direction, int64_t B, int64_t N, int64_t C,
                   void* out, void* zln, float* mean_in, float* rstd_in, void* a_cm, void* b_cm, void* gate,
                   void* x_cm, void* xln, float* mean_out, float* rstd_out,
                   void* workspace, int64_t workspace_bytes, int64_t rows_per_batch, int stages, void* stream);
int tpf_trimul_bwd_stages(const void* d_out, const void* z, const float* mask,
                   const float* p_in, const float* g_in, const float* p_out, const float* g_out,
                   const float* norm_in_w, const float* norm_out_w,
                   int direction, int64_t B, int64_t N, int64_t C,
                   const void* out, const void* zln, const float* mean_in, const float* rstd_in,
                   const void* a_cm, const void* b_cm, const void* gate, const void* x_cm, const void* xln,
                   const float* mean_out, const float* rstd_out,
                   void* d_z, float* d_p_in, float* d_g_in, float* d_p_out, float* d_g_out,
                   float* d_norm_in_w, float* d_norm_in_b, float* d_norm_out_w, float* d_norm_out_b,
                   void* workspace, int64_t workspace_bytes, int64_t rows_per_batch, int stages,
                   void* dx_cm, void* da_cm, void* db_cm, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TPF_B200_H_ */
