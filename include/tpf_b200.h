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
 *  - bf16 tensors are 16-byte aligned; extents are int64_t.
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
int tpf_attn_bwd(const void* q, const void* k, const void* v, const void* d_out,
                 const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const void* out, const float* lse,
                 const float* mask, int64_t mask_pitch,
                 const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* dq, void* dk, void* dv, float* dbias, float* delta,
                 void* workspace, int64_t workspace_bytes,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TPF_B200_H_ */
