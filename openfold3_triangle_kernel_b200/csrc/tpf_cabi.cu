// extern "C" surface of libtpf_b200.so (declarations: include/tpf_b200.h).
#include "../../include/tpf_b200.h"
#include "tpf_host.cuh"

namespace tpf {

char* last_error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int bmm_status_fetch_and_clear(int* out);
int bmm_bf16(const void* A, int64_t lda, int64_t bsa, int a_mn, const void* B, int64_t ldb, int64_t bsb, int b_mn,
             void* D, int64_t ldd, int64_t bsd, int out_f32, int64_t M, int64_t N, int64_t K, int64_t batch,
             int64_t k_per_split, int swizzle_bytes, cudaStream_t stream);

int attn_fwd_status_fetch_and_clear(int* out);
int attn_fwd(const void* q, const void* k, const void* v, const int64_t* q_strides, const int64_t* k_strides,
             const int64_t* v_strides, const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch,
             int64_t bias_batch, void* out, float* lse, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
             float scale, cudaStream_t stream);

int attn_bwd_status_fetch_and_clear(int* out);
int64_t attn_bwd_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t D);
int64_t attn_dbias_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t G);
int attn_bwd_dqkv(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                  const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                  const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch, int64_t bias_batch,
                  void* dq, void* dk, void* dv, float* delta, void* workspace, int64_t workspace_bytes, int64_t B,
                  int64_t O, int64_t H, int64_t N, int64_t D, float scale, int stages, cudaStream_t stream);
int attn_bwd_dbias(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                   const int64_t* k_strides, const int64_t* v_strides, const float* lse, const float* delta,
                   const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch, int64_t bias_batch,
                   float* dbias, void* workspace, int64_t workspace_bytes, int64_t B, int64_t O, int64_t H, int64_t N,
                   int64_t D, float scale, cudaStream_t stream);

int64_t attn_bwd_static_scratch_capacity();
int attn_bwd_static_scratch(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                            const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                            const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch,
                            int64_t bias_batch, void* dq, void* dk, void* dv, float* dbias, float* delta, int64_t B,
                            int64_t O, int64_t H, int64_t N, int64_t D, float scale, cudaStream_t stream);
int selftest_status_fetch_and_clear(int* out);
int selftest_bounded_wait(unsigned int* report, cudaStream_t stream);

int trimul_status_fetch_and_clear(int* out);
int64_t trimul_fwd_workspace_bytes(int64_t B, int64_t N, int64_t C);
int64_t trimul_bwd_workspace_bytes(int64_t B, int64_t N, int64_t C);
int trimul_fwd(const void* z, const float* mask, const float* p_in, const float* g_in, const float* p_out,
               const float* g_out, const float* gin, const float* bin, const float* gout, const float* bout,
               int incoming, int64_t B, int64_t N, int64_t C, void* out, void* zln, float* mean_in, float* rstd_in,
               void* a_cm, void* b_cm, void* gate, void* x_cm, void* xln, float* mean_out, float* rstd_out,
               void* workspace, int64_t workspace_bytes, int64_t NN, int stages, cudaStream_t stream);
int trimul_bwd(const void* d_out, const void* z, const float* mask, const float* p_in, const float* g_in,
               const float* p_out, const float* g_out, const float* gin, const float* gout, int incoming, int64_t B,
               int64_t N, int64_t C, const void* out, const void* zln, const float* mean_in, const float* rstd_in,
               const void* a_cm, const void* b_cm, const void* gate, const void* x_cm, const void* xln,
               const float* mean_out, const float* rstd_out, void* d_z, float* d_p_in, float* d_g_in, float* d_p_out,
               float* d_g_out, float* d_gin, float* d_bin, float* d_gout, float* d_bout, void* workspace,
               int64_t workspace_bytes, int64_t NN, int stages, void* dx_io, void* da_io, void* db_io,
               cudaStream_t stream);

}  // namespace tpf

extern "C" {

const char* tpf_version(void) { return "tpf_b200 0.1 sm_100a"; }

const char* tpf_last_error_string(void) { return tpf::last_error_buffer(); }

int64_t tpf_launch_count(void) { return tpf::launch_counter().load(); }

int tpf_device_status(int* status) {
  TPF_REQUIRE(status != nullptr, TPF_ERR_INVALID_ARGUMENT, "tpf_device_status: status is NULL");
  int total = 0, v = 0;
  int rc = tpf::bmm_status_fetch_and_clear(&v);
  if (rc) return rc;
  total |= v;
  if ((rc = tpf::attn_fwd_status_fetch_and_clear(&v))) return rc;
  total |= v;
  if ((rc = tpf::attn_bwd_status_fetch_and_clear(&v))) return rc;
  total |= v;
  if ((rc = tpf::trimul_status_fetch_and_clear(&v))) return rc;
  total |= v;
  if ((rc = tpf::selftest_status_fetch_and_clear(&v))) return rc;
  total |= v;
  *status = total;
  return TPF_OK;
}

int tpf_selftest_bounded_wait(unsigned int* report, void* stream) {
  return tpf::selftest_bounded_wait(report, static_cast<cudaStream_t>(stream));
}

int tpf_bmm_bf16(const void* A, int64_t lda, int64_t batch_stride_a, int a_mn, const void* B, int64_t ldb,
                 int64_t batch_stride_b, int b_mn, void* D, int64_t ldd, int64_t batch_stride_d, int out_f32,
                 int64_t M, int64_t N, int64_t K, int64_t batch, int64_t k_per_split, int swizzle_bytes,
                 void* stream) {
  return tpf::bmm_bf16(A, lda, batch_stride_a, a_mn, B, ldb, batch_stride_b, b_mn, D, ldd, batch_stride_d, out_f32,
                       M, N, K, batch, k_per_split, swizzle_bytes, static_cast<cudaStream_t>(stream));
}

int tpf_attn_fwd(const void* q, const void* k, const void* v, const int64_t* q_strides, const int64_t* k_strides,
                 const int64_t* v_strides, const float* mask, int64_t mask_pitch, const void* bias,
                 int64_t bias_pitch, int64_t bias_batch, void* out, float* lse, int64_t B, int64_t O, int64_t H,
                 int64_t N, int64_t D, float scale, void* stream) {
  TPF_REQUIRE(q_strides && k_strides && v_strides, TPF_ERR_INVALID_ARGUMENT, "tpf_attn_fwd: stride arrays are NULL");
  return tpf::attn_fwd(q, k, v, q_strides, k_strides, v_strides, mask, mask_pitch, bias, bias_pitch, bias_batch, out,
                       lse, B, O, H, N, D, scale, static_cast<cudaStream_t>(stream));
}

static int64_t round_up_256(int64_t x) { return (x + 255) / 256 * 256; }

int64_t tpf_attn_bwd_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, int64_t bias_batch) {
  if (B <= 0 || O <= 0 || H <= 0 || N <= 0 || (bias_batch != 1 && bias_batch != B)) return 0;
  return round_up_256(tpf::attn_bwd_workspace_bytes(B, O, H, N, D)) +
         round_up_256(tpf::attn_dbias_workspace_bytes(B, O, H, N, bias_batch));
}

int tpf_attn_bwd(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                 const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                 const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch, int64_t bias_batch,
                 void* dq, void* dk, void* dv, float* dbias, float* delta, void* workspace, int64_t workspace_bytes,
                 int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale, void* stream) {
  return tpf_attn_bwd_stages(q, k, v, d_out, q_strides, k_strides, v_strides, out, lse, mask, mask_pitch, bias,
                             bias_pitch, bias_batch, dq, dk, dv, dbias, delta, workspace, workspace_bytes, B, O, H, N,
                             D, scale, TPF_ATTN_BWD_STAGE_ALL, stream);
}

int tpf_attn_bwd_stages(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                        const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                        const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch,
                        int64_t bias_batch, void* dq, void* dk, void* dv, float* dbias, float* delta, void* workspace,
                        int64_t workspace_bytes, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D, float scale,
                        int stages, void* stream) {
  TPF_REQUIRE(stages > 0 && stages <= TPF_ATTN_BWD_STAGE_ALL, TPF_ERR_INVALID_ARGUMENT,
              "tpf_attn_bwd_stages: stages must be a non-empty mask of TPF_ATTN_BWD_STAGE_*");
  TPF_REQUIRE(q_strides && k_strides && v_strides, TPF_ERR_INVALID_ARGUMENT, "tpf_attn_bwd: stride arrays are NULL");
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, TPF_ERR_INVALID_ARGUMENT,
              "tpf_attn_bwd: workspace must be 256-byte aligned");
  TPF_REQUIRE(B > 0 && O > 0 && H > 0 && N > 0 && (bias_batch == 1 || bias_batch == B), TPF_ERR_INVALID_ARGUMENT,
              "tpf_attn_bwd: bad extents");
  const int64_t ws_a = round_up_256(tpf::attn_bwd_workspace_bytes(B, O, H, N, D));
  const int64_t ws_b = round_up_256(tpf::attn_dbias_workspace_bytes(B, O, H, N, bias_batch));
  TPF_REQUIRE(workspace_bytes >= ws_a + ws_b && (ws_a + ws_b == 0 || workspace), TPF_ERR_WORKSPACE,
              "tpf_attn_bwd: workspace of %lld bytes required, %lld given", (long long)(ws_a + ws_b),
              (long long)workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = TPF_OK;
  if (stages & (TPF_ATTN_BWD_STAGE_DELTA | TPF_ATTN_BWD_STAGE_DQKV))
    rc = tpf::attn_bwd_dqkv(q, k, v, d_out, q_strides, k_strides, v_strides, out, lse, mask, mask_pitch, bias,
                            bias_pitch, bias_batch, dq, dk, dv, delta, workspace, ws_a, B, O, H, N, D, scale,
                            stages & 3, st);
  if (rc) return rc;
  if (!(stages & TPF_ATTN_BWD_STAGE_DBIAS)) return TPF_OK;
  return tpf::attn_bwd_dbias(q, k, v, d_out, q_strides, k_strides, v_strides, lse, delta, mask, mask_pitch, bias,
                             bias_pitch, bias_batch, dbias, static_cast<char*>(workspace) + ws_a, ws_b, B, O, H, N, D,
                             scale, st);
}

int64_t tpf_attn_bwd_static_scratch_capacity(void) { return tpf::attn_bwd_static_scratch_capacity(); }

int tpf_attn_bwd_static_scratch(const void* q, const void* k, const void* v, const void* d_out,
                                const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                const void* out, const float* lse, const float* mask, int64_t mask_pitch,
                                const void* bias, int64_t bias_pitch, int64_t bias_batch, void* dq, void* dk, void* dv,
                                float* dbias, float* delta, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
                                float scale, void* stream) {
  TPF_REQUIRE(q_strides && k_strides && v_strides, TPF_ERR_INVALID_ARGUMENT,
              "tpf_attn_bwd_static_scratch: stride arrays are NULL");
  return tpf::attn_bwd_static_scratch(q, k, v, d_out, q_strides, k_strides, v_strides, out, lse, mask, mask_pitch,
                                      bias, bias_pitch, bias_batch, dq, dk, dv, dbias, delta, B, O, H, N, D, scale,
                                      static_cast<cudaStream_t>(stream));
}

static bool trimul_shape_ok(int64_t B, int64_t N, int64_t C) {
  return B > 0 && N > 0 && (C == 32 || C == 64 || C == 96 || C == 128);
}

int64_t tpf_trimul_fwd_workspace_bytes(int64_t B, int64_t N, int64_t C) {
  return trimul_shape_ok(B, N, C) ? tpf::trimul_fwd_workspace_bytes(B, N, C) : 0;
}

int64_t tpf_trimul_bwd_workspace_bytes(int64_t B, int64_t N, int64_t C) {
  return trimul_shape_ok(B, N, C) ? tpf::trimul_bwd_workspace_bytes(B, N * N, C) : 0;
}

int64_t tpf_trimul_bwd_stages_workspace_bytes(int64_t B, int64_t rows_per_batch, int64_t C) {
  return (trimul_shape_ok(B, 8, C) && rows_per_batch > 0) ? tpf::trimul_bwd_workspace_bytes(B, rows_per_batch, C) : 0;
}

int tpf_trimul_fwd_stages(const void* z, const float* mask, const float* p_in, const float* g_in, const float* p_out,
                          const float* g_out, const float* norm_in_w, const float* norm_in_b, const float* norm_out_w,
                          const float* norm_out_b, int direction, int64_t B, int64_t N, int64_t C, void* out, void* zln,
                          float* mean_in, float* rstd_in, void* a_cm, void* b_cm, void* gate, void* x_cm, void* xln,
                          float* mean_out, float* rstd_out, void* workspace, int64_t workspace_bytes,
                          int64_t rows_per_batch, int stages, void* stream) {
  TPF_REQUIRE(direction == 0 || direction == 1, TPF_ERR_INVALID_ARGUMENT,
              "tpf_trimul_fwd: direction must be 0 (outgoing) or 1 (incoming)");
  return tpf::trimul_fwd(z, mask, p_in, g_in, p_out, g_out, norm_in_w, norm_in_b, norm_out_w, norm_out_b, direction, B,
                         N, C, out, zln, mean_in, rstd_in, a_cm, b_cm, gate, x_cm, xln, mean_out, rstd_out, workspace,
                         workspace_bytes, rows_per_batch, stages, static_cast<cudaStream_t>(stream));
}

int tpf_trimul_fwd(const void* z, const float* mask, const float* p_in, const float* g_in, const float* p_out,
                   const float* g_out, const float* norm_in_w, const float* norm_in_b, const float* norm_out_w,
                   const float* norm_out_b, int direction, int64_t B, int64_t N, int64_t C, void* out, void* zln,
                   float* mean_in, float* rstd_in, void* a_cm, void* b_cm, void* gate, void* x_cm, void* xln,
                   float* mean_out, float* rstd_out, void* workspace, int64_t workspace_bytes, void* stream) {
  return tpf_trimul_fwd_stages(z, mask, p_in, g_in, p_out, g_out, norm_in_w, norm_in_b, norm_out_w, norm_out_b,
                               direction, B, N, C, out, zln, mean_in, rstd_in, a_cm, b_cm, gate, x_cm, xln, mean_out,
                               rstd_out, workspace, workspace_bytes, 0, 7, stream);
}

int tpf_trimul_bwd_stages(const void* d_out, const void* z, const float* mask, const float* p_in, const float* g_in,
                          const float* p_out, const float* g_out, const float* norm_in_w, const float* norm_out_w,
                          int direction, int64_t B, int64_t N, int64_t C, const void* out, const void* zln,
                          const float* mean_in, const float* rstd_in, const void* a_cm, const void* b_cm,
                          const void* gate, const void* x_cm, const void* xln, const float* mean_out,
                          const float* rstd_out, void* d_z, float* d_p_in, float* d_g_in, float* d_p_out,
                          float* d_g_out, float* d_norm_in_w, float* d_norm_in_b, float* d_norm_out_w,
                          float* d_norm_out_b, void* workspace, int64_t workspace_bytes, int64_t rows_per_batch,
                          int stages, void* dx_cm, void* da_cm, void* db_cm, void* stream) {
  TPF_REQUIRE(direction == 0 || direction == 1, TPF_ERR_INVALID_ARGUMENT,
              "tpf_trimul_bwd: direction must be 0 (outgoing) or 1 (incoming)");
  return tpf::trimul_bwd(d_out, z, mask, p_in, g_in, p_out, g_out, norm_in_w, norm_out_w, direction, B, N, C, out, zln,
                         mean_in, rstd_in, a_cm, b_cm, gate, x_cm, xln, mean_out, rstd_out, d_z, d_p_in, d_g_in,
                         d_p_out, d_g_out, d_norm_in_w, d_norm_in_b, d_norm_out_w, d_norm_out_b, workspace,
                         workspace_bytes, rows_per_batch, stages, dx_cm, da_cm, db_cm,
                         static_cast<cudaStream_t>(stream));
}

int tpf_trimul_bwd(const void* d_out, const void* z, const float* mask, const float* p_in, const float* g_in,
                   const float* p_out, const float* g_out, const float* norm_in_w, const float* norm_out_w,
                   int direction, int64_t B, int64_t N, int64_t C, const void* out, const void* zln,
                   const float* mean_in, const float* rstd_in, const void* a_cm, const void* b_cm, const void* gate,
                   const void* x_cm, const void* xln, const float* mean_out, const float* rstd_out, void* d_z,
                   float* d_p_in, float* d_g_in, float* d_p_out, float* d_g_out, float* d_norm_in_w,
                   float* d_norm_in_b, float* d_norm_out_w, float* d_norm_out_b, void* workspace,
                   int64_t workspace_bytes, void* stream) {
  return tpf_trimul_bwd_stages(d_out, z, mask, p_in, g_in, p_out, g_out, norm_in_w, norm_out_w, direction, B, N, C, out,
                               zln, mean_in, rstd_in, a_cm, b_cm, gate, x_cm, xln, mean_out, rstd_out, d_z, d_p_in,
                               d_g_in, d_p_out, d_g_out, d_norm_in_w, d_norm_in_b, d_norm_out_w, d_norm_out_b,
                               workspace, workspace_bytes, 0, 7, nullptr, nullptr, nullptr, stream);
}

}  // extern "C"
