// Batched bf16 GEMM on the tcgen05 engine: D[b] = A[b] * B[b]^T with either
// operand K-major or MN-major.  This is the TriMul k-contraction
// (reference: torch.bmm at turbopairformer_trimul.py:244-249 and :357-362) and
// the building block the other TriMul GEMM stages reuse with fused epilogues.
#include "tpf_gemm_host.cuh"

namespace tpf {

static __device__ int g_bmm_status;

int bmm_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  TPF_CUDA_OK(cudaMemcpyFromSymbol(&v, g_bmm_status, sizeof(int)));
  if (v) TPF_CUDA_OK(cudaMemcpyToSymbol(g_bmm_status, &zero, sizeof(int)));
  *out = v;
  return TPF_OK;
}

template <int SWZ, bool A_MN, bool B_MN, typename OutT>
int bmm_dispatch(const void* A, int64_t lda, int64_t bsa, const void* B, int64_t ldb, int64_t bsb, void* D,
                 int64_t ldd, int64_t bsd, const GemmShape& sh, int* status, cudaStream_t stream) {
  constexpr int kBK = (A_MN && B_MN) ? 64 : SWZ / 2;
  constexpr int kStages = (196608 / (256 * kBK * 2)) > 8 ? 8 : (196608 / (256 * kBK * 2));
  using Cfg = GemmCfg<128, 128, SWZ, A_MN, SWZ, B_MN, kStages>;
  using Epi = EpiStore<OutT>;
  typename Epi::Params ep{reinterpret_cast<OutT*>(D), ldd, bsd};
  return launch_gemm<Cfg, Epi>(A, lda, bsa, B, ldb, bsb, sh, ep, status, stream);
}

int bmm_bf16(const void* A, int64_t lda, int64_t bsa, int a_mn, const void* B, int64_t ldb, int64_t bsb, int b_mn,
             void* D, int64_t ldd, int64_t bsd, int out_f32, int64_t M, int64_t N, int64_t K, int64_t batch,
             int64_t k_per_split, int swizzle_bytes, cudaStream_t stream) {
  TPF_REQUIRE(A && B && D, TPF_ERR_INVALID_ARGUMENT, "bmm: null pointer");
  TPF_REQUIRE(M > 0 && N > 0 && K > 0 && batch > 0, TPF_ERR_INVALID_ARGUMENT, "bmm: M,N,K,batch must be positive");
  TPF_REQUIRE(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && batch < (1ll << 31),
              TPF_ERR_INVALID_ARGUMENT, "bmm: extent too large");
  TPF_REQUIRE(lda % 8 == 0 && ldb % 8 == 0 && bsa % 8 == 0 && bsb % 8 == 0, TPF_ERR_INVALID_ARGUMENT,
              "bmm: leading dimensions and batch strides must be multiples of 8 elements (16 bytes)");
  TPF_REQUIRE(k_per_split >= 0 && k_per_split % 64 == 0, TPF_ERR_INVALID_ARGUMENT,
              "bmm: k_per_split must be a non-negative multiple of 64");
  GemmShape sh{(int)M, (int)N, (int)K, (int)batch, (int)k_per_split};
  int* status = nullptr;
  {
    static PerDeviceAddress cache;
    if (int rc = device_symbol_address(g_bmm_status, cache, reinterpret_cast<void**>(&status))) return rc;
  }
#define TPF_BMM_CASE(SWZ, AM, BM)                                                                              \
  if (swizzle_bytes == SWZ && (a_mn != 0) == AM && (b_mn != 0) == BM)                                          \
    return out_f32 ? bmm_dispatch<SWZ, AM, BM, float>(A, lda, bsa, B, ldb, bsb, D, ldd, bsd, sh, status, stream) \
                   : bmm_dispatch<SWZ, AM, BM, __nv_bfloat16>(A, lda, bsa, B, ldb, bsb, D, ldd, bsd, sh, status, \
                                                              stream);
  TPF_BMM_CASE(128, false, false)
  TPF_BMM_CASE(128, true, true)
  TPF_BMM_CASE(128, true, false)
  TPF_BMM_CASE(128, false, true)
  TPF_BMM_CASE(64, false, false)
  TPF_BMM_CASE(64, true, true)
  TPF_BMM_CASE(32, false, false)
  TPF_BMM_CASE(32, true, true)
#undef TPF_BMM_CASE
  return fail(TPF_ERR_UNSUPPORTED, "bmm: unsupported (swizzle=%d, a_mn=%d, b_mn=%d)", swizzle_bytes, a_mn, b_mn);
}

}  // namespace tpf
