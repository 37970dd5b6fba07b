// Host-side launch helpers for the tcgen05 GEMM engine (tpf_gemm.cuh).
#pragma once

#include "tpf_gemm.cuh"
#include "tpf_host.cuh"

namespace tpf {

// Tensor map for one GEMM operand.  K-major: memory [batch][mn][k]; MN-major: memory [batch][k][mn].
inline int make_operand_tmap(CUtensorMap* tm, const void* base, bool mn_major, int64_t mn, int64_t k, int64_t ld,
                      int64_t batch, int64_t batch_stride, int swz, int tile_mn, int bk) {
  uint64_t dims[3];
  uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)(batch_stride ? batch_stride : 8) * 2};
  uint32_t box[3];
  if (!mn_major) {
    dims[0] = (uint64_t)k; dims[1] = (uint64_t)mn; dims[2] = (uint64_t)batch;
    box[0] = (uint32_t)bk; box[1] = (uint32_t)tile_mn; box[2] = 1;
  } else {
    dims[0] = (uint64_t)mn; dims[1] = (uint64_t)k; dims[2] = (uint64_t)batch;
    box[0] = (uint32_t)(swz / 2); box[1] = (uint32_t)bk; box[2] = 1;
  }
  return make_tmap_bf16(tm, base, 3, dims, strides, box, swz);
}

template <class Cfg, class Epi>
int launch_gemm(const void* A, int64_t lda, int64_t bsa, const void* B, int64_t ldb, int64_t bsb,
                const GemmShape& sh, const typename Epi::Params& ep, int* status, cudaStream_t stream,
                int max_ctas = 0) {
  CUtensorMap tmA, tmB;
  const int64_t tensor_batch = sh.k_per_split > 0 ? 1 : sh.batch;
  int rc = make_operand_tmap(&tmA, A, Cfg::A_MN, sh.M, sh.K, lda, tensor_batch, bsa, Cfg::SWZ_A, Cfg::BM, Cfg::BK);
  if (rc) return rc;
  rc = make_operand_tmap(&tmB, B, Cfg::B_MN, sh.N, sh.K, ldb, tensor_batch, bsb, Cfg::SWZ_B, Cfg::BN, Cfg::BK);
  if (rc) return rc;
  auto kern = gemm_umma_kernel<Cfg, Epi>;
  constexpr int smem_bytes = Cfg::SMEM_BYTES + Cfg::EPI_WARPS * Epi::kSmemPerWarp;
  static_assert(smem_bytes <= 232448, "shared memory budget");
  static PerDeviceOnce once;  // per instantiation
  if ((rc = ensure_dynamic_smem(kern, smem_bytes, once))) return rc;
  const int mt = (sh.M + Cfg::BM - 1) / Cfg::BM, nt = (sh.N + Cfg::BN - 1) / Cfg::BN;
  const int tiles = sh.batch * mt * nt;
  int grid = sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  if (grid > tiles) grid = tiles;
  if (grid < 1) return TPF_OK;
  if constexpr (Cfg::STAT != 0) {
    const int k_len = sh.k_per_split > 0 ? sh.k_per_split : sh.K;
    TPF_REQUIRE(k_len <= Cfg::STAT_KB * Cfg::BK, TPF_ERR_UNSUPPORTED,
                "gemm: K = %d exceeds the stationary operand buffer (%d)", k_len, Cfg::STAT_KB * Cfg::BK);
    const int per = (tiles + grid - 1) / grid;  // contiguous tiles per CTA; CTAs that would get none are not launched
    grid = (tiles + per - 1) / per;
  }
  launch_kernel(kern, dim3(grid), dim3(Cfg::THREADS), smem_bytes, stream, tmA, tmB, sh, ep, status);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

}  // namespace tpf
