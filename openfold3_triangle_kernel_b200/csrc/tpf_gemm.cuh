// Persistent, warp-specialised tcgen05 GEMM engine for sm_100a.
//
//   D[b][m][n] = sum_k A[b][m][k] * B[b][n][k]        (bf16 x bf16 -> fp32 in TMEM)
//
// One CTA per SM walks a static list of (batch, m-tile, n-tile) output tiles.
//   warp 0      : TMA producer  (one elected lane) - STAGES-deep smem ring
//   warp 1      : UMMA issuer   (one elected lane) - accumulators double-buffered in TMEM
//   warps 2..   : epilogue      (8 or 16 warps: two or four per 32 TMEM lanes = rows; they
//                               interleave 32-column chunks)
// Either operand may be K-major (k contiguous in memory) or MN-major (m / n
// contiguous); the shared-memory tiles are written by TMA in the swizzled
// canonical layouts the UMMA descriptors describe, so no thread touches them.
//
// The epilogue is a functor; the TriMul stages plug their fused epilogues in.
#pragma once

#include "tpf_ptx.cuh"

namespace tpf {

struct GemmShape {
  int M, N, K;
  int batch;        // number of independent problems, or number of K splits
  int k_per_split;  // 0: `batch` indexes the tensors' outer dim; >0: split-K, tile b covers
                    // k in [b*k_per_split, (b+1)*k_per_split) of ONE problem
};

template <int BM_, int BN_, int SWZ_A_, bool A_MN_, int SWZ_B_, bool B_MN_, int STAGES_, int EPI_WARPS_ = 8>
struct GemmCfg {
  static constexpr int BM = BM_, BN = BN_, SWZ_A = SWZ_A_, SWZ_B = SWZ_B_, STAGES = STAGES_;
  static constexpr bool A_MN = A_MN_, B_MN = B_MN_;
  static constexpr int EPI_WARPS = EPI_WARPS_;          // 8 or 16: warps per TMEM lane quarter x 4
  static constexpr int EPI_PER_Q = EPI_WARPS / 4;       // warps sharing one lane quarter; they interleave 32-column chunks
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int BK_A = A_MN ? 64 : SWZ_A / 2;
  static constexpr int BK_B = B_MN ? 64 : SWZ_B / 2;
  static constexpr int BK = BK_A < BK_B ? BK_A : BK_B;  // k elements per pipeline stage
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int CHUNK_A = SWZ_A / 2;  // MN-major: elements per swizzle row
  static constexpr int CHUNK_B = SWZ_B / 2;
  static constexpr int ACC_STRIDE = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;  // TMEM columns per accumulator
  static constexpr int TMEM_COLS = 2 * ACC_STRIDE;  // two accumulators; power of two >= 32
  static constexpr int SMEM_BYTES = STAGES * (A_BYTES + B_BYTES) + 256 + 1024;
  static_assert(EPI_WARPS == 8 || EPI_WARPS == 16, "epilogue warps");
  static_assert(BM == 128, "UMMA tile M is 128 (one TMEM lane per row)");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
  static_assert(TMEM_COLS == 32 || TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512,
                "TMEM allocation must be a power of two >= 32");
  static_assert(BN % 32 == 0, "the epilogue walks 32 accumulator columns at a time");
  static_assert(A_BYTES % 1024 == 0 && B_BYTES % 1024 == 0, "stage buffers keep 1024-byte alignment");
};

// ---- per-warp staging of a 32 x 32 bf16 block --------------------------------------------------
// In the epilogue lane = accumulator row, so a lane holds 32 consecutive columns (64 bytes) of its
// row.  Stored straight from the registers, one 16-byte store instruction touches 32 different
// rows: 32 memory transactions that each fill half a sector.  Staged through a 2 KiB per-warp
// shared-memory tile (16-byte pieces XOR-swizzled so that both phases are bank-conflict free),
// every store instruction covers 8 rows x 64 contiguous bytes.
__device__ __forceinline__ void warp_tile_put(uint8_t* tile, int lane, const uint32_t (&pk)[16]) {
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    *reinterpret_cast<uint4*>(tile + lane * 64 + ((i ^ sw) << 4)) =
        make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
}
__device__ __forceinline__ uint4 warp_tile_get(const uint8_t* tile, int row, int piece) {
  return *reinterpret_cast<const uint4*>(tile + row * 64 + ((piece ^ ((row >> 1) & 3)) << 4));
}
// row_ptr(r) -> address of the first of row r's 32 columns (16-byte aligned), or nullptr to skip the row.
// All 32 lanes must call this together.
template <class RowPtr>
__device__ __forceinline__ void warp_tile_store(uint8_t* tile, int lane, const uint32_t (&pk)[16], RowPtr row_ptr) {
  warp_tile_put(tile, lane, pk);
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = 8 * i + (lane >> 2), piece = lane & 3;
    __nv_bfloat16* dst = row_ptr(r);
    if (dst != nullptr) *reinterpret_cast<uint4*>(dst + 8 * piece) = warp_tile_get(tile, r, piece);
  }
  __syncwarp();
}

// Plain stores.  OutT = __nv_bfloat16 or float; row-major D[b][m][n] with leading dimension ldd.
template <typename OutT>
struct EpiStore {
  struct Params {
    OutT* D;
    int64_t ldd;
    int64_t batch_stride;
  };
  static constexpr bool kPaired = false;
  static constexpr bool kStaged = false;
  static constexpr int kSmemPerWarp = sizeof(OutT) == 2 ? 2048 : 0;  // bytes of per-warp epilogue scratch
  // Global-memory operands of the epilogue, requested before the accumulator wait so that their
  // latency hides behind the UMMAs instead of stalling the (few) epilogue warps chunk by chunk.
  struct Pre {};
  __device__ static __forceinline__ void prefetch(const Params&, const GemmShape&, int, int, int, int, Pre&) {}
  __device__ static __forceinline__ void apply(const Params& p, const GemmShape& sh, int b, int m, int n0,
                                               const float (&v)[32], float* wsm, int lane, const Pre&) {
    OutT* blk = p.D + (int64_t)b * p.batch_stride + n0;  // column n0 of row 0
    if constexpr (sizeof(OutT) == 2) {
      // warp-uniform test: whole 32-column block inside N and every row 16-byte aligned
      if (n0 + 32 <= sh.N && (p.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(blk) & 15) == 0) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
        const int m_base = m - lane;
        warp_tile_store(reinterpret_cast<uint8_t*>(wsm), lane, pk, [&](int r) -> __nv_bfloat16* {
          return m_base + r < sh.M ? blk + (int64_t)(m_base + r) * p.ldd : nullptr;
        });
        return;
      }
    }
    if (m >= sh.M) return;
    OutT* row = blk + (int64_t)m * p.ldd;
    if (sizeof(OutT) == 4 && n0 + 32 <= sh.N && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        reinterpret_cast<float4*>(row)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (n0 + i < sh.N) row[i] = static_cast<OutT>(v[i]);
    }
  }
};

template <class Cfg, class Epi>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmShape sh, const typename Epi::Params ep, int* __restrict__ status) {
  griddep_wait();
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint8_t* sA = smem;
  uint8_t* sB = smem + Cfg::STAGES * Cfg::A_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES));
  uint64_t* empty = full + Cfg::STAGES;
  uint64_t* tfull = empty + Cfg::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};
  // per-warp epilogue scratch (only when the epilogue asks for it) sits behind the 256-byte barrier block
  uint8_t* epi_smem = smem + Cfg::STAGES * (Cfg::A_BYTES + Cfg::B_BYTES) + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int mt = (sh.M + Cfg::BM - 1) / Cfg::BM;
  const int nt = (sh.N + Cfg::BN - 1) / Cfg::BN;
  const int tiles = sh.batch * mt * nt;
  const int k_len = sh.k_per_split > 0 ? sh.k_per_split : sh.K;
  const int kb_count = (k_len + Cfg::BK - 1) / Cfg::BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], Cfg::EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 1;
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int b = t / (mt * nt);
        const int r = t - b * (mt * nt);
        const int m0 = (r / nt) * Cfg::BM;
        const int n0 = (r % nt) * Cfg::BN;
        const int kbase = sh.k_per_split > 0 ? b * sh.k_per_split : 0;
        const int bc = sh.k_per_split > 0 ? 0 : b;
        for (int kb = 0; kb < kb_count; ++kb) {
          mbar_wait(&empty[s], ph, wctx);
          mbar_expect_tx(&full[s], Cfg::A_BYTES + Cfg::B_BYTES);
          const int k0 = kbase + kb * Cfg::BK;
          uint8_t* a_dst = sA + s * Cfg::A_BYTES;
          uint8_t* b_dst = sB + s * Cfg::B_BYTES;
          if constexpr (!Cfg::A_MN) {
            tma_load_3d(a_dst, &tmA, &full[s], k0, m0, bc);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BM / Cfg::CHUNK_A; ++c)
              tma_load_3d(a_dst + c * Cfg::BK * Cfg::SWZ_A, &tmA, &full[s], m0 + c * Cfg::CHUNK_A, k0, bc);
          }
          if constexpr (!Cfg::B_MN) {
            tma_load_3d(b_dst, &tmB, &full[s], k0, n0, bc);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::BN / Cfg::CHUNK_B; ++c)
              tma_load_3d(b_dst + c * Cfg::BK * Cfg::SWZ_B, &tmB, &full[s], n0 + c * Cfg::CHUNK_B, k0, bc);
          }
          if (++s == Cfg::STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(Cfg::BM, Cfg::BN, Cfg::A_MN, Cfg::B_MN);
      constexpr uint32_t sw_a = swizzle_mode_for_bytes(Cfg::SWZ_A);
      constexpr uint32_t sw_b = swizzle_mode_for_bytes(Cfg::SWZ_B);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 1;
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        mbar_wait(&tempty[acc], acc_ph, wctx);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        for (int kb = 0; kb < kb_count; ++kb) {
          mbar_wait(&full[s], ph, wctx);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * Cfg::A_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * Cfg::B_BYTES);
#pragma unroll
          for (int j = 0; j < Cfg::BK / 16; ++j) {
            const uint64_t ad = Cfg::A_MN ? make_smem_desc(a_addr + j * 16 * Cfg::SWZ_A, Cfg::BK * Cfg::SWZ_A,
                                                           8 * Cfg::SWZ_A, sw_a)
                                          : make_smem_desc(a_addr + j * 32, 16, 8 * Cfg::SWZ_A, sw_a);
            const uint64_t bd = Cfg::B_MN ? make_smem_desc(b_addr + j * 16 * Cfg::SWZ_B, Cfg::BK * Cfg::SWZ_B,
                                                           8 * Cfg::SWZ_B, sw_b)
                                          : make_smem_desc(b_addr + j * 32, 16, 8 * Cfg::SWZ_B, sw_b);
            umma_ss(d_tmem, ad, bd, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          if (++s == Cfg::STAGES) {
            s = 0;
            ph ^= 1;
          }
        }
        umma_commit(&tfull[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_ph ^= 1;
        }
      }
    }
  } else {
    // epilogue warps: EPI_PER_Q per TMEM lane quarter; they interleave 32-column chunks.
    // The epilogue's global-memory operands of tile t + 1 are requested while tile t is still being
    // worked on (the accumulators are usually ready long before the epilogue gets to them, so a request
    // made only at the top of a tile would expose the whole DRAM latency once per tile).
    const int lane_base = 32 * (warp & 3);
    const int chunk_par = (warp - 2) >> 2;
    float* wsm = reinterpret_cast<float*>(epi_smem + (warp - 2) * Epi::kSmemPerWarp);
    int acc = 0;
    uint32_t acc_ph = 0;
    constexpr int NCH = Epi::kPaired ? (Cfg::BN / 64 + Cfg::EPI_PER_Q - 1) / Cfg::EPI_PER_Q
                                     : (Cfg::BN / 32 + Cfg::EPI_PER_Q - 1) / Cfg::EPI_PER_Q;
    auto request = [&](int t, typename Epi::Pre (&pre)[NCH]) {
      const int b = t / (mt * nt);
      const int r = t - b * (mt * nt);
      const int m = (r / nt) * Cfg::BM + lane_base + lane;
      const int n0 = (r % nt) * Cfg::BN;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
        if constexpr (!Epi::kPaired) {
          if (c < Cfg::BN && n0 + c < sh.N) Epi::prefetch(ep, sh, b, m, n0 + c, lane, pre[k]);
        } else {
          if (c < Cfg::BN / 2) Epi::prefetch2(ep, sh, b, m, n0, c, lane, pre[k]);
        }
      }
    };
    typename Epi::Pre pre[NCH];
    if ((int)blockIdx.x < tiles) request(blockIdx.x, pre);
    for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
      const int b = t / (mt * nt);
      const int r = t - b * (mt * nt);
      const int m0 = (r / nt) * Cfg::BM;
      const int n0 = (r % nt) * Cfg::BN;
      const uint32_t t_acc = tmem_addr(tmem_base, lane_base, acc * Cfg::ACC_STRIDE);
      const int m = m0 + lane_base + lane;
      typename Epi::Pre nxt[NCH];
      mbar_wait(&tfull[acc], acc_ph, wctx);
      tc_fence_after();
      if constexpr (!Epi::kPaired) {
        uint32_t raw[NCH][32];
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN) tmem_ld32(t_acc + c, raw[k]);
        }
        if (t + (int)gridDim.x < tiles) request(t + gridDim.x, nxt);
        tmem_ld_wait();
        // the accumulator now lives in registers: hand the TMEM buffer back before the epilogue math
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN && n0 + c < sh.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[k][i]);
            Epi::apply(ep, sh, b, m, n0 + c, v, wsm, lane, pre[k]);
          }
        }
      } else {
        // Column c (first half of the tile) pairs with column c + BN/2.
        uint32_t raw0[NCH][32], raw1[NCH][32];
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN / 2) {
            tmem_ld32(t_acc + c, raw0[k]);
            tmem_ld32(t_acc + Cfg::BN / 2 + c, raw1[k]);
          }
        }
        // an epilogue that parks its operands in shared memory does so before the next tile's are requested,
        // so that both sets never hold registers at the same time
        if constexpr (Epi::kStaged && NCH == 1) Epi::stage(pre[0], wsm, lane);
        if (t + (int)gridDim.x < tiles) request(t + gridDim.x, nxt);
        tmem_ld_wait();
        // the accumulator now lives in registers: hand the TMEM buffer back before the epilogue math
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN / 2) {
            if constexpr (Epi::kStaged && NCH > 1) Epi::stage(pre[k], wsm, lane);
            float v0[32], v1[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              v0[i] = __uint_as_float(raw0[k][i]);
              v1[i] = __uint_as_float(raw1[k][i]);
            }
            Epi::apply2(ep, sh, b, m, n0, c, v0, v1, wsm, lane, pre[k]);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < NCH; ++k) pre[k] = nxt[k];
      if (++acc == 2) {
        acc = 0;
        acc_ph ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace tpf
