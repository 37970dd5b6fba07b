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

// STAT_: 0 = both operands stream through the stage ring; 1 = the A tile, 2 = the B tile is *stationary*:
// its whole K extent (at most STAT_KB_ k-blocks) is loaded once into a buffer of its own and kept for the
// run of consecutive tiles that share it, while only the other operand streams.  Tiles are then numbered
// so that such runs are long (the streamed operand's tile index runs fastest) and every CTA takes one
// contiguous range of them.  Without this every tile re-fetches both operands from L2, and with a short
// K that traffic, not the tensor pipe, bounds the kernel.
template <int BM_, int BN_, int SWZ_A_, bool A_MN_, int SWZ_B_, bool B_MN_, int STAGES_, int EPI_WARPS_ = 8,
          int STAT_ = 0, int STAT_KB_ = 0>
struct GemmCfg {
  static constexpr int BM = BM_, BN = BN_, SWZ_A = SWZ_A_, SWZ_B = SWZ_B_, STAGES = STAGES_;
  static constexpr bool A_MN = A_MN_, B_MN = B_MN_;
  static constexpr int STAT = STAT_, STAT_KB = STAT_KB_;
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
  static constexpr int STAT_BYTES = STAT == 1 ? STAT_KB * A_BYTES : STAT == 2 ? STAT_KB * B_BYTES : 0;
  static constexpr int STAGE_A = STAT == 1 ? 0 : A_BYTES;  // bytes of each operand in one ring stage
  static constexpr int STAGE_B = STAT == 2 ? 0 : B_BYTES;
  static constexpr int STAGE_BYTES = STAGE_A + STAGE_B;
  static constexpr int SMEM_BYTES = STAT_BYTES + STAGES * STAGE_BYTES + 256 + 1024;
  static_assert(STAT >= 0 && STAT <= 2 && (STAT == 0 || STAT_KB > 0), "stationary operand");
  static_assert(EPI_WARPS == 8 || EPI_WARPS == 16, "epilogue warps");
  static_assert(BM == 128, "UMMA tile M is 128 (one TMEM lane per row)");
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "UMMA N");
  static_assert(TMEM_COLS == 32 || TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512,
                "TMEM allocation must be a power of two >= 32");
  static_assert(BN % 32 == 0, "the epilogue walks 32 accumulator columns at a time");
  static_assert(A_BYTES % 1024 == 0 && B_BYTES % 1024 == 0, "stage buffers keep 1024-byte alignment");
  static_assert(STAGES <= 8, "barrier block");
};

// The tiles one CTA works on, in order.  Streaming: tile t = blockIdx.x, + gridDim.x, ... with the n index
// fastest.  Stationary operand: one contiguous range of a numbering in which the streamed operand's tile
// index runs fastest; `key` names the stationary tile.  The walk is a mixed-radix counter (batch, slow
// index, fast index) advanced by a fixed step, so the per-tile cost is a few adds: the roles that walk the
// tiles are single threads whose instruction stream is on the critical path of the tensor pipe.
template <class Cfg>
struct TileWalk {
  int r0, r1;          // radices of the fast and the slow digit
  int s0, s1, sb;      // the step, decomposed
  int d0, d1, b;       // current tile
  int count;           // tiles of this CTA
  __device__ TileWalk(const GemmShape& sh) {
    const int mt = (sh.M + Cfg::BM - 1) / Cfg::BM;
    const int nt = (sh.N + Cfg::BN - 1) / Cfg::BN;
    r0 = Cfg::STAT == 2 ? mt : nt;
    r1 = Cfg::STAT == 2 ? nt : mt;
    const int tiles = sh.batch * mt * nt;
    int first, step;
    if constexpr (Cfg::STAT == 0) {
      first = blockIdx.x;
      step = gridDim.x;
      count = first < tiles ? (tiles - first + step - 1) / step : 0;
    } else {
      const int per = (tiles + gridDim.x - 1) / gridDim.x;
      first = blockIdx.x * per;
      step = 1;
      count = first < tiles ? (tiles - first < per ? tiles - first : per) : 0;
    }
    b = first / (r0 * r1);
    int r = first - b * (r0 * r1);
    d1 = r / r0;
    d0 = r - d1 * r0;
    sb = step / (r0 * r1);
    r = step - sb * (r0 * r1);
    s1 = r / r0;
    s0 = r - s1 * r0;
  }
  __device__ __forceinline__ void next() {
    d0 += s0;
    if (d0 >= r0) {
      d0 -= r0;
      ++d1;
    }
    d1 += s1;
    if (d1 >= r1) {
      d1 -= r1;
      ++b;
    }
    b += sb;
  }
  __device__ __forceinline__ int m0() const { return (Cfg::STAT == 2 ? d0 : d1) * Cfg::BM; }
  __device__ __forceinline__ int n0() const { return (Cfg::STAT == 2 ? d1 : d0) * Cfg::BN; }
  __device__ __forceinline__ int key() const { return b * r1 + d1; }  // the slow digit names the stationary tile
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
  uint8_t* st_buf = smem;                      // stationary operand (STAT_BYTES, may be 0)
  uint8_t* ring = smem + Cfg::STAT_BYTES;      // STAGES x [A k-block | B k-block] (a stationary operand takes no room)
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* empty = full + Cfg::STAGES;
  uint64_t* tfull = empty + Cfg::STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* st_full = tempty + 2;   // stationary operand landed
  uint64_t* st_free = st_full + 1;  // every UMMA that reads it has completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(st_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};
  // per-warp epilogue scratch (only when the epilogue asks for it) sits behind the 256-byte barrier block
  uint8_t* epi_smem = ring + Cfg::STAGES * Cfg::STAGE_BYTES + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // A paired epilogue may ask for a tile with the operand roles exchanged (see the UMMA issuer).
  constexpr bool kCanSwap = Epi::kPaired && Cfg::BN == 256 && Cfg::BM == 128 && !Cfg::A_MN && !Cfg::B_MN &&
                            Cfg::SWZ_A == 128 && Cfg::SWZ_B == 128;

  const TileWalk<Cfg> walk(sh);
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
    mbar_init(st_full, 1);
    mbar_init(st_free, 1);
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
      // one k-block of an operand tile -> dst (the swizzled canonical layout the UMMA descriptors describe)
      auto load_a = [&](uint8_t* dst, uint64_t* bar, int k0, int m0, int bc) {
        if constexpr (!Cfg::A_MN) {
          tma_load_3d(dst, &tmA, bar, k0, m0, bc);
        } else {
#pragma unroll
          for (int c = 0; c < Cfg::BM / Cfg::CHUNK_A; ++c)
            tma_load_3d(dst + c * Cfg::BK * Cfg::SWZ_A, &tmA, bar, m0 + c * Cfg::CHUNK_A, k0, bc);
        }
      };
      auto load_b = [&](uint8_t* dst, uint64_t* bar, int k0, int n0, int bc) {
        if constexpr (!Cfg::B_MN) {
          tma_load_3d(dst, &tmB, bar, k0, n0, bc);
        } else {
#pragma unroll
          for (int c = 0; c < Cfg::BN / Cfg::CHUNK_B; ++c)
            tma_load_3d(dst + c * Cfg::BK * Cfg::SWZ_B, &tmB, bar, n0 + c * Cfg::CHUNK_B, k0, bc);
        }
      };
      int s = 0;
      uint32_t ph = 1;
      int cur_key = -1;
      uint32_t free_ph = 0;
      TileWalk<Cfg> w = walk;
      for (int i = 0; i < w.count; ++i, w.next()) {
        const int b = w.b, m0 = w.m0(), n0 = w.n0(), key = w.key();
        const int kbase = sh.k_per_split > 0 ? b * sh.k_per_split : 0;
        const int bc = sh.k_per_split > 0 ? 0 : b;
        if constexpr (Cfg::STAT != 0) {
          if (key != cur_key) {
            if (cur_key != -1) {  // the buffer is still being read by the previous run's UMMAs
              mbar_wait(st_free, free_ph, wctx);
              free_ph ^= 1;
            }
            cur_key = key;
            mbar_expect_tx(st_full, kb_count * (Cfg::STAT == 1 ? Cfg::A_BYTES : Cfg::B_BYTES));
            for (int kb = 0; kb < kb_count; ++kb) {
              if constexpr (Cfg::STAT == 1) load_a(st_buf + kb * Cfg::A_BYTES, st_full, kbase + kb * Cfg::BK, m0, bc);
              else load_b(st_buf + kb * Cfg::B_BYTES, st_full, kbase + kb * Cfg::BK, n0, bc);
            }
          }
        }
        for (int kb = 0; kb < kb_count; ++kb) {
          mbar_wait(&empty[s], ph, wctx);
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          const int k0 = kbase + kb * Cfg::BK;
          uint8_t* stage = ring + s * Cfg::STAGE_BYTES;
          if constexpr (Cfg::STAT != 1) load_a(stage, &full[s], k0, m0, bc);
          if constexpr (Cfg::STAT != 2) load_b(stage + Cfg::STAGE_A, &full[s], k0, n0, bc);
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
      // base descriptors of the operand area (K-major: 8-row groups SWZ x 8 bytes apart; MN-major: k groups
      // BK x SWZ bytes apart inside a chunk of SWZ / 2 rows)
      const uint64_t a_desc0 = Cfg::A_MN ? make_smem_desc(smem_u32(smem), Cfg::BK * Cfg::SWZ_A, 8 * Cfg::SWZ_A, sw_a)
                                         : make_smem_desc(smem_u32(smem), 16, 8 * Cfg::SWZ_A, sw_a);
      const uint64_t b_desc0 = Cfg::B_MN ? make_smem_desc(smem_u32(smem), Cfg::BK * Cfg::SWZ_B, 8 * Cfg::SWZ_B, sw_b)
                                         : make_smem_desc(smem_u32(smem), 16, 8 * Cfg::SWZ_B, sw_b);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      uint32_t acc_ph = 1;
      int cur_key = -1;
      uint32_t stat_ph = 0;
      TileWalk<Cfg> w = walk;
      // A barrier probe by this thread takes a few hundred cycles to answer even when the phase completed long
      // ago (its shared-memory operations queue behind the epilogue warps'), so every barrier is probed one step
      // early: the answer arrives while the UMMAs of the step before are being issued, and the blocking wait is
      // only the fallback.
      bool full_ready = false, acc_ready = false;
      if (w.count > 0) {
        acc_ready = mbar_test_wait(&tempty[0], 1);
        full_ready = mbar_test_wait(&full[0], 0);
      }
      for (int i = 0; i < w.count; ++i) {
        const int n0 = w.n0(), key = w.key();
        if constexpr (Cfg::STAT != 0) {
          if (key != cur_key) {
            mbar_wait(st_full, stat_ph, wctx);
            stat_ph ^= 1;
            cur_key = key;
          }
        }
        if (!acc_ready) mbar_wait(&tempty[acc], acc_ph, wctx);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_STRIDE;
        bool swap = false;
        if constexpr (kCanSwap) swap = Epi::swapped(ep, n0);
        for (int kb = 0; kb < kb_count; ++kb) {
          if (!full_ready) mbar_wait(&full[s], ph, wctx);
          tc_fence_after();
          // descriptors = a base descriptor + (byte offset >> 4) in the start-address field (no carry out of it:
          // shared memory is far smaller than the field's range)
          const uint32_t a_off = Cfg::STAT == 1 ? kb * Cfg::A_BYTES : Cfg::STAT_BYTES + s * Cfg::STAGE_BYTES;
          const uint32_t b_off = Cfg::STAT == 2 ? kb * Cfg::B_BYTES : Cfg::STAT_BYTES + s * Cfg::STAGE_BYTES + Cfg::STAGE_A;
          const uint64_t ad0 = a_desc0 + (a_off >> 4);
          const uint64_t bd0 = b_desc0 + (b_off >> 4);
          // probed while the UMMAs go out: the stage after this one (it may belong to the next tile) and the
          // accumulator the next tile will use
          const int sn = s + 1 == Cfg::STAGES ? 0 : s + 1;
          const uint32_t phn = s + 1 == Cfg::STAGES ? ph ^ 1 : ph;
          const uint32_t acc_phn = acc == 1 ? acc_ph ^ 1 : acc_ph;
          constexpr int A_STEP = Cfg::A_MN ? (16 * Cfg::SWZ_A >> 4) : 2;
          constexpr int B_STEP = Cfg::B_MN ? (16 * Cfg::SWZ_B >> 4) : 2;
          uint32_t probes = 0;
          bool swapped_now = false;
          if constexpr (kCanSwap) swapped_now = swap;
          if constexpr (Cfg::BK != 64) {
            // narrow swizzle modes (small K): fewer UMMAs per k-block, plain issue, blocking waits
#pragma unroll
            for (int j = 0; j < Cfg::BK / 16; ++j)
              umma_ss(d_tmem, ad0 + j * A_STEP, bd0 + j * B_STEP, idesc, (kb | j) != 0 ? 1u : 0u);
            umma_commit(&empty[s]);
          } else if (swapped_now) {
            // Operand roles exchanged: the two 128-row halves of the B tile are the M operands of two UMMAs
            // that share the A tile as their N operand.  Accumulator lane = row of the B tile (an output
            // column of the problem), accumulator column = row of the A tile; the first half's product sits
            // in columns [0, BM), the second half's in [BN / 2, BN / 2 + BM).
            constexpr uint32_t idesc_sw = make_idesc_bf16(128, Cfg::BM, false, false);
            probes = umma_ss_x4x2_probed<2, (128 * Cfg::SWZ_B >> 4)>(d_tmem, d_tmem + Cfg::BN / 2, bd0, ad0, idesc_sw,
                                                                    kb != 0 ? 1u : 0u, &empty[s], &full[sn], phn,
                                                                    &tempty[acc ^ 1], acc_phn);
          } else {
            probes = umma_ss_x4_probed<A_STEP, B_STEP>(d_tmem, ad0, bd0, idesc, kb != 0 ? 1u : 0u, &empty[s], &full[sn],
                                                       phn, &tempty[acc ^ 1], acc_phn);
          }
          full_ready = (kb + 1 < kb_count || i + 1 < w.count) && (probes & 1u);
          if (kb + 1 == kb_count) acc_ready = i + 1 < w.count && (probes & 2u);
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
        w.next();
        if constexpr (Cfg::STAT != 0) {
          // end of a run: the buffer may be overwritten once everything issued so far has completed
          if (i + 1 == w.count || w.key() != cur_key) umma_commit(st_free);
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
    auto request = [&](const TileWalk<Cfg>& tw, typename Epi::Pre (&pre)[NCH]) {
      const int b = tw.b, m0 = tw.m0(), n0 = tw.n0();
      const int m = m0 + lane_base + lane;
#pragma unroll
      for (int k = 0; k < NCH; ++k) {
        const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
        if constexpr (!Epi::kPaired) {
          if (c < Cfg::BN && n0 + c < sh.N) Epi::prefetch(ep, sh, b, m, n0 + c, lane, pre[k]);
        } else {
          bool swap = false;
          if constexpr (kCanSwap) swap = Epi::swapped(ep, n0);
          if (c < Cfg::BN / 2) Epi::prefetch2(ep, sh, b, m0, lane_base + lane, n0, c, lane, swap, pre[k]);
        }
      }
    };
    typename Epi::Pre pre[NCH];
    TileWalk<Cfg> w = walk;
    if (w.count > 0) request(w, pre);
    for (int i = 0; i < w.count; ++i) {
      const int b = w.b, m0 = w.m0(), n0 = w.n0();
      w.next();  // w now names the next tile (its operands are requested below)
      const uint32_t t_acc = tmem_addr(tmem_base, lane_base, acc * Cfg::ACC_STRIDE);
      typename Epi::Pre nxt[NCH];
      mbar_wait(&tfull[acc], acc_ph, wctx);
      tc_fence_after();
      if constexpr (!Epi::kPaired) {
        const int m = m0 + lane_base + lane;
        uint32_t raw[NCH][32];
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN) tmem_ld32(t_acc + c, raw[k]);
        }
        if (i + 1 < w.count) request(w, nxt);
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
            for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[k][e]);
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
        if (i + 1 < w.count) request(w, nxt);
        tmem_ld_wait();
        // the accumulator now lives in registers: hand the TMEM buffer back before the epilogue math
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        bool swap = false;
        if constexpr (kCanSwap) swap = Epi::swapped(ep, n0);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
          const int c = 32 * (chunk_par + Cfg::EPI_PER_Q * k);
          if (c < Cfg::BN / 2) {
            if constexpr (Epi::kStaged && NCH > 1) Epi::stage(pre[k], wsm, lane);
            float v0[32], v1[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              v0[e] = __uint_as_float(raw0[k][e]);
              v1[e] = __uint_as_float(raw1[k][e]);
            }
            Epi::apply2(ep, sh, b, m0, lane_base + lane, n0, c, v0, v1, wsm, lane, swap, pre[k]);
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
