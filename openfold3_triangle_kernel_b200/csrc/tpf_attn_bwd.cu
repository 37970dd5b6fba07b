// Triangle-attention backward for sm_100a: dQ, dK, dV (this file, kernel 1), the row
// scalar delta (kernel 0) and dBias (kernel 2 + fold).
//
// Reference interface replaced: turbopairformer_triangle_delta_out and
// turbopairformer_triangle_sr_backward_out
// (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_delta.cu:343-414,
//  openfold3/core/kernels/turbopairformer/turbopairformer_triangle_dq_dbias.cu:2526-2648).
// Same math: P = exp(S - lse) (0 where lse = -inf), dP = dO V^T, dS = P (dP - delta),
// dV = P^T dO, dK = scale dS^T Q, dQ = scale dS K, dBias = sum over outer rows of dS; P and dS
// are rounded to bf16 only as UMMA operands, all accumulation is fp32, no atomics anywhere.
//
// Machine mapping (differs from the reference, which keeps 64-key leaves and writes bf16
// dQ partials and dBias leaf planes to HBM):
//  * kernel 1 owns whole (b, o, h) planes.  For each 128x128 (query, key) tile the five GEMMs
//    run on tcgen05; dK/dV of up to KS key tiles and dQ of the current query tile stay in
//    TMEM until complete, so for N <= 128*KS nothing but the final gradients is written.
//    Longer sequences walk key strips and keep a per-CTA fp32 dQ running sum in a small
//    private scratch (same thread, fixed order).
//  * kernel 2 owns a (h, query tile, key tile) of dBias and walks the outer rows, recomputing
//    S and dP (two cheap K = D GEMMs) and summing dS in fp32 registers in ascending o.
//    A few independent o-chunks per tile fill the machine; their partial planes are folded
//    in fixed order by a tiny kernel.
#include <stdlib.h>

#include "tpf_host.cuh"
#include "tpf_ptx.cuh"

namespace tpf {

static __device__ int g_attn_bwd_status;

int attn_bwd_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  TPF_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn_bwd_status, sizeof(int)));
  if (v) TPF_CUDA_OK(cudaMemcpyToSymbol(g_attn_bwd_status, &zero, sizeof(int)));
  *out = v;
  return TPF_OK;
}

static int attn_bwd_status_address(int** out) {
  static PerDeviceAddress cache;
  return device_symbol_address(g_attn_bwd_status, cache, reinterpret_cast<void**>(out));
}

// =============================================================================================
// kernel 0: delta[b,o,h,q] = sum_d dO[b,o,q,h,d] * O[b,o,q,h,d]      (HBM bound)
// =============================================================================================
template <int D>
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ d_out,
                                                         const __nv_bfloat16* __restrict__ out,
                                                         float* __restrict__ delta, int64_t rows, int H, int N) {
  griddep_wait();
  // one thread handles D/8 ... : LANES threads per (b,o,q,h) row of D elements, 8 elements each
  constexpr int LANES = D / 8;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = gid / LANES;  // flat (b,o,q,h)
  const int part = (int)(gid % LANES);
  float acc = 0.f;
  if (r < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(d_out + r * D + part * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(out + r * D + part * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), acc);
      acc = fmaf(__uint_as_float(aw[i] & 0xFFFF0000u), __uint_as_float(bw[i] & 0xFFFF0000u), acc);
    }
  }
#pragma unroll
  for (int off = LANES / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (r < rows && part == 0) {
    const int h = (int)(r % H);
    const int64_t t = r / H;
    const int q = (int)(t % N);
    const int64_t bo = t / N;
    delta[(bo * H + h) * N + q] = acc;
  }
}

// =============================================================================================
// kernel 1: dQ, dK, dV
// =============================================================================================
struct AttnBwdParams {
  __nv_bfloat16 *dq, *dk, *dv;  // [B,O,H,N,D] contiguous
  const float* lse;             // [B,O,H,N]
  const float* delta;           // [B,O,H,N]
  float* dq_scratch;            // per-CTA [N][D] fp32 when the key axis needs several strips
  int B, O, H, N;
  int q_tiles, k_tiles, n_strips;
  int bias_broadcast;
  float scale;
  int n_items;
};

template <int D_>
struct AttnBwdCfg {
  static constexpr int D = D_;
  static constexpr int KS = D <= 32 ? 3 : 1;   // key tiles whose dK/dV stay in TMEM together
  static constexpr int NKV = 2, NQ = 2;
  static constexpr int NB = D <= 32 ? 2 : 1;   // bias stages
  static constexpr int NCW = 16;               // compute warps: four threads per query row, 32 keys each
  static constexpr int THREADS = 32 * (NCW + 2);
  static constexpr int WARP_TMA = NCW, WARP_MMA = NCW + 1;
  static constexpr int SWZ = 2 * D;
  static constexpr int TILE = 128 * D * 2;
  static constexpr int BIAS_STAGE = 32768, PD_BYTES = 32768;
  static constexpr int OFF_BIAS = 0;
  static constexpr int OFF_P = OFF_BIAS + NB * BIAS_STAGE;
  static constexpr int OFF_DS = OFF_P + PD_BYTES;
  static constexpr int OFF_Q = OFF_DS + PD_BYTES;        // [NQ]
  static constexpr int OFF_DO = OFF_Q + NQ * TILE;       // [NQ]
  static constexpr int OFF_K = OFF_DO + NQ * TILE;       // [NKV]
  static constexpr int OFF_V = OFF_K + NKV * TILE;       // [NKV]
  static constexpr int OFF_MASK = OFF_V + NKV * TILE;    // [NKV] x 512
  // two staging tiles through which finished dQ / dK / dV tiles leave as whole, contiguous 128 x D blocks
  // (only where shared memory has room for them; otherwise every thread stores its own piece)
  static constexpr int OFF_STG = OFF_MASK + NKV * 512;
  static constexpr bool STAGED = OFF_STG + 2 * TILE + 1024 + 256 <= 232448 - 1024;
  static constexpr int OFF_BAR = OFF_STG + (STAGED ? 2 * TILE : 0);
  static constexpr int N_BAR = 2 * NB + 2 * NQ + 2 * NKV + 6;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TM_S = 0, TM_DP = 128, TM_DQ = 256, TM_DK = 320, TM_DV = 320 + KS * D;
  static constexpr int TMEM_COLS = 512;
  static_assert(TM_DV + KS * D <= 512, "TMEM budget");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// Walks the (item, strip, query tile, key tile) sequence of one CTA.
struct BwdWalk {
  int n_items, q_tiles, k_tiles, KS, n_strips, step;
  int item, strip, qt, kk;
  __device__ void init(int first, int step_, int n_items_, int q_tiles_, int k_tiles_, int KS_, int n_strips_) {
    n_items = n_items_; q_tiles = q_tiles_; k_tiles = k_tiles_; KS = KS_; n_strips = n_strips_; step = step_;
    item = first; strip = 0; qt = 0; kk = 0;
  }
  __device__ bool valid() const { return item < n_items; }
  __device__ int strip_len() const { return min(KS, k_tiles - strip * KS); }
  __device__ int kt() const { return strip * KS + kk; }
  __device__ bool first_kk() const { return kk == 0; }
  __device__ bool last_kk() const { return kk == strip_len() - 1; }
  __device__ bool first_qt() const { return qt == 0; }
  __device__ bool last_qt() const { return qt == q_tiles - 1; }
  __device__ void next() {
    if (++kk < strip_len()) return;
    kk = 0;
    if (++qt < q_tiles) return;
    qt = 0;
    if (++strip < n_strips) return;
    strip = 0;
    item += step;
  }
};

// Sixteen compute warps: thread (row, part) owns query row `row` (= TMEM lane) and the 32 keys
// [32 part, 32 part + 32) of a 128 x 128 tile.  It walks them 16 columns at a time straight from
// TMEM (S and dP), forms P and dS, and keeps the bf16 results packed in 32 registers; only the
// shared-memory stores wait for the UMMAs of the previous tile to release the P / dS tiles, so
// the arithmetic of tile t+1 overlaps the dV / dK / dQ UMMAs of tile t.
template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmBias, const __grid_constant__ CUtensorMap tmMask,
                const AttnBwdParams p, int* __restrict__ status) {
  griddep_wait();
  constexpr int D = Cfg::D, KS = Cfg::KS, NKV = Cfg::NKV, NQ = Cfg::NQ, NB = Cfg::NB, NCW = Cfg::NCW;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* b_full = bars;
  uint64_t* b_empty = b_full + NB;
  uint64_t* q_full = b_empty + NB;
  uint64_t* q_empty = q_full + NQ;
  uint64_t* kv_full = q_empty + NQ;
  uint64_t* kv_empty = kv_full + NKV;
  uint64_t* misc = kv_empty + NKV;
  uint64_t* sdp_full = misc + 0;   // S and dP of a tile are in TMEM
  uint64_t* sdp_free = misc + 1;   // ... and have been read by all compute warps
  uint64_t* pds_ready = misc + 2;  // P and dS of a tile are in shared memory
  uint64_t* pds_free = misc + 3;   // ... and have been consumed by the dV / dK / dQ UMMAs
  uint64_t* dkv_full = misc + 4;
  uint64_t* dkv_free = misc + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], NCW);
    }
    for (int s = 0; s < NQ; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < NKV; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_free, NCW);
    mbar_init(pds_ready, NCW);
    mbar_init(pds_free, 1);
    mbar_init(dkv_full, 1);
    mbar_init(dkv_free, NCW);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmBias);
    tma_prefetch_desc(&tmMask);
  }
  if (warp == Cfg::WARP_MMA) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](int item, int& b, int& o, int& h) {
    h = item % p.H;
    const int r = item / p.H;
    o = r % p.O;
    b = r / p.O;
  };

  if (warp == Cfg::WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int q_s = 0, kv_s = 0, b_s = 0;
      uint32_t q_ph = 1, kv_ph = 1, b_ph = 1;
      BwdWalk w;
      w.init(blockIdx.x, gridDim.x, p.n_items, p.q_tiles, p.k_tiles, KS, p.n_strips);
      int b = 0, o = 0, h = 0, cur = -1;
      for (; w.valid(); w.next()) {
        if (w.item != cur) {
          cur = w.item;
          decode(cur, b, o, h);
        }
        if (w.first_kk()) {
          mbar_wait(&q_empty[q_s], q_ph, wctx);
          mbar_expect_tx(&q_full[q_s], 2 * Cfg::TILE);
          tma_load_5d(smem + Cfg::OFF_Q + q_s * Cfg::TILE, &tmQ, &q_full[q_s], 0, w.qt * 128, h, o, b);
          tma_load_5d(smem + Cfg::OFF_DO + q_s * Cfg::TILE, &tmDO, &q_full[q_s], 0, w.qt * 128, h, o, b);
          if (++q_s == NQ) {
            q_s = 0;
            q_ph ^= 1;
          }
        }
        const int kt = w.kt();
        mbar_wait(&kv_empty[kv_s], kv_ph, wctx);
        mbar_expect_tx(&kv_full[kv_s], 2 * Cfg::TILE + 512);
        tma_load_5d(smem + Cfg::OFF_K + kv_s * Cfg::TILE, &tmK, &kv_full[kv_s], 0, kt * 128, h, o, b);
        tma_load_5d(smem + Cfg::OFF_V + kv_s * Cfg::TILE, &tmV, &kv_full[kv_s], 0, kt * 128, h, o, b);
        tma_load_3d(smem + Cfg::OFF_MASK + kv_s * 512, &tmMask, &kv_full[kv_s], kt * 128, o, b);
        if (++kv_s == NKV) {
          kv_s = 0;
          kv_ph ^= 1;
        }
        const int bb = p.bias_broadcast ? 0 : b;
        mbar_wait(&b_empty[b_s], b_ph, wctx);
        mbar_expect_tx(&b_full[b_s], Cfg::BIAS_STAGE);
        tma_load_4d(smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE, &tmBias, &b_full[b_s], kt * 128, w.qt * 128, h, bb);
        tma_load_4d(smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE + 16384, &tmBias, &b_full[b_s], kt * 128 + 64,
                    w.qt * 128, h, bb);
        if (++b_s == NB) {
          b_s = 0;
          b_ph ^= 1;
        }
      }
    }
  } else if (warp == Cfg::WARP_MMA) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_sd = make_idesc_bf16(128, 128, false, false);  // S, dP
      constexpr uint32_t idesc_kv = make_idesc_bf16(128, D, true, true);      // dV, dK
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, false, true);     // dQ
      constexpr uint32_t swz = swizzle_mode_for_bytes(Cfg::SWZ);
      constexpr uint32_t swz128 = swizzle_mode_for_bytes(128);
      // Descriptors of stage 0 of every operand; a stage or a k-step only changes the start-address
      // field (bits 0-13, 16-byte units), so the per-UMMA work is one 64-bit add.
      const uint64_t dq_k = make_smem_desc(smem_u32(smem + Cfg::OFF_Q), 16, 8 * Cfg::SWZ, swz);     // Q, K-major (S)
      const uint64_t dk_k = make_smem_desc(smem_u32(smem + Cfg::OFF_K), 16, 8 * Cfg::SWZ, swz);     // K, K-major (S)
      const uint64_t ddo_k = make_smem_desc(smem_u32(smem + Cfg::OFF_DO), 16, 8 * Cfg::SWZ, swz);   // dO, K-major (dP)
      const uint64_t dv_k = make_smem_desc(smem_u32(smem + Cfg::OFF_V), 16, 8 * Cfg::SWZ, swz);     // V, K-major (dP)
      const uint64_t dp_mn = make_smem_desc(smem_u32(smem + Cfg::OFF_P), 16384, 1024, swz128);      // P^T as A (dV)
      const uint64_t dds_mn = make_smem_desc(smem_u32(smem + Cfg::OFF_DS), 16384, 1024, swz128);    // dS^T as A (dK)
      const uint64_t dds_k = make_smem_desc(smem_u32(smem + Cfg::OFF_DS), 16, 1024, swz128);        // dS as A (dQ)
      const uint64_t ddo_mn = make_smem_desc(smem_u32(smem + Cfg::OFF_DO), 128 * Cfg::SWZ, 8 * Cfg::SWZ, swz);  // dO as B (dV)
      const uint64_t dq_mn = make_smem_desc(smem_u32(smem + Cfg::OFF_Q), 128 * Cfg::SWZ, 8 * Cfg::SWZ, swz);    // Q as B (dK)
      const uint64_t dk_mn = make_smem_desc(smem_u32(smem + Cfg::OFF_K), 128 * Cfg::SWZ, 8 * Cfg::SWZ, swz);    // K as B (dQ)
      constexpr uint64_t kTile16 = Cfg::TILE >> 4;

      // stage trackers for the "ahead" stream (S, dP) and the "behind" stream (dV, dK, dQ)
      int aq_s = 0, akv_s = 0;
      uint32_t aq_ph = 0, akv_ph = 0;
      int bq_s = 0, bkv_s = 0;
      uint32_t sdpfree_ph = 1, pdsready_ph = 0, dkvfree_ph = 1;

      BwdWalk wa, wb;  // ahead / behind
      wa.init(blockIdx.x, gridDim.x, p.n_items, p.q_tiles, p.k_tiles, KS, p.n_strips);
      wb = wa;

      auto issue_sdp = [&]() {  // S and dP of tile wa, then advance wa
        if (wa.first_kk()) mbar_wait3(&q_full[aq_s], aq_ph, &kv_full[akv_s], akv_ph, sdp_free, sdpfree_ph, wctx);
        else mbar_wait2(&kv_full[akv_s], akv_ph, sdp_free, sdpfree_ph, wctx);
        sdpfree_ph ^= 1;
        tc_fence_after();
        const uint64_t qo = aq_s * kTile16, ko = akv_s * kTile16;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + Cfg::TM_S, dq_k + qo + 2 * ks, dk_k + ko + 2 * ks, idesc_sd, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + Cfg::TM_DP, ddo_k + qo + 2 * ks, dv_k + ko + 2 * ks, idesc_sd, ks != 0);
        umma_commit(sdp_full);
        if (++akv_s == NKV) {
          akv_s = 0;
          akv_ph ^= 1;
        }
        const bool last_kk = wa.last_kk();
        wa.next();
        if (last_kk) {
          if (++aq_s == NQ) {
            aq_s = 0;
            aq_ph ^= 1;
          }
        }
      };

      if (wa.valid()) issue_sdp();
      for (; wb.valid();) {
        // S and dP of the next tile as soon as the current pair has been read out of TMEM
        if (wa.valid()) issue_sdp();
        mbar_wait(pds_ready, pdsready_ph, wctx);
        pdsready_ph ^= 1;
        if (wb.first_qt() && wb.first_kk()) {
          // first accumulation of a strip overwrites dK/dV: the previous strip must have been read out
          mbar_wait(dkv_free, dkvfree_ph, wctx);
          dkvfree_ph ^= 1;
        }
        tc_fence_after();
        const uint64_t qo = bq_s * kTile16, ko = bkv_s * kTile16;
        const uint32_t acc_kv = wb.first_qt() ? 0u : 1u;
        // dV(kt) (+)= P^T dO ; dK(kt) (+)= dS^T Q   (16 queries per step)
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tmem_base + Cfg::TM_DV + wb.kk * D, dp_mn + (uint64_t)(ks * 128), ddo_mn + qo + (uint64_t)(ks * Cfg::SWZ),
                  idesc_kv, (ks != 0) ? 1u : acc_kv);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tmem_base + Cfg::TM_DK + wb.kk * D, dds_mn + (uint64_t)(ks * 128), dq_mn + qo + (uint64_t)(ks * Cfg::SWZ),
                  idesc_kv, (ks != 0) ? 1u : acc_kv);
        // dQ(qt) (+)= dS K   (16 keys per step)
        const uint32_t acc_q = wb.first_kk() ? 0u : 1u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tmem_base + Cfg::TM_DQ, dds_k + (uint64_t)((ks >> 2) * 1024 + (ks & 3) * 2),
                  dk_mn + ko + (uint64_t)(ks * Cfg::SWZ), idesc_dq, (ks != 0) ? 1u : acc_q);
        umma_commit(pds_free);
        umma_commit(&kv_empty[bkv_s]);
        if (++bkv_s == NKV) bkv_s = 0;
        const bool last_kk = wb.last_kk();
        const bool strip_done = last_kk && wb.last_qt();
        if (last_kk) {
          umma_commit(&q_empty[bq_s]);
          if (++bq_s == NQ) bq_s = 0;
        }
        (void)strip_done;  // the compute warps learn of a finished strip from pds_free of its last tile
        wb.next();
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int part = warp >> 2;                 // which 32-key slice of the tile
    const int row = 32 * (warp & 3) + lane;     // query row in the tile == TMEM lane
    const uint32_t lane_base = 32 * (warp & 3);
    const uint32_t t_s = tmem_addr(tmem_base, lane_base, Cfg::TM_S + 32 * part);
    const uint32_t t_dp = tmem_addr(tmem_base, lane_base, Cfg::TM_DP + 32 * part);
    constexpr int DQ = D / 4;                   // output columns per thread
    const uint32_t t_dq = tmem_addr(tmem_base, lane_base, Cfg::TM_DQ + DQ * part);
    // the thread's 32 keys are four 16-byte pieces of a 128-byte row of one 64-key half tile
    const int half_off = (part >> 1) * 16384 + row * 128;
    const int piece0 = (part & 1) * 4;
    constexpr float kLog2e = 1.4426950408889634f;
    const float scale = p.scale;
    const uint64_t scale2 = f2_pack(scale, scale);
    const uint64_t log2e2 = f2_pack(kLog2e, kLog2e);

    uint32_t sdpfull_ph = 0, pdsfree_ph = 1, kv_ph = 0, b_ph = 0, dkvfull_ph = 0;
    int kv_s = 0, b_s = 0;
    float neg_lse2 = -INFINITY, delta = 0.f;
    bool have_prev_dq = false;     // a finished dQ tile waits in TMEM
    bool have_prev_strip = false;  // the dK / dV accumulators of a finished strip wait in TMEM
    int prev_q0 = 0, prev_b = 0, prev_o = 0, prev_h = 0, prev_strip = 0;
    int sp_b = 0, sp_o = 0, sp_h = 0, sp_strip = 0, sp_nk = 0;
    int stg_slot = 0;

    // read DQ consecutive accumulator columns of this thread's row
    auto ld_cols = [&](uint32_t taddr, float (&v)[DQ]) {
      if constexpr (DQ == 4) {
        uint32_t r[4];
        tmem_ld4(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
      } else {
#pragma unroll
        for (int c = 0; c < DQ; c += 8) {
          uint32_t r[8];
          tmem_ld8(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) v[c + i] = __uint_as_float(r[i]);
        }
      }
    };
    auto st_cols = [&](__nv_bfloat16* dst, const float (&v)[DQ], float mul) {
      if constexpr (DQ == 4) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(v[0] * mul, v[1] * mul), pack_bf16x2(v[2] * mul, v[3] * mul));
      } else {
#pragma unroll
        for (int c = 0; c < DQ; c += 8)
          *reinterpret_cast<uint4*>(dst + c) =
              make_uint4(pack_bf16x2(v[c] * mul, v[c + 1] * mul), pack_bf16x2(v[c + 2] * mul, v[c + 3] * mul),
                         pack_bf16x2(v[c + 4] * mul, v[c + 5] * mul), pack_bf16x2(v[c + 6] * mul, v[c + 7] * mul));
      }
    };

    // One finished 128 x D tile (this thread holds DQ columns of row `row`) -> global memory at `gtile`
    // (row 0 of the tile; the tile is one contiguous block there).  Staged: every thread drops its piece
    // into a shared-memory copy of the block, then the 512 compute threads write the block out in
    // consecutive 16-byte pieces, so each store instruction covers 512 contiguous bytes instead of 32
    // half-used sectors.  All sixteen compute warps call this together.
    auto store_tile = [&](__nv_bfloat16* gtile, int rows_valid, const float (&v)[DQ], float mul) {
      if constexpr (Cfg::STAGED) {
        uint8_t* stg = smem + Cfg::OFF_STG + stg_slot * Cfg::TILE;
        stg_slot ^= 1;
        st_cols(reinterpret_cast<__nv_bfloat16*>(stg) + row * D + DQ * part, v, mul);
        named_barrier_sync(1, 32 * NCW);
#pragma unroll
        for (int i = threadIdx.x; i < Cfg::TILE / 16; i += 32 * NCW)
          if ((16 * i) / (2 * D) < rows_valid)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(gtile) + 16 * i) = *reinterpret_cast<const uint4*>(stg + 16 * i);
      } else {
        if (row < rows_valid) st_cols(gtile + row * D + DQ * part, v, mul);
      }
    };

    // store a finished dQ tile that has been read out of TMEM (or fold it into the per-CTA running sum)
    auto store_dq = [&](int b, int o, int h, int q0, int strip, float (&v)[DQ]) {
      if (p.n_strips == 1) {
        store_tile(p.dq + ((((int64_t)b * p.O + o) * p.H + h) * p.N + q0) * D, p.N - q0, v, scale);
        return;
      }
      const int q = q0 + row;
      if (q >= p.N) return;
      if (p.n_strips > 1) {
        float* sc = p.dq_scratch + ((int64_t)blockIdx.x * p.N + q) * D + DQ * part;
        if (strip > 0) {
#pragma unroll
          for (int c = 0; c < DQ; c += 4) {
            const float4 o4 = *reinterpret_cast<const float4*>(sc + c);
            v[c] += o4.x; v[c + 1] += o4.y; v[c + 2] += o4.z; v[c + 3] += o4.w;
          }
        }
        if (strip + 1 < p.n_strips) {
#pragma unroll
          for (int c = 0; c < DQ; c += 4) *reinterpret_cast<float4*>(sc + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
          return;
        }
      }
      st_cols(p.dq + ((((int64_t)b * p.O + o) * p.H + h) * p.N + q) * D + DQ * part, v, scale);
    };

    // lse / delta of this thread's query row, loaded one query tile ahead of their first use
    float l_pref = -INFINITY, d_pref = 0.f;
    auto prefetch_row_scalars = [&](const BwdWalk& t) {
      l_pref = -INFINITY;
      d_pref = 0.f;
      if (t.valid()) {
        int pb, po, phh;
        decode(t.item, pb, po, phh);
        const int pq = t.qt * 128 + row;
        if (pq < p.N) {
          const int64_t idx = (((int64_t)pb * p.O + po) * p.H + phh) * p.N + pq;
          l_pref = __ldg(p.lse + idx);
          d_pref = __ldg(p.delta + idx);
        }
      }
    };

    // Reads finished accumulators out of TMEM and sends them on their way: the dQ tile of a finished query
    // tile and, after the last tile of a strip, the strip's dK / dV tiles (then the UMMA issuer may start the
    // next strip in those columns).  Called by all compute warps once the UMMAs of the previous tile are done.
    auto drain_finished = [&]() {
      if (have_prev_dq) {
        float dqv[DQ];
        ld_cols(t_dq, dqv);
        have_prev_dq = false;
        store_dq(prev_b, prev_o, prev_h, prev_q0, prev_strip, dqv);
      }
      if (have_prev_strip) {
        have_prev_strip = false;
        for (int kk = 0; kk < sp_nk; ++kk) {
          const int key0 = (sp_strip * KS + kk) * 128;
          const int64_t base = ((((int64_t)sp_b * p.O + sp_o) * p.H + sp_h) * p.N + key0) * D;
          float vk1[DQ], vv1[DQ];
          ld_cols(tmem_addr(tmem_base, lane_base, Cfg::TM_DK + kk * D + DQ * part), vk1);
          ld_cols(tmem_addr(tmem_base, lane_base, Cfg::TM_DV + kk * D + DQ * part), vv1);
          store_tile(p.dk + base, p.N - key0, vk1, scale);
          store_tile(p.dv + base, p.N - key0, vv1, 1.f);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dkv_free);
      } else {
        tc_fence_before();
      }
    };

    BwdWalk w;
    w.init(blockIdx.x, gridDim.x, p.n_items, p.q_tiles, p.k_tiles, KS, p.n_strips);
    prefetch_row_scalars(w);
    int b = 0, o = 0, h = 0, cur = -1;
    for (; w.valid(); w.next()) {
      if (w.item != cur) {
        cur = w.item;
        decode(cur, b, o, h);
      }
      const int kt = w.kt();
      if (w.first_kk()) {
        // values fetched one query tile ahead; fetch the next tile's now
        neg_lse2 = (l_pref == -INFINITY) ? -INFINITY : -l_pref * kLog2e;
        delta = d_pref;
        BwdWalk nx = w;
        const int sl = w.strip_len();
        for (int t = 0; t < sl; ++t) nx.next();
        prefetch_row_scalars(nx);
      }
      const uint64_t nlse2 = f2_pack(neg_lse2, neg_lse2);
      const uint64_t ndel2 = f2_pack(-delta, -delta);

      mbar_wait3(sdp_full, sdpfull_ph, &kv_full[kv_s], kv_ph, &b_full[b_s], b_ph, wctx);
      sdpfull_ph ^= 1;
      tc_fence_after();
      const uint8_t* bias_row = smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE + half_off;
      const float* mask_row = reinterpret_cast<const float*>(smem + Cfg::OFF_MASK + kv_s * 512) + 32 * part;
      const bool tail = (kt + 1) * 128 > p.N;
      const bool general = tail || __any_sync(0xffffffffu, mask_row[lane] != 0.f);

      uint32_t ppk[16], dpk[16];  // bf16 pairs of P and dS of this thread's 32 keys
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {  // 16 keys per step
        uint32_t rs[16], rd[16];
        tmem_ld16(t_s + 16 * ch, rs);
        tmem_ld16(t_dp + 16 * ch, rd);
        const uint4 bv0 = *reinterpret_cast<const uint4*>(bias_row + (((piece0 + 2 * ch) ^ (row & 7)) << 4));
        const uint4 bv1 = *reinterpret_cast<const uint4*>(bias_row + (((piece0 + 2 * ch + 1) ^ (row & 7)) << 4));
        tmem_ld_wait();
        if (ch == 1) {
          // S, dP and the bias tile have been read: the next pair of UMMAs / the next bias load may overwrite them
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(sdp_free);
            mbar_arrive(&b_empty[b_s]);
          }
        }
        const uint32_t bw[8] = {bv0.x, bv0.y, bv0.z, bv0.w, bv1.x, bv1.y, bv1.z, bv1.w};
        uint64_t vv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          vv[e] = f2_fma(f2_pack_bits(rs[2 * e], rs[2 * e + 1]), scale2, f2_pack_bits(bw[e] << 16, bw[e] & 0xFFFF0000u));
        if (general) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 mk = *reinterpret_cast<const float2*>(mask_row + 16 * ch + 2 * e);
            float v0, v1;
            f2_unpack(f2_add(vv[e], f2_pack(mk.x, mk.y)), v0, v1);
            if (tail) {
              const int k0 = kt * 128 + 32 * part + 16 * ch + 2 * e;
              if (k0 >= p.N) v0 = -INFINITY;
              if (k0 + 1 >= p.N) v1 = -INFINITY;
            }
            vv[e] = f2_pack(v0, v1);
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint64_t v2 = vv[e];
          float a0, a1;
          f2_unpack(f2_fma(v2, log2e2, nlse2), a0, a1);
          const float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
          float d0, d1;
          f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack_bits(rd[2 * e], rd[2 * e + 1]), ndel2)), d0, d1);
          ppk[8 * ch + e] = pack_bf16x2(p0, p1);
          dpk[8 * ch + e] = pack_bf16x2(d0, d1);
        }
      }
      if (++b_s == NB) {
        b_s = 0;
        b_ph ^= 1;
      }
      if (++kv_s == NKV) {
        kv_s = 0;
        kv_ph ^= 1;
      }

      // the dV / dK / dQ UMMAs of the previous tile are done: the P and dS tiles are free and a finished dQ can be read
      mbar_wait(pds_free, pdsfree_ph, wctx);
      pdsfree_ph ^= 1;
      tc_fence_after();
      // the same completion covers the last tile of a strip: its dQ and the strip's dK / dV leave now,
      // before this tile's P / dS release the UMMAs that would overwrite them
      drain_finished();
      {
        uint8_t* p_row = smem + Cfg::OFF_P + half_off;
        uint8_t* ds_row = smem + Cfg::OFF_DS + half_off;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int off = ((piece0 + u) ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(p_row + off) = make_uint4(ppk[4 * u], ppk[4 * u + 1], ppk[4 * u + 2], ppk[4 * u + 3]);
          *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(dpk[4 * u], dpk[4 * u + 1], dpk[4 * u + 2], dpk[4 * u + 3]);
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);

      if (w.last_kk()) {
        have_prev_dq = true;
        prev_b = b; prev_o = o; prev_h = h; prev_q0 = w.qt * 128; prev_strip = w.strip;
      }
      if (w.last_kk() && w.last_qt()) {
        have_prev_strip = true;
        sp_b = b; sp_o = o; sp_h = h; sp_strip = w.strip; sp_nk = w.strip_len();
      }
    }
    // the last tile of this CTA: wait for its UMMAs, then the same drain
    if (have_prev_dq || have_prev_strip) {
      mbar_wait(pds_free, pdsfree_ph, wctx);
      pdsfree_ph ^= 1;
      tc_fence_after();
      drain_finished();
    }
  }


  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// =============================================================================================
// kernel 2: dBias partial planes.  One CTA = one (group, h, query tile, key tile) and a chunk of
// outer planes; dS summed over the chunk in ascending plane order, fp32, in registers.
// =============================================================================================
struct AttnDbiasParams {
  float* part;        // [n_chunks][G][H][N][N] fp32 (or the final buffer when n_chunks == 1)
  const float* lse;   // [B,O,H,N]
  const float* delta; // [B,O,H,N]
  int B, O, H, N;
  int G;              // bias batch (1 or B)
  int planes;         // outer planes per group = (B / G) * O
  int n_chunks, chunk_len;
  int q_tiles, k_tiles;
  float scale;
};

template <int D_>
struct AttnDbiasCfg {
  static constexpr int D = D_;
  static constexpr int SWZ = 2 * D;
  static constexpr int TILE = 128 * D * 2;
  static constexpr int STAGE = 4 * TILE + 1024;  // Q, dO, K, V, mask row
  static constexpr int NST = D <= 32 ? 4 : 2;
  static constexpr int NCW = 16;                 // compute warps: four threads per query row, 32 keys each
  static constexpr int OFF_BIAS32 = 0;           // the CTA's bias tile as fp32 * log2(e), 64 KiB, thread-major
  static constexpr int OFF_ST = 65536;
  // the bf16 bias tile is staged once: in the last stage buffer when that is large enough (the
  // producer waits for the conversion before it first fills that buffer), else in a region of its own
  static constexpr bool STAGE_HOLDS_BIAS = STAGE >= 32768 + 1024;
  static constexpr int OFF_BSTG = STAGE_HOLDS_BIAS ? OFF_ST + (NST - 1) * STAGE : OFF_ST + NST * STAGE;
  static constexpr int OFF_BAR = OFF_ST + NST * STAGE + (STAGE_HOLDS_BIAS ? 0 : 32768);
  static constexpr int N_BAR = 2 * NST + 4 + 2;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TMEM_COLS = 512;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// 16 compute warps: four threads share one query row (TMEM lane) and take 32 of the 128 keys of the
// tile each.  The bias tile of a CTA never changes, so it is converted once to fp32 (already
// multiplied by log2 e) and read back with conflict-free 16-byte loads; per logit the inner loop is
// three packed fp32x2 operations, one ex2 and (only for planes whose mask row is not all zero in
// this key range, or for a ragged key tail) the mask add.
template <class Cfg>
__global__ void __launch_bounds__(32 * (Cfg::NCW + 2), 1)
attn_dbias_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                  const __grid_constant__ CUtensorMap tmBias, const __grid_constant__ CUtensorMap tmMask,
                  const AttnDbiasParams p, int* __restrict__ status) {
  griddep_wait();
  constexpr int D = Cfg::D, NST = Cfg::NST, NCW = Cfg::NCW;
  constexpr int WARP_TMA = NCW, WARP_MMA = NCW + 1;
  constexpr int CPT = 32;                   // key columns per thread
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full = bars;
  uint64_t* empty = full + NST;
  uint64_t* sdp_full = empty + NST;   // [2]
  uint64_t* sdp_free = sdp_full + 2;  // [2]
  uint64_t* bias_full = sdp_free + 2;
  uint64_t* bias_done = bias_full + 1;  // the compute warps have converted the staged bias tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* bias_stage = smem + Cfg::OFF_BSTG;  // bf16 tile as TMA delivers it

  // work item
  int it = blockIdx.x;
  const int chunk = it % p.n_chunks; it /= p.n_chunks;
  const int kt = it % p.k_tiles; it /= p.k_tiles;
  const int qt = it % p.q_tiles; it /= p.q_tiles;
  const int h = it % p.H;
  const int g = it / p.H;
  const int pl0 = chunk * p.chunk_len;
  const int pl1 = min(p.planes, pl0 + p.chunk_len);
  const int b_per_g = p.B / p.G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1 + NCW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&sdp_free[s], NCW);
    }
    mbar_init(bias_full, 1);
    mbar_init(bias_done, NCW);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
    tma_prefetch_desc(&tmBias);
    tma_prefetch_desc(&tmMask);
  }
  if (warp == WARP_MMA) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == WARP_TMA) {
    if (lane == 0) {
      mbar_expect_tx(bias_full, 32768);
      tma_load_4d(bias_stage, &tmBias, bias_full, kt * 128, qt * 128, h, g);
      tma_load_4d(bias_stage + 16384, &tmBias, bias_full, kt * 128 + 64, qt * 128, h, g);
      int s = 0;
      uint32_t ph = 1;
      for (int pl = pl0; pl < pl1; ++pl) {
        const int b = g * b_per_g + pl / p.O, o = pl % p.O;
        if (pl - pl0 == NST - 1) mbar_wait(bias_done, 0, wctx);  // first use of the buffer the bias was staged in
        mbar_wait(&empty[s], ph, wctx);
        mbar_expect_tx(&full[s], 4 * Cfg::TILE + 512);
        uint8_t* st = smem + Cfg::OFF_ST + s * Cfg::STAGE;
        tma_load_5d(st, &tmQ, &full[s], 0, qt * 128, h, o, b);
        tma_load_5d(st + Cfg::TILE, &tmDO, &full[s], 0, qt * 128, h, o, b);
        tma_load_5d(st + 2 * Cfg::TILE, &tmK, &full[s], 0, kt * 128, h, o, b);
        tma_load_5d(st + 3 * Cfg::TILE, &tmV, &full[s], 0, kt * 128, h, o, b);
        tma_load_3d(st + 4 * Cfg::TILE, &tmMask, &full[s], kt * 128, o, b);
        if (++s == NST) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp == WARP_MMA) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t swz = swizzle_mode_for_bytes(Cfg::SWZ);
      int s = 0, buf = 0;
      uint32_t ph = 0, free_ph[2] = {1, 1};
      for (int pl = pl0; pl < pl1; ++pl) {
        mbar_wait2(&full[s], ph, &sdp_free[buf], free_ph[buf], wctx);
        free_ph[buf] ^= 1;
        tc_fence_after();
        const uint32_t st = smem_u32(smem + Cfg::OFF_ST + s * Cfg::STAGE);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + buf * 256, make_smem_desc(st + ks * 32, 16, 8 * Cfg::SWZ, swz),
                  make_smem_desc(st + 2 * Cfg::TILE + ks * 32, 16, 8 * Cfg::SWZ, swz), idesc, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + buf * 256 + 128, make_smem_desc(st + Cfg::TILE + ks * 32, 16, 8 * Cfg::SWZ, swz),
                  make_smem_desc(st + 3 * Cfg::TILE + ks * 32, 16, 8 * Cfg::SWZ, swz), idesc, ks != 0);
        umma_commit(&sdp_full[buf]);
        umma_commit(&empty[s]);
        buf ^= 1;
        if (++s == NST) {
          s = 0;
          ph ^= 1;
        }
      }
    }
  } else if (warp < NCW) {
    const int part = warp >> 2;               // which 32-column slice of the tile
    const int row = 32 * (warp & 3) + lane;
    const uint32_t lane_base = 32 * (warp & 3);
    constexpr float kLog2e = 1.4426950408889634f;
    const float c1 = p.scale * kLog2e;
    const uint64_t c2 = f2_pack(c1, c1);
    const uint64_t log2e2 = f2_pack(kLog2e, kLog2e);
    const int q = qt * 128 + row;
    const bool tail = (kt + 1) * 128 > p.N;

    // ---- bias tile -> fp32 * log2(e), laid out [part][16-column half][4-column group][row][4] so that
    //      the 32 lanes of a warp read 32 consecutive 16-byte pieces
    float4* bias32 = reinterpret_cast<float4*>(smem + Cfg::OFF_BIAS32);
    mbar_wait(bias_full, 0, wctx);
    {
      const int col0 = CPT * part;
      const uint8_t* brow = bias_stage + (col0 >> 6) * 16384 + row * 128;
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // 8 columns per 16-byte piece of the bf16 tile
        const uint4 bv = *reinterpret_cast<const uint4*>(brow + (((((col0 & 63) >> 3) + u) ^ (row & 7)) << 4));
        const float4 lo = make_float4(__uint_as_float(bv.x << 16) * kLog2e, __uint_as_float(bv.x & 0xFFFF0000u) * kLog2e,
                                      __uint_as_float(bv.y << 16) * kLog2e, __uint_as_float(bv.y & 0xFFFF0000u) * kLog2e);
        const float4 hi = make_float4(__uint_as_float(bv.z << 16) * kLog2e, __uint_as_float(bv.z & 0xFFFF0000u) * kLog2e,
                                      __uint_as_float(bv.w << 16) * kLog2e, __uint_as_float(bv.w & 0xFFFF0000u) * kLog2e);
        // piece u covers columns 8u .. 8u+7 of the slice: half = u / 2, groups 2 (u % 2) and 2 (u % 2) + 1
        bias32[(((part * 2 + (u >> 1)) * 4 + 2 * (u & 1)) * 128) + row] = lo;
        bias32[(((part * 2 + (u >> 1)) * 4 + 2 * (u & 1) + 1) * 128) + row] = hi;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bias_done);

    uint64_t acc[CPT / 2];
#pragma unroll
    for (int i = 0; i < CPT / 2; ++i) acc[i] = 0ull;

    // lse / delta of (plane, h, q): planes of one group are consecutive in memory, so the index
    // advances by H * N per step (no division in the loop)
    const int64_t row_stride = (int64_t)p.H * p.N;
    const int64_t row_idx0 = ((int64_t)g * b_per_g * p.O * p.H + h) * p.N + q;
    auto load_row_scalars = [&](int pl, float& l, float& dl) {
      l = INFINITY;  // a row without a finite log-sum-exp (fully masked, or past N) contributes nothing
      dl = 0.f;
      if (pl < pl1 && q < p.N) {
        const int64_t idx = row_idx0 + (int64_t)pl * row_stride;
        l = __ldg(p.lse + idx);
        dl = __ldg(p.delta + idx);
      }
    };

    int s = 0, buf = 0;
    uint32_t ph = 0, full_ph[2] = {0, 0};
    // row scalars travel two planes ahead of their use (they come from HBM on first touch)
    float l_n1, dl_n1, l_n2, dl_n2;
    load_row_scalars(pl0, l_n1, dl_n1);
    load_row_scalars(pl0 + 1, l_n2, dl_n2);
    for (int pl = pl0; pl < pl1; ++pl) {
      // exp2(t - lse log2e) with lse = -inf (fully masked row) must give 0, not NaN: use -inf there
      const float nl = (l_n1 == -INFINITY || l_n1 == INFINITY) ? -INFINITY : -l_n1 * kLog2e;
      const uint64_t nl2 = f2_pack(nl, nl);
      const uint64_t nd2 = f2_pack(-dl_n1, -dl_n1);
      l_n1 = l_n2;
      dl_n1 = dl_n2;
      load_row_scalars(pl + 2, l_n2, dl_n2);
      mbar_wait2(&sdp_full[buf], full_ph[buf], &full[s], ph, wctx);
      full_ph[buf] ^= 1;
      tc_fence_after();
      const float* mask_row =
          reinterpret_cast<const float*>(smem + Cfg::OFF_ST + s * Cfg::STAGE + 4 * Cfg::TILE) + CPT * part;
      const uint32_t t_s = tmem_addr(tmem_base, lane_base, buf * 256 + CPT * part);
      const uint32_t t_dp = tmem_addr(tmem_base, lane_base, buf * 256 + 128 + CPT * part);
      // 8 columns per step; the TMEM loads of step c+1 are in flight while step c is computed
      uint32_t rs[2][8], rd[2][8];
      tmem_ld8(t_s, rs[0]);
      tmem_ld8(t_dp, rd[0]);
      // the mask probe (shared-memory load + vote) runs under the latency of the first TMEM loads
      const bool general = tail || __any_sync(0xffffffffu, mask_row[lane] != 0.f);
#pragma unroll
      for (int c = 0; c < CPT / 8; ++c) {
        const float4 bb0 = bias32[((part * 2 + (c >> 1)) * 4 + 2 * (c & 1)) * 128 + row];
        const float4 bb1 = bias32[((part * 2 + (c >> 1)) * 4 + 2 * (c & 1) + 1) * 128 + row];
        tmem_ld_wait();  // step c has landed
        if (c + 1 < CPT / 8) {
          tmem_ld8(t_s + 8 * (c + 1), rs[(c + 1) & 1]);
          tmem_ld8(t_dp + 8 * (c + 1), rd[(c + 1) & 1]);
        } else {
          // the whole TMEM tile is in registers: the next S / dP pair may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sdp_free[buf]);
        }
        const uint32_t(&s8)[8] = rs[c & 1];
        const uint32_t(&d8)[8] = rd[c & 1];
        uint64_t t2[4];
        t2[0] = f2_fma(f2_pack_bits(s8[0], s8[1]), c2, f2_pack(bb0.x, bb0.y));
        t2[1] = f2_fma(f2_pack_bits(s8[2], s8[3]), c2, f2_pack(bb0.z, bb0.w));
        t2[2] = f2_fma(f2_pack_bits(s8[4], s8[5]), c2, f2_pack(bb1.x, bb1.y));
        t2[3] = f2_fma(f2_pack_bits(s8[6], s8[7]), c2, f2_pack(bb1.z, bb1.w));
        if (general) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 mk = *reinterpret_cast<const float2*>(mask_row + 8 * c + 2 * i);
            float v0, v1;
            f2_unpack(f2_fma(f2_pack(mk.x, mk.y), log2e2, t2[i]), v0, v1);
            if (tail) {
              const int k0 = kt * 128 + CPT * part + 8 * c + 2 * i;
              if (k0 >= p.N) v0 = -INFINITY;
              if (k0 + 1 >= p.N) v1 = -INFINITY;
            }
            t2[i] = f2_pack(v0, v1);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float a0, a1;
          f2_unpack(f2_add(t2[i], nl2), a0, a1);
          const uint64_t pr = f2_pack(ex2_approx(a0), ex2_approx(a1));
          const uint64_t gd = f2_add(f2_pack_bits(d8[2 * i], d8[2 * i + 1]), nd2);
          acc[4 * c + i] = f2_fma(pr, gd, acc[4 * c + i]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      buf ^= 1;
      if (++s == NST) {
        s = 0;
        ph ^= 1;
      }
    }

    if (q < p.N) {
      const int k0 = kt * 128 + CPT * part;
      float* dst = p.part + ((((int64_t)chunk * p.G + g) * p.H + h) * p.N + q) * p.N + k0;
      float a[CPT];
#pragma unroll
      for (int i = 0; i < CPT / 2; ++i) f2_unpack(acc[i], a[2 * i], a[2 * i + 1]);
      if ((p.N & 3) == 0 && k0 + CPT <= p.N) {
#pragma unroll
        for (int i = 0; i < CPT; i += 4)
          *reinterpret_cast<float4*>(dst + i) = make_float4(a[i], a[i + 1], a[i + 2], a[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < CPT; ++i)
          if (k0 + i < p.N) dst[i] = a[i];
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// dbias[i] = ((part[0][i] + part[1][i]) + part[2][i]) + ...   (ascending chunk order, fp32)
__global__ void __launch_bounds__(256) attn_dbias_fold_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                              int64_t n, int n_chunks) {
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float a = part[i];
    for (int c = 1; c < n_chunks; ++c) a = __fadd_rn(a, part[(int64_t)c * n + i]);
    out[i] = a;
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
int make_qkv_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
                  const int64_t* st, int swz);
int make_bias_tmap(CUtensorMap* tm, const void* base, int64_t Bb, int64_t H, int64_t N, int64_t pitch);
int make_mask_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t N, int64_t pitch);

template <int D>
int launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                    const CUtensorMap& tb, const CUtensorMap& tmk, AttnBwdParams& p, int* status, int grid,
                    cudaStream_t stream) {
  using Cfg = AttnBwdCfg<D>;
  auto kern = attn_bwd_kernel<Cfg>;
  static PerDeviceOnce once;  // per instantiation
  if (int rc = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, once)) return rc;
  launch_kernel(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, tq, tk, tv, tdo, tb, tmk, p, status);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

static int bwd_key_strip(int64_t D) { return D <= 32 ? 3 : 1; }

int64_t attn_bwd_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t D) {
  const int64_t k_tiles = (N + 127) / 128;
  const int64_t strips = (k_tiles + bwd_key_strip(D) - 1) / bwd_key_strip(D);
  if (strips <= 1) return 0;
  int64_t grid = sm_count();
  if (grid > B * O * H) grid = B * O * H;
  return grid * N * D * 4;
}

int attn_bwd_dqkv(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                  const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                  const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch, int64_t bias_batch,
                  void* dq, void* dk, void* dv, float* delta, void* workspace, int64_t workspace_bytes, int64_t B,
                  int64_t O, int64_t H, int64_t N, int64_t D, float scale, int stages, cudaStream_t stream) {
  TPF_REQUIRE(q && k && v && d_out && out && lse && mask && bias && dq && dk && dv && delta, TPF_ERR_INVALID_ARGUMENT,
              "attn_bwd: null pointer");
  TPF_REQUIRE(B > 0 && O > 0 && H > 0 && N > 0, TPF_ERR_INVALID_ARGUMENT, "attn_bwd: B,O,H,N must be positive");
  TPF_REQUIRE(D == 16 || D == 32 || D == 64, TPF_ERR_UNSUPPORTED, "attn_bwd: head dim %lld not in {16,32,64}",
              (long long)D);
  TPF_REQUIRE(bias_batch == 1 || bias_batch == B, TPF_ERR_INVALID_ARGUMENT, "attn_bwd: bias batch must be 1 or B");
  TPF_REQUIRE(bias_pitch >= N && bias_pitch % 8 == 0, TPF_ERR_INVALID_ARGUMENT,
              "attn_bwd: bias row pitch must be >= N and a multiple of 8 elements");
  TPF_REQUIRE(mask_pitch >= N && mask_pitch % 4 == 0, TPF_ERR_INVALID_ARGUMENT,
              "attn_bwd: mask row pitch must be >= N and a multiple of 4 elements");
  TPF_REQUIRE(B * O * H < (1ll << 31) && N <= (1 << 24), TPF_ERR_INVALID_ARGUMENT, "attn_bwd: extent too large");
  // dq / dk / dv rows and the delta pass's operands are accessed with 16-byte vectors
  TPF_REQUIRE_ALIGNED16(dq, "attn_bwd", "dq");
  TPF_REQUIRE_ALIGNED16(dk, "attn_bwd", "dk");
  TPF_REQUIRE_ALIGNED16(dv, "attn_bwd", "dv");
  TPF_REQUIRE_ALIGNED16(d_out, "attn_bwd", "d_out");
  TPF_REQUIRE_ALIGNED16(out, "attn_bwd", "out");
  const int64_t need = attn_bwd_workspace_bytes(B, O, H, N, D);
  TPF_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), TPF_ERR_WORKSPACE,
              "attn_bwd: workspace of %lld bytes required, %lld given", (long long)need, (long long)workspace_bytes);
  TPF_REQUIRE(need == 0 || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0, TPF_ERR_WORKSPACE,
              "attn_bwd: workspace must be 16-byte aligned");

  // delta = rowsum(dO * O)
  if (stages & 1) {
    const int64_t rows = B * O * N * H;
    const int lanes = (int)D / 8;
    const int64_t threads = rows * lanes;
    const int64_t blocks = (threads + 255) / 256;
    TPF_REQUIRE(blocks < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "attn_bwd: too many rows");
    const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(d_out);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(out);
    if (D == 16) launch_kernel(attn_delta_kernel<16>, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, delta, rows, (int)H, (int)N);
    else if (D == 32) launch_kernel(attn_delta_kernel<32>, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, delta, rows, (int)H, (int)N);
    else launch_kernel(attn_delta_kernel<64>, dim3((unsigned)blocks), dim3(256), 0, stream, a, b, delta, rows, (int)H, (int)N);
    TPF_LAUNCH_OK();
  }

  if (!(stages & 2)) return TPF_OK;
  const int swz = 2 * (int)D;
  CUtensorMap tq, tk, tv, tdo, tb, tm;
  int rc;
  if ((rc = make_qkv_tmap(&tq, q, B, O, H, N, D, q_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tk, k, B, O, H, N, D, k_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tv, v, B, O, H, N, D, v_strides, swz))) return rc;
  const int64_t do_strides[4] = {O * N * H * D, N * H * D, D, H * D};  // d_out is [B,O,N,H,D]
  if ((rc = make_qkv_tmap(&tdo, d_out, B, O, H, N, D, do_strides, swz))) return rc;
  if ((rc = make_bias_tmap(&tb, bias, bias_batch, H, N, bias_pitch))) return rc;
  if ((rc = make_mask_tmap(&tm, mask, B, O, N, mask_pitch))) return rc;

  AttnBwdParams p;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lse = lse;
  p.delta = delta;
  p.dq_scratch = reinterpret_cast<float*>(workspace);
  p.B = (int)B; p.O = (int)O; p.H = (int)H; p.N = (int)N;
  p.q_tiles = (int)((N + 127) / 128);
  p.k_tiles = p.q_tiles;
  const int ks = bwd_key_strip(D);
  p.n_strips = (p.k_tiles + ks - 1) / ks;
  p.bias_broadcast = bias_batch == 1 && B > 1 ? 1 : 0;
  p.scale = scale;
  p.n_items = (int)(B * O * H);
  int grid = sm_count();
  if (grid > p.n_items) grid = p.n_items;
  int* status = nullptr;
  if ((rc = attn_bwd_status_address(&status))) return rc;
  if (D == 16) return launch_attn_bwd<16>(tq, tk, tv, tdo, tb, tm, p, status, grid, stream);
  if (D == 32) return launch_attn_bwd<32>(tq, tk, tv, tdo, tb, tm, p, status, grid, stream);
  return launch_attn_bwd<64>(tq, tk, tv, tdo, tb, tm, p, status, grid, stream);
}

template <int D>
int launch_attn_dbias(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const CUtensorMap& tb, const CUtensorMap& tmk, AttnDbiasParams& p, int* status, int grid,
                      cudaStream_t stream) {
  using Cfg = AttnDbiasCfg<D>;
  auto kern = attn_dbias_kernel<Cfg>;
  static PerDeviceOnce once;  // per instantiation
  if (int rc = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, once)) return rc;
  launch_kernel(kern, dim3(grid), dim3(32 * (Cfg::NCW + 2)), Cfg::SMEM_BYTES, stream, tq, tk, tv, tdo, tb, tmk, p, status);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

// How the outer planes of one dBias tile are split into independent chunks.
static void dbias_plan(int64_t B, int64_t O, int64_t H, int64_t N, int64_t G, int* n_chunks, int* chunk_len) {
  const int64_t tiles = G * H * ((N + 127) / 128) * ((N + 127) / 128);
  const int64_t planes = (B / G) * O;
  int64_t c = sm_count() / tiles;
  if (c < 1) c = 1;
  if (c > planes) c = planes;
  const int64_t len = (planes + c - 1) / c;
  c = (planes + len - 1) / len;
  *n_chunks = (int)c;
  *chunk_len = (int)len;
}

int64_t attn_dbias_workspace_bytes(int64_t B, int64_t O, int64_t H, int64_t N, int64_t G) {
  int c, len;
  dbias_plan(B, O, H, N, G, &c, &len);
  return c > 1 ? (int64_t)c * G * H * N * N * 4 : 0;
}

int attn_bwd_dbias(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                   const int64_t* k_strides, const int64_t* v_strides, const float* lse, const float* delta,
                   const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch, int64_t bias_batch,
                   float* dbias, void* workspace, int64_t workspace_bytes, int64_t B, int64_t O, int64_t H, int64_t N,
                   int64_t D, float scale, cudaStream_t stream) {
  TPF_REQUIRE(dbias != nullptr, TPF_ERR_INVALID_ARGUMENT, "attn_bwd: dbias is NULL");
  TPF_REQUIRE_ALIGNED16(dbias, "attn_bwd", "dbias");  // rows are written with float4 stores
  const int64_t G = bias_batch;
  int n_chunks, chunk_len;
  dbias_plan(B, O, H, N, G, &n_chunks, &chunk_len);
  const int64_t need = attn_dbias_workspace_bytes(B, O, H, N, G);
  TPF_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), TPF_ERR_WORKSPACE,
              "attn_bwd: dBias workspace of %lld bytes required, %lld given", (long long)need,
              (long long)workspace_bytes);
  TPF_REQUIRE(need == 0 || (reinterpret_cast<uintptr_t>(workspace) & 15) == 0, TPF_ERR_WORKSPACE,
              "attn_bwd: dBias workspace must be 16-byte aligned");
  const int swz = 2 * (int)D;
  CUtensorMap tq, tk, tv, tdo, tb, tm;
  int rc;
  if ((rc = make_qkv_tmap(&tq, q, B, O, H, N, D, q_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tk, k, B, O, H, N, D, k_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tv, v, B, O, H, N, D, v_strides, swz))) return rc;
  const int64_t do_strides[4] = {O * N * H * D, N * H * D, D, H * D};
  if ((rc = make_qkv_tmap(&tdo, d_out, B, O, H, N, D, do_strides, swz))) return rc;
  if ((rc = make_bias_tmap(&tb, bias, bias_batch, H, N, bias_pitch))) return rc;
  if ((rc = make_mask_tmap(&tm, mask, B, O, N, mask_pitch))) return rc;
  AttnDbiasParams p;
  p.part = n_chunks > 1 ? reinterpret_cast<float*>(workspace) : dbias;
  p.lse = lse;
  p.delta = delta;
  p.B = (int)B; p.O = (int)O; p.H = (int)H; p.N = (int)N;
  p.G = (int)G;
  p.planes = (int)((B / G) * O);
  p.n_chunks = n_chunks;
  p.chunk_len = chunk_len;
  p.q_tiles = (int)((N + 127) / 128);
  p.k_tiles = p.q_tiles;
  p.scale = scale;
  const int64_t grid = (int64_t)G * H * p.q_tiles * p.k_tiles * n_chunks;
  TPF_REQUIRE(grid < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "attn_bwd: dBias grid too large");
  int* status = nullptr;
  if ((rc = attn_bwd_status_address(&status))) return rc;
  if (D == 16) rc = launch_attn_dbias<16>(tq, tk, tv, tdo, tb, tm, p, status, (int)grid, stream);
  else if (D == 32) rc = launch_attn_dbias<32>(tq, tk, tv, tdo, tb, tm, p, status, (int)grid, stream);
  else rc = launch_attn_dbias<64>(tq, tk, tv, tdo, tb, tm, p, status, (int)grid, stream);
  if (rc) return rc;
  if (n_chunks > 1) {
    const int64_t n = G * H * N * N;
    int blocks = (int)((n + 255) / 256);
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    launch_kernel(attn_dbias_fold_kernel, dim3(blocks), dim3(256), 0, stream, p.part, dbias, n, n_chunks);
    TPF_LAUNCH_OK();
  }
  return TPF_OK;
}

// =============================================================================================
// Backward with library-owned scratch: for callers that cannot allocate device memory themselves
// =============================================================================================
// Some hosts of this library may not call cudaMalloc (or any allocating routine) around the
// backward pass: code running between graph-capture begin/end, real-time or plugin hosts whose
// memory is handed out once at start-up, and foreign runtimes that own the device heap.  For them
// the scratch of the backward pass (per-CTA dQ running sums, dBias chunk planes) lives in a fixed
// array that is part of the library image.  Every GPU that loads the library holds these
// kStaticScratchBytes until the process exits.
constexpr int64_t kStaticScratchBytes = 16ll << 20;  // 16 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int64_t attn_bwd_static_scratch_capacity() { return kStaticScratchBytes; }

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address is looked up once per device (with that device current) and cached.
static int static_scratch_address(void** out) {
  static PerDeviceAddress cache;
  int rc = device_symbol_address(g_static_scratch, cache, out);
  if (rc) return rc;
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(*out) & 255) == 0, TPF_ERR_CUDA,
              "static scratch address lookup returned a misaligned pointer");
  return TPF_OK;
}

int attn_bwd_static_scratch(const void* q, const void* k, const void* v, const void* d_out, const int64_t* q_strides,
                            const int64_t* k_strides, const int64_t* v_strides, const void* out, const float* lse,
                            const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch,
                            int64_t bias_batch, void* dq, void* dk, void* dv, float* dbias, float* delta, int64_t B,
                            int64_t O, int64_t H, int64_t N, int64_t D, float scale, cudaStream_t stream) {
  TPF_REQUIRE(B > 0 && O > 0 && H > 0 && N > 0 && (bias_batch == 1 || bias_batch == B), TPF_ERR_INVALID_ARGUMENT,
              "attn_bwd (library scratch): bad extents");
  TPF_REQUIRE(D == 16 || D == 32 || D == 64, TPF_ERR_UNSUPPORTED,
              "attn_bwd (library scratch): head dim %lld not in {16,32,64}", (long long)D);
  const int64_t ws_a = (attn_bwd_workspace_bytes(B, O, H, N, D) + 255) / 256 * 256;
  const int64_t ws_b = (attn_dbias_workspace_bytes(B, O, H, N, bias_batch) + 255) / 256 * 256;
  TPF_REQUIRE(ws_a + ws_b <= kStaticScratchBytes, TPF_ERR_WORKSPACE,
              "attn_bwd (library scratch): this shape needs %lld bytes of scratch, the built-in array holds %lld; "
              "use tpf_attn_bwd with a caller-provided workspace",
              (long long)(ws_a + ws_b), (long long)kStaticScratchBytes);
  void* base = nullptr;
  int rc = static_scratch_address(&base);
  if (rc) return rc;
  // Nothing in the scratch has to start at zero: the dQ running sums are written by the first key
  // strip before they are read, and every dBias chunk plane is fully overwritten.
  rc = attn_bwd_dqkv(q, k, v, d_out, q_strides, k_strides, v_strides, out, lse, mask, mask_pitch, bias, bias_pitch,
                     bias_batch, dq, dk, dv, delta, base, ws_a, B, O, H, N, D, scale, 3, stream);
  if (rc) return rc;
  return attn_bwd_dbias(q, k, v, d_out, q_strides, k_strides, v_strides, lse, delta, mask, mask_pitch, bias,
                        bias_pitch, bias_batch, dbias, static_cast<char*>(base) + ws_a, ws_b, B, O, H, N, D, scale,
                        stream);
}

}  // namespace tpf
