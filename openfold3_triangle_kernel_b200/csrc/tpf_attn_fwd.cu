// Triangle-attention forward for sm_100a.
//
//   S[q,k]  = (Q K^T)[q,k] * scale + mask[k] + bias[q,k]      (fp32, logits never leave the SM)
//   out     = softmax_k(S) V  -> bf16 [B,O,N,H,D];   lse = logsumexp_k(S) -> fp32 [B,O,H,N]
//
// Stands in for the reference forward kernels
// (openfold3/core/kernels/turbopairformer/turbopairformer_triangle_forward.cu:775-1256 and :451-766):
// same math and rounding points (fp32 running max / sum, probabilities rounded to bf16 for P V,
// fully masked rows give out = 0 and lse = -inf), different machine mapping:
//
//  * A work item is one (b, o, h, 128-query tile); a CTA walks its items and, inside an item, the
//    64-key tiles.  CTAs are small (6 warps, about 55 KB of shared memory, 128 TMEM columns and about
//    70 registers per thread at D <= 32) so that FOUR of them are resident per SM: the latency of a
//    barrier hand-off, a TMA load or an MMA of one CTA is covered by the arithmetic of the others, and
//    the FMA / ALU work (bias add, maximum) of one overlaps the MUFU work (exponentials) of another.
//  * warps 0-3: softmax warps, one thread per query row (= TMEM lane).  warp 4: TMA producer.
//    warp 5: UMMA issuer.
//  * Q K^T runs on tcgen05 with S in TMEM.  The softmax warps walk a tile 16 columns at a time straight
//    from TMEM (one pass: bias add, running maximum, exponentials, row sum).  The bf16 probabilities go
//    back to TMEM (not to shared memory) and P V is issued with its A operand in TMEM; O accumulates
//    in TMEM across key tiles.  The reference maximum of a row is raised - and the row's partial
//    results rescaled - only when a chunk exceeds it by more than a fixed gap.
//  * A tile whose mask row is all zero and that has no ragged key tail (the common case) takes a
//    code path without the mask add.
#include "tpf_host.cuh"
#include "tpf_ptx.cuh"

namespace tpf {

static __device__ int g_attn_fwd_status;

int attn_fwd_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  TPF_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn_fwd_status, sizeof(int)));
  if (v) TPF_CUDA_OK(cudaMemcpyToSymbol(g_attn_fwd_status, &zero, sizeof(int)));
  *out = v;
  return TPF_OK;
}

struct AttnFwdParams {
  __nv_bfloat16* out;  // [B,O,N,H,D]
  float* lse;          // [B,O,H,N]
  int B, O, H, N;
  int q_tiles, k_tiles;  // 128-query tiles, 64-key tiles
  int bias_broadcast;    // 1: one bias for all b
  float scale;           // softmax scale applied to Q K^T
  int n_items;
};

template <int D_>
struct AttnFwdCfg {
  static constexpr int D = D_;
  static constexpr int KEYS = 64;                // keys per tile
  static constexpr int CTAS_PER_SM = D <= 32 ? 4 : 2;
  static constexpr int SWZ = 2 * D;              // bytes per smem row of a Q/K/V tile
  static constexpr int Q_TILE = 128 * D * 2;
  static constexpr int KV_TILE = KEYS * D * 2;
  static constexpr int NB = 2;                   // bias stages
  static constexpr int NKV = 3;                  // slots of the shared K / V ring (K0 V0 K1 V1 ...)
  static constexpr int NMASK = 4;                // mask-row slots (256 B each)
  static constexpr int BIAS_STAGE = 128 * KEYS * 2;
  static constexpr int OFF_BIAS = 0;
  static constexpr int OFF_Q = OFF_BIAS + NB * BIAS_STAGE;
  static constexpr int OFF_KV = OFF_Q + Q_TILE;                  // [NKV]
  static constexpr int OFF_MASK = OFF_KV + NKV * KV_TILE;        // [NMASK] x 256 B
  static constexpr int OFF_BAR = OFF_MASK + NMASK * 256;
  static constexpr int N_BAR = 2 * NB + 2 + 2 * NKV + 4;
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TM_S = 0;      // logits, fp32, 64 columns
  static constexpr int TM_P = 64;     // probabilities, bf16 pairs, 32 columns
  static constexpr int TM_O = 96;     // output accumulator, fp32, D columns
  static constexpr int TMEM_COLS = TM_O + D <= 128 ? 128 : 256;
  static constexpr int THREADS = 192;            // 4 softmax warps, TMA warp, UMMA warp
  static constexpr int WARP_TMA = 4, WARP_MMA = 5;
  static_assert(D == 16 || D == 32 || D == 64, "head dim lanes");
  static_assert(TMEM_COLS * CTAS_PER_SM <= 512, "TMEM budget");
  static_assert((SMEM_BYTES + 1024) * CTAS_PER_SM <= 233472, "shared memory budget");
  static_assert(KV_TILE % 1024 == 0 && Q_TILE % 1024 == 0, "tile buffers keep 1024-byte alignment");
};

// Softmax is done in ONE pass over each 64-key tile, 16 columns at a time straight out of TMEM, so a
// thread holds 16 logits at a time instead of a whole row segment (about 70 registers per thread,
// which is what lets four CTAs share an SM).  The exponentials of a chunk use the row's current
// reference maximum m; a chunk whose own maximum exceeds m by more than kGap first raises m and
// rescales what the row has accumulated so far (its sum, the part of P already stored for this tile,
// and O).  Every exponent argument is therefore bounded by kGap and the result does not depend on
// how often m was raised: lse = m + log(sum) at the end.
template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, Cfg::CTAS_PER_SM)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
                const __grid_constant__ CUtensorMap tmMask, const AttnFwdParams p, int* __restrict__ status) {
  griddep_wait();
  constexpr int D = Cfg::D, NKV = Cfg::NKV, NB = Cfg::NB, NMASK = Cfg::NMASK, KEYS = Cfg::KEYS;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* b_full = bars;                  // [NB]
  uint64_t* b_empty = b_full + NB;          // [NB]
  uint64_t* q_full = b_empty + NB;
  uint64_t* q_empty = q_full + 1;
  uint64_t* kv_full = q_empty + 1;          // [NKV]
  uint64_t* kv_empty = kv_full + NKV;       // [NKV]
  uint64_t* s_full = kv_empty + NKV;
  uint64_t* s_free = s_full + 1;
  uint64_t* p_ready = s_free + 1;
  uint64_t* pv_done = p_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 4);
    }
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < NKV; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
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

  const int KT = p.k_tiles;

  // item -> (b, h, qt, o); o fastest so that CTAs running at the same time read the same bias strip.
  // The coordinates are a mixed-radix counter advanced by the grid size: the divisions happen once, not per
  // item (an integer division by a run-time value costs a warp several hundred cycles on its critical path).
  struct ItemWalk {
    int o, qt, h, b;      // current item
    int so, sq, sh, sb;   // the step, decomposed
    int O, Q, H;
    __device__ void init(int item, int step, int O_, int Q_, int H_) {
      O = O_; Q = Q_; H = H_;
      o = item % O; int r = item / O;
      qt = r % Q; r /= Q;
      h = r % H; b = r / H;
      so = step % O; r = step / O;
      sq = r % Q; r /= Q;
      sh = r % H; sb = r / H;
    }
    __device__ __forceinline__ void next() {
      o += so;
      int c = o >= O ? 1 : 0;
      o -= c * O;
      qt += sq + c;
      c = qt >= Q ? 1 : 0;
      qt -= c * Q;
      h += sh + c;
      c = h >= H ? 1 : 0;
      h -= c * H;
      b += sb + c;
    }
  };

  if (warp == Cfg::WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    // Ring order K(0) V(0) K(1) V(1) ...: a K slot is free again once its Q K^T has run (early in the
    // tile), a V slot once its P V has run (end of the tile), so three slots keep K one tile and V
    // two tiles ahead.  The mask row of a tile arrives on the barrier of its K tile.
    if (lane == 0) {
      uint32_t q_ph = 1;
      int kv_s = 0, b_s = 0, m_s = 0;
      uint32_t kv_ph = 1, b_ph = 1;
      ItemWalk iw;
      iw.init(blockIdx.x, gridDim.x, p.O, p.q_tiles, p.H);
      for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, iw.next()) {
        const int b = iw.b, h = iw.h, qt = iw.qt, o = iw.o;
        const int bb = p.bias_broadcast ? 0 : b;
        mbar_wait(q_empty, q_ph, wctx);
        q_ph ^= 1;
        mbar_expect_tx(q_full, Cfg::Q_TILE);
        tma_load_5d(smem + Cfg::OFF_Q, &tmQ, q_full, 0, qt * 128, h, o, b);
        for (int j = 0; j < KT; ++j) {
          mbar_wait(&kv_empty[kv_s], kv_ph, wctx);
          mbar_expect_tx(&kv_full[kv_s], Cfg::KV_TILE + 256);
          tma_load_5d(smem + Cfg::OFF_KV + kv_s * Cfg::KV_TILE, &tmK, &kv_full[kv_s], 0, j * KEYS, h, o, b);
          tma_load_3d(smem + Cfg::OFF_MASK + m_s * 256, &tmMask, &kv_full[kv_s], j * KEYS, o, b);
          m_s = (m_s + 1) & (NMASK - 1);
          if (++kv_s == NKV) {
            kv_s = 0;
            kv_ph ^= 1;
          }
          mbar_wait(&b_empty[b_s], b_ph, wctx);
          mbar_expect_tx(&b_full[b_s], Cfg::BIAS_STAGE);
          tma_load_4d(smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE, &tmBias, &b_full[b_s], j * KEYS, qt * 128, h, bb);
          if (++b_s == NB) {
            b_s = 0;
            b_ph ^= 1;
          }
          mbar_wait(&kv_empty[kv_s], kv_ph, wctx);
          mbar_expect_tx(&kv_full[kv_s], Cfg::KV_TILE);
          tma_load_5d(smem + Cfg::OFF_KV + kv_s * Cfg::KV_TILE, &tmV, &kv_full[kv_s], 0, j * KEYS, h, o, b);
          if (++kv_s == NKV) {
            kv_s = 0;
            kv_ph ^= 1;
          }
        }
      }
    }
  } else if (warp == Cfg::WARP_MMA) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, KEYS, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      constexpr uint32_t swz = swizzle_mode_for_bytes(Cfg::SWZ);
      uint32_t q_ph = 0, sfree_ph = 1, pready_ph = 0;
      // ring positions of the next K tile and the next V tile (K and V alternate in the ring)
      int k_s = 0, v_s = 1;
      uint32_t k_ph = 0, v_ph = 0;
      const uint64_t q_desc0 = make_smem_desc(smem_u32(smem + Cfg::OFF_Q), 16, 8 * Cfg::SWZ, swz);
      const uint64_t k_desc0 = make_smem_desc(smem_u32(smem + Cfg::OFF_KV), 16, 8 * Cfg::SWZ, swz);
      const uint64_t v_desc0 = make_smem_desc(smem_u32(smem + Cfg::OFF_KV), KEYS * Cfg::SWZ, 8 * Cfg::SWZ, swz);
      auto advance2 = [&](int& s, uint32_t& ph) {
        s += 2;
        if (s >= NKV) {
          s -= NKV;
          ph ^= 1;
        }
      };

      auto issue_qk = [&](bool last) {
        // s_free: the softmax warps have read the whole previous S tile
        mbar_wait2(&kv_full[k_s], k_ph, s_free, sfree_ph, wctx);
        sfree_ph ^= 1;
        tc_fence_after();
        // descriptors differ from the hoisted ones only in the start-address field (bits 0-13, in 16-byte units)
        const uint64_t kd = k_desc0 + (uint64_t)((k_s * Cfg::KV_TILE) >> 4);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + Cfg::TM_S, q_desc0 + 2 * ks, kd + 2 * ks, idesc_qk, ks != 0);
        umma_commit(s_full);
        umma_commit(&kv_empty[k_s]);
        if (last) umma_commit(q_empty);
        advance2(k_s, k_ph);
      };

      bool first = true;
      for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
        if (first) {
          mbar_wait(q_full, q_ph, wctx);
          q_ph ^= 1;
          issue_qk(KT == 1);
          first = false;
        }
        const bool more_items = item + (int)gridDim.x < p.n_items;
        for (int j = 0; j < KT; ++j) {
          // Q K^T of the next tile (of this item or of the next one) as soon as S has been read
          if (j + 1 < KT) {
            issue_qk(j + 2 == KT);
          } else if (more_items) {
            mbar_wait(q_full, q_ph, wctx);
            q_ph ^= 1;
            issue_qk(KT == 1);
          }
          mbar_wait2(p_ready, pready_ph, &kv_full[v_s], v_ph, wctx);
          pready_ph ^= 1;
          tc_fence_after();
          const uint64_t vd = v_desc0 + (uint64_t)((v_s * Cfg::KV_TILE) >> 4);
#pragma unroll
          for (int ks = 0; ks < KEYS / 16; ++ks)  // 16 keys per step; A = P from TMEM (8 columns of bf16 pairs)
            umma_ts(tmem_base + Cfg::TM_O, tmem_base + Cfg::TM_P + 8 * ks, vd + (uint64_t)(ks * Cfg::SWZ), idesc_pv,
                    (ks | j) != 0);
          umma_commit(pv_done);
          umma_commit(&kv_empty[v_s]);
          advance2(v_s, v_ph);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: one thread per query row
    const int row = 32 * warp + lane;  // query row inside the tile == TMEM lane
    const uint32_t t_s = tmem_addr(tmem_base, 32 * warp, Cfg::TM_S);
    const uint32_t t_p = tmem_addr(tmem_base, 32 * warp, Cfg::TM_P);
    const uint32_t t_o = tmem_addr(tmem_base, 32 * warp, Cfg::TM_O);
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLn2 = 0.6931471805599453f;
    constexpr float kGap = 12.0f;  // largest exponent (natural units) a probability may have relative to m
    const uint64_t scale2 = f2_pack(p.scale, p.scale);
    const uint64_t log2e2 = f2_pack(kLog2e, kLog2e);

    uint32_t sfull_ph = 0, pv_ph = 0, b_ph = 0;
    int b_s = 0, m_s = 0;

    ItemWalk iw;
    iw.init(blockIdx.x, gridDim.x, p.O, p.q_tiles, p.H);
    for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, iw.next()) {
      const int b = iw.b, h = iw.h, qt = iw.qt, o = iw.o;
      float m_use = -INFINITY, l_run = 0.f;

      for (int j = 0; j < KT; ++j) {
        // s_full completes after Q K^T of this tile, hence after the K tile and the mask row that
        // arrives on the same barrier have landed
        mbar_wait(s_full, sfull_ph, wctx);
        sfull_ph ^= 1;
        const float* mask_row = reinterpret_cast<const float*>(smem + Cfg::OFF_MASK + m_s * 256);
        m_s = (m_s + 1) & (NMASK - 1);
        const bool tail = (j + 1) * KEYS > p.N;
        const float2 mprobe = *reinterpret_cast<const float2*>(mask_row + 2 * lane);
        const bool general = tail || __any_sync(0xffffffffu, (mprobe.x != 0.f) || (mprobe.y != 0.f));
        const uint8_t* bias_row = smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE + row * 128;
        if (j > 0) {
          // P V of the previous tile must be complete before P is overwritten or O is rescaled (it was
          // issued a whole tile ago)
          mbar_wait2(&b_full[b_s], b_ph, pv_done, pv_ph, wctx);
          pv_ph ^= 1;
        } else {
          mbar_wait(&b_full[b_s], b_ph, wctx);
        }
        tc_fence_after();
        float neg_m = (m_use == -INFINITY) ? 0.f : -m_use * kLog2e;
        uint64_t rs2 = 0ull;  // packed partial row sum of this tile

#pragma unroll
        for (int c = 0; c < KEYS / 16; ++c) {  // 16 key columns per step
          uint32_t raw[16];
          tmem_ld16(t_s + 16 * c, raw);
          const uint4 bv0 = *reinterpret_cast<const uint4*>(bias_row + (((2 * c) ^ (row & 7)) << 4));
          const uint4 bv1 = *reinterpret_cast<const uint4*>(bias_row + (((2 * c + 1) ^ (row & 7)) << 4));
          tmem_ld_wait();
          if (c == KEYS / 16 - 1) {
            // the whole S tile and bias tile have been read: the next Q K^T / bias load may overwrite them
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              mbar_arrive(s_free);
              mbar_arrive(&b_empty[b_s]);
            }
          }
          const uint32_t bw[8] = {bv0.x, bv0.y, bv0.z, bv0.w, bv1.x, bv1.y, bv1.z, bv1.w};
          uint64_t v2[8];
          float cmax0 = -INFINITY, cmax1 = -INFINITY;
          if (!general) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const uint64_t b2 = f2_pack_bits(bw[e] << 16, bw[e] & 0xFFFF0000u);
              v2[e] = f2_fma(f2_pack_bits(raw[2 * e], raw[2 * e + 1]), scale2, b2);
              float v0, v1;
              f2_unpack(v2[e], v0, v1);
              if (e & 1) cmax1 = max3(cmax1, v0, v1);
              else cmax0 = max3(cmax0, v0, v1);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const uint64_t b2 = f2_pack_bits(bw[e] << 16, bw[e] & 0xFFFF0000u);
              const float2 mk = *reinterpret_cast<const float2*>(mask_row + 16 * c + 2 * e);
              float v0, v1;
              f2_unpack(f2_add(f2_fma(f2_pack_bits(raw[2 * e], raw[2 * e + 1]), scale2, b2), f2_pack(mk.x, mk.y)), v0,
                        v1);
              if (tail) {
                const int k0 = j * KEYS + 16 * c + 2 * e;
                if (k0 >= p.N) v0 = -INFINITY;
                if (k0 + 1 >= p.N) v1 = -INFINITY;
              }
              v2[e] = f2_pack(v0, v1);
              if (e & 1) cmax1 = max3(cmax1, v0, v1);
              else cmax0 = max3(cmax0, v0, v1);
            }
          }
          const float cmax = fmaxf(cmax0, cmax1);
          if (__any_sync(0xffffffffu, cmax > m_use + kGap)) {
            // Raise the reference maximum of the rows that need it (f = 1 for the others) and rescale what
            // those rows have accumulated.  Runs for the first finite chunk of every row and then only
            // when the logits of a row grow by more than kGap.
            const bool grow = cmax > m_use + kGap;
            const float f = grow ? ex2_approx((m_use - cmax) * kLog2e) : 1.f;  // m_use = -inf gives 0; nothing accumulated then
            if (grow) m_use = cmax;
            neg_m = (m_use == -INFINITY) ? 0.f : -m_use * kLog2e;
            l_run *= f;
            {
              float r0, r1;
              f2_unpack(rs2, r0, r1);
              rs2 = f2_pack(r0 * f, r1 * f);
            }
            if (c > 0) tmem_st_wait();
#pragma unroll
            for (int cc = 0; cc < KEYS / 16; ++cc) {
              if (cc < c) {  // part of P already stored for this tile
                uint32_t pr[8];
                tmem_ld8(t_p + 8 * cc, pr);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  pr[i] = pack_bf16x2(__uint_as_float(pr[i] << 16) * f, __uint_as_float(pr[i] & 0xFFFF0000u) * f);
                tmem_st8(t_p + 8 * cc, pr);
              }
            }
            if (j > 0) {
#pragma unroll
              for (int cc = 0; cc < D; cc += 8) {
                uint32_t ro[8];
                tmem_ld8(t_o + cc, ro);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
                tmem_st8(t_o + cc, ro);
              }
            }
          }
          const uint64_t neg_m2 = f2_pack(neg_m, neg_m);
          uint32_t pk[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float a0, a1;
            f2_unpack(f2_fma(v2[e], log2e2, neg_m2), a0, a1);
            const float e0 = ex2_approx(a0), e1 = ex2_approx(a1);
            rs2 = f2_add(rs2, f2_pack(e0, e1));
            pk[e] = pack_bf16x2(e0, e1);
          }
          tmem_st8(t_p + 8 * c, pk);
        }
        {
          float r0, r1;
          f2_unpack(rs2, r0, r1);
          l_run += r0 + r1;
        }
        if (++b_s == NB) {
          b_s = 0;
          b_ph ^= 1;
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
      }

      // last tile's P V, then the accumulated output row
      mbar_wait(pv_done, pv_ph, wctx);
      pv_ph ^= 1;
      tc_fence_after();
      const int q = qt * 128 + row;
      const float inv = l_run > 0.f ? __fdividef(1.f, l_run) : 0.f;
      __nv_bfloat16* orow = p.out + ((((int64_t)b * p.O + o) * p.N + q) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 16) {
        uint32_t ro[16];
        tmem_ld16(t_o + c, ro);
        tmem_ld_wait();
        if (q < p.N) {
          uint4 pk0, pk1;
          pk0.x = pack_bf16x2(__uint_as_float(ro[0]) * inv, __uint_as_float(ro[1]) * inv);
          pk0.y = pack_bf16x2(__uint_as_float(ro[2]) * inv, __uint_as_float(ro[3]) * inv);
          pk0.z = pack_bf16x2(__uint_as_float(ro[4]) * inv, __uint_as_float(ro[5]) * inv);
          pk0.w = pack_bf16x2(__uint_as_float(ro[6]) * inv, __uint_as_float(ro[7]) * inv);
          pk1.x = pack_bf16x2(__uint_as_float(ro[8]) * inv, __uint_as_float(ro[9]) * inv);
          pk1.y = pack_bf16x2(__uint_as_float(ro[10]) * inv, __uint_as_float(ro[11]) * inv);
          pk1.z = pack_bf16x2(__uint_as_float(ro[12]) * inv, __uint_as_float(ro[13]) * inv);
          pk1.w = pack_bf16x2(__uint_as_float(ro[14]) * inv, __uint_as_float(ro[15]) * inv);
          *reinterpret_cast<uint4*>(orow + c) = pk0;
          *reinterpret_cast<uint4*>(orow + c + 8) = pk1;
        }
      }
      tc_fence_before();
      if (q < p.N)
        p.lse[(((int64_t)b * p.O + o) * p.H + h) * p.N + q] = l_run > 0.f ? m_use + log2f(l_run) * kLn2 : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

// 5-D map over a [B,O,H,N,D] bf16 tensor with element strides (sb, so, sh, sn), D contiguous.
// `rows` = sequence positions per box.
int make_qkv_tmap_rows(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
                       const int64_t* st, int swz, int rows) {
  uint64_t dims[5] = {(uint64_t)D, (uint64_t)N, (uint64_t)H, (uint64_t)O, (uint64_t)B};
  uint64_t strides[4] = {(uint64_t)st[3] * 2, (uint64_t)st[2] * 2, (uint64_t)st[1] * 2, (uint64_t)st[0] * 2};
  uint32_t box[5] = {(uint32_t)D, (uint32_t)rows, 1, 1, 1};
  return make_tmap_bf16(tm, base, 5, dims, strides, box, swz);
}
int make_qkv_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
                  const int64_t* st, int swz) {
  return make_qkv_tmap_rows(tm, base, B, O, H, N, D, st, swz, 128);
}

// 4-D map over the bf16 bias [Bb,H,N,N] whose rows are `pitch` elements apart.
int make_bias_tmap(CUtensorMap* tm, const void* base, int64_t Bb, int64_t H, int64_t N, int64_t pitch) {
  uint64_t dims[4] = {(uint64_t)N, (uint64_t)N, (uint64_t)H, (uint64_t)Bb};
  uint64_t strides[3] = {(uint64_t)pitch * 2, (uint64_t)pitch * N * 2, (uint64_t)pitch * N * H * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, 128);
}

// 3-D map over the fp32 additive mask [B,O,N] whose rows are `pitch` elements apart.
int make_mask_tmap_cols(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t N, int64_t pitch, int cols) {
  uint64_t dims[3] = {(uint64_t)N, (uint64_t)O, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)pitch * 4, (uint64_t)pitch * O * 4};
  uint32_t box[3] = {(uint32_t)cols, 1, 1};
  return make_tmap_f32(tm, base, 3, dims, strides, box);
}
int make_mask_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t N, int64_t pitch) {
  return make_mask_tmap_cols(tm, base, B, O, N, pitch, 128);
}

template <int D>
int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tb,
                    const CUtensorMap& tmk, const AttnFwdParams& p, int* status, cudaStream_t stream) {
  using Cfg = AttnFwdCfg<D>;
  auto kern = attn_fwd_kernel<Cfg>;
  static PerDeviceOnce once;  // per instantiation
  if (int rc = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, once)) return rc;
  int grid = Cfg::CTAS_PER_SM * sm_count();
  if (grid > p.n_items) grid = p.n_items;
  launch_kernel(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, tq, tk, tv, tb, tmk, p, status);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

int attn_fwd(const void* q, const void* k, const void* v, const int64_t* q_strides, const int64_t* k_strides,
             const int64_t* v_strides, const float* mask, int64_t mask_pitch, const void* bias, int64_t bias_pitch,
             int64_t bias_batch, void* out, float* lse, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
             float scale, cudaStream_t stream) {
  TPF_REQUIRE(q && k && v && mask && bias && out && lse, TPF_ERR_INVALID_ARGUMENT, "attn_fwd: null pointer");
  TPF_REQUIRE(B > 0 && O > 0 && H > 0 && N > 0, TPF_ERR_INVALID_ARGUMENT, "attn_fwd: B,O,H,N must be positive");
  TPF_REQUIRE(D == 16 || D == 32 || D == 64, TPF_ERR_UNSUPPORTED,
              "attn_fwd: head dim %lld not in {16,32,64} (pad on the host side)", (long long)D);
  TPF_REQUIRE(bias_batch == 1 || bias_batch == B, TPF_ERR_INVALID_ARGUMENT, "attn_fwd: bias batch must be 1 or B");
  TPF_REQUIRE(bias_pitch >= N && bias_pitch % 8 == 0, TPF_ERR_INVALID_ARGUMENT,
              "attn_fwd: bias row pitch must be >= N and a multiple of 8 elements");
  TPF_REQUIRE(mask_pitch >= N && mask_pitch % 4 == 0, TPF_ERR_INVALID_ARGUMENT,
              "attn_fwd: mask row pitch must be >= N and a multiple of 4 elements");
  TPF_REQUIRE(N <= (1 << 24) && B * O * H < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "attn_fwd: extent too large");
  TPF_REQUIRE_ALIGNED16(out, "attn_fwd", "out");
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(lse) & 3) == 0, TPF_ERR_INVALID_ARGUMENT,
              "attn_fwd: lse must be 4-byte aligned");
  const int swz = 2 * (int)D;
  CUtensorMap tq, tk, tv, tb, tm;
  int rc;
  if ((rc = make_qkv_tmap(&tq, q, B, O, H, N, D, q_strides, swz))) return rc;
  if ((rc = make_qkv_tmap_rows(&tk, k, B, O, H, N, D, k_strides, swz, 64))) return rc;
  if ((rc = make_qkv_tmap_rows(&tv, v, B, O, H, N, D, v_strides, swz, 64))) return rc;
  if ((rc = make_bias_tmap(&tb, bias, bias_batch, H, N, bias_pitch))) return rc;
  if ((rc = make_mask_tmap_cols(&tm, mask, B, O, N, mask_pitch, 64))) return rc;
  AttnFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = (int)B; p.O = (int)O; p.H = (int)H; p.N = (int)N;
  p.q_tiles = (int)((N + 127) / 128);
  p.k_tiles = (int)((N + 63) / 64);
  p.bias_broadcast = bias_batch == 1 && B > 1 ? 1 : 0;
  p.scale = scale;
  const int64_t items = B * H * p.q_tiles * O;
  TPF_REQUIRE(items < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "attn_fwd: too many work items");
  p.n_items = (int)items;
  int* status = nullptr;
  {
    static PerDeviceAddress cache;
    if ((rc = device_symbol_address(g_attn_fwd_status, cache, reinterpret_cast<void**>(&status)))) return rc;
  }
  if (D == 16) return launch_attn_fwd<16>(tq, tk, tv, tb, tm, p, status, stream);
  if (D == 32) return launch_attn_fwd<32>(tq, tk, tv, tb, tm, p, status, stream);
  return launch_attn_fwd<64>(tq, tk, tv, tb, tm, p, status, stream);
}

}  // namespace tpf
