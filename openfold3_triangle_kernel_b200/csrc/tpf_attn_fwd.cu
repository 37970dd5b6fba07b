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
//  * persistent CTAs, 18 working warps.  A work item is (b, h, 128-query tile, PAIR of outer rows o);
//    both rows of the pair use the same 128x128 bias tiles, so the bias - the largest
//    operand stream - is fetched once per pair.
//  * warps 0-7 / 8-15: two softmax groups, one per outer row; two threads per query row
//    (= TMEM lane), each owning 64 of the 128 keys of a tile, with packed fp32x2 arithmetic.
//    warp 16: TMA producer.  warp 17: UMMA issuer.
//  * Q K^T and P V run on tcgen05 with accumulators in TMEM.  The softmax group pulls the
//    logits of its rows into registers at once, releases the TMEM tile (so the next
//    Q K^T overlaps the exponentials), writes bf16 P into a swizzled smem tile for the
//    P V UMMA, which accumulates the output in TMEM across key tiles; the accumulator
//    is rescaled (TMEM load, multiply, store) only when a row maximum grows by more than
//    a fixed gap, so most tiles pay no rescale at all.
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
  int q_tiles, k_tiles, o_pairs;
  int bias_broadcast;  // 1: one bias for all b
  float scale;         // softmax scale applied to Q K^T
  int n_items;
};

template <int D_, int NKV_>
struct AttnFwdCfg {
  static constexpr int D = D_, NKV = NKV_;
  static constexpr int SWZ = 2 * D;              // bytes per smem row of a Q/K/V tile
  static constexpr int TILE = 128 * D * 2;       // one Q, K or V tile
  static constexpr int NB = D <= 32 ? 2 : 1;     // bias stages
  static constexpr int BIAS_STAGE = 128 * 128 * 2;
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int OFF_BIAS = 0;
  static constexpr int OFF_Q = OFF_BIAS + NB * BIAS_STAGE;       // [2]
  static constexpr int OFF_K = OFF_Q + 2 * TILE;                 // [2][NKV]
  static constexpr int OFF_V = OFF_K + 2 * NKV * TILE;           // [2][NKV]
  static constexpr int OFF_P = OFF_V + 2 * NKV * TILE;           // [2]
  static constexpr int OFF_MASK = OFF_P + 2 * P_BYTES;           // [2][NKV] x 512 B
  static constexpr int OFF_XCHG = OFF_MASK + 2 * NKV * 512;      // [2 parity][2 groups][2 halves][128] fp32
  static constexpr int OFF_BAR = OFF_XCHG + 2 * 2 * 2 * 128 * 4;
  static constexpr int N_BAR = 2 * NB + 2 * (2 + 4 * NKV + 4);
  static constexpr int SMEM_BYTES = OFF_BAR + N_BAR * 8 + 16 + 1024;
  static constexpr int TM_S = 0;      // S[w] at 128*w
  static constexpr int TM_O = 256;    // O[w] at 256 + 64*w
  static constexpr int TMEM_COLS = 512;
  static constexpr int THREADS = 640;            // 16 softmax warps, TMA warp, UMMA warp, 2 idle
  static constexpr int WARP_TMA = 16, WARP_MMA = 17;
  static_assert(D == 16 || D == 32 || D == 64, "head dim lanes");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmBias,
                const __grid_constant__ CUtensorMap tmMask, const AttnFwdParams p, int* __restrict__ status) {
  constexpr int D = Cfg::D, NKV = Cfg::NKV, NB = Cfg::NB;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* b_full = bars;                  // [NB]
  uint64_t* b_empty = b_full + NB;          // [NB]
  uint64_t* wg_bars = b_empty + NB;         // per group w: layout below
  constexpr int WG_STRIDE = 2 + 4 * NKV + 4;
  auto q_full = [&](int w) { return wg_bars + w * WG_STRIDE + 0; };
  auto q_empty = [&](int w) { return wg_bars + w * WG_STRIDE + 1; };
  auto k_full = [&](int w, int s) { return wg_bars + w * WG_STRIDE + 2 + s; };
  auto k_empty = [&](int w, int s) { return wg_bars + w * WG_STRIDE + 2 + NKV + s; };
  auto v_full = [&](int w, int s) { return wg_bars + w * WG_STRIDE + 2 + 2 * NKV + s; };
  auto v_empty = [&](int w, int s) { return wg_bars + w * WG_STRIDE + 2 + 3 * NKV + s; };
  auto s_full = [&](int w) { return wg_bars + w * WG_STRIDE + 2 + 4 * NKV + 0; };
  auto s_free = [&](int w) { return wg_bars + w * WG_STRIDE + 2 + 4 * NKV + 1; };
  auto p_ready = [&](int w) { return wg_bars + w * WG_STRIDE + 2 + 4 * NKV + 2; };
  auto pv_done = [&](int w) { return wg_bars + w * WG_STRIDE + 2 + 4 * NKV + 3; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + Cfg::N_BAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const WaitCtx wctx{abort_flag, status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(&b_full[s], 1);
      mbar_init(&b_empty[s], 16);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(q_full(w), 1);
      mbar_init(q_empty(w), 1);
      for (int s = 0; s < NKV; ++s) {
        mbar_init(k_full(w, s), 1);
        mbar_init(k_empty(w, s), 1);
        mbar_init(v_full(w, s), 1);
        mbar_init(v_empty(w, s), 1);
      }
      mbar_init(s_full(w), 1);
      mbar_init(s_free(w), 8);
      mbar_init(p_ready(w), 8);
      mbar_init(pv_done(w), 1);
    }
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

  // item -> (b, h, qt, o2); o2 fastest so that consecutive items reuse the same bias strip
  auto decode = [&](int item, int& b, int& h, int& qt, int& o2) {
    o2 = item % p.o_pairs;
    int r = item / p.o_pairs;
    qt = r % p.q_tiles;
    r /= p.q_tiles;
    h = r % p.H;
    b = r / p.H;
  };

  if (warp == Cfg::WARP_TMA) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t q_ph[2] = {1, 1};
      int k_s[2] = {0, 0}, v_s[2] = {0, 0};
      uint32_t k_ph[2] = {1, 1}, v_ph[2] = {1, 1};
      int b_s = 0;
      uint32_t b_ph = 1;
      for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
        int b, h, qt, o2;
        decode(item, b, h, qt, o2);
        const int bb = p.bias_broadcast ? 0 : b;
        for (int w = 0; w < 2; ++w) {
          const int o = 2 * o2 + w;
          if (o >= p.O) continue;
          mbar_wait(q_empty(w), q_ph[w], wctx);
          q_ph[w] ^= 1;
          mbar_expect_tx(q_full(w), Cfg::TILE);
          tma_load_5d(smem + Cfg::OFF_Q + w * Cfg::TILE, &tmQ, q_full(w), 0, qt * 128, h, o, b);
        }
        for (int j = 0; j < KT; ++j) {
          // K first (needed by the next Q K^T), then the bias tile, then V + mask row
          for (int w = 0; w < 2; ++w) {
            const int o = 2 * o2 + w;
            if (o >= p.O) continue;
            mbar_wait(k_empty(w, k_s[w]), k_ph[w], wctx);
            mbar_expect_tx(k_full(w, k_s[w]), Cfg::TILE);
            tma_load_5d(smem + Cfg::OFF_K + (w * NKV + k_s[w]) * Cfg::TILE, &tmK, k_full(w, k_s[w]), 0, j * 128, h,
                        o, b);
            if (++k_s[w] == NKV) {
              k_s[w] = 0;
              k_ph[w] ^= 1;
            }
          }
          mbar_wait(&b_empty[b_s], b_ph, wctx);
          mbar_expect_tx(&b_full[b_s], Cfg::BIAS_STAGE);
          tma_load_4d(smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE, &tmBias, &b_full[b_s], j * 128, qt * 128, h, bb);
          tma_load_4d(smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE + 16384, &tmBias, &b_full[b_s], j * 128 + 64,
                      qt * 128, h, bb);
          if (++b_s == NB) {
            b_s = 0;
            b_ph ^= 1;
          }
          for (int w = 0; w < 2; ++w) {
            const int o = 2 * o2 + w;
            if (o >= p.O) continue;
            mbar_wait(v_empty(w, v_s[w]), v_ph[w], wctx);
            mbar_expect_tx(v_full(w, v_s[w]), Cfg::TILE + 512);
            tma_load_5d(smem + Cfg::OFF_V + (w * NKV + v_s[w]) * Cfg::TILE, &tmV, v_full(w, v_s[w]), 0, j * 128, h,
                        o, b);
            tma_load_3d(smem + Cfg::OFF_MASK + (w * NKV + v_s[w]) * 512, &tmMask, v_full(w, v_s[w]), j * 128, o, b);
            if (++v_s[w] == NKV) {
              v_s[w] = 0;
              v_ph[w] ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == Cfg::WARP_MMA) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      constexpr uint32_t swz = swizzle_mode_for_bytes(Cfg::SWZ);
      uint32_t q_ph[2] = {0, 0};
      int k_s[2] = {0, 0}, v_s[2] = {0, 0};
      uint32_t k_ph[2] = {0, 0}, v_ph[2] = {0, 0};
      uint32_t sfree_ph[2] = {0, 0}, pready_ph[2] = {0, 0};

      auto issue_qk = [&](int w, bool last) {
        mbar_wait(k_full(w, k_s[w]), k_ph[w], wctx);
        tc_fence_after();
        const uint32_t qa = smem_u32(smem + Cfg::OFF_Q + w * Cfg::TILE);
        const uint32_t ka = smem_u32(smem + Cfg::OFF_K + (w * NKV + k_s[w]) * Cfg::TILE);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_ss(tmem_base + Cfg::TM_S + 128 * w, make_smem_desc(qa + ks * 32, 16, 8 * Cfg::SWZ, swz),
                  make_smem_desc(ka + ks * 32, 16, 8 * Cfg::SWZ, swz), idesc_qk, ks != 0);
        umma_commit(s_full(w));
        umma_commit(k_empty(w, k_s[w]));
        if (last) umma_commit(q_empty(w));
        if (++k_s[w] == NKV) {
          k_s[w] = 0;
          k_ph[w] ^= 1;
        }
      };

      for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
        int b, h, qt, o2;
        decode(item, b, h, qt, o2);
        bool valid[2] = {2 * o2 < p.O, 2 * o2 + 1 < p.O};
        for (int w = 0; w < 2; ++w) {
          if (!valid[w]) continue;
          mbar_wait(q_full(w), q_ph[w], wctx);
          q_ph[w] ^= 1;
          issue_qk(w, KT == 1);
        }
        for (int j = 0; j < KT; ++j) {
          for (int w = 0; w < 2; ++w) {
            if (!valid[w]) continue;
            // the group has copied S(j) to registers: S can be overwritten by the next Q K^T
            mbar_wait(s_free(w), sfree_ph[w], wctx);
            sfree_ph[w] ^= 1;
            if (j + 1 < KT) issue_qk(w, j + 2 == KT);
          }
          for (int w = 0; w < 2; ++w) {
            if (!valid[w]) continue;
            mbar_wait(p_ready(w), pready_ph[w], wctx);
            pready_ph[w] ^= 1;
            mbar_wait(v_full(w, v_s[w]), v_ph[w], wctx);
            tc_fence_after();
            const uint32_t pa = smem_u32(smem + Cfg::OFF_P + w * Cfg::P_BYTES);
            const uint32_t va = smem_u32(smem + Cfg::OFF_V + (w * NKV + v_s[w]) * Cfg::TILE);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ss(tmem_base + Cfg::TM_O + 64 * w,
                      make_smem_desc(pa + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, swizzle_mode_for_bytes(128)),
                      make_smem_desc(va + ks * 16 * Cfg::SWZ, 128 * Cfg::SWZ, 8 * Cfg::SWZ, swz), idesc_pv, (ks | j) != 0);
            umma_commit(pv_done(w));
            umma_commit(v_empty(w, v_s[w]));
            if (++v_s[w] == NKV) {
              v_s[w] = 0;
              v_ph[w] ^= 1;
            }
          }
        }
      }
    }
  } else if (warp < 16) {
    // ------------------------------------------------------------------ softmax warps
    // Two groups of 8 warps (one per outer row of the pair).  Inside a group, warps q and q+4
    // share the 32 query rows of TMEM lane quarter q and split the 128 keys of a tile in two
    // halves; they agree on the row maximum through a 64-thread named barrier.
    const int w = warp >> 3;
    const int hf = (warp >> 2) & 1;
    const int qd = warp & 3;
    const int row = 32 * qd + lane;  // query row inside the tile == TMEM lane
    constexpr int DH = D / 2;        // output columns per thread
    const uint32_t t_s = tmem_addr(tmem_base, 32 * qd, Cfg::TM_S + 128 * w + 64 * hf);
    const uint32_t t_o = tmem_addr(tmem_base, 32 * qd, Cfg::TM_O + 64 * w + DH * hf);
    uint8_t* p_row = smem + Cfg::OFF_P + w * Cfg::P_BYTES + hf * 16384 + row * 128;
    float* xchg = reinterpret_cast<float*>(smem + Cfg::OFF_XCHG);
    const int pair_bar = 1 + w * 4 + qd;
    constexpr float kLog2e = 1.4426950408889634f;
    constexpr float kLn2 = 0.6931471805599453f;
    const float scale = p.scale;
    const uint64_t scale2 = f2_pack(scale, scale);
    const uint64_t log2e2 = f2_pack(kLog2e, kLog2e);

    uint32_t sfull_ph = 0, pv_ph = 0, b_ph = 0, v_ph = 0;
    int b_s = 0, v_s = 0, par = 0;

    // value held by the partner thread (same row, other key half)
    auto exchange = [&](float mine) -> float {
      xchg[((par * 2 + w) * 2 + hf) * 128 + row] = mine;
      named_barrier_sync(pair_bar, 64);
      const float other = xchg[((par * 2 + w) * 2 + (hf ^ 1)) * 128 + row];
      par ^= 1;
      return other;
    };

    for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
      int b, h, qt, o2;
      decode(item, b, h, qt, o2);
      const int o = 2 * o2 + w;
      if (o >= p.O) {
        // keep the shared bias ring moving
        for (int j = 0; j < KT; ++j) {
          mbar_wait(&b_full[b_s], b_ph, wctx);
          __syncwarp();
          if (lane == 0) mbar_arrive(&b_empty[b_s]);
          if (++b_s == NB) {
            b_s = 0;
            b_ph ^= 1;
          }
        }
        continue;
      }

      // Running reference max (natural-log units) and this thread's share of the row sum.  The
      // output accumulates in TMEM across key tiles; it is rescaled only when the row max grows
      // by more than kRescaleGap, so the common case costs no TMEM round trip.
      float m_ref = -INFINITY, l_part = 0.f;
      constexpr float kRescaleGap = 5.0f;

      for (int j = 0; j < KT; ++j) {
        uint64_t s2[32];  // 64 logits as fp32 pairs
        mbar_wait(s_full(w), sfull_ph, wctx);
        sfull_ph ^= 1;
        mbar_wait(v_full(w, v_s), v_ph, wctx);  // mask row travels with V
        mbar_wait(&b_full[b_s], b_ph, wctx);
        tc_fence_after();
        {
          uint32_t(*raw)[32] = reinterpret_cast<uint32_t(*)[32]>(s2);
          tmem_ld32(t_s, raw[0]);
          tmem_ld32(t_s + 32, raw[1]);
          tmem_ld_wait();
        }
        const uint8_t* bias_row = smem + Cfg::OFF_BIAS + b_s * Cfg::BIAS_STAGE + hf * 16384 + row * 128;
        const float* mask_row =
            reinterpret_cast<const float*>(smem + Cfg::OFF_MASK + (w * NKV + v_s) * 512) + 64 * hf;
        const bool tail = (j + 1) * 128 > p.N;
        float tmax4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int u = 0; u < 8; ++u) {  // 8 key columns per step
          const uint4 bv = *reinterpret_cast<const uint4*>(bias_row + ((u ^ (row & 7)) << 4));
          const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
          const ulonglong2 mkA = *reinterpret_cast<const ulonglong2*>(mask_row + 8 * u);
          const ulonglong2 mkB = *reinterpret_cast<const ulonglong2*>(mask_row + 8 * u + 4);
          const uint64_t mk2[4] = {mkA.x, mkA.y, mkB.x, mkB.y};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint64_t b2 = f2_pack_bits(bw[e] << 16, bw[e] & 0xFFFF0000u);
            uint64_t v2 = f2_add(f2_fma(s2[4 * u + e], scale2, b2), mk2[e]);
            float v0, v1;
            f2_unpack(v2, v0, v1);
            if (tail) {
              const int k0 = j * 128 + 64 * hf + 8 * u + 2 * e;
              if (k0 >= p.N) v0 = -INFINITY;
              if (k0 + 1 >= p.N) v1 = -INFINITY;
              v2 = f2_pack(v0, v1);
            }
            s2[4 * u + e] = v2;
            tmax4[e] = max3(tmax4[e], v0, v1);
          }
        }
        // S, the bias tile and the mask row now live in registers
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(s_free(w));
          mbar_arrive(&b_empty[b_s]);
        }
        if (++b_s == NB) {
          b_s = 0;
          b_ph ^= 1;
        }
        if (++v_s == NKV) {
          v_s = 0;
          v_ph ^= 1;
        }

        const float tmax = fmaxf(fmaxf(tmax4[0], tmax4[1]), fmaxf(tmax4[2], tmax4[3]));
        const float m_new = max3(m_ref, tmax, exchange(tmax));
        if (j == 0) {
          m_ref = m_new;
        } else {
          // P V of the previous tile must be complete before P is overwritten or O is rescaled
          mbar_wait(pv_done(w), pv_ph, wctx);
          pv_ph ^= 1;
          tc_fence_after();
          if (__any_sync(0xffffffffu, m_new > m_ref + kRescaleGap)) {
            const float f = (m_new == -INFINITY) ? 1.f : ex2_approx((m_ref - m_new) * kLog2e);
#pragma unroll
            for (int c = 0; c < DH; c += 8) {
              uint32_t ro[8];
              tmem_ld8(t_o + c, ro);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 8; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * f);
              tmem_st8(t_o + c, ro);
            }
            tmem_st_wait();
            l_part *= f;
            m_ref = m_new;
          }
        }
        const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * kLog2e;
        const uint64_t neg_m2 = f2_pack(neg_m, neg_m);

        uint64_t rs2[2] = {0ull, 0ull};  // two packed partial sums (bit pattern of +0.f pairs)
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float a0, a1;
            f2_unpack(f2_fma(s2[4 * u + e], log2e2, neg_m2), a0, a1);
            const float e0 = ex2_approx(a0), e1 = ex2_approx(a1);
            rs2[e & 1] = f2_add(rs2[e & 1], f2_pack(e0, e1));
            pk[e] = pack_bf16x2(e0, e1);
          }
          *reinterpret_cast<uint4*>(p_row + ((u ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        {
          float r0, r1, r2, r3;
          f2_unpack(rs2[0], r0, r1);
          f2_unpack(rs2[1], r2, r3);
          l_part += (r0 + r1) + (r2 + r3);
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready(w));
      }

      // last tile's P V, then this thread's half of the accumulated output columns
      mbar_wait(pv_done(w), pv_ph, wctx);
      pv_ph ^= 1;
      tc_fence_after();
      float acc[DH];
#pragma unroll
      for (int c = 0; c < DH; c += 8) {
        uint32_t ro[8];
        tmem_ld8(t_o + c, ro);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[c + i] = __uint_as_float(ro[i]);
      }
      tc_fence_before();
      const float l_other = exchange(l_part);
      const float l_run = hf == 0 ? l_part + l_other : l_other + l_part;

      const int q = qt * 128 + row;
      if (q < p.N) {
        const float inv = l_run > 0.f ? __fdividef(1.f, l_run) : 0.f;
        __nv_bfloat16* orow = p.out + ((((int64_t)b * p.O + o) * p.N + q) * p.H + h) * D + DH * hf;
#pragma unroll
        for (int c = 0; c < DH; c += 8) {
          uint4 pk;
          pk.x = pack_bf16x2(acc[c + 0] * inv, acc[c + 1] * inv);
          pk.y = pack_bf16x2(acc[c + 2] * inv, acc[c + 3] * inv);
          pk.z = pack_bf16x2(acc[c + 4] * inv, acc[c + 5] * inv);
          pk.w = pack_bf16x2(acc[c + 6] * inv, acc[c + 7] * inv);
          *reinterpret_cast<uint4*>(orow + c) = pk;
        }
        if (hf == 0)
          p.lse[(((int64_t)b * p.O + o) * p.H + h) * p.N + q] =
              l_run > 0.f ? m_ref + log2f(l_run) * kLn2 : -INFINITY;
      }
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
int make_qkv_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t H, int64_t N, int64_t D,
                  const int64_t* st, int swz) {
  uint64_t dims[5] = {(uint64_t)D, (uint64_t)N, (uint64_t)H, (uint64_t)O, (uint64_t)B};
  uint64_t strides[4] = {(uint64_t)st[3] * 2, (uint64_t)st[2] * 2, (uint64_t)st[1] * 2, (uint64_t)st[0] * 2};
  uint32_t box[5] = {(uint32_t)D, 128, 1, 1, 1};
  return make_tmap_bf16(tm, base, 5, dims, strides, box, swz);
}

// 4-D map over the bf16 bias [Bb,H,N,N] whose rows are `pitch` elements apart.
int make_bias_tmap(CUtensorMap* tm, const void* base, int64_t Bb, int64_t H, int64_t N, int64_t pitch) {
  uint64_t dims[4] = {(uint64_t)N, (uint64_t)N, (uint64_t)H, (uint64_t)Bb};
  uint64_t strides[3] = {(uint64_t)pitch * 2, (uint64_t)pitch * N * 2, (uint64_t)pitch * N * H * 2};
  uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, 128);
}

// 3-D map over the fp32 additive mask [B,O,N] whose rows are `pitch` elements apart.
int make_mask_tmap(CUtensorMap* tm, const void* base, int64_t B, int64_t O, int64_t N, int64_t pitch) {
  uint64_t dims[3] = {(uint64_t)N, (uint64_t)O, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)pitch * 4, (uint64_t)pitch * O * 4};
  uint32_t box[3] = {128, 1, 1};
  return make_tmap_f32(tm, base, 3, dims, strides, box);
}

template <int D, int NKV>
int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tb,
                    const CUtensorMap& tmk, const AttnFwdParams& p, int* status, cudaStream_t stream) {
  using Cfg = AttnFwdCfg<D, NKV>;
  auto kern = attn_fwd_kernel<Cfg>;
  static PerDeviceOnce once;  // per instantiation
  if (int rc = ensure_dynamic_smem(kern, Cfg::SMEM_BYTES, once)) return rc;
  int grid = sm_count();
  if (grid > p.n_items) grid = p.n_items;
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tb, tmk, p, status);
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
  TPF_REQUIRE((reinterpret_cast<uintptr_t>(lse) & 3) == 0, TPF_ERR_INVALID_ARGUMENT, "attn_fwd: lse must be 4-byte aligned");
  const int swz = 2 * (int)D;
  CUtensorMap tq, tk, tv, tb, tm;
  int rc;
  if ((rc = make_qkv_tmap(&tq, q, B, O, H, N, D, q_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tk, k, B, O, H, N, D, k_strides, swz))) return rc;
  if ((rc = make_qkv_tmap(&tv, v, B, O, H, N, D, v_strides, swz))) return rc;
  if ((rc = make_bias_tmap(&tb, bias, bias_batch, H, N, bias_pitch))) return rc;
  if ((rc = make_mask_tmap(&tm, mask, B, O, N, mask_pitch))) return rc;
  AttnFwdParams p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = (int)B; p.O = (int)O; p.H = (int)H; p.N = (int)N;
  p.q_tiles = (int)((N + 127) / 128);
  p.k_tiles = p.q_tiles;
  p.o_pairs = (int)((O + 1) / 2);
  p.bias_broadcast = bias_batch == 1 && B > 1 ? 1 : 0;
  p.scale = scale;
  const int64_t items = B * H * p.q_tiles * p.o_pairs;
  TPF_REQUIRE(items < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "attn_fwd: too many work items");
  p.n_items = (int)items;
  int* status = nullptr;
  {
    static PerDeviceAddress cache;
    if ((rc = device_symbol_address(g_attn_fwd_status, cache, reinterpret_cast<void**>(&status)))) return rc;
  }
  if (D == 16) return launch_attn_fwd<16, 2>(tq, tk, tv, tb, tm, p, status, stream);
  if (D == 32) return launch_attn_fwd<32, 2>(tq, tk, tv, tb, tm, p, status, stream);
  return launch_attn_fwd<64, 1>(tq, tk, tv, tb, tm, p, status, stream);
}

}  // namespace tpf
