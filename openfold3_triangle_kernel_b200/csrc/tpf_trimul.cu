// Triangle multiplicative update (outgoing / incoming), forward and backward, for sm_100a.
//
//   zn  = LayerNorm_in(z)                                  a = (zn Wap^T) * sigmoid(zn Wag^T) * mask
//   x[i,j,c] = sum_k a[i,k,c] b[j,k,c]   (outgoing)        b = (zn Wbp^T) * sigmoid(zn Wbg^T) * mask
//   x[i,j,c] = sum_k a[k,i,c] b[k,j,c]   (incoming)        out = (LayerNorm_out(x) Wz^T) * sigmoid(zn Wg^T)
//
// Stands in for the reference's native TriMul stages and the cuBLAS calls between them
// (openfold3/core/kernels/turbopairformer/turbopairformer_trimul_cuda.cu:634-1047, 1202-1470,
//  1541-1809, 226-438 and turbopairformer_trimul.py:184-392).  Rounding points follow the
// reference: fp32 master weights are rounded to bf16 once, LayerNorm statistics are fp32 with
// var = E[x^2] - mean^2 and eps = 1e-5, intermediates (zn, a, b, gate logits, x) are bf16,
// weight gradients are fp32 sums folded in a fixed order.
//
// Every GEMM-shaped stage runs on the tcgen05 engine of tpf_gemm.cuh; gating, masking and the
// channel-major re-layout that the k-contraction wants are fused into GEMM epilogues.  The
// a / b / x tensors live channel-major ([B*C][N*N]) so that the k-contraction is a plain batched
// GEMM in both directions (K-major operands when outgoing, MN-major when incoming).
#include "tpf_gemm_host.cuh"

namespace tpf {

static __device__ int g_trimul_status;

int trimul_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  TPF_CUDA_OK(cudaMemcpyFromSymbol(&v, g_trimul_status, sizeof(int)));
  if (v) TPF_CUDA_OK(cudaMemcpyToSymbol(g_trimul_status, &zero, sizeof(int)));
  *out = v;
  return TPF_OK;
}

int bmm_bf16(const void* A, int64_t lda, int64_t bsa, int a_mn, const void* B, int64_t ldb, int64_t bsb, int b_mn,
             void* D, int64_t ldd, int64_t bsd, int out_f32, int64_t M, int64_t N, int64_t K, int64_t batch,
             int64_t k_per_split, int swizzle_bytes, cudaStream_t stream);

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

// =============================================================================================
// weight packing: fp32 masters -> bf16 W5 [5C,C] = [a_p; a_g; b_p; b_g; g], W5T [C,5C], Wz [C,C], WzT [C,C]
// =============================================================================================
__global__ void trimul_pack_weights_kernel(const float* __restrict__ p_in, const float* __restrict__ g_in,
                                           const float* __restrict__ p_out, const float* __restrict__ g_out,
                                           bf16* __restrict__ W5, bf16* __restrict__ W5T, bf16* __restrict__ Wz,
                                           bf16* __restrict__ WzT, int C) {
  griddep_wait();
  const int n = 5 * C * C;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int row = i / C, col = i % C;
    const int blk = row / C, r = row % C;
    float v;
    if (blk == 0) v = p_in[r * C + col];
    else if (blk == 1) v = g_in[r * C + col];
    else if (blk == 2) v = p_in[(C + r) * C + col];
    else if (blk == 3) v = g_in[(C + r) * C + col];
    else v = g_out[r * C + col];
    const bf16 h = __float2bfloat16(v);
    W5[i] = h;
    W5T[col * 5 * C + row] = h;
    if (i < C * C) {
      const bf16 hz = __float2bfloat16(p_out[i]);
      Wz[i] = hz;
      WzT[col * C + row] = hz;
    }
  }
}

// =============================================================================================
// LayerNorm over the last dim of a row-major [R,C] bf16 tensor (input norm), forward
// =============================================================================================
// Row-wise LayerNorm kernels: a lane owns 8 consecutive channels (one 16-byte load), the lanes of a row
// sit in a slot of LS lanes (a power of two; the lanes beyond C / 8 of a slot idle when C = 96), and a warp
// works on 32 / LS rows at a time.
template <int C>
struct RowLanes {
  static constexpr int LPR = C / 8;                               // lanes that hold a row
  static constexpr int LS = LPR <= 4 ? 4 : LPR <= 8 ? 8 : 16;     // lanes per row slot
  static constexpr int RPW = 32 / LS;                             // rows per warp step
};

template <int C>
__device__ __forceinline__ float slot_sum(float v) {
#pragma unroll
  for (int off = RowLanes<C>::LS / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
  x[0] = bf16_lo(u.x); x[1] = bf16_hi(u.x); x[2] = bf16_lo(u.y); x[3] = bf16_hi(u.y);
  x[4] = bf16_lo(u.z); x[5] = bf16_hi(u.z); x[6] = bf16_lo(u.w); x[7] = bf16_hi(u.w);
}

template <int C>
__global__ void __launch_bounds__(256) trimul_ln_fwd_kernel(const bf16* __restrict__ z, const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, bf16* __restrict__ zln,
                                                            float* __restrict__ mean, float* __restrict__ rstd,
                                                            int64_t R) {
  griddep_wait();
  using L = RowLanes<C>;
  constexpr int G = 4;  // row groups per warp, all loads issued before the first use
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int sub = lane / L::LS, part = lane % L::LS;
  const bool on = part < L::LPR;
  float g[8], b[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    g[e] = on ? gamma[part * 8 + e] : 0.f;
    b[e] = on ? beta[part * 8 + e] : 0.f;
  }
  uint4 u[G];
  bool active[G];
#pragma unroll
  for (int r = 0; r < G; ++r) {
    const int64_t row = (warp * G + r) * L::RPW + sub;
    active[r] = on && row < R;
    u[r] = make_uint4(0u, 0u, 0u, 0u);
    if (active[r]) u[r] = *reinterpret_cast<const uint4*>(z + row * C + part * 8);
  }
#pragma unroll
  for (int r = 0; r < G; ++r) {
    const int64_t row = (warp * G + r) * L::RPW + sub;
    float x[8];
    unpack8(u[r], x);
    float a1 = 0.f, a2 = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      a1 += x[e];
      a2 += x[e] * x[e];
    }
    const float s1 = slot_sum<C>(a1);
    const float s2 = slot_sum<C>(a2);
    const float mu = s1 * (1.f / C);
    const float var = fmaxf(s2 * (1.f / C) - mu * mu, 0.f);
    const float rs = rsqrtf(var + 1e-5f);
    if (active[r]) {
      uint4 o;
      o.x = pack_bf16x2((x[0] - mu) * rs * g[0] + b[0], (x[1] - mu) * rs * g[1] + b[1]);
      o.y = pack_bf16x2((x[2] - mu) * rs * g[2] + b[2], (x[3] - mu) * rs * g[3] + b[3]);
      o.z = pack_bf16x2((x[4] - mu) * rs * g[4] + b[4], (x[5] - mu) * rs * g[5] + b[5]);
      o.w = pack_bf16x2((x[6] - mu) * rs * g[6] + b[6], (x[7] - mu) * rs * g[7] + b[7]);
      *reinterpret_cast<uint4*>(zln + row * C + part * 8) = o;
      if (part == 0) {
        mean[row] = mu;
        rstd[row] = rs;
      }
    }
  }
}

// =============================================================================================
// Output norm forward: channel-major x [B*C][NN] -> row-major LayerNorm(x) [R,C] + mean/rstd
// =============================================================================================
// The channel-major -> row-major turn is done on 8x8 blocks of bf16 by ldmatrix.trans instead of element by
// element through shared memory: the tile is stored as it is loaded (16 bytes = 8 pair rows of one
// channel), every lane then holds, per 8-channel group, two neighbouring channels of ONE pair row, so
// the LayerNorm statistics are a register sum plus two shuffles, and the normalised row goes back
// through a row-major staging tile that is read out in 16-byte pieces.  About one shared-memory
// instruction per element instead of four.
template <int C>
__global__ void __launch_bounds__(256, 2) trimul_xnorm_fwd_kernel(const bf16* __restrict__ x_cm,
                                                                  const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta,
                                                                  bf16* __restrict__ xln, float* __restrict__ mean,
                                                                  float* __restrict__ rstd, int64_t NN,
                                                                  int tiles_per_batch, int n_tiles) {
  griddep_wait();
  constexpr int TR = 64;                    // pair rows per tile; warp w owns rows 8w .. 8w+7
  constexpr int IN_PITCH = TR * 2 + 16;     // bytes per channel row of the input tile (+16: conflict-free ldmatrix)
  constexpr int OUT_PITCH = C * 2 + 16;     // bytes per pair row of the staging tile
  constexpr int NG = C / 32;                // ldmatrix.x4 steps: 4 groups of 8 channels each
  extern __shared__ __align__(16) uint8_t xnorm_smem[];
  uint8_t* xs0 = xnorm_smem;                       // two input tiles: the next one is fetched (cp.async)
  uint8_t* ys = xnorm_smem + 2 * C * IN_PITCH;     // while the current one is processed
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k2 = 2 * (lane & 3);            // this lane's channel pair inside an 8-channel group
  const int rr = 8 * warp + (lane >> 2);    // this lane's pair row inside the tile
  float2 g[NG][4], bt[NG][4];
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      g[i][m] = *reinterpret_cast<const float2*>(gamma + 32 * i + 8 * m + k2);
      bt[i][m] = *reinterpret_cast<const float2*>(beta + 32 * i + 8 * m + k2);
    }
  // 16-byte copies: 8 consecutive pair rows of one channel (NN is a multiple of 8)
  auto fetch = [&](int tile, uint8_t* dst) {
    const int fb = tile / tiles_per_batch;
    const int64_t f0 = (int64_t)(tile % tiles_per_batch) * TR;
#pragma unroll
    for (int idx = threadIdx.x; idx < C * (TR / 8); idx += 256) {
      const int c = idx / (TR / 8), j8 = idx % (TR / 8);
      const bool ok = f0 + 8 * j8 < NN;
      cp_async_16(dst + c * IN_PITCH + 16 * j8, x_cm + ((int64_t)fb * C + c) * NN + (ok ? f0 + 8 * j8 : 0), ok);
    }
    cp_async_commit();
  };
  int buf = 0;
  if ((int)blockIdx.x < n_tiles) fetch(blockIdx.x, xs0);
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, buf ^= 1) {
    const int bb = tile / tiles_per_batch;
    const int64_t r0 = (int64_t)(tile % tiles_per_batch) * TR;
    uint8_t* xs = xs0 + buf * C * IN_PITCH;
    // the other buffer was last read (ldmatrix) before the barriers of the previous iteration
    if (tile + (int)gridDim.x < n_tiles) {
      fetch(tile + gridDim.x, xs0 + (buf ^ 1) * C * IN_PITCH);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    uint32_t fr[NG][4];
#pragma unroll
    for (int i = 0; i < NG; ++i)
      ldmatrix_x4_trans(fr[i], smem_u32(xs + (32 * i + lane) * IN_PITCH + 16 * warp));
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i)
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float v0 = bf16_lo(fr[i][m]), v1 = bf16_hi(fr[i][m]);
        s1 += v0 + v1;
        s2 += v0 * v0 + v1 * v1;
      }
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
    const float mu = s1 * (1.f / C);
    const float rs = rsqrtf(fmaxf(s2 * (1.f / C) - mu * mu, 0.f) + 1e-5f);
#pragma unroll
    for (int i = 0; i < NG; ++i)
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float y0 = (bf16_lo(fr[i][m]) - mu) * rs * g[i][m].x + bt[i][m].x;
        const float y1 = (bf16_hi(fr[i][m]) - mu) * rs * g[i][m].y + bt[i][m].y;
        *reinterpret_cast<uint32_t*>(ys + rr * OUT_PITCH + (32 * i + 8 * m + k2) * 2) = pack_bf16x2(y0, y1);
      }
    if ((lane & 3) == 0 && r0 + rr < NN) {
      mean[(int64_t)bb * NN + r0 + rr] = mu;
      rstd[(int64_t)bb * NN + r0 + rr] = rs;
    }
    __syncthreads();
    // row-major stores: 16 bytes (8 channels) per thread, a warp covers two whole rows
#pragma unroll
    for (int idx = threadIdx.x; idx < TR * (C / 8); idx += 256) {
      const int j = idx / (C / 8), c8 = idx % (C / 8);
      if (r0 + j < NN)
        *reinterpret_cast<uint4*>(xln + ((int64_t)bb * NN + r0 + j) * C + 8 * c8) =
            *reinterpret_cast<const uint4*>(ys + j * OUT_PITCH + 16 * c8);
    }
    // the next iteration's first barrier orders these reads before the staging tile is rewritten; the
    // input tile is rewritten only after every warp has passed the barrier above, i.e. after its ldmatrix
  }
}

// =============================================================================================
// GEMM epilogues
// =============================================================================================
// Projection + gating.  GEMM N axis = [a_p | a_g] [b_p | b_g] [g | pad], one tile of width 2C each.
// a and b are stored channel-major.  Each lane owns one row of the accumulator tile, which would
// make 2-byte scattered stores; the 32x32 block is transposed through a per-warp smem tile so
// that each lane writes 32 consecutive rows of ONE channel (4 x 16 bytes).
// Integer divisions by run-time values cost a lone epilogue warp 300-600 cycles each (a chain of conversions and
// a reciprocal on the XU pipe), once per tile and on its critical path, so the epilogues avoid them: the tile
// kind comes from comparisons, and the batch entry of a row is found by division only when there is more than one.
__device__ __forceinline__ int tile_kind(int n0, int C) { return n0 >= 4 * C ? 2 : n0 >= 2 * C ? 1 : 0; }
__device__ __forceinline__ void split_row(int row, int64_t NN, int M, int& bb, int& rr) {
  if ((int64_t)M <= NN) {  // one batch entry
    bb = 0;
    rr = row;
  } else {
    bb = (int)((uint32_t)row / (uint32_t)NN);
    rr = row - bb * (int)NN;
  }
}

struct EpiProjGate {
  struct Params {
    bf16* a_cm;        // [B*C][NN]
    bf16* b_cm;        // [B*C][NN]
    bf16* gate;        // [R][C] raw gate logits
    const float* mask; // [R]
    int C;
    int64_t NN;
  };
  static constexpr bool kPaired = true;
  static constexpr bool kStaged = false;
  static constexpr int kSmemPerWarp = 32 * 33 * 4;
  struct Pre {
    float mk;  // pair mask: of this lane's row, or (exchanged tile) of row `lane` of the warp's 32-row chunk
  };
  // At C = 128 the a and b tiles are computed with the operand roles exchanged: accumulator lane = channel,
  // accumulator column = pair row, so a lane holds 32 consecutive pair rows of ONE channel, which is 64
  // contiguous bytes of the channel-major output, and no transpose is needed.  The gate tile (row-major
  // output) keeps lane = pair row.
  __device__ static __forceinline__ bool swapped(const Params& p, int n0) { return n0 < 4 * p.C; }
  __device__ static __forceinline__ void prefetch2(const Params& p, const GemmShape& sh, int, int m0, int rit, int,
                                                   int c0, int lane, bool swap, Pre& pre) {
    const int m = swap ? m0 + c0 + lane : m0 + rit;
    pre.mk = (m < sh.M) ? p.mask[m] : 0.f;
  }
  __device__ static __forceinline__ void apply2(const Params& p, const GemmShape& sh, int, int m0, int rit, int n0,
                                                int c0, const float (&v0)[32], const float (&v1)[32], float* wsm,
                                                int lane, bool swap, const Pre& pre) {
    const int which = tile_kind(n0, p.C);
    if (swap) {
      // lane = channel `rit`; v0[i] / v1[i] = projection / gate logit of pair row m0 + c0 + i
      wsm[lane] = pre.mk;
      __syncwarp();
      const uint64_t half2 = f2_pack(0.5f, 0.5f);
      uint32_t ow[16];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 mk = reinterpret_cast<const float4*>(wsm)[q];  // same address in every lane: one broadcast
        const float mks[4] = {mk.x, mk.y, mk.z, mk.w};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int i = 4 * q + 2 * e;
          float h0, h1, a0, a1;
          f2_unpack(f2_mul(f2_pack(v1[i], v1[i + 1]), half2), h0, h1);
          const uint64_t sg = f2_fma(f2_pack(tanh_fast(h0), tanh_fast(h1)), half2, half2);
          const uint64_t pm = f2_mul(f2_pack(v0[i], v0[i + 1]), f2_pack(mks[2 * e], mks[2 * e + 1]));
          f2_unpack(f2_mul(pm, sg), a0, a1);
          ow[2 * q + e] = pack_bf16x2(a0, a1);
        }
      }
      __syncwarp();  // the mask row has been read: the scratch becomes the staging tile
      // Rows (and the sharded row count) are multiples of 64, so the 32-row chunk lies inside one batch entry
      // and is inside M as a whole or not at all.  A lane's 64 bytes go out through the staging tile so that one
      // store instruction covers 8 channels x 64 contiguous bytes instead of 32 channels x 16 bytes.
      const int r0 = m0 + c0;
      int bb, rr;
      split_row(r0, p.NN, sh.M, bb, rr);
      bf16* blk = (which == 0 ? p.a_cm : p.b_cm) + ((int64_t)bb * p.C + (rit - lane)) * p.NN + rr;  // channel of lane 0
      const bool ok = r0 < sh.M;
      warp_tile_store(reinterpret_cast<uint8_t*>(wsm), lane, ow,
                      [&](int r) -> bf16* { return ok ? blk + (int64_t)r * p.NN : nullptr; });
      return;
    }
    const int m = m0 + rit;
    const int m_base = m - lane;  // first row of this warp's 32-row block (a multiple of 32)
    if (which == 2) {
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(v0[2 * i], v0[2 * i + 1]);
      bf16* blk = p.gate + c0;
      warp_tile_store(reinterpret_cast<uint8_t*>(wsm), lane, pk, [&](int r) -> bf16* {
        return m_base + r < sh.M ? blk + (int64_t)(m_base + r) * p.C : nullptr;
      });
      return;
    }
    // a / b tile with lane = pair row (C < 128): each lane owns one row of the accumulator tile, which would
    // make 2-byte scattered stores; the 32x32 block is transposed through a per-warp smem tile so that each
    // lane writes 8 consecutive rows of four channels (4 x 16 bytes).
    const float mk = pre.mk;
#pragma unroll
    for (int i = 0; i < 32; ++i) wsm[lane * 33 + i] = v0[i] * sigmoid_fast(v1[i]) * mk;
    __syncwarp();
    // four lanes per channel: each store instruction covers 8 channels x 64 contiguous bytes (32 rows)
    int bb, rr;
    split_row(m_base, p.NN, sh.M, bb, rr);
    const int piece = lane & 3;  // rows 8*piece .. 8*piece+7 of the block
    bf16* dst = (which == 0 ? p.a_cm : p.b_cm) + ((int64_t)bb * p.C + c0 + (lane >> 2)) * p.NN + rr + 8 * piece;
    const float* col = wsm + (8 * piece) * 33 + (lane >> 2);
    const bool ok = m_base + 8 * piece + 7 < sh.M;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const float* cg = col + 8 * g;  // channel 8*g + lane/4
      uint4 u;
      u.x = pack_bf16x2(cg[0 * 33], cg[1 * 33]);
      u.y = pack_bf16x2(cg[2 * 33], cg[3 * 33]);
      u.z = pack_bf16x2(cg[4 * 33], cg[5 * 33]);
      u.w = pack_bf16x2(cg[6 * 33], cg[7 * 33]);
      if (ok) *reinterpret_cast<uint4*>(dst + (int64_t)(8 * g) * p.NN) = u;
    }
    __syncwarp();
  }
};

// Output projection: out = acc * sigmoid(gate)
struct EpiOutGate {
  struct Params {
    bf16* out;        // [R][C]
    const bf16* gate; // [R][C]
    int C;
  };
  static constexpr bool kPaired = false;
  static constexpr bool kStaged = false;
  static constexpr int kSmemPerWarp = 2048;
  struct Pre {
    uint4 g[4];  // 32 gate logits of this lane's row
  };
  __device__ static __forceinline__ void prefetch(const Params& p, const GemmShape& sh, int, int m, int n0, int,
                                                  Pre& pre) {
    if (m >= sh.M) return;
    const uint4* g = reinterpret_cast<const uint4*>(p.gate + (int64_t)m * p.C + n0);
#pragma unroll
    for (int i = 0; i < 4; ++i) pre.g[i] = g[i];
  }
  __device__ static __forceinline__ void apply(const Params& p, const GemmShape& sh, int, int m, int n0,
                                               const float (&v)[32], float* wsm, int lane, const Pre& pre) {
    uint32_t ow[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 gu = m < sh.M ? pre.g[i] : make_uint4(0u, 0u, 0u, 0u);
      const uint32_t gw[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        ow[4 * i + e] = pack_bf16x2(v[8 * i + 2 * e] * sigmoid_fast(bf16_lo(gw[e])),
                                    v[8 * i + 2 * e + 1] * sigmoid_fast(bf16_hi(gw[e])));
    }
    const int m_base = m - lane;
    bf16* blk = p.out + n0;
    warp_tile_store(reinterpret_cast<uint8_t*>(wsm), lane, ow, [&](int r) -> bf16* {
      return m_base + r < sh.M ? blk + (int64_t)(m_base + r) * p.C : nullptr;
    });
  }
};

// Backward of the gated projections: recomputed (p, g) pair + incoming d_a / d_b -> d_proj5[:, 0:4C]
struct EpiGateSplitBwd {
  struct Params {
    const bf16* da_cm;  // [B*C][NN]
    const bf16* db_cm;
    const float* mask;  // [R]
    bf16* d_proj5;      // [R][5C]
    int C;
    int64_t NN;
  };
  static constexpr bool kPaired = true;
  static constexpr bool kStaged = true;
  static constexpr int kSmemPerWarp = 32 * 33 * 4;
  struct Pre {
    uint4 d[4];  // incoming gradient, channel-major: d[g] = 8 consecutive rows of channel 8*g + lane/4
    float mk;    // pair mask of this lane's row
  };
  __device__ static __forceinline__ bool swapped(const Params&, int) { return false; }
  __device__ static __forceinline__ void prefetch2(const Params& p, const GemmShape& sh, int, int m0, int rit, int n0,
                                                   int c0, int lane, bool, Pre& pre) {
    const int which = tile_kind(n0, p.C);  // 0: a, 1: b
    const int m = m0 + rit;
    const int m_base = m - lane;
    int bb, rr;
    split_row(m_base, p.NN, sh.M, bb, rr);
    // four lanes per channel: load g reads rows 8*piece..+7 of channel 8*g + lane/4, so one load
    // instruction covers 8 channels x 64 contiguous bytes
    const int piece = lane & 3;
    const bf16* src = (which == 0 ? p.da_cm : p.db_cm) + ((int64_t)bb * p.C + c0 + (lane >> 2)) * p.NN + rr + 8 * piece;
    const bool ok = m_base + 8 * piece + 7 < sh.M;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      pre.d[g] = make_uint4(0u, 0u, 0u, 0u);
      if (ok) pre.d[g] = *reinterpret_cast<const uint4*>(src + (int64_t)(8 * g) * p.NN);
    }
    pre.mk = (m < sh.M) ? p.mask[m] : 0.f;
  }
  // The prefetched channel-major block is transposed through smem so that afterwards lane = row finds
  // its 32 channels at wsm[lane * 33 ..].
  __device__ static __forceinline__ void stage(const Pre& pre, float* wsm, int lane) {
    float* col = wsm + (8 * (lane & 3)) * 33 + (lane >> 2);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 u = pre.d[g];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        col[(2 * e) * 33 + 8 * g] = bf16_lo(w[e]);
        col[(2 * e + 1) * 33 + 8 * g] = bf16_hi(w[e]);
      }
    }
    __syncwarp();
  }
  __device__ static __forceinline__ void apply2(const Params& p, const GemmShape& sh, int, int m0, int rit, int n0,
                                                int c0, const float (&v0)[32], const float (&v1)[32], float* wsm,
                                                int lane, bool, const Pre& pre) {
    const int which = tile_kind(n0, p.C);  // 0: a, 1: b
    const int m = m0 + rit;
    // d = incoming gradient * mask; t = tanh(g / 2): sigmoid s = 0.5 + 0.5 t, s (1 - s) = 0.25 - 0.25 t^2.
    // Channel pairs (i, i + 1) go through packed fp32 arithmetic and are rounded to bf16 at once, so that
    // only the packed results stay live.
    const uint64_t mk2 = f2_pack(pre.mk, pre.mk);
    const uint64_t half2 = f2_pack(0.5f, 0.5f), quarter2 = f2_pack(0.25f, 0.25f), nquarter2 = f2_pack(-0.25f, -0.25f);
    uint32_t pk0[16], pk1[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint64_t d2 = f2_mul(f2_pack(wsm[lane * 33 + 2 * i], wsm[lane * 33 + 2 * i + 1]), mk2);
      float h0, h1, a0, a1, b0, b1;
      f2_unpack(f2_mul(f2_pack(v1[2 * i], v1[2 * i + 1]), half2), h0, h1);
      const uint64_t t2 = f2_pack(tanh_fast(h0), tanh_fast(h1));
      const uint64_t s2 = f2_fma(t2, half2, half2);
      const uint64_t ss2 = f2_fma(f2_mul(t2, nquarter2), t2, quarter2);
      f2_unpack(f2_mul(d2, s2), a0, a1);
      f2_unpack(f2_mul(f2_mul(d2, f2_pack(v0[2 * i], v0[2 * i + 1])), ss2), b0, b1);
      pk0[i] = pack_bf16x2(a0, a1);
      pk1[i] = pack_bf16x2(b0, b1);
    }
    __syncwarp();  // the transposed gradient block has been consumed: its smem is reused as staging tiles
    const int m_base = m - lane;
    bf16* dp = p.d_proj5 + which * 2 * p.C + c0;  // d_p block of row 0
    warp_tile_store(reinterpret_cast<uint8_t*>(wsm), lane, pk0, [&](int r) -> bf16* {
      return m_base + r < sh.M ? dp + (int64_t)(m_base + r) * 5 * p.C : nullptr;
    });
    warp_tile_store(reinterpret_cast<uint8_t*>(wsm) + 2048, lane, pk1, [&](int r) -> bf16* {
      return m_base + r < sh.M ? dp + p.C + (int64_t)(m_base + r) * 5 * p.C : nullptr;  // d_g: C columns further
    });
  }
};

// =============================================================================================
// backward elementwise stages
// =============================================================================================
// d_y = d_out * sigmoid(g);  d_glogit = d_out * out * (1 - sigmoid(g))  -> d_proj5[:, 4C:5C]
__global__ void __launch_bounds__(256) trimul_out_gate_bwd_kernel(const bf16* __restrict__ d_out,
                                                                  const bf16* __restrict__ out,
                                                                  const bf16* __restrict__ gate, bf16* __restrict__ d_y,
                                                                  bf16* __restrict__ d_proj5, int64_t R, int C) {
  griddep_wait();
  const int64_t n8 = R * C / 8;
  const int per_row = C / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 a = reinterpret_cast<const uint4*>(d_out)[i];
    const uint4 b = reinterpret_cast<const uint4*>(out)[i];
    const uint4 g = reinterpret_cast<const uint4*>(gate)[i];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, gw[4] = {g.x, g.y, g.z, g.w};
    uint32_t y[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float s0 = sigmoid_fast(bf16_lo(gw[e])), s1 = sigmoid_fast(bf16_hi(gw[e]));
      const float d0 = bf16_lo(aw[e]), d1 = bf16_hi(aw[e]);
      y[e] = pack_bf16x2(d0 * s0, d1 * s1);
      l[e] = pack_bf16x2(d0 * bf16_lo(bw[e]) * (1.f - s0), d1 * bf16_hi(bw[e]) * (1.f - s1));
    }
    reinterpret_cast<uint4*>(d_y)[i] = make_uint4(y[0], y[1], y[2], y[3]);
    const int64_t row = i / per_row;
    const int col8 = (int)(i % per_row);
    *reinterpret_cast<uint4*>(d_proj5 + row * 5 * C + 4 * C + col8 * 8) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// Output-norm backward.  d_xln row-major [R,C], x channel-major -> d_x channel-major; per-CTA partial sums
// for d_gamma / d_beta (fixed order inside the CTA, folded in CTA order later).
//
// Same data movement as the forward norm: x is stored as loaded and turned by ldmatrix.trans, so that a
// lane holds, for ONE pair row, two neighbouring channels of each 8-channel group; d_xln is staged
// row-major and read back in that same arrangement; d_x goes back through stmatrix.trans into the
// channel-major tile (in place: a warp only touches its own 8 pair rows of every channel) and leaves
// in 16-byte pieces.  The d_gamma / d_beta sums of a lane's channels stay in registers over all the
// tiles of the CTA and are reduced once at the end.
template <int C>
__global__ void __launch_bounds__(256, 2) trimul_xnorm_bwd_kernel(const bf16* __restrict__ d_xln,
                                                                  const bf16* __restrict__ x_cm,
                                                                  const float* __restrict__ gamma,
                                                                  const float* __restrict__ mean,
                                                                  const float* __restrict__ rstd,
                                                                  bf16* __restrict__ dx_cm, float* __restrict__ partials,
                                                                  int64_t NN, int tiles_per_batch, int n_tiles) {
  griddep_wait();
  constexpr int TR = 64;
  constexpr int IN_PITCH = TR * 2 + 16;
  constexpr int OUT_PITCH = C * 2 + 16;
  constexpr int NG = C / 32;
  extern __shared__ __align__(16) uint8_t xnorm_smem[];
  // two (x, d_xln) tile pairs: the next pair is fetched (cp.async) while the current one is processed
  uint8_t* xs0 = xnorm_smem;                          // x, later d_x: [channel][pair row]
  uint8_t* ds0 = xnorm_smem + 2 * C * IN_PITCH;       // d_xln: [pair row][channel]
  __shared__ float2 gsm[C / 2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k2 = 2 * (lane & 3);
  const int rr = 8 * warp + (lane >> 2);
  if (threadIdx.x < C / 2) gsm[threadIdx.x] = *reinterpret_cast<const float2*>(gamma + 2 * threadIdx.x);
  float2 ag[NG][4], ab[NG][4];  // running sums of d * xhat and d for this lane's channels
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int m = 0; m < 4; ++m) ag[i][m] = ab[i][m] = make_float2(0.f, 0.f);

  auto fetch = [&](int tile, uint8_t* xdst, uint8_t* ddst) {
    const int fb = tile / tiles_per_batch;
    const int64_t f0 = (int64_t)(tile % tiles_per_batch) * TR;
#pragma unroll
    for (int idx = threadIdx.x; idx < C * (TR / 8); idx += 256) {
      const int c = idx / (TR / 8), j8 = idx % (TR / 8);
      const bool ok = f0 + 8 * j8 < NN;
      cp_async_16(xdst + c * IN_PITCH + 16 * j8, x_cm + ((int64_t)fb * C + c) * NN + (ok ? f0 + 8 * j8 : 0), ok);
    }
#pragma unroll
    for (int idx = threadIdx.x; idx < TR * (C / 8); idx += 256) {
      const int j = idx / (C / 8), c8 = idx % (C / 8);
      const bool ok = f0 + j < NN;
      cp_async_16(ddst + j * OUT_PITCH + 16 * c8, d_xln + ((int64_t)fb * NN + (ok ? f0 + j : 0)) * C + 8 * c8, ok);
    }
    cp_async_commit();
  };
  int buf = 0;
  if ((int)blockIdx.x < n_tiles) fetch(blockIdx.x, xs0, ds0);
  for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, buf ^= 1) {
    const int bb = tile / tiles_per_batch;
    const int64_t r0 = (int64_t)(tile % tiles_per_batch) * TR;
    uint8_t* xs = xs0 + buf * C * IN_PITCH;
    uint8_t* ds = ds0 + buf * TR * OUT_PITCH;
    const bool row_ok = r0 + rr < NN;
    const float mu = row_ok ? mean[(int64_t)bb * NN + r0 + rr] : 0.f;
    const float rs = row_ok ? rstd[(int64_t)bb * NN + r0 + rr] : 0.f;
    // The other buffer pair was last touched in the previous iteration: its d_x read-out (plain loads) was
    // completed by every thread before that thread got here, but by OTHER threads only if they are past it too
    __syncthreads();
    if (tile + (int)gridDim.x < n_tiles) {
      fetch(tile + gridDim.x, xs0 + (buf ^ 1) * C * IN_PITCH, ds0 + (buf ^ 1) * TR * OUT_PITCH);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    uint32_t fx[NG][4], fd[NG][4];
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      ldmatrix_x4_trans(fx[i], smem_u32(xs + (32 * i + lane) * IN_PITCH + 16 * warp));
#pragma unroll
      for (int m = 0; m < 4; ++m)
        fd[i][m] = *reinterpret_cast<const uint32_t*>(ds + rr * OUT_PITCH + (32 * i + 8 * m + k2) * 2);
    }
    float a1 = 0.f, a2 = 0.f;
#pragma unroll
    for (int i = 0; i < NG; ++i)
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float2 gm = gsm[(32 * i + 8 * m + k2) >> 1];
        const float x0 = (bf16_lo(fx[i][m]) - mu) * rs, x1 = (bf16_hi(fx[i][m]) - mu) * rs;
        const float d0 = bf16_lo(fd[i][m]), d1 = bf16_hi(fd[i][m]);
        const float g0 = gm.x * d0, g1 = gm.y * d1;
        a1 += g0 + g1;
        a2 += g0 * x0 + g1 * x1;
        ag[i][m].x += d0 * x0;
        ag[i][m].y += d1 * x1;
        ab[i][m].x += d0;
        ab[i][m].y += d1;
      }
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    a2 += __shfl_xor_sync(0xffffffffu, a2, 1);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
    a2 += __shfl_xor_sync(0xffffffffu, a2, 2);
    const float m1 = a1 * (1.f / C), m2 = a2 * (1.f / C);
#pragma unroll
    for (int i = 0; i < NG; ++i) {
      uint32_t out[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const float2 gm = gsm[(32 * i + 8 * m + k2) >> 1];
        const float x0 = (bf16_lo(fx[i][m]) - mu) * rs, x1 = (bf16_hi(fx[i][m]) - mu) * rs;
        const float v0 = rs * (gm.x * bf16_lo(fd[i][m]) - m1 - x0 * m2);
        const float v1 = rs * (gm.y * bf16_hi(fd[i][m]) - m1 - x1 * m2);
        out[m] = pack_bf16x2(v0, v1);
      }
      stmatrix_x4_trans(smem_u32(xs + (32 * i + lane) * IN_PITCH + 16 * warp), out);
    }
    __syncthreads();
#pragma unroll
    for (int idx = threadIdx.x; idx < C * (TR / 8); idx += 256) {
      const int c = idx / (TR / 8), j8 = idx % (TR / 8);
      if (r0 + 8 * j8 < NN)
        *reinterpret_cast<uint4*>(dx_cm + ((int64_t)bb * C + c) * NN + r0 + 8 * j8) =
            *reinterpret_cast<const uint4*>(xs + c * IN_PITCH + 16 * j8);
    }
  }

  // ---- d_gamma / d_beta partials of this CTA: the 8 pair rows of a warp (lanes that differ in lane / 4) in
  //      shuffle order, then the 8 warps in warp order; a fixed tree, no atomics
  __syncthreads();
  float* red = reinterpret_cast<float*>(ds0);  // [8 warps][2][C]
#pragma unroll
  for (int i = 0; i < NG; ++i)
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      float v[4] = {ag[i][m].x, ag[i][m].y, ab[i][m].x, ab[i][m].y};
#pragma unroll
      for (int off = 4; off < 32; off <<= 1)
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] += __shfl_xor_sync(0xffffffffu, v[e], off);
      if (lane < 4) {
        const int c = 32 * i + 8 * m + k2;
        red[(warp * 2 + 0) * C + c] = v[0];
        red[(warp * 2 + 0) * C + c + 1] = v[1];
        red[(warp * 2 + 1) * C + c] = v[2];
        red[(warp * 2 + 1) * C + c + 1] = v[3];
      }
    }
  __syncthreads();
  if (threadIdx.x < 2 * C) {
    const int which = threadIdx.x / C, c = threadIdx.x % C;
    float t = red[(0 * 2 + which) * C + c];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += red[(w * 2 + which) * C + c];
    partials[(int64_t)blockIdx.x * 2 * C + which * C + c] = t;
  }
}

// Input-norm backward, row-major.  d_z = rstd (gamma d_zln - mean(gamma d_zln) - xhat mean(gamma d_zln xhat))
template <int C>
__global__ void __launch_bounds__(256) trimul_ln_bwd_kernel(const bf16* __restrict__ d_zln, const bf16* __restrict__ z,
                                                            const float* __restrict__ gamma,
                                                            const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, bf16* __restrict__ d_z,
                                                            float* __restrict__ partials, int64_t R,
                                                            int rows_per_block) {
  griddep_wait();
  using L = RowLanes<C>;
  __shared__ float red[8][2][C];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / L::LS, part = lane % L::LS;
  const bool on = part < L::LPR;
  const int64_t row_begin = (int64_t)blockIdx.x * rows_per_block;
  float g[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) g[e] = on ? gamma[part * 8 + e] : 0.f;
  float ag[8], ab[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) ag[e] = ab[e] = 0.f;
  constexpr int G = 4;  // row groups in flight per warp: all their loads are issued before the first use
  for (int it0 = warp * L::RPW; it0 < rows_per_block; it0 += G * 8 * L::RPW) {
    uint4 du[G], zu[G];
    float mu[G], rs[G];
    bool active[G];
#pragma unroll
    for (int r = 0; r < G; ++r) {
      const int it = it0 + r * 8 * L::RPW;
      const int64_t row = row_begin + it + sub;
      active[r] = on && it + sub < rows_per_block && row < R;
      du[r] = zu[r] = make_uint4(0u, 0u, 0u, 0u);
      mu[r] = rs[r] = 0.f;
      if (active[r]) {
        du[r] = *reinterpret_cast<const uint4*>(d_zln + row * C + part * 8);
        zu[r] = *reinterpret_cast<const uint4*>(z + row * C + part * 8);
        mu[r] = mean[row];
        rs[r] = rstd[row];
      }
    }
#pragma unroll
    for (int r = 0; r < G; ++r) {
      const int64_t row = row_begin + it0 + r * 8 * L::RPW + sub;
      float d[8], xh[8];
      unpack8(du[r], d);
      unpack8(zu[r], xh);
      float gd[8], a1 = 0.f, a2 = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        xh[e] = active[r] ? (xh[e] - mu[r]) * rs[r] : 0.f;
        gd[e] = g[e] * d[e];
        a1 += gd[e];
        a2 += gd[e] * xh[e];
      }
      const float m1 = slot_sum<C>(a1) * (1.f / C);
      const float m2 = slot_sum<C>(a2) * (1.f / C);
      if (active[r]) {
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e)
          o[e] = pack_bf16x2(rs[r] * (gd[2 * e] - m1 - xh[2 * e] * m2), rs[r] * (gd[2 * e + 1] - m1 - xh[2 * e + 1] * m2));
        *reinterpret_cast<uint4*>(d_z + row * C + part * 8) = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ag[e] += d[e] * xh[e];
          ab[e] += d[e];
        }
      }
    }
  }
  // fixed-order fold: the row slots of a warp (sub = 0 .. RPW-1), then the 8 warps
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float vg = ag[e], vb = ab[e];
    for (int s = 1; s < L::RPW; ++s) {
      const float og = __shfl_sync(0xffffffffu, ag[e], part + s * L::LS);
      const float ob = __shfl_sync(0xffffffffu, ab[e], part + s * L::LS);
      vg += og;
      vb += ob;
    }
    if (sub == 0 && on) {
      red[warp][0][part * 8 + e] = vg;
      red[warp][1][part * 8 + e] = vb;
    }
  }
  __syncthreads();
  if (threadIdx.x < 2 * C) {
    const int which = threadIdx.x / C, c = threadIdx.x % C;
    float s = red[0][which][c];
    for (int w = 1; w < 8; ++w) s += red[w][which][c];
    partials[(int64_t)blockIdx.x * 2 * C + which * C + c] = s;
  }
}

// out[j] = fixed-order sum over blocks of partials[blk][j], j < width.  One CTA per 32 columns;
// warp w adds blocks w, w+32, ... in ascending order, then the 32 warp sums are added in warp order.
__global__ void __launch_bounds__(1024) trimul_colsum_fold_kernel(const float* __restrict__ partials, int n_blocks,
                                                                 int width, float* __restrict__ out_a,
                                                                 float* __restrict__ out_b, int half) {
  griddep_wait();
  __shared__ float red[32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (j < width) {
#pragma unroll 4
    for (int b = warp; b < n_blocks; b += 32) s = __fadd_rn(s, partials[(int64_t)b * width + j]);
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && j < width) {
    float t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 32; ++w) t = __fadd_rn(t, red[w][lane]);
    if (j < half) out_a[j] = t;
    else out_b[j - half] = t;
  }
}

// Weight-gradient fold: out_row_block[r][c] = sum over splits (ascending) of part[s][m][c].
// Rows are routed in blocks of C rows to up to five destinations (W5 = [a_p; a_g; b_p; b_g; g]).
struct WgradDst {
  float* dst[5];
};
__global__ void __launch_bounds__(256) trimul_wgrad_fold_kernel(const float* __restrict__ part, int n_splits, int M,
                                                                int C, WgradDst d) {
  griddep_wait();
  // 32 output elements per CTA, 8 warps.  Warp g adds its contiguous range of splits in ascending
  // order (the loads of a batch of 8 splits are independent, so all are in flight before the first
  // add), then the 8 range sums are added in range order: a fixed summation tree, no atomics.
  __shared__ float red[8][32];
  const int g = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * 32 + lane;
  const int per = (n_splits + 7) / 8;
  const int k0 = g * per, k1 = min(n_splits, k0 + per);
  const int64_t stride = (int64_t)M * C;
  float s = 0.f;
  if (i < M * C) {
    const float* src = part + i;
    int k = k0;
    for (; k + 8 <= k1; k += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = src[(int64_t)(k + u) * stride];
#pragma unroll
      for (int u = 0; u < 8; ++u) s = __fadd_rn(s, v[u]);
    }
    for (; k < k1; ++k) s = __fadd_rn(s, src[(int64_t)k * stride]);
  }
  red[g][lane] = s;
  __syncthreads();
  if (g == 0 && i < M * C) {
    float t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t = __fadd_rn(t, red[w][lane]);
    const int row = i / C, col = i % C;
    d.dst[row / C][(row % C) * C + col] = t;
  }
}

// First level of the LayerNorm-gradient fold: out[s][j] = fixed-order sum of in[s*256 .. s*256+255][j].
__global__ void __launch_bounds__(1024) trimul_colsum_stage_kernel(const float* __restrict__ in, int n_in, int width,
                                                                   float* __restrict__ out) {
  griddep_wait();
  __shared__ float red[32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * 32 + lane;
  const int b0 = blockIdx.y * 256, b1 = min(n_in, b0 + 256);
  float s = 0.f;
  if (j < width)
    for (int b = b0 + warp; b < b1; b += 32) s = __fadd_rn(s, in[(int64_t)b * width + j]);
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && j < width) {
    float t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 32; ++w) t = __fadd_rn(t, red[w][lane]);
    out[(int64_t)blockIdx.y * width + j] = t;
  }
}

// =============================================================================================
// host orchestration
// =============================================================================================
struct TrimulPacked {
  bf16 *W5, *W5T, *Wz, *WzT;
};
static int64_t packed_weight_elems(int64_t C) { return 12 * C * C; }

static int pack_weights(const float* p_in, const float* g_in, const float* p_out, const float* g_out, void* buf,
                        int C, TrimulPacked* pk, cudaStream_t stream) {
  bf16* base = reinterpret_cast<bf16*>(buf);
  pk->W5 = base;
  pk->W5T = base + 5 * C * C;
  pk->Wz = base + 10 * C * C;
  pk->WzT = base + 11 * C * C;
  launch_kernel(trimul_pack_weights_kernel, dim3((5 * C * C + 255) / 256), dim3(256), 0, stream, p_in, g_in, p_out, g_out, pk->W5, pk->W5T,
                                                                          pk->Wz, pk->WzT, C);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

template <int C, class Epi>
static int proj_gemm(const bf16* zln, const bf16* W5, int64_t R, int n_cols, const typename Epi::Params& ep,
                     int* status, cudaStream_t stream) {
  // The gated epilogues are latency-bound: at C = 128 (four 32-column chunk pairs per tile) 16
  // epilogue warps keep one chunk pair each in flight; narrower tiles have work for 8 only.
  // The weight tile (2C rows x C) stays in shared memory while the CTA walks a contiguous range of row
  // tiles; only the activations stream.  CTAs j, j + n/3, j + 2n/3 walk the same rows for the a, b and
  // gate tiles at about the same time, so the activations come from DRAM once and from L2 twice.
  using Cfg = GemmCfg<128, 2 * C, 128, false, 128, false, 4, (C == 128 ? 16 : 8), 2, (C + 63) / 64>;
  GemmShape sh{(int)R, n_cols, C, 1, 0};
  return launch_gemm<Cfg, Epi>(zln, C, 0, W5, C, 0, sh, ep, status, stream);
}

template <int C>
static int trimul_fwd_t(const bf16* z, const float* mask, const TrimulPacked& pk, const float* gin, const float* bin,
                        const float* gout, const float* bout, int incoming, int64_t B, int64_t N, int64_t NN,
                        int stages, bf16* out, bf16* zln, float* mean_in, float* rstd_in, bf16* a_cm, bf16* b_cm,
                        bf16* gate, bf16* x_cm, bf16* xln, float* mean_out, float* rstd_out, int* status,
                        cudaStream_t stream) {
  // NN = pair rows per batch entry (N*N for a whole pair tensor, N_local*N for a row shard)
  const int64_t R = B * NN;
  using L = RowLanes<C>;
  int rc = TPF_OK;
  if (stages & 1) {
    const int64_t warps = (R + 4 * L::RPW - 1) / (4 * L::RPW);
    const int64_t blocks = (warps + 7) / 8;
    launch_kernel(trimul_ln_fwd_kernel<C>, dim3((unsigned)blocks), dim3(256), 0, stream, z, gin, bin, zln, mean_in, rstd_in, R);
    TPF_LAUNCH_OK();
    EpiProjGate::Params ep{a_cm, b_cm, gate, mask, C, NN};
    if ((rc = proj_gemm<C, EpiProjGate>(zln, pk.W5, R, 5 * C, ep, status, stream))) return rc;
  }
  if (stages & 2) {
    // k-contraction: batch = B*C problems of N x N x N
    rc = bmm_bf16(a_cm, N, NN, incoming, b_cm, N, NN, incoming, x_cm, N, NN, 0, N, N, N, B * C, 0, 128, stream);
    if (rc) return rc;
  }
  if (stages & 4) {
    const int tiles = (int)((NN + 63) / 64);
    int grid = (int)(B * tiles);
    if (grid > 2 * sm_count()) grid = 2 * sm_count();
    {
      auto kern = trimul_xnorm_fwd_kernel<C>;
      constexpr int smem = 2 * C * (64 * 2 + 16) + 64 * (C * 2 + 16);
      static PerDeviceOnce once;  // per instantiation
      if ((rc = ensure_dynamic_smem(kern, smem, once))) return rc;
      launch_kernel(kern, dim3(grid), dim3(256), smem, stream, x_cm, gout, bout, xln, mean_out, rstd_out, NN, tiles, (int)(B * tiles));
    }
    TPF_LAUNCH_OK();
    using Cfg = GemmCfg<128, C, 128, false, 128, false, 4>;
    GemmShape sh{(int)R, C, C, 1, 0};
    EpiOutGate::Params ep{out, gate, C};
    if ((rc = launch_gemm<Cfg, EpiOutGate>(xln, C, 0, pk.Wz, C, 0, sh, ep, status, stream))) return rc;
  }
  return TPF_OK;
}

static void split_plan(int64_t R, int tiles_mn, int* n_splits, int64_t* k_per_split) {
  int64_t s = sm_count() / (tiles_mn > 0 ? tiles_mn : 1);
  if (s < 1) s = 1;
  int64_t kps = ((R + s - 1) / s + 63) / 64 * 64;
  if (kps < 64) kps = 64;
  *k_per_split = kps;
  *n_splits = (int)((R + kps - 1) / kps);
}

struct TrimulBwdWorkspace {
  bf16 *wpack, *d_y, *d_proj5, *d_xln, *dx_cm, *da_cm, *db_cm;  // d_zln aliases d_xln
  float *part_w5, *part_wz, *part_ln_out, *part_ln_in, *part_lvl2;
  int splits_w5, splits_wz, blocks_ln_out, blocks_ln_in, rows_per_block_in;
  int64_t kps_w5, kps_wz;
  int64_t total_bytes;
};

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

static void plan_bwd_workspace(int64_t B, int64_t NN, int64_t C, char* base, TrimulBwdWorkspace* w) {
  const int64_t R = B * NN;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    char* p = base ? base + off : nullptr;
    off += align256(bytes);
    return p;
  };
  w->wpack = reinterpret_cast<bf16*>(take(packed_weight_elems(C) * 2));
  w->d_y = reinterpret_cast<bf16*>(take(R * C * 2));
  w->d_proj5 = reinterpret_cast<bf16*>(take(R * 5 * C * 2));
  w->d_xln = reinterpret_cast<bf16*>(take(R * C * 2));
  w->dx_cm = reinterpret_cast<bf16*>(take(R * C * 2));
  w->da_cm = reinterpret_cast<bf16*>(take(R * C * 2));
  w->db_cm = reinterpret_cast<bf16*>(take(R * C * 2));
  split_plan(R, (int)((5 * C + 127) / 128), &w->splits_w5, &w->kps_w5);
  split_plan(R, 1, &w->splits_wz, &w->kps_wz);
  w->part_w5 = reinterpret_cast<float*>(take((int64_t)w->splits_w5 * 5 * C * C * 4));
  w->part_wz = reinterpret_cast<float*>(take((int64_t)w->splits_wz * C * C * 4));
  {
    // one partial row per CTA of the output-norm backward kernel (persistent, two CTAs per SM)
    const int64_t tiles = B * ((NN + 63) / 64);
    w->blocks_ln_out = (int)(tiles < 2 * sm_count() ? tiles : 2 * sm_count());
  }
  w->rows_per_block_in = 128;
  w->blocks_ln_in = (int)((R + 127) / 128);
  w->part_ln_out = reinterpret_cast<float*>(take((int64_t)w->blocks_ln_out * 2 * C * 4));
  w->part_ln_in = reinterpret_cast<float*>(take((int64_t)w->blocks_ln_in * 2 * C * 4));
  {
    const int64_t most = w->blocks_ln_out > w->blocks_ln_in ? w->blocks_ln_out : w->blocks_ln_in;
    w->part_lvl2 = reinterpret_cast<float*>(take(((most + 255) / 256) * 2 * C * 4));
  }
  w->total_bytes = off;
}

template <int C>
static int trimul_bwd_t(const bf16* d_out, const bf16* z, const float* mask, const float* p_in, const float* g_in,
                        const float* p_out, const float* g_out, const float* gin, const float* gout, int incoming,
                        int64_t B, int64_t N, int64_t NN, int stages, bf16* dx_io, bf16* da_io, bf16* db_io,
                        const bf16* out, const bf16* zln, const float* mean_in,
                        const float* rstd_in, const bf16* a_cm, const bf16* b_cm, const bf16* gate, const bf16* x_cm,
                        const bf16* xln, const float* mean_out, const float* rstd_out, bf16* d_z, float* d_p_in,
                        float* d_g_in, float* d_p_out, float* d_g_out, float* d_gin, float* d_bin, float* d_gout,
                        float* d_bout, char* workspace, int* status, cudaStream_t stream) {
  const int64_t R = B * NN;
  TrimulBwdWorkspace w;
  plan_bwd_workspace(B, NN, C, workspace, &w);
  if (dx_io) w.dx_cm = dx_io;  // staged (sharded) use: the caller moves these between ranks
  if (da_io) w.da_cm = da_io;
  if (db_io) w.db_cm = db_io;
  TrimulPacked pk;
  int rc;
  if ((rc = pack_weights(p_in, g_in, p_out, g_out, w.wpack, C, &pk, stream))) return rc;

  if (stages & 1) {
  // 1. output gate: d_y, d_glogit
  {
    int blocks = (int)((R * C / 8 + 255) / 256);
    if (blocks > 16 * sm_count()) blocks = 16 * sm_count();
    launch_kernel(trimul_out_gate_bwd_kernel, dim3(blocks), dim3(256), 0, stream, d_out, out, gate, w.d_y, w.d_proj5, R, C);
    TPF_LAUNCH_OK();
  }
  // 2. d_xln = d_y Wz ; d_wz = d_y^T xln
  {
    using Cfg = GemmCfg<128, 128, 128, false, 128, false, 4>;
    using Epi = EpiStore<bf16>;
    GemmShape sh{(int)R, C, C, 1, 0};
    typename Epi::Params ep{w.d_xln, C, 0};
    if ((rc = launch_gemm<Cfg, Epi>(w.d_y, C, 0, pk.WzT, C, 0, sh, ep, status, stream))) return rc;
  }
  rc = bmm_bf16(w.d_y, C, 0, 1, xln, C, 0, 1, w.part_wz, C, (int64_t)C * C, 1, C, C, R, w.splits_wz, w.kps_wz, 128,
                stream);
  if (rc) return rc;
  {
    WgradDst d;
    for (int i = 0; i < 5; ++i) d.dst[i] = d_p_out;
    launch_kernel(trimul_wgrad_fold_kernel, dim3((C * C + 31) / 32), dim3(256), 0, stream, w.part_wz, w.splits_wz, C, C, d);
    TPF_LAUNCH_OK();
  }
  // 3. output norm backward -> d_x (channel-major), d_gamma_out, d_beta_out
  {
    const int tiles = (int)((NN + 63) / 64);
    {
      auto kern = trimul_xnorm_bwd_kernel<C>;
      constexpr int smem = 2 * C * (64 * 2 + 16) + 2 * 64 * (C * 2 + 16);
      static PerDeviceOnce once;  // per instantiation
      if ((rc = ensure_dynamic_smem(kern, smem, once))) return rc;
      launch_kernel(kern, dim3(w.blocks_ln_out), dim3(256), smem, stream, w.d_xln, x_cm, gout, mean_out, rstd_out, w.dx_cm, w.part_ln_out, NN,
                                                  tiles, (int)(B * tiles));
    }
    TPF_LAUNCH_OK();
    {
      const int lvl = (w.blocks_ln_out + 255) / 256;
      launch_kernel(trimul_colsum_stage_kernel, dim3(dim3((2 * C + 31) / 32, lvl)), dim3(1024), 0, stream, w.part_ln_out, w.blocks_ln_out,
                                                                                    2 * C, w.part_lvl2);
      TPF_LAUNCH_OK();
      launch_kernel(trimul_colsum_fold_kernel, dim3((2 * C + 31) / 32), dim3(1024), 0, stream, w.part_lvl2, lvl, 2 * C, d_gout, d_bout, C);
      TPF_LAUNCH_OK();
    }
  }
  }
  if (stages & 2) {
  // 4. contraction backward
  if (!incoming) {
    // d_a[c,i,k] = sum_j d_x[c,i,j] b[c,j,k] ; d_b[c,j,k] = sum_i d_x[c,i,j] a[c,i,k]
    if ((rc = bmm_bf16(w.dx_cm, N, NN, 0, b_cm, N, NN, 1, w.da_cm, N, NN, 0, N, N, N, B * C, 0, 128, stream))) return rc;
    if ((rc = bmm_bf16(w.dx_cm, N, NN, 1, a_cm, N, NN, 1, w.db_cm, N, NN, 0, N, N, N, B * C, 0, 128, stream))) return rc;
  } else {
    // d_a[c,k,i] = sum_j b[c,k,j] d_x[c,i,j] ; d_b[c,k,j] = sum_i a[c,k,i] d_x[c,i,j]
    if ((rc = bmm_bf16(b_cm, N, NN, 0, w.dx_cm, N, NN, 0, w.da_cm, N, NN, 0, N, N, N, B * C, 0, 128, stream))) return rc;
    if ((rc = bmm_bf16(a_cm, N, NN, 0, w.dx_cm, N, NN, 1, w.db_cm, N, NN, 0, N, N, N, B * C, 0, 128, stream))) return rc;
  }
  }
  if (stages & 4) {
  // 5. gated projections backward (recompute p, g) -> d_proj5[:, 0:4C]
  {
    EpiGateSplitBwd::Params ep{w.da_cm, w.db_cm, mask, w.d_proj5, C, NN};
    if ((rc = proj_gemm<C, EpiGateSplitBwd>(zln, pk.W5, R, 4 * C, ep, status, stream))) return rc;
  }
  // 6. d_zln = d_proj5 W5 ; dW5 = d_proj5^T zln
  bf16* d_zln = w.d_xln;
  {
    // d_proj5 streams from DRAM (W5^T comes from L2): six stages keep enough of it in flight per SM
    using Cfg = GemmCfg<128, 128, 128, false, 128, false, 6>;
    using Epi = EpiStore<bf16>;
    GemmShape sh{(int)R, C, 5 * C, 1, 0};
    typename Epi::Params ep{d_zln, C, 0};
    if ((rc = launch_gemm<Cfg, Epi>(w.d_proj5, 5 * C, 0, pk.W5T, 5 * C, 0, sh, ep, status, stream))) return rc;
  }
  rc = bmm_bf16(w.d_proj5, 5 * C, 0, 1, zln, C, 0, 1, w.part_w5, C, (int64_t)5 * C * C, 1, 5 * C, C, R, w.splits_w5,
                w.kps_w5, 128, stream);
  if (rc) return rc;
  {
    WgradDst d;
    d.dst[0] = d_p_in;              // a_p
    d.dst[1] = d_g_in;              // a_g
    d.dst[2] = d_p_in + C * C;      // b_p
    d.dst[3] = d_g_in + C * C;      // b_g
    d.dst[4] = d_g_out;             // g
    launch_kernel(trimul_wgrad_fold_kernel, dim3((5 * C * C + 31) / 32), dim3(256), 0, stream, w.part_w5, w.splits_w5, 5 * C, C, d);
    TPF_LAUNCH_OK();
  }
  // 7. input norm backward
  {
    launch_kernel(trimul_ln_bwd_kernel<C>, dim3(w.blocks_ln_in), dim3(256), 0, stream, d_zln, z, gin, mean_in, rstd_in, d_z, w.part_ln_in, R,
                                                                w.rows_per_block_in);
    TPF_LAUNCH_OK();
    {
      const int lvl = (w.blocks_ln_in + 255) / 256;
      launch_kernel(trimul_colsum_stage_kernel, dim3(dim3((2 * C + 31) / 32, lvl)), dim3(1024), 0, stream, w.part_ln_in, w.blocks_ln_in,
                                                                                    2 * C, w.part_lvl2);
      TPF_LAUNCH_OK();
      launch_kernel(trimul_colsum_fold_kernel, dim3((2 * C + 31) / 32), dim3(1024), 0, stream, w.part_lvl2, lvl, 2 * C, d_gin, d_bin, C);
      TPF_LAUNCH_OK();
    }
  }
  }
  return TPF_OK;
}

static int check_trimul_rows(const char* who, int64_t N, int64_t NN, int stages) {
  TPF_REQUIRE(stages >= 1 && stages <= 7, TPF_ERR_INVALID_ARGUMENT, "%s: stages must be a non-empty mask of 1|2|4", who);
  TPF_REQUIRE(NN > 0 && NN % 64 == 0, TPF_ERR_UNSUPPORTED, "%s: rows per batch (%lld) must be a positive multiple of 64",
              who, (long long)NN);
  TPF_REQUIRE(NN == N * N || !(stages & 2), TPF_ERR_INVALID_ARGUMENT,
              "%s: the contraction stage needs whole pair tensors (rows per batch == N*N)", who);
  return TPF_OK;
}

static int check_trimul_shape(const char* who, int64_t B, int64_t N, int64_t C) {
  TPF_REQUIRE(B > 0 && N > 0, TPF_ERR_INVALID_ARGUMENT, "%s: B and N must be positive", who);
  TPF_REQUIRE(C == 32 || C == 64 || C == 96 || C == 128, TPF_ERR_UNSUPPORTED, "%s: C=%lld not in {32,64,96,128}", who,
              (long long)C);
  TPF_REQUIRE(N % 8 == 0, TPF_ERR_UNSUPPORTED, "%s: N=%lld must be a multiple of 8 (pad on the host side)", who,
              (long long)N);
  TPF_REQUIRE(B * N * N < (1ll << 31), TPF_ERR_INVALID_ARGUMENT, "%s: B*N*N too large", who);
  return TPF_OK;
}

int64_t trimul_fwd_workspace_bytes(int64_t B, int64_t N, int64_t C) { return align256(packed_weight_elems(C) * 2); }

int64_t trimul_bwd_workspace_bytes(int64_t B, int64_t NN, int64_t C) {
  TrimulBwdWorkspace w;
  plan_bwd_workspace(B, NN, C, nullptr, &w);
  return w.total_bytes;
}

int trimul_fwd(const void* z, const float* mask, const float* p_in, const float* g_in, const float* p_out,
               const float* g_out, const float* gin, const float* bin, const float* gout, const float* bout,
               int incoming, int64_t B, int64_t N, int64_t C, void* out, void* zln, float* mean_in, float* rstd_in,
               void* a_cm, void* b_cm, void* gate, void* x_cm, void* xln, float* mean_out, float* rstd_out,
               void* workspace, int64_t workspace_bytes, int64_t NN, int stages, cudaStream_t stream) {
  int rc = check_trimul_shape("trimul_fwd", B, N, C);
  if (rc) return rc;
  if (NN == 0) NN = N * N;
  if ((rc = check_trimul_rows("trimul_fwd", N, NN, stages))) return rc;
  TPF_REQUIRE(z && mask && p_in && g_in && p_out && g_out && gin && bin && gout && bout && out && zln && mean_in &&
                  rstd_in && a_cm && b_cm && gate && x_cm && xln && mean_out && rstd_out,
              TPF_ERR_INVALID_ARGUMENT, "trimul_fwd: null pointer");
  TPF_REQUIRE(workspace && workspace_bytes >= trimul_fwd_workspace_bytes(B, N, C), TPF_ERR_WORKSPACE,
              "trimul_fwd: workspace of %lld bytes required", (long long)trimul_fwd_workspace_bytes(B, N, C));
  int* status = nullptr;
  {
    static PerDeviceAddress cache;
    if ((rc = device_symbol_address(g_trimul_status, cache, reinterpret_cast<void**>(&status)))) return rc;
  }
  TrimulPacked pk;
  if ((rc = pack_weights(p_in, g_in, p_out, g_out, workspace, (int)C, &pk, stream))) return rc;
#define TPF_TRIMUL_FWD(CC)                                                                                         \
  if (C == CC)                                                                                                     \
    return trimul_fwd_t<CC>((const bf16*)z, mask, pk, gin, bin, gout, bout, incoming, B, N, NN, stages, (bf16*)out, (bf16*)zln, \
                            mean_in, rstd_in, (bf16*)a_cm, (bf16*)b_cm, (bf16*)gate, (bf16*)x_cm, (bf16*)xln,       \
                            mean_out, rstd_out, status, stream);
  TPF_TRIMUL_FWD(32)
  TPF_TRIMUL_FWD(64)
  TPF_TRIMUL_FWD(96)
  TPF_TRIMUL_FWD(128)
#undef TPF_TRIMUL_FWD
  return fail(TPF_ERR_UNSUPPORTED, "trimul_fwd: unsupported C");
}

int trimul_bwd(const void* d_out, const void* z, const float* mask, const float* p_in, const float* g_in,
               const float* p_out, const float* g_out, const float* gin, const float* gout, int incoming, int64_t B,
               int64_t N, int64_t C, const void* out, const void* zln, const float* mean_in, const float* rstd_in,
               const void* a_cm, const void* b_cm, const void* gate, const void* x_cm, const void* xln,
               const float* mean_out, const float* rstd_out, void* d_z, float* d_p_in, float* d_g_in, float* d_p_out,
               float* d_g_out, float* d_gin, float* d_bin, float* d_gout, float* d_bout, void* workspace,
               int64_t workspace_bytes, int64_t NN, int stages, void* dx_io, void* da_io, void* db_io,
               cudaStream_t stream) {
  int rc = check_trimul_shape("trimul_bwd", B, N, C);
  if (rc) return rc;
  if (NN == 0) NN = N * N;
  if ((rc = check_trimul_rows("trimul_bwd", N, NN, stages))) return rc;
  TPF_REQUIRE(d_out && z && mask && p_in && g_in && p_out && g_out && gin && gout && out && zln && mean_in &&
                  rstd_in && a_cm && b_cm && gate && x_cm && xln && mean_out && rstd_out && d_z && d_p_in && d_g_in &&
                  d_p_out && d_g_out && d_gin && d_bin && d_gout && d_bout,
              TPF_ERR_INVALID_ARGUMENT, "trimul_bwd: null pointer");
  TPF_REQUIRE(workspace && workspace_bytes >= trimul_bwd_workspace_bytes(B, NN, C) &&
                  (reinterpret_cast<uintptr_t>(workspace) & 255) == 0,
              TPF_ERR_WORKSPACE, "trimul_bwd: 256-byte aligned workspace of %lld bytes required",
              (long long)trimul_bwd_workspace_bytes(B, NN, C));
  int* status = nullptr;
  {
    static PerDeviceAddress cache;
    if ((rc = device_symbol_address(g_trimul_status, cache, reinterpret_cast<void**>(&status)))) return rc;
  }
#define TPF_TRIMUL_BWD(CC)                                                                                            \
  if (C == CC)                                                                                                        \
    return trimul_bwd_t<CC>((const bf16*)d_out, (const bf16*)z, mask, p_in, g_in, p_out, g_out, gin, gout, incoming,  \
                            B, N, NN, stages, (bf16*)dx_io, (bf16*)da_io, (bf16*)db_io, (const bf16*)out, (const bf16*)zln, mean_in, rstd_in, (const bf16*)a_cm,            \
                            (const bf16*)b_cm, (const bf16*)gate, (const bf16*)x_cm, (const bf16*)xln, mean_out,      \
                            rstd_out, (bf16*)d_z, d_p_in, d_g_in, d_p_out, d_g_out, d_gin, d_bin, d_gout, d_bout,     \
                            (char*)workspace, status, stream);
  TPF_TRIMUL_BWD(32)
  TPF_TRIMUL_BWD(64)
  TPF_TRIMUL_BWD(96)
  TPF_TRIMUL_BWD(128)
#undef TPF_TRIMUL_BWD
  return fail(TPF_ERR_UNSUPPORTED, "trimul_bwd: unsupported C");
}

}  // namespace tpf

