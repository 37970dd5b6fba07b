"""tpf_bmm_bf16 (the tcgen05 GEMM engine behind the TriMul stages) on a B200 against an fp32 matmul of
the same bf16 operands: every (swizzle, operand-major) combination the C ABI accepts, ragged extents,
batches, split-K partial sums, fp32 and bf16 outputs.  The engine replaces torch.bmm / torch.mm in
openfold3/core/kernels/turbopairformer/turbopairformer_trimul.py:244-249, 357-362."""
import pytest
import torch

from openfold3_triangle_kernel_b200 import _cabi as C

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a CUDA device")]

# bf16 operands, fp32 accumulation: an fp32 result differs from the fp32 matmul only by summation order;
# a bf16 result carries one rounding (2^-9 relative)
TOL_F32 = 1e-5
TOL_BF16 = 4e-3

COMBOS = [(128, 0, 0), (128, 1, 1), (128, 1, 0), (128, 0, 1), (64, 0, 0), (64, 1, 1), (32, 0, 0), (32, 1, 1)]
SHAPES = [
    # M, N, K, batch
    (128, 128, 64, 1),
    (384, 384, 384, 3),      # the k-contraction of T384, three channels
    (200, 136, 72, 2),       # ragged in every extent
    (129, 40, 200, 1),
    (1, 8, 8, 1),
]


def _operand(rows, k, batch, mn_major, gen):
    """Returns (storage tensor, logical [batch, rows, k] view, leading dimension, batch stride)."""
    if not mn_major:
        ld = (k + 7) // 8 * 8
        buf = torch.zeros(batch, rows, ld, device="cuda", dtype=torch.bfloat16)
        buf[:, :, :k] = torch.randn(batch, rows, k, device="cuda", generator=gen).bfloat16()
        return buf, buf[:, :, :k], ld, rows * ld
    ld = (rows + 7) // 8 * 8
    buf = torch.zeros(batch, k, ld, device="cuda", dtype=torch.bfloat16)
    buf[:, :, :rows] = torch.randn(batch, k, rows, device="cuda", generator=gen).bfloat16()
    return buf, buf[:, :, :rows].transpose(1, 2), ld, k * ld


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


@pytest.mark.parametrize("swz,a_mn,b_mn", COMBOS)
@pytest.mark.parametrize("M,N,K,batch", SHAPES)
@pytest.mark.parametrize("out_f32", [0, 1])
def test_bmm_matches_fp32_matmul(swz, a_mn, b_mn, M, N, K, batch, out_f32):
    gen = torch.Generator(device="cuda").manual_seed(1000 * swz + 100 * a_mn + 10 * b_mn + M + N + K)
    a_buf, a, lda, bsa = _operand(M, K, batch, a_mn, gen)
    b_buf, b, ldb, bsb = _operand(N, K, batch, b_mn, gen)
    ldd = (N + 7) // 8 * 8
    d = torch.full((batch, M, ldd), float("nan"), device="cuda", dtype=torch.float32 if out_f32 else torch.bfloat16)
    C.call("tpf_bmm_bf16", C.ptr(a_buf), lda, bsa, a_mn, C.ptr(b_buf), ldb, bsb, b_mn, C.ptr(d), ldd, M * ldd, out_f32,
           M, N, K, batch, 0, swz, C.current_stream())
    torch.cuda.synchronize()
    assert C.device_status() == 0
    ref = torch.matmul(a.float(), b.float().transpose(1, 2))
    got = d[:, :, :N].float()
    assert torch.isfinite(got).all()
    assert _rel(got, ref) < (TOL_F32 if out_f32 else TOL_BF16)
    # the padding columns of D are not written
    if ldd > N:
        assert torch.isnan(d[:, :, N:].float()).all()


@pytest.mark.parametrize("swz,a_mn,b_mn", [(128, 1, 1), (128, 0, 0), (64, 1, 1)])
def test_bmm_split_k_partial_sums(swz, a_mn, b_mn):
    """k_per_split > 0: `batch` K-slices of ONE problem; slice b's partial sum lands in D[b]."""
    M, N, K, kps = 160, 128, 1000, 256
    splits = (K + kps - 1) // kps
    gen = torch.Generator(device="cuda").manual_seed(7)
    a_buf, a, lda, bsa = _operand(M, K, 1, a_mn, gen)
    b_buf, b, ldb, bsb = _operand(N, K, 1, b_mn, gen)
    d = torch.zeros(splits, M, N, device="cuda", dtype=torch.float32)
    C.call("tpf_bmm_bf16", C.ptr(a_buf), lda, 0, a_mn, C.ptr(b_buf), ldb, 0, b_mn, C.ptr(d), N, M * N, 1,
           M, N, K, splits, kps, swz, C.current_stream())
    torch.cuda.synchronize()
    assert C.device_status() == 0
    af, bf = a[0].float(), b[0].float()
    for s in range(splits):
        k0, k1 = s * kps, min(K, (s + 1) * kps)
        ref = af[:, k0:k1] @ bf[:, k0:k1].t()
        assert _rel(d[s], ref) < TOL_F32
    assert _rel(d.sum(0), af @ bf.t()) < TOL_F32


def test_bmm_many_tiles_per_cta():
    """More output tiles than CTAs: the persistent tile walk, both accumulators, every pipeline stage reused."""
    M, N, K, batch = 1024, 640, 192, 5
    gen = torch.Generator(device="cuda").manual_seed(11)
    a_buf, a, lda, bsa = _operand(M, K, batch, 0, gen)
    b_buf, b, ldb, bsb = _operand(N, K, batch, 0, gen)
    d = torch.empty(batch, M, N, device="cuda", dtype=torch.bfloat16)
    C.call("tpf_bmm_bf16", C.ptr(a_buf), lda, bsa, 0, C.ptr(b_buf), ldb, bsb, 0, C.ptr(d), N, M * N, 0,
           M, N, K, batch, 0, 128, C.current_stream())
    torch.cuda.synchronize()
    assert C.device_status() == 0
    assert _rel(d.float(), torch.matmul(a.float(), b.float().transpose(1, 2))) < TOL_BF16
