"""GPU parity: mm / addmm (ATen overrides through ``use_gems()``, the out variants and the
``torch.ops.flag_gems`` entries) against the fp64 CPU oracle.

Shapes and scalars follow tests/test_blas_ops.py:24-57,119-136 of FlagGems; the larger
shapes exercise the tcgen05 kernel including M/N/K tails and every operand majorness.
Tolerance (reference contract): rtol = dtype resolution, atol = 1e-4 * K."""
import ctypes

import pytest
import torch

from flaggems_b200 import _lib, workloads
from flaggems_b200.testing import assert_close
from oracle import reference_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
FLOAT_DTYPES = [torch.float16, torch.float32, torch.bfloat16]
MNK_SHAPES = [(1, 1, 32), (15, 160, 1024), (495, 5333, 71)]
SCALARS = [0.001, -0.999, 100.001, -111.999]


def _uses_tcgen05(a, b, c):
    p = _lib.GemmParams()
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    p.M, p.K = a.shape
    p.N = b.shape[1]
    p.a_stride0, p.a_stride1 = a.stride()
    p.b_stride0, p.b_stride1 = b.stride()
    p.c_stride0, p.c_stride1 = c.stride()
    p.dtype = _lib.dtype_code(c.dtype)
    return bool(_lib.load().fg_gemm_uses_tcgen05(ctypes.byref(p)))


@pytest.mark.parametrize("M,N,K", MNK_SHAPES)
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
@pytest.mark.parametrize("b_column_major", [True, False])
def test_mm(fg, M, N, K, dtype, b_column_major):
    torch.manual_seed(0)
    a = torch.randn((M, K), dtype=dtype, device=DEV)
    b = torch.randn((N, K), dtype=dtype, device=DEV).t() if b_column_major else torch.randn((K, N), dtype=dtype, device=DEV)
    ref = O.mm(a.cpu(), b.cpu())
    with fg.use_gems():
        before = _lib.launch_count()
        res = torch.mm(a, b)
        assert _lib.launch_count() > before, "torch.mm did not reach the flaggems_b200 kernel"
    assert_close(res.cpu(), ref, dtype, reduce_dim=K)


@pytest.mark.parametrize("M,N,K", MNK_SHAPES)
@pytest.mark.parametrize("scalar", SCALARS)
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
@pytest.mark.parametrize("b_column_major", [True, False])
def test_addmm(fg, M, N, K, scalar, dtype, b_column_major):
    torch.manual_seed(0)
    a = torch.randn((M, K), dtype=dtype, device=DEV)
    b = torch.randn((N, K), dtype=dtype, device=DEV).t() if b_column_major else torch.randn((K, N), dtype=dtype, device=DEV)
    for bias in (torch.randn((N,), dtype=dtype, device=DEV), torch.randn((M, N), dtype=dtype, device=DEV)):
        ref = O.addmm(bias.cpu(), a.cpu(), b.cpu(), alpha=scalar, beta=scalar)
        with fg.use_gems():
            res = torch.addmm(bias, a, b, alpha=scalar, beta=scalar)
        assert_close(res.cpu(), ref, dtype, reduce_dim=K)


TC_SHAPES = [(128, 256, 64), (256, 512, 4096), (1000, 776, 520), (4096, 4096, 4096), (129, 264, 72), (64, 64, 32),
             (2048, 6144, 4096), (300, 16, 4096), (8, 3000, 128),
             # 256x256 tiles whose last wave is cut into 128-row halves (162, 896 and 512 tiles on 148 SMs),
             # the first with a ragged last row tile
             (2100, 4608, 512), (2048, 28672, 256), (8192, 4096, 512)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_col,b_col", [(False, False), (False, True), (True, False), (True, True)])
def test_mm_tcgen05(fg, M, N, K, dtype, a_col, b_col):
    torch.manual_seed(1)
    a = torch.randn((K, M), dtype=dtype, device=DEV).t() if a_col else torch.randn((M, K), dtype=dtype, device=DEV)
    b = torch.randn((N, K), dtype=dtype, device=DEV).t() if b_col else torch.randn((K, N), dtype=dtype, device=DEV)
    res = fg.mm(a, b)
    # a column-major A needs a leading dimension that is a multiple of 16 bytes for TMA
    assert _uses_tcgen05(a, b, res) == (not a_col or M % 8 == 0), "unexpected kernel path for this shape"
    # CPU fp64 oracle on all rows when small, else on a sample that covers tile edges
    if M <= 512:
        rows = torch.arange(M, device=DEV)
    else:
        rows = torch.cat([torch.tensor([0, 1, 127, 128, 129, M - 129, M - 128, M - 1], device=DEV),
                          torch.randint(0, M, (120,), device=DEV)]).clamp_(0, M - 1)
    assert_close(res[rows].cpu(), O.mm(a[rows].cpu(), b.cpu()), dtype, reduce_dim=K)
    # every element against an independent fp32 product (loose: rounding of the result only)
    full = torch.mm(a.float(), b.float())
    torch.testing.assert_close(res.float(), full, rtol=2e-2, atol=1e-4 * K)


def test_addmm_tcgen05_epilogue_and_out_variants(fg):
    torch.manual_seed(2)
    M, N, K = 520, 1032, 768
    a = torch.randn((M, K), dtype=torch.bfloat16, device=DEV)
    b = torch.randn((K, N), dtype=torch.bfloat16, device=DEV) / K ** 0.5
    for bias in (torch.randn(N, dtype=torch.bfloat16, device=DEV), torch.randn(M, N, dtype=torch.bfloat16, device=DEV),
                 torch.randn(M, 1, dtype=torch.bfloat16, device=DEV)):
        ref = O.addmm(bias.cpu(), a.cpu(), b.cpu(), alpha=0.5, beta=-2.0)
        assert_close(fg.addmm(bias, a, b, alpha=0.5, beta=-2.0).cpu(), ref, torch.bfloat16, reduce_dim=K)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        assert fg.addmm_out(bias, a, b, alpha=0.5, beta=-2.0, out=out) is out
        assert_close(out.cpu(), ref, torch.bfloat16, reduce_dim=K)
        assert_close(torch.ops.flag_gems.addmm(bias, a, b, beta=-2.0, alpha=0.5).cpu(), ref, torch.bfloat16, reduce_dim=K)
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    with fg.use_gems():
        torch.mm(a, b, out=out)
    assert_close(out.cpu(), O.mm(a.cpu(), b.cpu()), torch.bfloat16, reduce_dim=K)
    assert_close(torch.ops.flag_gems.mm(a, b).cpu(), O.mm(a.cpu(), b.cpu()), torch.bfloat16, reduce_dim=K)
    # out with a padded leading dimension (row stride > N)
    wide = torch.zeros(M, N + 24, dtype=torch.bfloat16, device=DEV)
    fg.mm_out(a, b, out=wide[:, :N])
    assert_close(wide[:, :N].cpu(), O.mm(a.cpu(), b.cpu()), torch.bfloat16, reduce_dim=K)
    assert not wide[:, N:].any()


def test_gemm_edge_cases(fg):
    a = torch.randn(0, 16, device=DEV)
    assert fg.mm(a, torch.randn(16, 8, device=DEV)).shape == (0, 8)
    # K == 0: empty sum
    z = fg.mm(torch.randn(4, 0, device=DEV), torch.randn(0, 5, device=DEV))
    assert z.shape == (4, 5) and not z.any()
    bias = torch.randn(5, device=DEV)
    z = fg.addmm(bias, torch.randn(4, 0, device=DEV), torch.randn(0, 5, device=DEV), beta=2.0)
    torch.testing.assert_close(z, (bias * 2.0).expand(4, 5))
    with pytest.raises((AssertionError, RuntimeError)):
        fg.mm(torch.randn(4, 3, device=DEV), torch.randn(4, 3, device=DEV))
    with pytest.raises(RuntimeError):
        fg.mm(torch.randn(4, 3), torch.randn(3, 3))  # CPU tensors: no fallback


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_projection_shapes_linearity(fg, name):
    # Full benchmark shapes (M=8192): checked against the oracle on a sample of rows and
    # through a size-independent property: (2A) @ B == 2 (A @ B) exactly in bf16.
    a, b, bias = workloads.gemm_inputs(name, seed=4, device=DEV)
    K, N = workloads.GEMM_SHAPES[name]
    c = fg.mm(a, b)
    assert _uses_tcgen05(a, b, c)
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191], device=DEV)
    ref = O.mm(a[rows].cpu(), b.cpu())
    assert_close(c[rows].cpu(), ref, torch.bfloat16, reduce_dim=K)
    assert torch.equal(fg.mm(a * 2, b), c * 2)
    cb = fg.addmm(bias, a, b)
    assert_close(cb[rows].cpu(), O.addmm(bias.cpu(), a[rows].cpu(), b.cpu()), torch.bfloat16, reduce_dim=K)
    # column-major B (the nn.Linear weight form) gives the same product
    assert_close(fg.mm(a, b.t().contiguous().t())[rows].cpu(), ref, torch.bfloat16, reduce_dim=K)


# ---- bmm (aten::bmm override): the batch is the third dimension of the kernel's tensor maps
@pytest.mark.parametrize("M,N,K", MNK_SHAPES + [(256, 512, 128), (1000, 520, 264)])
@pytest.mark.parametrize("dtype", FLOAT_DTYPES)
def test_bmm(fg, M, N, K, dtype):
    # tests/test_blas_ops.py:95-111 (batch 4) plus shapes that take the tensor-core kernel
    torch.manual_seed(0)
    a = torch.randn((4, M, K), dtype=dtype, device=DEV)
    b = torch.randn((4, K, N), dtype=dtype, device=DEV)
    with fg.use_gems():
        out = torch.bmm(a, b)
    assert out.shape == (4, M, N) and out.dtype == dtype
    assert_close(out.cpu(), O.bmm(a.cpu(), b.cpu()), dtype, reduce_dim=K)


def test_bmm_layouts_and_batches(fg):
    torch.manual_seed(1)
    # transposed operands (column-major inner matrices), a broadcast batch and batch strides that
    # are not the packed ones; batch 1 and batch 33; empty batch
    a = torch.randn((6, 264, 384), dtype=torch.bfloat16, device=DEV)
    b = torch.randn((6, 512, 264), dtype=torch.bfloat16, device=DEV)
    out = fg.bmm(a.transpose(1, 2), b.transpose(1, 2))          # [6, 384, 264] x [6, 264, 512]
    assert_close(out.cpu(), O.bmm(a.transpose(1, 2).cpu(), b.transpose(1, 2).cpu()), torch.bfloat16, reduce_dim=264)
    w = torch.randn((264, 512), dtype=torch.bfloat16, device=DEV)
    out = fg.bmm(a.transpose(1, 2), w.expand(6, 264, 512))     # shared right operand
    assert_close(out.cpu(), O.bmm(a.transpose(1, 2).cpu(), w.expand(6, 264, 512).cpu()), torch.bfloat16, reduce_dim=264)
    big = torch.randn((33, 2, 128, 256), dtype=torch.float16, device=DEV)
    x, y = big[:, 0], big[:, 1].transpose(1, 2)                # batch stride 2 * 128 * 256
    assert_close(fg.bmm(x, y).cpu(), O.bmm(x.cpu(), y.cpu()), torch.float16, reduce_dim=256)
    assert_close(fg.bmm(x[:1], y[:1]).cpu(), O.bmm(x[:1].cpu(), y[:1].cpu()), torch.float16, reduce_dim=256)
    assert fg.bmm(x[:0], y[:0]).shape == (0, 128, 128)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1000, 1001, 1023), (513, 2049, 999), (2048, 2048, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b_col", [False, True])
def test_mm_unaligned_16bit_operands(fg, M, N, K, dtype, b_col):
    """Odd leading dimensions and views that start mid-row: the host pads such operands once so that
    the tensor-core kernel takes them; results against the fp64 oracle on every element."""
    torch.manual_seed(3)
    a_store = torch.randn((M, K + 3), dtype=dtype, device=DEV)
    a = a_store[:, 3:]                                   # base not 16-byte aligned, leading dimension K + 3
    b = torch.randn((N, K), dtype=dtype, device=DEV).t() if b_col else torch.randn((K, N), dtype=dtype, device=DEV)
    before = _lib.launch_count()
    res = fg.mm(a, b)
    assert _lib.launch_count() - before == 1
    assert res.shape == (M, N) and res.is_contiguous()
    assert_close(res.cpu(), O.mm(a.cpu(), b.cpu()), dtype, reduce_dim=K)
    bias = torch.randn((N,), dtype=dtype, device=DEV)
    with fg.use_gems():
        res2 = torch.addmm(bias, a, b, alpha=0.5, beta=2.0)
    assert_close(res2.cpu(), O.addmm(bias.cpu(), a.cpu(), b.cpu(), alpha=0.5, beta=2.0), dtype, reduce_dim=K)


@pytest.mark.parametrize("M,N,K", [(1536, 1664, 777), (2048, 1300, 64), (1500, 1536, 1025)])
@pytest.mark.parametrize("a_col,b_col", [(False, False), (True, True), (False, True)])
def test_mm_fp32_large_tiles(fg, M, N, K, a_col, b_col, monkeypatch):
    """fp32 (never TF32) on the 128 x 128 CUDA-core tiles, every operand majorness, M/N/K tails;
    the reference's fp32 tolerance against the fp64 oracle."""
    from flaggems_b200 import ops
    monkeypatch.setattr(ops, "_F32_SPLIT", False)      # keep these shapes on the CUDA-core kernel
    torch.manual_seed(4)
    a = torch.randn((K, M), device=DEV).t() if a_col else torch.randn((M, K), device=DEV)
    b = torch.randn((N, K), device=DEV).t() if b_col else torch.randn((K, N), device=DEV)
    res = fg.mm(a, b)
    assert_close(res.cpu(), O.mm(a.cpu(), b.cpu()), torch.float32, reduce_dim=K)
    bias = torch.randn((M, N), device=DEV)
    res2 = fg.addmm(bias, a, b, alpha=-0.999, beta=100.001)
    assert_close(res2.cpu(), O.addmm(bias.cpu(), a.cpu(), b.cpu(), alpha=-0.999, beta=100.001), torch.float32,
                 reduce_dim=K)


def _split_bytes(a, b, c):
    p = _lib.GemmParams()
    p.a, p.b, p.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    p.M, p.K = a.shape
    p.N = b.shape[1]
    p.a_stride0, p.a_stride1 = a.stride()
    p.b_stride0, p.b_stride1 = b.stride()
    p.c_stride0, p.c_stride1 = c.stride()
    p.dtype = _lib.dtype_code(c.dtype)
    return int(_lib.load().fg_gemm_f32_split_workspace_bytes(ctypes.byref(p)))


def _err(x, ref):
    d = (x.double() - ref).abs()
    return float(d.mean() / ref.abs().mean()), float(d.max() / ref.abs().max())


@pytest.mark.parametrize("M,N,K", [(1536, 1664, 777), (1000, 1111, 1300), (640, 2048, 4096), (129, 8200, 600)])
@pytest.mark.parametrize("a_col,b_col", [(False, False), (True, True), (False, True), (True, False)])
def test_mm_fp32_tensor_core_split(fg, M, N, K, a_col, b_col):
    """Large fp32 products on the tensor cores from three bf16 pieces per operand: every operand
    majorness, M/N/K tails.  The error against fp64 must stay at the level of an fp32 FMA loop
    (here: ATen's fp32 GEMM with TF32 off), not merely inside the reference's loose tolerance."""
    torch.manual_seed(5)
    a = torch.randn((K, M), device=DEV).t() if a_col else torch.randn((M, K), device=DEV)
    b = torch.randn((N, K), device=DEV).t() if b_col else torch.randn((K, N), device=DEV)
    assert _split_bytes(a, b, torch.empty((M, N), device=DEV)) > 0
    ref = a.double() @ b.double()
    res = fg.mm(a, b)
    assert_close(res.cpu(), ref.cpu(), torch.float32, reduce_dim=K)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        aten = torch.mm(a, b)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    mean_fg, max_fg = _err(res, ref)
    mean_at, max_at = _err(aten, ref)
    assert mean_fg <= 1.25 * mean_at + 1e-8, (mean_fg, mean_at)
    assert max_fg <= 2.0 * max_at + 1e-7, (max_fg, max_at)
    # addmm: full bias matrix and a row vector, scalars of the reference's grid
    bias = torch.randn((M, N), device=DEV)
    res2 = fg.addmm(bias, a, b, alpha=-0.999, beta=100.001)
    assert_close(res2.cpu(), O.addmm(bias.cpu(), a.cpu(), b.cpu(), alpha=-0.999, beta=100.001), torch.float32,
                 reduce_dim=K)
    row = torch.randn((N,), device=DEV)
    res3 = fg.addmm(row, a, b, alpha=0.001, beta=-111.999)
    assert_close(res3.cpu(), O.addmm(row.cpu(), a.cpu(), b.cpu(), alpha=0.001, beta=-111.999), torch.float32,
                 reduce_dim=K)


def test_mm_fp32_split_same_signed_data_and_output_views(fg):
    """Same-signed data is where a truncating accumulator shows: one tensor-core accumulator over
    K = 4096 is low by 1e-5 of the result; the chunked sums must stay below 1.5e-6.  Also an output
    view that allows no 16-byte stores."""
    torch.manual_seed(6)
    M, N, K = 512, 1024, 4096
    a = torch.rand((M, K), device=DEV)
    b = torch.rand((K, N), device=DEV)
    ref = a.double() @ b.double()
    res = fg.mm(a, b)
    rel = (res.double() - ref) / ref
    assert float(rel.abs().max()) < 1.5e-6, float(rel.abs().max())
    assert abs(float(rel.mean())) < 1.0e-6, float(rel.mean())
    buf = torch.full((M, N + 3), 7.0, device=DEV)
    out = buf[:, 1:N + 1]                       # rows start 4 bytes off a 16-byte boundary, odd pitch
    assert _split_bytes(a, b, out) > 0
    fg.mm_out(a, b, out=out)
    assert torch.equal(out, res)
    assert bool((buf[:, 0] == 7.0).all()) and bool((buf[:, N + 1:] == 7.0).all())


def test_mm_fp32_split_special_values(fg, monkeypatch):
    """An infinity or a NaN among the inputs: the pieces cannot carry it (inf times a zero piece
    is NaN), so the device-side flag hands the whole product to the CUDA-core kernel and the
    result is that kernel's, bit for bit."""
    from flaggems_b200 import ops
    torch.manual_seed(7)
    M, N, K = 512, 1024, 1024
    a = torch.randn((M, K), device=DEV)
    b = torch.randn((K, N), device=DEV)
    a[3, 5] = float("inf")
    b[7, 9] = float("nan")
    a[100, 0] = 3.4e38                             # rounds past the largest finite bf16: still finite
    assert _split_bytes(a, b, torch.empty((M, N), device=DEV)) > 0
    res = fg.mm(a, b)
    monkeypatch.setattr(ops, "_F32_SPLIT", False)
    simt = fg.mm(a, b)
    assert torch.equal(torch.nan_to_num(res, nan=1.5, posinf=2.5, neginf=-2.5),
                       torch.nan_to_num(simt, nan=1.5, posinf=2.5, neginf=-2.5))
    assert bool(torch.isinf(res[3]).any()) and bool(torch.isnan(res[:, 9]).all())
    # finite but huge values stay on the tensor cores and come out right
    monkeypatch.setattr(ops, "_F32_SPLIT", True)
    a2 = torch.randn((M, K), device=DEV)
    a2[100, 0] = 3.4e38
    b2 = torch.randn((K, N), device=DEV) * 1e-3
    r2 = fg.mm(a2, b2)
    ref2 = a2.double() @ b2.double()
    assert bool(torch.isfinite(r2).all())
    assert float(((r2.double() - ref2).abs() / ref2.abs().max()).max()) < 1e-6
