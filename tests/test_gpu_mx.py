"""MX block-scaled dot (`b200$block_scaled_dot$mx`, the stand-in for `__cublas$lt$matmul$mx`) against the
oracle's restatement of the reference's expansion (block_scaling_rewriter.cc:194-262): operands
dequantized element by element with one f8e8m0fnu scale per 32 values along K, then an f32 dot.

Tolerance.  The reference's own block-scaled tests compare a GPU run with the expanded HLO under
ErrorSpec{1e-4, 1e-5} for f32 results on inputs of modest size
(xla/backends/gpu/transforms/block_scaling_rewriter_cudnn_test.cc); here every element must satisfy
    |got - want| <= 2^-16 * sum_k |a_k * b_k|  (+ one step of the result type: 2^-23, 2^-7 or 2^-10 of |want|)
which bounds the f32 summation-order difference for K up to 4096 and is far below one scale step (a
wrong scale byte is off by a factor of two in a whole 32-block).
"""
import numpy as np
import pytest
import torch

from oracle import scaled_dot_oracle as o
from xla_b200 import cublas_lt_matmul_mx, device_status
from xla_b200.scaled_dot import BlockScaledDotCall, Buffer, F8E8M0FNU, XlaFfiError

pytestmark = pytest.mark.gpu

F8 = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def _dev(x, dev, dt=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    return t if dt is None else t.view(dt)


def _abs_dot(a, b, sa, sb, ka, kb):
    a_dq = np.abs(o.mx_dequantize(a, sa, ka)).astype(np.float64)
    b_dq = np.abs(o.mx_dequantize(b, sb, kb)).astype(np.float64)
    return np.matmul(a_dq, np.swapaxes(b_dq, -1, -2))


MX_256, MX_224 = 6, 7          # B200SD_KERNEL_MX_256 / _224: one accumulator of 256 columns, two of 224
WIDTHS = pytest.mark.parametrize("kernel", [MX_256, MX_224], ids=["tile256", "tile224"])


def _run(dev, a, b, sa, sb, ka="e4m3fn", kb="e4m3fn", out=torch.float32, alpha=1.0, kernel=0, block_size=None):
    d = cublas_lt_matmul_mx(_dev(a, dev, F8[ka]), _dev(b, dev, F8[kb]), _dev(sa, dev), _dev(sb, dev), out_dtype=out,
                            alpha_real=alpha, selected_algorithm=kernel, block_size=block_size)
    torch.cuda.synchronize()
    assert device_status() == 0
    return d


def _check(got_f32, want_f32, absdot, ulp):
    err = np.abs(got_f32.astype(np.float64) - want_f32.astype(np.float64))
    bound = absdot * 2.0 ** -16 + ulp * np.abs(want_f32) + 1e-30
    bad = err > bound
    assert not bad.any(), (int(bad.sum()), float((err / bound).max()), np.argwhere(bad)[:4].tolist())
    return float((err / (absdot + 1e-30)).max())


@pytest.mark.parametrize("m,n,k,batch", [
    (256, 512, 256, 0),       # one tile row, two tile columns, two k-blocks
    (16, 16, 256, 4),         # the reference's own test shape (block_scaling_rewriter_test.cc:90-123), batched
    (512, 256, 1024, 0),
    (384, 768, 512, 2),
    (128, 256, 128, 0),       # a single k-block; the pair's second CTA has no valid rows
])
@WIDTHS
def test_mx_dot_f32(cuda_device, m, n, k, batch, kernel):
    a, b, sa, sb = o.make_mx_operands(m * 7 + n, m, n, k, batch=batch)
    want = o.block_scaled_dot(a, b, sa, sb)
    got = _run(cuda_device, a, b, sa, sb, kernel=kernel).cpu().numpy()
    assert got.shape == want.shape
    _check(got, want, _abs_dot(a, b, sa, sb, "e4m3fn", "e4m3fn"), 2.0 ** -23)


@pytest.mark.parametrize("m,n,k", [(200, 136, 160), (300, 260, 96), (77, 33, 32), (129, 257, 416), (520, 700, 1024)])
@WIDTHS
def test_mx_dot_ragged_shapes(cuda_device, m, n, k, kernel):
    """Rows, columns and k-blocks that fill no tile, rows of scales that start on odd addresses
    (k / 32 not a multiple of 4: the scale loader's byte path) and results whose rows are not 16-byte
    multiples (scalar stores)."""
    a, b, sa, sb = o.make_mx_operands(m + n + k, m, n, k)
    want = o.block_scaled_dot(a, b, sa, sb)
    got = _run(cuda_device, a, b, sa, sb, kernel=kernel).cpu().numpy()
    _check(got, want, _abs_dot(a, b, sa, sb, "e4m3fn", "e4m3fn"), 2.0 ** -23)


@pytest.mark.parametrize("ka,kb", [("e5m2", "e4m3fn"), ("e4m3fn", "e5m2"), ("e5m2", "e5m2")])
def test_mx_dot_e5m2_operands(cuda_device, ka, kb):
    m, n, k = 256, 256, 384
    a, b, sa, sb = o.make_mx_operands(5, m, n, k, kind_a=ka, kind_b=kb)
    want = o.block_scaled_dot(a, b, sa, sb, a_kind=ka, b_kind=kb)
    got = _run(cuda_device, a, b, sa, sb, ka, kb).cpu().numpy()
    _check(got, want, _abs_dot(a, b, sa, sb, ka, kb), 2.0 ** -23)


@pytest.mark.parametrize("out,code,ulp", [(torch.bfloat16, o.BF16, 2.0 ** -7), (torch.float16, o.F16, 2.0 ** -10)])
@WIDTHS
def test_mx_dot_16_bit_results(cuda_device, out, code, ulp, kernel):
    m, n, k = 512, 384, 256
    # scales near one keep every value inside f16's range
    a, b, sa, sb = o.make_mx_operands(11, m, n, k, scale_lo=122, scale_hi=128)
    want = o.output_to_f32(o.block_scaled_dot(a, b, sa, sb, out_dtype=code), code)
    got = _run(cuda_device, a, b, sa, sb, out=out, kernel=kernel).float().cpu().numpy()
    _check(got, want, _abs_dot(a, b, sa, sb, "e4m3fn", "e4m3fn"), ulp)


@WIDTHS
def test_mx_scale_semantics(cuda_device, kernel):
    """Known answers that isolate the scale bytes: all-ones operands make every output
    sum_blocks 32 * 2^(sa - 127) * 2^(sb - 127); one block scale at a time is changed."""
    m, n, k = 256, 256, 256
    one = int(o.fp8_encode(np.array([1.0], np.float32))[0])
    a = np.full((m, k), one, np.uint8)
    b = np.full((n, k), one, np.uint8)
    sa = np.full((m, k // 32), 127, np.uint8)
    sb = np.full((n, k // 32), 127, np.uint8)
    rng = np.random.default_rng(3)
    for _ in range(6):
        r, j = int(rng.integers(m)), int(rng.integers(k // 32))
        sa[r, j] = 127 + int(rng.integers(-6, 7))
        c, j2 = int(rng.integers(n)), int(rng.integers(k // 32))
        sb[c, j2] = 127 + int(rng.integers(-6, 7))
    want = o.block_scaled_dot(a, b, sa, sb)
    got = _run(cuda_device, a, b, sa, sb, kernel=kernel).cpu().numpy()
    assert (got == want).all()          # powers of two: exact whatever the summation order
    assert want.min() != want.max()


def test_mx_alpha_and_nan_scale(cuda_device):
    m, n, k = 256, 256, 128
    a, b, sa, sb = o.make_mx_operands(21, m, n, k)
    sa[5, 2] = 255                     # f8e8m0fnu NaN: the whole row of D becomes NaN, nothing else
    want = o.block_scaled_dot(a, b, sa, sb, alpha=0.5)
    got = _run(cuda_device, a, b, sa, sb, alpha=0.5).cpu().numpy()
    assert np.isnan(got[5]).all() and np.isnan(want[5]).all()
    keep = np.ones(m, bool)
    keep[5] = False
    sa_ok = sa.copy()
    sa_ok[5, 2] = 127
    _check(got[keep], want[keep], 0.5 * _abs_dot(a, b, sa_ok, sb, "e4m3fn", "e4m3fn")[keep], 2.0 ** -23)


@WIDTHS
def test_mx_dot_full_size_sampled(cuda_device, kernel):
    """4096^3: every output row block is produced by the same code path; 96 sampled rows are compared
    with the oracle and the whole result against a linearity property (doubling one operand's scales
    doubles D exactly)."""
    m = n = k = 4096
    a, b, sa, sb = o.make_mx_operands(4096, m, n, k, scale_lo=121, scale_hi=131)
    d = _run(cuda_device, a, b, sa, sb, kernel=kernel)
    rows = np.random.default_rng(0).choice(m, 96, replace=False)
    want = o.block_scaled_dot(a[rows], b, sa[rows], sb)
    _check(d.cpu().numpy()[rows], want, _abs_dot(a[rows], b, sa[rows], sb, "e4m3fn", "e4m3fn"), 2.0 ** -23)
    d2 = _run(cuda_device, a, b, (sa + 1).astype(np.uint8), sb, kernel=kernel)
    assert torch.equal(d2, d * 2)


@pytest.mark.parametrize("m,n,k,batch,a_pad,b_pad", [
    (120, 120, 96, 4, (128, 4), (128, 4)),        # the reference's CudnnScaledDotPaddedScales shapes (block_scaling_rewriter_test.cc:329-345): byte loads
    (250, 250, 224, 0, (256, 8), (256, 8)),       # Mxfp8_PaddedScales (block_scaling_rewriter_cudnn_test.cc:105-121): 4-byte rows, 7 of 8 scales in use
    (300, 260, 512, 0, (304, 32), (264, 32)),     # rows of 32 bytes, 16 in use: TMA boxes over a strided corner
    (256, 512, 384, 0, (256, 16), (512, 16)),     # 12 of 16 in use: the box reaches past the corner, which must read as zero
    (384, 768, 512, 2, (400, 20), (768, 16)),     # batched; A's scales padded in both directions (word loads), B's not at all
    (200, 136, 1024, 2, (208, 48), (144, 64)),    # batched TMA path, two groups of four k-blocks, different padding per operand
])
@WIDTHS
def test_mx_padded_scales(cuda_device, m, n, k, batch, a_pad, b_pad, kernel):
    """Scale arrays larger than [rows, k / 32]: only the leading corner is read, as the reference slices it
    (block_scaling_rewriter.cc:469-518).  The padding holds NaN codes, so one padded byte taken for a scale, even
    against an all-zero block of values, shows in the result."""
    a, b, sa, sb = o.make_mx_operands(m + 3 * n + k, m, n, k, batch=batch)
    lead = (batch,) if batch else ()
    sa_p = np.full(lead + a_pad, 0xFF, np.uint8)
    sb_p = np.full(lead + b_pad, 0xFF, np.uint8)
    sa_p[..., :m, : k // 32] = sa
    sb_p[..., :n, : k // 32] = sb
    want = o.block_scaled_dot(a, b, sa, sb)
    assert np.array_equal(o.block_scaled_dot(a, b, sa_p, sb_p, block_size=32), want)
    got = _run(cuda_device, a, b, sa_p, sb_p, kernel=kernel, block_size=32).cpu().numpy()
    assert np.isfinite(got).all()
    _check(got, want, _abs_dot(a, b, sa, sb, "e4m3fn", "e4m3fn"), 2.0 ** -23)
    # and bit for bit what the same call gives on the unpadded arrays
    assert np.array_equal(got, _run(cuda_device, a, b, sa, sb, kernel=kernel).cpu().numpy())


def test_mx_call_frame_contract(cuda_device):
    """Operand count, scale shape and types are checked when the call site is instantiated."""
    dev = cuda_device
    a = torch.zeros((64, 128), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    b = torch.zeros((32, 128), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    s4 = torch.zeros((64, 4), dtype=torch.uint8, device=dev)
    t4 = torch.zeros((32, 4), dtype=torch.uint8, device=dev)
    d = torch.empty((64, 32), dtype=torch.float32, device=dev)

    def sc(t, dims=None):
        return Buffer(F8E8M0FNU, tuple(dims or t.shape), t.data_ptr())

    BlockScaledDotCall([a, b, sc(s4), sc(t4)], [d]).instantiate()
    with pytest.raises(XlaFfiError):          # three operands
        BlockScaledDotCall([a, b, sc(s4)], [d]).instantiate()
    with pytest.raises(XlaFfiError):          # block size 64
        BlockScaledDotCall([a, b, sc(s4, (64, 2)), sc(t4, (32, 2))], [d]).instantiate()
    with pytest.raises(XlaFfiError):          # scales that do not cover the rows
        BlockScaledDotCall([a, b, sc(s4, (60, 4)), sc(t4)], [d]).instantiate()
    s8 = torch.zeros((72, 8), dtype=torch.uint8, device=dev)
    BlockScaledDotCall([a, b, sc(s8, (72, 4)), sc(t4)], [d]).instantiate()                 # extra scale rows are taken as they are
    BlockScaledDotCall([a, b, sc(s8), sc(t4)], [d], block_size=32).instantiate()          # extra columns once the block size is stated
    with pytest.raises(XlaFfiError):          # ... and not otherwise: [72, 8] over k = 128 reads as block size 16
        BlockScaledDotCall([a, b, sc(s8), sc(t4)], [d]).instantiate()
    with pytest.raises(XlaFfiError):
        BlockScaledDotCall([a, b, sc(s4), sc(t4)], [d], block_size=16).instantiate()
    with pytest.raises(XlaFfiError):          # f32 scales
        BlockScaledDotCall([a, b, torch.zeros((64, 4), device=dev), torch.zeros((32, 4), device=dev)], [d]).instantiate()
    with pytest.raises(XlaFfiError):          # FP8 result
        BlockScaledDotCall([a, b, sc(s4), sc(t4)], [torch.empty((64, 32), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)]).instantiate()
