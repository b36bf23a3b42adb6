"""Quantiser parity on the GPU: e4m3 bytes and fp32 scales, bit for bit, against the
CPU oracle (IEEE division flavour), and the documented closeness of the
div.full.f32 flavour.  Calls go through the drop-in module, i.e. through the C ABI."""
import numpy as np
import pytest
import torch

from _util import assert_quant_equal, bits_of, bytes_of, ulp_distance
from cases import CASES, gen_input
from oracle import fp8_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    kernels.set_div_mode("rn")
    yield kernels
    kernels.set_div_mode("full")


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("rs", [False, True])
def test_rowwise_bit_exact(K, case, rs):
    name, seed, M, N, dtype, std, special = case
    x = gen_input(seed, M, N, dtype, std, special)
    q, s = K.quantize_fp8_rowwise(x.cuda(), 128, rs)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert_quant_equal(q, s, *O.quantize_rowwise(x, 128, rs), what=name)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("rs", [False, True])
def test_blockwise_bit_exact(K, case, rs):
    name, seed, M, N, dtype, std, special = case
    x = gen_input(seed, M, N, dtype, std, special)
    q, s = K.quantize_fp8_blockwise(x.cuda(), 128, 128, rs)
    assert_quant_equal(q, s, *O.quantize_blockwise(x, 128, 128, rs), what=name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_rowwise_layouts(K, dtype):
    g = torch.Generator().manual_seed(77)
    base = torch.randn(384, 512, generator=g).to(dtype)
    xc = base.cuda()
    # transposed view: tiles run along the strided axis (weight-gradient path)
    q, s = K.quantize_fp8_rowwise(xc.t(), 128, False)
    assert_quant_equal(q, s, *O.quantize_rowwise(base.t().contiguous(), 128, False), what="transposed view")
    # row slice with a pitch, column slice (misaligned start), every-other-column view
    for view_name, fn in {"pitched": lambda t: t[:, :256], "offset": lambda t: t[3:50, 5:300],
                          "strided": lambda t: t[:, ::2], "one_row": lambda t: t[7:8, :]}.items():
        q, s = K.quantize_fp8_rowwise(fn(xc), 128, True)
        assert_quant_equal(q, s, *O.quantize_rowwise(fn(base).contiguous(), 128, True), what=view_name)
        q, s = K.quantize_fp8_blockwise(fn(xc), 128, 128, False)
        assert_quant_equal(q, s, *O.quantize_blockwise(fn(base).contiguous(), 128, 128, False), what=view_name)


def test_transposed_view_ragged(K):
    g = torch.Generator().manual_seed(78)
    base = torch.randn(200, 136, generator=g).bfloat16()        # logical (136, 200): N = 200 is ragged
    q, s = K.quantize_fp8_rowwise(base.cuda().t(), 128, False)
    assert_quant_equal(q, s, *O.quantize_rowwise(base.t().contiguous(), 128, False), what="ragged transposed")
    base = torch.randn(272, 136, generator=g).bfloat16()        # N = 272: multiple of 16, not of 128
    q, s = K.quantize_fp8_rowwise(base.cuda().t(), 128, True)
    assert_quant_equal(q, s, *O.quantize_rowwise(base.t().contiguous(), 128, True), what="ragged transposed 272")


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("rs", [False, True])
def test_dual_rowwise_bit_exact(K, case, rs):
    """One pass, two quantisations: tiles along the columns and tiles along the rows of the transpose."""
    name, seed, M, N, dtype, std, special = case
    x = gen_input(seed, M, N, dtype, std, special)
    q_row, s_row, q_col, s_col = K.quantize_fp8_rowwise_dual(x.cuda(), rs)
    assert q_col.shape == (N, M) and s_col.shape == (N, (M + 127) // 128)
    assert_quant_equal(q_row, s_row, *O.quantize_rowwise(x, 128, rs), what=name + " rows")
    assert_quant_equal(q_col, s_col, *O.quantize_rowwise(x.t().contiguous(), 128, rs), what=name + " columns")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(256, 384), (144, 136), (16, 8), (400, 1000), (130, 264), (77, 200)])
def test_dual_rowwise_shapes(K, dtype, shape):
    """Fused path (rows a multiple of 16, columns of 8) and the ragged fallback, on a pitched view too."""
    M, N = shape
    g = torch.Generator().manual_seed(M * 1000 + N)
    base = (torch.randn(M, N + 16, generator=g) * torch.logspace(-3, 2, N + 16)[None, :]).to(dtype)
    base[M // 2, :] = 0                                               # an all-zero tile: floor 1e-4
    xc = base.cuda()
    for what, view, ref in (("contiguous", xc[:, :N].contiguous(), base[:, :N]), ("pitched", xc[:, 8:N + 8], base[:, 8:N + 8])):
        q_row, s_row, q_col, s_col = K.quantize_fp8_rowwise_dual(view, False)
        assert_quant_equal(q_row, s_row, *O.quantize_rowwise(ref.contiguous(), 128, False), what=what + " rows")
        assert_quant_equal(q_col, s_col, *O.quantize_rowwise(ref.t().contiguous(), 128, False), what=what + " columns")
        # and the same bytes as the two single-output calls
        q1, s1 = K.quantize_fp8_rowwise(view, 128, False)
        q2, s2 = K.quantize_fp8_rowwise(view.t(), 128, False)
        assert torch.equal(q1.view(torch.uint8), q_row.view(torch.uint8)) and torch.equal(s1, s_row)
        assert torch.equal(q2.view(torch.uint8), q_col.view(torch.uint8)) and torch.equal(s2, s_col)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(256, 384), (130, 272), (77, 208), (1000, 512), (16, 16)])
@pytest.mark.parametrize("rs", [False, True])
def test_rowwise_with_block_equals_separate_calls(K, dtype, shape, rs):
    """One pass over x: its 1x128 quantisation and the 128x128 re-quantisation of that, bit for bit what the row-wise
    quantiser followed by the row-to-block re-quantiser give, and what the oracle gives."""
    M, N = shape
    g = torch.Generator().manual_seed(M * 7 + N)
    base = (torch.randn(M, N + 16, generator=g) * torch.logspace(-3, 2, N + 16)[None, :]).to(dtype)
    base[M // 3, :] = 0
    xc = base.cuda()
    for view, ref in ((xc[:, :N].contiguous(), base[:, :N]), (xc[:, 16:N + 16], base[:, 16:N + 16])):
        q_row, s_row, q_blk, s_blk = K.quantize_fp8_rowwise_with_block(view, rs)
        q1, s1 = K.quantize_fp8_rowwise(view, 128, rs)
        q2, s2 = K.requantize_rowwise_to_blockwise(q1, s1)
        assert torch.equal(q_row.view(torch.uint8), q1.view(torch.uint8)) and torch.equal(s_row, s1)
        assert torch.equal(q_blk.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s_blk, s2)
        oq, os_ = O.quantize_rowwise(ref.contiguous(), 128, rs)
        assert_quant_equal(q_row, s_row, oq, os_, what="rows")
        assert_quant_equal(q_blk, s_blk, *O.requantize_row_to_block(oq, os_), what="blocks")


@pytest.mark.parametrize("rs", [False, True])
def test_every_bf16_amax(K, rs):
    """For bf16 input the scale is a function of the tile's amax alone: sweep every
    positive finite bf16 value as the amax of one tile."""
    bits = torch.arange(1, 0x7F80, dtype=torch.int32).to(torch.int16)
    vals = bits.view(torch.bfloat16)
    x = torch.zeros(vals.numel(), 128, dtype=torch.bfloat16)
    x[:, 0] = vals
    x[:, 1] = -vals * 0.5
    x[:, 2] = vals * 0.0625
    q, s = K.quantize_fp8_rowwise(x.cuda(), 128, rs)
    assert_quant_equal(q, s, *O.quantize_rowwise(x, 128, rs), what="bf16 amax sweep")


def test_other_tile_sizes(K):
    g = torch.Generator().manual_seed(79)
    x = torch.randn(50, 300, generator=g)
    for bs in (32, 64, 256):
        q, s = K.quantize_fp8_rowwise(x.cuda(), bs, False)
        assert_quant_equal(q, s, *O.quantize_rowwise(x, bs, False), what=f"block_size {bs}")
    q, s = K.quantize_fp8_blockwise(x.cuda(), 64, 32, True)
    assert_quant_equal(q, s, *O.quantize_blockwise(x, 64, 32, True), what="64x32 blocks")


def test_nan_inf_and_empty(K):
    x = torch.zeros(2, 256)
    x[0, 3] = float("nan")
    x[0, 4] = 2.0
    x[1, 130] = float("inf")
    x[1, 131] = -1.0
    q, s = K.quantize_fp8_rowwise(x.cuda(), 128)
    assert_quant_equal(q, s, *O.quantize_rowwise(x, 128), what="nan/inf")
    q, s = K.quantize_fp8_rowwise(torch.empty(0, 128, device="cuda"))
    assert q.shape == (0, 128) and s.shape == (0, 1)
    q, s = K.quantize_fp8_blockwise(torch.empty(0, 128, device="cuda"))
    assert q.shape == (0, 128) and s.shape == (0, 1)


def test_requantize_row_to_block(K):
    g = torch.Generator().manual_seed(80)
    for (M, Kd) in [(256, 512), (130, 144), (16, 128)]:
        x = torch.randn(M, Kd, generator=g).bfloat16()
        xq, xs = O.quantize_rowwise(x, 128, True)
        ref_q, ref_s = O.requantize_row_to_block(xq, xs)
        xq_g = xq.cuda().view(torch.float8_e4m3fn)
        q, s = K.requantize_rowwise_to_blockwise(xq_g, xs.cuda())
        assert_quant_equal(q, s, ref_q, ref_s, what=f"requant {M}x{Kd}")
        if M % 16 == 0:
            qt, st = K.requantize_rowwise_to_blockwise(xq_g, xs.cuda(), transpose_out=True)
            assert_quant_equal(qt, st, ref_q.t().contiguous(), ref_s, what=f"requant^T {M}x{Kd}")


def test_dequantisers(K, golden):
    for tag in ("deq_a", "deq_ragged"):
        codes = torch.from_numpy(golden[f"{tag}/codes"])
        scales = torch.from_numpy(golden[f"{tag}/scales"])
        y = K.dequantize_fp8_rowwise(codes.cuda().view(torch.float8_e4m3fn), scales.cuda(), 128)
        assert y.dtype == torch.float32
        assert np.array_equal(bits_of(y), golden[f"{tag}/out"].view(np.uint32))     # the reference's own output
    g = torch.Generator().manual_seed(81)
    x = torch.randn(200, 300, generator=g)
    q, s = O.quantize_blockwise(x, 128, 128)
    y = K.dequantize_fp8(q.cuda().view(torch.float8_e4m3fn), s.cuda(), 128, 128)
    ref = O.dequantize_block(q, s, 128, 128)
    assert y.dtype == torch.bfloat16 and torch.equal(y.cpu(), ref)


def test_reference_suite_cases(K):
    """The reference's own quantiser tests (tests/test_kernels.py:30-76) on seeded inputs."""
    g = torch.Generator().manual_seed(82)
    x = torch.randn(256, 512, generator=g).bfloat16().cuda()
    q, s = K.quantize_fp8_rowwise(x, block_size=128)
    assert q.shape == x.shape and q.dtype == torch.float8_e4m3fn and s.shape == (256, 4)
    w = torch.randn(512, 512, generator=g).bfloat16().cuda()
    wq, ws = K.quantize_fp8_blockwise(w, block_m=128, block_n=128)
    assert wq.shape == w.shape and ws.shape == (4, 4)
    rec = K.dequantize_fp8(q, s, block_m=1, block_n=128)
    rel = (x.float() - rec.float()).abs() / (x.float().abs() + 1e-6)
    assert rel.mean().item() < 0.1
    x[0, 0] = 1000.0
    x[100, 200] = -500.0
    q, s = K.quantize_fp8_rowwise(x, block_size=128)
    rec = K.dequantize_fp8(q, s, block_m=1, block_n=128)
    assert not torch.isnan(rec).any() and not torch.isinf(rec).any()


def test_hoisted_reciprocal_equals_div_full(K):
    """The default flavour multiplies by one rcp.approx per scale; on this GPU that product must have the bits of
    div.full.f32 for every 16-bit input and every scale a 16-bit amax can produce."""
    assert K.selfcheck_division() == 0


def test_full_division_flavour_is_close(K):
    """div.full.f32 (what Triton emits for the reference on a GPU) is a <= 2 ulp division:
    scales stay within 2 ulp of the IEEE ones and a byte moves by at most one e4m3 step."""
    x = gen_input(1001, 512, 1024, torch.bfloat16, 1.0, None)
    K.set_div_mode("full")
    try:
        q, s = K.quantize_fp8_rowwise(x.cuda(), 128, False)
        q2, s2 = K.quantize_fp8_rowwise(x.cuda(), 128, True)
    finally:
        K.set_div_mode("rn")
    rq, rs_ = O.quantize_rowwise(x, 128, False)
    assert ulp_distance(bits_of(s), rs_.numpy().view(np.uint32)).max() <= 2
    dq = O.e4m3_decode(bytes_of(q)).astype(np.float64)
    dr = O.e4m3_decode(rq.numpy()).astype(np.float64)
    step = np.maximum(np.abs(dr) * 0.125, 2.0 ** -9)
    assert np.all(np.abs(dq - dr) <= step + 1e-12)
    frac = float((bytes_of(q) != rq.numpy()).mean())
    assert frac < 2e-3, frac
    # power-of-two scales: the division by the scale is exact in both flavours
    rq2, rs2 = O.quantize_rowwise(x, 128, True)
    m, _ = torch.frexp(s2.cpu())
    assert torch.all(m == 0.5)
    same_scale = (bits_of(s2) == rs2.numpy().view(np.uint32))
    assert same_scale.mean() > 0.999
    rows_ok = np.repeat(same_scale, 128, axis=1)
    assert np.array_equal(bytes_of(q2)[rows_ok], rq2.numpy()[rows_ok])


def test_config2_activation_full_size(K):
    """x of the FFN-width configuration, 16384 x 7168 bf16: full bit-exact parity."""
    x = gen_input(1002, 16384, 7168, torch.bfloat16, 1.0, None)
    xc = x.cuda()
    q, s = K.quantize_fp8_rowwise(xc, 128, False)
    assert_quant_equal(q, s, *O.quantize_rowwise(x, 128, False), what="C2 x")
    # transposed-view kernel at size: compare a band of logical rows
    qt, st = K.quantize_fp8_rowwise(xc.t(), 128, False)
    band = slice(1024, 1024 + 256)
    rq, rs_ = O.quantize_rowwise(x[:, band].t().contiguous(), 128, False)
    assert_quant_equal(qt[band], st[band], rq, rs_, what="C2 x^T band")
    # idempotence: quantising the de-quantised tensor reproduces bytes and scales
    y = K.dequantize_fp8_rowwise(q, s, 128)
    q2, s2 = K.quantize_fp8_rowwise(y, 128, False)
    assert torch.equal(s2, s)
    assert (q2.view(torch.uint8) != q.view(torch.uint8)).float().mean().item() < 1e-6


@pytest.mark.parametrize("shape", [(256, 512), (384, 640), (132, 200), (16, 128), (2048, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_blockwise_with_transposed_copy(K, shape, dtype):
    """One pass, two layouts: (M, N) and its byte transpose (N, M), one set of scales (src/kernels.py:747-748)."""
    M, N = shape
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn(M, N, generator=g) * 0.02).to(dtype)
    q, s, q_t = K.quantize_fp8_blockwise_t(x.cuda())
    assert_quant_equal(q, s, *O.quantize_blockwise(x, 128, 128, False), what="block copy")
    assert q_t.shape == (N, M) and torch.equal(q_t.view(torch.uint8), q.view(torch.uint8).t())


@pytest.mark.parametrize("shape", [(256, 512), (144, 272), (1024, 896), (16, 16), (130, 72), (7, 13), (64, 4)])
def test_byte_transposer(K, shape):
    R, C = shape
    g = torch.Generator().manual_seed(R * C)
    x = torch.randint(0, 256, (R, C), generator=g, dtype=torch.uint8).cuda()
    assert torch.equal(K.transpose_fp8(x), x.t().contiguous())
    wide = torch.randint(0, 256, (R, C + 8), generator=g, dtype=torch.uint8).cuda()
    assert torch.equal(K.transpose_fp8(wide[:, :C]), wide[:, :C].t().contiguous())        # pitched rows


@pytest.mark.parametrize("shape", [(256, 512), (144, 272), (16, 128), (1040, 384)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rs", [False, True])
def test_rowwise_with_transposed_block_copy(K, shape, dtype, rs):
    """The row + block pass with the block copy written (N, M): same bytes as the untransposed variant, transposed."""
    M, N = shape
    g = torch.Generator().manual_seed(3 * M + N)
    x = torch.randn(M, N, generator=g).to(dtype).cuda()
    q_row, s_row, q_blk, s_blk = K.quantize_fp8_rowwise_with_block(x, rs)
    q_row2, s_row2, q_blk_t, s_blk2 = K.quantize_fp8_rowwise_with_block(x, rs, transpose_block=True)
    assert torch.equal(q_row.view(torch.uint8), q_row2.view(torch.uint8)) and torch.equal(s_row, s_row2)
    assert torch.equal(s_blk, s_blk2)
    assert q_blk_t.shape == (N, M) and torch.equal(q_blk_t.view(torch.uint8), q_blk.view(torch.uint8).t())
    ref_q, ref_s = O.requantize_row_to_block(*O.quantize_rowwise(x.cpu(), 128, rs))
    assert_quant_equal(q_blk, s_blk, ref_q, ref_s, what="block copy")
