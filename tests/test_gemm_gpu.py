"""Block-scaled FP8 GEMM parity: CUDA (through the C ABI) against the float64
dequantise -> matmul oracle.  Tolerance from the specification: relative
Frobenius error <= 1e-3 on the fp32 result; the bf16 result is compared with the
float64 result rounded to bf16."""
import numpy as np
import pytest
import torch

from _util import assert_bf16_close, bits_of, bytes_of, rel_fro
from oracle import fp8_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-3          # rel-Frobenius bound of the specification (fp32 output)


@pytest.fixture(scope="module")
def K():
    from cinnamon_b200 import kernels
    kernels.set_div_mode("rn")
    yield kernels
    assert kernels.device_status() == 0, "a kernel gave up on a bounded wait"
    kernels.set_div_mode("full")


def _operands(M, N, Kd, seed):
    x, w, _ = O.make_linear_case(M, Kd, N, seed)
    xq, xs = O.quantize_rowwise(x, 128)
    wq, ws = O.quantize_blockwise(w.float(), 128, 128)
    return xq, xs, wq, ws


def _f8(t):
    return t.cuda().view(torch.float8_e4m3fn)


SHAPES = [(128, 256, 128), (256, 512, 512), (130, 576, 512), (130, 576, 640), (1, 128, 256), (300, 64, 1024),
          (4096, 2048, 512), (257, 1000, 144)]


@pytest.mark.parametrize("M,N,Kd", SHAPES)
def test_gemm_weight_layout_nk(K, M, N, Kd):
    """B given as the (N, K) weight seen through .t(): the forward layout."""
    xq, xs, wq, ws = _operands(M, N, Kd, seed=M + N + Kd)
    ref = O.fp8_matmul_f64(xq, wq.t(), xs, ws.t())
    out32 = K.fp8_matmul_dsv3(_f8(xq), _f8(wq).t(), xs.cuda(), ws.cuda().t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    err = rel_fro(out32, ref)
    maxabs = float((out32.cpu().double() - ref).abs().max())
    print(f"[{M}x{N}x{Kd}] fp32 rel-Fro {err:.3e} max-abs {maxabs:.3e}")
    assert err <= TOL
    assert err <= 2e-5          # e4m3 products are exact, only fp32 accumulation rounds
    out16 = K.fp8_matmul_dsv3(_f8(xq), _f8(wq).t(), xs.cuda(), ws.cuda().t())
    assert out16.dtype == torch.bfloat16
    assert_bf16_close(out16, ref, "bf16 output")
    assert (out16.cpu() != ref.to(torch.bfloat16)).float().mean().item() < 1e-2


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 128), (256, 512, 512), (130, 576, 640), (300, 64, 1024), (4096, 2048, 512)])
def test_gemm_layout_kn(K, M, N, Kd):
    """B stored (K, N) as fp8_matmul_dsv3 documents (src/kernels.py:669)."""
    xq, xs, wq, ws = _operands(M, N, Kd, seed=7 + M + N + Kd)
    b = wq.t().contiguous()
    bs = ws.t().contiguous()
    ref = O.fp8_matmul_f64(xq, b, xs, bs)
    out32 = K.fp8_matmul_dsv3(_f8(xq), _f8(b), xs.cuda(), bs.cuda(), out_dtype=torch.float32)
    err = rel_fro(out32, ref)
    print(f"[KN {M}x{N}x{Kd}] fp32 rel-Fro {err:.3e}")
    assert err <= TOL and err <= 2e-5


PAIR_SCRIPT = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from cinnamon_b200 import kernels as K
from oracle import fp8_oracle as O
M, N, Kd = 2304, 2560, 640          # 9 x 10 tiles of 256 x 256: enough for the two-SM kernel, ragged against nothing
xq, xs = O.quantize_rowwise(O.make_linear_case(M, Kd, N, 77)[0], 128)
w = O.make_linear_case(M, Kd, N, 77)[1]
wq, ws = O.quantize_blockwise(w.float(), 128, 128)
f8 = lambda t: t.cuda().view(torch.float8_e4m3fn)
nk = K.fp8_matmul_dsv3(f8(xq), f8(wq).t(), xs.cuda(), ws.cuda().t(), out_dtype=torch.float32)
b = wq.t().contiguous(); bs = ws.t().contiguous()
kn = K.fp8_matmul_dsv3(f8(xq), f8(b), xs.cuda(), bs.cuda(), out_dtype=torch.float32)
torch.cuda.synchronize()
assert K.device_status() == 0
torch.save({"nk": nk.cpu(), "kn": kn.cpu()}, sys.argv[2])
"""


def test_two_sm_and_one_sm_kernels_agree(K, tmp_path):
    """CINN_GEMM_PAIR=0 forces the one-SM kernel, =2 the two-SM (cta_group::2) kernel for both B layouts."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "pair.py"
    script.write_text(PAIR_SCRIPT)
    outs = {}
    for mode in ("0", "2"):
        out = tmp_path / f"out{mode}.pt"
        subprocess.check_call([sys.executable, str(script), root, str(out)], env=dict(os.environ, CINN_GEMM_PAIR=mode),
                              timeout=300)
        outs[mode] = torch.load(out)
    M, N, Kd = 2304, 2560, 640
    x, w, _ = O.make_linear_case(M, Kd, N, 77)
    xq, xs = O.quantize_rowwise(x, 128)
    wq, ws = O.quantize_blockwise(w.float(), 128, 128)
    ref = O.fp8_matmul_f64(xq, wq.t(), xs, ws.t())
    for mode in ("0", "2"):
        for layout in ("nk", "kn"):
            err = rel_fro(outs[mode][layout], ref)
            assert err <= TOL and err <= 2e-5, (mode, layout, err)
    assert rel_fro(outs["2"]["nk"], outs["0"]["nk"].double()) < 1e-6
    assert rel_fro(outs["2"]["kn"], outs["0"]["kn"].double()) < 1e-6


def test_gemm_is_deterministic(K):
    xq, xs, wq, ws = _operands(512, 1024, 1024, seed=5)
    a = K.fp8_matmul_dsv3(_f8(xq), _f8(wq).t(), xs.cuda(), ws.cuda().t(), out_dtype=torch.float32)
    b = K.fp8_matmul_dsv3(_f8(xq), _f8(wq).t(), xs.cuda(), ws.cuda().t(), out_dtype=torch.float32)
    assert torch.equal(a, b)


@pytest.mark.parametrize("M,Kd,N,rs", [(256, 512, 384, False), (512, 256, 640, True), (4096, 512, 2048, False)])
def test_autograd_function_matches_oracle(K, M, Kd, N, rs):
    """FP8MatmulFunction forward / dgrad / wgrad (src/kernels.py:739-794)."""
    x, w, dy = O.make_linear_case(M, Kd, N, seed=11 + M)
    ref_out, saved = O.fp8_linear_forward(x, w, rs)
    ref_gx, ref_gw = O.fp8_linear_backward(dy, saved, rs)
    xg = x.cuda().requires_grad_(True)
    wg = w.float().cuda().requires_grad_(True)
    out = K.FP8MatmulFunction.apply(xg, wg, rs)
    out.backward(dy.cuda())
    assert out.dtype == torch.bfloat16 and xg.grad.shape == x.shape and wg.grad.shape == w.shape
    for name, got, ref in (("fwd", out, ref_out), ("dgrad", xg.grad, ref_gx), ("wgrad", wg.grad, ref_gw)):
        err = rel_fro(got.detach().float(), ref)
        print(f"{name}: rel-Fro(bf16 out) {err:.3e}")
        assert_bf16_close(got.detach().to(torch.bfloat16), ref, name)
        assert err < 4e-3, name          # bf16 rounding alone costs ~1.7e-3


def test_fp8_linear_weight_cache(K):
    """The optional e4m3 weight cache: same outputs and gradients, one quantiser launch fewer per call while the
    weight is unchanged, refreshed after an in-place update."""
    torch.manual_seed(5)
    a = K.FP8Linear(256, 384).cuda()
    b = K.FP8Linear(256, 384, cache_quantized_weight=True).cuda()
    b.load_state_dict(a.state_dict())
    x = torch.randn(64, 256, device="cuda")
    for step in range(3):
        ya, yb = a(x), b(x)
        assert torch.equal(ya, yb)
        ya.sum().backward()
        yb.sum().backward()
        assert torch.equal(a.weight.grad, b.weight.grad)
        if step == 1:                                              # an optimiser step: the cache must notice
            with torch.no_grad():
                a.weight.add_(0.01)
                b.weight.add_(0.01)
        a.weight.grad = b.weight.grad = None
    n0 = K.launch_count
    b(x)
    cached = K.launch_count - n0
    n0 = K.launch_count
    a(x)
    assert K.launch_count - n0 == cached + 1


def test_grouped_gemm_scattered_rows(K):
    """Output rows stored at per-row addresses (the expert-parallel way home): here a permutation inside a local
    buffer, with a dropped row (address 0) and ragged expert sizes; same bits as the plain grouped GEMM."""
    g = torch.Generator().manual_seed(41)
    E, d_in, d_out = 4, 256, 384
    counts = [130, 0, 77, 200]
    T = sum(counts)
    x = torch.randn(T, d_in, generator=g).bfloat16().cuda()
    w = (torch.randn(E, d_out, d_in, generator=g) * 0.05).bfloat16().cuda()
    ends = torch.tensor(counts).cumsum(0).cuda()
    starts = ends - torch.tensor(counts).cuda()
    xq, xs = K.quantize_fp8_rowwise(x)
    wq, ws = K.quantize_expert_weights(w)
    ref = K.fp8_grouped_gemm(xq, xs, wq, ws, starts, ends, out_dtype=torch.bfloat16)
    perm = torch.randperm(T, generator=g).cuda()
    out = torch.full((T + 3, d_out), 7.0, dtype=torch.bfloat16, device="cuda")
    table = out.data_ptr() + perm * (d_out * 2)
    table[5] = 0                                                            # this row has no destination
    K.fp8_grouped_gemm_scatter(xq, xs, wq, ws, starts, ends, table.contiguous(), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    keep = torch.ones(T, dtype=torch.bool, device="cuda")
    keep[5] = False
    assert torch.equal(out[perm[keep]], ref[keep])
    assert torch.all(out[perm[5]] == 7.0) and torch.all(out[T:] == 7.0)     # untouched


def test_fp8_linear_module(K):
    g = torch.Generator().manual_seed(3)
    lin = K.FP8Linear(256, 384, bias=True, round_scale=True).cuda()
    x = torch.randn(2, 65, 256, generator=g).cuda()
    y = lin(x)
    assert y.shape == (2, 65, 384)
    ref, _ = O.fp8_linear_forward(x.cpu().reshape(-1, 256), lin.weight.detach().cpu(), True)
    ref = ref.reshape(2, 65, 384) + lin.bias.detach().cpu().double()
    assert rel_fro(y.float(), ref) < 4e-3
    y.sum().backward()
    assert lin.weight.grad is not None and lin.weight.grad.dtype == torch.float32


def test_weight_caches_and_updates_through_data(K):
    """The e4m3 copies follow every update that goes through the tensor (version counter); an update through
    ``.data`` leaves them stale until ``invalidate_weight_cache`` is called - the documented behaviour."""
    torch.manual_seed(6)
    E, d, h, T = 3, 256, 128, 96
    w = (torch.randn(E, h, d, device="cuda") * 0.02)
    x = torch.randn(T, d, device="cuda").bfloat16()
    starts = torch.tensor([0, 32, 64], device="cuda")
    ends = torch.tensor([32, 64, 96], device="cuda")
    y0 = K.moe_grouped_gemm(x, w, starts, ends)
    n0 = K.launch_count
    assert torch.equal(K.moe_grouped_gemm(x, w, starts, ends), y0)
    assert K.launch_count - n0 == 2                                 # token quantiser + GEMM: the weights came from the cache
    w.mul_(2.0)                                                     # in place through the tensor: noticed
    y1 = K.moe_grouped_gemm(x, w, starts, ends)
    torch.testing.assert_close(y1.float(), 2 * y0.float(), rtol=2e-2, atol=1e-3)
    w.data.mul_(0.5)                                                # behind autograd's back: not noticed ...
    assert torch.equal(K.moe_grouped_gemm(x, w, starts, ends), y1)
    K.invalidate_weight_cache()                                     # ... until the caches are dropped
    assert torch.equal(K.moe_grouped_gemm(x, w, starts, ends), y0)
    lin = K.FP8Linear(256, 128, cache_quantized_weight=True).cuda()
    z0 = lin(x)
    lin.weight.data.mul_(2.0)
    assert torch.equal(lin(x), z0)
    K.invalidate_weight_cache(lin)
    torch.testing.assert_close(lin(x).float(), 2 * z0.float(), rtol=2e-2, atol=1e-3)


def _grouped_case(E, d_in, d_out, counts, seed, gap=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(counts) + gap
    x = torch.randn(T, d_in, generator=g).bfloat16()
    w = (torch.randn(E, d_out, d_in, generator=g) * 0.02).bfloat16()
    ends = torch.tensor(counts).cumsum(0)
    starts = ends - torch.tensor(counts)
    return x, w, starts, ends


GROUPED = {
    "equal_reference_case": (8, 512, 128, [32] * 8),                       # tests/test_kernels.py:131-155
    "ragged": (6, 256, 384, [5, 0, 130, 1, 257, 64]),
    "empty_first_last": (5, 384, 256, [0, 200, 0, 129, 0]),
    "one_owns_all": (4, 256, 512, [0, 0, 700, 0]),
    "single_tokens": (16, 128, 128, [1] * 16),
    "wide_k": (3, 1024, 320, [100, 300, 28]),
}


@pytest.mark.parametrize("name", list(GROUPED))
def test_grouped_gemm(K, name):
    E, d_in, d_out, counts = GROUPED[name]
    x, w, starts, ends = _grouped_case(E, d_in, d_out, counts, seed=len(name), gap=9)
    ref = O.grouped_gemm_fp8_f64(x, w, starts, ends)
    xq, xs = K.quantize_fp8_rowwise(x.cuda())
    wq, ws = K.quantize_expert_weights(w.cuda())
    T = x.shape[0]
    out = torch.full((T, d_out), 777.0, dtype=torch.float32, device="cuda")       # canary everywhere
    K.fp8_grouped_gemm(xq, xs, wq, ws, starts.cuda(), ends.cuda(), out=out)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    used = int(ends[-1])
    assert torch.all(out[used:] == 777.0), "rows outside every expert's range were written"
    err = rel_fro(out[:used], ref[:used])
    print(f"{name}: rel-Fro {err:.3e}")
    assert err <= TOL and err <= 2e-5
    # the drop-in entry point: fp16 result like the reference, loose check like its own test
    out16 = K.moe_grouped_gemm(x.cuda(), w.cuda(), starts.cuda(), ends.cuda())
    assert out16.dtype == torch.float16 and out16.shape == (T, d_out)
    plain = O.grouped_gemm_f64(x, w, starts, ends)
    rel = ((plain[:used] - out16[:used].cpu().double()).abs() / (plain[:used].abs() + 1e-6))
    assert rel.median().item() < 0.08


@pytest.mark.parametrize("name", list(GROUPED))
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_grouped_gemm_16bit(K, name, dtype):
    """The grouped GEMM in the reference's precision (16-bit operands, fp32 accumulation on the tensor cores) against
    the float64 product of the same 16-bit operands; canary rows; then the drop-in in its "16bit" mode, forward and
    backward."""
    E, d_in, d_out, counts = GROUPED[name]
    x, w, starts, ends = _grouped_case(E, d_in, d_out, counts, seed=7 + len(name), gap=9)
    x, w = x.to(dtype), w.to(dtype)
    T, used = x.shape[0], int(ends[-1])
    ref = torch.zeros(T, d_out, dtype=torch.float64)
    for e in range(E):
        s, t = int(starts[e]), int(ends[e])
        ref[s:t] = x[s:t].double() @ w[e].double().t()
    out = torch.full((T, d_out), 777.0, dtype=torch.float32, device="cuda")
    K.grouped_gemm_16bit(x.cuda(), w.cuda(), starts.cuda(), ends.cuda(), out=out)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert torch.all(out[used:] == 777.0), "rows outside every expert's range were written"
    err = rel_fro(out[:used], ref[:used])
    print(f"{name} {dtype}: rel-Fro {err:.3e}")
    assert err < 2e-6                                            # exact products, fp32 accumulation
    out16 = K.grouped_gemm_16bit(x.cuda(), w.cuda(), starts.cuda(), ends.cuda(), out_dtype=torch.float16)
    torch.testing.assert_close(out16[:used].float().cpu(), ref[:used].float(), rtol=2e-3, atol=2e-3)
    prev = K.set_moe_grouped_precision("16bit")
    try:
        xg = x.float().cuda().requires_grad_(True)               # fp32 rows, as the reference's MoE passes them
        wg = w.float().cuda().requires_grad_(True)
        y = K.moe_grouped_gemm(xg, wg, starts.cuda(), ends.cuda())
        assert y.dtype == torch.float16
        rel = ((ref[:used] - y[:used].detach().cpu().double()).abs() / (ref[:used].abs() + 1e-6)).mean().item()
        assert rel < 0.01, rel                                   # the reference's own bound (tests/test_kernels.py:155)
        y.float().pow(2).mean().backward()
        assert torch.isfinite(xg.grad).all() and torch.isfinite(wg.grad).all() and wg.grad.abs().sum() > 0
    finally:
        K.set_moe_grouped_precision(prev)


def test_config2_full_size_sampled(K):
    """16384 x 18432 x 7168 forward; rows sampled for the float64 check."""
    M, Kd, N = 16384, 7168, 18432
    g = torch.Generator().manual_seed(1002)
    x = torch.randn(M, Kd, generator=g).bfloat16().cuda()
    w = (torch.randn(N, Kd, generator=g) * 0.02).bfloat16().cuda()
    xq, xs = K.quantize_fp8_rowwise(x)
    wq, ws = K.quantize_fp8_blockwise(w)
    out = K.fp8_matmul_dsv3(xq, wq.t(), xs, ws.t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    rows = torch.tensor([0, 1, 127, 128, 5000, 8191, 12345, 16383])
    ref = O.fp8_matmul_f64(xq[rows.cuda()].view(torch.uint8).cpu(), wq.view(torch.uint8).cpu().t(),
                           xs[rows.cuda()].cpu(), ws.cpu().t())
    err = rel_fro(out[rows.cuda()], ref)
    print(f"C2 forward sampled rows: rel-Fro {err:.3e}")
    assert err <= TOL and err <= 2e-5
    # linearity in the activation scales: doubling sA doubles the result exactly
    out2 = K.fp8_matmul_dsv3(xq, wq.t(), xs * 2, ws.t(), out_dtype=torch.float32)
    assert torch.equal(out2, out * 2)


@pytest.mark.parametrize("k_in,n_out", [(7168, 1536), (7168, 576), (1536, 24576), (512, 16384)])
def test_mla_projection_shapes_sampled(K, k_in, n_out):
    """Tall-skinny / small-N / small-K GEMMs of the MLA projections at 16384 tokens (quantised on the GPU,
    float64 check on sampled rows)."""
    Mt = 16384
    g = torch.Generator().manual_seed(1003 + n_out)
    x = torch.randn(Mt, k_in, generator=g).bfloat16().cuda()
    w = (torch.randn(n_out, k_in, generator=g) * 0.02).bfloat16().cuda()
    xq, xs = K.quantize_fp8_rowwise(x)
    wq, ws = K.quantize_fp8_blockwise(w)
    out = K.fp8_matmul_dsv3(xq, wq.t(), xs, ws.t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    rows = torch.tensor([0, 127, 128, 4097, 9999, 16383])
    ref = O.fp8_matmul_f64(xq[rows.cuda()].view(torch.uint8).cpu(), wq.view(torch.uint8).cpu().t(),
                           xs[rows.cuda()].cpu(), ws.cpu().t())
    err = rel_fro(out[rows.cuda()], ref)
    print(f"MLA {k_in}->{n_out}: rel-Fro {err:.3e}")
    assert err <= TOL and err <= 2e-5
    out16 = K.fp8_matmul_dsv3(xq, wq.t(), xs, ws.t())
    assert_bf16_close(out16[rows.cuda()], ref, "bf16 output")


@pytest.mark.parametrize("name", ["ragged", "empty_first_last", "wide_k"])
def test_grouped_gemm_backward(K, name):
    """moe_grouped_gemm is differentiable here (it is not in the reference): grouped dgrad in one launch,
    weight gradient per expert, both with the arithmetic of the dense backward."""
    E, d_in, d_out, counts = GROUPED[name]
    x, w, starts, ends = _grouped_case(E, d_in, d_out, counts, seed=40 + len(name))
    g = torch.Generator().manual_seed(41)
    dy = torch.randn(x.shape[0], d_out, generator=g).bfloat16()
    ref_dx, ref_dw = O.grouped_gemm_fp8_backward_f64(x, w, starts, ends, dy)
    xg = x.cuda().requires_grad_(True)
    wg = w.float().cuda().requires_grad_(True)
    out = K.moe_grouped_gemm(xg, wg, starts.cuda(), ends.cuda(), dtype=torch.bfloat16)
    out.backward(dy.cuda())
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert xg.grad.dtype == torch.bfloat16 and wg.grad.dtype == torch.float32
    assert_bf16_close(xg.grad, ref_dx, "grouped dgrad")
    assert_bf16_close(wg.grad.to(torch.bfloat16), ref_dw, "grouped wgrad")
    for e, c in enumerate(counts):
        if c == 0:
            assert torch.all(wg.grad[e] == 0)


def test_config2_backward_full_size_sampled(K):
    """Forward + backward of FP8MatmulFunction at the FFN width (x [16384, 7168], W [18432, 7168], dy [16384, 18432]),
    i.e. the step the benchmark times, with the fused quantiser passes in the loop.  dgrad is checked on sampled token
    rows, wgrad on sampled weight rows (all 7168 columns each), both against the float64 product of operands the CPU
    oracle quantised (src/kernels.py:763-794: dy row-wise, dy^T row-wise, x row-wise then re-quantised in blocks)."""
    M, Kd, N = 16384, 7168, 18432
    g = torch.Generator().manual_seed(1002)
    x = torch.randn(M, Kd, generator=g).bfloat16()
    w = torch.randn(N, Kd, generator=g) * 0.02
    dy = torch.randn(M, N, generator=g).bfloat16()
    xg = x.cuda().requires_grad_(True)
    wg = w.cuda().requires_grad_(True)
    out = K.FP8MatmulFunction.apply(xg, wg, False)
    out.backward(dy.cuda())
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert xg.grad.shape == (M, Kd) and wg.grad.shape == (N, Kd) and wg.grad.dtype == torch.float32
    wq, ws = O.quantize_blockwise(w, 128, 128)
    # dgrad: sampled token rows
    rows = torch.tensor([0, 1, 127, 128, 4097, 8191, 12345, 16383])
    dq, ds = O.quantize_rowwise(dy[rows], 128)
    ref_dx = O.fp8_matmul_f64(dq, wq, ds, ws)
    assert_bf16_close(xg.grad[rows.cuda()], ref_dx, "C2 dgrad")
    err_dx = rel_fro(xg.grad[rows.cuda()].float(), ref_dx)
    # wgrad: sampled weight rows; the reduction runs over all 16384 tokens
    nrows = torch.tensor([0, 127, 128, 255, 9000, 18431])
    dtq, dts = O.quantize_rowwise(dy[:, nrows].t().contiguous(), 128)
    xq, xs = O.quantize_rowwise(x, 128)
    xbq, xbs = O.requantize_row_to_block(xq, xs)
    ref_dw = O.fp8_matmul_f64(dtq, xbq, dts, xbs)
    assert_bf16_close(wg.grad[nrows.cuda()].to(torch.bfloat16), ref_dw, "C2 wgrad")
    err_dw = rel_fro(wg.grad[nrows.cuda()], ref_dw)
    # forward once more on sampled rows (bf16 result of the autograd path)
    ref_out = O.fp8_matmul_f64(xq[rows], wq.t(), xs[rows], ws.t())
    assert_bf16_close(out[rows.cuda()], ref_out, "C2 forward")
    print(f"C2 backward sampled: dgrad rel-Fro {err_dx:.3e}, wgrad rel-Fro {err_dw:.3e} (bf16 results)")
    assert err_dx < 4e-3 and err_dw < 4e-3          # bf16 rounding alone is 1.7e-3


def test_config4_grouped_gemm_literal_routing_sampled(K):
    """Grouped GEMMs of the MoE configuration at full size: 256 experts, 32768 tokens, top-8 (262144 rows), d = 7168,
    up-projection 7168 -> 4096 and down-projection 2048 -> 7168, with the row ranges that the literal routing
    specification produces (sigmoid scores + bias ~ N(0, 1): about 30 experts receive rows, several receive every
    token).  Gaps of a few rows that belong to no expert are inserted between some experts and a canary is written
    everywhere first.  Sampled rows - the first and last row of several experts among them - are checked against
    the float64 product."""
    from cinnamon_b200 import moe
    E, d, I, T, k = 256, 7168, 2048, 32768, 8
    g = torch.Generator(device="cuda").manual_seed(1004)
    xt = torch.randn(T, d, generator=g, device="cuda").bfloat16()
    router = torch.randn(E, d, generator=g, device="cuda") * 0.02
    bias = torch.randn(E, generator=g, device="cuda")
    r = moe.route(xt, router, bias, k)
    counts = r.counts.cpu()
    active = [e for e in range(E) if counts[e] > 0]
    assert int(counts.sum()) == T * k and len(active) < 64 and int(counts.max()) > 0.9 * T, "the literal routing is heavily skewed"
    # ranges with a 5-row gap in front of every third active expert
    starts, ends, pos = torch.zeros(E, dtype=torch.int64), torch.zeros(E, dtype=torch.int64), 0
    for e in range(E):
        if counts[e] > 0 and active.index(e) % 3 == 1:
            pos += 5
        starts[e], ends[e] = pos, pos + int(counts[e])
        pos = int(ends[e])
    R = pos + 9
    src = torch.zeros(R, dtype=torch.int64)
    for e in active:
        seg = r.token_indices[int(counts[:e].sum()):int(counts[:e + 1].sum())].cpu()
        src[int(starts[e]):int(ends[e])] = seg
    xq_t, xs_t = K.quantize_fp8_rowwise(xt)
    xq, xs = K.gather_quantized_rows(xq_t, xs_t, src.cuda())
    del xt, xq_t, xs_t
    covered = torch.zeros(R, dtype=torch.bool)
    for e in active:
        covered[int(starts[e]):int(ends[e])] = True
    sample = []
    for e in active[:4] + active[-3:] + [int(counts.argmax())]:
        s, t = int(starts[e]), int(ends[e])
        sample += [(e, s), (e, t - 1), (e, s + (t - s) // 2)]
        if t - s > 300:
            sample += [(e, s + 127), (e, s + 128), (e, t - 129)]
    rows = torch.tensor([p for _, p in sample])
    for name, d_in, d_out in (("up", d, 2 * I), ("down", I, d)):
        gw = torch.Generator(device="cuda").manual_seed(2004 + d_in)
        wq = torch.empty(E, d_out, d_in, dtype=torch.float8_e4m3fn, device="cuda")
        wsc = torch.empty(E, d_out // 128, d_in // 128, device="cuda")
        for e0 in range(0, E, 32):                                   # 32 experts at a time: the bf16 masters are large
            wpart = (torch.randn(32, d_out, d_in, generator=gw, device="cuda") * 0.02).bfloat16()
            wq[e0:e0 + 32], wsc[e0:e0 + 32] = K.quantize_expert_weights(wpart)
        del wpart
        if name == "up":
            aq, asc = xq, xs
        else:
            h = torch.randn(R, I, generator=gw, device="cuda").bfloat16()
            aq, asc = K.quantize_fp8_rowwise(h)
            del h
        out = torch.full((R, d_out), 777.0, dtype=torch.bfloat16, device="cuda")
        K.fp8_grouped_gemm(aq, asc, wq, wsc, starts.cuda(), ends.cuda(), out=out)
        torch.cuda.synchronize()
        assert K.device_status() == 0
        untouched = (out[(~covered).cuda()] == 777.0).all()
        assert bool(untouched), f"{name}: rows that belong to no expert were written"
        got = out[rows.cuda()].float().cpu()
        worst = 0.0
        for i, (e, p) in enumerate(sample):
            ref = O.fp8_matmul_f64(aq[p:p + 1].view(torch.uint8).cpu(), wq[e].view(torch.uint8).cpu().t(),
                                   asc[p:p + 1].cpu(), wsc[e].cpu().t())
            assert_bf16_close(got[i:i + 1].to(torch.bfloat16), ref, f"{name} row {p} of expert {e}")
            worst = max(worst, rel_fro(got[i:i + 1], ref))
        print(f"C4 {name}-projection, {len(active)} active experts, {len(sample)} sampled rows: worst rel-Fro {worst:.3e} (bf16)")
        del wq, wsc, out


FUSED_WGRAD = {
    "ragged": (6, 512, 256, [5, 0, 130, 1, 257, 64]),
    "one_owns_all": (4, 256, 512, [0, 0, 700, 0]),
    "empty_first_last": (5, 256, 256, [0, 128, 0, 129, 0]),
    "many_small": (16, 256, 256, [1, 2, 3, 127, 128, 129, 0, 0, 255, 256, 257, 16, 17, 15, 64, 1]),
}


@pytest.mark.parametrize("name", list(FUSED_WGRAD))
def test_grouped_weight_gradient_in_one_gemm(K, name):
    """cinn_fp8_grouped_wgrad_fused (segments padded to tiles on the device, two quantiser launches, one grouped-K
    GEMM, no host read-back) against the float64 oracle and against the per-expert loop, whose bytes and sums it
    must reproduce exactly; a gap of rows that belong to no expert and canary values in dW."""
    E, d_in, d_out, counts = FUSED_WGRAD[name]
    x, w, starts, ends = _grouped_case(E, d_in, d_out, counts, seed=60 + len(name), gap=7)
    g = torch.Generator().manual_seed(61)
    dy = torch.randn(x.shape[0], d_out, generator=g).bfloat16()
    _, ref_dw = O.grouped_gemm_fp8_backward_f64(x, w, starts, ends, dy)
    xq, xs = K.quantize_fp8_rowwise(x.cuda())
    args = (dy.cuda(), xq, xs, starts.cuda(), ends.cuda(), E, d_in, d_out)
    fused = K.fp8_grouped_wgrad(*args, w_dtype=torch.float32, fused=True)
    loop = K.fp8_grouped_wgrad(*args, w_dtype=torch.float32, fused=False)
    torch.cuda.synchronize()
    assert K.device_status() == 0
    assert torch.equal(fused, loop), float((fused - loop).abs().max())
    assert_bf16_close(fused.to(torch.bfloat16), ref_dw, "grouped wgrad, one GEMM")
    for e, c in enumerate(counts):
        if c == 0:
            assert torch.all(fused[e] == 0)
    assert torch.equal(K.fp8_grouped_wgrad(*args, w_dtype=torch.bfloat16, fused=True), fused.to(torch.bfloat16))
    # the same call that also hands back the row-wise quantisation of dY (one pass over dY for both): same dW bits,
    # and inside the expert ranges the bytes and scales of the row-wise quantiser
    both, gq, gs = K.fp8_grouped_wgrad(*args, w_dtype=torch.float32, fused=True, with_row_quant=True)
    wq, ws = K.quantize_fp8_rowwise(dy.cuda())
    assert torch.equal(both, fused)
    inside = torch.zeros(x.shape[0], dtype=torch.bool)
    for a, b in zip(starts.tolist(), ends.tolist()):
        inside[a:b] = True
    assert inside.any() and not inside.all()
    ins = inside.numpy()
    assert np.array_equal(bytes_of(gq)[ins], bytes_of(wq)[ins]) and np.array_equal(bits_of(gs)[ins], bits_of(ws)[ins])
    for dt in (torch.float16, torch.float32):                     # fp32 gradients take the two-pass route
        both, gq, gs = K.fp8_grouped_wgrad(dy.cuda().to(dt), *args[1:], w_dtype=torch.float32, fused=True, with_row_quant=True)
        wq, ws = K.quantize_fp8_rowwise(dy.cuda().to(dt))
        assert torch.equal(both, fused)
        assert np.array_equal(bytes_of(gq)[ins], bytes_of(wq)[ins]) and np.array_equal(bits_of(gs)[ins], bits_of(ws)[ins])


def test_zero_rows_outside_ranges(K):
    """cinn_zero_rows_outside clears exactly the rows that no range covers (gaps, empty / reversed / overlapping /
    out-of-bounds ranges, a row size that is not a multiple of 16), and the grouped input gradient built on it
    gives zero rows where no expert has rows."""
    import ctypes
    from cinnamon_b200 import _lib
    dev = torch.device("cuda")
    for T, row_bytes in ((1000, 256), (517, 36), (128, 16)):
        buf = torch.full((T, row_bytes), 7, dtype=torch.uint8, device=dev)
        starts = torch.tensor([-5, 40, 300, 290, 700, 650, 990], dtype=torch.int64, device=dev)
        ends = torch.tensor([10, 40, 420, 310, 650, 660, 5000], dtype=torch.int64, device=dev)
        _lib.check(_lib.lib.cinn_zero_rows_outside(ctypes.c_void_p(buf.data_ptr()), T, row_bytes, ctypes.c_void_p(starts.data_ptr()),
                                                   ctypes.c_void_p(ends.data_ptr()), starts.numel(), None), "zero")
        covered = torch.zeros(T, dtype=torch.bool)
        for s, e in zip(starts.tolist(), ends.tolist()):
            covered[max(s, 0):max(min(e, T), 0)] = True
        want = torch.where(covered[:, None], torch.tensor(7, dtype=torch.uint8), torch.tensor(0, dtype=torch.uint8)).expand(T, row_bytes)
        assert torch.equal(buf.cpu(), want)
    g = torch.Generator(device=dev).manual_seed(5)
    E, d_in, d_out, T = 3, 256, 384, 700
    dy = torch.randn(T, d_out, generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn(E, d_out, d_in, generator=g, device=dev) * 0.05).to(torch.bfloat16)
    dq, dsc = K.quantize_fp8_rowwise(dy)
    wq, wsc = K.quantize_expert_weights(w)
    starts = torch.tensor([10, 300, 300], dtype=torch.int64, device=dev)
    ends = torch.tensor([200, 300, 650], dtype=torch.int64, device=dev)
    dx = K.fp8_grouped_gemm_dgrad(dq, dsc, wq, wsc, starts, ends)
    assert torch.count_nonzero(dx[:10]) == 0 and torch.count_nonzero(dx[200:300]) == 0 and torch.count_nonzero(dx[650:]) == 0
    assert torch.count_nonzero(dx[10:200]) > 0 and torch.isfinite(dx.float()).all()
