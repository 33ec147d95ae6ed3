"""GPU: the reference's OWN nonlinear operators (the unmodified Triton kernels of Jetfire/Nonlinear/*.py, compiled for this GPU
by the installed Triton) against this package's CUDA operators on the same device tensors.

What this adds to the golden fixtures (the same kernels under the Triton interpreter, 128 x 256 inputs): the comparison runs at a
size where this package's kernels loop over several tiles per warp, and the stochastic operators run in the reference's own
noise mode -- `Nonlinear.set_sr_noise("torch")` draws `uniform_(-0.5, 0.5)` from torch's generator exactly as the reference
does, so after the same `torch.manual_seed` both sides must round identically without any noise tensor being handed over.

Expected agreement.  The COMPILED reference is not bit-identical to the INTERPRETED reference that generated the golden fixtures
(and that this package matches bit for bit): compiled Triton lowers the fp32 `/` of the scale computation `absmax / 127.` to the
approximate `div.full.f32` (only `tl.div_rn` is IEEE), contracts multiply-add pairs into fma, and uses libdevice's erf / exp.  A
scale that comes out one fp32 ulp different moves a payload by one step where the quotient sits on a rounding boundary.  So every
comparison here is "payloads within one step on at most a stated small fraction of elements, fp16 scales within one ulp", with
the measured fractions printed; the bounds in the asserts are a few times the measured values.  Pure data movement (transpose,
and dequantize, whose product is a single fp16 multiplication) is bit for bit.

The autotuner of every reference kernel is cut to its first configuration (tile shape and stage count do not change results)
to keep compilation short.  Skipped when the reference files are not reachable (tests/stage_reference.py stages them).
"""
import pytest
import torch

from gpu_util import DEV, outlier_randn

pytestmark = pytest.mark.gpu

M, N = 2048, 3072          # 6144 quantisation blocks: several tiles per warp in every kernel of this package
BOUND = 1e-3               # largest tolerated fraction of payloads one step apart (measured: at most 1.9e-4; printed)


@pytest.fixture(scope="module")
def R():
    from oracle import build_ref
    try:
        mod = build_ref.load_nonlinear(first_config_only=True)
    except ImportError as e:                          # no Triton in the environment
        pytest.skip(f"the reference's Triton operators cannot be imported: {e}")
    if mod is None:
        pytest.skip("reference files not reachable (python tests/stage_reference.py with a reference checkout)")
    try:                                              # can the installed Triton compile and launch them here at all?
        mod.int8_quantize(torch.zeros(32, 32, device=DEV), 32)
        torch.cuda.synchronize()
    except Exception as e:
        pytest.skip(f"the reference's Triton kernels do not run in this environment: {type(e).__name__}: {str(e)[:200]}")
    return mod


@pytest.fixture()
def torch_noise(NL):
    prev = NL.set_sr_noise("torch")
    yield
    NL.set_sr_noise(prev)


def _cmp(tag, got, ref, max_step=0, max_frac=0.0):
    """int8 payloads: fraction that differs and by how much."""
    d = (got.to(torch.int32) - ref.to(torch.int32)).abs()
    frac = float((d != 0).float().mean())
    print(f"{tag}: {frac:.2e} of payloads differ (max {int(d.max())} step)")
    assert int(d.max()) <= max_step and frac <= max_frac, tag


def _cmp_scale(tag, got, ref, max_ulp=0):
    d = (got.view(torch.int16).to(torch.int32) - ref.view(torch.int16).to(torch.int32)).abs()
    print(f"{tag}: scales differ by at most {int(d.max())} fp16 ulp ({float((d != 0).float().mean()):.2e} of them)")
    assert int(d.max()) <= max_ulp, tag


def _x(seed, scale=1.0):
    return (scale * outlier_randn(torch.Generator().manual_seed(seed), M, N)).to(DEV)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_quantize_transpose_dequantize(R, NL, dt):
    x = _x(1).to(dt)
    q, s = NL.int8_quantize(x, 32)
    qr, sr = R.int8_quantize(x, 32)
    _cmp(f"quantize {dt}", q, qr, 1, BOUND); _cmp_scale(f"quantize {dt}", s, sr, 1)
    q2, s2, qt = NL.int8_quantize_transpose(x, 32)
    qr2, sr2, qtr = R.int8_quantize_transpose(x, 32)
    _cmp(f"quantize_transpose {dt}", q2, qr2, 1, BOUND); _cmp(f"quantize_transpose {dt} (transposed copy)", qt, qtr, 1, BOUND)
    _cmp_scale(f"quantize_transpose {dt}", s2, sr2, 1)
    assert torch.equal(NL.int8_transpose(qr), R.int8_transpose(qr))
    assert torch.equal(NL.int8_dequantize(qr, sr, 32), R.int8_dequantize(qr, sr, 32).float())


def test_quantize_sr_same_seed_same_rounding(R, NL, torch_noise):
    x = _x(2).to(torch.bfloat16)
    torch.manual_seed(1234)
    q, s = NL.int8_quantize(x, 32, stochastic=True)
    torch.manual_seed(1234)
    qr, sr = R.int8_quantize(x, 32, stochastic=True)
    _cmp("quantize_sr", q, qr, 1, BOUND); _cmp_scale("quantize_sr", s, sr, 1)
    torch.manual_seed(1234)
    q2, s2, qt = NL.int8_quantize_transpose(x, 32, stochastic=True)
    torch.manual_seed(1234)
    qr2, sr2, qtr = R.int8_quantize_transpose(x, 32, stochastic=True)
    _cmp("quantize_transpose_sr", q2, qr2, 1, BOUND); _cmp("quantize_transpose_sr (transposed copy)", qt, qtr, 1, BOUND)
    torch.manual_seed(99)                     # a different seed rounds differently: about half of the payloads sit between two steps
    q3, _ = NL.int8_quantize(x, 32, stochastic=True)
    other = float((q3 != q).float().mean())
    print(f"quantize_sr: another seed changes {other:.3f} of the payloads")
    assert other > 0.2


def test_gelu_forward_and_backward(R, NL, torch_noise):
    qx, sx = NL.int8_quantize(_x(3), 32)
    qg, sg = NL.int8_quantize(_x(4, 1e-2), 32)
    qy, sy = NL.int8_gelu_forward(qx, sx, 32)
    qyr, syr = R.int8_gelu_forward(qx, sx, 32)
    _cmp("gelu_fwd", qy, qyr, 1, BOUND); _cmp_scale("gelu_fwd", sy, syr, 1)
    qd, sd = NL.int8_gelu_backward(qx, sx, qg, sg, 32, stochastic=False)
    qdr, sdr = R.int8_gelu_backward(qx, sx, qg, sg, 32, stochastic=False)
    _cmp("gelu_bwd", qd, qdr, 1, BOUND); _cmp_scale("gelu_bwd", sd, sdr, 1)
    torch.manual_seed(7)
    qd, sd = NL.int8_gelu_backward(qx, sx, qg, sg, 32, stochastic=True)
    torch.manual_seed(7)
    qdr, sdr = R.int8_gelu_backward(qx, sx, qg, sg, 32, stochastic=True)
    _cmp("gelu_bwd_sr", qd, qdr, 1, BOUND); _cmp_scale("gelu_bwd_sr", sd, sdr, 1)


def test_layernorm_forward_and_backward(R, NL, torch_noise):
    x = _x(5)
    qx, sx = NL.int8_quantize(x, 32)
    xd = NL.int8_dequantize(qx, sx, 32)
    mean = xd.mean(-1)
    rstd = 1.0 / xd.var(-1, unbiased=False).sqrt()
    gamma = (1.0 + 0.1 * torch.randn(N, generator=torch.Generator().manual_seed(6))).to(DEV)
    qy, sy, _ = NL.int8_layernorm_forward(qx, sx, gamma, mean, rstd, 32)
    qyr, syr, _ = R.int8_layernorm_forward(qx, sx, gamma, mean, rstd, 32)
    _cmp("ln_fwd", qy, qyr, 1, BOUND); _cmp_scale("ln_fwd", sy, syr, 1)
    qg, sg = NL.int8_quantize(_x(7, 1e-2), 32)
    for stochastic in (False, True):
        torch.manual_seed(11)
        qd, sd, dw = NL.int8_layernorm_backward(qx, sx, qg, sg, gamma, 32, mean, rstd, stochastic=stochastic)
        torch.manual_seed(11)
        qdr, sdr, dwr = R.int8_layernorm_backward(qx, sx, qg, sg, gamma, 32, mean, rstd, stochastic=stochastic)
        tag = "ln_bwd_sr" if stochastic else "ln_bwd"
        # the row sums c1, c2 are reduced in a device-specific order on both sides
        _cmp(tag, qd, qdr, 1, BOUND); _cmp_scale(tag, sd, sdr, 1)
        rel = float((dw.float() - dwr.float()).abs().max() / dwr.float().abs().max())
        print(f"{tag}: d_gamma max deviation {rel:.2e} of max |d_gamma|")
        assert rel < 5e-3


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_residual_add(R, NL, torch_noise, dt):
    x1 = _x(8).to(dt)
    q2, s2 = NL.int8_quantize(_x(9), 32)
    y1, qy, sy = NL.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, 32)
    y1r, qyr, syr = R.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, 32)
    assert torch.equal(y1, y1r.float())
    _cmp(f"add {dt}", qy, qyr, 1, BOUND); _cmp_scale(f"add {dt}", sy, syr, 1)
    torch.manual_seed(21)
    y1, qy, sy = NL.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, 32, stochastic=True)
    torch.manual_seed(21)
    y1r, qyr, syr = R.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, 32, stochastic=True)
    assert torch.equal(y1, y1r.float())
    _cmp(f"add_sr {dt}", qy, qyr, 1, BOUND); _cmp_scale(f"add_sr {dt}", sy, syr, 1)
    y1, qy, sy, mean, rstd = NL.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, q2, s2, 32)
    y1r, qyr, syr, meanr, rstdr = R.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, q2, s2, 32)
    assert torch.equal(y1, y1r.float())
    _cmp(f"add_meanvar {dt}", qy, qyr, 1, BOUND); _cmp_scale(f"add_meanvar {dt}", sy, syr, 1)
    torch.testing.assert_close(mean.float().reshape(-1), meanr.float().reshape(-1), rtol=1e-3, atol=1e-5)
    torch.testing.assert_close(rstd.float().reshape(-1), rstdr.float().reshape(-1), rtol=1e-3, atol=1e-5)
