"""GPU parity of the nonlinear operators: CUDA kernels (through the ctypes C ABI) against
  (1) the golden vectors produced by the reference's own Triton kernels, and
  (2) the CPU oracle on seeded inputs at further shapes (ragged N, 3-D, larger).
Rules: integer payloads and scales bit-exact wherever every rounding point is defined by the reference (quantize,
transpose, dequantize, LayerNorm forward, residual add); where the reference leaves a last-ulp freedom (libdevice
erf/exp in GELU, tree-order row sums in LayerNorm backward and in the row statistics) payloads may differ by one step on
a stated small fraction of elements and floating-point outputs must agree to rel-err <= 1e-3."""
import numpy as np
import pytest
import torch

from conftest import load_golden, to_np
from gpu_util import DEV, assert_bits_equal, assert_payload_close, assert_scales_close, n, outlier_randn, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def NL():
    from jetfire_int8training_b200 import Nonlinear
    return Nonlinear


# ------------------------------------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("tag,dt", [("f32", torch.float32), ("f16", torch.float16), ("bf16", torch.bfloat16)])
def test_quantize_golden(NL, tag, dt):
    d = load_golden("quantize_" + tag)
    x = t(d["x"], dt)
    q, s = NL.int8_quantize(x, 32)
    assert_bits_equal(n(q), d["q"], "q"); assert_bits_equal(n(s), d["s"], "s")
    d = load_golden("quantize_transpose_" + tag)
    q, s, qt = NL.int8_quantize_transpose(t(d["x"], dt), 32)
    assert_bits_equal(n(q), d["q"], "q"); assert_bits_equal(n(s), d["s"], "s"); assert_bits_equal(n(qt), d["qt"], "qt")


def test_quantize_sr_golden_with_reference_noise(NL):
    d = load_golden("quantize_sr_bf16")
    q, s = NL.int8_quantize(t(d["x"]), 32, stochastic=True, noise=t(d["noise"]))
    assert_bits_equal(n(q), d["q"], "q"); assert_bits_equal(n(s), d["s"], "s")


def test_quantize_3d_golden(NL):
    d = load_golden("quantize_3d_f32")
    q, s = NL.int8_quantize(t(d["x"]), 32)
    assert q.shape == (2, 64, 128) and s.shape == (2, 2, 4)
    assert_bits_equal(n(q), d["q"], "q"); assert_bits_equal(n(s), d["s"], "s")


def test_transpose_dequantize_golden(NL):
    d = load_golden("transpose")
    assert_bits_equal(n(NL.int8_transpose(t(d["x"]))), d["y"], "transpose")
    d = load_golden("dequantize")
    assert_bits_equal(n(NL.int8_dequantize(t(d["q"]), t(d["s"]), 32)), d["y"], "dequantize")


def test_gelu_golden(NL):
    d = load_golden("gelu_fwd")
    q, s = NL.int8_gelu_forward(t(d["qx"]), t(d["sx"]), 32)
    assert_payload_close(n(q), d["qy"], 2e-3, "gelu_fwd"); assert_scales_close(n(s), d["sy"], 1, "gelu_fwd")
    d = load_golden("gelu_bwd")
    q, s = NL.int8_gelu_backward(t(d["qx"]), t(d["sx"]), t(d["qg"]), t(d["sg"]), 32)
    assert_payload_close(n(q), d["qd"], 2e-3, "gelu_bwd"); assert_scales_close(n(s), d["sd"], 1, "gelu_bwd")
    d = load_golden("gelu_bwd_sr")
    q, s = NL.int8_gelu_backward(t(d["qx"]), t(d["sx"]), t(d["qg"]), t(d["sg"]), 32, stochastic=True, noise=t(d["noise"]))
    assert_payload_close(n(q), d["qd"], 2e-3, "gelu_bwd_sr"); assert_scales_close(n(s), d["sd"], 1, "gelu_bwd_sr")


def test_layernorm_golden(NL):
    d = load_golden("ln_fwd")
    q, s, _ = NL.int8_layernorm_forward(t(d["qx"]), t(d["sx"]), t(d["gamma"]), t(d["mean"]), t(d["rstd"]), 32)
    assert_bits_equal(n(q), d["qy"], "ln_fwd q"); assert_bits_equal(n(s), d["sy"], "ln_fwd s")
    for name in ("ln_bwd", "ln_bwd_sr"):
        d = load_golden(name)
        kw = dict(stochastic=True, noise=t(d["noise"])) if "noise" in d else {}
        q, s, dw = NL.int8_layernorm_backward(t(d["qx"]), t(d["sx"]), t(d["qg"]), t(d["sg"]), t(d["gamma"]), 32, t(d["mean"]),
                                              t(d["rstd"]), **kw)
        assert_payload_close(n(q), d["qd"], 1e-2, name); assert_scales_close(n(s), d["sd"], 1, name)
        # the reference sums each 32-row partial of dgamma in fp16; the kernel accumulates the same fp16 products in fp32
        assert np.abs(n(dw) - d["dw"]).max() <= 5e-3 * np.abs(d["dw"]).max()


@pytest.mark.parametrize("tag,dt", [("f32", torch.float32), ("bf16", torch.bfloat16)])
def test_add_golden(NL, tag, dt):
    d = load_golden("add_" + tag)
    y, q, s = NL.int8_add_Ifp_Ig16_Ofp_Og(t(d["x1"], dt), t(d["q2"]), t(d["s2"]), 32)
    assert_bits_equal(n(y), d["y1"], "y1"); assert_bits_equal(n(q), d["qy"], "q"); assert_bits_equal(n(s), d["sy"], "s")
    d = load_golden("add_sr_" + tag)
    y, q, s = NL.int8_add_Ifp_Ig16_Ofp_Og(t(d["x1"], dt), t(d["q2"]), t(d["s2"]), 32, stochastic=True, noise=t(d["noise"]))
    assert_bits_equal(n(y), d["y1"], "y1"); assert_bits_equal(n(q), d["qy"], "q"); assert_bits_equal(n(s), d["sy"], "s")
    d = load_golden("add_meanvar_" + tag)
    y, q, s, mean, rstd = NL.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(t(d["x1"], dt), t(d["q2"]), t(d["s2"]), 32)
    assert_bits_equal(n(y), d["y1"], "y1"); assert_bits_equal(n(q), d["qy"], "q"); assert_bits_equal(n(s), d["sy"], "s")
    np.testing.assert_allclose(n(mean), d["mean"], rtol=1e-3, atol=1e-6)   # tolerance: rel-err 1e-3
    np.testing.assert_allclose(n(rstd), d["rstd"], rtol=1e-3)


# ------------------------------------------------------------------------------------------------ oracle, more shapes
SHAPES = [(32, 32), (64, 160), (256, 768), (96, 3072), (1024, 2304)]


@pytest.mark.parametrize("M,N", SHAPES)
@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_quantize_vs_oracle(NL, oracle, M, N, dt):
    g = torch.Generator().manual_seed(M * 7 + N)
    x = outlier_randn(g, M, N).to(dt)
    if M >= 64:
        x[32:64, 0:32] = 0
    q, s, qt = NL.int8_quantize_transpose(x.to(DEV), 32)
    qo, so, qto = oracle.int8_quantize_transpose(x.float().numpy())
    assert_bits_equal(n(q), qo, "q"); assert_bits_equal(n(s), so, "s"); assert_bits_equal(n(qt), qto, "qt")
    q2, s2 = NL.int8_quantize(x.to(DEV), 32)
    assert_bits_equal(n(q2), qo, "q"); assert_bits_equal(n(s2), so, "s")
    assert_bits_equal(n(NL.int8_transpose(q2)), qto, "transpose")
    assert_bits_equal(n(NL.int8_dequantize(q2, s2, 32)), oracle.int8_dequantize(qo, so), "dequantize")


@pytest.mark.parametrize("M,N", [(64, 160), (256, 768)])
def test_quantize_philox_bit_exact_and_unbiased(NL, oracle, M, N):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, N, generator=g).to(torch.bfloat16)
    key = (0x1234567890ABCDEF, 42)
    q, s = NL.int8_quantize(x.to(DEV), 32, stochastic=True, sr_key=key)
    noise = oracle.sr_noise(M, N, *key)
    qo, so = oracle.int8_quantize(x.float().numpy(), noise)
    assert_bits_equal(n(q), qo, "q (fixed Philox key)"); assert_bits_equal(n(s), so, "s")
    # same key -> same bits; next offset -> different noise
    q_again, _ = NL.int8_quantize(x.to(DEV), 32, stochastic=True, sr_key=key)
    assert torch.equal(q, q_again)
    q_other, _ = NL.int8_quantize(x.to(DEV), 32, stochastic=True, sr_key=(key[0], 43))
    assert not torch.equal(q, q_other)
    # unbiasedness: mean of dequantised draws approaches x
    acc = torch.zeros(M, N, device=DEV)
    R = 200
    for r in range(R):
        qr, sr = NL.int8_quantize(x.to(DEV), 32, stochastic=True, sr_key=(99, r))
        acc += NL.int8_dequantize(qr, sr, 32)
    err = (acc / R - x.float().to(DEV)).abs().mean() / x.float().abs().mean()
    q0, s0 = NL.int8_quantize(x.to(DEV), 32)
    err_rn = (NL.int8_dequantize(q0, s0, 32) - x.float().to(DEV)).abs().mean() / x.float().abs().mean()
    assert float(err) < 0.25 * float(err_rn)


@pytest.mark.parametrize("M,N", [(64, 160), (256, 768), (512, 3072)])
def test_gelu_vs_oracle(NL, oracle, M, N):
    g = torch.Generator().manual_seed(N)
    qx, sx = oracle.int8_quantize(outlier_randn(g, M, N).numpy())
    qg, sg = oracle.int8_quantize((1e-2 * torch.randn(M, N, generator=g)).numpy())
    q, s = NL.int8_gelu_forward(t(qx), t(sx), 32)
    qo, so = oracle.int8_gelu_forward(qx, sx)
    assert_payload_close(n(q), qo, 2e-3, "gelu_fwd"); assert_scales_close(n(s), so, 1)
    key = (7, 11)
    q, s = NL.int8_gelu_backward(t(qx), t(sx), t(qg), t(sg), 32, stochastic=True, sr_key=key)
    qo, so = oracle.int8_gelu_backward(qx, sx, qg, sg, oracle.sr_noise(M, N, *key))
    assert_payload_close(n(q), qo, 2e-3, "gelu_bwd"); assert_scales_close(n(s), so, 1)


@pytest.mark.parametrize("M,N", [(64, 128), (256, 768), (128, 3072), (64, 160), (96, 1600)])
def test_layernorm_vs_oracle(NL, oracle, M, N):
    g = torch.Generator().manual_seed(N + 1)
    xf = outlier_randn(g, M, N)
    qx, sx = oracle.int8_quantize(xf.numpy())
    gamma = (1.0 + 0.1 * torch.randn(N, generator=g)).numpy()
    xd = oracle.int8_dequantize(qx, sx)
    mean = xd.mean(-1).astype(np.float32)
    rstd = (1.0 / np.sqrt(xd.var(-1) + 1e-5)).astype(np.float32)
    q, s, _ = NL.int8_layernorm_forward(t(qx), t(sx), t(gamma), t(mean), t(rstd), 32)
    qo, so = oracle.int8_layernorm_forward(qx, sx, gamma, mean, rstd)
    assert_bits_equal(n(q), qo, "ln_fwd q"); assert_bits_equal(n(s), so, "ln_fwd s")
    qg, sg = oracle.int8_quantize((1e-2 * torch.randn(M, N, generator=g)).numpy())
    key = (3, 5)
    qd, sd, dw = NL.int8_layernorm_backward(t(qx), t(sx), t(qg), t(sg), t(gamma), 32, t(mean), t(rstd), stochastic=True, sr_key=key)
    qo, so, dwo = oracle.int8_layernorm_backward(qx, sx, qg, sg, gamma, mean, rstd, oracle.sr_noise(M, N, *key), dw_accum="fp32")
    assert_payload_close(n(qd), qo, 1e-2, "ln_bwd"); assert_scales_close(n(sd), so, 1)
    assert np.abs(n(dw) - dwo).max() <= 1e-4 * np.abs(dwo).max() + 1e-7    # fp32 sums in a different order


@pytest.mark.parametrize("M,N", [(64, 160), (256, 768), (128, 3072)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_add_vs_oracle(NL, oracle, M, N, dt):
    g = torch.Generator().manual_seed(N + 2)
    x1 = outlier_randn(g, M, N).to(dt)
    q2, s2 = oracle.int8_quantize(torch.randn(M, N, generator=g).numpy())
    key = (21, 2)
    y, q, s = NL.int8_add_Ifp_Ig16_Ofp_Og(x1.to(DEV), t(q2), t(s2), 32, stochastic=True, sr_key=key)
    yo, qo, so = oracle.int8_add(x1.float().numpy(), q2, s2, oracle.sr_noise(M, N, *key))
    assert_bits_equal(n(y), yo, "y1"); assert_bits_equal(n(q), qo, "q"); assert_bits_equal(n(s), so, "s")
    y, q, s, mean, rstd = NL.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1.to(DEV), t(q2), t(s2), 32)
    yo, qo, so, mo, ro = oracle.int8_add_meanvar(x1.float().numpy(), q2, s2)
    assert_bits_equal(n(y), yo, "y1"); assert_bits_equal(n(q), qo, "q"); assert_bits_equal(n(s), so, "s")
    np.testing.assert_allclose(n(mean), mo, rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(n(rstd), ro, rtol=1e-3)


def test_3d_inputs_keep_the_batch_dimension(NL, oracle):
    g = torch.Generator().manual_seed(9)
    x = torch.randn(2, 64, 256, generator=g)
    q, s = NL.int8_quantize(x.to(DEV), 32)
    assert q.shape == (2, 64, 256) and s.shape == (2, 2, 8)
    y, sy = NL.int8_gelu_forward(q, s, 32)
    assert y.shape == q.shape and sy.shape == s.shape
    qt = NL.int8_transpose(q, transpose_output_2d=True)
    assert qt.shape == (256, 128)
    # the reference's callers pass int8 payloads viewed as float8_e4m3fn between autograd Functions
    y2, _ = NL.int8_gelu_forward(q.view(torch.float8_e4m3fn), s, 32)
    assert torch.equal(y, y2)


def test_full_size_properties(NL):
    """Size-independent properties at the benchmark's full sizes ([8192, 3072])."""
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(8192, 3072, generator=g, device=DEV, dtype=torch.bfloat16)
    q, s, qt = NL.int8_quantize_transpose(x, 32)
    # each block hits +-127 at its absmax; dequantisation error is bounded by half a step
    blk = q.view(256, 32, 96, 32).abs().amax((1, 3))
    assert int(blk.min()) == 127 and int(blk.max()) == 127
    deq = NL.int8_dequantize(q, s, 32)
    step = s.float().repeat_interleave(32, 0).repeat_interleave(32, 1)
    assert bool(((deq - x.float()).abs() <= 0.65 * step + 1e-6).all())
    # transpose twice is the identity; quantising the dequantised tensor is idempotent on the payload
    assert torch.equal(NL.int8_transpose(qt), q)
    q2, s2 = NL.int8_quantize(deq, 32)
    assert torch.equal(q2, q)


def test_errors(NL):
    with pytest.raises(RuntimeError):
        NL.int8_quantize(torch.randn(32, 32), 32)                       # CPU tensor: no fallback
    with pytest.raises(Exception):
        NL.int8_quantize(torch.randn(48, 32, device=DEV), 32)          # rows not a multiple of 32
    with pytest.raises(ValueError):
        NL.int8_quantize(torch.randn(32, 32, device=DEV), 16)          # only QB = 32
