"""GPU: the reference's OWN GEMM kernels (its BlockQuantizeCUDA extension, rebuilt for sm_100 by oracle/build_ref.py from the
reference checkout) against the CPU oracle -- the one pin of the GEMM oracle's fp32 accumulation and re-quantising epilogue
that comes from the reference itself -- and against this package's kernels on the same operands.

The reference builds with -use_fast_math (approximate division in the epilogue) and draws its stochastic-rounding noise from
curand seeded by libc rand(), so these comparisons are tolerance-level by nature; what is asserted is what the reference's own
test scripts assert (JetfireGEMMKernel/tests/test_int8igemmoutputIntQuantizeBiasRowCol.py:49-54: allclose(rtol 1e-1, atol 5)
on dequantised values) plus the measured payload agreement.  Shapes are the reference's own (M, N multiples of 128).
Skipped when oracle/_ref/BlockQuantizeCUDA.so has not been built.
"""
import numpy as np
import pytest
import torch

from gpu_util import DEV, n, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ext():
    from oracle import build_ref
    mod = build_ref.load()
    if mod is None:
        pytest.skip("oracle/_ref/BlockQuantizeCUDA.so not built (python oracle/build_ref.py with a reference checkout)")
    return mod


def _operands(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = rng.integers(-127, 128, (M, K), dtype=np.int8)
    b = rng.integers(-127, 128, (N, K), dtype=np.int8)
    sa = rng.uniform(1e-3, 1e-1, (M // 32, K // 32)).astype(np.float16)
    sb = rng.uniform(1e-3, 1e-1, (N // 32, K // 32)).astype(np.float16)
    return a, b, sa, sb


def _deq(q, s):
    return q.astype(np.float32).reshape(q.shape[0] // 32, 32, q.shape[1] // 32, 32) * s.astype(np.float32)[:, None, :, None]


@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (512, 512, 512), (1024, 2048, 512)])
def test_reference_forward_kernel_agrees_with_the_oracle(ref_ext, oracle, M, N, K):
    a, b, sa, sb = _operands(M, N, K, M + K)
    A, B = t(a), t(b)
    SAt, SBt = t(sa).t().contiguous(), t(sb).t().contiguous()
    bias = torch.zeros(N, device=DEV); biasmax = torch.zeros(1, device=DEV)
    o, so = ref_ext.igemm_output_int_quantize_bias_rowcol(A, B.t(), bias, biasmax, SAt, SBt, M, N, K)
    torch.cuda.synchronize()
    qo, sco = oracle.linear_forward(a, sa, b, sb)
    d = np.abs(n(o).astype(np.int32) - qo.astype(np.int32))
    frac = np.count_nonzero(d) / d.size
    sdiff = np.abs(n(so).view(np.int16).astype(np.int32) - sco.view(np.int16).astype(np.int32)).max()
    print(f"reference fwd kernel vs oracle [{M}x{N}x{K}]: {frac:.2e} of payloads differ (max {d.max()} step), scales max {sdiff} ulp")
    assert d.max() <= 1 and frac <= 2e-3 and sdiff <= 1        # fast-math division: rounding ties only
    np.testing.assert_allclose(_deq(n(o), n(so)), _deq(qo, sco), rtol=1e-1, atol=5)   # the reference's own bar
    # this package's kernel on the same operands is bit-identical to the oracle
    from jetfire_int8training_b200 import Linear
    y8, sy = Linear.int8_linear_forward(A, t(sa), B, t(sb), True, 32)
    assert np.array_equal(n(y8), qo) and np.array_equal(n(sy).view(np.uint16), sco.view(np.uint16))


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (1024, 2048, 512)])
def test_reference_wgrad_and_dgrad_kernels_agree_with_the_oracle(ref_ext, oracle, M, N, K):
    """igemm_output_fp_no_quantize (A [M,K] row-major, B [K,N] row-major -> fp16) and igemm_output_int_quantize_stochastic."""
    a, b, sa, sb = _operands(M, N, K, 7 * M + K)
    bt = np.ascontiguousarray(b.T)                                   # [K, N]
    A, Bt = t(a), t(bt)
    SAt, SBt = t(sa).t().contiguous(), t(sb).t().contiguous()
    o = ref_ext.igemm_output_fp_no_quantize(A, Bt, SAt, SBt, M, N, K)
    torch.cuda.synchronize()
    acc = oracle.gemm_accumulate(a, b, sa, sb)
    want = acc.astype(np.float16)
    ulp = np.abs(n(o).view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
    print(f"reference wgrad-style kernel vs oracle [{M}x{N}x{K}]: {np.count_nonzero(ulp) / ulp.size:.2e} of fp16 outputs differ, max {ulp.max()} ulp")
    # same sequential fp32 FMA chain, no division in this epilogue: identical up to the compiler's freedom under fast-math
    assert ulp.max() <= 1 and np.count_nonzero(ulp) <= 1e-3 * ulp.size
    # stochastic kernel: its noise stream is curand's, so payloads are compared with the round-to-nearest oracle: the same
    # scales, every payload within one step (stochastic rounding picks floor or ceil), and the mean signed deviation of the
    # payloads close to zero (unbiased)
    q, s = ref_ext.igemm_output_int_quantize_stochastic(A, Bt, SAt, SBt, M, N, K)
    torch.cuda.synchronize()
    qo, sco = oracle.requant(acc)
    sdiff = np.abs(n(s).view(np.int16).astype(np.int32) - sco.view(np.int16).astype(np.int32)).max()
    dev = n(q).astype(np.int32) - qo.astype(np.int32)
    print(f"reference dgrad kernel vs round-to-nearest oracle: payload max {np.abs(dev).max()} step (stochastic), "
          f"mean deviation {dev.mean():+.2e}, scales max {sdiff} ulp")
    assert sdiff <= 1 and np.abs(dev).max() <= 1 and abs(dev.mean()) < 5e-3
