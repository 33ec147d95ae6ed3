"""GPU parity of the per-block INT8 GEMMs (tcgen05 kernels, through the ctypes C ABI) against the CPU oracle.
Everything here is integer / exactly-specified fp32 work, so the bar is bit-exact: int32 block products, int8 payloads,
fp16 scales, fp16 dense outputs -- for round-to-nearest and, with a fixed Philox key, for stochastic rounding.
Every forward / backward / split-K case runs on BOTH GEMM paths: the int8-operand kernel (kind::i8 + conversion in the
consumers) and the fp16-operand kernel (conversion passes + kind::f16), which the library picks by size in production."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from gpu_util import DEV, assert_bits_equal, n, outlier_randn, t

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def LIN():
    from jetfire_int8training_b200 import Linear
    return Linear


@pytest.fixture(scope="module")
def L():
    from jetfire_int8training_b200._lib import lib
    return lib()


@pytest.fixture(params=[False, True], ids=["i8ops", "f16ops"])
def op16(request):
    """operand_scratch argument of the Linear wrappers: False = int8-operand kernel, True = fp16-operand kernel."""
    return request.param


@pytest.fixture(autouse=True)
def _no_expired_wait(L):
    yield
    torch.cuda.synchronize()
    assert L.jf_igemm_error_flag() == 0, "a bounded wait inside the GEMM kernel expired"


def rand_operands(seed, M, N, K):
    """int8 payloads uniform in [-127,127], scales uniform in [1e-3, 1e-1] (the GEMM sweep's input distribution)."""
    rng = np.random.default_rng(seed)
    A = rng.integers(-127, 128, (M, K), dtype=np.int8)
    B = rng.integers(-127, 128, (N, K), dtype=np.int8)
    SA = rng.uniform(1e-3, 1e-1, (M // 32, K // 32)).astype(np.float16)
    SB = rng.uniform(1e-3, 1e-1, (N // 32, K // 32)).astype(np.float16)
    return A, B, SA, SB


def int32_gemm(L, A, B):
    M, K = A.shape
    N = B.shape[0]
    a, b = t(A), t(B)
    c = torch.empty((M, N), dtype=torch.int32, device=DEV)
    st = L.jf_igemm_int32(a.data_ptr(), b.data_ptr(), M, N, K, c.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0, st
    return n(c)


def test_int32_known_answer_fixture(L):
    """The reference's A/B/CPU.txt fixture (128x128x32), through the tensor-core path."""
    d = load_golden("gemm_basic_int8_128_128_32")
    got = int32_gemm(L, d["A"], np.ascontiguousarray(d["B"].T))
    assert np.array_equal(got, d["C"])


@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (128, 128, 128), (128, 128, 160), (256, 384, 512), (32, 32, 32), (96, 160, 224),
                                   (1024, 2048, 3072)])
def test_int32_exact(L, oracle, M, N, K):
    A, B, _, _ = rand_operands(K + M, M, N, K)
    got = int32_gemm(L, A, B)
    assert np.array_equal(got, oracle.gemm_int32(A, B))


FWD_SHAPES = [(128, 128, 32), (128, 128, 256), (32, 64, 96), (160, 288, 416), (512, 512, 512), (1024, 2048, 512),
              (2048, 3072, 768), (256, 4224, 1600)]


@pytest.mark.parametrize("M,N,K", FWD_SHAPES)
def test_forward_bit_exact(LIN, oracle, op16, M, N, K):
    A, B, SA, SB = rand_operands(M + N + K, M, N, K)
    q, s = LIN.int8_linear_forward(t(A), t(SA), t(B), t(SB), True, 32, operand_scratch=op16)
    qo, so, do = oracle.linear_forward(A, SA, B, SB, dequantized=True)
    assert_bits_equal(n(q), qo, "payload"); assert_bits_equal(n(s), so, "scales")
    y16 = LIN.int8_linear_forward(t(A), t(SA), t(B), t(SB), False, 32, operand_scratch=op16)
    assert_bits_equal(n(y16), do, "dequantised fp16")


@pytest.mark.parametrize("M,N,K", FWD_SHAPES)
def test_backward_bit_exact(LIN, oracle, op16, M, N, K):
    """dgrad (M x Cin x Cout) with a fixed Philox key and wgrad (Cout x Cin x tokens), operands in their natural layouts."""
    tokens, Cin, Cout = M, N, K
    rng = np.random.default_rng(tokens + Cin * 3 + Cout)
    G = rng.integers(-127, 128, (tokens, Cout), dtype=np.int8)
    X = rng.integers(-127, 128, (tokens, Cin), dtype=np.int8)
    W = rng.integers(-127, 128, (Cout, Cin), dtype=np.int8)
    SG = rng.uniform(1e-3, 1e-1, (tokens // 32, Cout // 32)).astype(np.float16)
    SX = rng.uniform(1e-3, 1e-1, (tokens // 32, Cin // 32)).astype(np.float16)
    SW = rng.uniform(1e-3, 1e-1, (Cout // 32, Cin // 32)).astype(np.float16)
    key = (0xC0FFEE, 3)
    gx, gs, gw = LIN.int8_linear_backward(t(X), t(SX), t(G), t(SG), None, t(W), t(SW), 32, stochastic=True, sr_key=key,
                                          wgrad_split_k=1, operand_scratch=op16)
    noise = oracle.sr_noise(tokens, Cin, *key)
    qo, so = oracle.linear_dgrad(G, SG, W, SW, noise)
    assert_bits_equal(n(gx), qo, "dgrad payload"); assert_bits_equal(n(gs), so, "dgrad scales")
    assert_bits_equal(n(gw), oracle.linear_wgrad(G, SG, X, SX), "wgrad fp16")
    # round-to-nearest and dequantised variants
    gx, gs, _ = LIN.int8_linear_backward(t(X), t(SX), t(G), t(SG), None, t(W), t(SW), 32, stochastic=False, wgrad_split_k=1,
                                         operand_scratch=op16)
    qo, so, do = oracle.linear_dgrad(G, SG, W, SW, None, dequantized=True)
    assert_bits_equal(n(gx), qo, "dgrad RN payload"); assert_bits_equal(n(gs), so, "dgrad RN scales")
    g16, _ = LIN.int8_linear_backward(t(X), t(SX), t(G), t(SG), None, t(W), t(SW), 32, stochastic=False, dgrad_quantize=False,
                                      wgrad_split_k=1, operand_scratch=op16)
    assert_bits_equal(n(g16), do, "dgrad dequantised")


@pytest.mark.parametrize("tokens,Cin,Cout,split", [(2048, 128, 128, 4), (4096, 768, 768, 0), (1024, 96, 160, 3)])
def test_wgrad_split_k_is_deterministic_and_matches_oracle(LIN, L, oracle, op16, tokens, Cin, Cout, split):
    rng = np.random.default_rng(tokens + split)
    G = rng.integers(-127, 128, (tokens, Cout), dtype=np.int8)
    X = rng.integers(-127, 128, (tokens, Cin), dtype=np.int8)
    SG = rng.uniform(1e-3, 1e-1, (tokens // 32, Cout // 32)).astype(np.float16)
    SX = rng.uniform(1e-3, 1e-1, (tokens // 32, Cin // 32)).astype(np.float16)
    eff = L.jf_igemm_wgrad_plan(Cout, Cin, tokens, split)
    assert eff >= 1
    for dt, ndt in ((torch.float32, np.float32), (torch.float16, np.float16)):
        dw = LIN.int8_linear_wgrad(t(X), t(SX), t(G), t(SG), dt, split, operand_scratch=op16)
        want = oracle.linear_wgrad(G, SG, X, SX, split_k=eff, out_dtype=ndt)
        assert_bits_equal(n(dw), want, f"wgrad split {eff} {ndt.__name__}")
        assert torch.equal(dw, LIN.int8_linear_wgrad(t(X), t(SX), t(G), t(SG), dt, split))


def test_config1_linear_layer(LIN, oracle):
    """Single linear layer forward + backward on the benchmark's first configuration: X bf16 [2048,768] N(0,1) with 0.5% outlier
    channels x30, W bf16 [3072,768] N(0,0.02), dY N(0,1e-2) [2048,3072], all block-quantised, seed 0."""
    from jetfire_int8training_b200 import Nonlinear as NL
    g = torch.Generator().manual_seed(0)
    X = outlier_randn(g, 2048, 768).to(torch.bfloat16)
    W = (0.02 * torch.randn(3072, 768, generator=g)).to(torch.bfloat16)
    dY = (1e-2 * torch.randn(2048, 3072, generator=g)).to(torch.bfloat16)
    (qx, sx), (qw, sw), (qg, sg) = [NL.int8_quantize(v.to(DEV), 32) for v in (X, W, dY)]
    for v, (q, s) in ((X, (qx, sx)), (W, (qw, sw)), (dY, (qg, sg))):
        qo, so = oracle.int8_quantize(v.float().numpy())
        assert_bits_equal(n(q), qo); assert_bits_equal(n(s), so)
    y, sy = LIN.int8_linear_forward(qx, sx, qw, sw, True, 32)
    qo, so = oracle.linear_forward(n(qx), n(sx), n(qw), n(sw))
    assert_bits_equal(n(y), qo, "Y"); assert_bits_equal(n(sy), so, "SY")
    key = (0, 0)
    gx, gs, gw = LIN.int8_linear_backward(qx, sx, qg, sg, None, qw, sw, 32, stochastic=True, sr_key=key, wgrad_split_k=1)
    qo, so = oracle.linear_dgrad(n(qg), n(sg), n(qw), n(sw), oracle.sr_noise(2048, 768, *key))
    assert_bits_equal(n(gx), qo, "dX"); assert_bits_equal(n(gs), so, "SdX")
    assert_bits_equal(n(gw), oracle.linear_wgrad(n(qg), n(sg), n(qx), n(sx)), "dW")
    # FP tolerance of the whole layer against the unquantised product: the reference's own acceptance test (rtol 1e-1 level)
    ref = X.float() @ W.float().t()
    deq = NL.int8_dequantize(y, sy, 32).cpu()
    assert float((deq - ref).norm() / ref.norm()) < 5e-2


def test_dgrad_stochastic_rounding_is_unbiased(LIN, oracle):
    """Mean over many draws approaches the unrounded accumulator (the reference's test averages 100-1000 runs,
    JetfireGEMMKernel/tests/test_int8igemmoutputIntQuantizeStochastic.py:70-120)."""
    tokens, Cin, Cout = 128, 128, 256
    rng = np.random.default_rng(1)
    G = rng.integers(-127, 128, (tokens, Cout), dtype=np.int8)
    W = rng.integers(-127, 128, (Cout, Cin), dtype=np.int8)
    SG = rng.uniform(1e-3, 1e-1, (tokens // 32, Cout // 32)).astype(np.float16)
    SW = rng.uniform(1e-3, 1e-1, (Cout // 32, Cin // 32)).astype(np.float16)
    X = np.zeros((tokens, Cin), np.int8); SX = np.ones((tokens // 32, Cin // 32), np.float16)
    acc = oracle.gemm_accumulate(G, W.T, SG, SW.T)
    tot = torch.zeros(tokens, Cin, device=DEV)
    R = 300
    gt, sgt, wt, swt, xt, sxt = t(G), t(SG), t(W), t(SW), t(X), t(SX)
    for r in range(R):
        gx, gs, _ = LIN.int8_linear_backward(xt, sxt, gt, sgt, None, wt, swt, 32, stochastic=True, sr_key=(5, r), wgrad_split_k=1)
        tot += gx.float() * gs.float().repeat_interleave(32, 0).repeat_interleave(32, 1)
    mean = (tot / R).cpu().numpy()
    err_sr = np.abs(mean - acc).mean()
    qo, so = oracle.linear_dgrad(G, SG, W, SW, None)
    err_rn = np.abs(qo.astype(np.float32) * np.kron(so.astype(np.float32), np.ones((32, 32), np.float32)) - acc).mean()
    assert err_sr < 0.3 * err_rn


def test_full_size_properties(LIN, L):
    """8192^3 (the headline shape): linearity in the scales and agreement of the three layouts with one another."""
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(0)
    A = torch.randint(-127, 128, (M, K), generator=g, device=DEV, dtype=torch.int8)
    B = torch.randint(-127, 128, (N, K), generator=g, device=DEV, dtype=torch.int8)
    SA = (torch.rand(M // 32, K // 32, generator=g, device=DEV) * 0.099 + 1e-3).half()
    SB = (torch.rand(N // 32, K // 32, generator=g, device=DEV) * 0.099 + 1e-3).half()
    q, s = LIN.int8_linear_forward(A, SA, B, SB, True, 32)
    # doubling every A scale (exact in fp16) doubles every output scale and leaves the payload unchanged
    q2, s2 = LIN.int8_linear_forward(A, SA * 2, B, SB, True, 32)
    assert torch.equal(q, q2) and torch.equal(s2.float(), s.float() * 2)
    # the same product through the dgrad layout (B given as [K, N]) with rounding to nearest
    Bt = B.t().contiguous()
    Z8 = torch.zeros((M, 32), dtype=torch.int8, device=DEV); ZS = torch.ones((M // 32, 1), dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    q3 = torch.empty_like(q); s3 = torch.empty_like(s)
    SBt = SB.t().contiguous()
    rc = L.jf_igemm_dgrad(A.data_ptr(), Bt.data_ptr(), SA.data_ptr(), SA.stride(0), SA.stride(1), SBt.data_ptr(), SBt.stride(0),
                          SBt.stride(1), M, N, K, 0, q3.data_ptr(), s3.data_ptr(), None, 0, None, 0, 0, None, 0, st)
    assert rc == 0
    assert torch.equal(q, q3) and torch.equal(s, s3)
    # a 512-row slab against the exact integer product with unit scales
    ones_a = torch.ones_like(SA); ones_b = torch.ones_like(SB)
    c = torch.empty((512, 512), dtype=torch.int32, device=DEV)
    rc = L.jf_igemm_int32(A.data_ptr(), B.data_ptr(), 512, 512, K, c.data_ptr(), st)
    assert rc == 0
    ref = (A[:512].double() @ B[:512].double().t())
    assert torch.equal(c.double(), ref)


def test_errors(L):
    st = torch.cuda.current_stream().cuda_stream
    a = torch.zeros((64, 64), dtype=torch.int8, device=DEV)
    s = torch.ones((2, 2), dtype=torch.float16, device=DEV)
    assert L.jf_igemm_forward(a.data_ptr(), a.data_ptr(), s.data_ptr(), 2, 1, s.data_ptr(), 2, 1, 64, 48, 64, 0, a.data_ptr(),
                              s.data_ptr(), None, None, 0, st) == -2              # N not a multiple of 32
    assert L.jf_igemm_forward(None, a.data_ptr(), s.data_ptr(), 2, 1, s.data_ptr(), 2, 1, 64, 64, 64, 0, a.data_ptr(),
                              s.data_ptr(), None, None, 0, st) == -1              # NULL operand
    assert L.jf_igemm_forward(a.data_ptr() + 1, a.data_ptr(), s.data_ptr(), 2, 1, s.data_ptr(), 2, 1, 64, 64, 64, 0,
                              a.data_ptr(), s.data_ptr(), None, None, 0, st) == -3   # misaligned operand
