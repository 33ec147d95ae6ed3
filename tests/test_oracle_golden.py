"""CPU: the oracle against the golden vectors produced by the reference's own Triton kernels (interpreter) and against
the reference's GEMM known-answer fixture.  These pins are what makes the oracle trustworthy as the GPU checker."""
import numpy as np
import pytest

from conftest import load_golden, to_np


def _eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("tag", ["f32", "f16", "bf16"])
def test_quantize_bit_exact(oracle, tag):
    d = load_golden("quantize_" + tag)
    q, s = oracle.int8_quantize(to_np(d["x"]))
    _eq(q, d["q"]); _eq(s, d["s"])
    d = load_golden("quantize_transpose_" + tag)
    q, s, qt = oracle.int8_quantize_transpose(to_np(d["x"]))
    _eq(q, d["q"]); _eq(s, d["s"]); _eq(qt, d["qt"])


def test_quantize_all_zero_block_gives_zero_scale_and_payload(oracle):
    d = load_golden("quantize_f32")
    assert np.all(d["q"][32:64, 64:96] == 0) and d["s"][1, 2] == 0
    q, s = oracle.int8_quantize(d["x"])
    assert np.all(q[32:64, 64:96] == 0) and s[1, 2] == 0


def test_quantize_stochastic_with_reference_noise(oracle):
    d = load_golden("quantize_sr_bf16")
    q, s = oracle.int8_quantize(to_np(d["x"]), d["noise"])
    _eq(q, d["q"]); _eq(s, d["s"])


def test_quantize_3d(oracle):
    d = load_golden("quantize_3d_f32")
    q, s = oracle.int8_quantize(d["x"])
    _eq(q, d["q"].reshape(q.shape)); _eq(s, d["s"].reshape(s.shape))


def test_transpose_and_dequantize(oracle):
    d = load_golden("transpose")
    _eq(oracle.int8_transpose(d["x"]), d["y"])
    d = load_golden("dequantize")
    _eq(oracle.int8_dequantize(d["q"], d["s"]), d["y"])


def test_gelu(oracle):
    d = load_golden("gelu_fwd")
    q, s = oracle.int8_gelu_forward(d["qx"], d["sx"])
    _eq(q, d["qy"]); _eq(s, d["sy"])
    d = load_golden("gelu_bwd")
    q, s = oracle.int8_gelu_backward(d["qx"], d["sx"], d["qg"], d["sg"])
    _eq(q, d["qd"]); _eq(s, d["sd"])
    d = load_golden("gelu_bwd_sr")
    q, s = oracle.int8_gelu_backward(d["qx"], d["sx"], d["qg"], d["sg"], d["noise"])
    _eq(q, d["qd"]); _eq(s, d["sd"])


def test_layernorm(oracle):
    d = load_golden("ln_fwd")
    q, s = oracle.int8_layernorm_forward(d["qx"], d["sx"], d["gamma"], d["mean"], d["rstd"])
    _eq(q, d["qy"]); _eq(s, d["sy"])
    for name in ("ln_bwd", "ln_bwd_sr"):
        d = load_golden(name)
        q, s, dw = oracle.int8_layernorm_backward(d["qx"], d["sx"], d["qg"], d["sg"], d["gamma"], d["mean"], d["rstd"],
                                                  d.get("noise"))
        _eq(q, d["qd"]); _eq(s, d["sd"]); _eq(dw, d["dw"])


def test_layernorm_backward_is_the_slab_formula_not_the_row_formula(oracle):
    d = load_golden("ln_bwd")
    q_row, _, _ = oracle.int8_layernorm_backward(d["qx"], d["sx"], d["qg"], d["sg"], d["gamma"], d["mean"], d["rstd"], slab=None)
    assert np.count_nonzero(q_row != d["qd"]) > 1000   # the full-row reduction is NOT what the reference computes


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_add(oracle, tag):
    d = load_golden("add_" + tag)
    y, q, s = oracle.int8_add(to_np(d["x1"]), d["q2"], d["s2"])
    _eq(y, d["y1"]); _eq(q, d["qy"]); _eq(s, d["sy"])
    d = load_golden("add_sr_" + tag)
    y, q, s = oracle.int8_add(to_np(d["x1"]), d["q2"], d["s2"], d["noise"])
    _eq(y, d["y1"]); _eq(q, d["qy"]); _eq(s, d["sy"])
    d = load_golden("add_meanvar_" + tag)
    y, q, s, mean, rstd = oracle.int8_add_meanvar(to_np(d["x1"]), d["q2"], d["s2"])
    _eq(y, d["y1"]); _eq(q, d["qy"]); _eq(s, d["sy"])
    np.testing.assert_allclose(mean, d["mean"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(rstd, d["rstd"], rtol=1e-6)


def test_gemm_known_answer(oracle):
    d = load_golden("gemm_basic_int8_128_128_32")
    A, B, C = d["A"], d["B"], d["C"]
    assert np.array_equal(oracle.gemm_int32(A, B.T), C)
    # the per-block path with unit scales must reproduce the same integers exactly
    one = np.ones((4, 1), np.float16)
    acc = oracle.gemm_accumulate(A, np.ascontiguousarray(B.T), one, one)
    assert np.array_equal(acc.astype(np.int64), C.astype(np.int64))


def test_gemm_matches_torch_level_emulation(oracle):
    """The reference's own test recipe (JetfireGEMMKernel/tests/test_int8igemmoutputIntQuantizeStochastic.py:24-51):
    dequantise, fp matmul, compare at rtol 1e-1 -- plus the exact per-block restatement in float64."""
    rng = np.random.default_rng(0)
    M, N, K = 64, 96, 128
    A = rng.integers(-127, 128, (M, K), dtype=np.int8)
    B = rng.integers(-127, 128, (N, K), dtype=np.int8)
    SA = rng.uniform(1e-3, 1e-1, (M // 32, K // 32)).astype(np.float16)
    SB = rng.uniform(1e-3, 1e-1, (N // 32, K // 32)).astype(np.float16)
    acc = oracle.gemm_accumulate(A, B, SA, SB)
    ra = A.astype(np.float64) * np.kron(SA.astype(np.float64), np.ones((32, 32)))
    rb = B.astype(np.float64) * np.kron(SB.astype(np.float64), np.ones((32, 32)))
    ref = ra @ rb.T
    assert np.abs(acc - ref).max() / np.abs(ref).max() < 1e-5
    q, s = oracle.requant(acc)
    deq = q.astype(np.float64) * np.kron(s.astype(np.float64), np.ones((32, 32)))
    assert np.linalg.norm(deq - ref) / np.linalg.norm(ref) < 2e-2
    # layouts: dgrad / wgrad helpers agree with the generic routine on transposed views
    W = np.ascontiguousarray(B.T)            # [K, N]
    SW = np.ascontiguousarray(SB.T)
    q2, s2 = oracle.linear_dgrad(A, SA, W, SW)
    assert np.array_equal(q2, q) and np.array_equal(s2, s)
    G = np.ascontiguousarray(A.T)            # [K(tokens), M]
    SG = np.ascontiguousarray(SA.T)
    dw = oracle.linear_wgrad(G, SG, W, SW, out_dtype=np.float32)
    assert np.array_equal(dw, acc)
    dw2 = oracle.linear_wgrad(G, SG, W, SW, split_k=2, out_dtype=np.float32)
    assert np.abs(dw2 - acc).max() / np.abs(acc).max() < 1e-6


def test_philox_known_answers(oracle):
    """Random123 known-answer vectors for philox4x32-10."""
    def run(c, k):
        return [int(x) for x in oracle.philox4x32_10(*[np.uint32(v) for v in c], k[0], k[1])]
    assert run((0, 0, 0, 0), (0, 0)) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert run((0xffffffff,) * 4, (0xffffffff, 0xffffffff)) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert run((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0)) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_sr_noise_is_centred_and_in_range(oracle):
    n = oracle.sr_noise(256, 256, seed=1234, offset=7)
    assert n.dtype == np.float32 and np.all(n >= -0.5) and np.all(n < 0.5)
    assert abs(float(n.mean())) < 5e-3
    assert not np.array_equal(n, oracle.sr_noise(256, 256, seed=1234, offset=8))
