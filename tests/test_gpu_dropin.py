"""GPU: the package as a drop-in UNDER the reference's own, unmodified caller code.

  * INT8_GPT2/qmodel.py (QGPT, its five autograd Functions and modules) imported as the reference ships it, on top of this
    package's `Nonlinear` / `Linear` modules registered by compat.install() -- forward + backward on a tiny configuration;
  * Jetfire/Linear/linear_fwd.py and linear_bwd.py, the reference's glue around its `BlockQuantizeCUDA` extension, on top of
    this package's `BlockQuantizeCUDA` shim: transposed scale copies, the `W8.t()` view, the materialised dY^T with
    g_transposed = 1 -- results bit for bit against the CPU oracle.

The reference files come from $JETFIRE_REFERENCE, a checkout at the default location, or the copies staged by
tests/stage_reference.py; without any of them the tests skip.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import pytest
import torch

from gpu_util import DEV, assert_bits_equal, n, t
from stage_reference import reference_files_root

pytestmark = pytest.mark.gpu

REF = reference_files_root()
needs_ref = pytest.mark.skipif(REF is None, reason="no reference checkout and nothing staged by tests/stage_reference.py")


def _load(name, relpath):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, relpath))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def installed():
    from jetfire_int8training_b200 import compat
    compat.install()
    import BlockQuantizeCUDA
    import Linear
    import Nonlinear
    assert Nonlinear.__name__.startswith("jetfire_int8training_b200") and Linear.__name__.startswith("jetfire_int8training_b200")
    return BlockQuantizeCUDA


@needs_ref
def test_reference_qmodel_runs_unmodified_on_this_package(installed):
    """QGPT of the reference's qmodel.py: forward + backward, loss next to this package's own harness on the same weights."""
    from jetfire_int8training_b200 import gpt2, rng
    qmodel = _load("jetfire_reference_qmodel", "INT8_GPT2/qmodel.py")
    torch.manual_seed(0)
    rng.manual_seed(11)
    cfg = qmodel.GPTConfig(block_size=64, vocab_size=512, n_layer=2, n_head=2, n_embd=128, dropout=0.0, bias=False)
    qargs = types.SimpleNamespace(qgroup_size_non=32, qgroup_size_lin=32)
    model = qmodel.QGPT(cfg, qargs).to(DEV)
    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, 512, (4, 64), generator=g).to(DEV)
    tgt = torch.randint(0, 512, (4, 64), generator=g).to(DEV)
    with torch.autocast("cuda", dtype=torch.float16):
        logits, loss = model(idx, tgt)
    assert logits.shape == (4, 64, 512) and torch.isfinite(loss)
    assert abs(float(loss) - float(np.log(512))) < 0.3            # random init: loss ~ ln(vocab)
    loss.backward()
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        assert float(p.grad.abs().max()) > 0, name
    # the same weights in this package's own harness (same data flow, written independently) give the same loss
    ours = gpt2.QGPT(gpt2.GPTConfig(block_size=64, vocab_size=512, n_layer=2, n_head=2, n_embd=128)).to(DEV)
    with torch.no_grad():
        ours.wte.weight.copy_(model.transformer.wte.weight); ours.wpe.weight.copy_(model.transformer.wpe.weight)
        ours.ln_f.copy_(model.transformer.ln_f.weight)
        for b, rb in zip(ours.blocks, model.transformer.h):
            at, ml = rb.attn_residual, rb.mlp_residual
            b.ln_1.copy_(at.ln_1.weight); b.c_attn.copy_(at.c_attn.weight); b.c_proj.copy_(at.c_proj.weight)
            b.ln_2.copy_(ml.ln_2.weight); b.c_fc.copy_(ml.c_fc.weight); b.c_proj2.copy_(ml.c_proj.weight)
    loss_ours = ours(idx, tgt)
    assert abs(float(loss_ours) - float(loss)) < 2e-2 * float(loss)   # fp16 vs bf16 LM head, otherwise the same operators
    # ... and the same gradients: the reference's autograd Functions and this package's harness wire the backward operators
    # the same way (different stochastic-rounding draws, so cosine and norm instead of bits)
    loss_ours.backward()
    pairs = [("wte", ours.wte.weight, model.transformer.wte.weight), ("wpe", ours.wpe.weight, model.transformer.wpe.weight),
             ("ln_f", ours.ln_f, model.transformer.ln_f.weight)]
    for i, (b, rb) in enumerate(zip(ours.blocks, model.transformer.h)):
        at, ml = rb.attn_residual, rb.mlp_residual
        pairs += [(f"h{i}.ln_1", b.ln_1, at.ln_1.weight), (f"h{i}.c_attn", b.c_attn, at.c_attn.weight), (f"h{i}.c_proj", b.c_proj, at.c_proj.weight),
                  (f"h{i}.ln_2", b.ln_2, ml.ln_2.weight), (f"h{i}.c_fc", b.c_fc, ml.c_fc.weight), (f"h{i}.c_proj2", b.c_proj2, ml.c_proj.weight)]
    worst = (2.0, 1.0, "")
    for name, po, pr in pairs:
        a, r = po.grad.flatten().float(), pr.grad.flatten().float()
        cos, ratio = float(torch.dot(a, r) / (a.norm() * r.norm())), float(a.norm() / r.norm())
        worst = min(worst, (cos, ratio, name))
        assert cos > 0.98 and 0.9 < ratio < 1.1, (name, cos, ratio)
    print(f"gradients of this package's harness vs the reference's qmodel.py on the same operators: lowest cosine {worst[0]:.4f} ({worst[2]})")


@needs_ref
def test_reference_linear_glue_on_the_extension_shim(installed, oracle):
    """Jetfire/Linear/linear_fwd.py + linear_bwd.py (unmodified) driving this package's BlockQuantizeCUDA functions."""
    from jetfire_int8training_b200 import rng
    fwd = _load("jetfire_reference_linear_fwd", "Jetfire/Linear/linear_fwd.py")
    bwd = _load("jetfire_reference_linear_bwd", "Jetfire/Linear/linear_bwd.py")
    assert sys.modules["BlockQuantizeCUDA"] is installed
    B, T, Cin, Cout = 2, 128, 160, 384          # M = 256 tokens; widths that are multiples of 32 but not of 128
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B * T, Cin, generator=g)
    x[:, 3] *= 30
    w = 0.02 * torch.randn(Cout, Cin, generator=g)
    dy = 1e-2 * torch.randn(B * T, Cout, generator=g)
    qx, sx = oracle.int8_quantize(x.numpy())
    qw, sw = oracle.int8_quantize(w.numpy())
    qg, sg = oracle.int8_quantize(dy.numpy())
    X8 = t(qx).reshape(B, T, Cin); SX = t(sx).reshape(B, T // 32, Cin // 32)
    G8 = t(qg).reshape(B, T, Cout); SG = t(sg).reshape(B, T // 32, Cout // 32)
    W8, SW = t(qw), t(sw)
    # forward, quantised and dequantised outputs
    o8, so = fwd.int8_linear_forward(X8, SX, W8, SW, True, 32)
    qo, sco, deq = oracle.linear_forward(qx, sx, qw, sw, dequantized=True)
    assert o8.shape == (B, T, Cout) and so.shape == (B, T // 32, Cout // 32)
    assert_bits_equal(n(o8).reshape(B * T, Cout), qo, "forward payload"); assert_bits_equal(n(so).reshape(sco.shape), sco, "forward scales")
    o16 = fwd.int8_linear_forward(X8, SX, W8, SW, False, 32)
    assert o16.dtype == torch.float16
    assert_bits_equal(n(o16).reshape(B * T, Cout), deq, "forward dequantised")
    # backward: the reference passes the materialised transpose of dY and always rounds stochastically
    G8T = G8.reshape(B * T, Cout).t().contiguous()
    key = (77, 3)
    rng.manual_seed(*key)
    gx8, gsx, gw = bwd.int8_linear_backward(X8, SX, G8, SG, G8T, W8, SW, 32)
    qdx, sdx = oracle.linear_dgrad(qg, sg, qw, sw, oracle.sr_noise(B * T, Cin, *key))
    assert_bits_equal(n(gx8).reshape(B * T, Cin), qdx, "dgrad payload"); assert_bits_equal(n(gsx).reshape(sdx.shape), sdx, "dgrad scales")
    assert gw.dtype == torch.float16
    assert_bits_equal(n(gw).view(np.uint16), oracle.linear_wgrad(qg, sg, qx, sx).view(np.uint16), "wgrad")
    rng.manual_seed(*key)
    gx16, gw2 = bwd.int8_linear_backward(X8, SX, G8, SG, G8T, W8, SW, 32, dgrad_quantize=False)
    _, _, deq = oracle.linear_dgrad(qg, sg, qw, sw, oracle.sr_noise(B * T, Cin, *key), dequantized=True)
    assert_bits_equal(n(gx16).reshape(B * T, Cin), deq, "dgrad dequantised"); assert torch.equal(gw, gw2)


def test_extension_shim_refuses_a_bias(installed):
    """The reference's forward kernel adds `bias` / `biasmax` (always zero in Jetfire); the shim does not implement them and
    must say so instead of ignoring a non-zero tensor."""
    BQC = installed
    M = N = K = 32
    X = torch.zeros(M, K, dtype=torch.int8, device=DEV); W = torch.zeros(N, K, dtype=torch.int8, device=DEV)
    S = torch.ones(1, 1, dtype=torch.float16, device=DEV)
    z = torch.zeros(N, device=DEV); zm = torch.zeros(1, device=DEV)
    BQC.igemm_output_int_quantize_bias_rowcol(X, W.t(), z, zm, S, S, M, N, K)
    with pytest.raises(NotImplementedError):
        BQC.igemm_output_int_quantize_bias_rowcol(X, W.t(), z + 1, zm, S, S, M, N, K)
    with pytest.raises(NotImplementedError):
        BQC.igemm_output_int_quantize_bias_rowcol(X, W.t(), z, zm + 1, S, S, M, N, K)
