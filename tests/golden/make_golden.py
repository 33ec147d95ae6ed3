#!/usr/bin/env python
"""Generate the golden input/output vectors under tests/golden/ from the reference itself.

Runs only where the reference checkout is available (pass its root with --reference).
It executes the reference's own, unmodified Triton kernels (Jetfire/Nonlinear/*.py) on CPU
under TRITON_INTERPRET=1 and stores inputs + outputs as small .npz fixtures, and converts
the reference's only complete GEMM known-answer fixture
(JetfireGEMMKernel/cppsrc/igemm/igemm_BasicInt8Gemm_128_128_32/{A,B,CPU}.txt) to .npz.

Harness-level shims (no reference file is edited):
  * the autotuner needs a GPU driver -> run the first config directly;
  * triton.language.extra.cuda.libdevice is not patched by the interpreter -> numpy-backed
    llrint / signbit / erf / sqrt / pow;
  * list grids -> tuples; device="cuda" allocations -> CPU.

Usage:  python tests/golden/make_golden.py --reference /path/to/Jetfire-INT8Training
"""
import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import scipy.special
import torch
import triton
import triton.language as tl
from triton.runtime import interpreter as _interp
from triton.runtime.autotuner import Autotuner
from triton.language.extra.cuda import libdevice as _libdevice

HERE = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------- shims
def _install_shims():
    def _run_first_config(self, *args, **kwargs):
        cfg = self.configs[0]
        kw = dict(kwargs)
        kw.update(cfg.all_kwargs())
        return self.fn.run(*args, **kw)

    Autotuner.run = _run_first_config

    TH = _interp.TensorHandle

    def _wrap(data, dtype, like=None):
        data = np.asarray(data)
        if data.ndim == 0:
            data = data.reshape(1)
        h = TH(data, dtype)
        if data.shape == (1,) and (like is None or not like.type.is_block()):
            return tl.tensor(h, dtype)
        return tl.tensor(h, tl.block_type(dtype, list(data.shape)))

    def _as_np(x):
        if isinstance(x, tl.tensor):
            return x.handle.data, x.dtype, x
        if isinstance(x, tl.constexpr):
            x = x.value
        return np.array([x], dtype=np.float32), tl.float32, None

    def llrint(x, **_):
        d, _t, like = _as_np(x)
        return _wrap(np.rint(d).astype(np.int64), tl.int64, like)

    def signbit(x, **_):
        d, _t, like = _as_np(x)
        return _wrap(np.signbit(d).astype(np.int32), tl.int32, like)

    def erf(x, **_):
        d, t, like = _as_np(x)
        return _wrap(scipy.special.erf(d).astype(d.dtype), t, like)

    def sqrt(x, **_):
        d, t, like = _as_np(x)
        return _wrap(np.sqrt(d).astype(d.dtype), t, like)

    def pow_(x, y, **_):
        d, t, like = _as_np(x)
        e = y.value if isinstance(y, tl.constexpr) else y
        if isinstance(e, tl.tensor):
            e = e.handle.data
        return _wrap(np.power(d, np.asarray(e).astype(d.dtype)).astype(d.dtype), t, like)

    _libdevice.llrint = llrint
    _libdevice.signbit = signbit
    _libdevice.erf = erf
    _libdevice.sqrt = sqrt
    _libdevice.pow = pow_

    _orig_init = _interp.GridExecutor.__init__

    def _init(self, fn, arg_names, grid, *a, **k):
        if isinstance(grid, list):
            grid = tuple(grid)
        elif callable(grid):
            g0 = grid

            def grid(meta, _g=g0):
                r = _g(meta)
                return tuple(r) if isinstance(r, list) else r
        _orig_init(self, fn, arg_names, grid, *a, **k)

    _interp.GridExecutor.__init__ = _init

    for name in ("empty", "empty_like", "zeros", "zeros_like"):
        orig = getattr(torch, name)

        def _cpu(*a, __orig=orig, **k):
            if str(k.get("device", "")).startswith("cuda"):
                k["device"] = "cpu"
            return __orig(*a, **k)

        setattr(torch, name, _cpu)


# --------------------------------------------------------------------------- inputs
def block_quantize_ref(x, QB=32):
    """fp32 block absmax quantize used only to *prepare* int8 inputs for the ops."""
    M, N = x.shape
    xb = x.float().reshape(M // QB, QB, N // QB, QB)
    s = xb.abs().amax((1, 3)) / 127.0
    q = torch.round(xb / s[:, None, :, None]).reshape(M, N).to(torch.int8)
    return q, s.half()


def outlier_randn(g, M, N, frac=0.005, mult=30.0):
    x = torch.randn(M, N, generator=g)
    k = max(1, round(frac * N))
    idx = torch.randperm(N, generator=g)[:k]
    x[:, idx] *= mult
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("JETFIRE_REFERENCE"), required="JETFIRE_REFERENCE" not in os.environ,
                    help="checkout of thu-ml/Jetfire-INT8Training (or set JETFIRE_REFERENCE)")
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()

    _install_shims()
    sys.path.insert(0, os.path.join(args.reference, "Jetfire"))
    import Nonlinear as R  # the reference's operator package, unmodified
    from Nonlinear.dequantize import int8_dequantize as ref_dequantize

    QB = 32
    out = {}

    def save(name, **arrs):
        conv = {}
        for k, v in arrs.items():
            if isinstance(v, torch.Tensor):
                if v.dtype == torch.bfloat16:
                    v = v.view(torch.int16)
                    k = k + "__bf16"
                v = v.numpy()
            conv[k] = v
        np.savez_compressed(os.path.join(args.out, name + ".npz"), **conv)
        print("wrote", name, {k: (v.shape, str(v.dtype)) for k, v in conv.items()})

    # ---------------- quantize (RN) for fp32 / fp16 / bf16, and SR with explicit noise
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16"), (torch.bfloat16, "bf16")):
        g = torch.Generator().manual_seed(100)
        x = outlier_randn(g, 128, 256).to(dt)
        x[32:64, 64:96] = 0  # an all-zero block
        q, s = R.int8_quantize(x, QB)
        save(f"quantize_{tag}", x=x, q=q, s=s)
        q2, s2, qt = R.int8_quantize_transpose(x, QB)
        save(f"quantize_transpose_{tag}", x=x, q=q2, s=s2, qt=qt)

    g = torch.Generator().manual_seed(101)
    x = outlier_randn(g, 128, 256).to(torch.bfloat16)
    torch.manual_seed(7)
    noise = torch.empty_like(x, dtype=torch.float32).uniform_(-0.5, 0.5)
    torch.manual_seed(7)  # the op draws the identical tensor from the global generator
    q, s = R.int8_quantize(x, QB, stochastic=True)
    save("quantize_sr_bf16", x=x, noise=noise, q=q, s=s)

    # 3-D input path
    g = torch.Generator().manual_seed(102)
    x3 = torch.randn(2, 64, 128, generator=g)
    q, s = R.int8_quantize(x3, QB)
    save("quantize_3d_f32", x=x3, q=q, s=s)

    # ---------------- transpose
    g = torch.Generator().manual_seed(103)
    xi = torch.randint(-128, 128, (128, 192), generator=g, dtype=torch.int8)
    save("transpose", x=xi, y=R.int8_transpose(xi))

    # ---------------- dequantize
    g = torch.Generator().manual_seed(104)
    qx, sx = block_quantize_ref(outlier_randn(g, 128, 256))
    save("dequantize", q=qx, s=sx, y=ref_dequantize(qx, sx, QB))

    # ---------------- GELU forward / backward
    g = torch.Generator().manual_seed(105)
    qx, sx = block_quantize_ref(outlier_randn(g, 128, 256))
    qy, sy = R.int8_gelu_forward(qx, sx, QB)
    save("gelu_fwd", qx=qx, sx=sx, qy=qy, sy=sy)

    qg, sg = block_quantize_ref(1e-2 * torch.randn(128, 256, generator=g))
    qd, sd = R.int8_gelu_backward(qx, sx, qg, sg, QB, stochastic=False)
    save("gelu_bwd", qx=qx, sx=sx, qg=qg, sg=sg, qd=qd, sd=sd)
    torch.manual_seed(8)
    noise = torch.empty(128, 256, dtype=torch.float32).uniform_(-0.5, 0.5)
    torch.manual_seed(8)
    qd, sd = R.int8_gelu_backward(qx, sx, qg, sg, QB, stochastic=True)
    save("gelu_bwd_sr", qx=qx, sx=sx, qg=qg, sg=sg, noise=noise, qd=qd, sd=sd)

    # ---------------- LayerNorm forward / backward (stats supplied by the caller)
    g = torch.Generator().manual_seed(106)
    xf = outlier_randn(g, 128, 256)
    qx, sx = block_quantize_ref(xf)
    gamma = 1.0 + 0.1 * torch.randn(256, generator=g)
    xd = (qx.float().reshape(4, 32, 8, 32) * sx.float()[:, None, :, None]).reshape(128, 256)
    mean = xd.mean(-1)
    rstd = 1.0 / xd.var(-1, unbiased=False).sqrt()
    qy, sy, _ = R.int8_layernorm_forward(qx, sx, gamma, mean, rstd, QB)
    save("ln_fwd", qx=qx, sx=sx, gamma=gamma, mean=mean, rstd=rstd, qy=qy, sy=sy)

    qg, sg = block_quantize_ref(1e-2 * torch.randn(128, 256, generator=g))
    qd, sd, dw = R.int8_layernorm_backward(qx, sx, qg, sg, gamma, QB, mean, rstd, stochastic=False)
    save("ln_bwd", qx=qx, sx=sx, qg=qg, sg=sg, gamma=gamma, mean=mean, rstd=rstd, qd=qd, sd=sd, dw=dw)
    torch.manual_seed(9)
    noise = torch.empty(128, 256, dtype=torch.float32).uniform_(-0.5, 0.5)
    torch.manual_seed(9)
    qd, sd, dw = R.int8_layernorm_backward(qx, sx, qg, sg, gamma, QB, mean, rstd, stochastic=True)
    save("ln_bwd_sr", qx=qx, sx=sx, qg=qg, sg=sg, gamma=gamma, mean=mean, rstd=rstd, noise=noise,
         qd=qd, sd=sd, dw=dw)

    # ---------------- residual add (+SR) and add + mean/var
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        g = torch.Generator().manual_seed(107)
        x1 = outlier_randn(g, 128, 256).to(dt)
        q2, s2 = block_quantize_ref(torch.randn(128, 256, generator=g))
        y1, qy, sy = R.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, QB, stochastic=False)
        save(f"add_{tag}", x1=x1, q2=q2, s2=s2, y1=y1, qy=qy, sy=sy)
        torch.manual_seed(10)
        noise = torch.empty(128, 256, dtype=torch.float32).uniform_(-0.5, 0.5)
        torch.manual_seed(10)
        y1, qy, sy = R.int8_add_Ifp_Ig16_Ofp_Og(x1, q2, s2, QB, stochastic=True)
        save(f"add_sr_{tag}", x1=x1, q2=q2, s2=s2, noise=noise, y1=y1, qy=qy, sy=sy)
        y1, qy, sy, mean, rstd = R.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, q2, s2, QB)
        save(f"add_meanvar_{tag}", x1=x1, q2=q2, s2=s2, y1=y1, qy=qy, sy=sy, mean=mean, rstd=rstd)

    # ---------------- GEMM known-answer fixture shipped by the reference
    kd = os.path.join(args.reference, "JetfireGEMMKernel", "cppsrc", "igemm", "igemm_BasicInt8Gemm_128_128_32")
    A = np.loadtxt(os.path.join(kd, "A.txt"), dtype=np.int64).reshape(128, 32).astype(np.int8)
    B = np.loadtxt(os.path.join(kd, "B.txt"), dtype=np.int64).reshape(32, 128).astype(np.int8)
    C = np.loadtxt(os.path.join(kd, "CPU.txt"), dtype=np.int64).reshape(128, 128).astype(np.int32)
    assert np.array_equal(A.astype(np.int32) @ B.astype(np.int32), C)
    np.savez_compressed(os.path.join(args.out, "gemm_basic_int8_128_128_32.npz"), A=A, B=B, C=C)
    print("wrote gemm_basic_int8_128_128_32")


if __name__ == "__main__":
    main()
