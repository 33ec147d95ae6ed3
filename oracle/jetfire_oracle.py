"""CPU oracle for the Jetfire INT8 hot path.  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arms may import this
module; the product package never does (it fails loudly when its CUDA library is missing).

Every function restates, in IEEE arithmetic on the CPU, one operator of the reference
(thu-ml/Jetfire-INT8Training; citations are paths inside that project).  Parity pinning:
  * the nonlinear operators are checked against golden vectors produced by the reference's own
    Triton kernels run under the Triton CPU interpreter (tests/golden/*.npz, generator beside them);
  * the int32 block product is checked against the reference's A/B/CPU.txt known-answer fixture;
  * the fp32 rescale/accumulate order and the re-quantising GEMM epilogues are pinned only by this
    restatement of the CUDA sources (the reference's own tests use rtol=1e-1) -> "parity unpinned"
    for those bits;
  * stochastic-rounding *noise streams* are unpinned (the reference uses torch.uniform_ / curand
    seeded by libc rand()); with an explicit noise tensor the rounding itself is pinned.

Conventions: int8 payload q[M,N] row-major, scales s[M/32,N/32] float16 (block absmax/127), QB = 32.
"""
import ctypes
import os
import subprocess

import numpy as np
import scipy.special

QB = 32
_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")
_LIB = os.path.join(_BUILD, "libjf_oracle.so")

f32 = np.float32
f16 = np.float16


# --------------------------------------------------------------------------------------------
# C part (GEMM): built on demand with gcc
# --------------------------------------------------------------------------------------------
def build_c_oracle(force=False):
    src = os.path.join(_HERE, "gemm_oracle.c")
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(src):
        return _LIB
    os.makedirs(_BUILD, exist_ok=True)
    cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC",
           src, "-o", _LIB, "-lm"]
    subprocess.check_call(cmd)
    return _LIB


_clib = None


def _c():
    global _clib
    if _clib is None:
        build_c_oracle()
        lib = ctypes.CDLL(_LIB)
        i64, vp = ctypes.c_int64, ctypes.c_void_p
        lib.jf_oracle_gemm_accumulate.argtypes = [vp, i64, i64, vp, i64, i64, vp, i64, i64, vp, i64, i64,
                                                  vp, i64, i64, i64, i64, i64]
        lib.jf_oracle_gemm_int32.argtypes = [vp, i64, i64, vp, i64, i64, vp, i64, i64, i64]
        lib.jf_oracle_requant.argtypes = [vp, i64, i64, vp, vp, vp, vp]
        lib.jf_oracle_to_half.argtypes = [vp, i64, vp]
        lib.jf_oracle_sum_partials.argtypes = [vp, i64, i64, vp]
        lib.jf_oracle_set_threads.argtypes = [ctypes.c_int]
        lib.jf_oracle_set_threads.restype = None
        lib.jf_oracle_max_threads.restype = ctypes.c_int
        lib.jf_oracle_markstein_div.argtypes = [ctypes.c_float, ctypes.c_float]
        lib.jf_oracle_markstein_div.restype = ctypes.c_float
        lib.jf_oracle_markstein_mismatches.argtypes = [vp, vp, i64]
        lib.jf_oracle_markstein_mismatches.restype = i64
        lib.jf_oracle_markstein_sweep_mantissas.argtypes = [ctypes.c_float, ctypes.c_int]
        lib.jf_oracle_markstein_sweep_mantissas.restype = i64
        for f in (lib.jf_oracle_gemm_accumulate, lib.jf_oracle_gemm_int32, lib.jf_oracle_requant,
                  lib.jf_oracle_to_half, lib.jf_oracle_sum_partials):
            f.restype = None
        _clib = lib
    return _clib


def set_threads(n):
    """Number of OpenMP threads of the C part (launchers like torchrun export OMP_NUM_THREADS=1); returns the value in effect."""
    _c().jf_oracle_set_threads(int(n))
    return int(_c().jf_oracle_max_threads())


def markstein_mismatches(a, b):
    """How many of the quotients a[i] / b[i] the CUDA kernels' exact-division sequence gets wrong (expected: none)."""
    a = np.ascontiguousarray(a, dtype=f32)
    b = np.ascontiguousarray(b, dtype=f32)
    assert a.shape == b.shape
    return int(_c().jf_oracle_markstein_mismatches(_ptr(a), _ptr(b), a.size))


def markstein_sweep_mantissas(b, e=0):
    """Mismatches over all 2^23 dividend mantissas (times 2^e) for the divisor b."""
    return int(_c().jf_oracle_markstein_sweep_mantissas(float(np.float32(b)), int(e)))


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _strides(a):
    return [s // a.itemsize for s in a.strides]


# --------------------------------------------------------------------------------------------
# Philox4x32-10 counter-based generator (the published Random123 algorithm) and the SR noise map
# --------------------------------------------------------------------------------------------
_PH_M0, _PH_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PH_W0, _PH_W1 = 0x9E3779B9, 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox4x32 with 10 rounds.  c* are uint32 arrays (or scalars), k* python ints."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK32 for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    for r in range(10):
        if r > 0:
            k0 = (k0 + _PH_W0) & 0xFFFFFFFF
            k1 = (k1 + _PH_W1) & 0xFFFFFFFF
        p0 = _PH_M0 * c0
        p1 = _PH_M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ np.uint64(k0)), lo1, (hi0 ^ c3 ^ np.uint64(k1)), lo0
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


def sr_noise(M, N, seed, offset):
    """Noise in [-0.5, 0.5) for element (row, col) of an [M, N] tensor, as the CUDA kernels generate it.

    One Philox4x32-10 call serves 8 consecutive elements: group g = e // 8 of element e = row*N + col, key = (seed_lo, seed_hi),
    counter = (g_lo, g_hi, offset_lo, offset_hi); element e takes the 16-bit half (e & 1) of word (e >> 1) & 3 and
    noise = h * 2**-16 - 0.5 (a multiple of 2**-16, exact in fp32).
    """
    total = M * N
    g = np.arange((total + 7) // 8, dtype=np.uint64)
    w = philox4x32_10(g & _MASK32, g >> np.uint64(32), np.uint64(offset & 0xFFFFFFFF),
                      np.uint64((offset >> 32) & 0xFFFFFFFF), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    words = np.stack(w, axis=1)                                   # [groups, 4]
    halves = np.stack([words & np.uint32(0xFFFF), words >> np.uint32(16)], axis=2).reshape(-1)[:total]
    return (halves.astype(np.float64) * 2.0 ** -16 - 0.5).astype(f32).reshape(M, N)


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
def _blk(a):
    M, N = a.shape
    return a.reshape(M // QB, QB, N // QB, QB)


def _unblk(a):
    return a.reshape(a.shape[0] * QB, a.shape[2] * QB)


def _bc(s):
    return s[:, None, :, None]


def _amax(y):
    return np.abs(_blk(y)).max(axis=(1, 3)).astype(f32)


def _sr(v, noise):
    """Jetfire/Nonlinear/quantize.py:119-126: sign * clamp(|v| + noise, -128, 127)."""
    sign = (1 - 2 * np.signbit(v).astype(np.int32)).astype(f32)
    mag = (np.abs(v) + noise).astype(f32)
    return (sign * np.clip(mag, f32(-128), f32(127))).astype(f32)


def _to_int8_rne(v):
    """libdevice.llrint then .to(int8): round-half-even, NaN -> 0, wrap like a narrowing cast."""
    with np.errstate(invalid="ignore"):
        r = np.rint(v)
        r = np.where(np.isnan(r), 0, r)
        return r.astype(np.int64).astype(np.int8)


def _to_int8_trunc(v):
    """A plain float -> int8 cast (truncation toward zero), Jetfire/Nonlinear/add.py:139."""
    with np.errstate(invalid="ignore"):
        r = np.trunc(v)
        r = np.where(np.isnan(r), 0, r)
        return r.astype(np.int64).astype(np.int8)


def _div(a, b):
    with np.errstate(invalid="ignore", divide="ignore"):
        return (a / b).astype(f32)


def _exp32(x):
    """Correctly rounded fp32 exponential (evaluated in fp64, rounded once).  numpy's own float32 exp is a SIMD
    approximation whose last bit depends on the host CPU; the oracle must not."""
    return np.exp(np.asarray(x, dtype=np.float64)).astype(f32)


def _erf32(x):
    """Correctly rounded fp32 error function (fp64 evaluation rounded once; scipy's float32 loop does the same)."""
    return scipy.special.erf(np.asarray(x, dtype=np.float64)).astype(f32)


def _as2d(x):
    x = np.asarray(x)
    return x.reshape(-1, x.shape[-1])


# --------------------------------------------------------------------------------------------
# nonlinear operators
# --------------------------------------------------------------------------------------------
def int8_quantize(x, noise=None):
    """Jetfire/Nonlinear/quantize.py:33-117.  fp32 math; quantises with the fp32 scale amax/127, stores it as fp16."""
    x = _as2d(x).astype(f32)
    s32 = (_amax(x) / f32(127.0)).astype(f32)
    v = _unblk(_div(_blk(x), _bc(s32)))
    if noise is not None:
        v = _sr(v, noise.astype(f32))
    return _to_int8_rne(v), s32.astype(f16)


def int8_quantize_transpose(x, noise=None):
    """Jetfire/Nonlinear/quantize_transpose.py:33-129: quantize and also return q^T."""
    q, s = int8_quantize(x, noise)
    return q, s, np.ascontiguousarray(q.T)


def int8_transpose(q):
    """Jetfire/Nonlinear/transpose.py:29-67."""
    return np.ascontiguousarray(_as2d(q).T)


def _deq16(q, s):
    """int8 * fp16 -> fp16 product (Jetfire/Nonlinear/gelu_fwd.py:78, layernorm.py:131, dequantize.py:70)."""
    return _unblk((_blk(q).astype(f32) * _bc(s.astype(f32))).astype(f16))


def _deq32(q, s):
    """fp32 product (Jetfire/Nonlinear/gelu_bwd.py:101-102, add.py:89-95)."""
    return _unblk((_blk(q).astype(f32) * _bc(s.astype(f32))).astype(f32))


def int8_dequantize(q, s):
    """Jetfire/Nonlinear/dequantize.py:28-84: fp16 product widened to fp32."""
    return _deq16(_as2d(q), _as2d(s)).astype(f32)


def int8_gelu_forward(q, s):
    """Jetfire/Nonlinear/gelu_fwd.py:34-126: fp16 dequant, erf GELU in fp32, amax + 5e-5, IEEE divide, RNE."""
    x = _deq16(_as2d(q), _as2d(s)).astype(f32)
    sqrt2 = np.sqrt(f32(2.0))
    cdf = ((f32(1.0) + _erf32((x / sqrt2).astype(f32))) / f32(2.0)).astype(f32)
    y = (cdf * x).astype(f32)
    amax = (_amax(y) + f32(5e-5)).astype(f32)
    sc = (amax / f32(127.0)).astype(f32)
    return _to_int8_rne(_unblk(_div(_blk(y), _bc(sc)))), sc.astype(f16)


def int8_gelu_backward(qx, sx, qg, sg, noise=None):
    """Jetfire/Nonlinear/gelu_bwd.py:28-171: fp32 dequant, dgelu = Phi(x) + x*phi(x), quantise (+SR)."""
    x = _deq32(_as2d(qx), _as2d(sx))
    g = _deq32(_as2d(qg), _as2d(sg))
    sqrt2 = np.sqrt(f32(2.0))
    cdf = (f32(0.5) * (f32(1.0) + _erf32((x / sqrt2).astype(f32)))).astype(f32)
    sqrt2pi = np.sqrt(f32(2 * 3.141592653589793))
    e = _exp32((-(x * x).astype(f32) / f32(2.0)).astype(f32))
    ex = ((x / f32(sqrt2pi)).astype(f32) * e).astype(f32)
    d = ((cdf + ex).astype(f32) * g).astype(f32)
    sc = (_amax(d) / f32(127.0)).astype(f32)
    v = _unblk(_div(_blk(d), _bc(sc)))
    if noise is not None:
        v = _sr(v, noise.astype(f32))
    return _to_int8_rne(v), sc.astype(f16)


def int8_layernorm_forward(q, s, gamma, mean, rstd):
    """Jetfire/Nonlinear/layernorm.py:74-190 (wrapper :430-465): statistics are inputs, bias is zero, eps unused."""
    x = _deq16(_as2d(q), _as2d(s)).astype(f32)
    xhat = ((x - mean.astype(f32)[:, None]).astype(f32) * rstd.astype(f32)[:, None]).astype(f32)
    y = ((xhat * gamma.astype(f32)[None, :]).astype(f32) + f32(0.0)).astype(f32)
    sc = (_amax(y) / f32(127.0)).astype(f32)
    return _to_int8_rne(_unblk(_div(_blk(y), _bc(sc)))), sc.astype(f16)


def _seq_sum_last(a):
    """((a0 + a1) + a2) + ... along the last axis, one fp32 rounding per step."""
    acc = a[..., 0].astype(f32)
    for j in range(1, a.shape[-1]):
        acc = (acc + a[..., j]).astype(f32)
    return acc


def _tree8(a):
    """((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7)) along the last axis (length 8), fp32."""
    p = (a[..., 0::2] + a[..., 1::2]).astype(f32)
    p = (p[..., 0::2] + p[..., 1::2]).astype(f32)
    return (p[..., 0] + p[..., 1]).astype(f32)


def _slab_sums(a, slab, order):
    """Row sums of a [M, nsl*slab] fp32 array over each slab.  order="numpy": numpy's pairwise summation (what the Triton
    interpreter, and therefore the golden vectors, use); order="kernel": the CUDA kernel's order -- each 16-column chunk summed
    left to right, the eight chunks of a 128-column slab combined as a balanced tree (the reference's GPU lowering of tl.sum
    is a shuffle tree as well; the reference itself leaves the order undefined)."""
    M = a.shape[0]
    nsl = a.shape[1] // slab
    if order == "numpy":
        return a.reshape(M, nsl, slab).sum(-1, dtype=f32)
    assert slab == 128, "the kernel order is defined for the reference's 128-column slab"
    return _tree8(_seq_sum_last(a.reshape(M, nsl, 8, 16)))


def int8_layernorm_backward(qx, sx, qg, sg, gamma, mean, rstd, noise=None, slab=128, dw_accum="fp16", order="numpy"):
    """Jetfire/Nonlinear/layernorm.py:197-428 (wrapper :467-526).

    Rounding points of the reference: mean, rstd -> fp16; x and dy dequantised in fp16; xhat in fp16;
    wdy = gamma*dy, c1, c2 in fp32 with the row sums taken over each `slab`-column slab only but divided
    by the full N; dx -> fp16; scale = fp32(amax16)/127 and quotient in fp32; dgamma partials per 32 rows
    summed in fp16 (dw_accum="fp16") then across partials in fp32.  slab=None sums over the row.

    The ORDER of the 128-term fp32 row sums and of the dgamma column sums is not defined by the reference (tree reductions
    whose shape the compiler picks).  order="numpy" is the order of the Triton interpreter that produced the golden vectors
    (bit-exact against them); order="kernel" is the CUDA kernel's documented order and, with dw_accum="kernel", makes the
    whole operator bit-comparable with the GPU.  Every other rounding point is identical in the two modes.
    Returns (qdx, sdx, dgamma)."""
    qx, sx, qg, sg = _as2d(qx), _as2d(sx), _as2d(qg), _as2d(sg)
    M, N = qx.shape
    slab = N if slab is None else slab
    m16 = mean.astype(f32).astype(f16)[:, None]
    r16 = rstd.astype(f32).astype(f16)[:, None]
    x = _deq16(qx, sx)
    dy = _deq16(qg, sg)
    xhat = ((x - m16).astype(f16) * r16).astype(f16)
    wdy = (gamma.astype(f32)[None, :] * dy.astype(f32)).astype(f32)
    xw = (xhat.astype(f32) * wdy).astype(f32)
    # The reference needs N % 128 == 0 (layernorm.py:482, 515); for other N (multiples of 32, e.g. GPT-2 XL's 1600) the last
    # slab is simply shorter -- modelled by zero padding, which does not change the sums.
    nsl = -(-N // slab)
    pad = nsl * slab - N
    c1 = (_slab_sums(np.pad(xw, ((0, 0), (0, pad))), slab, order) / f32(N)).astype(f32)
    c2 = (_slab_sums(np.pad(wdy, ((0, 0), (0, pad))), slab, order) / f32(N)).astype(f32)
    c1 = np.repeat(c1, slab, axis=1)[:, :N]
    c2 = np.repeat(c2, slab, axis=1)[:, :N]
    t = ((xhat.astype(f32) * c1).astype(f32) + c2).astype(f32)
    dx = (((wdy - t).astype(f32)) * r16.astype(f32)).astype(f32).astype(f16)
    amax16 = np.abs(_blk(dx)).max(axis=(1, 3))
    sc32 = (amax16.astype(f32) / f32(127.0)).astype(f32)   # a division involving fp16 is carried out in fp32
    v = _unblk(_div(_blk(dx).astype(f32), _bc(sc32)))
    if noise is not None:
        v = _sr(v, noise.astype(f32))
    qd = _to_int8_rne(v)
    prod = (dy * xhat).astype(f16)
    if dw_accum == "fp16":   # reference-faithful: each 32-row partial is summed in fp16, partials in fp32
        dw = prod.reshape(M // QB, QB, N).sum(1, dtype=f16).astype(f32).sum(0, dtype=f32)
    elif dw_accum == "kernel":
        # the CUDA kernel: fp32 sums of the fp16 products.  Inside a 32-row tile a lane owns rows rg, rg+8, rg+16, rg+24
        # (summed in that order), the eight lanes are combined as a balanced tree; the M/32 partial rows are then summed by
        # eight interleaved groups (rows g, g+8, ...) left to right, and the eight group sums left to right.
        p32 = prod.astype(f32).reshape(M // QB, 4, 8, N)                       # [tile, pass, rg, col]
        lane = _seq_sum_last(np.moveaxis(p32, 1, -1))                           # [tile, rg, col]
        part = _tree8(np.moveaxis(lane, 1, -1))                                 # [tile, col]
        rows = part.shape[0]
        grp = np.zeros((8, N), f32)
        for r in range(rows):
            grp[r % 8] = (grp[r % 8] + part[r]).astype(f32)
        dw = _seq_sum_last(np.ascontiguousarray(grp.T))
    else:                    # plain fp32 accumulation of the fp16 products, numpy order
        dw = prod.astype(f32).reshape(M // QB, QB, N).sum(1, dtype=f32).sum(0, dtype=f32)
    return qd, sc32.astype(f16), dw


def int8_add(x1, q2, s2, noise=None):
    """Jetfire/Nonlinear/add.py:29-162: y = x1 + q2*s2 in fp32; stores fp32 y, and q(y) by *truncation*."""
    x1 = _as2d(x1).astype(f32)
    y = (x1 + _deq32(_as2d(q2), _as2d(s2))).astype(f32)
    sc = (_amax(y) / f32(127.0)).astype(f32)
    v = _unblk(_div(_blk(y), _bc(sc)))
    if noise is not None:
        v = _sr(v, noise.astype(f32))
    return y, _to_int8_trunc(v), sc.astype(f16)


def int8_add_meanvar(x1, q2, s2):
    """Jetfire/Nonlinear/add_mean_var.py:28-231: add (no SR) plus row mean and rstd = 1/sqrt(E[y^2] - mean^2)
    of the fp32 sum (biased variance, no eps).  The reference sums 64-column partials then the partials; the
    summation order is not part of the contract (fp tolerance)."""
    y, q, sc = int8_add(x1, q2, s2)
    N = y.shape[1]
    w = 64 if N % 64 == 0 else 32          # the reference only runs at N % 64 == 0
    part = y.reshape(y.shape[0], N // w, w)
    mean = (part.sum(-1, dtype=f32).sum(-1, dtype=f32) / f32(N)).astype(f32)
    sq = ((part * part).astype(f32).sum(-1, dtype=f32).sum(-1, dtype=f32) / f32(N)).astype(f32)
    var = (sq - (mean * mean).astype(f32)).astype(f32)
    with np.errstate(invalid="ignore", divide="ignore"):
        rstd = (f32(1.0) / np.sqrt(var)).astype(f32)
    return y, q, sc, mean, rstd


# --------------------------------------------------------------------------------------------
# GEMMs (C implementation)
# --------------------------------------------------------------------------------------------
def gemm_int32(A, B_nk):
    """Plain int8 x int8 -> int32 product A[M,K] * B[N,K]^T."""
    A = np.asarray(A)
    B = np.asarray(B_nk)
    M, K = A.shape
    N = B.shape[0]
    C = np.empty((M, N), np.int32)
    (am, ak), (bn, bk) = _strides(A), _strides(B)
    _c().jf_oracle_gemm_int32(_ptr(A), am, ak, _ptr(B), bn, bk, _ptr(C), M, N, K)
    return C


def gemm_accumulate(A_mk, B_nk, SA_ip, SB_jp, acc=None, p_begin=0, p_end=None):
    """fp32 accumulator of the per-block GEMM.  A_mk / B_nk / SA_ip / SB_jp may be arbitrary strided views
    (pass X.T etc. to express the dgrad / wgrad layouts without copies)."""
    M, K = A_mk.shape
    N = B_nk.shape[0]
    assert B_nk.shape[1] == K and SA_ip.shape == (M // QB, K // QB) and SB_jp.shape == (N // QB, K // QB)
    assert A_mk.dtype == np.int8 and B_nk.dtype == np.int8 and SA_ip.dtype == f16 and SB_jp.dtype == f16
    if acc is None:
        acc = np.zeros((M, N), f32)
    p_end = K // QB if p_end is None else p_end
    (am, ak), (bn, bk), (si, sp), (sj, sq) = _strides(A_mk), _strides(B_nk), _strides(SA_ip), _strides(SB_jp)
    _c().jf_oracle_gemm_accumulate(_ptr(A_mk), am, ak, _ptr(B_nk), bn, bk, _ptr(SA_ip), si, sp, _ptr(SB_jp), sj, sq,
                                   _ptr(acc), M, N, K, p_begin, p_end)
    return acc


def requant(acc, noise=None, dequantized=False):
    M, N = acc.shape
    q = np.empty((M, N), np.int8)
    s = np.empty((M // QB, N // QB), f16)
    deq = np.empty((M, N), f16) if dequantized else None
    nz = None if noise is None else np.ascontiguousarray(noise, dtype=f32)
    _c().jf_oracle_requant(_ptr(np.ascontiguousarray(acc)), M, N, _ptr(nz), _ptr(q), _ptr(s), _ptr(deq))
    return (q, s, deq) if dequantized else (q, s)


def linear_forward(X8, SX, W8, SW, dequantized=False):
    """Y = X W^T.  Jetfire/Linear/linear_fwd.py:4-32 + igemm_output_int_quantize_bias_rowcol (bias = 0).
    X8 [M,K], SX [M/32,K/32], W8 [N,K], SW [N/32,K/32]."""
    return requant(gemm_accumulate(X8, W8, SX, SW), None, dequantized)


def linear_dgrad(G8, SG, W8, SW, noise=None, dequantized=False):
    """dX = dY W.  Jetfire/Linear/linear_bwd.py:17 + igemm_output_int_quantize_stochastic.
    G8 [M,Cout], SG [M/32,Cout/32], W8 [Cout,Cin], SW [Cout/32,Cin/32]."""
    return requant(gemm_accumulate(G8, W8.T, SG, SW.T), noise, dequantized)


def linear_wgrad(G8, SG, X8, SX, split_k=1, out_dtype=f16):
    """dW = dY^T X.  Jetfire/Linear/linear_bwd.py:19 + igemm_output_fp_no_quantize (fp16 dense output).
    G8 [T,Cout], SG [T/32,Cout/32], X8 [T,Cin], SX [T/32,Cin/32].  split_k > 1 models the deterministic
    split-K of the CUDA kernel: K blocks are cut into `split_k` contiguous ranges of ceil(nb/split_k) blocks,
    each accumulated from zero, then summed in ascending order."""
    T = G8.shape[0]
    nb = T // QB
    if split_k <= 1:
        acc = gemm_accumulate(G8.T, X8.T, SG.T, SX.T)
    else:
        per = (nb + split_k - 1) // split_k
        parts = []
        for k in range(split_k):
            b, e = k * per, min(nb, (k + 1) * per)
            if b >= e:
                break
            parts.append(gemm_accumulate(G8.T, X8.T, SG.T, SX.T, None, b, e))
        stack = np.ascontiguousarray(np.stack(parts))
        acc = np.empty_like(parts[0])
        _c().jf_oracle_sum_partials(_ptr(stack), len(parts), acc.size, _ptr(acc))
    if out_dtype == f32:
        return acc
    out = np.empty(acc.shape, f16)
    _c().jf_oracle_to_half(_ptr(np.ascontiguousarray(acc)), acc.size, _ptr(out))
    return out
