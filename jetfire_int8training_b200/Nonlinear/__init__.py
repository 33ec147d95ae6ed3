"""INT8-in / INT8-out nonlinear operators with the reference's names, signatures and return conventions
(Jetfire/Nonlinear/__init__.py:1-8 of thu-ml/Jetfire-INT8Training), executed by hand-written sm_100a kernels
through the C ABI in include/jetfire_b200.h.

Conventions kept from the reference: tensors are CUDA tensors, 2-D or 3-D (3-D inputs are flattened over the leading
dimensions and outputs get the leading batch dimension back); outputs are freshly allocated; everything runs on the
current stream; QB must be 32.

Extras not in the reference (keyword-only): `noise=` feeds an explicit fp32 noise tensor to a stochastic operator
(used to reproduce the reference's rounding bit for bit), `sr_key=(seed, offset)` pins the Philox key of one call.
`set_sr_noise("torch")` makes every stochastic operator draw its noise the way the reference does -- one fp32 tensor
`uniform_(-0.5, 0.5)` per call from torch's CUDA generator (Jetfire/Nonlinear/quantize.py:143-144, gelu_bwd.py:192,
layernorm.py:493, add.py:185) -- so that a run seeded with `torch.manual_seed` rounds exactly like the reference run with the
same seed, at the price of writing and reading 4 bytes of noise per element; the default "philox" generates 16 noise bits per
element inside the kernel.
"""
import torch

from .. import rng
from .._lib import lib, check

__all__ = [
    "int8_quantize", "int8_quantize_many", "int8_quantize_transpose", "int8_transpose", "int8_dequantize",
    "int8_gelu_forward", "int8_gelu_backward", "int8_layernorm_forward", "int8_layernorm_backward",
    "int8_add_Ifp_Ig16_Ofp_Og", "int8_add_Ifp_Ig16_Ofp_Og_MeanVar", "set_sr_noise",
]

_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
TILE_N = 128
_SR_NOISE = "philox"


def set_sr_noise(mode):
    """"philox": in-kernel Philox4x32-10 keyed by rng.next_key() (default).  "torch": the reference's noise stream."""
    global _SR_NOISE
    if mode not in ("philox", "torch"):
        raise ValueError("sr noise mode is 'philox' or 'torch'")
    previous, _SR_NOISE = _SR_NOISE, mode
    return previous


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("jetfire_int8training_b200 operators need CUDA tensors (there is no CPU path)")


def _qb(QB):
    if QB != 32:
        raise ValueError("only the 32x32 quantisation block of the reference recipe is implemented")


def _flat(x):
    """(2-D view, batch or None): the reference's 3-D -> 2-D convention."""
    if x.dim() == 2:
        return x.contiguous(), None
    return x.reshape(-1, x.shape[-1]).contiguous(), x.shape[0]


def _unflat(y, bs):
    return y if bs is None else y.reshape(bs, -1, y.shape[-1])


def _p(t):
    return None if t is None else t.data_ptr()


def _sr_args(stochastic, noise, sr_key, like):
    if not stochastic:
        return 0, None, 0, 0, None
    if noise is not None:
        noise = noise.reshape(like.shape).to(device=like.device, dtype=torch.float32).contiguous()
        return 1, noise.data_ptr(), 0, 0, noise
    if sr_key is None and _SR_NOISE == "torch":
        noise = torch.empty(like.shape, dtype=torch.float32, device=like.device).uniform_(-0.5, 0.5)
        return 1, noise.data_ptr(), 0, 0, noise
    seed, offset = sr_key if sr_key is not None else rng.next_key()
    return 1, None, seed, offset, None


def _as_i8(t):
    return t.view(torch.int8) if t.dtype != torch.int8 else t


def int8_quantize(x, QB, stochastic=False, *, noise=None, sr_key=None):
    """Jetfire/Nonlinear/quantize.py:128-164.  Returns (q int8, scale fp16)."""
    _qb(QB); _need_cuda(x)
    x2, bs = _flat(x)
    if x2.dtype not in _DTYPE:
        x2 = x2.float()
    M, N = x2.shape
    q = torch.empty((M, N), dtype=torch.int8, device=x.device)
    s = torch.empty((M // 32, N // 32), dtype=torch.float16, device=x.device)
    st, nz, seed, off, keep = _sr_args(stochastic, noise, sr_key, x2)
    check(lib().jf_int8_quantize(x2.data_ptr(), _DTYPE[x2.dtype], M, N, q.data_ptr(), s.data_ptr(), None, st, nz, seed, off,
                                 _stream()), "int8_quantize")
    return _unflat(q, bs), _unflat(s, bs)


def int8_quantize_many(tensors, QB):
    """Round-to-nearest int8_quantize of several 2-D tensors (same dtype and device) with one kernel launch per 8 tensors: the
    weight matrices that the reference quantises one by one at the start of every forward pass (INT8_GPT2/qmodel.py:92, 139,
    199-200).  Returns [(q, scale), ...], bit-identical to int8_quantize on each tensor."""
    import ctypes
    _qb(QB)
    tensors = [t if t.dtype in _DTYPE else t.float() for t in tensors]
    _need_cuda(*tensors)
    assert all(t.dim() == 2 and t.dtype == tensors[0].dtype and t.device == tensors[0].device for t in tensors)
    tensors = [t.contiguous() for t in tensors]
    outs = []
    for i in range(0, len(tensors), 8):
        grp = tensors[i:i + 8]
        n = len(grp)
        qs = [torch.empty(t.shape, dtype=torch.int8, device=t.device) for t in grp]
        ss = [torch.empty((t.shape[0] // 32, t.shape[1] // 32), dtype=torch.float16, device=t.device) for t in grp]
        vp, i64 = ctypes.c_void_p * n, ctypes.c_int64 * n
        check(lib().jf_int8_quantize_multi(n, vp(*[t.data_ptr() for t in grp]), _DTYPE[grp[0].dtype], i64(*[t.shape[0] for t in grp]),
                                           i64(*[t.shape[1] for t in grp]), vp(*[q.data_ptr() for q in qs]),
                                           vp(*[s.data_ptr() for s in ss]), _stream()), "int8_quantize_many")
        outs += list(zip(qs, ss))
    return outs


def int8_quantize_transpose(x, QB, stochastic=False, transpose_output_2d=False, *, noise=None, sr_key=None):
    """Jetfire/Nonlinear/quantize_transpose.py:131-171.  Returns (q, scale, q^T)."""
    _qb(QB); _need_cuda(x)
    x2, bs = _flat(x)
    if x2.dtype not in _DTYPE:
        x2 = x2.float()
    M, N = x2.shape
    q = torch.empty((M, N), dtype=torch.int8, device=x.device)
    s = torch.empty((M // 32, N // 32), dtype=torch.float16, device=x.device)
    qt = torch.empty((N, M), dtype=torch.int8, device=x.device)
    st, nz, seed, off, keep = _sr_args(stochastic, noise, sr_key, x2)
    check(lib().jf_int8_quantize(x2.data_ptr(), _DTYPE[x2.dtype], M, N, q.data_ptr(), s.data_ptr(), qt.data_ptr(), st, nz, seed,
                                 off, _stream()), "int8_quantize_transpose")
    if bs is not None and not transpose_output_2d:
        qt = qt.reshape(bs, -1, qt.shape[-1])
    return _unflat(q, bs), _unflat(s, bs), qt


def int8_transpose(x, transpose_output_2d=False):
    """Jetfire/Nonlinear/transpose.py:69-97."""
    _need_cuda(x)
    x2, bs = _flat(_as_i8(x))
    M, N = x2.shape
    y = torch.empty((N, M), dtype=torch.int8, device=x.device)
    check(lib().jf_int8_transpose(x2.data_ptr(), M, N, y.data_ptr(), _stream()), "int8_transpose")
    if bs is not None and not transpose_output_2d:
        y = y.reshape(bs, -1, y.shape[-1])
    return y


def int8_dequantize(x, s_x, QB):
    """Jetfire/Nonlinear/dequantize.py:86-116.  Returns fp32."""
    _qb(QB); _need_cuda(x, s_x)
    x2, bs = _flat(_as_i8(x))
    s2, _ = _flat(s_x)
    M, N = x2.shape
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    check(lib().jf_int8_dequantize(x2.data_ptr(), s2.data_ptr(), M, N, y.data_ptr(), _stream()), "int8_dequantize")
    return _unflat(y, bs)


def int8_gelu_forward(x, s_x, QB):
    """Jetfire/Nonlinear/gelu_fwd.py:128-162."""
    _qb(QB); _need_cuda(x, s_x)
    x2, bs = _flat(_as_i8(x))
    s2, _ = _flat(s_x)
    M, N = x2.shape
    y = torch.empty_like(x2)
    sy = torch.empty_like(s2, dtype=torch.float16)
    check(lib().jf_int8_gelu_forward(x2.data_ptr(), s2.data_ptr(), M, N, y.data_ptr(), sy.data_ptr(), _stream()),
          "int8_gelu_forward")
    return _unflat(y, bs), _unflat(sy, bs)


def int8_gelu_backward(x, s_x, g, s_g, QB, stochastic=False, *, noise=None, sr_key=None):
    """Jetfire/Nonlinear/gelu_bwd.py:173-215."""
    _qb(QB); _need_cuda(x, s_x, g, s_g)
    x2, bs = _flat(_as_i8(x))
    s2, _ = _flat(s_x)
    g2, _ = _flat(_as_i8(g))
    sg2, _ = _flat(s_g)
    M, N = x2.shape
    y = torch.empty_like(x2)
    sy = torch.empty_like(s2, dtype=torch.float16)
    st, nz, seed, off, keep = _sr_args(stochastic, noise, sr_key, x2)
    check(lib().jf_int8_gelu_backward(x2.data_ptr(), s2.data_ptr(), g2.data_ptr(), sg2.data_ptr(), M, N, y.data_ptr(),
                                      sy.data_ptr(), st, nz, seed, off, _stream()), "int8_gelu_backward")
    return _unflat(y, bs), _unflat(sy, bs)


def int8_layernorm_forward(x, sx, weight, mean, rstd, QB, eps=1e-6):
    """Jetfire/Nonlinear/layernorm.py:430-465.  mean / rstd are inputs; no bias; eps is accepted and unused,
    exactly as in the reference.  Returns (y, sy, (mean, rstd))."""
    _qb(QB); _need_cuda(x, sx, weight, mean, rstd)
    x2, bs = _flat(_as_i8(x))
    s2, _ = _flat(sx)
    M, N = x2.shape
    w = weight.detach().float().contiguous()
    mu = mean.reshape(-1).float().contiguous()
    rs = rstd.reshape(-1).float().contiguous()
    y = torch.empty_like(x2)
    sy = torch.empty_like(s2, dtype=torch.float16)
    check(lib().jf_int8_layernorm_forward(x2.data_ptr(), s2.data_ptr(), w.data_ptr(), mu.data_ptr(), rs.data_ptr(), M, N,
                                          y.data_ptr(), sy.data_ptr(), _stream()), "int8_layernorm_forward")
    return _unflat(y, bs), _unflat(sy, bs), (mean, rstd)


def int8_layernorm_backward(x, sx, g, sg, w, QB, m, v, stochastic=False, eps=1e-6, *, noise=None, sr_key=None):
    """Jetfire/Nonlinear/layernorm.py:467-526.  Returns (dx int8, sdx fp16, dw).  The two row reductions of dx are taken
    over 128-column slabs, as the reference's kernel does."""
    _qb(QB); _need_cuda(x, sx, g, sg, w, m, v)
    x2, bs = _flat(_as_i8(x))
    s2, _ = _flat(sx)
    g2, _ = _flat(_as_i8(g))
    sg2, _ = _flat(sg)
    M, N = x2.shape
    wf = w.detach().float().contiguous()
    mu = m.reshape(-1).float().contiguous()
    rs = v.reshape(-1).float().contiguous()
    dx = torch.empty((M, N), dtype=torch.int8, device=x.device)
    sdx = torch.empty((M // 32, N // 32), dtype=torch.float16, device=x.device)
    dw = torch.empty((N,), dtype=torch.float32, device=x.device)
    scratch = torch.empty(((M // 32) * N,), dtype=torch.float32, device=x.device)
    st, nz, seed, off, keep = _sr_args(stochastic, noise, sr_key, x2)
    check(lib().jf_int8_layernorm_backward(x2.data_ptr(), s2.data_ptr(), g2.data_ptr(), sg2.data_ptr(), wf.data_ptr(),
                                           mu.data_ptr(), rs.data_ptr(), M, N, TILE_N, dx.data_ptr(), sdx.data_ptr(),
                                           dw.data_ptr(), scratch.data_ptr(), st, nz, seed, off, _stream()),
          "int8_layernorm_backward")
    return _unflat(dx, bs), _unflat(sdx, bs), dw.to(w.dtype)


def int8_add_Ifp_Ig16_Ofp_Og(x1, x2, s_x2, QB, stochastic=False, *, noise=None, sr_key=None):
    """Jetfire/Nonlinear/add.py:164-211.  Returns (y1 fp32, y2 int8, s_y2 fp16)."""
    _qb(QB); _need_cuda(x1, x2, s_x2)
    a, bs = _flat(x1)
    if a.dtype not in _DTYPE:
        a = a.float()
    q2, _ = _flat(_as_i8(x2))
    s2, _ = _flat(s_x2)
    assert a.shape == q2.shape
    M, N = a.shape
    y1 = torch.empty((M, N), dtype=torch.float32, device=a.device)
    y2 = torch.empty_like(q2)
    sy = torch.empty_like(s2, dtype=torch.float16)
    st, nz, seed, off, keep = _sr_args(stochastic, noise, sr_key, a)
    check(lib().jf_int8_add(a.data_ptr(), _DTYPE[a.dtype], q2.data_ptr(), s2.data_ptr(), M, N, y1.data_ptr(), y2.data_ptr(),
                            sy.data_ptr(), st, nz, seed, off, _stream()), "int8_add_Ifp_Ig16_Ofp_Og")
    return _unflat(y1, bs), _unflat(y2, bs), _unflat(sy, bs)


def int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, x2, s_x2, QB):
    """Jetfire/Nonlinear/add_mean_var.py:179-231.  Returns (y1 fp32, y2 int8, s_y2 fp16, mean, rstd)."""
    _qb(QB); _need_cuda(x1, x2, s_x2)
    a, bs = _flat(x1)
    if a.dtype not in _DTYPE:
        a = a.float()
    q2, _ = _flat(_as_i8(x2))
    s2, _ = _flat(s_x2)
    assert a.shape == q2.shape
    M, N = a.shape
    y1 = torch.empty((M, N), dtype=torch.float32, device=a.device)
    y2 = torch.empty_like(q2)
    sy = torch.empty_like(s2, dtype=torch.float16)
    mean = torch.empty((M,), dtype=torch.float32, device=a.device)
    rstd = torch.empty((M,), dtype=torch.float32, device=a.device)
    scratch = torch.empty((2 * M * ((N + TILE_N - 1) // TILE_N),), dtype=torch.float32, device=a.device)
    check(lib().jf_int8_add_meanvar(a.data_ptr(), _DTYPE[a.dtype], q2.data_ptr(), s2.data_ptr(), M, N, y1.data_ptr(),
                                    y2.data_ptr(), sy.data_ptr(), mean.data_ptr(), rstd.data_ptr(), scratch.data_ptr(),
                                    _stream()), "int8_add_Ifp_Ig16_Ofp_Og_MeanVar")
    if bs is not None:
        mean = mean.reshape(bs, -1)
        rstd = rstd.reshape(bs, -1)
    return _unflat(y1, bs), _unflat(y2, bs), _unflat(sy, bs), mean, rstd
