"""Test infrastructure: the reference's INT8 recipe restated with plain torch tensor operations (any device).

Each function has the name, arguments and return convention of the operator it stands for (the reference's
Jetfire/Nonlinear/*.py and Jetfire/Linear/*.py), so that `gpt2.QGPT` can be run on it by swapping the two operator modules.
It is the "reference INT8 recipe" side of the end-to-end loss-curve comparison (pinned to the golden vectors of the reference's
own kernels by tests/test_recipe_golden.py; `noise=` injects a given rounding-noise tensor for that purpose): same quantisation points, same block size,
same truncation / rounding rules, stochastic rounding from torch's generator (the reference draws torch.uniform_ noise too,
Jetfire/Nonlinear/quantize.py:143-144).  The GEMMs are evaluated on the dequantised operands in fp64 and rounded to fp32, i.e.
with exact per-block integer products and an accumulation at least as accurate as the reference's fp32 one.
Never imported by the package.
"""
import math

import torch

QB = 32


def _blocks(x):
    M, N = x.shape
    return x.reshape(M // QB, QB, N // QB, QB)


def _flat(x):
    if x.dim() == 2:
        return x, None
    return x.reshape(-1, x.shape[-1]), x.shape[0]


def _unflat(y, bs):
    return y if bs is None else y.reshape(bs, -1, y.shape[-1])


def _quant(y, stochastic, trunc=False, amax_adj=0.0, noise=None):
    """fp32 [M,N] -> (int8 payload, fp16 scales): quantize.py:73-96 (+ _stochastic_rounding :119-126); add.py:139 truncates."""
    y = y.float()
    b = _blocks(y)
    amax = b.abs().amax(dim=(1, 3), keepdim=True) + amax_adj
    scale = amax / 127.0
    v = torch.where(scale > 0, b / scale, torch.zeros_like(b))
    if stochastic:
        noise = (torch.rand_like(v) - 0.5) if noise is None else _blocks(noise.float())
        v = torch.sign(v) * torch.clamp(v.abs() + noise, max=127.0)
    q = torch.trunc(v) if trunc else torch.round(v)
    q = q.clamp(-127, 127).to(torch.int8).reshape(y.shape)
    return q, scale.reshape(y.shape[0] // QB, y.shape[1] // QB).half()


def _deq(q, s, half_product=False):
    """payload * block scale; half_product: the product is formed in fp16 (gelu_fwd.py:78, layernorm.py:131, dequantize.py:70-72)."""
    q = q.view(torch.int8) if q.dtype != torch.int8 else q
    b = _blocks(q.float())
    sc = s.float().reshape(s.shape[0], 1, s.shape[1], 1)
    if half_product:
        return (b.half() * sc.half()).float().reshape(q.shape)
    return (b * sc).reshape(q.shape)


# ------------------------------------------------------------------------------------------------ Nonlinear
def int8_quantize(x, B, stochastic=False, noise=None):
    x2, bs = _flat(x)
    q, s = _quant(x2, stochastic, noise=noise)
    return _unflat(q, bs), _unflat(s, bs)


def int8_quantize_many(tensors, B):
    """The weight quantisations of one step, one after the other (the package does them eight per launch)."""
    return [int8_quantize(t, B) for t in tensors]


def int8_gelu_forward(x, s_x, B):
    x2, bs = _flat(x); s2, _ = _flat(s_x)
    v = _deq(x2, s2, half_product=True)
    y = v * 0.5 * (1.0 + torch.erf(v * 0.7071067811865476))          # gelu_fwd.py:81-82
    q, s = _quant(y, False, amax_adj=5e-5)                            # gelu_fwd.py:90
    return _unflat(q, bs), _unflat(s, bs)


def int8_gelu_backward(x, s_x, g, s_g, B, stochastic=False, noise=None):
    x2, bs = _flat(x); sx2, _ = _flat(s_x); g2, _ = _flat(g); sg2, _ = _flat(s_g)
    v, gv = _deq(x2, sx2), _deq(g2, sg2)
    cdf = 0.5 * (1.0 + torch.erf(v * 0.7071067811865476))
    pdf = torch.exp(-0.5 * v * v) * 0.3989422804014327
    q, s = _quant((cdf + v * pdf) * gv, stochastic, noise=noise)      # gelu_bwd.py:101-107
    return _unflat(q, bs), _unflat(s, bs)


def int8_layernorm_forward(x, sx, weight, mean, rstd, B, eps=1e-6):
    x2, bs = _flat(x); s2, _ = _flat(sx)
    v = _deq(x2, s2, half_product=True)
    y = (v - mean.reshape(-1, 1).float()) * rstd.reshape(-1, 1).float() * weight.float()      # layernorm.py:131-140
    q, s = _quant(y, False)
    return _unflat(q, bs), _unflat(s, bs), (mean, rstd)


def int8_layernorm_backward(x, sx, g, sg, w, B, m, v, stochastic=False, eps=1e-6, noise=None):
    """layernorm.py:310-336: statistics, x, dy and xhat in fp16; row sums over the 128-column slab divided by N; dx -> fp16."""
    x2, bs = _flat(x); sx2, _ = _flat(sx); g2, _ = _flat(g); sg2, _ = _flat(sg)
    M, N = x2.shape
    mu = m.reshape(-1, 1).half(); rs = v.reshape(-1, 1).half()
    xv = _deq(x2, sx2, half_product=True).half()
    dy = _deq(g2, sg2, half_product=True).half()
    xhat = ((xv - mu) * rs).float()
    wdy = w.float() * dy.float()
    slab = 128
    pad = (-N) % slab
    padded = lambda a: torch.nn.functional.pad(a, (0, pad)).reshape(M, -1, slab)      # a shorter last slab = zero padding
    c1 = padded(xhat * wdy).sum(-1, keepdim=True) / N
    c2 = padded(wdy).sum(-1, keepdim=True) / N
    dx = ((padded(wdy) - (padded(xhat) * c1 + c2)) * rs.float().reshape(M, 1, 1)).reshape(M, -1)[:, :N]
    dx = dx.half().float()
    dw = (dy.float() * xhat).sum(0)
    q, s = _quant(dx, stochastic, noise=noise)
    return _unflat(q, bs), _unflat(s, bs), dw.to(w.dtype)


def int8_add_Ifp_Ig16_Ofp_Og(x1, x2, s_x2, B, stochastic=False, noise=None):
    a, bs = _flat(x1); q2, _ = _flat(x2); s2, _ = _flat(s_x2)
    y = a.float() + _deq(q2, s2)                                       # add.py:120-139 (truncating cast)
    q, s = _quant(y, stochastic, trunc=True, noise=noise)
    return _unflat(y, bs), _unflat(q, bs), _unflat(s, bs)


def int8_add_Ifp_Ig16_Ofp_Og_MeanVar(x1, x2, s_x2, B):
    a, bs = _flat(x1); q2, _ = _flat(x2); s2, _ = _flat(s_x2)
    y = a.float() + _deq(q2, s2)
    q, s = _quant(y, False, trunc=True)
    N = y.shape[1]
    mean = y.sum(1) / N
    var = (y * y).sum(1) / N - mean * mean                              # add_mean_var.py:219-221 (biased, no eps)
    rstd = 1.0 / torch.sqrt(var)
    lead = x1.shape[:-1]
    return _unflat(y, bs), _unflat(q, bs), _unflat(s, bs), mean.reshape(lead), rstd.reshape(lead)


# ------------------------------------------------------------------------------------------------ Linear
def int8_linear_forward(X8_3D, SX16_3D, W8, SW16, output_quantized, B):
    x2, bs = _flat(X8_3D); sx2, _ = _flat(SX16_3D)
    y = (_deq(x2, sx2).double() @ _deq(W8, SW16).double().t()).float()      # linear_fwd.py:4-32
    q, s = _quant(y, False)
    if output_quantized:
        return _unflat(q, bs), _unflat(s, bs)
    # linear_fwd.py:30: the quantised output is dequantised again (int8 * fp16 scale, a product in fp16), not the raw accumulator
    return _unflat(_deq(q, s, half_product=True).half(), bs)


def int8_linear_backward(X8_3D, SX16_3D, G8_3D, SG16_3D, G8T, W8, SW16, B, stochastic=True, dgrad_quantize=True, *,
                         wgrad_out_dtype=torch.float16, **_):
    x2, bs = _flat(X8_3D); sx2, _ = _flat(SX16_3D); g2, _ = _flat(G8_3D); sg2, _ = _flat(SG16_3D)
    gd, xd, wd = _deq(g2, sg2).double(), _deq(x2, sx2).double(), _deq(W8, SW16).double()
    gx = (gd @ wd).float()                                               # linear_bwd.py:17
    gw = (gd.t() @ xd).float().to(wgrad_out_dtype)                       # linear_bwd.py:19
    q, s = _quant(gx, True)                                              # the reference's dgrad kernel always rounds stochastically
    if dgrad_quantize:
        return _unflat(q, bs), _unflat(s, bs), gw
    return _unflat(_deq(q, s, half_product=True).half(), bs), gw         # linear_bwd.py:27: dequantised again, fp16 product
