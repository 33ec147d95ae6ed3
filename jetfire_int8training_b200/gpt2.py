"""GPT-2 with the Jetfire INT8 data flow, as the caller of the hot path.

This is the integration harness for the operators of this package: a nanoGPT-shaped decoder (no biases) whose linear layers,
LayerNorms, GELU and residual adds run on the per-block INT8 operators, following the data flow of the reference's quantised
model (INT8_GPT2/qmodel.py:35-362): between blocks the activations travel as (fp residual, int8 payload, fp16 block scales,
row mean, row rstd); in the backward pass the gradient travels as (fp residual gradient, int8 payload, fp16 scales) with
stochastic rounding.  int8 payloads cross autograd boundaries viewed as float8_e4m3fn, as in the reference, because autograd
only tracks floating tensors.  Attention itself (scaled-dot-product), the embedding, the final LayerNorm and the LM head stay
in floating point, as they do in the reference.

Differences from the reference's module, none of which touch the operators' semantics: weight gradients are produced in fp32
(the reference's fp16 overflows under its 2^24 loss scale), the materialised dY^T copies are not made (the GEMMs read dY
in place), and the weight matrices are quantised eight per kernel launch at the start of the forward pass.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
from torch.nn import functional as F

from . import Linear as L
from . import Nonlinear as NL
from .lm_loss import lm_cross_entropy

QB = 32
F8 = torch.float8_e4m3fn


@dataclass
class GPTConfig:
    block_size: int = 1024
    vocab_size: int = 50304
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768


def _f8(t):
    return t.view(F8)


def quantized_weight(w):
    """(int8 payload, fp16 scales) of a weight matrix for the forward pass that is running: the pair that
    quantise_weights() stored on the parameter at the start of this pass, else a fresh quantisation."""
    hit = getattr(w, "_jf_q", None)
    if hit is not None:
        return hit
    return NL.int8_quantize(w.detach(), QB)


def quantise_weights(weights, reuse=False):
    """Quantise the weight matrices of a model for one forward pass, eight tensors per kernel launch, and store the results
    where quantized_weight finds them (the reference quantises each weight where it is used, INT8_GPT2/qmodel.py:92, 139,
    199-200: 4 * n_layer launches, each smaller than one wave of the GPU at GPT-2 124M sizes).

    `reuse=True` keeps the quantisations of the previous pass.  Only the caller knows that the weights have not changed since --
    the further micro-steps of a gradient-accumulation step -- and has to say so: a parameter's version counter is NOT a safe
    key, because fused optimisers (torch.optim.AdamW(fused=True)) update parameters without advancing it."""
    if reuse and all(getattr(w, "_jf_q", None) is not None for w in weights):
        return
    for w, pair in zip(weights, NL.int8_quantize_many([w.detach() for w in weights], QB)):
        w._jf_q = pair


def _i8(t):
    return t.view(torch.int8)


class _Begin(torch.autograd.Function):
    """Entry of the INT8 stream: quantise the embedding output (reference: QModel_bgn_func, qmodel.py:309-326)."""

    @staticmethod
    def forward(ctx, x):
        qx, sx = NL.int8_quantize(x, QB)
        return x, _f8(qx), sx

    @staticmethod
    def backward(ctx, g, qg, sg):
        return g


class _End(torch.autograd.Function):
    """Exit of the INT8 stream: in the backward pass the incoming fp gradient is block-quantised with stochastic rounding and
    seeds the INT8 gradient stream (reference: QModel_end_func, qmodel.py:343-362)."""

    @staticmethod
    def forward(ctx, x, qx, sx):
        return x.clone()

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        qg, sg = NL.int8_quantize(g, QB, stochastic=True)
        return g, _f8(qg), sg


class _AttnIn(torch.autograd.Function):
    """LayerNorm + QKV projection (reference: _QAttentionPart1, qmodel.py:86-132).  Output: dequantised fp16 QKV."""

    @staticmethod
    def forward(ctx, residual, qx, sx, w_qkv, ln_w, mean, rstd):
        qx = _i8(qx)
        qw, sw = quantized_weight(w_qkv)
        qn, sn, _ = NL.int8_layernorm_forward(qx, sx, ln_w, mean, rstd, QB)
        y = L.int8_linear_forward(qn, sn, qw, sw, False, QB)
        ctx.save_for_backward(qx, sx, qn, sn, qw, sw, ln_w, mean, rstd)
        return residual, y

    @staticmethod
    def backward(ctx, fpg, g):
        qx, sx, qn, sn, qw, sw, ln_w, mean, rstd = ctx.saved_tensors
        qg, sg = NL.int8_quantize(g.contiguous(), QB, stochastic=True)
        qg, sg, dw = _linear_backward(qn, sn, qg, sg, qw, sw)
        qg, sg, dln = NL.int8_layernorm_backward(qx, sx, qg, sg, ln_w, QB, mean, rstd, stochastic=True)
        res_g, qg, sg = NL.int8_add_Ifp_Ig16_Ofp_Og(fpg.contiguous(), qg, sg, QB, stochastic=True)
        return res_g, _f8(qg), sg, dw, dln, None, None


class _AttnOut(torch.autograd.Function):
    """Attention output projection + residual add with row statistics (reference: _QAttentionPart2, qmodel.py:134-170)."""

    @staticmethod
    def forward(ctx, residual, y, w_proj):
        qw, sw = quantized_weight(w_proj)
        qy, sy = NL.int8_quantize(y.contiguous(), QB)
        qo, so = L.int8_linear_forward(qy, sy, qw, sw, True, QB)
        fpx, qx, sx, mean, rstd = NL.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(residual.contiguous(), qo, so, QB)
        ctx.save_for_backward(qy, sy, qw, sw)
        ctx.mark_non_differentiable(mean, rstd)
        return fpx, _f8(qx), sx, mean, rstd

    @staticmethod
    def backward(ctx, fpg, qg, sg, _m, _r):
        qy, sy, qw, sw = ctx.saved_tensors
        g16, dw = _linear_backward(qy, sy, _i8(qg), sg, qw, sw, dgrad_quantize=False)
        return fpg, g16, dw


class _MLP(torch.autograd.Function):
    """LayerNorm + FC1 + GELU + FC2 + residual add with row statistics (reference: _QMLPResidual, qmodel.py:190-267)."""

    @staticmethod
    def forward(ctx, residual, qx, sx, w1, w2, ln_w, mean, rstd):
        qx = _i8(qx)
        qw1, sw1 = quantized_weight(w1)
        qw2, sw2 = quantized_weight(w2)
        qn, sn, _ = NL.int8_layernorm_forward(qx, sx, ln_w, mean, rstd, QB)
        qh, sh = L.int8_linear_forward(qn, sn, qw1, sw1, True, QB)
        qa, sa = NL.int8_gelu_forward(qh, sh, QB)
        qo, so = L.int8_linear_forward(qa, sa, qw2, sw2, True, QB)
        fpx, qy, sy, mean2, rstd2 = NL.int8_add_Ifp_Ig16_Ofp_Og_MeanVar(residual.contiguous(), qo, so, QB)
        ctx.save_for_backward(qx, sx, qn, sn, qh, sh, qa, sa, qw1, sw1, qw2, sw2, ln_w, mean, rstd)
        ctx.mark_non_differentiable(mean2, rstd2)
        return fpx.to(torch.bfloat16), _f8(qy), sy, mean2, rstd2

    @staticmethod
    def backward(ctx, fpg, qg, sg, _m, _r):
        qx, sx, qn, sn, qh, sh, qa, sa, qw1, sw1, qw2, sw2, ln_w, mean, rstd = ctx.saved_tensors
        qg, sg, dw2 = _linear_backward(qa, sa, _i8(qg), sg, qw2, sw2)
        qg, sg = NL.int8_gelu_backward(qh, sh, qg, sg, QB, stochastic=True)
        qg, sg, dw1 = _linear_backward(qn, sn, qg, sg, qw1, sw1)
        qg, sg, dln = NL.int8_layernorm_backward(qx, sx, qg, sg, ln_w, QB, mean, rstd, stochastic=True)
        res_g, qg, sg = NL.int8_add_Ifp_Ig16_Ofp_Og(fpg.contiguous(), qg, sg, QB, stochastic=True)
        return res_g, _f8(qg), sg, dw1, dw2, dln, None, None


def _linear_backward(qx, sx, qg, sg, qw, sw, dgrad_quantize=True):
    """Input gradient (stochastically rounded INT8, or dequantised fp16) and fp32 weight gradient of one linear layer."""
    return L.int8_linear_backward(qx, sx, qg, sg, None, qw, sw, QB, stochastic=True, dgrad_quantize=dgrad_quantize,
                                  wgrad_out_dtype=torch.float32)


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        C = cfg.n_embd
        self.n_head = cfg.n_head
        self.ln_1 = nn.Parameter(torch.ones(C))
        self.c_attn = nn.Parameter(torch.empty(3 * C, C))
        self.c_proj = nn.Parameter(torch.empty(C, C))
        self.ln_2 = nn.Parameter(torch.ones(C))
        self.c_fc = nn.Parameter(torch.empty(4 * C, C))
        self.c_proj2 = nn.Parameter(torch.empty(C, 4 * C))

    def forward(self, x, qx, sx, mean, rstd):
        B, T, C = x.shape
        residual, qkv = _AttnIn.apply(x, qx, sx, self.c_attn, self.ln_1, mean, rstd)
        q, k, v = qkv.split(C, dim=2)
        hs = C // self.n_head
        q = q.view(B, T, self.n_head, hs).transpose(1, 2)
        k = k.view(B, T, self.n_head, hs).transpose(1, 2)
        v = v.view(B, T, self.n_head, hs).transpose(1, 2)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        y = y.transpose(1, 2).contiguous().view(B, T, C)
        x, qx, sx, mean, rstd = _AttnOut.apply(residual, y, self.c_proj)
        return _MLP.apply(x, qx, sx, self.c_fc, self.c_proj2, self.ln_2, mean, rstd)


class QGPT(nn.Module):
    def __init__(self, cfg: GPTConfig):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.vocab_size, cfg.n_embd)
        self.wpe = nn.Embedding(cfg.block_size, cfg.n_embd)
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.Parameter(torch.ones(cfg.n_embd))
        std = 0.02
        nn.init.normal_(self.wte.weight, 0.0, std)
        nn.init.normal_(self.wpe.weight, 0.0, std)
        for b in self.blocks:
            nn.init.normal_(b.c_attn, 0.0, std)
            nn.init.normal_(b.c_fc, 0.0, std)
            nn.init.normal_(b.c_proj, 0.0, std / math.sqrt(2 * cfg.n_layer))
            nn.init.normal_(b.c_proj2, 0.0, std / math.sqrt(2 * cfg.n_layer))

    def num_params(self):
        return sum(p.numel() for p in self.parameters()) - self.wpe.weight.numel()

    def forward(self, idx, targets, reuse_quantised_weights=False):
        """`reuse_quantised_weights`: the weights have not changed since the previous forward pass (micro-steps 2.. of a
        gradient-accumulation step), keep their quantisations."""
        B, T = idx.shape
        pos = torch.arange(T, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        quantise_weights([w for b in self.blocks for w in (b.c_attn, b.c_proj, b.c_fc, b.c_proj2)], reuse=reuse_quantised_weights)
        x, qx, sx = _Begin.apply(x)
        mean = x.mean(-1)
        rstd = 1.0 / x.var(-1).sqrt()
        for blk in self.blocks:
            x, qx, sx, mean, rstd = blk(x, qx, sx, mean.detach(), rstd.detach())
        x = _End.apply(x, qx, sx)
        x = F.layer_norm(x.float(), (self.cfg.n_embd,), self.ln_f, None, 1e-5)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = F.linear(x, self.wte.weight)
        return lm_cross_entropy(logits, targets)       # no fp32 copy of the [tokens, vocab] logits; gradient written in place
