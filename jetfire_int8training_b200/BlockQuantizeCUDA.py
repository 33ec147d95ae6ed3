"""Drop-in for the three functions of the reference's pybind module `BlockQuantizeCUDA` that the hot path uses
(JetfireGEMMKernel/BlockQuantize/cpp_extension/bindings.cpp:7-27), with the reference's argument order and layouts, so the
reference's own Jetfire/Linear glue can run on the sm_100a kernels unmodified.

Layouts (as the reference passes them): scale tensors are the TRANSPOSED copies [K/32, rows/32]; `Wt` of the forward call
is a `.t()` view whose storage is W [N, K] row-major; `X` of the weight-gradient call is the materialised dY^T [M, K].
"""
import torch

from . import rng
from ._lib import lib, check


def _stream():
    return torch.cuda.current_stream().cuda_stream


def igemm_output_int_quantize_bias_rowcol(X, Wt, bias, biasmax, SXt, SWt, M, N, K):
    """Forward Y = X W^T -> (int8 [M,N], fp16 [M/32,N/32]).  `bias` / `biasmax` must be zero (Jetfire always passes
    zeros, Jetfire/Linear/linear_fwd.py:20-21): the reference kernel adds them before re-quantising
    (igemm_BlockSquare32OutputIntQuantizeBiasRowCol.cu:341, 357), this one does not, so a non-zero tensor is refused.  The
    check reads the two tensors back (one small device-to-host copy per call); `Linear.int8_linear_forward` does not pay it."""
    if (bias is not None and bool(torch.count_nonzero(bias))) or (biasmax is not None and bool(torch.count_nonzero(biasmax))):
        raise NotImplementedError("BlockQuantizeCUDA shim: a non-zero bias / biasmax is not implemented (Jetfire passes zeros)")
    dev = X.device
    O = torch.empty((M, N), dtype=torch.int8, device=dev)
    SO = torch.empty((M // 32, N // 32), dtype=torch.float16, device=dev)
    SXt, SWt = SXt.contiguous(), SWt.contiguous()
    check(lib().jf_igemm_forward(X.data_ptr(), Wt.data_ptr(), SXt.data_ptr(), 1, SXt.stride(0), SWt.data_ptr(), 1, SWt.stride(0),
                                 M, N, K, 0, O.data_ptr(), SO.data_ptr(), None, None, 0, _stream()), "igemm_output_int_quantize_bias_rowcol")
    return O, SO


def igemm_output_int_quantize_stochastic(X, W, SXt, SW, M, N, K):
    """Input gradient dX = dY W with stochastic rounding -> (int8 [M,N], fp16 [M/32,N/32])."""
    dev = X.device
    O = torch.empty((M, N), dtype=torch.int8, device=dev)
    SO = torch.empty((M // 32, N // 32), dtype=torch.float16, device=dev)
    SXt, SW = SXt.contiguous(), SW.contiguous()
    seed, off = rng.next_key()
    check(lib().jf_igemm_dgrad(X.data_ptr(), W.data_ptr(), SXt.data_ptr(), 1, SXt.stride(0), SW.data_ptr(), SW.stride(0), 1,
                               M, N, K, 0, O.data_ptr(), SO.data_ptr(), None, 1, None, seed, off, None, 0, _stream()),
          "igemm_output_int_quantize_stochastic")
    return O, SO


def igemm_output_fp_no_quantize(X, W, SXt, SW, M, N, K):
    """Weight gradient dW = X W with X = dY^T [M,K] (materialised), W = activations [K,N] -> fp16 [M,N]."""
    dev = X.device
    L = lib()
    O = torch.empty((M, N), dtype=torch.float16, device=dev)
    SXt, SW = SXt.contiguous(), SW.contiguous()
    splits = L.jf_igemm_wgrad_plan(M, N, K, 1)
    check(L.jf_igemm_wgrad(X.data_ptr(), 1, W.data_ptr(), SXt.data_ptr(), SXt.stride(0), 1, SW.data_ptr(), SW.stride(0), 1,
                           M, N, K, 1, O.data_ptr(), splits, None, None, 0, _stream()), "igemm_output_fp_no_quantize")
    return O
