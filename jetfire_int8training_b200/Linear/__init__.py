"""The INT8 linear layer with the reference's function names and conventions
(Jetfire/Linear/linear_fwd.py:4-32 and linear_bwd.py:4-28 of thu-ml/Jetfire-INT8Training).

Differences that do not change results: scale tensors are read in their natural [rows/32, cols/32] layout (the
reference makes transposed copies), W and dY are read in place by the GEMMs (the `G8T` argument, the materialised
transpose of dY, is accepted and ignored), the "dequantised output" variants are produced by the GEMM epilogue
instead of two torch kernels, and large GEMMs run on exact fp16 copies of their operands (`operand_scratch`: the tensor core
then delivers the block products as floats; bit-identical results).
"""
import torch

from .. import rng
from .._lib import lib, check

__all__ = ["int8_linear_forward", "int8_linear_backward", "int8_linear_wgrad"]

JF_OUT_INT8, JF_OUT_DEQUANT_F16 = 0, 1
JF_F32, JF_F16 = 0, 1


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _i8(t):
    return t.view(torch.int8) if t.dtype != torch.int8 else t


# "auto": let the library decide from the GEMM's dimensions whether the fp16-operand kernel pays for its conversion passes
# (large GEMMs); True / False force it on / off.  Results are bit-identical either way.
OPERAND_SCRATCH = "auto"


def _op16(M, N, K, device, mode=None):
    """(pointer, bytes, keep-alive tensor) of the fp16 operand scratch for a GEMM, or (None, 0, None)."""
    mode = OPERAND_SCRATCH if mode is None else mode
    if mode is False:
        return None, 0, None
    nbytes = 2 * (M * K + N * K) if mode is True else lib().jf_igemm_op16_bytes(M, N, K)
    if nbytes <= 0:
        return None, 0, None
    buf = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    return buf.data_ptr(), nbytes, buf


def int8_linear_forward(X8_3D, SX16_3D, W8, SW16, output_quantized, B, *, operand_scratch=None):
    """Y = X W^T.  X8 int8 [..., K] with scales [..., K/32] (leading dims flattened), W8 int8 [N, K], SW16 [N/32, K/32].
    Returns (Y8, SY16) when output_quantized, else the dequantised fp16 tensor fp16(q) * scale."""
    if B != 32:
        raise ValueError("only the 32x32 quantisation block of the reference recipe is implemented")
    if not X8_3D.is_cuda:
        raise RuntimeError("jetfire_int8training_b200 operators need CUDA tensors (there is no CPU path)")
    K = X8_3D.shape[-1]
    N = W8.shape[0]
    X8 = _i8(X8_3D).reshape(-1, K).contiguous()
    SX = SX16_3D.reshape(-1, SX16_3D.shape[-1]).contiguous()
    W8c = _i8(W8).contiguous()
    SWc = SW16.contiguous()
    M = X8.shape[0]
    out_shape = list(X8_3D.shape[:-1]) + [N]
    s_shape = list(SX16_3D.shape[:-1]) + [N // 32]
    dev = X8.device
    op, opn, _keep = _op16(M, N, K, dev, operand_scratch)
    if output_quantized:
        y8 = torch.empty((M, N), dtype=torch.int8, device=dev)
        sy = torch.empty((M // 32, N // 32), dtype=torch.float16, device=dev)
        check(lib().jf_igemm_forward(X8.data_ptr(), W8c.data_ptr(), SX.data_ptr(), SX.stride(0), SX.stride(1), SWc.data_ptr(),
                                     SWc.stride(0), SWc.stride(1), M, N, K, JF_OUT_INT8, y8.data_ptr(), sy.data_ptr(), None,
                                     op, opn, _stream()), "int8_linear_forward")
        return y8.reshape(out_shape), sy.reshape(s_shape)
    y16 = torch.empty((M, N), dtype=torch.float16, device=dev)
    check(lib().jf_igemm_forward(X8.data_ptr(), W8c.data_ptr(), SX.data_ptr(), SX.stride(0), SX.stride(1), SWc.data_ptr(),
                                 SWc.stride(0), SWc.stride(1), M, N, K, JF_OUT_DEQUANT_F16, None, None, y16.data_ptr(),
                                 op, opn, _stream()), "int8_linear_forward")
    return y16.reshape(out_shape)


def int8_linear_wgrad(X8, SX, G8, SG, out_dtype=torch.float16, split_k=0, operand_scratch=None):
    """dW[Cout, Cin] = dY^T X with dY = G8 [T, Cout], X8 [T, Cin] (2-D, natural layouts, read in place)."""
    T, Cout = G8.shape
    Cin = X8.shape[1]
    L = lib()
    splits = L.jf_igemm_wgrad_plan(Cout, Cin, T, split_k)
    if splits < 1:
        check(splits, "int8_linear_wgrad(plan)")
    dw = torch.empty((Cout, Cin), dtype=out_dtype, device=G8.device)
    scratch = torch.empty((splits * Cout * Cin,), dtype=torch.float32, device=G8.device) if splits > 1 else None
    op, opn, _keep = _op16(Cout, Cin, T, G8.device, operand_scratch)
    check(L.jf_igemm_wgrad(G8.data_ptr(), 0, X8.data_ptr(), SG.data_ptr(), SG.stride(0), SG.stride(1), SX.data_ptr(), SX.stride(0),
                           SX.stride(1), Cout, Cin, T, JF_F16 if out_dtype == torch.float16 else JF_F32, dw.data_ptr(), splits,
                           None if scratch is None else scratch.data_ptr(), op, opn, _stream()), "int8_linear_wgrad")
    return dw


def int8_linear_backward(X8_3D, SX16_3D, G8_3D, SG16_3D, G8T, W8, SW16, B, stochastic=True, dgrad_quantize=True, *,
                         sr_key=None, noise=None, wgrad_split_k=0, wgrad_out_dtype=torch.float16, operand_scratch=None):
    """dX = dY W (block-quantised with stochastic rounding, or dequantised fp16 when dgrad_quantize is False) and
    dW = dY^T X (dense fp16).  Returns (GX8, GSX16, GW) or (GX16, GW), as the reference does.
    The reference ignores `stochastic` and always rounds stochastically; here stochastic=False rounds to nearest.
    `wgrad_out_dtype=torch.float32` (extra) returns dW in fp32 instead of the reference's fp16."""
    if B != 32:
        raise ValueError("only the 32x32 quantisation block of the reference recipe is implemented")
    if not G8_3D.is_cuda:
        raise RuntimeError("jetfire_int8training_b200 operators need CUDA tensors (there is no CPU path)")
    Cout, Cin = W8.shape
    G8 = _i8(G8_3D).reshape(-1, Cout).contiguous()
    SG = SG16_3D.reshape(-1, SG16_3D.shape[-1]).contiguous()
    X8 = _i8(X8_3D).reshape(-1, Cin).contiguous()
    SX = SX16_3D.reshape(-1, SX16_3D.shape[-1]).contiguous()
    W8c = _i8(W8).contiguous()
    SWc = SW16.contiguous()
    M = G8.shape[0]
    dev = G8.device
    gx_shape = list(G8_3D.shape[:-1]) + [Cin]
    gs_shape = list(SG16_3D.shape[:-1]) + [Cin // 32]
    st, nz, seed, off = 0, None, 0, 0
    if stochastic:
        st = 1
        if noise is not None:
            noise = noise.reshape(M, Cin).to(device=dev, dtype=torch.float32).contiguous()
            nz = noise.data_ptr()
        else:
            seed, off = sr_key if sr_key is not None else rng.next_key()
    L = lib()
    op, opn, _keep = _op16(M, Cin, Cout, dev, operand_scratch)
    if dgrad_quantize:
        gx8 = torch.empty((M, Cin), dtype=torch.int8, device=dev)
        gsx = torch.empty((M // 32, Cin // 32), dtype=torch.float16, device=dev)
        check(L.jf_igemm_dgrad(G8.data_ptr(), W8c.data_ptr(), SG.data_ptr(), SG.stride(0), SG.stride(1), SWc.data_ptr(), SWc.stride(0),
                               SWc.stride(1), M, Cin, Cout, JF_OUT_INT8, gx8.data_ptr(), gsx.data_ptr(), None, st, nz, seed, off,
                               op, opn, _stream()), "int8_linear_backward(dgrad)")
    else:
        gx16 = torch.empty((M, Cin), dtype=torch.float16, device=dev)
        check(L.jf_igemm_dgrad(G8.data_ptr(), W8c.data_ptr(), SG.data_ptr(), SG.stride(0), SG.stride(1), SWc.data_ptr(), SWc.stride(0),
                               SWc.stride(1), M, Cin, Cout, JF_OUT_DEQUANT_F16, None, None, gx16.data_ptr(), st, nz, seed, off,
                               op, opn, _stream()), "int8_linear_backward(dgrad)")
    gw = int8_linear_wgrad(X8, SX, G8, SG, wgrad_out_dtype, wgrad_split_k, operand_scratch)
    if dgrad_quantize:
        return gx8.reshape(gx_shape), gsx.reshape(gs_shape), gw
    return gx16.reshape(gx_shape), gw
