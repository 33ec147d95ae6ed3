"""Cross-entropy of the language-model head on bf16 logits, without an fp32 copy of the logits.

`lm_cross_entropy(logits, targets)` equals `F.cross_entropy(logits.float().view(-1, V), targets.view(-1), ignore_index=-1)`
(the loss at the end of the reference's quantised GPT-2, INT8_GPT2/qmodel.py:433-439) up to fp32 rounding.  The forward pass
reads the logits once; the backward pass overwrites them IN PLACE with their gradient (the logits are an intermediate that
nothing else needs: the backward of the producing matmul uses its inputs, not its output), so no second [tokens, vocab] tensor
is ever allocated.  There is no CPU path.
"""
import torch

from ._lib import lib, check

__all__ = ["lm_cross_entropy"]


class _LMLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        if not logits.is_cuda:
            raise RuntimeError("jetfire_int8training_b200 operators need CUDA tensors (there is no CPU path)")
        if logits.dtype != torch.bfloat16:
            raise TypeError("lm_cross_entropy takes bf16 logits")
        V = logits.shape[-1]
        x = logits.reshape(-1, V)
        if not x.is_contiguous():
            x = x.contiguous()
        t = targets.reshape(-1).to(torch.int64).contiguous()
        rows = x.shape[0]
        lse = torch.empty(rows, dtype=torch.float32, device=x.device)
        loss_rows = torch.empty(rows, dtype=torch.float32, device=x.device)
        st = torch.cuda.current_stream().cuda_stream
        check(lib().jf_lm_loss_forward(x.data_ptr(), t.data_ptr(), rows, V, lse.data_ptr(), loss_rows.data_ptr(), st), "lm_cross_entropy")
        count = ((t >= 0) & (t < V)).sum().clamp(min=1).to(torch.float32)
        ctx.save_for_backward(x, t, lse, count)
        ctx.shape = logits.shape
        return loss_rows.sum() / count

    @staticmethod
    def backward(ctx, grad_out):
        x, t, lse, count = ctx.saved_tensors
        rows, V = x.shape
        g = (grad_out.to(torch.float32) / count).reshape(1).contiguous()
        st = torch.cuda.current_stream().cuda_stream
        check(lib().jf_lm_loss_backward(x.data_ptr(), t.data_ptr(), lse.data_ptr(), g.data_ptr(), 1.0, rows, V, st),
              "lm_cross_entropy(backward)")
        return x.view(ctx.shape), None


def lm_cross_entropy(logits, targets):
    """Mean softmax cross-entropy over the positions whose target lies in [0, vocab).  `logits` (bf16, [..., vocab]) is
    consumed: after backward() it holds its own gradient."""
    return _LMLoss.apply(logits, targets)
