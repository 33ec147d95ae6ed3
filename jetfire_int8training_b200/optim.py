"""Loss scaling + gradient clipping by global norm + AdamW as one call into the CUDA library (csrc/optim.cu).

Replaces  scaler.scale(loss).backward(); scaler.unscale_(optimizer); clip_grad_norm_(params, max_norm); scaler.step(optimizer);
scaler.update()  at the end of the reference's training step (INT8_GPT2/train.py:216-217, 320-329: fp16 autocast with torch's
GradScaler, init_scale 2^24; optimiser groups: weight decay on tensors with two or more dimensions, none on the others,
INT8_GPT2/qmodel.py:525-537).  The loss scale matters for the INT8 path: the gradients that cross the attention are fp16 tensors,
and at GPT-2 124M sizes (12 x 1024 tokens per batch) they underflow without it.  The parameters are moved into one flat fp32 buffer (each `p.data` becomes a view of it, so the
model, DDP and checkpoints keep working); first and second moments are two more flat buffers; gradients stay where autograd puts
them.  Construct it BEFORE wrapping the model in DistributedDataParallel.
"""
import ctypes
import math

import torch

from ._lib import lib, check


class ClipAdamW:
    """`groups`: iterable of (parameters, weight_decay).

    loss_scale=None: no loss scaling.  loss_scale=s: `scale_loss(loss)` multiplies the loss by the current scale (initially s);
    a step whose gradients are not finite changes nothing but the scale (x backoff_factor), and after growth_interval good
    steps in a row the scale is multiplied by growth_factor -- torch.amp.GradScaler's rule, kept in device memory (no host
    synchronisation).  step() returns a device tensor [gradient norm, factor applied to the raw gradients, 1 if skipped]."""

    def __init__(self, groups, lr, betas=(0.9, 0.95), eps=1e-8, max_norm=1.0, loss_scale=None, growth_interval=2000,
                 growth_factor=2.0, backoff_factor=0.5):
        self.lr, self.betas, self.eps, self.max_norm = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(max_norm)
        self.growth_interval = int(growth_interval) if loss_scale is not None else 0
        self.growth_factor, self.backoff_factor = float(growth_factor), float(backoff_factor)
        self.params, wds = [], []
        for ps, wd in groups:
            for p in ps:
                if not p.requires_grad:
                    continue
                if p.dtype != torch.float32 or not p.is_cuda or p.numel() % 4 != 0:
                    raise ValueError("ClipAdamW needs fp32 CUDA parameters whose sizes are multiples of 4")
                self.params.append(p)
                wds.append(float(wd))
        if not self.params:
            raise ValueError("no parameters")
        self.chunk = int(lib().jf_adamw_chunk_elements())
        dev = self.params[0].device
        n = len(self.params)
        starts, c = [], 0
        for p in self.params:
            starts.append(c)
            c += (p.numel() + self.chunk - 1) // self.chunk
        self.total_chunks = c
        self.flat = torch.zeros(c * self.chunk, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros_like(self.flat)
        self.exp_avg_sq = torch.zeros_like(self.flat)
        with torch.no_grad():
            for p, s in zip(self.params, starts):
                view = self.flat[s * self.chunk: s * self.chunk + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
        self._numel = (ctypes.c_int64 * n)(*[p.numel() for p in self.params])
        self._starts = (ctypes.c_int64 * n)(*starts)
        self._wd = (ctypes.c_float * n)(*wds)
        self._partial = torch.empty(c, dtype=torch.float32, device=dev)
        self._GradArray = ctypes.c_void_p * n
        # [scale, steps since the scale changed, optimiser steps taken, norm, applied factor, skipped, 2 x scratch]
        self.state = torch.zeros(8, dtype=torch.float32, device=dev)
        self.state[0] = 1.0 if loss_scale is None else float(loss_scale)

    def scale_loss(self, loss):
        """loss x current loss scale (a device-side multiplication); call backward() on the result."""
        return loss * self.state[0]

    @property
    def step_count(self):
        """Optimiser steps actually taken (skipped steps do not count).  Synchronises."""
        return int(self.state[2].item())

    def _segment(self, buf, i):
        s = self._starts[i] * self.chunk
        return buf[s: s + self.params[i].numel()].view(self.params[i].shape)

    def step(self):
        grads = []
        for p in self.params:
            g = p.grad
            if g is None:
                raise RuntimeError("ClipAdamW.step(): a parameter has no gradient")
            if g.dtype != torch.float32 or not g.is_contiguous():
                g = g.float().contiguous()
                p.grad = g
            grads.append(g)
        check(lib().jf_adamw_clip_step(len(self.params), self._GradArray(*[g.data_ptr() for g in grads]), self._numel, self._starts,
                                       self._wd, self.flat.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                                       self.total_chunks, self.lr, self.betas[0], self.betas[1], self.eps, self.max_norm,
                                       self.state.data_ptr(), self.growth_interval, self.growth_factor, self.backoff_factor,
                                       self._partial.data_ptr(), torch.cuda.current_stream().cuda_stream), "adamw_clip_step")
        out = self.state[3:6].clone()          # [gradient norm, applied factor, skipped]
        # the parameters were updated in place through the flat buffer by a kernel autograd does not know about: advance their
        # version counters (what an in-place torch operation would have done)
        torch.autograd.graph.increment_version(self.params)
        return out

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def state_dict(self):
        return {"state": self.state.clone(), "lr": self.lr, "betas": self.betas, "eps": self.eps, "max_norm": self.max_norm,
                "exp_avg": self.exp_avg.clone(), "exp_avg_sq": self.exp_avg_sq.clone()}

    def load_state_dict(self, sd):
        self.state.copy_(sd["state"])
        self.lr, self.betas, self.eps, self.max_norm = float(sd["lr"]), tuple(sd["betas"]), float(sd["eps"]), float(sd["max_norm"])
        self.exp_avg.copy_(sd["exp_avg"]); self.exp_avg_sq.copy_(sd["exp_avg_sq"])
