"""Gradient clipping by global norm + AdamW as one call into the CUDA library (csrc/optim.cu).

Replaces the pair  torch.nn.utils.clip_grad_norm_(params, max_norm); torch.optim.AdamW(...).step()  at the end of the reference's
training step (INT8_GPT2/train.py:320-329; its optimiser groups: weight decay on tensors with two or more dimensions, none on the
others, INT8_GPT2/qmodel.py:525-537).  The parameters are moved into one flat fp32 buffer (each `p.data` becomes a view of it, so the
model, DDP and checkpoints keep working); first and second moments are two more flat buffers; gradients stay where autograd puts
them.  Construct it BEFORE wrapping the model in DistributedDataParallel.
"""
import ctypes
import math

import torch

from ._lib import lib, check


class ClipAdamW:
    """`groups`: iterable of (parameters, weight_decay).  step() returns a device tensor [grad_norm, applied_factor]."""

    def __init__(self, groups, lr, betas=(0.9, 0.95), eps=1e-8, max_norm=1.0):
        self.lr, self.betas, self.eps, self.max_norm = float(lr), (float(betas[0]), float(betas[1])), float(eps), float(max_norm)
        self.step_count = 0
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
        self.step_count += 1
        out = torch.empty(2, dtype=torch.float32, device=self.flat.device)
        check(lib().jf_adamw_clip_step(len(self.params), self._GradArray(*[g.data_ptr() for g in grads]), self._numel, self._starts,
                                       self._wd, self.flat.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                                       self.total_chunks, self.lr, self.betas[0], self.betas[1], self.eps, self.step_count,
                                       self.max_norm, self._partial.data_ptr(), out.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream), "adamw_clip_step")
        # the parameters were updated in place through the flat buffer by a kernel autograd does not know about: advance their
        # version counters (what an in-place torch operation would have done; caches keyed on the version see the change)
        torch.autograd.graph.increment_version(self.params)
        return out

    def zero_grad(self, set_to_none=True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def state_dict(self):
        return {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps, "max_norm": self.max_norm,
                "exp_avg": self.exp_avg.clone(), "exp_avg_sq": self.exp_avg_sq.clone()}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        self.lr, self.betas, self.eps, self.max_norm = float(sd["lr"]), tuple(sd["betas"]), float(sd["eps"]), float(sd["max_norm"])
        self.exp_avg.copy_(sd["exp_avg"]); self.exp_avg_sq.copy_(sd["exp_avg_sq"])
