"""INT8 linear layer steps (forward + input gradient + weight gradient) fed from and drained to pinned HOST buffers.

`Linear.int8_linear_forward/backward` take device tensors, as the reference's functions do (Jetfire/Linear/linear_fwd.py:4-32,
linear_bwd.py:5-21).  When the operands of every step live in host memory, the copies cost more than the three GEMMs
(470 MB per 8192^3 step), so this helper runs the steps as a three-stream pipeline: the copy engine brings in the operands of
step i+1 (double-buffered on the device) while the GEMMs of step i run and the results of step i-1 go back to the host.
Every step still moves all of its operands in and all of its results out; nothing is cached between steps.
"""
import torch

from . import Linear


class LinearStepPipeline:
    """submit(host_in, host_out) queues one step; finish() waits until every queued result has reached the host.

    host_in  = (X8 [M,K] int8, SX [M/32,K/32] fp16, W8 [N,K] int8, SW fp16, G8 [M,N] int8, SG fp16), pinned
    host_out = (Y8 [M,N] int8, SY fp16, GX8 [M,K] int8, GSX fp16, GW [N,K] fp16), pinned
    `after_backward(gw)` (optional) runs on the compute stream after the weight gradient (e.g. the data-parallel all-reduce).
    """

    def __init__(self, device, stochastic=True, after_backward=None):
        self.dev = torch.device(device)
        self.stochastic = stochastic
        self.after_backward = after_backward
        # The compute stream is the stream that is current when the pipeline is built; submit() runs its GEMMs on it whatever
        # stream is current at that time, because all of the pipeline's events are ordered against this one stream.
        self.s_comp = torch.cuda.current_stream(self.dev)
        self.s_in = torch.cuda.Stream(self.dev)
        self.s_out = torch.cuda.Stream(self.dev)
        self.dev_in = [None, None]
        self.free_ev = [None, None]   # the compute of the step that last used an input set has finished
        self.i = 0
        self.prefetched = None        # (step index, events) of operands already on their way
        self.last_out = None

    def _h2d(self, i, host_in):
        with torch.cuda.stream(self.s_in):
            if self.dev_in[i % 2] is None:
                # Allocated under the copy stream, so the caching allocator hands out memory that is free with respect to THIS
                # stream.  Its first use is still ordered after everything queued on the compute stream so far: a block that the
                # allocator recycled from the compute stream may be read by kernels that are still queued there.
                first = torch.cuda.Event()
                first.record(self.s_comp)
                self.s_in.wait_event(first)
                self.dev_in[i % 2] = [torch.empty_like(t, device=self.dev) for t in host_in]
            buf = self.dev_in[i % 2]
            if self.free_ev[i % 2] is not None:
                self.s_in.wait_event(self.free_ev[i % 2])
            for d, h in zip(buf[:4], host_in[:4]):          # forward operands first, so that the forward GEMM can start
                d.copy_(h, non_blocking=True)
            ev_fwd = torch.cuda.Event(); ev_fwd.record(self.s_in)
            for d, h in zip(buf[4:], host_in[4:]):
                d.copy_(h, non_blocking=True)
            ev_bwd = torch.cuda.Event(); ev_bwd.record(self.s_in)
        return ev_fwd, ev_bwd

    def submit(self, host_in, host_out, next_host_in=None):
        """Queue one step.  `next_host_in`: the operands of the following step, if known, are prefetched behind this one's."""
        i = self.i
        if self.prefetched is not None and self.prefetched[0] == i:
            ev_fwd, ev_bwd = self.prefetched[1]
        else:
            ev_fwd, ev_bwd = self._h2d(i, host_in)
        self.prefetched = (i + 1, self._h2d(i + 1, next_host_in)) if next_host_in is not None else None
        x8, sx, w8, sw, g8, sg = self.dev_in[i % 2]
        s_comp, s_out = self.s_comp, self.s_out
        with torch.cuda.stream(s_comp):      # the operators launch on the current stream: make it the pipeline's compute stream
            for d in self.dev_in[i % 2]:
                d.record_stream(s_comp)      # allocated under the copy stream, read here
            s_comp.wait_event(ev_fwd)
            y8, sy = Linear.int8_linear_forward(x8, sx, w8, sw, True, 32)
            ev_y = torch.cuda.Event(); ev_y.record(s_comp)
            s_comp.wait_event(ev_bwd)
            gx8, gsx, gw = Linear.int8_linear_backward(x8, sx, g8, sg, None, w8, sw, 32, stochastic=self.stochastic)
            if self.after_backward is not None:
                self.after_backward(gw)
            ev_b = torch.cuda.Event(); ev_b.record(s_comp)
        self.free_ev[i % 2] = ev_b
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_y)
            for h, o in zip(host_out[:2], (y8, sy)):
                o.record_stream(s_out)
                h.copy_(o, non_blocking=True)
            s_out.wait_event(ev_b)
            for h, o in zip(host_out[2:], (gx8, gsx, gw)):
                o.record_stream(s_out)
                h.copy_(o, non_blocking=True)
            self.last_out = torch.cuda.Event(); self.last_out.record(s_out)
        self.i = i + 1

    def finish(self):
        """Make the compute stream wait for the last device-to-host copy (call torch.cuda.synchronize() to block the host)."""
        if self.last_out is not None:
            self.s_comp.wait_event(self.last_out)
