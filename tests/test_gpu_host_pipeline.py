"""The host-buffer pipeline must give exactly what the device-tensor operator calls give, step by step."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(seed, M, N, K):
    g = torch.Generator().manual_seed(seed)
    def q(r, c):
        return torch.randint(-127, 128, (r, c), generator=g, dtype=torch.int8).pin_memory()
    def s(r, c):
        return (torch.rand(r, c, generator=g) * 0.05 + 1e-3).half().pin_memory()
    return (q(M, K), s(M // 32, K // 32), q(N, K), s(N // 32, K // 32), q(M, N), s(M // 32, N // 32))


def test_pipeline_matches_direct_calls():
    from jetfire_int8training_b200 import Linear, rng
    from jetfire_int8training_b200.host_pipeline import LinearStepPipeline
    dev = torch.device("cuda", 0)
    M, N, K = 256, 384, 512
    steps = [_operands(s, M, N, K) for s in (1, 2, 3)]

    rng.manual_seed(99)
    want = []
    for h in steps:
        x8, sx, w8, sw, g8, sg = [t.to(dev) for t in h]
        y8, sy = Linear.int8_linear_forward(x8, sx, w8, sw, True, 32)
        gx8, gsx, gw = Linear.int8_linear_backward(x8, sx, g8, sg, None, w8, sw, 32, stochastic=True)
        want.append([t.cpu() for t in (y8, sy, gx8, gsx, gw)])

    rng.manual_seed(99)
    pipe = LinearStepPipeline(dev, stochastic=True)
    outs = [[torch.empty_like(t).pin_memory() for t in want[0]] for _ in steps]
    for i, h in enumerate(steps):
        pipe.submit(h, outs[i], next_host_in=steps[i + 1] if i + 1 < len(steps) else None)
    pipe.finish()
    torch.cuda.synchronize()
    for i in range(len(steps)):
        for got, ref in zip(outs[i], want[i]):
            assert torch.equal(got, ref), f"step {i}"


def test_pipeline_built_and_driven_from_a_side_stream_after_queued_work():
    """The pipeline's compute stream is the stream that is current when it is built; its device buffers are allocated while
    kernels are still queued on that stream, and submit() is called with yet another stream current.  Results must equal the
    serial path (stream-ordering bugs show up as stale or overwritten operands)."""
    from jetfire_int8training_b200 import Linear, rng
    from jetfire_int8training_b200.host_pipeline import LinearStepPipeline
    dev = torch.device("cuda", 0)
    M, N, K = 512, 384, 768
    steps = [_operands(s, M, N, K) for s in (11, 12, 13, 14)]
    rng.manual_seed(5)
    want = []
    for h in steps:
        x8, sx, w8, sw, g8, sg = [t.to(dev) for t in h]
        y8, sy = Linear.int8_linear_forward(x8, sx, w8, sw, True, 32)
        gx8, gsx, gw = Linear.int8_linear_backward(x8, sx, g8, sg, None, w8, sw, 32, stochastic=True)
        want.append([t.cpu() for t in (y8, sy, gx8, gsx, gw)])
    torch.cuda.synchronize()

    side, other = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    rng.manual_seed(5)
    with torch.cuda.stream(side):
        # queue work on the side stream that reads freshly freed blocks, then build the pipeline behind it
        junk = [torch.randn(2048, 2048, device=dev) for _ in range(3)]
        acc = junk[0]
        for _ in range(20):
            acc = acc @ junk[1]
        del junk, acc
        pipe = LinearStepPipeline(dev, stochastic=True)
    outs = [[torch.empty_like(t).pin_memory() for t in want[0]] for _ in steps]
    with torch.cuda.stream(other):        # a different stream is current while the steps are submitted
        for i, h in enumerate(steps):
            pipe.submit(h, outs[i], next_host_in=steps[i + 1] if i + 1 < len(steps) else None)
        pipe.finish()
    torch.cuda.synchronize()
    for i in range(len(steps)):
        for got, ref in zip(outs[i], want[i]):
            assert torch.equal(got, ref), f"step {i}"
