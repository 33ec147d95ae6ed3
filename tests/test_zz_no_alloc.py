"""GPU: the allocation-free add + mean/var entry point against the regular one.

Some callers cannot supply a workspace or let the library allocate one (plug-in interfaces that pass only inputs and
outputs, runtimes with a single fixed device arena, loops that must not call cudaMalloc).  jf_int8_add_meanvar_noalloc
serves them from a fixed array inside the library.  This test calls it through the C ABI twice in a row, with different
inputs, and requires the same bits as jf_int8_add_meanvar with a caller-provided workspace: the second call checks that
whatever the first one left in the shared array does not leak into the result.  It is collected last so that a run which
stops at the first failure has already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _run(L, fn_noalloc, x1, q2, s2):
    M, N = x1.shape
    st = torch.cuda.current_stream().cuda_stream
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x1.dtype]

    def outs():
        return (torch.empty((M, N), dtype=torch.float32, device=DEV), torch.empty((M, N), dtype=torch.int8, device=DEV),
                torch.empty((M // 32, N // 32), dtype=torch.float16, device=DEV), torch.empty((M,), dtype=torch.float32, device=DEV),
                torch.empty((M,), dtype=torch.float32, device=DEV))
    a = outs()
    if fn_noalloc:
        rc = L.jf_int8_add_meanvar_noalloc(x1.data_ptr(), dt, q2.data_ptr(), s2.data_ptr(), M, N, a[0].data_ptr(), a[1].data_ptr(),
                                           a[2].data_ptr(), a[3].data_ptr(), a[4].data_ptr(), st)
    else:
        scratch = torch.empty((2 * M * ((N + 127) // 128),), dtype=torch.float32, device=DEV)
        rc = L.jf_int8_add_meanvar(x1.data_ptr(), dt, q2.data_ptr(), s2.data_ptr(), M, N, a[0].data_ptr(), a[1].data_ptr(),
                                   a[2].data_ptr(), a[3].data_ptr(), a[4].data_ptr(), scratch.data_ptr(), st)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return a


def test_noalloc_matches_regular_entry_point_twice():
    from jetfire_int8training_b200._lib import lib
    L = lib()
    g = torch.Generator().manual_seed(31)
    for (M, N, dt) in ((256, 768, torch.float32), (96, 160, torch.bfloat16)):   # second call: other shape, ragged tile
        x1 = torch.randn(M, N, generator=g).to(dt).to(DEV)
        q2 = torch.randint(-127, 128, (M, N), generator=g, dtype=torch.int8).to(DEV)
        s2 = (torch.rand(M // 32, N // 32, generator=g) * 0.05 + 1e-3).half().to(DEV)
        want = _run(L, False, x1, q2, s2)
        got = _run(L, True, x1, q2, s2)
        for w, h in zip(want, got):
            assert torch.equal(w.view(torch.uint8), h.view(torch.uint8))   # bit-exact: the same kernels run
        assert bool(torch.isfinite(got[3]).all()) and bool(torch.isfinite(got[4]).all())


def test_noalloc_rejects_shapes_beyond_its_workspace():
    from jetfire_int8training_b200._lib import lib
    L = lib()
    x = torch.zeros(32, device=DEV)
    p = x.data_ptr()
    # 2 * M * ceil(N/128) = 2 * 65536 * 16 floats > 1048576: refused before anything is launched
    assert L.jf_int8_add_meanvar_noalloc(p, 0, p, p, 65536, 2048, p, p, p, p, p, None) == -2
    assert L.jf_int8_add_meanvar_noalloc(p, 0, p, p, 48, 128, p, p, p, p, p, None) == -2


def test_noalloc_at_exactly_its_limit():
    """2 * M * ceil(N/128) == 1048576 floats is the last shape the built-in workspace holds: it must run and give the regular
    entry point's bits; one more block row must be refused."""
    from jetfire_int8training_b200._lib import lib
    L = lib()
    M, N = 524288, 32
    g = torch.Generator(device=DEV).manual_seed(7)
    x1 = torch.randn(M, N, generator=g, device=DEV)
    q2 = torch.randint(-127, 128, (M, N), generator=g, device=DEV, dtype=torch.int8)
    s2 = (torch.rand(M // 32, N // 32, generator=g, device=DEV) * 0.05 + 1e-3).half()
    want = _run(L, False, x1, q2, s2)
    got = _run(L, True, x1, q2, s2)
    for w, h in zip(want, got):
        assert torch.equal(w.view(torch.uint8), h.view(torch.uint8))
    p = x1.data_ptr()
    assert L.jf_int8_add_meanvar_noalloc(p, 0, p, p, M + 32, N, p, p, p, p, p, None) == -2
