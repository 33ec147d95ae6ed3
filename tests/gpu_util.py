"""Helpers shared by the GPU parity tests: seeded inputs and comparison rules."""
import numpy as np
import torch

DEV = "cuda"


def t(a, dtype=None):
    x = a if isinstance(a, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        x = x.to(dtype)
    return x.to(DEV)


def n(x):
    if x.dtype == torch.bfloat16:
        return x.float().cpu().numpy()
    return x.detach().cpu().numpy()


def assert_bits_equal(got, want, what=""):
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert got.dtype == want.dtype, (what, got.dtype, want.dtype)
    neq = np.count_nonzero(got.view(np.uint8).reshape(-1) != want.view(np.uint8).reshape(-1))
    assert neq == 0, f"{what}: {neq} differing bytes of {got.nbytes}"


def assert_payload_close(got, want, max_frac, what=""):
    """int8 payloads equal except for at most max_frac of the elements, which may differ by one step."""
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1, f"{what}: payload differs by {d.max()} steps"
    frac = np.count_nonzero(d) / d.size
    assert frac <= max_frac, f"{what}: {frac:.2e} of the payload differs (allowed {max_frac:.1e})"


def assert_scales_close(got, want, ulps=1, what=""):
    """fp16 scales within `ulps` units in the last place."""
    a = got.view(np.int16).astype(np.int32)
    b = want.view(np.int16).astype(np.int32)
    assert np.abs(a - b).max() <= ulps, f"{what}: scales differ by {np.abs(a - b).max()} ulp"


def outlier_randn(g, M, N, frac=0.005, mult=30.0):
    """N(0,1) with a fraction of the channels scaled up (the activation-outlier model of the benchmark configs)."""
    x = torch.randn(M, N, generator=g)
    k = max(1, round(frac * N))
    idx = torch.randperm(N, generator=g)[:k]
    x[:, idx] *= mult
    return x
