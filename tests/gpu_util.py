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


def outlier_randn(g, M, N, frac=0.005, mult=30.0):
    """N(0,1) with a fraction of the channels scaled up (the activation-outlier model of the benchmark configs)."""
    x = torch.randn(M, N, generator=g)
    k = max(1, round(frac * N))
    idx = torch.randperm(N, generator=g)[:k]
    x[:, idx] *= mult
    return x
