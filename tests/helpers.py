"""Shared helpers for the test-suite: seeded inputs, golden-case enumeration, digests."""
import hashlib

import numpy as np
import torch

CONSTS = dict(alpha=0.25, thresh=0.25, beta=1.0, interval=0.5)  # reference snnlib_func.py:11-14


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def fire_cases(golden):
    """Names of the golden cases that carry x, g, u, s, gx for the plain LIF layer."""
    return sorted({k[:-2] for k in golden.files if k.endswith("_u")})


def seeded_inputs(T, N, seed, dtype=torch.float32, batch=1):
    """Input currents ~ N(0.5, 1), upstream gradients ~ N(0, 1), as the benchmark configs use."""
    gen = torch.Generator().manual_seed(seed)
    x = 0.5 + torch.randn((T, batch, N // batch), generator=gen)
    g = torch.randn((T, batch, N // batch), generator=gen)
    return x.to(dtype), g.to(dtype)


def config1_inputs():
    """The single-layer case: T=8, [32,128,16,16], seed 1234 (x first, then the gradient)."""
    gen = torch.Generator().manual_seed(1234)
    shape = (8, 32, 128, 16, 16)
    x = 0.5 + torch.randn(shape, generator=gen)
    g = torch.randn(shape, generator=gen)
    return x, g


def assert_grad_close(got, want, rtol=1e-4, atol=1e-6, what="grad"):
    """Gradient parity: within 1e-4 relative, with an absolute floor for near-zero entries."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} entries off; "
                           f"max err {err.max():.3e} at value {want.flat[err.argmax()]:.6g}")
