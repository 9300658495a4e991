"""Shared helpers of the test-suite."""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "reference_cuda.npz")

# north-star tolerances: forward rtol 1e-5 (fp32) / 2e-3 (fp16); fp32 gradients 1e-4 relative.
# A purely relative test is meaningless at zero crossings, so every comparison adds the same
# fraction of the tensor's rms as absolute slack:  |a - b| <= tol * (|b| + rms(b)).
FWD_TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.float64: 1e-12}
# Half gradients are accumulated by atomics IN HALF, in whatever order the hardware serves them
# (the reference does the same): two runs of the reference's own kernel differ by several
# half ulps of the running sum, so the half backward bound is that run-to-run spread.
BWD_TOL = {torch.float32: 1e-4, torch.float16: 6e-2, torch.float64: 1e-11}


def bits(t):
    """Integer view for exact comparison (distinguishes nothing but the bit pattern)."""
    t = t.detach().cpu().contiguous()
    return t.view({2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()])


def n_mismatch(a, b):
    a, b = a.detach().cpu(), b.detach().cpu()
    # +0 and -0 compare equal on purpose: no consumer of the op can tell them apart
    return int((a.double() != b.double()).sum())


def assert_close(a, b, tol, what=""):
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    assert a.shape == b.shape, (a.shape, b.shape)
    rms = float(b.pow(2).mean().sqrt()) if b.numel() else 0.0
    err = (a - b).abs()
    bound = tol * (b.abs() + rms)
    bad = err > bound
    assert not bool(bad.any()), "%s: %d of %d elements differ beyond tol %g (max abs err %g, rms %g)" % (
        what, int(bad.sum()), a.numel(), tol, float(err.max()), rms)


def load_golden():
    z = np.load(GOLDEN)
    return z


def golden_tensor(z, key, dtype):
    a = z[key]
    t = torch.from_numpy(a.copy())
    if dtype == torch.float16:
        t = t.view(torch.int16).view(torch.float16) if t.dtype != torch.int16 else t.view(torch.float16)
    return t
