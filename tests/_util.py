"""Shared helpers for the tests: golden-fixture loading and error norms."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        out[k] = torch.from_numpy(a) if a.ndim > 0 else a.item()
    return out


def opt_mask(t):
    return None if (t is None or t.numel() == 0) else t.bool()


def rel_l2(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    d = (a - b).norm()
    n = b.norm()
    return float(d / n) if n > 0 else float(d)


def make_ema_params(gen, dim, ndim, bidirectional=False, device="cpu"):
    k = 2 * dim if bidirectional else dim
    alpha = torch.randn(k, ndim, 1, generator=gen) * 0.2
    delta = torch.randn(k, ndim, 1, generator=gen) * 0.2
    val = torch.ones(ndim, 1)
    val[1::2] = -1.0
    beta = torch.randn(k, ndim, 1, generator=gen) * 0.02 + val
    gamma = torch.randn(k, ndim, generator=gen)
    omega = torch.randn(dim, generator=gen)
    return [t.to(device) for t in (alpha, delta, beta, gamma, omega)]


def right_pad_mask(gen, bsz, length, frac):
    mask = torch.zeros(bsz, length, dtype=torch.bool)
    for b in range(bsz):
        n = int(torch.rand((), generator=gen).item() * frac * length)
        if n:
            mask[b, length - n:] = True
    return mask
