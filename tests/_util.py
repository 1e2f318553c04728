"""Seeded input builders shared by the GPU parity tests."""
import numpy as np
import torch

RTOL = 2e-2  # bf16 outputs against the fp32 oracle
ATOL = 2e-2


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    """Round to bf16 and return as fp32: what the oracle sees when the kernels see bf16."""
    return t.to(torch.bfloat16).float()


def gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def zipf_indices(t: int, k: int, n: int, s: float, seed: int) -> torch.Tensor:
    """Expert ids drawn with replacement from p(e) ~ (e+1)^-s by inverse CDF."""
    rng = np.random.default_rng(seed)
    p = (np.arange(1, n + 1, dtype=np.float64)) ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = rng.random((t, k))
    return torch.from_numpy(np.minimum(np.searchsorted(cdf, u), n - 1).astype(np.int32))


def assert_close(actual: torch.Tensor, expected: torch.Tensor, rtol=RTOL, atol=ATOL, what=""):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    bad = (a - e).abs() > atol + rtol * e.abs()
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.numel()} elements outside rtol={rtol} atol={atol}; "
                           f"max abs err {float((a - e).abs().max()):.4g}")
