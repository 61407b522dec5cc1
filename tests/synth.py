"""Seeded synthetic inputs shared by the tests, the golden-fixture generator and the benchmark.

Everything is drawn on the CPU from ``torch.Generator().manual_seed(seed)`` in a
fixed order, so the oracle, the reference and the CUDA path see identical bits.
The recipes restate the benchmark configurations: standard-normal values times a
per-channel (last dimension) log-normal scale with sparse x20 outliers, and a
Student-t (nu = 4) variant with a wider channel spread.
"""
from __future__ import annotations

import torch

EDGE_NUMELS = (0, 1, 31, 32, 33, 65, 1024, 1027)


def config0_style(seed: int, shape) -> torch.Tensor:
    """bf16 tensor: N(0,1) x lognormal(0, 0.5) per channel, 0.1 % of entries x 20."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    ch = torch.exp(0.5 * torch.randn(shape[-1], generator=g))
    x = x * ch
    mask = torch.rand(shape, generator=g) < 0.001
    x = torch.where(mask, 20 * x, x)
    return x.to(torch.bfloat16)


def config0_chunks(seed: int, total: int, seq_len: int, dim: int, chunk: int = 128):
    """Yields [<=chunk, seq_len, dim] bf16 blocks drawn from ONE generator in sample order."""
    g = torch.Generator().manual_seed(seed)
    ch = None
    done = 0
    while done < total:
        b = min(chunk, total - done)
        x = torch.randn((b, seq_len, dim), generator=g)
        if ch is None:
            ch = torch.exp(0.5 * torch.randn(dim, generator=g))
        x = x * ch
        mask = torch.rand((b, seq_len, dim), generator=g) < 0.001
        yield torch.where(mask, 20 * x, x).to(torch.bfloat16)
        done += b


def config2_slices(n_slices: int, seed: int = 2, rows: int = 1024, cols: int = 1024) -> torch.Tensor:
    """First ``n_slices`` leading slices of the Student-t(4) x lognormal(0,1) tensor, bf16."""
    g = torch.Generator().manual_seed(seed)
    ch = torch.exp(1.0 * torch.randn(cols, generator=g))
    out = torch.empty((n_slices, rows, cols), dtype=torch.bfloat16)
    for b in range(n_slices):
        z = torch.randn((rows, cols), generator=g)
        w = torch.randn((4, rows, cols), generator=g)
        out[b] = (z / torch.sqrt((w * w).sum(0) / 4) * ch).to(torch.bfloat16)
    return out


def config3_tensors(seed: int = 3, rows_x: int = 8192, rows_w: int = 14336, k: int = 4096):
    """(X bf16 [rows_x, k] ~ N(0,1), W bf16 [rows_w, k] ~ N(0, std 0.02)).

    W is drawn first so that it does not depend on how many rows of X are asked for.
    """
    g = torch.Generator().manual_seed(seed)
    W = (0.02 * torch.randn((rows_w, k), generator=g)).to(torch.bfloat16)
    X = torch.randn((rows_x, k), generator=g).to(torch.bfloat16)
    return X, W


def edge_values() -> torch.Tensor:
    """fp32 [4096]: NaN / +-Inf, constant groups, huge and tiny magnitudes."""
    g = torch.Generator().manual_seed(103)
    x = torch.randn(4096, generator=g)
    x[5] = float("nan")
    x[40] = float("inf")
    x[41] = float("-inf")
    x[64:96] = float("nan")
    x[128:160] = 3.0
    x[160:192] = -3.0
    x[192:224] = 0.0
    x[224:256] = 1e30
    x[300] = -1e38
    x[301] = 3e38
    x[320:352] = torch.randn(32, generator=g) * 1e-39
    x[352:384] = 1e-30
    x[400:464] = torch.randn(64, generator=g) * 6e4
    return x
