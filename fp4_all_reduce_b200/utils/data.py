"""Deterministic synthetic inputs.

* `partial(rows, rank)`        the benchmark distribution: N(0,1) times a per-row lognormal(0,1) scale with
                               0.1 % of the elements multiplied by 50, generated from seed = rank.
* `gaussian_mags(rows, src, seed)`  the reference project's gate input in spirit (harness/ref.cuh:11-28):
                               N(0,1) times a per-source magnitude plus 32 outliers of +-40 x magnitude.
* `special_rows(rows, src)`    twelve classes of adversarial rows (all zero, all -0, random finite bits,
                               subnormal rows whose row scale overflows, huge rows, one 1e30 outlier, E2M1
                               rounding midpoints, saturating blocks, smallest subnormals, BF16 max, an
                               exponent ramp, mixed blocks), the classes of bench/codec/codec_bench.cu:702-723.

All generators return torch.bfloat16 tensors of shape [rows, 6144] on the requested device and are
pure functions of their arguments.
"""
from __future__ import annotations

import numpy as np
import torch

H = 6144
MAGS = (1.0, 0.5, 2.0, 0.25, 1.5, 0.75, 3.0, 0.125)


def partial(rows: int, rank: int, device="cpu", seed_offset: int = 0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(rank + 1000003 * seed_offset)
    x = torch.randn(rows, H, generator=g)
    scale = torch.exp(torch.randn(rows, 1, generator=g))
    mask = torch.rand(rows, H, generator=g) < 1e-3
    x = x * scale
    x = torch.where(mask, x * 50.0, x)
    return x.to(torch.bfloat16).to(device)


def gaussian_mags(rows: int, src: int, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(1000 + 17 * rows + 7777 * seed + 131 * src)
    mag = MAGS[src & 7]
    x = torch.randn(rows, H, generator=g) * mag
    n = rows * H
    pos = torch.randint(0, n, (32,), generator=g)
    sign = torch.randint(0, 2, (32,), generator=g).float() * 2 - 1
    x.view(-1)[pos] = sign * 40.0 * mag
    return x.to(torch.bfloat16).to(device)


def residual(rows: int, seed: int = 12345, device="cpu") -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(rows, H, generator=g).to(torch.bfloat16).to(device)


def norm_weight(seed: int = 777, device="cpu") -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(H, generator=g) * 0.02).to(torch.bfloat16).to(device)


def special_rows(rows: int, src: int, device="cpu") -> torch.Tensor:
    """Row r is of class (r + 7 * src) % 16 for classes 0..11; classes 12..15 are plain Gaussian rows."""
    rng = np.random.default_rng(1234 + src)
    base = gaussian_mags(rows, src, 99).view(torch.int16).numpy().view(np.uint16).copy()

    def sign():
        return (rng.integers(0, 2, H, dtype=np.uint16) << 15).astype(np.uint16)

    for r in range(rows):
        k = (r + 7 * src) % 16
        p = base[r]
        if k == 0:
            p[:] = 0
        elif k == 1:
            p[:] = 0x8000
        elif k == 2:   # random finite bit patterns
            u = rng.integers(0, 1 << 16, H, dtype=np.uint32).astype(np.uint16)
            u[((u >> 7) & 0xFF) == 0xFF] &= 0xBFFF
            p[:] = u
        elif k == 3:   # tiny / subnormal: the row scale's inverse overflows to inf
            p[:] = (rng.integers(0, 128, H, dtype=np.uint16) | (rng.integers(0, 2, H, dtype=np.uint16) << 7)) | sign()
        elif k == 4:   # huge
            p[:] = 0x7E00 | rng.integers(0, 256, H, dtype=np.uint16) | sign()
        elif k == 5:   # blocks of zero / tiny / large / signed zero
            b = (np.arange(H) // 16) % 4
            tiny = 0x0100 | rng.integers(0, 128, H, dtype=np.uint16) | sign()
            large = 0x4500 | rng.integers(0, 256, H, dtype=np.uint16) | sign()
            p[:] = np.where(b == 0, 0, np.where(b == 1, tiny, np.where(b == 2, large, sign())))
        elif k == 6:   # one 1e30 outlier: every other block scale underflows
            p[:] = 0x3F00 | rng.integers(0, 256, H, dtype=np.uint16) | sign()
            p[rng.integers(0, H)] = 0x7149
        elif k == 7:   # E2M1 rounding midpoints 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5 (and 6.5)
            mid = np.array([0x3E80, 0x3F40, 0x3FA0, 0x3FE0, 0x4020, 0x4060, 0x40A0, 0x40D0], np.uint16)
            p[:] = mid[rng.integers(0, 8, H)] | sign()
            p[0] = 0x40C0  # a 6.0 so that the row maximum maps exactly onto the grid
        elif k == 8:   # one large value per block, the rest small
            small = 0x3800 | rng.integers(0, 128, H, dtype=np.uint16) | sign()
            p[:] = np.where(np.arange(H) % 16 == 0, 0x43E0, small)
        elif k == 9:   # smallest subnormals
            p[:] = 0x0001 | sign()
        elif k == 10:  # +-BF16 max
            p[:] = 0x7F7F | sign()
        elif k == 11:  # block-wise exponent ramp
            p[:] = ((0x30 + (np.arange(H) // 16) % 0x20).astype(np.uint16) << 8) | rng.integers(0, 256, H, dtype=np.uint16) | sign()
    return torch.from_numpy(base.view(np.int16)).view(torch.bfloat16).to(device)
