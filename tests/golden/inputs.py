"""Seeded inputs shared by the golden-vector generator and the tests (CPU generators, so the same
values are produced in the build container and on a GPU box)."""
from __future__ import annotations

import torch

# (M, K, dtype) cases of the symmetric product
SYRK_CASES = [(96, 80, torch.float32), (128, 96, torch.bfloat16), (200, 72, torch.bfloat16)]
# Newton-Schulz input shapes: wide, tall, square, not multiples of any tile
NS_SHAPES = [(64, 96), (96, 64), (128, 128), (100, 72)]

MUON_HP = dict(lr=0.02, weight_decay=0.01, momentum=0.95, nesterov=True, ns_steps=5)
# three numel groups: 1536 (4 params, wide/tall mix), 1600 (3 params -> partial round at ws 2),
# 288 (a conv filter and a matrix of the same numel)
MUON_SHAPES = [(32, 48), (48, 32), (40, 40), (32, 48), (8, 4, 3, 3), (64, 24), (40, 40), (16, 18),
               (40, 40)]


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def syrk_input(m: int, k: int, dtype: torch.dtype) -> torch.Tensor:
    return (torch.randn(m, k, generator=_gen(100 + m + k)) / k ** 0.5).to(dtype)


def ns_input(rows: int, cols: int) -> torch.Tensor:
    return torch.randn(rows, cols, generator=_gen(200 + 7 * rows + cols))


def muon_case(steps: int, shapes=MUON_SHAPES, dtype=torch.bfloat16, seed: int = 0):
    """Returns (params, grads_per_step): params ~ N(0, 0.02), grads ~ N(0, 1e-3), in ``dtype``."""
    g = _gen(seed)
    params = [(torch.randn(*s, generator=g) * 0.02).to(dtype) for s in shapes]
    grads = []
    for t in range(steps):
        gt = _gen(1000 + t + seed)
        grads.append([(torch.randn(*s, generator=gt) * 1e-3).to(dtype) for s in shapes])
    return params, grads
