"""TEST INFRASTRUCTURE -- plain-torch restatement of the reference's Muon hot path.

Nothing in the product imports this module: only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` do, as the checker or the timed CPU
baseline, never as the thing shipped.

Every function restates one piece of nil0x9/flash-muon line by line with ordinary torch ops, so it
runs on CPU tensors (the oracle proper) and, unchanged, on CUDA tensors (where it is the
"plain PyTorch" comparison for the floating-point kernels).

Pinning: the reference holds no tests, golden vectors or fixtures.  The oracle is pinned against
outputs of the reference itself run on CPU (``tests/golden/make_golden.py`` imports a checkout of
the reference: ``benchmark.py``'s torch functions unmodified; ``flash_muon/muon.py`` with its
Triton launch replaced by a CPU matmul, the only part that cannot execute without a GPU; the Triton
kernel itself under the interpreter in fp32).  ``tests/test_oracle_golden.py`` checks the oracle
against those committed fixtures.
"""
from __future__ import annotations

import torch
from torch import Tensor

NS_COEFFS = (3.4445, -4.7750, 2.0315)  # flash_muon/muon.py:14


def matmul_transpose(x: Tensor, native: bool = False) -> Tensor:
    """``x @ x.T`` as the reference kernel produces it.

    flash_muon/matmul_transpose_triton.py:53 accumulates in fp32, :63 casts once to the input
    dtype, :43-44 computes only tiles on or above the diagonal and :71-75 stores each of them
    transposed as well, so the lower triangle is a copy of the upper one.

    ``native=True`` lets the device's matmul of the input dtype do the product (on CUDA: 16-bit
    operands on tensor cores, fp32 accumulation, one rounding -- what ``tl.dot`` does at :58);
    the default upcasts first, which is exact fp32 accumulation on any device.  Both have the same
    rounding points and differ only in the order of the fp32 additions.
    """
    assert x.ndim == 2
    y = (x @ x.T) if native else (x.float() @ x.float().T).to(x.dtype)
    upper = torch.triu(y)
    return upper + torch.triu(y, diagonal=1).T


def torch_matmul_transpose(x: Tensor) -> Tensor:
    """The reference's baseline ``G @ G.T`` (benchmark.py:20-21)."""
    return x @ x.T


def newtonschulz(G: Tensor, steps: int = 5, native: bool = False) -> Tensor:
    """``fast_newtonschulz`` (flash_muon/muon.py:6-33) with its rounding points.

    :15 cast to bf16, :16-17 transpose tall inputs, :23 normalise (norm, +1e-7 and the quotient
    are three bf16 results), :26-27 two symmetric products rounded to bf16, :28 three bf16
    elementwise results, :29 a bf16 matmul and two bf16 elementwise results, :31-32 transpose back.
    """
    assert G.ndim >= 2
    a, b, c = NS_COEFFS
    X = G.bfloat16()
    if G.size(-2) > G.size(-1):
        X = X.mT
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        buf1 = matmul_transpose(X, native)
        buf2 = matmul_transpose(buf1, native)
        B = b * buf1 + c * buf2
        X = a * X + B @ X
    if G.size(-2) > G.size(-1):
        X = X.mT
    return X


def torch_newtonschulz5(G: Tensor, steps: int = 5) -> Tensor:
    """The reference's plain-torch baseline (benchmark.py:23-47); note ``c * A @ A`` there
    parses as ``(c * A) @ A``."""
    assert len(G.shape) == 2
    a, b, c = NS_COEFFS
    X = G.bfloat16()
    if G.size(0) > G.size(1):
        X = X.T
    X = X / (X.norm() + 1e-7)
    for _ in range(steps):
        A = X @ X.T
        B = b * A + c * A @ A
        X = a * X + B @ X
    if G.size(0) > G.size(1):
        X = X.T
    return X


def momentum_update(g: Tensor, buf: Tensor, momentum: float, nesterov: bool) -> Tensor:
    """flash_muon/muon.py:99-100, in place on ``buf`` and (Nesterov) on ``g``; returns the
    tensor the reference hands to Newton-Schulz."""
    buf.lerp_(g, 1 - momentum)
    return g.lerp_(buf, momentum) if nesterov else buf


def apply_update(p: Tensor, g_flat: Tensor, lr: float, weight_decay: float) -> None:
    """flash_muon/muon.py:87-89, in place on ``p``."""
    p.mul_(1 - lr * weight_decay)
    p.add_(g_flat.view_as(p), alpha=-lr * max(1, p.size(-2) / p.size(-1)) ** 0.5)


def owner_of(index_in_group: int, world_size: int) -> int:
    """Round-robin ownership inside a numel group (flash_muon/muon.py:90-92)."""
    return index_in_group % world_size


def muon_step(params: list[Tensor], grads: list[Tensor], momentum_buffers: dict, *,
              lr: float = 0.02, weight_decay: float = 0.01, momentum: float = 0.95,
              nesterov: bool = True, ns_steps: int = 5, world_size: int = 1,
              native: bool = False) -> None:
    """One ``Muon.step()`` (flash_muon/muon.py:75-110) for ALL ranks of a data-parallel job,
    simulated in one process.

    Every rank holds identical ``params`` and ``grads``, so the replicas are represented once.
    ``momentum_buffers`` maps parameter index -> buffer and stands for the union of the
    per-owner states (:95-98).  Groups are keyed by numel (:68); inside a group rank ``r`` owns
    ``params[base + r]`` (:90-92), computes momentum (:99-100), flattens conv filters (:101-102),
    orthogonalises (:103); the all-gather (:108) hands every update to every rank, which applies
    weight decay and the scaled update to every parameter (:86-89).  ``grads[i]`` is overwritten
    by the Nesterov lerp as ``p.grad`` is in the reference (:100).
    """
    sizes = sorted({p.numel() for p in params})
    for size in sizes:
        idx = [i for i, p in enumerate(params) if p.numel() == size]
        for base in range(0, len(idx), world_size):
            round_idx = idx[base: base + world_size]
            updates = []
            for i in round_idx:  # each is computed by rank owner_of(position, world_size)
                g = grads[i]
                if i not in momentum_buffers:
                    momentum_buffers[i] = torch.zeros_like(g)
                g = momentum_update(g, momentum_buffers[i], momentum, nesterov)
                if g.ndim == 4:
                    g = g.view(len(g), -1)
                updates.append(newtonschulz(g, steps=ns_steps, native=native).flatten())
            for i, u in zip(round_idx, updates):
                apply_update(params[i], u, lr, weight_decay)
