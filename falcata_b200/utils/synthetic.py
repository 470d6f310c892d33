"""Seeded synthetic data of the five benchmark shapes.

Rows are generated in fixed chunks of ``CHUNK`` rows, each from its own generator seeded by the
chunk index, so rows ``[offset, offset + n)`` are the same numbers whichever rank (and however many
ranks) asks for them: a model trained on 1, 2, 4 or 8 shards sees the same global data set.
Everything derived from the random draws (interaction features, logits, labels) is computed on the
WHOLE chunk and sliced afterwards: a reduction or matrix product over a slice whose shape depends on
the shard may pick another kernel and round differently, which would flip a label near its threshold.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

CHUNK = 1 << 18


def _gen(seed: int, chunk: int, device: torch.device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + chunk) & 0x7FFFFFFFFFFF)
    return g


def _chunks(offset: int, n: int):
    c = offset // CHUNK
    pos = offset
    end = offset + n
    while pos < end:
        lo = pos - c * CHUNK
        hi = min(CHUNK, end - c * CHUNK)
        yield c, lo, hi
        pos = c * CHUNK + hi
        c += 1


def binary_small(n: int = 10000, f: int = 28, seed: int = 0, device: str = "cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """10k x 28 N(0,1); label = 1[x.w + 0.5 eps > 0] (the CPU benchmark shape)."""
    dev = torch.device(device)
    g = _gen(seed, 0, dev)
    x = torch.randn(n, f, generator=g, device=dev)
    w = torch.randn(f, generator=g, device=dev)
    eps = torch.randn(n, generator=g, device=dev)
    return x, ((x @ w + 0.5 * eps) > 0).float()


def binary_higgs_like(n: int, offset: int = 0, seed: int = 0, device: str = "cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """28 features: 21 N(0,1) + 7 |x_i * x_j| interactions; label ~ Bernoulli(sigmoid(x.w + 0.5 x0 x1))."""
    dev = torch.device(device)
    gw = _gen(seed, 1 << 30, torch.device("cpu"))
    w = (torch.randn(28, generator=gw) * 0.3).to(dev)
    pairs = torch.randint(0, 21, (7, 2), generator=gw)
    xs, ys = [], []
    for c, lo, hi in _chunks(offset, n):
        g = _gen(seed, c, dev)
        base = torch.randn(CHUNK, 21, generator=g, device=dev)
        u = torch.rand(CHUNK, generator=g, device=dev)
        inter = torch.stack([(base[:, int(i)] * base[:, int(j)]).abs() for i, j in pairs.tolist()], dim=1)
        x = torch.cat([base, inter], dim=1)
        logit = x @ w + 0.5 * x[:, 0] * x[:, 1]
        label = (u < torch.sigmoid(logit)).float()
        xs.append(x[lo:hi].clone())
        ys.append(label[lo:hi].clone())
        del base, inter, x, logit, label, u
    return torch.cat(xs), torch.cat(ys)


def regression_wide(n: int, f: int = 2000, offset: int = 0, seed: int = 0, device: str = "cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """Integer features: 0 with p=0.8 else uniform in 1..15; y = sum over 50 features of sin(x_f) c_f + N(0,1)."""
    dev = torch.device(device)
    gw = _gen(seed, 1 << 30, torch.device("cpu"))
    sel = torch.randperm(f, generator=gw)[:50].to(dev)
    coef = (torch.rand(50, generator=gw) * 4 - 2).to(dev)
    xs, ys = [], []
    for c, lo, hi in _chunks(offset, n):
        g = _gen(seed, c, dev)
        nz = torch.rand(CHUNK, f, generator=g, device=dev) >= 0.8
        val = torch.randint(1, 16, (CHUNK, f), generator=g, device=dev, dtype=torch.int8)
        x = torch.where(nz, val, torch.zeros_like(val))
        del nz, val
        noise = torch.randn(CHUNK, generator=g, device=dev)
        y = (torch.sin(x[:, sel].float()) * coef).sum(1) + noise
        xs.append(x[lo:hi].clone()); ys.append(y[lo:hi].clone())
        del x, y, noise
    return torch.cat(xs), torch.cat(ys)


def multiclass(n: int, f: int = 100, k: int = 10, offset: int = 0, seed: int = 0, device: str = "cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """N(0,1) features; label = argmax(x W + Gumbel)."""
    dev = torch.device(device)
    gw = _gen(seed, 1 << 30, torch.device("cpu"))
    W = torch.randn(f, k, generator=gw).to(dev)
    xs, ys = [], []
    for c, lo, hi in _chunks(offset, n):
        g = _gen(seed, c, dev)
        x = torch.randn(CHUNK, f, generator=g, device=dev)
        u = torch.rand(CHUNK, k, generator=g, device=dev).clamp_(1e-9, 1 - 1e-9)
        gum = -torch.log(-torch.log(u))
        label = (x @ W + gum).argmax(1).float()
        xs.append(x[lo:hi].clone()); ys.append(label[lo:hi].clone())
        del x, u, gum, label
    return torch.cat(xs), torch.cat(ys)


def ranking(num_queries: int, docs: int = 100, f: int = 136, query_offset: int = 0, seed: int = 0, device: str = "cuda"):
    """U(0,1) features with 30% exact zeros; relevance 0..4 from per-query quintiles of x.w + N(0, 0.5^2)."""
    dev = torch.device(device)
    gw = _gen(seed, 1 << 30, torch.device("cpu"))
    w = torch.randn(f, generator=gw).to(dev)
    qchunk = max(1, CHUNK // docs)
    xs, ys = [], []
    q = query_offset
    end = query_offset + num_queries
    while q < end:
        c = q // qchunk
        lo = q - c * qchunk
        hi = min(qchunk, end - c * qchunk)
        g = _gen(seed, c, dev)
        x = torch.rand(qchunk * docs, f, generator=g, device=dev)
        z = torch.rand(qchunk * docs, f, generator=g, device=dev) < 0.3
        x = torch.where(z, torch.zeros_like(x), x)
        s = x @ w + 0.5 * torch.randn(qchunk * docs, generator=g, device=dev)
        s = s.view(qchunk, docs)
        rank = s.argsort(dim=1).argsort(dim=1)
        rel = (rank * 5 // docs).float().view(-1)
        xs.append(x[lo * docs:hi * docs]); ys.append(rel[lo * docs:hi * docs])
        q = c * qchunk + hi
    group = torch.full((num_queries,), docs, dtype=torch.int32)
    return torch.cat(xs), torch.cat(ys), group


def shard(total: int, rank: int, world: int, align: int = 1) -> Tuple[int, int]:
    """(offset, count) of this rank's contiguous row range; ``align`` keeps query groups whole."""
    units = total // align
    per = (units + world - 1) // world
    lo = min(units, rank * per)
    hi = min(units, lo + per)
    return lo * align, (hi - lo) * align
