"""Seeded synthetic inputs with the shapes and distributions of the benchmark
configurations, and comparison helpers shared by the tests."""
from __future__ import annotations

import numpy as np


def normal_logits(rows, V, sigma, seed):
    return (np.random.default_rng(seed).standard_normal((rows, V), dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def gumbel_logits(rows, V, scale, seed):
    u = np.random.default_rng(seed).random((rows, V), dtype=np.float64)
    u = np.clip(u, 1e-300, 1.0 - 1e-16)
    return (scale * -np.log(-np.log(u))).astype(np.float32)


def histories(rows, H, V, seed):
    return np.random.default_rng(seed).integers(0, V, size=(rows, H), dtype=np.int32)


def seq_states(oracle_port, seed, n):
    """One reference generator seeded with `seed`; entry r is its state after r draws,
    so a batch of n single-row sequences reproduces a CPU loop over rows with one rng."""
    s = oracle_port.rng_seed(seed)
    out = np.empty(n, np.uint64)
    for r in range(n):
        out[r] = s
        s = oracle_port.rng_advance(s, 1)
    return out


def independent_states(oracle_port, seed, n):
    return np.array([oracle_port.rng_seed(seed + i) for i in range(n)], dtype=np.uint64)


def to_dev(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def u64_to_dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, np.uint64).view(np.int64)).cuda()


def u64_from_dev(t):
    return t.cpu().numpy().view(np.uint64)


def per_seq(n, T, K, P):
    import torch
    T = np.broadcast_to(np.asarray(T, np.float32), (n,))
    K = np.broadcast_to(np.asarray(K, np.int32), (n,))
    P = np.broadcast_to(np.asarray(P, np.float32), (n,))
    return to_dev(T), to_dev(K), to_dev(P)


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-30)) if a.size else 0.0
