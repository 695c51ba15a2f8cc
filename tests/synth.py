"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (no dataset is involved: the reference measures on none)."""
from __future__ import annotations

import numpy as np


def gaussian_rows(n: int, dim: int, seed: int) -> np.ndarray:
    """n x dim float32, entries i.i.d. N(0,1) (rows are normalised by the index itself)."""
    return np.random.default_rng(seed).standard_normal((n, dim), dtype=np.float32)


def clustered_rows(n: int, dim: int, seed: int, centres: int = 256, sigma: float = 0.1) -> np.ndarray:
    """Half the rows (odd ones) sit around `centres` un-normalised Gaussian centres with
    per-coordinate noise sigma, which makes their int8 scores collide often."""
    rng = np.random.default_rng(seed)
    rows = rng.standard_normal((n, dim), dtype=np.float32)
    cen = np.random.default_rng(seed + 2000).standard_normal((centres, dim), dtype=np.float32)
    odd = np.arange(1, n, 2)
    rows[odd] = cen[(odd // 2) % centres] + np.float32(sigma) * rows[odd]
    return rows


def phash_set(n: int, seed: int, dup_frac: float = 0.1, max_flips: int = 6) -> np.ndarray:
    """n uint64 hashes: (1-dup_frac) uniform random, the rest near-duplicates of a random
    base hash with 0..max_flips distinct bits flipped; then shuffled."""
    rng = np.random.default_rng(seed)
    n_dup = int(n * dup_frac)
    n_base = n - n_dup
    base = rng.integers(0, 2**64, size=n_base, dtype=np.uint64)
    src = rng.integers(0, max(n_base, 1), size=n_dup)
    dup = base[src].copy()
    flips = rng.integers(0, max_flips + 1, size=n_dup)
    for i in range(n_dup):
        bits = rng.choice(64, size=flips[i], replace=False)
        for b in bits:
            dup[i] ^= np.uint64(1) << np.uint64(b)
    allh = np.concatenate([base, dup])
    rng.shuffle(allh)
    return allh
