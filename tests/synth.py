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


def seed_scoring_case(n_cand: int, n_seed: int, people: int, dims: int, vetoes: bool, cannot_links: bool,
                      users: bool, seed: int):
    """The scenario shape of the reference's grouped-vs-one-at-a-time test
    (media-server/tasks/face_score_kernel_test.go:80-150) over this repo's own seeded generator:
    people with tight seed clouds (spread 0.02), every third candidate near a person's centre
    (spread 0.03), the rest junk; optional vetoes (every 4th candidate from 1), cannot-links
    (every 6th from 2) and user seeds (every 5th)."""
    rng = np.random.default_rng(seed)

    def unit(v):
        v = v.astype(np.float32)
        return (v / np.sqrt(np.sum(v.astype(np.float64) ** 2))).astype(np.float32)

    centres = [unit(rng.standard_normal(dims)) for _ in range(people)]
    seed_ids = [i + 1 for i in range(n_seed)]
    seed_person = [i % people + 1 for i in range(n_seed)]
    seed_user = [bool(users and i % 5 == 0) for i in range(n_seed)]
    seed_vecs = np.stack([unit(centres[seed_person[i] - 1] + 0.02 * rng.standard_normal(dims)) for i in range(n_seed)])
    cand_ids = [1_000_000 + i for i in range(n_cand)]
    cand_vecs = np.stack([unit(centres[i % people] + 0.03 * rng.standard_normal(dims)) if i % 3 == 0
                          else unit(rng.standard_normal(dims)) for i in range(n_cand)])
    veto = {cand_ids[i]: {i % people + 1} for i in range(1, n_cand, 4)} if vetoes else {}
    cannot = {cand_ids[i]: {seed_ids[(i * 3) % n_seed]} for i in range(2, n_cand, 6)} if cannot_links else {}
    return dict(cand_ids=cand_ids, cand_vecs=cand_vecs, seed_ids=seed_ids, seed_vecs=seed_vecs,
                seed_person=seed_person, seed_user=seed_user, vetoes=veto, cannot=cannot)


# (name, n_cand, n_seed, people, dims, threshold, vetoes, cannot-links, user seeds): the reference's table
SEED_SCORING_CASES = [
    ("plain", 200, 500, 10, 64, 0.42, False, False, False),
    ("candidate count not a multiple of the group width", 203, 501, 7, 64, 0.42, False, False, False),
    ("seed count straddling the chunk boundary", 64, 257, 5, 64, 0.42, False, False, False),
    ("with user seeds", 200, 500, 8, 64, 0.42, False, False, True),
    ("with vetoes", 200, 500, 8, 64, 0.42, True, False, True),
    ("with cannot-links", 200, 500, 8, 64, 0.42, False, True, True),
    ("everything at once, low threshold", 300, 800, 12, 32, 0.20, True, True, True),
    ("single candidate", 1, 300, 4, 64, 0.42, True, True, True),
    ("fewer candidates than the group width", 3, 300, 4, 64, 0.42, True, True, True),
]


def device_corpus(lk, n: int, dim: int, store: int, seed: int, clustered: bool = False, centres: int = 256,
                  sigma: float = 0.1, sample_every: int = 4099, chunk: int = 62_500, device: int = 0):
    """A corpus of a benchmark configuration's full size, generated on the GPU in chunks
    (seeded N(0,1); with `clustered` the odd rows sit around un-normalised Gaussian centres) and
    handed to the index as device rows, so that no multi-gigabyte float array crosses the host.
    Returns (index, sample_ids, sample_rows): the float32 input of every `sample_every`-th row,
    kept on the host to check the stored form of those rows against the oracle."""
    import torch

    dev = torch.device("cuda", device)
    idx = lk.DeviceIndex(dim, store, device=device)
    idx.reserve(n)
    gen = torch.Generator(device=dev)
    cen = None
    if clustered:
        gen.manual_seed(seed + 2000)
        cen = torch.randn((centres, dim), generator=gen, device=dev, dtype=torch.float32)
    ids, rows = [], []
    for c0 in range(0, n, chunk):
        m = min(chunk, n - c0)
        gen.manual_seed(seed * 1_000_003 + c0)
        block = torch.randn((m, dim), generator=gen, device=dev, dtype=torch.float32)
        if clustered:
            gid = torch.arange(c0, c0 + m, device=dev)
            odd = (gid % 2) == 1
            block[odd] = cen[(gid[odd] // 2) % centres] + sigma * block[odd]
        torch.cuda.synchronize(dev)
        idx.upsert_device(c0, m, block.data_ptr())
        pick = np.arange((-c0) % sample_every, m, sample_every)
        if pick.size:
            ids.append(pick + c0)
            rows.append(block[torch.as_tensor(pick, device=dev)].cpu().numpy())
        del block
    assert len(idx) == n
    return idx, np.concatenate(ids), np.concatenate(rows)
