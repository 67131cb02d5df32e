"""Per-tensor digests for the committed golden fixtures. TEST INFRASTRUCTURE ONLY: never imported by the product.

A fixture cannot hold the 10^8 gradients of a full-size model, and an L2 norm alone says nothing about
direction (a sign error keeps it). Besides the norm, the mean and a set of fixed entries, a digest therefore
holds a sketch: the inner products of the flattened tensor with NPROJ fixed pseudo-random +-1 vectors. For two
tensors a and b the mean of (proj_k(a) - proj_k(b))^2 over k is an unbiased estimate of |a - b|^2, so a test
can bound the relative L2 distance of a tensor it computed to the one the oracle computed, at 8 * NPROJ bytes
per tensor in the fixture. The sign vectors depend only on the element count and k (numpy PCG64, stable across
numpy versions), so the test re-creates them."""
from __future__ import annotations

import numpy as np

NPROJ = 16
NSAMPLES = 32


_CHUNK = 1 << 22


def sketch(a, nproj: int = NPROJ) -> list:
    """Inner products of the flattened tensor with nproj (<= 16) +-1 vectors. Element i of vector k is bit k of
    the i-th 16-bit word of a PCG64 stream seeded with the element count."""
    assert 1 <= nproj <= 16
    flat = np.ascontiguousarray(np.asarray(a).ravel(), dtype=np.float32)
    rng = np.random.Generator(np.random.PCG64(1000003 + flat.size))
    acc = np.zeros(16, dtype=np.float64)
    total = 0.0
    for o in range(0, flat.size, _CHUNK):
        x = flat[o:o + _CHUNK]
        words = rng.integers(0, 65536, size=x.size, dtype=np.uint16)
        bits = np.unpackbits(words.view(np.uint8).reshape(-1, 2), axis=1, bitorder="little").astype(np.float32)
        acc += (x @ bits).astype(np.float64)
        total += float(x.sum(dtype=np.float64))
    return [float(2.0 * acc[k] - total) for k in range(nproj)]


def sample_index(n: int, samples: int = NSAMPLES) -> np.ndarray:
    return np.linspace(0, n - 1, num=min(samples, n)).astype(np.int64)


def digest(arrays: dict, samples: int = NSAMPLES, nproj: int = NPROJ) -> dict:
    out = {}
    for k, a in arrays.items():
        flat = np.asarray(a, dtype=np.float64).ravel()
        idx = sample_index(flat.size, samples)
        out[k] = {"n": int(flat.size), "l2": float(np.sqrt((flat ** 2).sum())), "mean": float(flat.mean()),
                  "idx": idx.tolist(), "val": [float(flat[i]) for i in idx], "proj": sketch(flat, nproj)}
    return out


def sketch_distance(a, d: dict) -> float:
    """Estimate of |a - b| / |b| for the tensor b behind digest d (relative standard error of the estimate:
    sqrt(2 / NPROJ) / 2, about 18 % with 16 projections)."""
    pa = np.asarray(sketch(a, len(d["proj"])))
    pb = np.asarray(d["proj"])
    return float(np.sqrt(np.mean((pa - pb) ** 2)) / (d["l2"] + 1e-300))


def sample_distance(a, d: dict) -> float:
    """Root-mean-square deviation of the sampled entries, relative to the tensor's root-mean-square entry."""
    flat = np.asarray(a, dtype=np.float64).ravel()
    got = flat[np.asarray(d["idx"], dtype=np.int64)]
    rms = d["l2"] / np.sqrt(d["n"]) + 1e-300
    return float(np.sqrt(np.mean((got - np.asarray(d["val"])) ** 2)) / rms)
