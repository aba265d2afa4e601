"""Shared test helpers: configurations named in BASELINE.json and seeded inputs."""
import numpy as np

from inferred_thoughts_b200.configs import TINY, MID, ODD, M35B, L177B  # noqa: F401


def oracle_dims(d):
    from oracle import oracle_py as O
    return O.ModelDims(**d)


def prompt_ids(seed, n, n_vocab):
    """Uniform-random token ids from a seeded generator."""
    return np.random.default_rng(seed).integers(0, n_vocab, n).astype(np.uint32)


def noise(n, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(n) * scale).astype(np.float32)


def host_dims(d):
    from inferred_thoughts_b200 import host
    return host.ModelDims(**d)


def cosine(a, b):
    a = a.astype(np.float64); b = b.astype(np.float64)
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))
