"""Shared helpers of the GPU parity tests."""
import functools

import numpy as np
import pytest

import kalosm_b200 as kb
from oracle import oracle as O

TYPES = {"q4_0": O.Q4_0, "q8_0": O.Q8_0, "q4k": O.Q4K, "q6k": O.Q6K}


@functools.lru_cache(maxsize=1)
def device():
    """The test session's device handle. Fails (does not skip) when the CUDA library or a GPU is
    missing: GPU tests never fall back to a CPU path."""
    return kb.Device(0)


@pytest.fixture(scope="session")
def dev():
    return device()


def weights(seed, n, k, ty, sigma=0.02):
    """Seeded N(0, sigma) weights quantised by the oracle's encoder; both sides use these bytes."""
    return O.random_qweights(seed, sigma, n * k, ty)


def activations(seed, m, k):
    return O.normal(1000 + seed, 1.0, m * k).reshape(m, k)
