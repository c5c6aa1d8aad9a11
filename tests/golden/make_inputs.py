"""Seeded inputs shared by make_golden.py and the tests (numpy PCG64, no torch RNG)."""

import numpy as np


def layer_cfg1_weights(seed=0, D=128, ff=512, E=8):
    """Weights N(0, 0.02) for the config-1 layer, from numpy's PCG64 (also used by the tests)."""
    rng = np.random.default_rng(seed)
    router = (rng.standard_normal((E, D)) * 0.02).astype(np.float32)
    w1 = (rng.standard_normal((E, ff, D)) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((E, D, ff)) * 0.02).astype(np.float32)
    x = rng.standard_normal((256, D)).astype(np.float32)
    target = rng.standard_normal((256, D)).astype(np.float32)
    return router, w1, w2, x, target
