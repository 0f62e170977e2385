"""Lloyd-Max scalar codebooks for coordinates of a randomly rotated unit vector.

Mirrors the interface of the reference's ``aither_kvcache/codebook.py``
(``get_codebook`` :62-82, ``get_theory_bounds`` :85-89): for d >= 64 a
coordinate is close to N(0, 1/d), so the tabulated N(0,1) quantiser (Max 1960)
is scaled by 1/sqrt(d); decision boundaries are midpoints.  The tables are
constants of the kernels (passed as device arrays per call).
"""
from __future__ import annotations

import math
from typing import Tuple

import numpy as np

# positive halves of the odd-symmetric N(0,1) tables, and the per-vector MSE they give
_POSITIVE = {
    1: ((0.798284,), 0.363480),
    2: ((0.452781, 1.510469), 0.117517),
    3: ((0.245104, 0.756031, 1.344134, 2.152090), 0.034506),
    4: ((0.128350, 0.388089, 0.656804, 0.942391, 1.256233, 1.618002, 2.069016, 2.733266), 0.009497),
}


def get_codebook(d: int, bits: int) -> Tuple[np.ndarray, np.ndarray, float]:
    """(centroids[2^bits], inner boundaries[2^bits-1], total MSE on the unit sphere), float64."""
    if bits not in _POSITIVE:
        raise ValueError(f"Supported bit-widths: {list(_POSITIVE)}. Got {bits}")
    pos, mse = _POSITIVE[bits]
    pos = np.asarray(pos, dtype=np.float64)
    centroids = np.concatenate([-pos[::-1], pos]) * (1.0 / math.sqrt(d))
    boundaries = (centroids[:-1] + centroids[1:]) / 2
    return centroids, boundaries, mse


def get_theory_bounds(bits: int) -> Tuple[float, float]:
    """Lower / upper bound on E||x - x_hat||^2 for b-bit quantisation of unit vectors."""
    return 1.0 / 4 ** bits, (3 * math.pi / 2) / 4 ** bits
