"""Shared pieces of the parity tests: tolerances and the oracle import (tests may use oracle/, the product may not)."""
from __future__ import annotations

import numpy as np

from oracle import np_oracle, sl_oracle  # noqa: F401  (re-exported for the tests)

TYPE_OF = {2: "Q4_0", 6: "Q5_0", 8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 20: "IQ4_NL"}
FMT_OF = {v: k for k, v in TYPE_OF.items()}

# fp32 outputs: max relative error 1e-3 against the oracle's integer-dot result on the same quantized inputs.
# Outputs that cancel to (almost) nothing are measured against EPS_FLOOR x the row's RMS instead of their own size.
MAX_REL = 1e-3
EPS_FLOOR = 1e-2


def max_rel_error(y: np.ndarray, ref: np.ndarray) -> float:
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    if y.size == 0:
        return 0.0
    rms = np.sqrt(np.mean(ref * ref, axis=-1, keepdims=True))
    denom = np.maximum(np.abs(ref), EPS_FLOOR * rms)
    denom = np.where(denom == 0, 1.0, denom)
    return float(np.max(np.abs(y - ref) / denom))


def relative_rms(y: np.ndarray, ref: np.ndarray) -> float:
    """sqrt(sum (y - ref)^2 / sum ref^2): the measure of QuantTests.MatMulWithIntDotMatchesReference."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    den = float(np.sum(ref * ref))
    return float(np.sqrt(np.sum((y - ref) ** 2) / den)) if den > 0 else float(np.sqrt(np.sum((y - ref) ** 2)))


def same_floats(a: np.ndarray, b: np.ndarray) -> bool:
    """Equal as numbers (+0 == -0), NaN matching NaN."""
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return bool(np.all((a == b) | (np.isnan(a) & np.isnan(b))))
