"""Shared helpers of the GPU parity tests."""
import glob
import os

import numpy as np

# self-attention fixtures; the cross_* file (query rows != keys) has its own tests
GOLDEN = sorted(p for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))
                if not os.path.basename(p).startswith("cross_"))
GOLDEN_CROSS = os.path.join(os.path.dirname(__file__), "golden", "cross_b1h2q96k192d64.npz")

# Tolerance of the int8 output against the quantised CPU oracle: |diff| <= 1 LSB on at least
# 99.9 % of the elements and <= 2 LSB everywhere.
MIN_FRAC_WITHIN_1 = 0.999
MAX_ABS_DIFF = 2


def parity_stats(got, want):
    d = np.abs(np.asarray(got, np.int32) - np.asarray(want, np.int32))
    return int(d.max()) if d.size else 0, float((d <= 1).mean()) if d.size else 1.0, float((d == 0).mean()) if d.size else 1.0


def assert_parity(got, want, what=""):
    mx, f1, f0 = parity_stats(got, want)
    assert mx <= MAX_ABS_DIFF and f1 >= MIN_FRAC_WITHIN_1, f"{what}: max|diff|={mx} within1={f1:.6f} exact={f0:.6f}"
    return mx, f1, f0


def sample_rows(B, H, S, per_head, valid=None, seed=0):
    """Flattened row ids (bh*S + i): first/last rows, rows around tile edges and the valid-length
    edge, plus random rows, `per_head` per (b,h)."""
    rng = np.random.default_rng(seed)
    rows = []
    for bh in range(B * H):
        fixed = {0, 1, 63, 64, 127, 128, S - 1, S - 64, S // 2}
        if valid is not None:
            L = int(valid[bh // H])
            fixed |= {max(L - 1, 0), min(L, S - 1)}
        fixed = {r for r in fixed if 0 <= r < S}
        extra = rng.integers(0, S, max(per_head - len(fixed), 0))
        for r in sorted(fixed | set(int(x) for x in extra)):
            rows.append(bh * S + r)
    return np.asarray(rows, np.int64)
