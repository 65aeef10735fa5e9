"""Helpers shared by the tests: dtype plumbing and the parity measures."""
import numpy as np
import torch

from oracle import mta_oracle as orc

ROUND = {torch.float32: orc.ROUND_NONE, torch.bfloat16: orc.ROUND_BF16, torch.float16: orc.ROUND_FP16}


def npf(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().contiguous().numpy()


def rel_fro(a: np.ndarray, ref: np.ndarray) -> float:
    fin = np.isfinite(ref)
    assert np.array_equal(fin, np.isfinite(a)), "non-finite entries are in different places"
    assert np.array_equal(a[~fin], ref[~fin]), "non-finite entries differ"
    d = np.linalg.norm((a[fin] - ref[fin]).astype(np.float64))
    n = np.linalg.norm(ref[fin].astype(np.float64))
    return float(d / n) if n > 0 else float(d)


def rel_max(a: np.ndarray, ref: np.ndarray) -> float:
    fin = np.isfinite(ref)
    m = float(np.max(np.abs(ref[fin]))) if fin.any() else 0.0
    d = float(np.max(np.abs(a[fin] - ref[fin]))) if fin.any() else 0.0
    return d / m if m > 0 else d


def max_abs(a: np.ndarray, ref: np.ndarray) -> float:
    fin = np.isfinite(ref)
    return float(np.max(np.abs(a[fin] - ref[fin]))) if fin.any() else 0.0


# Tolerances of the parity contract: fp32 max abs error <= 1e-3; 16-bit dtypes <= 2e-2 relative, applied
# norm-wise (Frobenius and max-abs over max-abs) against the oracle evaluated on the same rounded inputs.
FP32_MAX_ABS = 1e-3
BF16_REL = 2e-2


def assert_parity(a: np.ndarray, ref: np.ndarray, dtype: torch.dtype, what: str = "") -> None:
    if dtype == torch.float32:
        e = max_abs(a, ref)
        rel_fro(a, ref)  # also checks the non-finite pattern
        assert e <= FP32_MAX_ABS, f"{what}: max abs {e:.3e} > {FP32_MAX_ABS}"
    else:
        f, m = rel_fro(a, ref), rel_max(a, ref)
        assert f <= BF16_REL and m <= BF16_REL, f"{what}: rel fro {f:.3e}, rel max {m:.3e} > {BF16_REL}"
