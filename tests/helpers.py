"""Shared tolerances and comparison helpers for the parity tests."""
import numpy as np
import torch

# Tolerances of the target: bf16 kernels against the fp32 oracle.
O_MAX_ABS = 1e-2
O_REL_FRO = 5e-3
ML_REL = 1e-3
# fp32 kernels against the fp32 oracle (same arithmetic, different summation order / exp).
F32_MAX_ABS = 2e-5
F32_REL_FRO = 2e-5


def to_np(x):
    if isinstance(x, torch.Tensor):
        return x.detach().float().cpu().numpy()
    return np.asarray(x, dtype=np.float32)


def rel_fro(a, b):
    a, b = to_np(a).astype(np.float64), to_np(b).astype(np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


def max_abs(a, b):
    return float(np.max(np.abs(to_np(a).astype(np.float64) - to_np(b).astype(np.float64)))) if to_np(a).size else 0.0


def assert_O(got, want, bf16=True, what="O"):
    ma, rf = max_abs(got, want), rel_fro(got, want)
    lim_a, lim_r = (O_MAX_ABS, O_REL_FRO) if bf16 else (F32_MAX_ABS, F32_REL_FRO)
    assert ma <= lim_a and rf <= lim_r, f"{what}: max-abs {ma:.3e} (<= {lim_a}), rel-Fro {rf:.3e} (<= {lim_r})"


def assert_stats(m, l, m_ref, l_ref, what="m/l"):
    """m, l relative <= 1e-3; rows with no visible key must be exactly -inf / 0."""
    m, l, m_ref, l_ref = (to_np(x).astype(np.float64) for x in (m, l, m_ref, l_ref))
    empty = ~np.isfinite(m_ref)
    assert np.array_equal(np.isneginf(m), empty), f"{what}: -inf pattern differs"
    assert np.all(l[empty] == 0.0), f"{what}: l of empty rows not 0"
    ok = ~empty
    if ok.any():
        # m is compared through exp(m) (a shift of m by eps rescales l by e^eps), l relatively
        dm = np.abs(m[ok] - m_ref[ok])
        assert np.all(dm <= ML_REL * np.maximum(1.0, np.abs(m_ref[ok]))), f"{what}: m off by {dm.max():.3e}"
        dl = np.abs(l[ok] - l_ref[ok]) / np.abs(l_ref[ok])
        assert np.all(dl <= ML_REL), f"{what}: l rel err {dl.max():.3e}"


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()
