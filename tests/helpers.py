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
    """Target tolerance: max-abs <= 1e-2 and relative Frobenius <= 5e-3.  A bf16 OUTPUT
    cannot meet an absolute 1e-2 where |O| >= 4 (its spacing there is 2^-5), so each element
    is allowed 1e-2 plus one bf16 rounding step (2^-8 |O|) of the value it has to represent."""
    g, w = to_np(got).astype(np.float64), to_np(want).astype(np.float64)
    rf = rel_fro(got, want)
    ma = max_abs(got, want)
    peak = float(np.abs(w).max()) if w.size else 0.0
    print(f"[parity] {what}: max-abs {ma:.3e}  rel-Fro {rf:.3e}  max|O| {peak:.3g}")     # shown by pytest -s / on failure
    if bf16:
        excess = np.abs(g - w) - (O_MAX_ABS + np.abs(w) * 2.0 ** -8)
        worst = float(excess.max()) if excess.size else -1.0
        assert worst <= 0 and rf <= O_REL_FRO, \
            f"{what}: max-abs {ma:.3e} exceeds 1e-2 + 2^-8|O| by {worst:.3e}; rel-Fro {rf:.3e} (<= {O_REL_FRO})"
        if peak < 2.0:
            # every value lies where rounding the OUTPUT to bf16 costs at most 2^-9 |O| < 4e-3, so the plain
            # target applies (in [2, 4) that rounding alone may take 7.8e-3 of the 1e-2)
            assert ma <= O_MAX_ABS, f"{what}: max-abs {ma:.3e} > {O_MAX_ABS} although max|O| = {peak:.3g} < 2"
    else:
        assert ma <= F32_MAX_ABS and rf <= F32_REL_FRO, \
            f"{what}: max-abs {ma:.3e} (<= {F32_MAX_ABS}), rel-Fro {rf:.3e} (<= {F32_REL_FRO})"


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
        dl = np.abs(l[ok] - l_ref[ok]) / np.abs(l_ref[ok])
        print(f"[parity] {what}: m abs err {dm.max():.3e}  l rel err {dl.max():.3e}")
        assert np.all(dm <= ML_REL * np.maximum(1.0, np.abs(m_ref[ok]))), f"{what}: m off by {dm.max():.3e}"
        assert np.all(dl <= ML_REL), f"{what}: l rel err {dl.max():.3e}"


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()
