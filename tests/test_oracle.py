"""CPU tests of the oracle itself: it is checked against golden vectors recorded
from the reference's own kernels, against an independent torch fp64 mirror, and
for the algebraic identities the kernels rely on."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import dmla_oracle as orc
from oracle import torch_mirror as tm

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_attn_golden.npz")


def _cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})


@pytest.mark.skipif(not os.path.exists(GOLDEN), reason="golden vectors not recorded yet")
def test_oracle_matches_reference_kernel_outputs():
    """Pins oracle_attn_plain to what vanilla_attn_forward / fa1_forward /
    fa2_forward (reference csrc/attention/*.cu, unmodified, run on a B200) gave."""
    g = np.load(GOLDEN)
    seen = 0
    for name in _cases(g):
        Q, K, V, scale = g[f"{name}/Q"], g[f"{name}/K"], g[f"{name}/V"], float(g[f"{name}/scale"])
        O, _, _ = orc.attn_plain(Q, K, V, scale)
        # vanilla and fa1 are fp32 end to end (they differ from the oracle by __expf and
        # summation order); fa2 rounds Q and K to fp16 for the tensor-core product.
        for kern, tol in (("vanilla", 2e-5), ("fa1", 2e-5), ("fa2", 5e-3)):
            key = f"{name}/O_{kern}"
            if key not in g.files:
                continue
            ref = g[key]
            assert np.isfinite(ref).all(), f"{key}: reference output not finite"
            err = np.abs(O - ref).max()
            assert err <= tol, f"{key}: oracle differs from the reference kernel by {err:.3e}"
            seen += 1
    assert seen >= 8


@pytest.mark.parametrize("B,H,Sq,Skv,dq,dv,causal", [
    (2, 3, 17, 29, 48, 32, True), (1, 2, 33, 33, 160, 128, True), (2, 2, 8, 40, 24, 24, False),
    (1, 2, 12, 5, 16, 8, True),   # Sq > Skv: leading rows see no key
    (1, 1, 1, 70, 64, 32, True),  # decode-like
])
def test_cache_latent_matches_fp64_mirror(B, H, Sq, Skv, dq, dv, causal):
    torch.manual_seed(B * 100 + Sq)
    Q = torch.randn(B, H, Sq, dq) * 0.5
    K = torch.randn(B, Skv, dq) * 0.5
    sc = 1 / math.sqrt(dq)
    O, m, l = orc.fwd_cache_latent(Q, K, dv, sc, causal)
    O2, m2, l2 = tm.fwd_cache_latent(Q, K, dv, sc, causal)
    assert np.abs(O - O2.numpy()).max() < 1e-5
    fin = np.isfinite(m2.numpy())
    assert np.array_equal(np.isfinite(m), fin)
    assert np.abs(m[fin] - m2.numpy()[fin]).max() < 1e-5
    assert np.abs(l - l2.numpy()).max() / max(1.0, l2.max().item()) < 1e-5
    assert (l[~fin] == 0).all() and (O[~fin] == 0).all()


def test_config0_shapes_and_statistics():
    """BASELINE config 0 exactly: B=2,H=8,S=256,d_lat=128,d_rope=32, fp32, causal."""
    from flashdmla import synthetic
    Q, K = synthetic.cache_latent_inputs(2, 8, 256, 256, 160, std=0.5, seed=1)
    sc = 1 / math.sqrt(160)
    O, m, l = orc.fwd_cache_latent(Q, K, 128, sc, True)
    O2, m2, l2 = tm.fwd_cache_latent(Q, K, 128, sc, True)
    assert O.shape == (2, 8, 256, 128) and m.shape == (2, 8, 256)
    assert np.abs(O - O2.numpy()).max() < 2e-5
    assert np.abs(m - m2.numpy()).max() < 1e-5
    assert (np.abs(l - l2.numpy()) / l2.numpy()).max() < 1e-5
    # first causal row attends exactly one key: l = 1, O = V_0
    assert np.allclose(l[:, :, 0], 1.0) and np.allclose(O[:, :, 0], K[:, None, 0, :128].numpy(), atol=1e-6)


def test_online_tiles_equal_three_pass():
    rs = np.random.RandomState(0)
    Q, K, V = rs.randn(9, 32).astype(np.float32), rs.randn(77, 32).astype(np.float32), rs.randn(77, 20).astype(np.float32)
    O, m, l = orc.attn_plain(Q, K, V, 0.2)
    for tile in (1, 16, 64, 200):
        O2, m2, l2 = orc.attn_online(Q, K, V, 0.2, tile)
        assert np.abs(O - O2).max() < 1e-5 and np.abs(m - m2).max() < 1e-6
        assert (np.abs(l - l2) / l).max() < 1e-5


def test_on_the_fly_and_backward_match_autograd():
    torch.manual_seed(3)
    B, H, Sq, Skv, dm, dl = 2, 2, 19, 23, 24, 16
    Q, K, V = torch.randn(B, H, Sq, dl), torch.randn(B, H, Skv, dm), torch.randn(B, H, Skv, dm)
    WK, WV = torch.randn(dm, dl) * 0.2, torch.randn(dm, dl) * 0.2
    for causal in (True, False):
        O, m, l = orc.fwd_on_the_fly(Q, K, V, WK, WV, 0.25, causal)
        O2, m2, l2 = tm.fwd_on_the_fly(Q, K, V, WK, WV, 0.25, causal)
        assert np.abs(O - O2.numpy()).max() < 1e-5
        dO = torch.randn(B, H, Sq, dl)
        got = orc.bwd_on_the_fly(Q, K, V, WK, WV, O, m, l, dO, 0.25, causal)
        want = tm.bwd_on_the_fly_autograd(Q, K, V, WK, WV, dO, 0.25, causal)
        for a, b, name in zip(got, want, ("dQ", "dK", "dV", "dWK", "dWV")):
            assert np.abs(a - b.numpy()).max() < 2e-5 * max(1.0, b.abs().max().item()), name


def test_cache_latent_backward_matches_autograd():
    torch.manual_seed(4)
    B, H, Sq, Skv, dq, dv = 2, 3, 10, 14, 24, 16
    Q, K = torch.randn(B, H, Sq, dq) * 0.5, torch.randn(B, Skv, dq) * 0.5
    O, m, l = orc.fwd_cache_latent(Q, K, dv, 0.2, True)
    dO = torch.randn(B, H, Sq, dv)
    dQ, dK = orc.bwd_cache_latent(Q, K, O, m, l, dO, 0.2, True)
    dQ2, dK2 = tm.bwd_cache_latent_autograd(Q, K, dv, dO, 0.2, True)
    assert np.abs(dQ - dQ2.numpy()).max() < 2e-5 and np.abs(dK - dK2.numpy()).max() < 2e-5


def _paged_problem(seed=5, B=3, H=4, d=32, ps=8, lens=(21, 8, 40)):
    from flashdmla import synthetic
    return synthetic.paged_decode_inputs(B, H, lens, d, ps, seed=seed, std=0.5, dtype=torch.float32)


def test_paged_gather_is_index_select_and_permutation_invariant():
    Q, pool, table, lens = _paged_problem()
    O, m, l = orc.decode_paged(Q, pool, table, lens, 16, 0.3)
    O2, m2, l2 = tm.decode_paged(Q, pool, table, lens, 16, 0.3)
    assert np.abs(O - O2.numpy()).max() < 1e-5
    # dense equivalent: gather rows then plain attention
    for b in range(3):
        rows = tm.gather_pages(pool, table, b, int(lens[b]))
        Ob, mb, lb = orc.attn_plain(Q[b], rows, rows[:, :16], 0.3)
        assert np.array_equal(Ob, O[b]) and np.array_equal(mb, m[b]) and np.array_equal(lb, l[b])
    # permuting physical pages (and the table with them) changes nothing, bit for bit
    perm = torch.randperm(pool.shape[0], generator=torch.Generator().manual_seed(9))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(pool.shape[0])
    O3, m3, l3 = orc.decode_paged(Q, pool[perm], inv[table.long()].to(torch.int32), lens, 16, 0.3)
    assert np.array_equal(O, O3) and np.array_equal(m, m3) and np.array_equal(l, l3)


def test_split_and_merge_equals_unsplit():
    Q, pool, table, lens = _paged_problem(lens=(37, 64, 5))
    O, m, l = orc.decode_paged(Q, pool, table, lens, 16, 0.3)
    cuts = [0, 16, 16, 40, 64]           # includes an empty slice and slices past short sequences
    parts = [orc.decode_paged(Q, pool, table, lens, 16, 0.3, a, b) for a, b in zip(cuts[:-1], cuts[1:])]
    Op, mp, lp = (np.stack([p[i] for p in parts]) for i in range(3))
    Om, mm, lm = orc.merge_partials(Op, mp, lp)
    assert np.abs(Om - O).max() < 1e-5 and np.abs(mm - m).max() < 1e-6 and (np.abs(lm - l) / l).max() < 1e-5
    Ot, mt, lt = tm.merge_partials(torch.from_numpy(Op).double(), torch.from_numpy(mp).double(), torch.from_numpy(lp).double())
    assert np.abs(Om - Ot.numpy()).max() < 1e-5


def test_merge_all_empty_rows():
    Op = np.zeros((3, 4, 8), np.float32)
    mp = np.full((3, 4), -np.inf, np.float32)
    lp = np.zeros((3, 4), np.float32)
    O, m, l = orc.merge_partials(Op, mp, lp)
    assert (O == 0).all() and np.isneginf(m).all() and (l == 0).all()


def test_split_range_is_the_reference_partition_rule():
    """fa2_fwd_mpi.cu:47-53: base = n / size, rem = n % size, first `rem` ranks get one more."""
    from flashdmla.parallel import shard_range
    for n, parts in ((10, 3), (8, 8), (5, 8), (131072 // 64, 8), (0, 4)):
        offs = [orc.split_range(n, parts, r) for r in range(parts)]
        assert sum(ln for _, ln in offs) == n
        assert all(offs[r][0] + offs[r][1] == offs[r + 1][0] for r in range(parts - 1))
        assert max(ln for _, ln in offs) - min(ln for _, ln in offs) <= 1
        assert offs == [shard_range(n, parts, r) for r in range(parts)]
