"""GPU parity tests: every operator, called through the C ABI (ctypes), against
the CPU oracle on the same seeded inputs.  Tolerances are the target's:
O max-abs <= 1e-2 and relative Frobenius <= 5e-3 (bf16 against the fp32 oracle),
m and l relative <= 1e-3, page-table indexing bit-exact."""
import math

import numpy as np
import pytest
import torch

from helpers import assert_O, assert_stats, max_abs, rel_fro, to_np
from oracle import dmla_oracle as orc

pytestmark = pytest.mark.gpu

# portable: CUDA-core kernels; auto: tcgen05 kernels wherever the shape qualifies (2-CTA kernel
# for the MLA dimensions); auto1: the same but MLA shapes stay on the single-CTA tcgen05 kernel
BACKENDS = ["portable", "auto", "auto1"]


@pytest.fixture(params=BACKENDS)
def backend(request, cuda):
    import flashdmla
    flashdmla.set_backend(flashdmla.BACKEND_PORTABLE if request.param == "portable" else flashdmla.BACKEND_AUTO)
    flashdmla.set_single_cta(request.param == "auto1")
    yield request.param
    flashdmla.set_single_cta(False)
    flashdmla.set_backend(flashdmla.BACKEND_AUTO)
    assert flashdmla.device_error_flag() == 0


def _rand(shape, std, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype)


# ----------------------------------------------------------------------------- cache-latent forward
CL_SHAPES = [
    # B, H, Sq, Skv, d_qk, d_v, causal
    (2, 3, 17, 29, 48, 32, True),
    (1, 2, 33, 33, 160, 128, True),
    (2, 2, 8, 40, 24, 24, False),
    (1, 2, 12, 5, 16, 8, True),       # Sq > Skv: leading rows see nothing
    (1, 5, 1, 70, 64, 32, True),      # decode-like
    (1, 2, 130, 200, 576, 512, True),  # MLA dims, ragged tiles
    (2, 4, 64, 64, 64, 64, True),
    (1, 1, 300, 300, 128, 64, False),
]


@pytest.mark.parametrize("shape", CL_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_latent_forward(shape, dtype, backend, cuda):
    import flashdmla
    B, H, Sq, Skv, dq, dv, causal = shape
    Q = _rand((B, H, Sq, dq), 0.5, 11, dtype)
    K = _rand((B, Skv, dq), 0.5, 12, dtype)
    sc = 1 / math.sqrt(dq)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q.to(cuda), K.to(cuda), dv, sc, causal)
    Or, mr, lr = orc.fwd_cache_latent(Q.float(), K.float(), dv, sc, causal)
    assert O.dtype == dtype and m.dtype == torch.float32
    assert_O(O, Or, bf16=(dtype == torch.bfloat16))
    assert_stats(m, l, mr, lr)


def test_config0_exact(backend, cuda):
    """BASELINE config 0: B=2,H=8,Sq=Skv=256,d_lat=128,d_rope=32, fp32, causal, N(0,0.5^2)."""
    import flashdmla
    from flashdmla import synthetic
    Q, K = synthetic.cache_latent_inputs(2, 8, 256, 256, 160, std=0.5, seed=1)
    sc = 1 / math.sqrt(160)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q.to(cuda), K.to(cuda), 128, sc, True)
    Or, mr, lr = orc.fwd_cache_latent(Q, K, 128, sc, True)
    assert O.shape == (2, 8, 256, 128) and m.shape == (2, 8, 256) and l.shape == (2, 8, 256)
    assert_O(O, Or, bf16=False)
    assert_stats(m, l, mr, lr)


# ----------------------------------------------------------------------------- on-the-fly forward
OTF_SHAPES = [
    # B, H, Sq, Skv, d_model, d_lat, causal
    (2, 2, 19, 23, 24, 16, True),
    (1, 3, 64, 64, 128, 64, True),
    (2, 2, 100, 140, 128, 64, False),
    (1, 2, 200, 200, 96, 32, True),
]


@pytest.mark.parametrize("shape", OTF_SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_on_the_fly_forward(shape, dtype, backend, cuda):
    import flashdmla
    B, H, Sq, Skv, dm, dl, causal = shape
    Q = _rand((B, H, Sq, dl), 1.0, 21, dtype)
    K = _rand((B, H, Skv, dm), 1.0, 22, dtype)
    V = _rand((B, H, Skv, dm), 1.0, 23, dtype)
    WK = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 24, dtype)
    WV = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 25, dtype)
    sc = 1 / math.sqrt(dl)
    O, m, l = flashdmla.flash_dmla_on_the_fly(*(t.to(cuda) for t in (Q, K, V, WK, WV)), sc, causal)
    f = [t.float() for t in (Q, K, V, WK, WV)]
    bf = dtype == torch.bfloat16
    # a bf16 kernel stores the projected latents in bf16 (tensor-core operands); the row
    # statistics are compared with an oracle that rounds the latents the same way, and O is
    # additionally held to the target tolerance against the unrounded oracle
    Or, mr, lr = orc.fwd_on_the_fly(*f, sc, causal, latents_bf16=bf)
    assert_O(O, Or, bf16=bf)
    assert_stats(m, l, mr, lr)
    if bf:
        Ou, _, _ = orc.fwd_on_the_fly(*f, sc, causal)
        assert_O(O, Ou, bf16=True, what="O vs unrounded-latent oracle")


# ----------------------------------------------------------------------------- paged decode
def _paged(B, H, lens, d, ps, dtype, seed=31, std=0.3):
    from flashdmla import synthetic
    return synthetic.paged_decode_inputs(B, H, lens, d, ps, seed=seed, std=std, dtype=dtype)


@pytest.mark.parametrize("dims", [(64, 32, 16), (576, 512, 64), (160, 128, 8)])
@pytest.mark.parametrize("splits", [1, 2, 3, 7, None])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_decode_ragged(dims, splits, dtype, backend, cuda):
    import flashdmla
    dq, dv, ps = dims
    lens = [5 * ps + 3, ps, 1, 9 * ps, 2 * ps - 1]     # partial last pages, one-token sequence
    B, H = len(lens), 6
    Q, pool, table, sl = _paged(B, H, lens, dq, ps, dtype)
    sc = 1 / math.sqrt(dq)
    O, m, l = flashdmla.flash_dmla_paged_decode(Q.to(cuda), pool.to(cuda), table.to(cuda), sl.to(cuda), dv, sc,
                                                num_splits=splits)
    Or, mr, lr = orc.decode_paged(Q.float(), pool.float(), table, sl, dv, sc)
    assert_O(O, Or, bf16=(dtype == torch.bfloat16))
    assert_stats(m, l, mr, lr)


@pytest.mark.parametrize("case", [((576, 512, 64), 128, 1), ((576, 512, 64), 128, 2), ((576, 512, 64), 128, 5), ((576, 512, 64), 128, 21),
                                  ((576, 512, 64), 6, 4), ((576, 512, 64), 128, None), ((64, 32, 16), 6, 3), ((160, 128, 8), 6, 1)])
def test_paged_decode_partial_for_the_exchange(case, backend, cuda):
    """fdmla_decode_paged_partial: one rank's fp32 (O, m, l) over its whole cache, whatever the schedule behind it
    (one piece, equal splits or balanced runs of tiles with every piece a partial), an empty sequence included."""
    from flashdmla import ops
    (dq, dv, ps), H, splits = case
    lens = [37 * ps + 5, 0, ps, 90 * ps, 1, 11 * ps - 1]
    B = len(lens)
    Q, pool, table, sl = _paged(B, H, lens, dq, ps, torch.bfloat16, std=0.1)
    sc = 1 / math.sqrt(dq)
    O, m, l = ops.flash_dmla_paged_decode_partial(Q.to(cuda), pool.to(cuda), table.to(cuda), sl.to(cuda), dv, sc, num_splits=splits)
    assert O.dtype == torch.float32 and tuple(O.shape) == (B, H, dv)
    Or, mr, lr = orc.decode_paged(Q.float(), pool.float(), table, sl, dv, sc)
    assert_O(O.to(torch.bfloat16), Or)
    assert_stats(m, l, mr, lr)
    assert float(O[1].abs().max()) == 0.0 and float(l[1].abs().max()) == 0.0      # the empty sequence


def test_paged_decode_heads_128_and_window(backend, cuda):
    """H=128 (one full 128-row tile), 576/512 dims, and an attended window with partials."""
    import flashdmla
    lens = [700, 64, 1000]
    Q, pool, table, sl = _paged(3, 128, lens, 576, 64, torch.bfloat16, std=0.1)
    sc = 1 / math.sqrt(192)
    dev = [t.to(cuda) for t in (Q, pool, table, sl)]
    O, m, l = flashdmla.flash_dmla_paged_decode(*dev, 512, sc, num_splits=3)
    Or, mr, lr = orc.decode_paged(Q.float(), pool.float(), table, sl, 512, sc)
    assert_O(O, Or)
    assert_stats(m, l, mr, lr)
    # window [128, 640): partial results, then merged
    Op, mp, lp = flashdmla.flash_dmla_paged_decode(*dev, 512, sc, num_splits=2, kv_begin=128, kv_end=640,
                                                   partial_only=True)
    Om, mm, lm = flashdmla.merge_partials(Op, mp, lp)
    Ow, mw, lw = orc.decode_paged(Q.float(), pool.float(), table, sl, 512, sc, 128, 640)
    assert_O(Om, Ow)
    assert_stats(mm, lm, mw, lw)   # sequence 1 (64 tokens) is empty in this window: -inf / 0 / 0


def test_page_table_indexing_is_bit_exact(backend, cuda):
    """Identity vs permuted physical pages give identical bits; gather == index_select."""
    import flashdmla
    lens = [300, 64, 129, 1]
    Q, pool, table, sl = _paged(4, 16, lens, 576, 64, torch.bfloat16, std=0.1)
    dev = [t.to(cuda) for t in (Q, pool, table, sl)]
    sc = 1 / math.sqrt(192)
    O1, m1, l1 = flashdmla.flash_dmla_paged_decode(*dev, 512, sc, num_splits=2)
    perm = torch.randperm(pool.shape[0], generator=torch.Generator().manual_seed(5))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(pool.shape[0])
    pool2, table2 = pool[perm].contiguous(), inv[table.long()].to(torch.int32)
    O2, m2, l2 = flashdmla.flash_dmla_paged_decode(Q.to(cuda), pool2.to(cuda), table2.to(cuda), sl.to(cuda), 512, sc,
                                                   num_splits=2)
    assert torch.equal(O1, O2) and torch.equal(m1, m2) and torch.equal(l1, l2)
    n = max(lens)
    got = flashdmla.cache_gather(dev[1], dev[2], dev[3], n).cpu()
    flat = pool.view(-1, 576)
    for b, s in enumerate(lens):
        t = torch.arange(s)
        rows = table[b, t // 64].long() * 64 + t % 64
        assert torch.equal(got[b, :s], flat.index_select(0, rows))
        assert (got[b, s:] == 0).all()


def test_cache_append_then_decode(backend, cuda):
    import flashdmla
    ps, d, B = 16, 64, 3
    lens = [20, 3, 33]
    Q, pool, table, sl = _paged(B, 4, [l + 5 for l in lens], d, ps, torch.bfloat16)
    pool_d, table_d = pool.to(cuda), table.to(cuda)
    new = _rand((B, 5, d), 0.3, 77, torch.bfloat16)
    start = torch.tensor(lens, dtype=torch.int32)
    flashdmla.cache_append(new.to(cuda), pool_d, table_d, start.to(cuda))
    full = torch.tensor([l + 5 for l in lens], dtype=torch.int32)
    got = flashdmla.cache_gather(pool_d, table_d, full.to(cuda), max(lens) + 5).cpu()
    for b, s in enumerate(lens):
        assert torch.equal(got[b, s:s + 5], new[b])
    O, m, l = flashdmla.flash_dmla_paged_decode(Q.to(cuda), pool_d, table_d, full.to(cuda), 32, 0.125)
    Or, mr, lr = orc.decode_paged(Q.float(), pool_d.cpu().float(), table, full, 32, 0.125)
    assert_O(O, Or)
    assert_stats(m, l, mr, lr)


def test_merge_matches_oracle(cuda):
    import flashdmla
    g = torch.Generator().manual_seed(3)
    P, rows, dv = 5, 37, 96
    Op = torch.randn(P, rows, dv, generator=g)
    mp = torch.randn(P, rows, generator=g) * 3
    lp = torch.rand(P, rows, generator=g) * 10 + 0.1
    lp[1] = 0
    mp[1] = -math.inf          # an empty part
    lp[:, 5] = 0
    mp[:, 5] = -math.inf       # a row empty in every part
    O, m, l = flashdmla.merge_partials(Op.to(cuda), mp.to(cuda), lp.to(cuda))
    Or, mr, lr = orc.merge_partials(Op, mp, lp)
    assert_O(O, Or, bf16=False)
    assert_stats(m, l, mr, lr)


# ----------------------------------------------------------------------------- backward
@pytest.mark.parametrize("shape", [(2, 2, 19, 23, 24, 16, True), (1, 3, 64, 64, 128, 64, True),
                                   (1, 2, 70, 100, 128, 64, False), (2, 2, 300, 333, 128, 64, True),
                                   (1, 2, 333, 300, 128, 64, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_on_the_fly_backward(shape, dtype, backend, cuda):
    import flashdmla
    B, H, Sq, Skv, dm, dl, causal = shape
    Q = _rand((B, H, Sq, dl), 1.0, 41, dtype)
    K = _rand((B, H, Skv, dm), 1.0, 42, dtype)
    V = _rand((B, H, Skv, dm), 1.0, 43, dtype)
    WK = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 44, dtype)
    WV = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 45, dtype)
    dO = _rand((B, H, Sq, dl), 1.0, 46, dtype)
    sc = 1 / math.sqrt(dl)
    ts = [t.to(cuda).requires_grad_(True) for t in (Q, K, V, WK, WV)]
    O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, sc, causal)
    O.backward(dO.to(cuda))
    f = [t.float() for t in (Q, K, V, WK, WV)]
    Or, mr, lr = orc.fwd_on_the_fly(*f, sc, causal)
    want = orc.bwd_on_the_fly(*f, Or, mr, lr, dO.float(), sc, causal)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    for t, w, name in zip(ts, want, ("dQ", "dK", "dV", "dWK", "dWV")):
        assert t.grad is not None and t.grad.dtype == dtype
        assert rel_fro(t.grad, w) <= tol, f"{name}: rel-Fro {rel_fro(t.grad, w):.3e}"


def test_on_the_fly_backward_ignores_the_neighbouring_head(cuda):
    """Sq is no multiple of the 128-row tile, so the last tile the tensor-core backward streams for head 0 also
    holds the first rows of head 1.  Those rows carry NaN here (host-made inputs); they are masked, and a masked
    row must not reach head 0's gradients as 0 x NaN either."""
    import flashdmla
    B, H, S, dm, dl = 1, 2, 192, 128, 64
    dtype = torch.bfloat16
    Q = _rand((B, H, S, dl), 1.0, 141, dtype)
    K = _rand((B, H, S, dm), 1.0, 142, dtype)
    V = _rand((B, H, S, dm), 1.0, 143, dtype)
    WK = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 144, dtype)
    WV = _rand((dm, dl), math.sqrt(2.0 / (dm + dl)), 145, dtype)
    dO = _rand((B, H, S, dl), 1.0, 146, dtype)
    sc = 1 / math.sqrt(dl)
    bad = [t.clone() for t in (Q, K, V, dO)]
    for t in bad:
        t[:, 1] = float("nan")
    ts = [t.to(cuda).requires_grad_(True) for t in (bad[0], bad[1], bad[2], WK, WV)]
    O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, sc, True)
    assert flashdmla.last_kernel() == "tcgen05"
    O.backward(bad[3].to(cuda))
    f = [t[:, :1].float() for t in (Q, K, V)] + [WK.float(), WV.float()]
    Or, mr, lr = orc.fwd_on_the_fly(*f, sc, True)
    want = orc.bwd_on_the_fly(*f, Or, mr, lr, dO[:, :1].float(), sc, True)
    assert torch.isfinite(O[:, 0].float()).all()
    for t, w, name in zip(ts[:3], want[:3], ("dQ", "dK", "dV")):
        got = t.grad[:, :1]
        assert torch.isfinite(got.float()).all(), f"{name} of head 0 picked up the neighbouring head's NaN"
        assert rel_fro(got, w) <= 2e-2, f"{name}: rel-Fro {rel_fro(got, w):.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_cache_latent_backward(dtype, backend, cuda):
    import flashdmla
    B, H, Sq, Skv, dq, dv = 2, 3, 40, 50, 160, 128
    Q = _rand((B, H, Sq, dq), 0.5, 51, dtype)
    K = _rand((B, Skv, dq), 0.5, 52, dtype)
    dO = _rand((B, H, Sq, dv), 1.0, 53, dtype)
    sc = 1 / math.sqrt(dq)
    Qd, Kd = Q.to(cuda).requires_grad_(True), K.to(cuda).requires_grad_(True)
    O, m, l = flashdmla.flash_dmla_cache_latent(Qd, Kd, dv, sc, True)
    O.backward(dO.to(cuda))
    Or, mr, lr = orc.fwd_cache_latent(Q.float(), K.float(), dv, sc, True)
    dQ, dK = orc.bwd_cache_latent(Q.float(), K.float(), Or, mr, lr, dO.float(), sc, True)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert rel_fro(Qd.grad, dQ) <= tol and rel_fro(Kd.grad, dK) <= tol


@pytest.mark.parametrize("shape", [(2, 3, 100, 128, 192, 128, True), (1, 4, 64, 192, 576, 512, True), (1, 2, 300, 256, 576, 512, False),
                                   (1, 2, 130, 64, 64, 64, True), (1, 3, 512, 512, 576, 512, True), (1, 2, 384, 640, 192, 128, True)])
def test_cache_latent_backward_on_tensor_cores(shape, cuda):
    """bf16 with d_qk, d_v and Skv multiples of 64: the backward runs as GEMMs on the tensor cores over a score
    workspace (row counts that are not multiples of the 128-row tile, Sq != Skv, causal and not; the two largest
    shapes have score tiles that no query row sees, which the score GEMMs leave out, and row tiles that run over the
    end of a head)."""
    import flashdmla
    B, H, Sq, Skv, dq, dv, causal = shape
    Q = _rand((B, H, Sq, dq), 0.3, 61, torch.bfloat16)
    K = _rand((B, Skv, dq), 0.3, 62, torch.bfloat16)
    dO = _rand((B, H, Sq, dv), 1.0, 63, torch.bfloat16)
    sc = 1 / math.sqrt(dq)
    Qd, Kd = Q.to(cuda).requires_grad_(True), K.to(cuda).requires_grad_(True)
    O, m, l = flashdmla.flash_dmla_cache_latent(Qd, Kd, dv, sc, causal)
    O.backward(dO.to(cuda))
    # the same call through the C ABI on this thread (autograd runs the backward on a thread of its own, and the name
    # of the last kernel family is kept per thread)
    from flashdmla import _lib
    L = _lib.lib()
    dQ2, dK2 = torch.empty_like(Qd), torch.empty_like(Kd)
    ws = torch.empty(L.fdmla_bwd_cache_latent_workspace_bytes(B, H, Sq, Skv, dq, dv, _lib.BF16), dtype=torch.uint8, device=cuda)
    dOd = dO.to(cuda)
    rc = L.fdmla_bwd_cache_latent(Qd.data_ptr(), Kd.data_ptr(), O.data_ptr(), m.data_ptr(), l.data_ptr(), dOd.data_ptr(),
                                  dQ2.data_ptr(), dK2.data_ptr(), ws.data_ptr(), ws.numel(), B, H, Sq, Skv, dq, dv, sc, int(causal),
                                  _lib.BF16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and flashdmla.last_kernel() == "tcgen05"
    assert torch.equal(dQ2, Qd.grad) and torch.equal(dK2, Kd.grad)
    Or, mr, lr = orc.fwd_cache_latent(Q.float(), K.float(), dv, sc, causal)
    dQ, dK = orc.bwd_cache_latent(Q.float(), K.float(), Or, mr, lr, dO.float(), sc, causal)
    print(f"[parity] cache-latent backward {shape}: dQ rel-Fro {rel_fro(Qd.grad, dQ):.3e}, dK rel-Fro {rel_fro(Kd.grad, dK):.3e}")
    assert rel_fro(Qd.grad, dQ) <= 2e-2 and rel_fro(Kd.grad, dK) <= 2e-2
    assert flashdmla.device_error_flag() == 0


def test_production_shapes_run_on_tensor_cores(cuda):
    """bf16 MLA / d=64 shapes dispatch to the tcgen05 kernels, and no kernel reported a
    timed-out wait or a bad page id."""
    import flashdmla
    flashdmla.set_backend(flashdmla.BACKEND_AUTO)
    Q = _rand((1, 4, 128, 576), 0.1, 1, torch.bfloat16).to(cuda)
    K = _rand((1, 128, 576), 0.1, 2, torch.bfloat16).to(cuda)
    flashdmla.flash_dmla_cache_latent(Q, K, 512, 0.07, True)
    assert flashdmla.last_kernel() == "tcgen05"
    Q, pool, table, sl = _paged(2, 128, [130, 64], 576, 64, torch.bfloat16)
    flashdmla.flash_dmla_paged_decode(Q.to(cuda), pool.to(cuda), table.to(cuda), sl.to(cuda), 512, 0.07)
    assert flashdmla.last_kernel() == "tcgen05"
    Qo = _rand((1, 2, 128, 64), 1.0, 3, torch.bfloat16).to(cuda)
    Ko = _rand((1, 2, 128, 128), 1.0, 4, torch.bfloat16).to(cuda)
    W = _rand((128, 64), 0.1, 5, torch.bfloat16).to(cuda)
    flashdmla.flash_dmla_on_the_fly(Qo, Ko, Ko, W, W, 0.125, True)
    assert flashdmla.last_kernel() == "tcgen05"
    flashdmla.flash_dmla_cache_latent(Qo.float(), Ko[:, 0, :, :64].float().contiguous(), 32, 0.1, True)
    assert flashdmla.last_kernel() == "portable"      # fp32 stays on the CUDA-core kernels
    assert flashdmla.device_error_flag() == 0


# ----------------------------------------------------------------------------- properties
def test_runs_are_deterministic(backend, cuda):
    import flashdmla
    Q = _rand((2, 4, 128, 64), 1.0, 61, torch.bfloat16).to(cuda)
    K = _rand((2, 4, 128, 128), 1.0, 62, torch.bfloat16).to(cuda)
    V = _rand((2, 4, 128, 128), 1.0, 63, torch.bfloat16).to(cuda)
    WK = _rand((128, 64), 0.1, 64, torch.bfloat16).to(cuda)
    WV = _rand((128, 64), 0.1, 65, torch.bfloat16).to(cuda)
    outs = []
    for _ in range(2):
        ts = [t.clone().requires_grad_(True) for t in (Q, K, V, WK, WV)]
        O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, 0.125, True)
        O.backward(torch.ones_like(O))
        outs.append([O, m, l] + [t.grad for t in ts])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_batch_and_head_shards_reproduce_the_full_run(backend, cuda):
    """What each GPU computes under batch/head sharding equals its slice of the 1-GPU run."""
    import flashdmla
    Q = _rand((4, 8, 96, 576), 0.1, 71, torch.bfloat16).to(cuda)
    K = _rand((4, 96, 576), 0.1, 72, torch.bfloat16).to(cuda)
    sc = 1 / math.sqrt(192)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, 512, sc, True)
    Oh, mh, lh = flashdmla.flash_dmla_cache_latent(Q[:, 2:4].contiguous(), K, 512, sc, True)       # head shard
    Ob, mb, lb = flashdmla.flash_dmla_cache_latent(Q[1:3].contiguous(), K[1:3].contiguous(), 512, sc, True)
    if backend == "portable":
        assert torch.equal(O[:, 2:4], Oh) and torch.equal(m[:, 2:4], mh)
        assert torch.equal(O[1:3], Ob) and torch.equal(l[1:3], lb)
    else:   # tile boundaries may move with the shard; results stay within tolerance
        assert_O(Oh, O[:, 2:4])
        assert_O(Ob, O[1:3])


def test_errors_are_reported(cuda):
    import flashdmla
    Q = torch.zeros(1, 2, 4, 16, device=cuda)
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.flash_dmla_cache_latent(Q, torch.zeros(1, 4, 8, device=cuda), 8)          # d_qk mismatch
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.flash_dmla_cache_latent(Q, torch.zeros(1, 4, 16, device=cuda), 32)        # d_v > d_qk
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.flash_dmla_cache_latent(Q.half(), torch.zeros(1, 4, 16, device=cuda).half(), 8)   # fp16
    with pytest.raises(flashdmla.FlashDMLAError):
        flashdmla.flash_dmla_paged_decode(Q[:, :, 0], torch.zeros(2, 4, 16, device=cuda),
                                          torch.zeros(1, 1, dtype=torch.int64, device=cuda),
                                          torch.ones(1, dtype=torch.int32, device=cuda), 8)
    # empty inputs are a no-op that still returns correctly shaped outputs
    O, m, l = flashdmla.flash_dmla_cache_latent(torch.zeros(0, 2, 4, 16, device=cuda), torch.zeros(0, 4, 16, device=cuda), 8)
    assert O.shape == (0, 2, 4, 8)
    # Skv = 0: every row is empty
    O, m, l = flashdmla.flash_dmla_cache_latent(Q, torch.zeros(1, 0, 16, device=cuda), 8)
    assert (O == 0).all() and torch.isneginf(m).all() and (l == 0).all()


@pytest.mark.parametrize("heads,slabs", [(128, 2), (16, 2), (16, 3), (128, 6), (16, 64)])
def test_paged_decode_balanced_schedule(heads, slabs, cuda):
    """Final output with spare partial slabs on the 576/512 tensor path: the keys are dealt out as
    contiguous runs of 256-key tiles, sequences that straddle two runs are cut and merged.  Ragged
    lengths with empty and one-token sequences, against the oracle and against the unsplit result."""
    import flashdmla
    g = torch.Generator().manual_seed(77 + slabs)
    lens = torch.randint(0, 6001, (40,), generator=g).tolist()
    lens[3] = 0
    lens[17] = 1
    lens[22] = 6000
    lens[39] = 0          # an empty sequence at the very end of the line
    B = len(lens)
    Q, pool, table, sl = _paged(B, heads, lens, 576, 64, torch.bfloat16, seed=5, std=0.1)
    sc = 1 / math.sqrt(192)
    dev = [t.to(cuda) for t in (Q, pool, table, sl)]
    O, m, l = flashdmla.flash_dmla_paged_decode(*dev, 512, sc, num_splits=slabs)
    assert flashdmla.last_kernel() == "tcgen05" and flashdmla.device_error_flag() == 0
    O1, m1, l1 = flashdmla.flash_dmla_paged_decode(*dev, 512, sc, num_splits=1)
    assert_O(O, O1.float())
    assert_stats(m, l, m1, l1)
    hs = slice(0, min(heads, 8))
    Or, mr, lr = orc.decode_paged(Q[:, hs].float(), pool.float(), table, sl, 512, sc)
    assert_O(O[:, hs], Or)
    assert_stats(m[:, hs], l[:, hs], mr, lr)
    for b in (3, 39):     # empty sequences: zeros, -inf, 0
        assert (O[b] == 0).all() and (l[b] == 0).all() and torch.isinf(m[b]).all()


def test_sequence_length_beyond_the_page_table_is_clamped_and_reported(cuda):
    """seqlens[b] > max_pages * page_size cannot be served by the page table: the kernels attend the
    max_pages * page_size keys the table describes and report it (error flag 4, which does not stop
    later launches).  Without the clamp the balanced schedule would cut such a sequence into more
    pieces than there are partial slabs."""
    import flashdmla
    lens = [700, 300, 1000]
    Q, pool, table, sl = _paged(len(lens), 128, lens, 576, 64, torch.bfloat16, seed=15, std=0.1)
    sc = 1 / math.sqrt(192)
    cap = table.shape[1] * 64
    bad, clamped = sl.clone(), sl.clone()
    bad[1], clamped[1] = 10 ** 6, cap
    Qd, pd, td = Q.to(cuda), pool.to(cuda), table.to(cuda)
    assert flashdmla.device_error_flag(reset=True) in (0, 4)
    for splits in (1, 3, 5):
        want = flashdmla.flash_dmla_paged_decode(Qd, pd, td, clamped.to(cuda), 512, sc, num_splits=splits)
        assert flashdmla.device_error_flag() == 0
        got = flashdmla.flash_dmla_paged_decode(Qd, pd, td, bad.to(cuda), 512, sc, num_splits=splits)
        assert flashdmla.device_error_flag(reset=True) == 4
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    assert flashdmla.device_error_flag() == 0
