"""GPU parity at the BASELINE configurations' full sizes.  The kernels run the whole
problem; the CPU oracle checks sampled units (it would need minutes to hours for all of
them), and size-independent properties cover the rest: invariance to the physical page
order, to the split count and to the rank count of a sequence split, and consistency
between dK and dWK."""
import math

import numpy as np
import pytest
import torch

from helpers import assert_O, assert_stats, rel_fro
from oracle import dmla_oracle as orc

pytestmark = pytest.mark.gpu
SC_MLA = 1 / math.sqrt(192)


def _gpu_randn(shape, std, seed, dev, dtype=torch.bfloat16):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)


def test_config1_on_the_fly_forward_full_size(cuda):
    """B=4,H=16,Sq=Skv=2048, K,V [.,.,.,128], WK,WV [128,64] Xavier, bf16, causal, scale 1/8."""
    import flashdmla
    B, H, S, dm, dl = 4, 16, 2048, 128, 64
    Q, K, V = (_gpu_randn((B, H, S, d), 1.0, s, cuda) for d, s in ((dl, 1), (dm, 2), (dm, 3)))
    bound = math.sqrt(6.0 / (dm + dl))
    g = torch.Generator(device=cuda).manual_seed(4)
    WK = ((torch.rand(dm, dl, generator=g, device=cuda) * 2 - 1) * bound).to(torch.bfloat16)
    WV = ((torch.rand(dm, dl, generator=g, device=cuda) * 2 - 1) * bound).to(torch.bfloat16)
    O, m, l = flashdmla.flash_dmla_on_the_fly(Q, K, V, WK, WV, 0.125, True)
    assert flashdmla.last_kernel() == "tcgen05"
    for b, h in ((0, 0), (3, 15), (1, 7)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        Or, mr, lr = orc.fwd_on_the_fly(Q[sl].float(), K[sl].float(), V[sl].float(), WK.float(), WV.float(), 0.125, True,
                                        latents_bf16=True)
        assert_O(O[sl], Or)
        assert_stats(m[sl], l[sl], mr, lr)


@pytest.fixture(scope="module")
def config2(cuda):
    """B=128,H=128,Skv=4096, pool 8192 pages x 64 x 576 bf16 ~0.1 N(0,1), table = seeded randperm."""
    B, H, SKV = 128, 128, 4096
    n_pages = B * SKV // 64
    pool = _gpu_randn((n_pages, 64, 576), 0.1, 21, cuda)
    Q = _gpu_randn((B, H, 576), 0.1, 22, cuda)
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(23)).to(torch.int32).view(B, SKV // 64).to(cuda)
    seqlens = torch.full((B,), SKV, dtype=torch.int32, device=cuda)
    return Q, pool, table, seqlens


def test_config2_paged_decode_full_size(config2, cuda):
    import flashdmla
    Q, pool, table, seqlens = config2
    O, m, l = flashdmla.flash_dmla_paged_decode(Q, pool, table, seqlens, 512, SC_MLA)
    assert flashdmla.last_kernel() == "tcgen05"
    rows = flashdmla.cache_gather(pool, table, seqlens, 4096)
    for b in (0, 77, 127):
        Kb = rows[b].float().cpu()
        Or, mr, lr = orc.attn_plain(Q[b].float().cpu(), Kb, Kb[:, :512], SC_MLA)
        assert_O(O[b], Or)
        assert_stats(m[b], l[b], mr, lr)
    # split count does not change the result beyond rounding; the physical page order not at all
    O4, m4, l4 = flashdmla.flash_dmla_paged_decode(Q, pool, table, seqlens, 512, SC_MLA, num_splits=4)
    assert_O(O4, O.float())
    assert_stats(m4, l4, m, l)
    perm = torch.randperm(pool.shape[0], generator=torch.Generator().manual_seed(5)).to(cuda)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(pool.shape[0], device=cuda)
    O2, m2, l2 = flashdmla.flash_dmla_paged_decode(Q, pool[perm].contiguous(), inv[table.long()].to(torch.int32),
                                                   seqlens, 512, SC_MLA)
    assert torch.equal(O, O2) and torch.equal(m, m2) and torch.equal(l, l2)


def test_config3_causal_prefill_full_size(cuda):
    """B=4,H=128,Sq=Skv=8192, d=576/512, bf16, causal."""
    import flashdmla
    B, H, S = 4, 128, 8192
    K = _gpu_randn((B, S, 576), 0.1, 31, cuda)
    Q = torch.empty(B, H, S, 576, dtype=torch.bfloat16, device=cuda)
    for b in range(B):
        Q[b] = _gpu_randn((H, S, 576), 0.1, 32 + b, cuda)
    O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, 512, SC_MLA, True)
    assert flashdmla.last_kernel() == "tcgen05"
    for b, h, i in ((0, 0, 0), (0, 5, 127), (1, 64, 128), (2, 127, 4095), (3, 3, 8191), (3, 100, 6000), (1, 9, 255), (2, 77, 256)):
        Kb = K[b, : i + 1].float().cpu()
        Or, mr, lr = orc.attn_plain(Q[b, h, i:i + 1].float().cpu(), Kb, Kb[:, :512], SC_MLA)
        assert_O(O[b, h, i:i + 1], Or, what=f"O[{b},{h},{i}]")
        assert_stats(m[b, h, i:i + 1], l[b, h, i:i + 1], mr, lr)
    # whole 128-row tiles (both CTAs of a pair, both key halves, the diagonal tile): the last tile of the
    # sequence and one in the middle.  Rows [r0, r0 + 128) against keys [0, r0 + 128) with the bottom-right
    # causal mask are exactly those rows of the full problem.
    for b, h, r0 in ((3, 127, S - 128), (1, 40, 4096)):
        Or, mr, lr = orc.fwd_cache_latent(Q[b:b + 1, h:h + 1, r0:r0 + 128].float().cpu(), K[b:b + 1, : r0 + 128].float().cpu(),
                                          512, SC_MLA, True)
        assert_O(O[b:b + 1, h:h + 1, r0:r0 + 128], Or, what=f"O[{b},{h},{r0}:{r0 + 128}]")
        assert_stats(m[b:b + 1, h:h + 1, r0:r0 + 128], l[b:b + 1, h:h + 1, r0:r0 + 128], mr, lr)
    assert torch.isfinite(O.float()).all() and torch.isfinite(m).all() and (l > 0).all()
    del Q, O


def test_config4a_long_context_sequence_split(cuda):
    """B=8,H=128, Skv ~ U{16384..131072}, page 64; the KV sequence is cut into 8 contiguous page-aligned
    slices (the remainder rule of the reference's fa2_fwd_mpi.cu:47-53), each slice is attended on its
    own as one rank would, and the partial (O,m,l) are merged."""
    import flashdmla
    from flashdmla.parallel import pack_partial, split_sequence_pages, unpack_partials
    B, H, W = 8, 128, 8
    lens = torch.randint(16384, 131073, (B,), generator=torch.Generator().manual_seed(41)).tolist()
    pages = [(s + 63) // 64 for s in lens]
    n_pages = sum(pages)
    pool = _gpu_randn((n_pages, 64, 576), 0.1, 42, cuda)
    Q = _gpu_randn((B, H, 576), 0.1, 43, cuda)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(44)).to(torch.int32)
    table = torch.zeros(B, max(pages), dtype=torch.int32)
    cur = 0
    for b in range(B):
        table[b, : pages[b]] = perm[cur:cur + pages[b]]
        cur += pages[b]
    seqlens = torch.tensor(lens, dtype=torch.int32)
    O, m, l = flashdmla.flash_dmla_paged_decode(Q, pool, table.to(cuda), seqlens.to(cuda), 512, SC_MLA,
                                                max_seqlen=max(lens))
    msgs = []
    for r in range(W):
        parts = split_sequence_pages(lens, 64, W, r)
        ltab = torch.zeros(B, max(n for _, n, _ in parts), dtype=torch.int32)
        llen = torch.zeros(B, dtype=torch.int32)
        for b, (first, n, ntok) in enumerate(parts):
            ltab[b, :n] = table[b, first:first + n]
            llen[b] = ntok
        Op, mp, lp = flashdmla.flash_dmla_paged_decode(Q, pool, ltab.to(cuda), llen.to(cuda), 512, SC_MLA,
                                                       num_splits=1, partial_only=True)
        msgs.append(pack_partial(Op[0], mp[0], lp[0]))
    Om, mm, lm = flashdmla.merge_partials(*unpack_partials(torch.stack(msgs), (B, H), 512), out_dtype=torch.bfloat16)
    assert_O(Om, O.float())
    assert_stats(mm, lm, m, l)
    rows = flashdmla.cache_gather(pool, table.to(cuda), seqlens.to(cuda), max(lens))
    b = int(np.argmax(lens))
    Kb = rows[b, : lens[b]].float().cpu()
    Or, mr, lr = orc.attn_plain(Q[b, :8].float().cpu(), Kb, Kb[:, :512], SC_MLA)
    assert_O(Om[b, :8], Or)
    assert_stats(mm[b, :8], lm[b, :8], mr, lr)


def test_config4b_backward_full_size(cuda):
    """On-the-fly backward, B=8,H=16,S=4096, dO ~ N(0,1): dQ/dK/dV of one (b,h) against the oracle, and
    dWK/dWV against the latent gradients recovered from dK/dV (dK = dK_lat WK^T, dWK = sum K^T dK_lat)."""
    import flashdmla
    B, H, S, dm, dl = 8, 16, 4096, 128, 64
    Q, K, V = (_gpu_randn((B, H, S, d), 1.0, s, cuda) for d, s in ((dl, 51), (dm, 52), (dm, 53)))
    bound = math.sqrt(6.0 / (dm + dl))
    g = torch.Generator(device=cuda).manual_seed(54)
    WK = ((torch.rand(dm, dl, generator=g, device=cuda) * 2 - 1) * bound).to(torch.bfloat16)
    WV = ((torch.rand(dm, dl, generator=g, device=cuda) * 2 - 1) * bound).to(torch.bfloat16)
    dO = _gpu_randn((B, H, S, dl), 1.0, 55, cuda)
    ts = [t.requires_grad_(True) for t in (Q, K, V, WK, WV)]
    O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, 0.125, True)
    O.backward(dO)
    b, h = 5, 11
    sl = (slice(b, b + 1), slice(h, h + 1))
    f = [Q[sl].float(), K[sl].float(), V[sl].float(), WK.float(), WV.float()]
    Or, mr, lr = orc.fwd_on_the_fly(*f, 0.125, True, latents_bf16=True)
    dQr, dKr, dVr, _, _ = orc.bwd_on_the_fly(*f, Or, mr, lr, dO[sl].float(), 0.125, True)
    assert rel_fro(Q.grad[sl], dQr) <= 2e-2 and rel_fro(K.grad[sl], dKr) <= 2e-2 and rel_fro(V.grad[sl], dVr) <= 2e-2
    # dK = dK_lat WK^T  =>  dK_lat = dK WK (WK^T WK)^-1 ; then dWK = sum_{rows} K^T dK_lat
    for X, W, dX, dW in ((K, WK, K.grad, WK.grad), (V, WV, V.grad, WV.grad)):
        Wf = W.detach().float()
        dlat = dX.float().reshape(-1, dm) @ Wf @ torch.linalg.inv(Wf.T @ Wf)
        dW_check = X.detach().float().reshape(-1, dm).T @ dlat
        assert rel_fro(dW, dW_check) <= 3e-2
