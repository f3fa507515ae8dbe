"""Absorbed MLA block around the decode kernel: the algebra on the CPU, the full step on the GPU."""
import math

import pytest
import torch


def test_absorption_is_an_identity_cpu():
    """[q_nope W_UK^T | rope(q_rope)] . [c | k_rope] equals the per-head score, and (sum p c) W_UV the per-head output."""
    from flashdmla.mla import AbsorbedMLA, rope
    blk = AbsorbedMLA(d_model=96, n_heads=4, d_lat=32, d_rope=8, d_nope=16, d_vhead=12, dtype=torch.float32, device="cpu", seed=3)
    g = torch.Generator().manual_seed(4)
    T = 19
    hs = torch.randn(T, 96, generator=g)
    rows = blk.cache_rows(hs[None], torch.arange(T)[None])[0]            # [T, 40]
    h = hs[-1]
    Qp = blk.absorbed_query_torch(h[None], torch.tensor([T - 1]))[0]     # [H, 40]
    s = (Qp @ rows.T) * blk.scale
    p = torch.softmax(s, dim=-1)
    o_lat = p @ rows[:, :32]
    out = torch.einsum("hl,hlv->hv", o_lat, blk.W_UV).reshape(-1) @ blk.W_O
    want = blk.reference_decode(rows, h, T - 1)
    assert torch.allclose(out, want, rtol=1e-4, atol=1e-5)
    # rope is a rotation: norms are preserved and relative positions are what the score sees
    x = torch.randn(5, 8, generator=g)
    assert torch.allclose(rope(x, torch.arange(5)).norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    a, b = torch.randn(8, generator=g), torch.randn(8, generator=g)
    d1 = rope(a[None], torch.tensor([7]))[0] @ rope(b[None], torch.tensor([3]))[0]
    d2 = rope(a[None], torch.tensor([14]))[0] @ rope(b[None], torch.tensor([10]))[0]
    assert abs(float(d1 - d2)) < 1e-4


@pytest.mark.gpu
def test_absorbed_decode_step_matches_per_head_attention(cuda):
    from flashdmla.cache import PagedLatentCache
    from flashdmla.mla import AbsorbedMLA
    import flashdmla
    blk = AbsorbedMLA(d_model=256, n_heads=16, device=cuda, seed=5)
    cache = PagedLatentCache(num_pages=32, page_size=64, d_qk=576, max_seqs=4, max_pages_per_seq=8, device=cuda)
    g = torch.Generator().manual_seed(6)
    slots = [cache.new_sequence() for _ in range(3)]
    lens = [150, 64, 1]
    for s, n in zip(slots, lens):                                        # prompts of different lengths
        h = (torch.randn(1, n, 256, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
        cache.append([s], blk.cache_rows(h, torch.arange(n, device=cuda)[None]))
    for step in range(3):                                                # three decode steps
        h = (torch.randn(3, 256, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
        pos = torch.tensor([cache.length(s) for s in slots], device=cuda)
        Qk, Qt = blk.absorbed_query(h, pos), blk.absorbed_query_torch(h, pos)     # the GEMM + RoPE kernels against torch
        assert (Qk.float() - Qt.float()).abs().max() <= 2e-2 * Qt.float().abs().max()
        out = blk.decode(cache, slots, h)
        assert flashdmla.last_kernel() == "tcgen05"
        rows = cache.gather(slots, max(lens) + step + 1)
        for i, s in enumerate(slots):
            n = cache.length(s)
            want = blk.reference_decode(rows[i, :n], h[i], n - 1)
            err = (out[i].float() - want).norm() / want.norm()
            assert err < 2e-2, f"sequence {i} step {step}: rel err {float(err):.3e}"
