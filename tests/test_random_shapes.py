"""Seeded random shapes on the GPU: every decode schedule must agree with the unsplit result, and the
tcgen05 forward with the CUDA-core forward, with no wait inside a kernel giving up."""
import math
import random

import pytest
import torch

from helpers import rel_fro

pytestmark = pytest.mark.gpu
SC = 1 / math.sqrt(192)


def test_decode_schedules_agree_on_random_batches(cuda):
    import flashdmla
    rnd = random.Random(11)
    for case in range(60):
        B = rnd.choice([1, 2, 3, 7, 16, 40, 74, 75, 128, 150])
        H = rnd.choice([1, 16, 64, 128])
        mx = rnd.choice([64, 300, 1000, 4096, 9000])
        lens = [rnd.choice([0, 1, rnd.randint(1, mx), mx]) for _ in range(B)]
        ps = rnd.choice([64, 128])
        pages = [(s + ps - 1) // ps for s in lens]
        n_pages = max(1, sum(pages))
        g = torch.Generator(device=cuda).manual_seed(case)
        pool = (torch.randn(n_pages, ps, 576, generator=g, device=cuda) * 0.1).to(torch.bfloat16)
        Q = (torch.randn(B, H, 576, generator=g, device=cuda) * 0.1).to(torch.bfloat16)
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(case)).to(torch.int32)
        table = torch.zeros(B, max(1, max(pages)), dtype=torch.int32)
        cur = 0
        for b in range(B):
            table[b, :pages[b]] = perm[cur:cur + pages[b]]
            cur += pages[b]
        td, sd = table.to(cuda), torch.tensor(lens, dtype=torch.int32, device=cuda)
        O1, m1, l1 = flashdmla.flash_dmla_paged_decode(Q, pool, td, sd, 512, SC, num_splits=1)
        fin = torch.isfinite(m1)
        empty = torch.tensor(lens, device=cuda) == 0
        for s in (None, 2, rnd.choice([3, 5, 9, 33])):
            what = f"case {case}: B={B} H={H} page={ps} slabs={s} lens={lens[:6]}"
            O, m, l = flashdmla.flash_dmla_paged_decode(Q, pool, td, sd, 512, SC, num_splits=s)
            assert flashdmla.device_error_flag() == 0, what
            assert rel_fro(O, O1.float()) < 6e-3, what
            assert torch.equal(torch.isfinite(m), fin), what
            if fin.any():
                assert float((m[fin] - m1[fin]).abs().max()) < 1e-3, what
                assert float(((l[fin] - l1[fin]).abs() / l1[fin].clamp_min(1e-6)).max()) < 2e-3, what
            assert (O[empty] == 0).all() and (l[empty] == 0).all(), what


def test_tensor_forward_agrees_with_cuda_core_forward_on_random_shapes(cuda):
    import flashdmla
    rnd = random.Random(12)
    try:
        for case in range(80):
            B, H = rnd.choice([1, 2, 3]), rnd.choice([1, 3, 8, 16])
            Sq = rnd.choice([1, 2, 17, 64, 128, 129, 300, 700])
            Skv = rnd.choice([Sq, Sq + 5, Sq + 256, 64, 1000])
            causal = rnd.choice([True, False])
            if causal and Skv < Sq:
                Skv = Sq
            what = f"case {case}: B={B} H={H} Sq={Sq} Skv={Skv} causal={causal}"
            g = torch.Generator(device=cuda).manual_seed(case)
            Q = (torch.randn(B, H, Sq, 576, generator=g, device=cuda) * 0.1).to(torch.bfloat16)
            K = (torch.randn(B, Skv, 576, generator=g, device=cuda) * 0.1).to(torch.bfloat16)
            flashdmla.set_backend(flashdmla.BACKEND_AUTO)
            O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, 512, SC, causal)
            assert flashdmla.last_kernel() == "tcgen05" and flashdmla.device_error_flag() == 0, what
            flashdmla.set_backend(flashdmla.BACKEND_PORTABLE)
            Or, mr, lr = flashdmla.flash_dmla_cache_latent(Q, K, 512, SC, causal)
            assert rel_fro(O, Or.float()) < 6e-3, what
            assert float((m - mr).abs().max()) < 1e-3 and float(((l - lr).abs() / lr).max()) < 2e-3, what
    finally:
        flashdmla.set_backend(flashdmla.BACKEND_AUTO)


def test_tensor_backward_agrees_with_cuda_core_backward_on_random_shapes(cuda):
    """On-the-fly mode with 64-wide latents: O and the five gradients from the tcgen05 kernels against the
    CUDA-core kernels.  Gradients that are zero in exact arithmetic (one visible key) are compared against a
    noise floor instead of their own norm."""
    import flashdmla
    rnd = random.Random(13)

    def run(ts, dO, causal):
        for t in ts:
            t.grad = None
        O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, 0.125, causal)
        O.backward(dO)
        return [O.detach().float()] + [t.grad.float() for t in ts]
    try:
        for case in range(60):
            B, H = rnd.choice([1, 2]), rnd.choice([1, 2, 5])
            Sq = rnd.choice([1, 17, 64, 128, 129, 300, 513])
            Skv = rnd.choice([Sq, Sq + 5, Sq + 256, 64, 700])
            causal = rnd.choice([True, False])
            if causal and Skv < Sq:
                Skv = Sq
            what = f"case {case}: B={B} H={H} Sq={Sq} Skv={Skv} causal={causal}"
            g = torch.Generator(device=cuda).manual_seed(case)
            mk = lambda *sh, s=1.0: (torch.randn(*sh, generator=g, device=cuda) * s).to(torch.bfloat16)
            ts = [mk(B, H, Sq, 64), mk(B, H, Skv, 128), mk(B, H, Skv, 128), mk(128, 64, s=0.1), mk(128, 64, s=0.1)]
            ts = [t.requires_grad_(True) for t in ts]
            dO = mk(B, H, Sq, 64)
            flashdmla.set_backend(flashdmla.BACKEND_AUTO)
            a = run(ts, dO, causal)
            assert flashdmla.last_kernel() == "tcgen05" and flashdmla.device_error_flag() == 0, what
            flashdmla.set_backend(flashdmla.BACKEND_PORTABLE)
            b = run(ts, dO, causal)
            for x, y, name in zip(a, b, ("O", "dQ", "dK", "dV", "dWK", "dWV")):
                den = max(float(y.norm()), 0.05 * math.sqrt(y.numel()))
                assert float((x - y).norm()) / den < 3e-2, f"{what}: {name}"
    finally:
        flashdmla.set_backend(flashdmla.BACKEND_AUTO)
