"""The decode entry point that allocates nothing (fdmla_decode_paged_noalloc).

Some callers cannot allocate device memory when they need a decode step: all of it may
already belong to a pool they do not own, the host they are plugged into may not let an
operator call the allocator, or an allocation would synchronise a latency-critical path.
For them the split-KV partials live in a fixed array inside the library.  This test calls
that entry point through the C ABI, several times in a row with different problems (the array
is shared and keeps what the previous call left in it), and checks each result against the
ordinary entry point given caller-provided scratch and against the CPU oracle.  It is collected
last on purpose.
"""
import ctypes
import math

import pytest
import torch

from helpers import assert_O, assert_stats

pytestmark = pytest.mark.gpu


def _problem(lens, H, seed, cuda):
    from flashdmla import synthetic
    Q, pool, table, sl = synthetic.paged_decode_inputs(len(lens), H, lens, 576, 64, seed=seed, std=0.1)
    return [t.to(cuda) for t in (Q, pool, table, sl)]


def _call_noalloc(L, Q, pool, table, sl, splits, scale):
    B, H, d_qk = Q.shape
    O = torch.full((B, H, 512), float("nan"), dtype=torch.bfloat16, device=Q.device)
    m = torch.full((B, H), float("nan"), dtype=torch.float32, device=Q.device)
    l = torch.full((B, H), float("nan"), dtype=torch.float32, device=Q.device)
    rc = L.fdmla_decode_paged_noalloc(Q.data_ptr(), pool.data_ptr(), table.data_ptr(), sl.data_ptr(), O.data_ptr(),
                                      m.data_ptr(), l.data_ptr(), B, H, d_qk, 512, pool.shape[1], table.shape[1],
                                      pool.shape[0], splits, scale, 1, torch.cuda.current_stream().cuda_stream)
    return rc, O, m, l


def test_noalloc_decode_matches_the_ordinary_entry_point_twice(cuda):
    import ctypes as ct
    import flashdmla
    from flashdmla import _lib
    from oracle import dmla_oracle as orc
    L = _lib.lib()
    scale = 1 / math.sqrt(192)
    ragged = torch.randint(2000, 4097, (40,), generator=torch.Generator().manual_seed(9)).tolist()
    ragged[0] = 4096
    # first call: 3 splits, long ragged sequences; second call: a smaller problem with another
    # split count, so stale partials of the first call sit right where the second one works; third
    # call: forty longer sequences, which the library hands out as balanced runs of tiles merged inside
    # the attention kernel - the schedule whose arrival counters have to start at zero although the
    # array still holds whatever the first two calls left there
    plans = []
    for lens, H, splits, seed in (([1500, 64, 2100, 700, 129], 128, 3, 5), ([300, 1000], 64, 2, 6), (ragged, 64, 4, 7)):
        Q, pool, table, sl = _problem(lens, H, seed, cuda)
        plans.append(L.fdmla_decode_plan(len(lens), H, 576, 512, 64, table.shape[1], splits, 1, None, None))
        rc, O, m, l = _call_noalloc(L, Q, pool, table, sl, splits, scale)
        assert rc == 0, L.fdmla_status_string(rc)
        Or, mr, lr = flashdmla.flash_dmla_paged_decode(Q, pool, table, sl, 512, scale, num_splits=splits)
        torch.cuda.synchronize()
        assert_O(O, Or.float())
        assert_stats(m, l, mr, lr)
        assert torch.equal(O, Or) and torch.equal(m, mr) and torch.equal(l, lr)   # same kernels, same split plan
        # and against the CPU oracle, on the first sequences and heads
        nb, nh = min(3, len(lens)), 8
        Oo, mo, lo = orc.decode_paged(Q[:nb, :nh].float().cpu(), pool.float().cpu(), table[:nb].cpu(), sl[:nb].cpu(), 512, scale)
        assert_O(O[:nb, :nh], Oo)
        assert_stats(m[:nb, :nh], l[:nb, :nh], mo, lo)
    assert plans[2] == 2, f"the third problem was meant to take the in-kernel balanced schedule (plans {plans})"
    assert flashdmla.device_error_flag() == 0


def test_noalloc_decode_refuses_what_does_not_fit(cuda):
    from flashdmla import _lib
    L = _lib.lib()
    max_rows = L.fdmla_decode_paged_noalloc_max_rows(512)
    assert 16000 <= max_rows <= 16400                      # 32 MiB / ((512 + 2) * 4 B)
    Q, pool, table, sl = _problem([200, 300], 128, 7, cuda)
    splits = max_rows // (2 * 128) + 1                      # one split too many for the built-in array
    rc, O, m, l = _call_noalloc(L, Q, pool, table, sl, splits, 0.07)
    assert rc == -5 and b"built-in scratch" in L.fdmla_status_string(rc)
    torch.cuda.synchronize()
    assert torch.isnan(O.float()).all()                    # nothing was launched
    rc, O, m, l = _call_noalloc(L, Q, pool, table, sl, 1, 0.07)   # a single split needs no scratch at all
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.isfinite(O.float()).all()
