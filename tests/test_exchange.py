"""fdmla_exchange_merge on ONE GPU: the kernel's own half of the exchange against the merge kernel, and its time limit.

The peers of a real exchange are other GPUs (tests/test_multi_gpu.py runs that on two).  Here rank 0 of a world of two
runs alone: its "peer's" buffer is a second local buffer, and what the peer would have stored into rank 0's buffer -
its partial rows and data flags for the row blocks rank 0 owns (the even ones), the merged rows and result flags for
the blocks the peer owns - is written by the host before the launch, so the kernel never waits for another kernel.
The time-limit case leaves the flags unset: the wait runs out, the kernel returns, the error flag reads 31.
"""
import ctypes

import pytest
import torch

GRID = 128        # thread blocks of the exchange kernel = flag words per rank


class _Raw:
    def __init__(self, ptr, n_floats):
        self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def _alloc(L, nbytes, cuda):
    buf, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    assert L.fdmla_exchange_alloc(nbytes, ctypes.byref(buf), handle) == 0
    return buf, torch.as_tensor(_Raw(buf.value, nbytes // 4), device=cuda)


def _message(rows, d_v, seed, empty_rows=()):
    g = torch.Generator().manual_seed(seed)
    O = torch.randn(rows, d_v, generator=g)
    m = torch.randn(rows, generator=g) * 3
    l = torch.rand(rows, generator=g) * 50 + 0.5
    for r in empty_rows:          # a rank whose slice of that sequence is empty: l = 0, m = -inf, O = 0
        O[r] = 0
        m[r] = float("-inf")
        l[r] = 0
    return torch.cat([O.reshape(-1), m, l])


def test_exchange_argument_validation_needs_no_gpu():
    from flashdmla import _lib
    L = _lib.lib()
    assert L.fdmla_exchange_bytes(0, 8, 512) == 0 and L.fdmla_exchange_bytes(17, 8, 512) == 0
    assert L.fdmla_exchange_bytes(2, 8, 510) == 0
    n = 8 * 514
    assert L.fdmla_exchange_bytes(2, 8, 512) == (2 * 3 * n + 2 * GRID + 2 * GRID) * 4      # 2 slots x (2 messages + results), flags
    assert L.fdmla_exchange_merge(None, None, 2, 0, 0, 512, None, None, None, 0, 100, None) == 0      # no rows: no-op
    assert L.fdmla_exchange_merge(None, None, 2, 0, 8, 512, None, None, None, 0, 100, None) == -1
    assert L.fdmla_exchange_merge(None, None, 2, 2, 8, 512, None, None, None, 0, 100, None) == -1     # rank outside the world
    assert L.fdmla_exchange_merge(None, None, 2, 0, 8, 512, None, None, None, 0, 0, None) == -1       # no time limit
    assert L.fdmla_exchange_alloc(0, None, None) == -1 and L.fdmla_exchange_open(None, None) == -1
    assert L.fdmla_exchange_close(None) == 0 and L.fdmla_exchange_free(None) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,d_v,out_dtype", [(1024, 512, torch.bfloat16), (130, 512, torch.float32), (7, 64, torch.float32)])
def test_exchange_merge_against_merge_kernel(rows, d_v, out_dtype, cuda):
    import flashdmla
    from flashdmla import _lib
    from flashdmla.parallel import message_views
    L = _lib.lib()
    n = rows * (d_v + 2)
    stride = (n + 3) // 4 * 4
    nbytes = L.fdmla_exchange_bytes(2, rows, d_v)
    with torch.cuda.device(cuda):
        own, own_t = _alloc(L, nbytes, cuda)
        peer, peer_t = _alloc(L, nbytes, cuda)
        assert float(own_t.abs().sum()) == 0.0                       # allocated zeroed
        bufs = (ctypes.c_void_p * 2)(own.value, peer.value)
        slot_floats, flags_off = 3 * stride, 2 * 3 * stride          # a slot: two messages and the result area
        code = _lib.F32 if out_dtype == torch.float32 else _lib.BF16
        per = (rows + GRID - 1) // GRID
        block_of_row = torch.arange(rows) // per
        mine = (block_of_row % 2 == 0).to(cuda)                      # rows whose block rank 0 owns
        for step in (1, 2, 3):                                       # slots 1, 0, 1
            msg0 = _message(rows, d_v, 10 * step, empty_rows=(0,)).to(cuda)
            msg1 = _message(rows, d_v, 10 * step + 1, empty_rows=(0, rows - 1)).to(cuda)
            O_p, m_p, l_p = message_views(torch.stack([msg0, msg1]), (rows,), d_v)
            Ow, mw, lw = flashdmla.merge_partials(O_p, m_p, l_p, out_dtype)
            slot = (step & 1) * slot_floats
            stepw = torch.full((GRID,), step, dtype=torch.int32).view(torch.float32).to(cuda)
            # what rank 1 would have stored here.  For the blocks rank 0 owns: its partial rows in message [1] of the
            # slot and the step number in data flags [1][*] ...
            own_t[slot + stride: slot + stride + n] = msg1
            own_t[flags_off + GRID: flags_off + 2 * GRID] = stepw
            # ... for the blocks rank 1 owns: the merged rows in the slot's result area and the step number in the
            # result flags (only those rows: the others hold a marker that must not reach the output)
            res = own_t[slot + 2 * stride: slot + 3 * stride]
            res[:] = 12345.0
            res_O = res.view(out_dtype)[: rows * d_v].view(rows, d_v)
            res_O[~mine] = Ow[~mine]
            res[rows * d_v: rows * d_v + rows][~mine] = mw[~mine]
            res[rows * d_v + rows: rows * d_v + 2 * rows][~mine] = lw[~mine]
            own_t[flags_off + 2 * GRID: flags_off + 3 * GRID] = stepw
            peer_t[slot: slot + 3 * stride] = -777.0
            O = torch.full((rows, d_v), float("nan"), dtype=out_dtype, device=cuda)
            m = torch.full((rows,), float("nan"), device=cuda)
            l = torch.full((rows,), float("nan"), device=cuda)
            torch.cuda.synchronize()
            rc = L.fdmla_exchange_merge(msg0.data_ptr(), bufs, 2, 0, rows, d_v, O.data_ptr(), m.data_ptr(), l.data_ptr(),
                                        code, 2000, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0
            torch.cuda.synchronize()
            assert flashdmla.last_kernel() == "exchange_merge_kernel"
            assert torch.equal(O, Ow) and torch.equal(m, mw) and torch.equal(l, lw)        # bit for bit
            # and both against the merge rule written out in fp32 (an odd number of rows puts the second gathered
            # message off the 16-byte grid: the merge kernel must not read it with vector loads)
            w = l_p * torch.exp(m_p - m_p.max(dim=0).values.clamp_min(-1e30))
            ref = (w[..., None] * O_p).sum(0) / w.sum(0).clamp_min(1e-30)[..., None]
            assert float((O.float()[1:] - ref[1:]).abs().max()) <= (2e-2 if out_dtype == torch.bfloat16 else 1e-4)
            assert float(l[0]) == 0.0 and float(m[0]) == float("-inf") and float(O[0].float().abs().sum()) == 0.0
            # what it stored for its peer.  Blocks the peer owns: rank 0's partial rows in message [0] of the peer's slot
            # and the step number in the peer's data flags [0][odd blocks] ...
            sent_O, sent_m, sent_l = message_views(peer_t[slot: slot + n], (rows,), d_v)
            mO0, mm0, ml0 = message_views(msg0, (rows,), d_v)
            assert torch.equal(sent_O[~mine], mO0[~mine]) and torch.equal(sent_m[~mine], mm0[~mine]) and torch.equal(sent_l[~mine], ml0[~mine])
            assert bool((sent_O[mine] == -777.0).all())                  # nothing else travels
            flags = peer_t[flags_off: flags_off + 3 * GRID].view(torch.int32)
            odd = torch.arange(GRID, device=cuda) % 2 == 1
            assert bool((flags[:GRID][odd] == step).all()) and bool((flags[:GRID][~odd] == 0).all())
            # ... blocks rank 0 owns: the merged rows in the peer's result area and the step number in its result flags
            pres = peer_t[slot + 2 * stride: slot + 3 * stride]
            assert torch.equal(pres.view(out_dtype)[: rows * d_v].view(rows, d_v)[mine], Ow[mine])
            assert torch.equal(pres[rows * d_v: rows * d_v + rows][mine], mw[mine])
            assert torch.equal(pres[rows * d_v + rows: rows * d_v + 2 * rows][mine], lw[mine])
            assert bool((flags[2 * GRID:][~odd] == step).all()) and bool((flags[2 * GRID:][odd] == 0).all())
        assert flashdmla.device_error_flag() == 0
        del own_t, peer_t
        assert L.fdmla_exchange_free(own) == 0 and L.fdmla_exchange_free(peer) == 0


@pytest.mark.gpu
def test_exchange_peer_that_never_arrives_times_out(cuda):
    """Nothing sets the peer's flags: every block's wait runs out after the limit, the kernel returns, the result is
    left unwritten and the device error flag names the exchange.  The context stays usable."""
    import flashdmla
    from flashdmla import _lib
    L = _lib.lib()
    rows, d_v = 64, 512
    nbytes = L.fdmla_exchange_bytes(2, rows, d_v)
    with torch.cuda.device(cuda):
        own, own_t = _alloc(L, nbytes, cuda)
        peer, peer_t = _alloc(L, nbytes, cuda)
        bufs = (ctypes.c_void_p * 2)(own.value, peer.value)
        msg0 = _message(rows, d_v, 5).to(cuda)
        O = torch.full((rows, d_v), 7.0, device=cuda)
        m = torch.full((rows,), 7.0, device=cuda)
        l = torch.full((rows,), 7.0, device=cuda)
        assert flashdmla.device_error_flag(reset=True) in (0, 31)
        rc = L.fdmla_exchange_merge(msg0.data_ptr(), bufs, 2, 0, rows, d_v, O.data_ptr(), m.data_ptr(), l.data_ptr(),
                                    _lib.F32, 50, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        assert flashdmla.device_error_flag() == 31
        assert flashdmla.device_error_flag(reset=True) == 31 and flashdmla.device_error_flag() == 0
        assert float((O - 7.0).abs().sum()) == 0.0 and float((l - 7.0).abs().sum()) == 0.0       # nothing merged
        # the context still works
        assert float((torch.ones(4, device=cuda) * 2).sum()) == 8.0
        del own_t, peer_t
        assert L.fdmla_exchange_free(own) == 0 and L.fdmla_exchange_free(peer) == 0
