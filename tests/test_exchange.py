"""fdmla_exchange_merge on ONE GPU: the kernel's own half of the exchange against the merge kernel, and its time limit.

The peers of a real exchange are other GPUs (tests/test_multi_gpu.py runs that on two).  Here rank 0 of a world of two
runs alone: its "peer's" buffer is a second local buffer, and what the peer would have stored into rank 0's buffer -
its partial rows and data flags, and in the owner form the merged rows and result flags of the row blocks the peer
owns - is written by the host before the launch, so the kernel never waits for another kernel.
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
    assert L.fdmla_exchange_bytes(2, 8, 512) == (2 * 3 * n + 2 * GRID + 2 * GRID) * 4      # 2 slots x (2 messages + results), flags, counters
    assert L.fdmla_exchange_merge(None, None, 2, 0, 0, 512, None, None, None, 0, 100, None) == 0      # no rows: no-op
    assert L.fdmla_exchange_merge(None, None, 2, 0, 8, 512, None, None, None, 0, 100, None) == -1
    assert L.fdmla_exchange_merge(None, None, 2, 2, 8, 512, None, None, None, 0, 100, None) == -1     # rank outside the world
    assert L.fdmla_exchange_merge(None, None, 2, 0, 8, 512, None, None, None, 0, 0, None) == -1       # no time limit
    assert L.fdmla_exchange_alloc(0, None, None) == -1 and L.fdmla_exchange_open(None, None) == -1
    assert L.fdmla_exchange_close(None) == 0 and L.fdmla_exchange_free(None) == 0
    assert L.fdmla_exchange_merge_parts(None, None, None, 0, None, None, 2, 0, 8, 512, None, None, None, 0, 100, None) == -1   # no pieces
    # the host side refuses anything but CUDA devices before it touches the process group: there is no CPU path
    from flashdmla.exchange import PeerExchange
    with pytest.raises(_lib.FlashDMLAError):
        PeerExchange(8, 512, "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("pieces", [0, 5])
@pytest.mark.parametrize("world", [2, 5])
@pytest.mark.parametrize("rows,d_v,out_dtype", [(1024, 512, torch.bfloat16), (130, 512, torch.float32), (7, 64, torch.float32)])
def test_exchange_merge_against_merge_kernel(rows, d_v, out_dtype, world, pieces, cuda):
    """world 2 runs the all-gather form (whole messages to every peer, every rank merges everything), world 5 the owner
    form (rows to the rank that owns their block, merged rows back).  pieces > 0: rank 0's own partial result arrives in
    that many unmerged pieces (fdmla_exchange_merge_parts: the kernel merges them into the message first)."""
    import flashdmla
    from flashdmla import _lib
    from flashdmla.parallel import message_views
    L = _lib.lib()
    W = world
    gather = W <= 4
    n = rows * (d_v + 2)
    stride = (n + 3) // 4 * 4
    nbytes = L.fdmla_exchange_bytes(W, rows, d_v)
    with torch.cuda.device(cuda):
        raw, t = zip(*[_alloc(L, nbytes, cuda) for _ in range(W)])       # t[0]: rank 0's own buffer; t[p]: "peer" p's
        assert float(t[0].abs().sum()) == 0.0                            # allocated zeroed
        bufs = (ctypes.c_void_p * W)(*[r.value for r in raw])
        slot_floats, flags_off = (W + 1) * stride, 2 * (W + 1) * stride  # a slot: W messages and the result area
        code = _lib.F32 if out_dtype == torch.float32 else _lib.BF16
        per = (rows + GRID - 1) // GRID
        owner_of_row = ((torch.arange(rows) // per) % W).to(cuda)
        owner_of_block = torch.arange(GRID, device=cuda) % W
        mine = torch.ones(rows, dtype=torch.bool, device=cuda) if gather else owner_of_row == 0
        for step in (1, 2, 3):                                           # slots 1, 0, 1
            msgs = [_message(rows, d_v, 10 * step + q, empty_rows=(0,) if q == 0 else (0, rows - 1)).to(cuda) for q in range(W)]
            if pieces:
                # rank 0's message = the merge kernel's result over its pieces (piece 1 empty everywhere, row 0 empty in all)
                pm = [_message(rows, d_v, 100 * step + q, empty_rows=range(rows) if q == 1 else (0,)).to(cuda) for q in range(pieces)]
                pO, pmm, pl = (t.contiguous() for t in message_views(torch.stack(pm), (rows,), d_v))
                msgs[0] = torch.cat([t.reshape(-1) for t in flashdmla.merge_partials(pO, pmm, pl, torch.float32)])
            O_p, m_p, l_p = message_views(torch.stack(msgs), (rows,), d_v)
            Ow, mw, lw = flashdmla.merge_partials(O_p, m_p, l_p, out_dtype)
            slot = (step & 1) * slot_floats
            stepw = torch.full((GRID,), step, dtype=torch.int32).view(torch.float32).to(cuda)
            # what the peers would have stored here.  Their partial rows in messages [1..] of the slot and the step
            # number in data flags [p][*] (the owner form reads only the rows of the blocks rank 0 owns) ...
            for q in range(1, W):
                t[0][slot + q * stride: slot + q * stride + n] = msgs[q]
                t[0][flags_off + q * GRID: flags_off + (q + 1) * GRID] = stepw
            # ... and, owner form, for the blocks they own: the merged rows in the slot's result area and the step number
            # in the result flags (only those rows: the others hold a marker that must not reach the output)
            res = t[0][slot + W * stride: slot + (W + 1) * stride]
            res[:] = 12345.0
            if not gather:
                res.view(out_dtype)[: rows * d_v].view(rows, d_v)[~mine] = Ow[~mine]
                res[rows * d_v: rows * d_v + rows][~mine] = mw[~mine]
                res[rows * d_v + rows: rows * d_v + 2 * rows][~mine] = lw[~mine]
                t[0][flags_off + W * GRID: flags_off + (W + 1) * GRID] = stepw
            for q in range(1, W):
                t[q][slot: slot + (W + 1) * stride] = -777.0
            O = torch.full((rows, d_v), float("nan"), dtype=out_dtype, device=cuda)
            m = torch.full((rows,), float("nan"), device=cuda)
            l = torch.full((rows,), float("nan"), device=cuda)
            torch.cuda.synchronize()
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            if pieces:
                built = torch.full((n,), float("nan"), device=cuda)
                rc = L.fdmla_exchange_merge_parts(pO.data_ptr(), pmm.data_ptr(), pl.data_ptr(), pieces, built.data_ptr(), bufs, W, 0,
                                                  rows, d_v, O.data_ptr(), m.data_ptr(), l.data_ptr(), code, 2000, stream)
            else:
                rc = L.fdmla_exchange_merge(msgs[0].data_ptr(), bufs, W, 0, rows, d_v, O.data_ptr(), m.data_ptr(), l.data_ptr(),
                                            code, 2000, stream)
            assert rc == 0
            torch.cuda.synchronize()
            if pieces:
                assert torch.equal(built, msgs[0])                    # the message it built from the pieces, bit for bit
            assert flashdmla.last_kernel() == "exchange_merge_kernel"
            assert torch.equal(O, Ow) and torch.equal(m, mw) and torch.equal(l, lw)        # bit for bit
            # and both against the merge rule written out in fp32 (an odd number of rows puts the later gathered
            # messages off the 16-byte grid: the merge kernel must not read them with vector loads)
            w = l_p * torch.exp(m_p - m_p.max(dim=0).values.clamp_min(-1e30))
            ref = (w[..., None] * O_p).sum(0) / w.sum(0).clamp_min(1e-30)[..., None]
            assert float((O.float()[1:] - ref[1:]).abs().max()) <= (2e-2 if out_dtype == torch.bfloat16 else 1e-4)
            assert float(l[0]) == 0.0 and float(m[0]) == float("-inf") and float(O[0].float().abs().sum()) == 0.0
            mO0, mm0, ml0 = message_views(msgs[0], (rows,), d_v)
            for q in range(1, W):
                # what it stored for peer q: rank 0's partial rows in message [0] of the peer's slot (all-gather form: all
                # rows; owner form: the rows of the blocks the peer owns, nothing else) and the step number in the
                # peer's data flags [0][those blocks]
                sent_O, sent_m, sent_l = message_views(t[q][slot: slot + n], (rows,), d_v)
                theirs = torch.ones(rows, dtype=torch.bool, device=cuda) if gather else owner_of_row == q
                their_blocks = torch.ones(GRID, dtype=torch.bool, device=cuda) if gather else owner_of_block == q
                assert torch.equal(sent_O[theirs], mO0[theirs]) and torch.equal(sent_m[theirs], mm0[theirs]) and torch.equal(sent_l[theirs], ml0[theirs])
                assert bool((sent_O[~theirs] == -777.0).all())
                flags = t[q][flags_off: flags_off + (W + 1) * GRID].view(torch.int32)
                assert bool((flags[:GRID][their_blocks] == step).all()) and bool((flags[:GRID][~their_blocks] == 0).all())
                if gather:
                    continue
                # owner form, blocks rank 0 owns: the merged rows in the peer's result area, the step number in its result flags
                pres = t[q][slot + W * stride: slot + (W + 1) * stride]
                assert torch.equal(pres.view(out_dtype)[: rows * d_v].view(rows, d_v)[mine], Ow[mine])
                assert torch.equal(pres[rows * d_v: rows * d_v + rows][mine], mw[mine])
                assert torch.equal(pres[rows * d_v + rows: rows * d_v + 2 * rows][mine], lw[mine])
                my_blocks = owner_of_block == 0
                assert bool((flags[W * GRID:][my_blocks] == step).all()) and bool((flags[W * GRID:][~my_blocks] == 0).all())
        assert flashdmla.device_error_flag() == 0
        del t
        for r in raw:
            assert L.fdmla_exchange_free(r) == 0


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
