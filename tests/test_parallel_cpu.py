"""Host-side logic of the multi-GPU paths, run as world_size-2 gloo ranks on CPU.
The per-rank attention and the merge are stood in for by the CPU oracle (the
product operators have no CPU path); what is tested is the sharding rule, the
message packing, the all-gather and the failure detection around it."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD = 2
LENS = [300, 64, 129, 1, 1000]
H, D_QK, D_V, PS = 4, 64, 32, 16


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_decode(Q, pool, table, lens, d_v, scale):
    from oracle import dmla_oracle as orc
    O, m, l = orc.decode_paged(Q, pool, table, lens, d_v, scale)
    return torch.from_numpy(O), torch.from_numpy(m), torch.from_numpy(l)


def _oracle_merge(O_p, m_p, l_p, out_dtype):
    from oracle import dmla_oracle as orc
    O, m, l = orc.merge_partials(O_p.numpy(), m_p.numpy(), l_p.numpy())
    return torch.from_numpy(O).to(out_dtype), torch.from_numpy(m), torch.from_numpy(l)


def _local_slice(rank, world):
    """Full problem -> this rank's slice of every sequence as a local pool / table / seqlens."""
    from flashdmla import synthetic
    from flashdmla.parallel import split_sequence_pages
    Q, pool, table, sl = synthetic.paged_decode_inputs(len(LENS), H, LENS, D_QK, PS, seed=9, std=0.5, dtype=torch.float32)
    parts = split_sequence_pages(LENS, PS, world, rank)
    max_local = max(1, max(n for _, n, _ in parts))
    ltable = torch.zeros(len(LENS), max_local, dtype=torch.int32)
    llens = torch.zeros(len(LENS), dtype=torch.int32)
    for b, (first, n, ntok) in enumerate(parts):
        ltable[b, :n] = table[b, first:first + n]
        llens[b] = ntok
    return Q, pool, table, sl, ltable, llens


def _worker(rank, world, port, mode, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "ds-flashdmla-moe_b200")]
    from flashdmla import parallel
    try:
        timeout = datetime.timedelta(seconds=4 if mode == "absent" else 60)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, timeout=timeout)
        Q, pool, table, sl, ltable, llens = _local_slice(rank, world)
        if mode == "absent" and rank == 1:
            q.put((rank, "left"))        # this rank never joins the exchange
            return

        def decode_fn(*a):
            O, m, l = _oracle_decode(*a)
            if mode == "poison" and rank == 1:
                O[0, 0, 0] = float("nan")
            return O, m, l
        O, m, l = parallel.sequence_parallel_decode(Q, pool, ltable, llens, D_V, 0.2, decode_fn=decode_fn,
                                                    merge_fn=_oracle_merge, out_dtype=torch.float32, validate=True)
        Of, mf, lf = _oracle_decode(Q, pool, table, sl, D_V, 0.2)
        err = max(float((O - Of).abs().max()), float((m - mf).abs().max()), float(((l - lf) / lf).abs().max()))
        q.put((rank, "ok", err))
    except Exception as e:       # reported to the parent, which asserts on it
        q.put((rank, "error", type(e).__name__ + ": " + str(e)[:200]))
    finally:
        if dist.is_initialized() and mode != "absent":
            dist.destroy_process_group()


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, WORLD, port, mode, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(WORLD)]
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    return sorted(out)


def test_sequence_split_decode_matches_unsplit():
    out = _run("normal")
    assert all(o[1] == "ok" for o in out), out
    assert max(o[2] for o in out) < 1e-5


def test_poisoned_partial_is_detected_on_every_rank():
    out = _run("poison")
    assert all(o[1] == "error" and "PartialCheckError" in o[2] and "[1]" in o[2] for o in out), out


def test_absent_rank_ends_the_exchange_with_an_error():
    out = _run("absent")
    r0 = [o for o in out if o[0] == 0][0]
    assert r0[1] == "error", out       # the short process-group timeout surfaces as an exception


def test_split_sequence_pages_covers_each_sequence_once():
    from flashdmla.parallel import split_sequence_pages
    for world in (1, 2, 8):
        tot = [0] * len(LENS)
        for r in range(world):
            prev_end = None
            for b, (first, n, ntok) in enumerate(split_sequence_pages(LENS, PS, world, r)):
                tot[b] += ntok
                assert 0 <= ntok <= n * PS
        assert tot == LENS


def test_pack_unpack_roundtrip():
    from flashdmla.parallel import pack_partial, unpack_partials
    O, m, l = torch.randn(3, 4, 8), torch.randn(3, 4), torch.rand(3, 4)
    buf = torch.stack([pack_partial(O, m, l), pack_partial(2 * O, m + 1, l)])
    O2, m2, l2 = unpack_partials(buf, (3, 4), 8)
    assert torch.equal(O2[0], O) and torch.equal(O2[1], 2 * O) and torch.equal(m2[1], m + 1) and torch.equal(l2[0], l)
    # the parts are views of the gathered buffer, one message apart: nothing is copied on the receiving side
    assert O2.data_ptr() == buf.data_ptr() and O2.stride(0) == buf.shape[1] and O2[0].is_contiguous()
    assert m2.stride(0) == l2.stride(0) == buf.shape[1]
