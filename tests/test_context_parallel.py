"""Context-parallel causal prefill: chunk bookkeeping and the gloo exchange on the CPU (the
per-rank attention stood in for by the oracle), the real kernels on the GPU with the ranks
run one after another over an in-process gather."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_O, assert_stats

B, H, S, D_QK, D_V = 2, 3, 48, 16, 8


def _problem(seed=4, dtype=torch.float32, b=B, h=H, s=S, dq=D_QK, std=0.5):
    g = torch.Generator().manual_seed(seed)
    Q = (torch.randn(b, h, s, dq, generator=g) * std).to(dtype)
    K = (torch.randn(b, s, dq, generator=g) * std).to(dtype)
    return Q, K


def _oracle_attn(Q, K, d_v, scale):
    from oracle import dmla_oracle as orc
    O, m, l = orc.fwd_cache_latent(Q.float().numpy(), K.float().numpy(), d_v, scale, causal=True)
    return torch.from_numpy(O), torch.from_numpy(m), torch.from_numpy(l)


def test_chunks_cover_the_sequence_and_balance_the_triangle():
    from flashdmla.parallel import context_chunks
    for world in (1, 2, 4, 8):
        owned = sorted(c for r in range(world) for c in context_chunks(world, r))
        assert owned == list(range(2 * world))
        work = {sum(c + 1 for c in context_chunks(world, r)) for r in range(world)}
        assert work == {2 * world + 1}                    # every rank: the same number of chunk blocks
        assert [context_chunks(world, r, zigzag=False) for r in range(world)] == [[r] for r in range(world)]


@pytest.mark.parametrize("zigzag", [True, False])
def test_shard_then_assemble_is_the_identity(zigzag):
    from flashdmla.parallel import assemble_context, shard_context
    x = torch.arange(2 * 48 * 3, dtype=torch.float32).view(2, 48, 3)
    for world in (1, 2, 4):
        gathered = torch.stack([shard_context(x, world, r, zigzag, dim=1) for r in range(world)])
        assert torch.equal(assemble_context(gathered, zigzag), x)
    with pytest.raises(ValueError):
        shard_context(x, 5, 0, zigzag, dim=1)


@pytest.mark.parametrize("zigzag", [True, False])
def test_every_rank_in_turn_matches_the_unsharded_problem(zigzag):
    """No process group: the gather is a stack of all ranks' shards."""
    from flashdmla.parallel import context_parallel_prefill, shard_context
    Q, K = _problem()
    sc = 0.3
    Of, mf, lf = _oracle_attn(Q, K, D_V, sc)
    for world in (1, 3):
        k_all = torch.stack([shard_context(K, world, r, zigzag, dim=1) for r in range(world)])
        for r in range(world):
            O, m, l = context_parallel_prefill(shard_context(Q, world, r, zigzag), k_all[r], D_V, sc, zigzag=zigzag,
                                               attn_fn=_oracle_attn, gather_fn=lambda local: k_all, world=world, rank=r)
            assert torch.allclose(O, shard_context(Of, world, r, zigzag), atol=1e-6)
            assert torch.allclose(m, shard_context(mf, world, r, zigzag, dim=-1), atol=1e-6)
            assert torch.allclose(l, shard_context(lf, world, r, zigzag, dim=-1), rtol=1e-6)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "ds-flashdmla-moe_b200"), os.path.join(root, "tests")]
    from flashdmla import parallel
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        Q, K = _problem()
        Of, mf, lf = _oracle_attn(Q, K, D_V, 0.3)
        O, m, l = parallel.context_parallel_prefill(parallel.shard_context(Q, world, rank), parallel.shard_context(K, world, rank, dim=1),
                                                    D_V, 0.3, attn_fn=_oracle_attn)
        err = max(float((O - parallel.shard_context(Of, world, rank)).abs().max()),
                  float((m - parallel.shard_context(mf, world, rank, dim=-1)).abs().max()),
                  float((l / parallel.shard_context(lf, world, rank, dim=-1) - 1).abs().max()))
        q.put((rank, "ok", err))
    except Exception as e:
        q.put((rank, "error", type(e).__name__ + ": " + str(e)[:200]))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_two_gloo_ranks_gather_the_latent_rows_and_match():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert all(o[1] == "ok" for o in out), out
    assert max(o[2] for o in out) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("world,zigzag", [(4, True), (2, False)])
def test_kernels_on_each_ranks_chunks_match_the_oracle(cuda, world, zigzag):
    """The product operator on every rank's chunks (ranks one after another on one GPU, the gather
    a stack of the shards) against the oracle on the unsharded problem, 576/512 bf16."""
    from flashdmla.parallel import context_parallel_prefill, shard_context
    from flashdmla import last_kernel
    Q, K = _problem(seed=21, dtype=torch.bfloat16, b=1, h=16, s=1024, dq=576, std=0.1)
    sc = 1 / math.sqrt(192)
    Of, mf, lf = _oracle_attn(Q, K, 512, sc)
    k_all = torch.stack([shard_context(K, world, r, zigzag, dim=1) for r in range(world)]).to(cuda)
    for r in range(world):
        O, m, l = context_parallel_prefill(shard_context(Q, world, r, zigzag).to(cuda), k_all[r], 512, sc, zigzag=zigzag,
                                           gather_fn=lambda local: k_all, world=world, rank=r)
        assert last_kernel() == "tcgen05"
        assert_O(O, shard_context(Of, world, r, zigzag))
        assert_stats(m, l, shard_context(mf, world, r, zigzag, dim=-1), shard_context(lf, world, r, zigzag, dim=-1))
