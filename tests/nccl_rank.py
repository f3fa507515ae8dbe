"""One NCCL rank of the multi-GPU exchange checks (launched by test_multi_gpu.py through
torch.distributed.run, one process per GPU).  Every rank builds the same seeded global problem,
keeps its shard, runs the product path with the real collective and compares its result with
the CPU oracle on the unsharded problem.  Exits non-zero on any mismatch."""
import datetime
import math
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "ds-flashdmla-moe_b200"), os.path.join(ROOT, "tests")]

from helpers import assert_O, assert_stats          # noqa: E402
from oracle import dmla_oracle as orc               # noqa: E402


def context_parallel_case(dev, world, rank):
    from flashdmla import device_error_flag, last_kernel
    from flashdmla.parallel import context_parallel_prefill, shard_context
    g = torch.Generator().manual_seed(33)
    Q = (torch.randn(1, 16, 1024, 576, generator=g) * 0.1).to(torch.bfloat16)
    K = (torch.randn(1, 1024, 576, generator=g) * 0.1).to(torch.bfloat16)
    sc = 1 / math.sqrt(192)
    Of, mf, lf = (torch.from_numpy(x) for x in orc.fwd_cache_latent(Q.float().numpy(), K.float().numpy(), 512, sc, causal=True))
    for zigzag in (True, False):
        O, m, l = context_parallel_prefill(shard_context(Q, world, rank, zigzag).to(dev),
                                           shard_context(K, world, rank, zigzag, dim=1).to(dev), 512, sc, zigzag=zigzag)
        assert last_kernel() == "tcgen05" and device_error_flag() == 0
        assert_O(O, shard_context(Of, world, rank, zigzag))
        assert_stats(m, l, shard_context(mf, world, rank, zigzag, dim=-1), shard_context(lf, world, rank, zigzag, dim=-1))


def sequence_parallel_case(dev, world, rank):
    from flashdmla import synthetic
    from flashdmla.parallel import sequence_parallel_decode, split_sequence_pages
    lens, H, ps = [5000, 333, 64, 2049, 1], 128, 64
    Q, pool, table, sl = synthetic.paged_decode_inputs(len(lens), H, lens, 576, ps, seed=12)
    parts = split_sequence_pages(lens, ps, world, rank)
    ltable = torch.zeros(len(lens), max(1, max(n for _, n, _ in parts)), dtype=torch.int32)
    llens = torch.zeros(len(lens), dtype=torch.int32)
    for b, (first, n, ntok) in enumerate(parts):
        ltable[b, :n] = table[b, first:first + n]
        llens[b] = ntok
    sc = 1 / math.sqrt(192)
    O, m, l = sequence_parallel_decode(Q.to(dev), pool.to(dev), ltable.to(dev), llens.to(dev), 512, sc, validate=True)
    Of, mf, lf = orc.decode_paged(Q.float().numpy(), pool.float().numpy(), table.numpy(), sl.numpy(), 512, sc)
    assert_O(O, Of)
    assert_stats(m, l, mf, lf)
    # the same step with every buffer allocated once, eagerly and replayed from a CUDA graph (three split counts:
    # the attention kernel writing the message itself, and split-KV partials merged into it)
    import flashdmla
    from flashdmla.parallel import SequenceParallelDecoder
    Qd, pd, td, ld = Q.to(dev), pool.to(dev), ltable.to(dev), llens.to(dev)
    for splits in (1, 3, None):
        dec = SequenceParallelDecoder(len(lens), H, 576, 512, ps, int(llens.max()), dev, scale=sc, num_splits=splits)
        O2, m2, l2 = (t.clone() for t in dec.step(Qd, pd, td, ld))
        assert_O(O2, Of)
        assert_stats(m2, l2, mf, lf)
        dec.capture(Qd, pd, td, ld)
        for t in dec.out:
            t.zero_()
        O3, m3, l3 = dec.replay()
        torch.cuda.synchronize()
        assert torch.equal(O3, O2) and torch.equal(m3, m2) and torch.equal(l3, l2)
        # the exchange and the merge as ONE kernel over peer memory: bit-identical to all-gather + merge, on several
        # steps in a row (both slots of the exchange buffers, the step counters) and replayed from a CUDA graph
        peer = SequenceParallelDecoder(len(lens), H, 576, 512, ps, int(llens.max()), dev, scale=sc, num_splits=splits,
                                       exchange="peer")
        for _ in range(3):
            for t in peer.out:
                t.zero_()
            O4, m4, l4 = peer.step(Qd, pd, td, ld)
            torch.cuda.synchronize()
            assert torch.equal(O4, O2) and torch.equal(m4, m2) and torch.equal(l4, l2)
        assert flashdmla.last_kernel() == "exchange_merge_kernel"
        peer.capture(Qd, pd, td, ld)
        for _ in range(3):
            for t in peer.out:
                t.zero_()
            O5, m5, l5 = peer.replay()
            torch.cuda.synchronize()
            assert torch.equal(O5, O2) and torch.equal(m5, m2) and torch.equal(l5, l2)
        assert flashdmla.device_error_flag() == 0
        peer.xch.close()


def absent_peer_case(dev, world, rank):
    """A rank that does not take part in a step of the peer exchange: the others' kernels give up their wait after the
    time limit, return, and report error code 31 through the device flag; the context stays usable and a new exchange
    works again.  The absent rank is simply not launching (it sits in a host barrier), nothing is killed."""
    import flashdmla
    from flashdmla.exchange import PeerExchange
    rows, d_v = 64, 512
    g = torch.Generator().manual_seed(900 + rank)
    msg = torch.cat([torch.randn(rows * d_v, generator=g), torch.randn(rows, generator=g), torch.rand(rows, generator=g) + 0.5]).to(dev)
    out = (torch.full((rows, d_v), 7.0, device=dev), torch.full((rows,), 7.0, device=dev), torch.full((rows,), 7.0, device=dev))
    xch = PeerExchange(rows, d_v, dev, timeout_ms=300)
    xch.merge(msg, out)                                   # a step everybody takes part in
    torch.cuda.synchronize()
    assert flashdmla.device_error_flag() == 0 and float(out[2].min()) > 0.0 and float((out[2] - 7.0).abs().min()) > 0.0
    dist.barrier()
    for t in out:
        t.fill_(7.0)
    if rank != world - 1:                                 # the last rank stays away from this step
        xch.merge(msg, out)
        torch.cuda.synchronize()
        assert flashdmla.device_error_flag() == 31
        assert flashdmla.device_error_flag(reset=True) == 31 and flashdmla.device_error_flag() == 0
        if world == 2:                                    # every row needed the absent rank: nothing was written
            assert all(float((t - 7.0).abs().max()) == 0.0 for t in out)
    dist.barrier()
    xch.close()
    again = PeerExchange(rows, d_v, dev, timeout_ms=2000)   # fresh buffers and counters: the ranks are in step again
    again.merge(msg, out)
    torch.cuda.synchronize()
    assert flashdmla.device_error_flag() == 0 and float((out[2] - 7.0).abs().min()) > 0.0
    dist.barrier()
    again.close()


def expert_parallel_case(dev, world, rank):
    from flashdmla.moe import MoEFFN
    layer = MoEFFN(d_model=128, d_ff=256, n_experts=12, top_k=3, capacity_factor=1.0, device=dev, seed=4)    # same weights on every rank
    x = (torch.randn(150 + 7 * rank, 128, generator=torch.Generator().manual_seed(50 + rank)) * 0.5).to(torch.bfloat16).to(dev)
    cap = layer.capacity(160)                             # one capacity for all ranks (they hold 150, 157, ... tokens)
    got = layer.forward_ep(x, capacity=cap)               # experts sharded 12 -> world ranks, rows over NCCL all-to-all
    want = layer.forward(x, capacity=cap)                 # all experts here
    err = float((got.float() - want.float()).norm() / want.float().norm())
    assert err < 5e-3, err                                # same arithmetic, other GEMM batch shapes
    if layer.E % world == 0:
        got2 = layer.forward_ep_batched(x, cap)  # padded rows, equal splits, no host read-back
        err2 = float((got2.float() - want.float()).norm() / want.float().norm())
        assert err2 < 5e-3, err2


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=90))   # a mismatch ends in an error, not a hang
    try:
        orc.build()
        context_parallel_case(dev, world, rank)
        sequence_parallel_case(dev, world, rank)
        expert_parallel_case(dev, world, rank)
        absent_peer_case(dev, world, rank)
        torch.cuda.synchronize()
        dist.barrier()
        print(f"rank {rank} of {world}: exchange checks passed", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
