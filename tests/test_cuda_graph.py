"""A whole decode step - append the new latent row, advance the lengths, attend - captured once as a
CUDA graph and replayed with fresh inputs.  Nothing on the path may allocate, synchronise or read
the device from the host while the stream is capturing, and everything that changes from step to
step (queries, new rows, lengths) is read from device memory by the kernels."""
import math

import pytest
import torch

from helpers import assert_O, assert_stats
from oracle import dmla_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("splits", [1, 3])
def test_decode_step_replays_as_a_cuda_graph(cuda, splits):
    import flashdmla
    from flashdmla import ops
    g = torch.Generator().manual_seed(77 + splits)
    B, H, dq, dv, ps, max_pages = 3, 128, 576, 512, 64, 8
    sc = 1 / math.sqrt(192)
    lens0 = [130, 63, 300]                                  # 63 -> 64 -> 65 crosses a page boundary during the replays
    n_pages = B * max_pages
    perm = torch.randperm(n_pages, generator=g).to(torch.int32).view(B, max_pages)      # pages reserved up front
    pool_h = torch.zeros(n_pages, ps, dq, dtype=torch.bfloat16)
    hist = []
    for b, n in enumerate(lens0):
        rows = (torch.randn(n, dq, generator=g) * 0.1).to(torch.bfloat16)
        hist.append(rows)
        for t in range(n):
            pool_h[perm[b, t // ps], t % ps] = rows[t]
    pool, table = pool_h.to(cuda), perm.to(cuda)
    lens = torch.tensor(lens0, dtype=torch.int32, device=cuda)
    q_in = torch.zeros(B, H, dq, dtype=torch.bfloat16, device=cuda)           # static inputs of the graph
    row_in = torch.zeros(B, 1, dq, dtype=torch.bfloat16, device=cuda)
    ws = flashdmla.DecodeWorkspace()

    def step():
        ops.cache_append(row_in, pool, table, lens)          # the new row goes to position lens[b]
        lens.add_(1)
        return flashdmla.flash_dmla_paged_decode(q_in, pool, table, lens, dv, sc, num_splits=splits, workspace=ws,
                                                 max_seqlen=max_pages * ps)

    # warm-up outside the capture (first-use queries of the library, workspace allocation), then undo it
    side = torch.cuda.Stream(device=cuda)
    with torch.cuda.stream(side):
        step()
    torch.cuda.synchronize()
    lens.sub_(1)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        O, m, l = step()
    for it in range(3):
        q = (torch.randn(B, H, dq, generator=g) * 0.1).to(torch.bfloat16)
        new = (torch.randn(B, 1, dq, generator=g) * 0.1).to(torch.bfloat16)
        q_in.copy_(q.to(cuda))
        row_in.copy_(new.to(cuda))
        graph.replay()
        torch.cuda.synchronize()
        for b in range(B):
            hist[b] = torch.cat([hist[b], new[b]])
        assert lens.tolist() == [n + it + 1 for n in lens0]
        for b in range(B):
            K = hist[b].float()
            Or, mr, lr = orc.attn_plain(q[b].float(), K, K[:, :dv], sc)
            assert_O(O[b], Or)
            assert_stats(m[b], l[b], mr, lr)
    assert flashdmla.last_kernel() == "tcgen05" and flashdmla.device_error_flag() == 0
