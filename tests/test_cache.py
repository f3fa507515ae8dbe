"""Paged latent cache: page allocator on the CPU, append -> decode round trip on the GPU."""
import math

import pytest
import torch

from helpers import assert_O, assert_stats
from oracle import dmla_oracle as orc


def test_allocator_bookkeeping_needs_no_gpu():
    from flashdmla.cache import PagedLatentCache
    from flashdmla import FlashDMLAError
    c = PagedLatentCache(num_pages=10, page_size=4, d_qk=8, max_seqs=3, max_pages_per_seq=4, device="cpu")
    a, b = c.new_sequence(), c.new_sequence()
    assert c.reserve([a, b], 5).tolist() == [0, 0]           # 2 pages each
    assert c.length(a) == 5 and len(c.pages_of(a)) == 2 and c.free_pages == 6
    assert c.reserve([a], 3).tolist() == [5]                 # 5 + 3 = 8 tokens still fit 2 pages
    assert len(c.pages_of(a)) == 2
    assert c.reserve([a], 1).tolist() == [8]                 # a third page
    assert len(c.pages_of(a)) == 3 and c.free_pages == 5
    live = c.pages_of(a) + c.pages_of(b)
    assert len(set(live)) == len(live)                       # no page belongs to two sequences
    assert c.h_table[a, :3].tolist() == c.pages_of(a)
    with pytest.raises(FlashDMLAError):                      # 4 pages per sequence at most; nothing changes
        c.reserve([a], 100)
    assert c.length(a) == 9 and c.free_pages == 5
    with pytest.raises(FlashDMLAError):
        c.reserve([a, a], 1)
    d = c.new_sequence()
    with pytest.raises(FlashDMLAError):
        c.new_sequence()                                     # max_seqs = 3
    c.reserve([a], 4)                                        # a: 13 tokens, 4 pages; 4 pages left
    with pytest.raises(FlashDMLAError):                      # b needs 2 more pages, d needs 3: nothing is changed
        c.reserve([b, d], 11)
    assert c.free_pages == 4 and c.length(d) == 0 and c.length(b) == 5
    freed = c.pages_of(a)
    c.free_sequence(a)
    assert c.free_pages == 8
    with pytest.raises(FlashDMLAError):
        c.length(a)                                          # the slot is dead
    e = c.new_sequence()
    c.reserve([e], 4)
    assert c.pages_of(e)[0] in freed                         # pages are recycled


@pytest.mark.gpu
def test_append_then_decode_matches_oracle(cuda):
    from flashdmla.cache import PagedLatentCache
    g = torch.Generator().manual_seed(9)
    H, dq, dv, ps = 16, 576, 512, 64
    c = PagedLatentCache(num_pages=64, page_size=ps, d_qk=dq, max_seqs=4, max_pages_per_seq=16, device=cuda)
    slots = [c.new_sequence() for _ in range(3)]
    hist = {s: [] for s in slots}

    def add(ss, n):
        rows = (torch.randn(len(ss), n, dq, generator=g) * 0.1).to(torch.bfloat16)
        c.append(ss, rows.to(cuda))
        for i, s in enumerate(ss):
            hist[s].append(rows[i])
    add(slots, 100)                 # prefill of all three
    add(slots[:2], 37)              # two of them grow across a page boundary
    for _ in range(5):              # decode steps, one row at a time
        add(slots, 1)
    c.free_sequence(slots[1])       # its pages go back and are reused by a new sequence
    s_new = c.new_sequence()
    slots[1] = s_new
    hist[s_new] = []
    add([s_new], 70)
    want = {s: torch.cat(hist[s]) for s in slots}
    got = c.gather(slots, 160).cpu()
    for i, s in enumerate(slots):
        n = want[s].shape[0]
        assert c.length(s) == n
        assert torch.equal(got[i, :n], want[s]) and (got[i, n:] == 0).all()
    Q = (torch.randn(3, H, dq, generator=g) * 0.1).to(torch.bfloat16)
    sc = 1 / math.sqrt(192)
    O, m, l = c.decode(Q.to(cuda), slots, dv, sc)
    for i, s in enumerate(slots):
        K = want[s].float()
        Or, mr, lr = orc.attn_plain(Q[i].float(), K, K[:, :dv], sc)
        assert_O(O[i], Or)
        assert_stats(m[i], l[i], mr, lr)
