"""Multi-GPU use of the Flash-DMLA operators: one process per GPU.

Two patterns, as the path shards:
  * batch (decode) or head (prefill) sharding - every rank runs the same
    operator on its shard, no collective on the data path;
  * long-context decode - the KV sequence of every request is split into
    contiguous page-aligned slices, one per rank (the balanced-with-remainder
    rule of the reference's csrc/attention/fa2_fwd_mpi.cu:47-53).  Each rank
    attends its own slice and the partial (O, m, l) are all-gathered over
    NCCL/NVLink and merged with the log-sum-exp rule.  The reference's MPI
    wrapper all-gathers the keys and values themselves on the host
    (fa2_fwd_mpi.cu:65-74); gathering the partials moves (d_v+2) floats per
    row instead of the whole cache.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """(offset, length) of rank's contiguous share of n items; the remainder
    goes to the first ranks (rows_of/off_of in fa2_fwd_mpi.cu:47-53)."""
    base, rem = divmod(int(n), int(world))
    length = base + (1 if rank < rem else 0)
    offset = rank * base + min(rank, rem)
    return offset, length


def split_sequence_pages(seqlens: List[int], page_size: int, world: int, rank: int):
    """Per sequence: (first_page, n_pages, n_tokens) of rank's KV slice."""
    out = []
    for s in seqlens:
        pages = (int(s) + page_size - 1) // page_size
        off, ln = shard_range(pages, world, rank)
        lo = off * page_size
        hi = min((off + ln) * page_size, int(s))
        out.append((off, ln, max(hi - lo, 0)))
    return out


def pack_partial(O: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """[..., d_v] + [...] + [...] -> one [..., d_v + 2] fp32 message."""
    return torch.cat([O.float(), m.float()[..., None], l.float()[..., None]], dim=-1).contiguous()


def unpack_partials(buf: torch.Tensor):
    """[W, ..., d_v + 2] -> O_p [W, ..., d_v], m_p, l_p [W, ...] (contiguous)."""
    return buf[..., :-2].contiguous(), buf[..., -2].contiguous(), buf[..., -1].contiguous()


class PartialCheckError(RuntimeError):
    """A gathered partial (O, m, l) is not a possible softmax partial."""


def check_partials(O_p: torch.Tensor, m_p: torch.Tensor, l_p: torch.Tensor) -> None:
    """Host-side failure detection for the exchange step: every rank's partial must
    have finite O, l >= 0, and m finite or -inf exactly where l == 0.  Names the
    first offending rank."""
    bad_O = ~torch.isfinite(O_p).flatten(1).all(dim=1)
    bad_l = (~torch.isfinite(l_p) | (l_p < 0)).flatten(1).any(dim=1)
    bad_m = (torch.isnan(m_p) | (torch.isinf(m_p) & ((m_p > 0) | (l_p != 0)))).flatten(1).any(dim=1)
    bad = (bad_O | bad_l | bad_m).nonzero().flatten().tolist()
    if bad:
        raise PartialCheckError(f"invalid partial attention result received from rank(s) {bad}")


def sequence_parallel_decode(Q, local_pool, local_page_table, local_seqlens, d_v, scale=None,
                             group: Optional[dist.ProcessGroup] = None, out_dtype=None,
                             num_splits: Optional[int] = None,
                             decode_fn: Optional[Callable] = None,
                             merge_fn: Optional[Callable] = None, validate: bool = False):
    """Decode when every rank holds one slice of each sequence's paged cache.

    Q [B,H,d_qk] is replicated; local_* describe this rank's slice only.
    Returns the merged O [B,H,d_v], m, l [B,H] on every rank.
    decode_fn / merge_fn default to the CUDA operators; tests of the host-side
    protocol may inject CPU stand-ins.
    """
    if decode_fn is None or merge_fn is None:
        from . import ops
        if decode_fn is None:
            def decode_fn(Q, pool, table, lens, d_v, scale):
                Op, mp, lp = ops.flash_dmla_paged_decode(Q, pool, table, lens, d_v, scale,
                                                         num_splits=num_splits, partial_only=True)
                if Op.shape[0] == 1:
                    return Op[0], mp[0], lp[0]
                return ops.merge_partials(Op, mp, lp, torch.float32)
        if merge_fn is None:
            merge_fn = ops.merge_partials
    O_loc, m_loc, l_loc = decode_fn(Q, local_pool, local_page_table, local_seqlens, d_v, scale)
    msg = pack_partial(O_loc, m_loc, l_loc)
    world = dist.get_world_size(group)
    flat = torch.empty((world * msg.shape[0],) + tuple(msg.shape[1:]), dtype=msg.dtype, device=msg.device)
    dist.all_gather_into_tensor(flat, msg, group=group)      # concatenated along dim 0, rank-major
    gathered = flat.view((world,) + tuple(msg.shape))
    O_p, m_p, l_p = unpack_partials(gathered)
    if validate:          # synchronises; meant for debugging and for the failure-detection tests
        check_partials(O_p, m_p, l_p)
    return merge_fn(O_p, m_p, l_p, out_dtype or Q.dtype)
