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
    row instead of the whole cache;
  * context-parallel prefill - the sequence dimension of a causal prefill is cut
    into chunks, every rank owns the queries and the latent rows of its chunks,
    the bf16 latent rows are all-gathered once (the counterpart of the
    reference's host all-gather of K and V, fa2_fwd_mpi.cu:65-74: 1152 bytes per
    token here, against H (d_v + 2) floats per token for gathered partials) and
    every rank attends its own query chunks over the key prefix they may see.
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


# One rank's partial result travels as ONE fp32 message laid out in blocks,
#   [ O (rows x d_v) | m (rows) | l (rows) ],
# so that the decode (or the local merge) writes its three outputs straight into the message and the
# receiver merges the gathered messages where they lie, as strided parts: nothing is packed or unpacked.
def message_views(buf: torch.Tensor, lead: Tuple[int, ...], d_v: int):
    """Views (O [*lead, d_v], m [*lead], l [*lead]) of one message, or of a [W, n] stack of messages
    ([W, *lead, d_v], [W, *lead], [W, *lead]; the parts are then n elements apart)."""
    rows = 1
    for x in lead:
        rows *= int(x)
    n = rows * (d_v + 2)
    if buf.dim() == 1:
        if buf.numel() != n:
            raise ValueError("message size does not match its shape")
        return (buf[: rows * d_v].view(*lead, d_v), buf[rows * d_v: rows * d_v + rows].view(*lead),
                buf[rows * d_v + rows:].view(*lead))
    W = buf.shape[0]
    if buf.dim() != 2 or buf.shape[1] != n:
        raise ValueError("expected a [world, message] stack")
    return (buf[:, : rows * d_v].unflatten(1, (*lead, d_v)), buf[:, rows * d_v: rows * d_v + rows].unflatten(1, lead),
            buf[:, rows * d_v + rows:].unflatten(1, lead))


def pack_partial(O: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """(O [..., d_v], m [...], l [...]) -> one message (a copy; the CUDA path writes into message_views instead)."""
    return torch.cat([O.float().reshape(-1), m.float().reshape(-1), l.float().reshape(-1)])


def unpack_partials(buf: torch.Tensor, lead: Tuple[int, ...], d_v: int):
    """[W, n] stack of messages -> O_p [W, *lead, d_v], m_p, l_p [W, *lead] (views)."""
    return message_views(buf, tuple(lead), d_v)


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
                             merge_fn: Optional[Callable] = None, validate: bool = False,
                             workspace=None, timing_events=None):
    """Decode when every rank holds one slice of each sequence's paged cache.

    Q [B,H,d_qk] is replicated; local_* describe this rank's slice only.
    Returns the merged O [B,H,d_v], m, l [B,H] on every rank.
    decode_fn / merge_fn default to the CUDA operators; tests of the host-side
    protocol may inject CPU stand-ins.  workspace: a flashdmla.DecodeWorkspace to
    reuse across steps.  timing_events: four CUDA events recorded on the current
    stream at the start, after the local partial, after the all-gather and after
    the merge (measurement only).
    """
    B, H = Q.shape[0], Q.shape[1]
    world = dist.get_world_size(group)
    n = B * H * (d_v + 2)
    rec = (lambda i: timing_events[i].record()) if timing_events is not None else (lambda i: None)
    rec(0)
    msg = torch.empty(n, dtype=torch.float32, device=Q.device)
    mO, mm, ml = message_views(msg, (B, H), d_v)
    if decode_fn is None:
        from . import ops
        # the rank's partial straight into its message: one call, the library picks the schedule and merges its pieces
        if num_splits is None:
            num_splits = (ops.suggest_partial_slabs(B, H, int(local_page_table.shape[1]) * int(local_pool.shape[1]),
                                                    int(local_pool.shape[1])) if (Q.shape[-1], d_v) == (576, 512) else 1)
        scratch = workspace.get(num_splits, B, H, d_v, Q.device) if (workspace is not None and num_splits > 1) else None
        ops.flash_dmla_paged_decode_partial(Q, local_pool, local_page_table, local_seqlens, d_v, scale,
                                            num_splits=num_splits, out=(mO, mm, ml), scratch=scratch)
    else:
        O_loc, m_loc, l_loc = decode_fn(Q, local_pool, local_page_table, local_seqlens, d_v, scale)
        mO.copy_(O_loc); mm.copy_(m_loc); ml.copy_(l_loc)
    if merge_fn is None:
        from . import ops
        merge_fn = ops.merge_partials
    rec(1)
    flat = torch.empty(world * n, dtype=torch.float32, device=Q.device)
    dist.all_gather_into_tensor(flat, msg, group=group)      # rank-major
    rec(2)
    O_p, m_p, l_p = message_views(flat.view(world, n), (B, H), d_v)
    if validate:          # synchronises; meant for debugging and for the failure-detection tests
        check_partials(O_p, m_p, l_p)
    res = merge_fn(O_p, m_p, l_p, out_dtype or Q.dtype)
    rec(3)
    return res


class SequenceParallelDecoder:
    """`sequence_parallel_decode` for a serving loop: every buffer of the step (split-KV partials, the rank's
    message, the gathered stack, the result) is allocated once, the split count is chosen once, and the step can
    be captured into a CUDA graph - local attention, local merge, the NCCL all-gather and the final merge replay as
    one launch, which matters when a rank's slice is attended in tens of microseconds and a Python host would
    otherwise spend longer enqueueing the step than the GPUs spend running it.

    B, H, d_qk, d_v, page_size: the problem; max_local_tokens: the longest slice any sequence has on this rank
    (fixes the split count).  The tensors handed to `step` may change from call to call; a captured graph replays on
    the tensors it was captured with (update them in place).

    exchange="nccl": all-gather of the messages with NCCL, then the merge kernel.  exchange="peer" (ranks of one
    node): `flashdmla.exchange.PeerExchange` - one kernel per rank sends its partial rows over NVLink to the ranks that
    own them, merges the rows it owns and hands the merged rows to every peer; same result bit for bit, one launch
    instead of a collective and a merge.
    """

    def __init__(self, B: int, H: int, d_qk: int, d_v: int, page_size: int, max_local_tokens: int, device,
                 dtype=torch.bfloat16, scale: Optional[float] = None, group: Optional[dist.ProcessGroup] = None,
                 num_splits: Optional[int] = None, exchange: str = "nccl"):
        from . import ops
        if exchange not in ("nccl", "peer"):
            raise ValueError("exchange must be 'nccl' or 'peer'")
        self.xch = None
        if exchange == "peer":
            from .exchange import PeerExchange
            self.xch = PeerExchange(B * H, d_v, device, group)
        self.B, self.H, self.d_v, self.scale, self.group = B, H, d_v, scale, group
        self.world = dist.get_world_size(group)
        n = B * H * (d_v + 2)
        self.msg = torch.empty(n, dtype=torch.float32, device=device)
        self.flat = None if self.xch is not None else torch.empty(self.world * n, dtype=torch.float32, device=device)
        self.out = (torch.empty(B, H, d_v, dtype=dtype, device=device), torch.empty(B, H, dtype=torch.float32, device=device),
                    torch.empty(B, H, dtype=torch.float32, device=device))
        self.splits = int(num_splits) if num_splits else (ops.suggest_partial_slabs(B, H, max(int(max_local_tokens), 1), page_size)
                                                          if (d_qk, d_v) == (576, 512) else 1)
        s = self.splits
        self.part = None if s == 1 else (torch.empty(s, B, H, d_v, dtype=torch.float32, device=device),
                                         torch.empty(s, B, H, dtype=torch.float32, device=device),
                                         torch.empty(s, B, H, dtype=torch.float32, device=device))
        self.graph = None

    def step(self, Q, local_pool, local_page_table, local_seqlens):
        """One decode step; returns (O [B,H,d_v], m, l) - the same tensors every call."""
        from . import ops
        if self.xch is not None and self.part is not None:
            # the pieces of the local slice stay in the scratch slabs; one kernel merges them, exchanges and merges again
            ops.flash_dmla_paged_decode_partial(Q, local_pool, local_page_table, local_seqlens, self.d_v, self.scale,
                                                num_splits=self.splits, scratch=self.part, pieces_only=True)
            return self.xch.merge_parts(self.part, self.msg, self.out)
        mO, mm, ml = message_views(self.msg, (self.B, self.H), self.d_v)
        ops.flash_dmla_paged_decode_partial(Q, local_pool, local_page_table, local_seqlens, self.d_v, self.scale,
                                            num_splits=self.splits, out=(mO, mm, ml), scratch=self.part)
        if self.xch is not None:
            return self.xch.merge(self.msg, self.out)
        dist.all_gather_into_tensor(self.flat, self.msg, group=self.group)
        O_p, m_p, l_p = message_views(self.flat.view(self.world, -1), (self.B, self.H), self.d_v)
        ops.merge_partials(O_p, m_p, l_p, self.out[0].dtype, out=self.out)
        return self.out

    def capture(self, Q, local_pool, local_page_table, local_seqlens, warmup: int = 3):
        """Capture one step on these tensors into a CUDA graph (after `warmup` eager steps, which also bring up the
        NCCL communicator); `replay()` then runs it.  Every rank must capture and replay the same number of times."""
        for _ in range(max(1, warmup)):
            self.step(Q, local_pool, local_page_table, local_seqlens)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device=Q.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                self.step(Q, local_pool, local_page_table, local_seqlens)
        torch.cuda.synchronize()
        self.graph = graph
        return self

    def replay(self):
        self.graph.replay()
        return self.out


# --------------------------------------------------------------------------- #
# context-parallel causal prefill
# --------------------------------------------------------------------------- #
def context_chunks(world: int, rank: int, zigzag: bool = True) -> List[int]:
    """Sequence chunks a rank owns, in the order they sit in its local tensors.

    zigzag: the sequence is cut into 2*world chunks and rank r owns chunks r and
    2*world-1-r.  Chunk c attends (c+1) chunks of keys, so every rank does
    (r+1) + (2*world-r) = 2*world+1 chunk-blocks of work: the causal triangle is
    balanced.  Otherwise: world chunks, rank r owns chunk r (the contiguous
    split of fa2_fwd_mpi.cu:47-53; rank world-1 then does world times the work
    of rank 0)."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    return [rank, 2 * world - 1 - rank] if zigzag else [rank]


def assemble_context(gathered: torch.Tensor, zigzag: bool = True) -> torch.Tensor:
    """[world, B, S_local, d] as all-gathered (rank-major) -> [B, S, d] in sequence order."""
    world, B, s_loc, d = gathered.shape
    if not zigzag:
        return gathered.permute(1, 0, 2, 3).reshape(B, world * s_loc, d)
    if s_loc % 2:
        raise ValueError("zigzag layout needs an even local length")
    lc = s_loc // 2
    first = gathered[:, :, :lc].permute(1, 0, 2, 3)                 # chunks 0 .. world-1
    second = gathered[:, :, lc:].flip(0).permute(1, 0, 2, 3)        # chunks world .. 2 world-1
    return torch.cat([first, second], dim=1).reshape(B, 2 * world * lc, d)


def shard_context(x: torch.Tensor, world: int, rank: int, zigzag: bool = True, dim: int = -2) -> torch.Tensor:
    """A rank's local part of a tensor whose dimension `dim` is the full sequence (the inverse
    of assemble_context; for laying out inputs and for comparing results)."""
    n_chunks = 2 * world if zigzag else world
    S = x.shape[dim]
    if S % n_chunks:
        raise ValueError(f"sequence length {S} is not a multiple of {n_chunks} chunks")
    lc = S // n_chunks
    return torch.cat([x.narrow(dim, c * lc, lc) for c in context_chunks(world, rank, zigzag)], dim=dim).contiguous()


def context_parallel_prefill(Q_local, K_lat_local, d_v, scale=None, group: Optional[dist.ProcessGroup] = None,
                             zigzag: bool = True, attn_fn: Optional[Callable] = None,
                             gather_fn: Optional[Callable] = None, world: Optional[int] = None,
                             rank: Optional[int] = None):
    """Causal cache-latent prefill with the sequence sharded across ranks (forward only).

    Q_local [B,H,S_local,d_qk] and K_lat_local [B,S_local,d_qk] hold this rank's
    chunks (context_chunks order).  Returns O [B,H,S_local,d_v], m, l [B,H,S_local]
    for the same rows.  One all-gather of the latent rows; no other exchange.
    attn_fn(Q, K_lat, d_v, scale) -> (O, m, l) defaults to the CUDA operator with
    causal=True (bottom-right aligned, so a chunk of queries against the key prefix
    that ends with the same chunk is exactly its slice of the full causal problem);
    gather_fn(local) -> [world, ...] defaults to all_gather_into_tensor.  Tests
    inject stand-ins for both.
    """
    if world is None:
        world = dist.get_world_size(group)
    if rank is None:
        rank = dist.get_rank(group)
    if attn_fn is None:
        from . import ops

        def attn_fn(Q, K, d_v, scale):
            return ops.flash_dmla_cache_latent(Q, K, d_v, scale, causal=True)
    if gather_fn is None:
        def gather_fn(local):
            flat = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(flat, local.contiguous(), group=group)
            return flat.view((world,) + tuple(local.shape))
    if Q_local.dim() != 4 or K_lat_local.dim() != 3 or Q_local.shape[2] != K_lat_local.shape[1]:
        raise ValueError("expected Q_local [B,H,S_local,d_qk] and K_lat_local [B,S_local,d_qk]")
    chunks = context_chunks(world, rank, zigzag)
    s_loc = Q_local.shape[2]
    if s_loc % len(chunks):
        raise ValueError("zigzag layout needs an even local length")
    lc = s_loc // len(chunks)
    if scale is None:
        scale = 1.0 / (Q_local.shape[3] ** 0.5)
    K_full = assemble_context(gather_fn(K_lat_local), zigzag)
    outs = []
    with torch.no_grad():
        for i, c in enumerate(chunks):
            q = Q_local[:, :, i * lc:(i + 1) * lc].contiguous()
            k = K_full[:, :(c + 1) * lc].contiguous()
            outs.append(attn_fn(q, k, d_v, scale))
    if len(outs) == 1:
        return outs[0]
    return tuple(torch.cat([o[j] for o in outs], dim=2) for j in range(3))
