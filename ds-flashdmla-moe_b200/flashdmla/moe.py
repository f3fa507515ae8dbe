"""MoE FFN around the library's gate / pack / gather / combine kernels (the "unfused reference path"
the reference describes at README.md:17-20, and its single-node expert parallelism, README.md:21-23).

    idx, w          = route_topk(logits, k)                  # gate
    pos, perm, offs = pack(idx, E, capacity)                 # bucket + exclusive scan, deterministic
    xp              = scatter(x, pos, rows)                  # rows in expert order (or gather(x, perm, offs))
    yp              = expert MLP on xp[offs[e]:offs[e+1]]    # plain GEMMs (torch.matmul = vendor library)
    out             = combine(yp, pos, w, shared)            # renormalised weights, shared expert added

`MoEFFN.forward` runs that on one GPU.  `MoEFFN.forward_ep` shards the experts over the ranks of a
process group (one process per GPU): packed rows are ordered by expert, so the rows for rank r's
experts are one contiguous range; counts and rows are exchanged with `all_to_all_single`, every
rank runs its own experts, and the results travel back the same way.  Forward only.
"""
from __future__ import annotations

import math
from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib
from ._lib import FlashDMLAError, check
from .ops import _dtype_code, _need_cuda, _ptr, _stream


def route_topk(logits: torch.Tensor, k: int):
    """logits [T,E] fp32 -> idx [T,k] int32, w [T,k] fp32."""
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise FlashDMLAError("logits must be [T,E] float32")
    logits = logits.contiguous()
    T, E = logits.shape
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device):
        check(_lib.lib().fdmla_moe_route_topk(_ptr(logits), _ptr(idx), _ptr(w), T, E, int(k), _stream(logits)),
              "fdmla_moe_route_topk")
    return idx, w


def pack(idx: torch.Tensor, n_experts: int, capacity: int, padded: bool = False):
    """idx [T,k] int32 -> pos [T,k], perm [min(T k, E capacity)], offsets [E+1] (all int32, on the device).
    padded: every expert owns `capacity` packed rows (offsets[e] = e capacity; perm has E capacity entries)."""
    _need_cuda(idx)
    if idx.dtype != torch.int32 or idx.dim() != 2:
        raise FlashDMLAError("idx must be [T,k] int32")
    idx = idx.contiguous()
    T, k = idx.shape
    dev = idx.device
    pos = torch.empty(T, k, dtype=torch.int32, device=dev)
    perm = torch.empty(max(1, n_experts * capacity if padded else min(T * k, n_experts * capacity)), dtype=torch.int32, device=dev)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        L = _lib.lib()
        nbytes = L.fdmla_moe_pack_workspace_bytes(T, k, n_experts)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
        check(L.fdmla_moe_pack(_ptr(idx), _ptr(pos), _ptr(perm), _ptr(offsets), _ptr(ws), ws.numel(), T, k,
                               int(n_experts), int(capacity), int(bool(padded)), _stream(idx)), "fdmla_moe_pack")
    return pos, perm, offsets


def gather(x: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """x [T,d] -> packed [len(perm), d]; rows at and past offsets[-1] are left unwritten."""
    _need_cuda(x, perm, offsets)
    x = x.contiguous()
    packed = torch.empty(perm.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.lib().fdmla_moe_gather(_ptr(x), _ptr(perm), _ptr(offsets), _ptr(packed), perm.shape[0],
                                          offsets.shape[0] - 1, x.shape[1], _dtype_code(x), _stream(x)), "fdmla_moe_gather")
    return packed


def scatter(x: torch.Tensor, pos: torch.Tensor, n_rows: int) -> torch.Tensor:
    """x [T,d], pos [T,k] -> packed [n_rows, d] (the same rows as `gather`, each token row read once)."""
    _need_cuda(x, pos)
    x = x.contiguous()
    packed = torch.empty(n_rows, x.shape[1], dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.lib().fdmla_moe_scatter(_ptr(x), _ptr(pos.contiguous()), _ptr(packed), pos.shape[0], pos.shape[1],
                                           x.shape[1], _dtype_code(x), _stream(x)), "fdmla_moe_scatter")
    return packed


def combine(y: torch.Tensor, pos: torch.Tensor, w: torch.Tensor, shared: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y [rows,d], pos [T,k], w [T,k] -> out [T,d] (+ shared [T,d])."""
    _need_cuda(y, pos, w, shared)
    y = y.contiguous()
    T, k = pos.shape
    if shared is not None:
        shared = shared.contiguous()
        if shared.dtype != y.dtype or tuple(shared.shape) != (T, y.shape[1]):
            raise FlashDMLAError("shared must be [T,d] in y's dtype")
    out = torch.empty(T, y.shape[1], dtype=y.dtype, device=y.device)
    with torch.cuda.device(y.device):
        check(_lib.lib().fdmla_moe_combine(_ptr(y), _ptr(pos.contiguous()), _ptr(w.contiguous()), _ptr(shared), _ptr(out),
                                           T, k, y.shape[1], _dtype_code(y), _stream(y)), "fdmla_moe_combine")
    return out


def swiglu_mlp(x, W1, W3, W2):
    """(silu(x W1) * (x W3)) W2 with library GEMMs."""
    return (torch.nn.functional.silu(x @ W1) * (x @ W3)) @ W2


def _expert_mlp_batched(xb, W1, W3, W2):
    """[E, rows, d] through every expert's SwiGLU MLP on the library's tensor-core GEMM (gate fused into the first
    GEMM's epilogue).  On a GPU there is no other path: a dtype or width the kernel does not take is an error.  CPU
    tensors - the exchange tests run the host logic of the expert-parallel forward on gloo - use torch.bmm."""
    if xb.is_cuda:
        from . import gemm
        return gemm.expert_mlp(xb.contiguous(), W1.contiguous(), W3.contiguous(), W2.contiguous())
    return torch.bmm(torch.nn.functional.silu(torch.bmm(xb, W1)) * torch.bmm(xb, W3), W2)


def expert_ranges(n_experts: int, world: int):
    """Experts of every rank as (first, count): contiguous, the remainder to the first ranks."""
    base, rem = divmod(n_experts, world)
    out, first = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append((first, n))
        first += n
    return out


class MoEFFN:
    """Weights of one MoE FFN layer (random init) and its forward, on one GPU or expert-parallel."""

    def __init__(self, d_model: int, d_ff: int, n_experts: int, top_k: int, capacity_factor: float = 1.25,
                 shared_expert: bool = True, dtype=torch.bfloat16, device="cuda", seed: int = 0):
        g = torch.Generator().manual_seed(seed)

        def w(*shape, fan_in):
            return (torch.randn(*shape, generator=g) / math.sqrt(fan_in)).to(dtype).to(device)
        self.d, self.f, self.E, self.k, self.cf = d_model, d_ff, n_experts, top_k, capacity_factor
        self.Wg = (torch.randn(d_model, n_experts, generator=g) / math.sqrt(d_model)).to(device)      # gate in fp32
        self.W1, self.W3 = w(n_experts, d_model, d_ff, fan_in=d_model), w(n_experts, d_model, d_ff, fan_in=d_model)
        self.W2 = w(n_experts, d_ff, d_model, fan_in=d_ff)
        self.shared = (w(d_model, d_ff, fan_in=d_model), w(d_model, d_ff, fan_in=d_model),
                       w(d_ff, d_model, fan_in=d_ff)) if shared_expert else None

    def capacity(self, n_tokens: int) -> int:
        return max(1, int(math.ceil(self.cf * n_tokens * self.k / self.E)))

    def _route(self, x, capacity):
        idx, w = route_topk(x.float() @ self.Wg, self.k)
        pos, perm, offsets = pack(idx, self.E, capacity)
        return idx, w, pos, perm, offsets

    def forward(self, x: torch.Tensor, capacity: Optional[int] = None) -> torch.Tensor:
        """x [T,d] -> [T,d], all experts on this GPU."""
        cap = self.capacity(x.shape[0]) if capacity is None else int(capacity)
        idx, w, pos, perm, offsets = self._route(x, cap)
        xp = scatter(x, pos, perm.shape[0])
        # one grouped GEMM launch per MLP stage: the experts' row ranges are read from `offsets` on the device, no padding
        # rows are multiplied and nothing comes back to the host
        from . import gemm
        yp = gemm.expert_mlp_grouped(xp, offsets, self.W1, self.W3, self.W2)
        sh = swiglu_mlp(x, *self.shared) if self.shared is not None else None
        return combine(yp, pos, w, sh)

    def forward_batched(self, x: torch.Tensor, capacity: Optional[int] = None) -> torch.Tensor:
        """The same layer with padded packing: the packed rows are an [E, capacity, d] batch, the expert MLPs
        three batched GEMMs, and nothing is read back to the host (so the step can be captured in a CUDA graph).
        Rows past an expert's count are multiplied too - that is the price - and never combined."""
        cap = self.capacity(x.shape[0]) if capacity is None else int(capacity)
        idx, w = route_topk(x.float() @ self.Wg, self.k)
        pos, perm, offsets = pack(idx, self.E, cap, padded=True)
        xp = torch.zeros(self.E * cap, x.shape[1], dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            check(_lib.lib().fdmla_moe_scatter(_ptr(x.contiguous()), _ptr(pos), _ptr(xp), x.shape[0], self.k, x.shape[1],
                                               _dtype_code(x), _stream(x)), "fdmla_moe_scatter")
        xb = xp.view(self.E, cap, x.shape[1])
        yb = _expert_mlp_batched(xb, self.W1, self.W3, self.W2)
        sh = swiglu_mlp(x, *self.shared) if self.shared is not None else None
        return combine(yb.view(self.E * cap, x.shape[1]), pos, w, sh)

    def forward_ep_batched(self, x: torch.Tensor, capacity: int, group: Optional[dist.ProcessGroup] = None,
                           route_fn: Optional[Callable] = None, scatter_fn: Optional[Callable] = None,
                           combine_fn: Optional[Callable] = None) -> torch.Tensor:
        """Expert parallelism without a host read-back: padded packing makes every rank's share of the packed
        rows the same size ([experts per rank, capacity, d]), so the two all-to-alls have equal, known splits and
        the experts of a rank run as three batched GEMMs over [experts per rank, world x capacity, d].  Needs
        n_experts divisible by the number of ranks and THE SAME `capacity` ON EVERY RANK (it fixes the message
        sizes; ranks may hold different numbers of tokens).  Unused rows travel and are multiplied too."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if self.E % world:
            raise FlashDMLAError("forward_ep_batched needs n_experts divisible by the number of ranks")
        n_loc = self.E // world
        cap = int(capacity)
        if route_fn is None:
            idx, w = route_topk(x.float() @ self.Wg, self.k)
            pos, perm, offsets = pack(idx, self.E, cap, padded=True)
        else:
            idx, w, pos = route_fn(x, cap)
        if scatter_fn is None:
            xp = torch.zeros(self.E * cap, x.shape[1], dtype=x.dtype, device=x.device)
            with torch.cuda.device(x.device):
                check(_lib.lib().fdmla_moe_scatter(_ptr(x.contiguous()), _ptr(pos), _ptr(xp), x.shape[0], self.k, x.shape[1],
                                                   _dtype_code(x), _stream(x)), "fdmla_moe_scatter")
        else:
            xp = scatter_fn(x, pos, self.E * cap)
        x_in = torch.empty_like(xp)                                   # [world (source), n_loc, cap, d]
        dist.all_to_all_single(x_in, xp, group=group)
        d = x.shape[1]
        xb = x_in.view(world, n_loc, cap, d).permute(1, 0, 2, 3).reshape(n_loc, world * cap, d)
        lo = rank * n_loc
        W1, W3, W2 = self.W1[lo:lo + n_loc], self.W3[lo:lo + n_loc], self.W2[lo:lo + n_loc]
        yb = _expert_mlp_batched(xb, W1, W3, W2)
        y_out = yb.view(n_loc, world, cap, d).permute(1, 0, 2, 3).contiguous().view(self.E * cap, d)
        y_back = torch.empty_like(y_out)
        dist.all_to_all_single(y_back, y_out, group=group)
        sh = swiglu_mlp(x, *self.shared) if self.shared is not None else None
        return (combine_fn or combine)(y_back, pos, w, sh)

    def forward_ep(self, x: torch.Tensor, group: Optional[dist.ProcessGroup] = None, capacity: Optional[int] = None,
                   route_fn: Optional[Callable] = None, gather_fn: Optional[Callable] = None,
                   combine_fn: Optional[Callable] = None) -> torch.Tensor:
        """x [T_local,d] on every rank; rank r holds the weights of its experts only (indexing by global
        expert id is done here, so `self.W1` etc. may be the full tensors or a dict-like view).  The
        capacity applies per rank of origin.  route_fn / gather_fn / combine_fn default to the CUDA
        operators; tests of the exchange on CPU pass stand-ins."""
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        cap = self.capacity(x.shape[0]) if capacity is None else int(capacity)
        idx, w, pos, perm, offsets = (route_fn or self._route)(x, cap)
        xp = (gather_fn or gather)(x, perm, offsets)
        offs = offsets.tolist()
        ranges = expert_ranges(self.E, world)
        # rows this rank sends to each rank (its packed rows are ordered by expert = by owning rank)
        send_rows = [offs[f + n] - offs[f] for f, n in ranges]
        my_first, my_n = ranges[rank]
        # per-expert counts: every rank tells every other how many rows come for each of its experts
        counts_out = torch.tensor([offs[e + 1] - offs[e] for e in range(self.E)], dtype=torch.int64, device=x.device)
        counts_in = torch.empty(world * my_n, dtype=torch.int64, device=x.device)
        dist.all_to_all_single(counts_in, counts_out, output_split_sizes=[my_n] * world,
                               input_split_sizes=[n for _, n in ranges], group=group)
        counts_in = counts_in.view(world, my_n).tolist()
        recv_rows = [sum(c) for c in counts_in]
        x_in = torch.empty(sum(recv_rows), x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(x_in, xp[: offs[self.E]].contiguous(), output_split_sizes=recv_rows,
                               input_split_sizes=send_rows, group=group)
        # run my experts on what arrived: source-rank blocks, each ordered by expert
        y_in = torch.empty_like(x_in)
        base = 0
        for src in range(world):
            for j in range(my_n):
                n = counts_in[src][j]
                if n:
                    e = my_first + j
                    y_in[base:base + n] = swiglu_mlp(x_in[base:base + n], self.W1[e], self.W3[e], self.W2[e])
                base += n
        yp = torch.zeros_like(xp)
        y_back = torch.empty(offs[self.E], x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(y_back, y_in, output_split_sizes=send_rows, input_split_sizes=recv_rows, group=group)
        yp[: offs[self.E]] = y_back
        sh = swiglu_mlp(x, *self.shared) if self.shared is not None else None
        return (combine_fn or combine)(yp, pos, w, sh)
