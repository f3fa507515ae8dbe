"""CPU restatement of the MoE FFN the reference advertises (test infrastructure only).

PARITY UNPINNED: the reference ships no MoE source (csrc/moe/*.cu, tests/test_moe.py are listed in
its README.md:37-60 but absent), so there is nothing to run or to take golden vectors from.  This
file restates the "unfused reference path" of README.md:17-20 - Top-K gate -> per-expert packing
(bucket + exclusive scan) -> expert MLP -> combine & shared-expert add, "gate weight
renormalization under capacity; overflow tokens are masked" - with every choice the README leaves
open written down here:

  * gate: p = softmax(logits) in fp32 over all experts; the k largest logits win (ties: lower expert
    index; listed in descending order); w = p[selected] / sum(p[selected]);
  * packing: assignments are numbered a = token * k + j; within an expert they keep that order;
    an expert keeps its first `capacity` assignments, the rest are dropped (pos = -1);
    offsets = exclusive scan of the kept counts; packed row offsets[e] + rank holds the token;
  * renormalisation: a token's kept weights are rescaled to sum to 1 (all dropped: zero output
    from the routed experts);
  * expert MLP: (silu(x W1[e]) * (x W3[e])) W2[e]; the shared expert is the same MLP applied to
    every token and added unweighted.

Only tests, the smoke check and the CPU baseline may import this module.
"""
from __future__ import annotations

import numpy as np


def route_topk(logits: np.ndarray, k: int):
    x = logits.astype(np.float32)
    p = np.exp(x - x.max(axis=1, keepdims=True))
    p = p / p.sum(axis=1, keepdims=True, dtype=np.float32)
    # stable: descending logit (the same order as descending p, without p's rounding ties), ties by lower index
    order = np.argsort(-x, axis=1, kind="stable")[:, :k]
    sel = np.take_along_axis(p, order, axis=1)
    w = sel / sel.sum(axis=1, keepdims=True, dtype=np.float32)
    return order.astype(np.int32), w.astype(np.float32)


def pack(idx: np.ndarray, n_experts: int, capacity: int):
    T, k = idx.shape
    flat = idx.reshape(-1)
    rank = np.zeros(T * k, np.int64)
    seen = np.zeros(n_experts, np.int64)
    for a, e in enumerate(flat):
        rank[a] = seen[e]
        seen[e] += 1
    counts = np.minimum(seen, capacity)
    offsets = np.zeros(n_experts + 1, np.int32)
    offsets[1:] = np.cumsum(counts)
    kept = rank < capacity
    pos = np.where(kept, offsets[flat] + rank, -1).astype(np.int32)
    perm = np.full(int(offsets[-1]), -1, np.int32)
    perm[pos[kept]] = (np.arange(T * k) // k)[kept]
    return pos.reshape(T, k), perm, offsets


def renormalise(w: np.ndarray, pos: np.ndarray):
    kept = (pos >= 0).astype(np.float32)
    s = (w * kept).sum(axis=1, keepdims=True, dtype=np.float32)
    return np.where(s > 0, w * kept / np.where(s > 0, s, 1), 0).astype(np.float32)


def swiglu_mlp(x, W1, W3, W2):
    a = x @ W1
    return ((a / (1 + np.exp(-a))) * (x @ W3)) @ W2


def moe_ffn(x, Wg, W1, W3, W2, k, capacity, shared=None):
    """x [T,d]; Wg [d,E]; W1, W3 [E,d,f]; W2 [E,f,d]; shared = (W1s, W3s, W2s) or None.  All fp32."""
    x = x.astype(np.float32)
    E = Wg.shape[1]
    idx, w = route_topk(x @ Wg.astype(np.float32), k)
    pos, perm, offsets = pack(idx, E, capacity)
    wn = renormalise(w, pos)
    y = np.zeros((len(perm), x.shape[1]), np.float32)
    for e in range(E):
        lo, hi = offsets[e], offsets[e + 1]
        if hi > lo:
            y[lo:hi] = swiglu_mlp(x[perm[lo:hi]], W1[e].astype(np.float32), W3[e].astype(np.float32), W2[e].astype(np.float32))
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(k):
            if pos[t, j] >= 0:
                out[t] += wn[t, j] * y[pos[t, j]]
    if shared is not None:
        out += swiglu_mlp(x, *(s.astype(np.float32) for s in shared))
    return out, dict(idx=idx, w=w, pos=pos, perm=perm, offsets=offsets, wn=wn)
