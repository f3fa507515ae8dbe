"""MoE FFN plumbing: the oracle's own invariants and the expert-parallel exchange on the CPU (gloo, world
size 2, kernels stood in for by the oracle), every kernel and the whole layer against the oracle on the GPU.
Index work (expert ids, packing) is compared bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as morc


def _assignments(T, k, E, seed, skew=False):
    g = np.random.default_rng(seed)
    logits = g.standard_normal((T, E)).astype(np.float32)
    if skew:
        logits[:, : max(1, E // 8)] += 2.0           # a few hot experts, so that capacity bites
    return logits


def test_oracle_packing_invariants():
    for T, k, E, cap, skew in ((37, 2, 8, 6, True), (64, 4, 16, 1000, False), (5, 1, 4, 0, False), (0, 2, 4, 3, False)):
        idx, w = morc.route_topk(_assignments(T, k, E, 3, skew), k) if T else (np.zeros((0, k), np.int32), np.zeros((0, k), np.float32))
        pos, perm, offs = morc.pack(idx, E, cap)
        assert offs[0] == 0 and (np.diff(offs) >= 0).all() and (np.diff(offs) <= cap).all()
        kept = pos >= 0
        assert sorted(pos[kept].tolist()) == list(range(int(offs[-1])))          # a bijection onto the packed rows
        for t in range(T):
            for j in range(k):
                if kept[t, j]:
                    e = idx[t, j]
                    assert offs[e] <= pos[t, j] < offs[e + 1] and perm[pos[t, j]] == t
        if T:
            assert np.allclose(w.sum(axis=1), 1, atol=1e-6) and (np.diff(w, axis=1) <= 1e-7).all()
            wn = morc.renormalise(w, pos)
            s = wn.sum(axis=1)
            assert np.all((np.abs(s - 1) < 1e-6) | (~kept.any(axis=1) & (s == 0)))


def test_argument_validation_needs_no_gpu():
    from flashdmla import _lib
    L = _lib.lib()
    assert L.fdmla_moe_route_topk(None, None, None, 4, 8, 2, None) == -1
    assert L.fdmla_moe_route_topk(1, 1, 1, 4, 8, 9, None) == -2          # k > E
    assert L.fdmla_moe_pack_workspace_bytes(1000, 8, 256) == ((1000 * 8 + 255) // 256 * 256 + 8000 + 256) * 4
    assert L.fdmla_moe_pack(1, 1, 1, 1, None, 0, 4, 2, 8, 3, 0, None) == -4
    assert L.fdmla_moe_gather(16, 16, 16, 16, 4, 8, 7, 1, None) == -2    # 14-byte rows
    assert L.fdmla_moe_combine(1, 1, 1, None, 1, 4, 2, 8, 5, None) == -1
    from flashdmla.moe import expert_ranges, route_topk
    assert expert_ranges(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
    with pytest.raises(_lib.FlashDMLAError):
        route_topk(torch.zeros(4, 8), 2)                                 # CPU tensor: no fallback


# ------------------------------------------------------------------ expert parallelism on gloo
D, F, E, K, T_LOCAL = 16, 24, 6, 2, 11


def _layer_weights(seed=5):
    g = np.random.default_rng(seed)
    n = lambda *s: (g.standard_normal(s) / np.sqrt(s[-2])).astype(np.float32)
    return dict(Wg=n(D, E), W1=n(E, D, F), W3=n(E, D, F), W2=n(E, F, D), shared=(n(D, F), n(D, F), n(F, D)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "ds-flashdmla-moe_b200")]
    from flashdmla.moe import MoEFFN
    try:
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        W = _layer_weights()
        x = np.random.default_rng(100 + rank).standard_normal((T_LOCAL + rank, D)).astype(np.float32)
        layer = MoEFFN.__new__(MoEFFN)                       # weights from numpy, fp32, on the CPU
        layer.d, layer.f, layer.E, layer.k, layer.cf = D, F, E, K, 1.0
        layer.Wg, layer.W1, layer.W3, layer.W2 = (torch.from_numpy(W[n]) for n in ("Wg", "W1", "W3", "W2"))
        layer.shared = tuple(torch.from_numpy(s) for s in W["shared"])
        cap = 5

        def route_fn(xt, capacity):
            idx, w = morc.route_topk(xt.numpy() @ W["Wg"], K)
            pos, perm, offs = morc.pack(idx, E, capacity)
            return tuple(torch.from_numpy(a) for a in (idx, w, pos, perm, offs))

        def gather_fn(xt, perm, offs):
            return xt[perm.long()]

        def combine_fn(yp, pos, w, sh):
            wn = torch.from_numpy(morc.renormalise(w.numpy(), pos.numpy()))
            out = torch.zeros(pos.shape[0], yp.shape[1])
            for t in range(pos.shape[0]):
                for j in range(pos.shape[1]):
                    if pos[t, j] >= 0:
                        out[t] += wn[t, j] * yp[pos[t, j]]
            return out + sh
        out = layer.forward_ep(torch.from_numpy(x), capacity=cap, route_fn=route_fn, gather_fn=gather_fn, combine_fn=combine_fn)
        want, _ = morc.moe_ffn(x, W["Wg"], W["W1"], W["W3"], W["W2"], K, cap, W["shared"])
        err = float(np.abs(out.numpy() - want).max())

        # the padded, read-back-free exchange: same kept assignments, rows at expert * capacity + rank
        def route_padded(xt, capacity):
            idx, w = morc.route_topk(xt.numpy() @ W["Wg"], K)
            pos, perm, offs = morc.pack(idx, E, capacity)
            ppos = np.where(pos >= 0, pos - offs[idx] + idx * capacity, -1).astype(np.int32)
            return torch.from_numpy(idx), torch.from_numpy(w), torch.from_numpy(ppos)

        def scatter_fn(xt, pos, n_rows):
            xp = torch.zeros(n_rows, xt.shape[1])
            for t in range(pos.shape[0]):
                for j in range(pos.shape[1]):
                    if pos[t, j] >= 0:
                        xp[pos[t, j]] = xt[t]
            return xp
        out2 = layer.forward_ep_batched(torch.from_numpy(x), cap, route_fn=route_padded, scatter_fn=scatter_fn,
                                        combine_fn=combine_fn)
        err = max(err, float(np.abs(out2.numpy() - want).max()))
        q.put((rank, "ok", err))
    except Exception as e:
        q.put((rank, "error", type(e).__name__ + ": " + str(e)[:300]))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def test_expert_parallel_exchange_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert all(o[1] == "ok" for o in out), out
    assert max(o[2] for o in out) < 1e-4


# ------------------------------------------------------------------ kernels on the GPU
@pytest.mark.gpu
@pytest.mark.parametrize("T,k,E,cap,skew", [(1000, 8, 256, 40, True), (37, 2, 8, 6, True), (4096, 6, 64, 10 ** 6, False),
                                            (5, 1, 4, 0, False), (300, 3, 7, 100, True), (1, 4, 4, 1, False)])
def test_gate_and_packing_match_the_oracle_bit_for_bit(cuda, T, k, E, cap, skew):
    from flashdmla import moe
    logits = _assignments(T, k, E, 11, skew)
    idx, w = moe.route_topk(torch.from_numpy(logits).to(cuda), k)
    idx_r, w_r = morc.route_topk(logits, k)
    assert np.array_equal(idx.cpu().numpy(), idx_r)
    assert np.allclose(w.cpu().numpy(), w_r, rtol=2e-5, atol=1e-7)
    pos, perm, offs = moe.pack(idx, E, cap)
    pos_r, perm_r, offs_r = morc.pack(idx_r, E, cap)
    assert np.array_equal(offs.cpu().numpy(), offs_r)
    assert np.array_equal(pos.cpu().numpy(), pos_r)
    assert np.array_equal(perm.cpu().numpy()[: offs_r[-1]], perm_r)
    # gather is a row copy: bit exact
    x = torch.randn(T, 64, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    xp = moe.gather(x.to(cuda), perm, offs).cpu()
    assert torch.equal(xp[: offs_r[-1]], x[torch.from_numpy(perm_r).long()])
    xs = moe.scatter(x.to(cuda), pos, perm.shape[0]).cpu()          # the same rows, written from the token side
    assert torch.equal(xs[: offs_r[-1]], xp[: offs_r[-1]])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_combine_renormalises_kept_weights_and_adds_the_shared_expert(cuda, dtype):
    from flashdmla import moe
    T, k, E, d, cap = 200, 4, 8, 96, 60
    logits = _assignments(T, k, E, 4, True)
    idx, w = morc.route_topk(logits, k)
    pos, perm, offs = morc.pack(idx, E, cap)
    assert (pos < 0).any() and (pos < 0).all(axis=1).sum() >= 0
    g = torch.Generator().manual_seed(8)
    y = torch.randn(int(offs[-1]), d, generator=g).to(dtype)
    sh = torch.randn(T, d, generator=g).to(dtype)
    out = moe.combine(y.to(cuda), torch.from_numpy(pos).to(cuda), torch.from_numpy(w).to(cuda), sh.to(cuda)).float().cpu().numpy()
    wn = morc.renormalise(w, pos)
    want = sh.float().numpy().copy()
    for t in range(T):
        for j in range(k):
            if pos[t, j] >= 0:
                want[t] += wn[t, j] * y[pos[t, j]].float().numpy()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert np.abs(out - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.gpu
def test_whole_layer_matches_the_oracle(cuda):
    from flashdmla.moe import MoEFFN
    layer = MoEFFN(d_model=128, d_ff=256, n_experts=16, top_k=4, capacity_factor=1.0, device=cuda, seed=3)
    x = (torch.randn(300, 128, generator=torch.Generator().manual_seed(9)) * 0.5).to(torch.bfloat16)
    out = layer.forward(x.to(cuda)).float().cpu().numpy()
    f = lambda t: t.float().cpu().numpy()
    # the oracle routes on the logits the GPU computed (fp32 GEMM), so that a near-tie cannot flip an expert
    logits = f(x.to(cuda).float() @ layer.Wg)
    idx, w = morc.route_topk(logits, layer.k)
    cap = layer.capacity(300)
    pos, perm, offs = morc.pack(idx, layer.E, cap)
    assert (pos < 0).any()                                   # capacity factor 1.0 drops something
    wn = morc.renormalise(w, pos)
    xf = f(x)
    want = morc.swiglu_mlp(xf, *(f(s) for s in layer.shared))
    for t in range(300):
        for j in range(layer.k):
            if pos[t, j] >= 0:
                e = idx[t, j]
                want[t] += wn[t, j] * morc.swiglu_mlp(xf[t:t + 1], f(layer.W1[e]), f(layer.W3[e]), f(layer.W2[e]))[0]
    err = np.linalg.norm(out - want) / np.linalg.norm(want)
    assert err <= 1.5e-2, err                                # bf16 GEMMs and a bf16 result against fp32
    # padded packing + batched GEMMs: the same routing, the same kept assignments
    out_b = layer.forward_batched(x.to(cuda)).float().cpu().numpy()
    err_b = np.linalg.norm(out_b - want) / np.linalg.norm(want)
    assert err_b <= 1.5e-2, err_b
    from flashdmla import moe
    idx_g, _ = moe.route_topk(x.to(cuda).float() @ layer.Wg, layer.k)
    pos_p, perm_p, offs_p = moe.pack(idx_g, layer.E, cap, padded=True)
    assert offs_p.tolist() == [e * cap for e in range(layer.E + 1)]
    pp = pos_p.cpu().numpy()
    assert np.array_equal(pp >= 0, pos >= 0)
    assert np.array_equal(np.where(pp >= 0, pp - idx * cap, -1), np.where(pos >= 0, pos - offs[idx], -1))   # same rank inside the expert
    # rows of the padded layout that hold no assignment are marked -1 and gathered as zeros
    used = np.zeros(layer.E * cap, dtype=bool)
    used[pp[pp >= 0]] = True
    perm_np = perm_p.cpu().numpy()
    assert (perm_np[~used] == -1).all() and (perm_np[used] >= 0).all()
    xg = moe.gather(x.to(cuda), perm_p, offs_p).float().cpu().numpy()
    assert (xg[~used] == 0).all()
    assert np.array_equal(xg[used], f(x)[perm_np[used]])


@pytest.mark.gpu
def test_batched_layer_replays_as_a_cuda_graph(cuda):
    """forward_batched reads nothing back to the host, so a whole MoE layer captures as one CUDA graph."""
    from flashdmla.moe import MoEFFN
    layer = MoEFFN(d_model=128, d_ff=128, n_experts=8, top_k=2, capacity_factor=1.5, device=cuda, seed=6)
    g = torch.Generator().manual_seed(10)
    x_in = torch.zeros(96, 128, dtype=torch.bfloat16, device=cuda)
    side = torch.cuda.Stream(device=cuda)
    with torch.cuda.stream(side):
        layer.forward_batched(x_in)                      # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.forward_batched(x_in)
    for _ in range(2):
        x = (torch.randn(96, 128, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
        x_in.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        want = layer.forward_batched(x)
        assert torch.equal(out, want)
    # the ragged layer (grouped GEMM over device-side row ranges) reads nothing back either
    with torch.cuda.stream(side):
        layer.forward(x_in)
    torch.cuda.synchronize()
    graph2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph2):
        out2 = layer.forward(x_in)
    x = (torch.randn(96, 128, generator=g) * 0.5).to(torch.bfloat16).to(cuda)
    x_in.copy_(x)
    graph2.replay()
    torch.cuda.synchronize()
    assert torch.equal(out2, layer.forward(x))
    assert (out2.float() - layer.forward_batched(x).float()).abs().max() <= 2e-2 * out2.float().abs().max()
