"""Where the time of one paged-decode launch goes, pair by pair (development aid).

    python ds-flashdmla-moe_b200/build.py --timeline [--ablate BITS]
    python ds-flashdmla-moe_b200/timeline_report.py [--batch 128] [--skv 4096] [--splits 1] [--ablate 0,1,2,4,3]
    python ds-flashdmla-moe_b200/timeline_report.py --prefill 1,16,8192

Runs the DeepSeek-V3-shape decode (H=128, 576-wide rows, page 64, seeded synthetic cache) on the library built with
-DFDMLA_TIMELINE, which stamps what every CTA pair of the 2-CTA forward kernel does (global timer) and adds up the SM
cycles each role spends in each kind of wait, and prints medians over the pairs of the last of three launches.  With
--ablate the same launch is repeated on the libraries that leave out one pipeline stage (1: K/V copies, 2: softmax
arithmetic, 4: MMAs; results of those runs are garbage, only their timing means something).  Needs a GPU.
"""
from __future__ import annotations

import argparse
import math
import os
import struct
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

TL_CLUSTERS, TL_TILES, TW_KINDS = 128, 40, 8
WAIT_NAMES = {
    0: ("producer", ["Q free", "K slots free", "V slots free", "tail copies", "issue K", "issue V", "item set-up", "whole role"]),
    1: ("MMA issuer", ["Q landed", "S buffer free", "K slots landed", "P written", "V slots landed", "tail zeroed", "O read out", "whole role"]),
    2: ("softmax thread 0", ["scores ready", "P V done (rescale)", "P quarter read", "P V done (end)", "epilogue", "ticket + merge", "", "whole role"]),
}


def lib_path(ablate: int) -> str:
    return os.path.join(HERE, "flashdmla", "libflashdmla_timeline" + (f"_abl{ablate}" if ablate else "") + ".so")


def parse(path):
    import numpy as np
    data = open(path, "rb").read()
    recs, off = [], 0
    while off < len(data):
        ncl, dec, nslots, nitems = struct.unpack_from("4i", data, off); off += 16
        take = lambda dt, n: np.frombuffer(data, dtype=dt, count=n, offset=off).copy()
        st = take(np.uint64, TL_CLUSTERS * nslots).reshape(TL_CLUSTERS, nslots); off += st.nbytes
        ti = take(np.int32, TL_CLUSTERS * nitems).reshape(TL_CLUSTERS, nitems); off += ti.nbytes
        wa = take(np.int64, TL_CLUSTERS * 2 * 3 * TW_KINDS).reshape(TL_CLUSTERS, 2, 3, TW_KINDS); off += wa.nbytes
        tt = take(np.uint64, TL_CLUSTERS * TL_TILES).reshape(TL_CLUSTERS, TL_TILES); off += tt.nbytes
        tc = take(np.int64, TL_CLUSTERS * TL_TILES).reshape(TL_CLUSTERS, TL_TILES); off += tc.nbytes
        recs.append((ncl, dec, st, ti, wa, tt, tc))
    return recs


def summarise(rec, label):
    import numpy as np
    ncl, dec, st, ti, wa, tt, tc = rec
    st, wa = st[:ncl].astype(np.float64), wa[:ncl].astype(np.float64)
    tt, tc = tt[:ncl].astype(np.float64), tc[:ncl].astype(np.float64)
    t0 = st[:, 0].min()
    us = lambda a: (a - t0) / 1e3
    print(f"== {label}: {ncl} CTA pairs; times in us after the first pair entered the kernel")
    print(f"   set-up done (median) {np.median(us(st[:, 1])):.1f}; scores of the first tile ready: median {np.median(us(st[:, 2])):.1f}, "
          f"last pair {us(st[:, 2]).max():.1f}")
    for i in range(ti.shape[1]):
        have = st[:, 4 + 3 * i] > 0
        if not have.any():
            break
        nt = ti[:ncl, i][have]
        a, b, c = us(st[have, 2 + 3 * i]), us(st[have, 3 + 3 * i]), us(st[have, 4 + 3 * i])
        print(f"   item {i}: {int(have.sum())} pairs, {np.median(nt):.0f} tiles (median); first scores {np.median(a):.1f}, last P V "
              f"{np.median(b):.1f}, result written {np.median(c):.1f} (epilogue {np.median(c - b):.2f})")
    print(f"   roles finished: first pair {us(st[:, 30]).min():.1f}, median {np.median(us(st[:, 30])):.1f}, last {us(st[:, 30]).max():.1f}; "
          f"last exit {us(st[:, 31]).max():.1f}")
    with np.errstate(all="ignore"):
        d = np.diff(tt, axis=1) / 1e3
        d[(tt[:, 1:] == 0) | (tt[:, :-1] == 0)] = np.nan
        ghz = np.diff(tc, axis=1) / (d * 1e3)
        cols = [j for j in range(d.shape[1]) if np.isfinite(d[:, j]).any()]
        print("   us between the scores of consecutive tiles of a pair (median over pairs): " + " ".join(f"{np.nanmedian(d[:, j]):.2f}" for j in cols))
        print("   SM clock over the same spans, GHz: " + " ".join(f"{np.nanmedian(ghz[:, j]):.2f}" for j in cols))
    for role, (rname, names) in WAIT_NAMES.items():
        for rk in (0, 1):
            w = wa[:, rk, role, :]
            if w[:, 7].max() == 0:
                continue
            s = ", ".join(f"{names[k]} {np.median(w[:, k]) / 1e3:.1f}" for k in range(TW_KINDS) if names[k])
            print(f"   {rname}, CTA {rk}, thousands of SM cycles (median): {s}")


def run_prefill(args):
    import torch
    import flashdmla
    dev = torch.device("cuda:0")
    Bp, Hp, Sp = (int(x) for x in args.prefill.split(","))
    g = torch.Generator(device=dev).manual_seed(77)
    K = (torch.randn(Bp, Sp, 576, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    Q = (torch.randn(Bp, Hp, Sp, 576, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    for _ in range(3):
        flashdmla.flash_dmla_cache_latent(Q, K, 512, 1 / math.sqrt(192), True)
    torch.cuda.synchronize()
    summarise(parse(os.environ["FDMLA_TIMELINE_FILE"])[-1], f"causal prefill B={Bp} H={Hp} S={Sp} ablate={args.one}")
    print(f"   device error flag {flashdmla.device_error_flag()}")


def run_one(args):
    if args.prefill:
        return run_prefill(args)
    import torch
    import flashdmla
    dev = torch.device("cuda:0")
    B, H, S, D, P = args.batch, 128, args.skv, 576, 64
    g = torch.Generator(device=dev).manual_seed(1000)
    n_pages = B * S // P
    pool = (torch.randn(n_pages, P, D, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    Q = (torch.randn(B, H, D, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1000)).to(torch.int32).view(B, S // P).to(dev)
    seqlens = torch.full((B,), S, dtype=torch.int32, device=dev)
    ws = flashdmla.DecodeWorkspace()
    for _ in range(3):
        flashdmla.flash_dmla_paged_decode(Q, pool, table, seqlens, 512, 1 / math.sqrt(192), num_splits=args.splits, workspace=ws, max_seqlen=S)
    torch.cuda.synchronize()
    summarise(parse(os.environ["FDMLA_TIMELINE_FILE"])[-1], f"B={B} Skv={S} slabs={args.splits} ablate={args.one}")
    print(f"   device error flag {flashdmla.device_error_flag()}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--skv", type=int, default=4096)
    ap.add_argument("--splits", type=int, default=1)
    ap.add_argument("--ablate", default="0", help="comma-separated list of ablation builds to run (0 = none)")
    ap.add_argument("--prefill", default="", help="B,H,S: time a causal prefill of that shape instead of the decode")
    ap.add_argument("--one", type=int, default=-1, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.one >= 0:
        return run_one(args)
    for abl in [int(x) for x in args.ablate.split(",")]:
        lib = lib_path(abl)
        if not os.path.exists(lib):
            raise SystemExit(f"{lib} is missing: python {os.path.join(HERE, 'build.py')} --timeline" + (f" --ablate {abl}" if abl else ""))
        with tempfile.TemporaryDirectory() as tmp:
            env = dict(os.environ, FLASHDMLA_LIB=lib, FDMLA_TIMELINE_FILE=os.path.join(tmp, "timeline.bin"))
            subprocess.run([sys.executable, os.path.abspath(__file__), "--batch", str(args.batch), "--skv", str(args.skv),
                            "--splits", str(args.splits), "--one", str(abl)] + (["--prefill", args.prefill] if args.prefill else []),
                           env=env, check=True)


if __name__ == "__main__":
    main()
