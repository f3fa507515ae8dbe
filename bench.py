#!/usr/bin/env python
"""Benchmark of the Flash-DMLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (one "step"): DeepSeek-V3-shape paged MLA decode, bf16,
B=128 sequences per GPU, H=128, Skv=4096, 576-wide latent rows (V = first 512),
page size 64, page table = seeded random permutation of the pool, scale
1/sqrt(192), entries 0.1*N(0,1).  Sequences are sharded over GPUs with no
collective (weak scaling: every GPU decodes its own 128 sequences).  The line
also carries the causal-prefill figure (B=4, H=128, S=8192, heads sharded) and, on
more than one GPU, the long-context decode whose KV sequence is split over the
GPUs (B=8, Skv in [16384, 131072]: the one exchange step of the path, an NCCL
all-gather of the partial results) and a context-parallel prefill.

`--impl reference` times the CPU oracle (the restatement of the reference's
naive attention; the reference ships no CPU code and no DMLA kernels) on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "ds-flashdmla-moe_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

# ---- workload constants (BASELINE configs 2 and 3) -------------------------------------------
B, H, SKV, D_QK, D_V, PAGE = 128, 128, 4096, 576, 512, 64
SCALE = 1.0 / math.sqrt(192.0)
DECODE_BYTES = (B * SKV * D_QK * 2          # latent rows read once
                + B * H * D_QK * 2          # Q
                + B * H * D_V * 2           # O
                + 2 * B * H * 4             # m, l
                + B * (SKV // PAGE) * 4)    # page table            = 639 795 200
DECODE_FLOP = 2 * B * H * SKV * (D_QK + D_V)
# DRAM bytes per sequence of one decode launch, from the ncu capture of the B=32 case
# (profiles/fwd_tc2_kernel_decode_b32.md: read 157.63 MB + write 3.66 MB for 32 sequences); traffic grows in
# proportion to the sequences, so a launch of B sequences moves B times this.
NCU_DRAM_BYTES_PER_SEQ = (157_634_048 + 3_657_728) / 32
PF_B, PF_H, PF_S = 4, 128, 8192
PREFILL_FLOP_CAUSAL = 2 * PF_B * PF_H * (PF_S * (PF_S + 1) // 2) * (D_QK + D_V)


def set_batch(b: int) -> None:
    """Reduced decode case (fewer sequences, same per-sequence shape) for profiler captures."""
    global B, DECODE_BYTES, DECODE_FLOP
    B = int(b)
    DECODE_BYTES = B * SKV * D_QK * 2 + B * H * D_QK * 2 + B * H * D_V * 2 + 2 * B * H * 4 + B * (SKV // PAGE) * 4
    DECODE_FLOP = 2 * B * H * SKV * (D_QK + D_V)


def set_prefill_shape(b: int, h: int, s: int) -> None:
    global PF_B, PF_H, PF_S, PREFILL_FLOP_CAUSAL
    PF_B, PF_H, PF_S = b, h, s
    PREFILL_FLOP_CAUSAL = 2 * PF_B * PF_H * (PF_S * (PF_S + 1) // 2) * (D_QK + D_V)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle sampling while the timed region runs (rank 0)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc, self.idx = None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def make_decode_inputs(dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    n_pages = B * SKV // PAGE
    pool = (torch.randn(n_pages, PAGE, D_QK, generator=g, device=dev, dtype=torch.float32) * 0.1).to(torch.bfloat16)
    Q = (torch.randn(B, H, D_QK, generator=g, device=dev, dtype=torch.float32) * 0.1).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    table = perm.view(B, SKV // PAGE).contiguous().to(dev)
    seqlens = torch.full((B,), SKV, dtype=torch.int32, device=dev)
    return Q, pool, table, seqlens


def time_steps(fn, steps, warmup, world):
    """W untimed + exactly K timed steps between barrier+synchronize; device time, ms total."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def median_launch_ms(fn, launches=200, warmup=10):
    """Median device time of one call of `fn` on the current stream: an event between every two of
    `launches` back-to-back calls (the stream never runs dry: a call is enqueued in far less time than it
    runs), independent of --steps."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(launches + 1)]
    ev[0].record()
    for i in range(launches):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return statistics.median(ev[i].elapsed_time(ev[i + 1]) for i in range(launches))


def pin_to_cores(local: int, world: int):
    """Give every rank its own share of the host cores before it allocates pinned memory (first touch
    then lands near the cores that drive the copies).  Returns the cores, or None if the platform has no
    affinity call."""
    try:
        avail = sorted(os.sched_getaffinity(0))
        per = max(1, len(avail) // max(world, 1))
        mine = avail[local * per:(local + 1) * per] or avail
        os.sched_setaffinity(0, mine)
        return mine
    except (AttributeError, OSError):
        return None


def decode_config(world):
    """The workload both arms are measured on (the GPU arm's tuning choices are reported under `plan`)."""
    return {"workload": "paged_mla_decode", "B_per_gpu": B, "H": H, "Skv": SKV, "d_qk": D_QK, "d_v": D_V,
            "page_size": PAGE, "parallelism": f"batch-sharded x{world}, no collective",
            "l2": f"working set {B * SKV * D_QK * 2 / 1e6:.0f} MB per step exceeds the 126 MB L2 (no flush needed)"}


def cpu_baseline_sample(target_s=12.0):
    """Oracle (port of the reference's naive attention) on the host cores, bounded sample."""
    from flashdmla import synthetic
    from oracle import dmla_oracle as orc
    orc.use_all_cores()
    def run(nseq):
        Q, pool, table, sl = synthetic.paged_decode_inputs(nseq, H, [SKV] * nseq, D_QK, PAGE, seed=3, std=0.1,
                                                          dtype=torch.float32)
        t = time.perf_counter()
        orc.decode_paged(Q, pool, table, sl, D_V, SCALE)
        return time.perf_counter() - t
    t1 = run(2) / 2.0
    nseq = int(max(2, min(B, target_s / max(t1, 1e-3))))
    dt = run(nseq)
    return {"value": nseq / dt, "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{nseq} of {B} sequences x {H} heads x {SKV} keys, fp32 oracle (oracle/dmla_oracle.c), "
                      f"{dt:.2f} s, all host threads"}


def run_reference(args, rank, world):
    """The reference arm: the CPU oracle on the host cores, same metric and config."""
    if rank != 0:
        return
    from flashdmla import synthetic
    from oracle import dmla_oracle as orc
    orc.use_all_cores()
    probe = 2
    Q, pool, table, sl = synthetic.paged_decode_inputs(probe, H, [SKV] * probe, D_QK, PAGE, seed=3, std=0.1,
                                                      dtype=torch.float32)
    t = time.perf_counter()
    orc.decode_paged(Q, pool, table, sl, D_V, SCALE)
    t1 = (time.perf_counter() - t) / probe
    per_step_s = 150.0 / max(1, args.steps + args.warmup)       # whole run within a few minutes
    nseq = int(max(1, min(B, min(2.0, per_step_s) / max(t1, 1e-3))))
    Q, pool, table, sl = synthetic.paged_decode_inputs(nseq, H, [SKV] * nseq, D_QK, PAGE, seed=3, std=0.1,
                                                      dtype=torch.float32)
    for _ in range(args.warmup):
        orc.decode_paged(Q, pool, table, sl, D_V, SCALE)
    t = time.perf_counter()
    for _ in range(args.steps):
        orc.decode_paged(Q, pool, table, sl, D_V, SCALE)
    dt = time.perf_counter() - t
    value = nseq * args.steps / dt
    sample = (f"{nseq} of {B} sequences x {H} heads x {SKV} keys per step, fp32 oracle "
              f"(oracle/dmla_oracle.c, restating the reference's csrc/attention/vanallia_attn.cu), all host threads")
    print(json.dumps({
        "impl": "reference", "metric": "paged_mla_decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": decode_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-prefill", action="store_true", help="skip the secondary causal-prefill measurement")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--splits", type=int, default=0, help="override the decode split count (0 = library choice)")
    ap.add_argument("--prefill-shape", default="",
                    help="B,H,S of the prefill measurement (default 4,128,8192); a reduced shape is used for ncu captures")
    ap.add_argument("--only-prefill", action="store_true", help="run only the prefill measurement (profiling aid)")
    ap.add_argument("--only-moe", action="store_true", help="run only the MoE plumbing measurement (profiling aid)")
    ap.add_argument("--only-long-context", action="store_true",
                    help="run only the long-context decode over N GPUs (KV split, exchange, merge; profiling aid)")
    ap.add_argument("--only-otf", action="store_true", help="run only the on-the-fly forward/backward measurement (profiling aid)")
    ap.add_argument("--otf-shape", default="", help="B,H,S of the on-the-fly measurement (a reduced shape for ncu captures)")
    ap.add_argument("--only-gemm", action="store_true", help="run only the batched-GEMM measurement (profiling aid)")
    ap.add_argument("--gemm-experts", type=int, default=64, help="experts of the GEMM measurement (fewer for ncu captures)")
    ap.add_argument("--kernel-launches", type=int, default=200,
                    help="launches behind the kernel-only median timings (fewer for ncu launch lists)")
    ap.add_argument("--batch", type=int, default=0,
                    help="decode sequences per GPU (default 128); smaller values give the reduced case used for ncu captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.batch:
        set_batch(args.batch)
    if args.prefill_shape:
        set_prefill_shape(*[int(x) for x in args.prefill_shape.split(",")])

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    cores = pin_to_cores(local, world) if world > 1 else sorted(os.sched_getaffinity(0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    import flashdmla
    from flashdmla import _lib

    hbm_peak, tf_burst, tf_sust, peak_src = peaks()
    if args.only_prefill:
        pf = bench_prefill(dev, rank, world, tf_burst, tf_sust)
        if rank == 0:
            print(json.dumps({"prefill": pf, "device_error_flag": flashdmla.device_error_flag()}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only_otf:
        if rank == 0:
            shape = tuple(int(x) for x in args.otf_shape.split(",")) if args.otf_shape else None
            print(json.dumps({"on_the_fly": bench_on_the_fly(dev, tf_burst, only_shape=shape),
                              "device_error_flag": flashdmla.device_error_flag()}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only_gemm:
        if rank == 0:
            print(json.dumps({"gemm": bench_gemm(dev, tf_burst, hbm_peak, E=args.gemm_experts),
                              "device_error_flag": flashdmla.device_error_flag()}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only_long_context:
        if world < 2:
            raise SystemExit("--only-long-context needs --gpus N > 1 under torch.distributed.run")
        lc = bench_long_context(dev, rank, world)
        if rank == 0:
            print(json.dumps({"long_context": lc, "device_error_flag": flashdmla.device_error_flag()}), flush=True)
        dist.destroy_process_group()
        return
    if args.only_moe:
        mp_ = bench_moe_plumbing(dev, hbm_peak)
        if rank == 0:
            print(json.dumps({"moe_plumbing": mp_}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    Q, pool, table, seqlens = make_decode_inputs(dev, seed=1000 + rank)
    splits = args.splits or flashdmla.suggest_splits(B, H, SKV, D_QK, D_V, PAGE)
    ws = flashdmla.DecodeWorkspace()
    L = _lib.lib()
    import ctypes
    qmin, units = ctypes.c_int(0), ctypes.c_int(0)
    mode = L.fdmla_decode_plan(B, H, D_QK, D_V, PAGE, SKV // PAGE, splits, _lib.BF16, ctypes.byref(qmin), ctypes.byref(units))
    mode_name = {0: "equal splits" if splits > 1 else "one work item per sequence", 1: "balanced runs + merge kernel",
                 2: "balanced runs, merged in the attention kernel"}.get(mode, "?")
    # kernels of this library per step: the attention kernel, plus the merge kernel where one runs (the balanced
    # in-kernel schedule also enqueues a 1 KB memset node, which is not a kernel of ours)
    launches_per_step = 1 if (splits == 1 or mode == 2) else 2
    n_units = units.value or 74
    tiles_total = B * (SKV // 256)
    if mode in (1, 2):
        tiles_per_pair_max = max(-(-tiles_total // n_units), qmin.value)
    else:
        tiles_per_pair_max = -(-(B * splits) // n_units) * -(-(SKV // 256) // splits)
    pairs_idle_frac = 1.0 - tiles_total / float(n_units * tiles_per_pair_max)

    def step():
        return flashdmla.flash_dmla_paged_decode(Q, pool, table, seqlens, D_V, SCALE, num_splits=splits,
                                                 workspace=ws, max_seqlen=SKV)

    O, m, l = step()
    torch.cuda.synchronize()
    kernel_family = flashdmla.last_kernel()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total_ms = time_steps(step, args.steps, args.warmup, world)
    ms_per_step = total_ms / args.steps
    value = world * B / (ms_per_step * 1e-3)

    # the dominant kernel alone, through the C ABI, CUDA events on its stream, median of 200 launches: the whole call
    # where the attention kernel also merges (or nothing is to merge), the partial-only call (O = NULL) where a merge
    # kernel would follow
    Op, mp, lp = ws.get(splits, B, H, D_V, dev) if splits > 1 else (None, None, None)
    stream = torch.cuda.current_stream().cuda_stream
    only_partials = launches_per_step == 2
    ptr = lambda t: None if t is None else t.data_ptr()

    def kernel_call(tab):
        def f():
            _lib.check(L.fdmla_decode_paged(Q.data_ptr(), pool.data_ptr(), tab.data_ptr(), seqlens.data_ptr(),
                                            None if only_partials else O.data_ptr(), m.data_ptr(), l.data_ptr(), ptr(Op),
                                            ptr(mp), ptr(lp), B, H, D_QK, D_V, PAGE, SKV // PAGE, pool.shape[0], splits, 0,
                                            -1, SCALE, _lib.BF16, stream), "fdmla_decode_paged")
        return f
    k_ms = median_launch_ms(kernel_call(table), launches=args.kernel_launches)
    # control: the same launch with every sequence's page table aliased onto the pages of 8 sequences
    # (38 MB of distinct cache rows, resident in L2), i.e. the kernel with HBM taken out of the picture
    alias_table = table[:8].repeat((B + 7) // 8, 1)[:B].contiguous()
    k_l2_ms = median_launch_ms(kernel_call(alias_table), launches=args.kernel_launches)
    achieved = DECODE_BYTES / (k_ms * 1e-3) / 1e9

    e2e = bench_e2e(dev, world, Q, pool, table, seqlens, splits, ws, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    prefill = on_the_fly = moe_plumbing = long_context = context_prefill = gemm_line = cl_bwd = None
    if not args.no_prefill:
        prefill = bench_prefill(dev, rank, world, tf_burst, tf_sust)
        if world > 1:
            del pool
            torch.cuda.empty_cache()
            long_context = bench_long_context(dev, rank, world)
            context_prefill = bench_context_prefill(dev, rank, world)
        if rank == 0:
            on_the_fly = bench_on_the_fly(dev, tf_burst)
            moe_plumbing = bench_moe_plumbing(dev, hbm_peak)
            gemm_line = bench_gemm(dev, tf_burst, hbm_peak)
            cl_bwd = bench_cache_latent_bwd(dev, tf_burst)

    err = flashdmla.device_error_flag()
    if rank == 0:
        cpu = None if (args.no_cpu or world > 1) else cpu_baseline_sample()
        line = {
            "metric": "paged_mla_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": decode_config(world),
            "plan": {"num_splits": splits, "schedule": mode_name, "kernel_family": kernel_family,
                     "host_cores_of_rank0": len(cores) if cores else None},
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps * world,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                         "frac": achieved / hbm_peak, "traffic": NCU_DRAM_BYTES_PER_SEQ * B,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the B=32 capture, "
                                           "scaled by the number of sequences",
                         "peak_source": peak_src,
                         "kernel": "fwd_tc2_kernel (2-CTA tcgen05 split-KV decode)", "kernel_ms": k_ms,
                         "kernel_ms_method": f"median of {args.kernel_launches} back-to-back C-ABI calls, one CUDA event between calls",
                         "algorithmic_bytes": DECODE_BYTES, "tensor_tflops": DECODE_FLOP / (k_ms * 1e-3) / 1e12,
                         "kernel_ms_l2_resident_control": k_l2_ms,
                         "tiles_per_pair_max": tiles_per_pair_max, "pairs": n_units, "pairs_idle_frac": pairs_idle_frac,
                         "frac_of_8TBs_spec": achieved / 8000.0},
            "decode_hbm_gbs_per_gpu": DECODE_BYTES / (ms_per_step * 1e-3) / 1e9,
            "prefill": prefill,
            "long_context": long_context,
            "context_parallel_prefill": context_prefill,
            "on_the_fly": on_the_fly,
            "moe_plumbing": moe_plumbing,
            "gemm": gemm_line,
            "cache_latent_bwd": cl_bwd,
            "device_error_flag": err,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def bench_e2e(dev, world, Q, pool, table, seqlens, splits, ws, steps):
    """End to end through the public operator with HOST buffers: every step copies its inputs (Q, page table,
    lengths) from pinned host memory and its results (O, m, l) back.  One staging buffer per direction - the three
    tensors packed at 256-byte offsets - so that a step is ONE copy in and ONE copy out; the device side works on
    views of the staging buffers.  The copies run on their own streams with three sets of buffers, so the copy-in of
    step i+1 and the copy-out of step i-1 overlap the kernel of step i.  The same schedule without the kernel gives
    the ceiling the host link sets (`copy_only_ms`)."""
    import flashdmla
    al = lambda n: (n + 255) & ~255
    nQ, ntab, nlen = Q.numel() * 2, table.numel() * 4, seqlens.numel() * 4
    o_tab, o_len, n_in = al(nQ), al(nQ) + al(ntab), al(nQ) + al(ntab) + al(nlen)
    nO, nm = B * H * D_V * 2, B * H * 4
    o_m, o_l, n_out = al(nO), al(nO) + al(nm), al(nO) + 2 * al(nm)
    NB = 3
    h_in = torch.empty(n_in, dtype=torch.uint8).pin_memory()
    h_in[:nQ].copy_(Q.cpu().view(torch.uint8).reshape(-1))
    h_in[o_tab:o_tab + ntab].copy_(table.cpu().view(torch.uint8).reshape(-1))
    h_in[o_len:o_len + nlen].copy_(seqlens.cpu().view(torch.uint8).reshape(-1))
    h_out = [torch.empty(n_out, dtype=torch.uint8).pin_memory() for _ in range(NB)]
    d_in = [torch.empty(n_in, dtype=torch.uint8, device=dev) for _ in range(NB)]
    d_out = [torch.empty(n_out, dtype=torch.uint8, device=dev) for _ in range(NB)]
    vQ = [d[:nQ].view(torch.bfloat16).view(B, H, D_QK) for d in d_in]
    vtab = [d[o_tab:o_tab + ntab].view(torch.int32).view(B, -1) for d in d_in]
    vlen = [d[o_len:o_len + nlen].view(torch.int32) for d in d_in]
    vout = [(d[:nO].view(torch.bfloat16).view(B, H, D_V), d[o_m:o_m + nm].view(torch.float32).view(B, H),
             d[o_l:o_l + nm].view(torch.float32).view(B, H)) for d in d_out]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev_in = [torch.cuda.Event() for _ in range(NB)]
    ev_done = [torch.cuda.Event() for _ in range(NB)]
    ev_out = [torch.cuda.Event() for _ in range(NB)]
    counter = [0]

    def e2e_step(with_kernel):
        i = counter[0]
        counter[0] += 1
        b = i % NB
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(s_in):
            if i >= NB:
                s_in.wait_event(ev_done[b])              # the kernel that read this input set is finished
            d_in[b].copy_(h_in, non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        if i >= NB:
            cur.wait_event(ev_out[b])                    # the copy that read this output set is finished
        if with_kernel:
            flashdmla.flash_dmla_paged_decode(vQ[b], pool, vtab[b], vlen[b], D_V, SCALE, num_splits=splits,
                                              workspace=ws, max_seqlen=SKV, out=vout[b])
        ev_done[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b])
            h_out[b].copy_(d_out[b], non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_time(n, warmup, with_kernel):
        counter[0] = 0
        for _ in range(warmup):
            e2e_step(with_kernel)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        cur = torch.cuda.current_stream()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        s_in.wait_event(e0)
        s_out.wait_event(e0)
        for _ in range(n):
            e2e_step(with_kernel)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        e1.record(cur)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / n
    e2e_ms = e2e_time(steps, 4, True)
    got = vout[(counter[0] - 1) % NB]
    torch.cuda.synchronize()
    O_ref, m_ref, l_ref = flashdmla.flash_dmla_paged_decode(Q, pool, table, seqlens, D_V, SCALE, num_splits=splits, workspace=ws)
    same = bool(torch.equal(got[0], O_ref) and torch.equal(got[1], m_ref))
    copy_ms = e2e_time(steps, 4, False)
    return {"value": world * B / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": n_in,
            "d2h_bytes_per_step": n_out, "ms_per_step": e2e_ms, "copy_only_ms": copy_ms,
            "frac_of_copy_ceiling": copy_ms / e2e_ms,
            "h2d_gbs_per_gpu": n_in / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_gpu": n_out / (e2e_ms * 1e-3) / 1e9,
            "host_link_gbs_all_gpus": world * (n_in + n_out) / (e2e_ms * 1e-3) / 1e9,
            "result_matches_resident_run": same,
            "note": "paged KV pool stays resident in HBM (it is the cache); every step moves Q, page table, seqlens in "
                    "and O, m, l out, one copy per direction from/to one pinned staging buffer, on their own streams, "
                    "three sets of buffers; copy_only_ms is the same schedule without the kernel"}


def _median_over_ranks(ms, world):
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def bench_long_context(dev, rank, world, steps=50, warmup=10):
    """Long-context decode (B=8, H=128, Skv ~ U{16384..131072}, page 64): the KV sequence of every request is cut
    into `world` contiguous page-aligned slices (remainder to the first ranks, the rule of the reference's
    csrc/attention/fa2_fwd_mpi.cu:47-53), every rank attends its slice, the partial (O, m, l) travel in one
    NCCL all-gather and every rank merges them.  Timed per phase with CUDA events (median over the steps, max over
    ranks) and as a whole like the headline (K steps between barriers, max over ranks).  Then the same step with the
    exchange and the merge as one kernel over peer memory (flashdmla.exchange), which must return the same bits; the
    faster of the two graph replays is the reported step."""
    import flashdmla
    from flashdmla import parallel
    B8 = 8
    lens = torch.randint(16384, 131073, (B8,), generator=torch.Generator().manual_seed(4100)).tolist()
    pages = [(x + PAGE - 1) // PAGE for x in lens]
    n_pages = sum(pages)
    g = torch.Generator(device=dev).manual_seed(4101)          # the same cache on every rank
    pool = torch.empty(n_pages, PAGE, D_QK, dtype=torch.bfloat16, device=dev)
    for p0 in range(0, n_pages, 1024):
        p1 = min(n_pages, p0 + 1024)
        pool[p0:p1] = (torch.randn(p1 - p0, PAGE, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    Q = (torch.randn(B8, H, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(4102)).to(torch.int32)
    table = torch.zeros(B8, max(pages), dtype=torch.int32)
    cur = 0
    for b in range(B8):
        table[b, :pages[b]] = perm[cur:cur + pages[b]]
        cur += pages[b]
    seqlens = torch.tensor(lens, dtype=torch.int32, device=dev)
    table_d = table.to(dev)
    # the unsplit problem on one GPU: reference result and 1-GPU time
    ws1 = flashdmla.DecodeWorkspace()
    one = lambda: flashdmla.flash_dmla_paged_decode(Q, pool, table_d, seqlens, D_V, SCALE, workspace=ws1, max_seqlen=max(lens))
    O1, m1, l1 = one()
    one_ms = _median_over_ranks(median_launch_ms(one, launches=steps, warmup=warmup), world)
    # this rank's slice: its own pool holding only its pages
    parts = parallel.split_sequence_pages(lens, PAGE, world, rank)
    ids = torch.cat([table[b, first:first + n] for b, (first, n, _) in enumerate(parts)]).long()
    lpool = pool[ids.to(dev)].contiguous()
    ltab = torch.zeros(B8, max(max(n for _, n, _ in parts), 1), dtype=torch.int32)
    llen = torch.zeros(B8, dtype=torch.int32)
    cur = 0
    for b, (first, n, ntok) in enumerate(parts):
        ltab[b, :n] = torch.arange(cur, cur + n, dtype=torch.int32)
        cur += n
        llen[b] = ntok
    ltab, llen = ltab.to(dev), llen.to(dev)
    del pool
    torch.cuda.empty_cache()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    res = [None]

    def make_step(ev):
        def f():
            res[0] = parallel.sequence_parallel_decode(Q, lpool, ltab, llen, D_V, SCALE, timing_events=ev)
        return f
    plain = make_step(None)
    for _ in range(warmup):
        plain()
    torch.cuda.synchronize()
    dist.barrier()
    for i in range(steps):
        make_step(evs[i])()
    torch.cuda.synchronize()
    med = lambda a, b: statistics.median(e[a].elapsed_time(e[b]) for e in evs)
    local_ms, ag_ms, merge_ms = (_median_over_ranks(med(0, 1), world), _median_over_ranks(med(1, 2), world),
                                 _median_over_ranks(med(2, 3), world))
    eager_ms = time_steps(plain, steps, 3, world) / steps
    # the step as a serving loop would run it: buffers allocated once, captured into a CUDA graph, replayed
    dec = parallel.SequenceParallelDecoder(B8, H, D_QK, D_V, PAGE, int(llen.max().item()), dev, scale=SCALE)
    dec.step(Q, lpool, ltab, llen)
    torch.cuda.synchronize()
    dist.barrier()
    prealloc_ms = time_steps(lambda: dec.step(Q, lpool, ltab, llen), steps, 3, world) / steps
    graph_ms = None
    captured = 1
    try:
        dec.capture(Q, lpool, ltab, llen)
    except Exception as exc:                          # capture of the collective refused by this NCCL / torch build
        captured = 0
        sys.stderr.write(f"rank {rank}: long-context step not captured into a CUDA graph: {exc}\n")
    flag = torch.tensor([captured], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)       # every rank replays, or none does
    if int(flag.item()) == 1:
        graph_ms = time_steps(dec.replay, steps, 3, world) / steps
        res[0] = dec.replay()
    else:
        res[0] = dec.step(Q, lpool, ltab, llen)
    torch.cuda.synchronize()
    # the same step with the exchange and the merge as one kernel over peer memory (no collective library on the path)
    peer_eager_ms = peer_graph_ms = None
    peer_equal = None
    peer_ok = 1
    pdec = None
    try:
        pdec = parallel.SequenceParallelDecoder(B8, H, D_QK, D_V, PAGE, int(llen.max().item()), dev, scale=SCALE, exchange="peer")
    except Exception as exc:                          # CUDA IPC between the ranks' processes refused on this machine
        peer_ok = 0
        sys.stderr.write(f"rank {rank}: peer exchange not set up: {exc}\n")
    flag = torch.tensor([peer_ok], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if int(flag.item()) == 1:
        want = tuple(t.clone() for t in res[0])
        got = pdec.step(Q, lpool, ltab, llen)
        torch.cuda.synchronize()
        peer_equal = bool(all(torch.equal(a, b) for a, b in zip(got, want)))
        dist.barrier()
        peer_eager_ms = time_steps(lambda: pdec.step(Q, lpool, ltab, llen), steps, 3, world) / steps
        pdec.capture(Q, lpool, ltab, llen)
        dist.barrier()
        peer_graph_ms = time_steps(pdec.replay, steps, 3, world) / steps
        torch.cuda.synchronize()
        if peer_equal and flashdmla.device_error_flag() == 0 and (graph_ms is None or peer_graph_ms < graph_ms):
            res[0] = pdec.replay()
            torch.cuda.synchronize()
    use_peer = peer_graph_ms is not None and peer_equal and (graph_ms is None or peer_graph_ms < graph_ms)
    peer_eager_wins = use_peer and peer_eager_ms < peer_graph_ms        # two launches: the host can keep up without a graph
    total_ms = (min(peer_graph_ms, peer_eager_ms) if use_peer else (graph_ms if graph_ms is not None else prealloc_ms))
    O, m, l = res[0]
    err = float((O.float() - O1.float()).abs().max())
    msg_bytes = B8 * H * (D_V + 2) * 4
    local_tokens = int(llen.sum().item())
    return {"workload": f"long-context decode B={B8} H={H} Skv~U[16384,131072] page={PAGE}, KV split over {world} GPUs "
                        f"(sequence lengths {lens})",
            "tokens_per_s": B8 / (total_ms * 1e-3), "ms_per_step": total_ms,
            "ms_per_step_how": ("two launches per step enqueued from Python: local attention, then local merge + exchange + merge "
                                "as one kernel over peer memory (SequenceParallelDecoder, exchange='peer')" if peer_eager_wins else
                                "whole step replayed from a CUDA graph: local attention, then local merge + exchange + merge as one "
                                "kernel over peer memory (SequenceParallelDecoder, exchange='peer')" if use_peer else
                                "whole step replayed from a CUDA graph (SequenceParallelDecoder)" if graph_ms is not None
                                else "eager steps on preallocated buffers (SequenceParallelDecoder)"),
            "ms_per_step_eager_python": eager_ms, "ms_per_step_preallocated": prealloc_ms, "ms_per_step_graph": graph_ms,
            "ms_per_step_peer_exchange_eager": peer_eager_ms, "ms_per_step_peer_exchange_graph": peer_graph_ms,
            "peer_exchange_bit_identical_to_nccl_path": peer_equal,
            "phase_times_note": "local / all-gather / merge are CUDA-event spans of the eager Python step: they include the "
                                "host's enqueue gaps",
            "local_splits": dec.splits,
            "local_ms": local_ms, "allgather_ms": ag_ms, "merge_ms": merge_ms,
            "bytes_out": msg_bytes, "bytes_in": (world - 1) * msg_bytes,
            "allgather_busbw_gbs": (world - 1) * msg_bytes / (ag_ms * 1e-3) / 1e9,
            "vs_1gpu_ms": one_ms, "speedup_over_1gpu": one_ms / total_ms,
            "local_hbm_gbs_rank0": local_tokens * D_QK * 2 / (local_ms * 1e-3) / 1e9,
            "max_abs_vs_unsplit": err, "collective": ("exchange_merge_kernel: peer stores over NVLink into buffers mapped with CUDA IPC, the merge in the same kernel "
                           "(the NCCL all-gather + merge path is timed beside it: ms_per_step_graph)" if use_peer else
                           "torch.distributed.all_gather_into_tensor (NCCL), one message per rank"),
            "limiter": max((("local attention", local_ms), ("all-gather", ag_ms), ("merge", merge_ms)), key=lambda kv: kv[1])[0]}


def bench_context_prefill(dev, rank, world, iters=10):
    """Context-parallel causal prefill, B=1, H=128, S=1024 per GPU: zigzag chunks, one NCCL all-gather of the bf16
    latent rows, then the tensor-core forward on this rank's two query chunks."""
    import flashdmla
    from flashdmla import parallel
    S = 1024 * world
    g = torch.Generator(device=dev).manual_seed(4200)          # the same tensors on every rank, then sharded
    K = (torch.randn(1, S, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    Kl = parallel.shard_context(K, world, rank, dim=1)
    Ql = (torch.randn(1, PF_H, S // world, D_QK, generator=torch.Generator(device=dev).manual_seed(4300 + rank), device=dev)
          * 0.1).to(torch.bfloat16)
    del K
    step = lambda: parallel.context_parallel_prefill(Ql, Kl, D_V, SCALE)
    flat = torch.empty((world,) + tuple(Kl.shape), dtype=Kl.dtype, device=dev)
    gather = lambda: dist.all_gather_into_tensor(flat.view(world * Kl.shape[0], *Kl.shape[1:]), Kl)
    for _ in range(3):
        step(); gather()
    tot, ag = [], []
    for _ in range(iters):
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record(); step(); e[1].record(); gather(); e[2].record()
        torch.cuda.synchronize()
        tot.append(e[0].elapsed_time(e[1])); ag.append(e[1].elapsed_time(e[2]))
    total_ms = _median_over_ranks(statistics.median(tot), world)
    ag_ms = _median_over_ranks(statistics.median(ag), world)
    flop = 2.0 * PF_H * (S * (S + 1) / 2) * (D_QK + D_V)
    return {"workload": f"context-parallel causal prefill B=1 H={PF_H} S={S} over {world} GPUs (zigzag chunks)",
            "ms": total_ms, "allgather_ms_alone": ag_ms, "allgather_share": ag_ms / total_ms,
            "allgather_bytes_in": (world - 1) * Kl.numel() * 2, "tflops_total": flop / (total_ms * 1e-3) / 1e12,
            "tokens_per_s": S / (total_ms * 1e-3)}


def bench_prefill(dev, rank, world, tf_burst, tf_sust, iters=10, warmup=3):
    """Causal prefill, B=4,H=128,S=8192, d=576/512, heads sharded over ranks (K_lat replicated); median of `iters`
    launches after `warmup`, max over ranks."""
    import flashdmla
    Hl = PF_H // world
    g = torch.Generator(device=dev).manual_seed(77)
    K = (torch.randn(PF_B, PF_S, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    Q = torch.empty(PF_B, Hl, PF_S, D_QK, dtype=torch.bfloat16, device=dev)
    for b in range(PF_B):       # generated per batch entry to bound the fp32 temporary
        Q[b] = (torch.randn(Hl, PF_S, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16)

    def step():
        return flashdmla.flash_dmla_cache_latent(Q, K, D_V, SCALE, True)
    if world > 1:
        dist.barrier()
    ms = _median_over_ranks(median_launch_ms(step, launches=iters, warmup=warmup), world)
    tflops = PREFILL_FLOP_CAUSAL / (ms * 1e-3) / 1e12
    return {"workload": f"causal prefill B={PF_B} H={PF_H} S={PF_S} d=576/512, heads sharded", "ms": ms, "tflops_total": tflops,
            "tflops_per_gpu": tflops / world, "frac_of_measured_bf16_peak": tflops / world / tf_burst,
            "frac_of_measured_bf16_sustained": tflops / world / tf_sust,
            "frac_of_2250_spec": tflops / world / 2250.0, "kernel_family": flashdmla.last_kernel(),
            "timing": f"median of {iters} launches after {warmup} warm-ups, CUDA events",
            "tokens_per_s": PF_B * PF_S / (ms * 1e-3)}


def bench_on_the_fly(dev, tf_peak, iters=5, only_shape=None):
    """On-the-fly mode (per-head K, V projected to 64-wide latents), causal, forward and backward through the
    autograd operator, at B=8,H=16,S=4096 (the training-backward configuration) and at B=4,H=16,S=2048 (the
    single-GPU forward configuration).  FLOP: attention 4 S(S+1)/2 64 per head forward (two GEMMs), five GEMMs
    backward, plus the latent projections (2 forward, 2 recomputed + 2 gradient + 2 weight-gradient backward)."""
    import flashdmla

    def one(B4, H4, S4, dm=128, dl=64):
        g = torch.Generator(device=dev).manual_seed(99)
        mk = lambda *sh, s=1.0: (torch.randn(*sh, generator=g, device=dev) * s).to(torch.bfloat16)
        Q, K, V = mk(B4, H4, S4, dl), mk(B4, H4, S4, dm), mk(B4, H4, S4, dm)
        WK, WV = mk(dm, dl, s=0.1), mk(dm, dl, s=0.1)
        dO = mk(B4, H4, S4, dl)
        ts = [t.requires_grad_(True) for t in (Q, K, V, WK, WV)]
        attn = 2.0 * B4 * H4 * (S4 * (S4 + 1) / 2) * dl            # one causal GEMM
        proj = 2.0 * B4 * H4 * S4 * dm * dl                        # one projection-sized GEMM
        fwd_flop, bwd_flop = 2 * attn + 2 * proj, 5 * attn + 6 * proj
        fwd_ms, bwd_ms = [], []
        for _ in range(iters + 2):
            for t in ts:
                t.grad = None
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            O, m, l = flashdmla.flash_dmla_on_the_fly(*ts, 0.125, True)
            e[1].record()
            O.backward(dO)
            e[2].record()
            torch.cuda.synchronize()
            fwd_ms.append(e[0].elapsed_time(e[1]))
            bwd_ms.append(e[1].elapsed_time(e[2]))
        f, b = statistics.median(fwd_ms[2:]), statistics.median(bwd_ms[2:])
        return {"workload": f"on-the-fly B={B4} H={H4} S={S4} d_model={dm} d_lat={dl} causal (autograd operator)",
                "fwd_ms": f, "bwd_ms": b, "fwd_tflops": fwd_flop / (f * 1e-3) / 1e12, "bwd_tflops": bwd_flop / (b * 1e-3) / 1e12,
                "fwd_frac_of_measured_bf16_peak": fwd_flop / (f * 1e-3) / 1e12 / tf_peak,
                "bwd_frac_of_measured_bf16_peak": bwd_flop / (b * 1e-3) / 1e12 / tf_peak,
                "tokens_per_s_fwd": B4 * S4 / (f * 1e-3), "kernel_family": flashdmla.last_kernel()}
    if only_shape is not None:
        return one(*only_shape)
    out = one(8, 16, 4096)
    out["config1"] = one(4, 16, 2048)
    return out


def bench_cache_latent_bwd(dev, tf_peak, iters=5):
    """Cache-latent backward at B=1, H=128, Sq=Skv=1024, d=576/512, causal, through the autograd operator: tensor-core
    GEMMs over a score workspace (unfused).  FLOP counted for the visible half only: 2 (3 x 576 + 2 x 512) per score."""
    import flashdmla
    Bc, Hc, Sc = 1, 128, 1024
    g = torch.Generator(device=dev).manual_seed(55)
    Q = (torch.randn(Bc, Hc, Sc, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16).requires_grad_(True)
    K = (torch.randn(Bc, Sc, D_QK, generator=g, device=dev) * 0.1).to(torch.bfloat16).requires_grad_(True)
    dO = torch.randn(Bc, Hc, Sc, D_V, generator=g, device=dev).to(torch.bfloat16)
    ts = []
    for _ in range(iters + 2):
        Q.grad = K.grad = None
        O, m, l = flashdmla.flash_dmla_cache_latent(Q, K, D_V, SCALE, True)
        a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); O.backward(dO); b2.record(); torch.cuda.synchronize()
        ts.append(a.elapsed_time(b2))
    ms = statistics.median(ts[2:])
    flop = 2.0 * Bc * Hc * (Sc * (Sc + 1) / 2) * (3 * D_QK + 2 * D_V)
    return {"workload": f"cache-latent backward B={Bc} H={Hc} Sq=Skv={Sc} d=576/512 causal (autograd operator)", "ms": ms,
            "tflops_visible_half": flop / (ms * 1e-3) / 1e12, "frac_of_measured_bf16_peak": flop / (ms * 1e-3) / 1e12 / tf_peak,
            "kernel_family": flashdmla.last_kernel(),
            "how": "five tcgen05 GEMM launches and one elementwise kernel per chunk of query rows (causal: score tiles nobody sees are left out "
                   "of the S, dP and dQ GEMMs; the dK GEMMs run over the masked half too)"}


def bench_gemm(dev, tf_burst, hbm_peak, E=64):
    """The library's batched tensor-core GEMM on its three uses: the expert MLPs of a MoE layer over padded packing
    (E=64 experts x 640 rows, d=4096, d_ff=1024: gate+up GEMM with the SwiGLU gate in its epilogue, then the down
    GEMM), with the same arithmetic on the vendor library's batched GEMM beside it for scale, and the absorbed
    query / output projections of an MLA block at the decode batch (n=128 tokens, H=128 heads; replayed from a CUDA
    graph, because one launch is shorter than a Python call)."""
    from flashdmla import gemm
    g = torch.Generator(device=dev).manual_seed(5)
    mk = lambda *sh, std=0.1: (torch.randn(*sh, generator=g, device=dev) * std).to(torch.bfloat16)
    rows, d, f = 640, 4096, 1024
    xb, W1, W3, W2 = mk(E, rows, d), mk(E, d, f, std=0.02), mk(E, d, f, std=0.02), mk(E, f, d, std=0.02)
    h = torch.empty(E, rows, f, dtype=torch.bfloat16, device=dev)
    y = torch.empty(E, rows, d, dtype=torch.bfloat16, device=dev)
    g1 = lambda: gemm.gemm_batched(xb.view(E * rows, d), W1.view(E * d, f), h.view(E * rows, f), E, rows, f, d,
                                   a_brow=rows, b_brow=d, c_brow=rows, gate=W3.view(E * d, f))
    g2 = lambda: gemm.gemm_batched(h.view(E * rows, f), W2.view(E * f, d), y.view(E * rows, d), E, rows, d, f,
                                   a_brow=rows, b_brow=f, c_brow=rows)
    t1, t2 = median_launch_ms(g1, launches=20, warmup=3), median_launch_ms(g2, launches=20, warmup=3)
    lib_ms = median_launch_ms(lambda: torch.bmm(torch.nn.functional.silu(torch.bmm(xb, W1)) * torch.bmm(xb, W3), W2),
                              launches=20, warmup=3)
    fl1, fl2 = 2.0 * E * rows * d * 2 * f, 2.0 * E * rows * f * d
    del xb, W1, W3, W2, h, y
    n, Hh = 128, 128
    q, WUK, WUV, o_lat = mk(n, Hh, 192), mk(Hh, 512, 128), mk(Hh, 512, 128), mk(n, Hh, 512)
    Qo = torch.empty(n, Hh, 576, dtype=torch.bfloat16, device=dev)
    oo = torch.empty(n, Hh, 128, dtype=torch.bfloat16, device=dev)
    ga = lambda: gemm.gemm_batched(q.view(n, Hh * 192), WUK.view(Hh * 512, 128), Qo.view(n, Hh * 576), Hh, n, 512, 128,
                                   a_bcol=192, b_brow=512, b_k_major=True, c_bcol=576)
    gp = lambda: gemm.gemm_batched(o_lat.view(n, Hh * 512), WUV.view(Hh * 512, 128), oo.view(n, Hh * 128), Hh, n, 128, 512,
                                   a_bcol=512, b_brow=512, c_bcol=128)

    def graph_ms(fn, reps=20):
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                for _ in range(reps):
                    fn()
        torch.cuda.synchronize()
        return median_launch_ms(gr.replay, launches=10, warmup=2) / reps
    ta, tp = graph_ms(ga), graph_ms(gp)
    del q, WUK, WUV, o_lat, Qo, oo
    # the CTA-pair form of the kernel (256 x 256 tiles over two SMs) on a problem whose rows fill such tiles
    Mp = 8192
    Ap, Bp, Cp = mk(Mp, Mp), mk(Mp, Mp, std=0.02), torch.empty(Mp, Mp, dtype=torch.bfloat16, device=dev)
    t_pair = median_launch_ms(lambda: gemm.gemm_batched(Ap, Bp, Cp, 1, Mp, Mp, Mp), launches=10, warmup=3)
    t_vend = median_launch_ms(lambda: torch.matmul(Ap, Bp, out=Cp), launches=10, warmup=3)
    del Ap, Bp, Cp
    ba, bp = (n * Hh * 128 + Hh * 512 * 128 + n * Hh * 512) * 2, (n * Hh * 512 + Hh * 512 * 128 + n * Hh * 128) * 2
    return {"kernel": "tcg::gemm_kernel (tcgen05, TMA ring of 4 x 48 KB, 128 x 256 tiles, two accumulators in tensor memory; "
                      "CTA pairs with 256 x 256 tiles and 6 x 32 KB stages where the rows fill them)",
            "pair_form_8192_cubed_ms": t_pair, "pair_form_8192_cubed_tflops": 2.0 * Mp ** 3 / (t_pair * 1e-3) / 1e12,
            "pair_form_8192_cubed_frac_of_measured_bf16_peak": 2.0 * Mp ** 3 / (t_pair * 1e-3) / 1e12 / tf_burst,
            "vendor_library_8192_cubed_tflops": 2.0 * Mp ** 3 / (t_vend * 1e-3) / 1e12,
            "expert_mlp_workload": f"E={E} x {rows} rows, d={d}, d_ff={f}, bf16 (padded packing of T=4096, top-8, capacity 1.25)",
            "gate_up_gemm_ms": t1, "gate_up_gemm_tflops": fl1 / (t1 * 1e-3) / 1e12, "down_gemm_ms": t2,
            "down_gemm_tflops": fl2 / (t2 * 1e-3) / 1e12,
            "expert_mlp_tflops": (fl1 + fl2) / ((t1 + t2) * 1e-3) / 1e12,
            "expert_mlp_frac_of_measured_bf16_peak": (fl1 + fl2) / ((t1 + t2) * 1e-3) / 1e12 / tf_burst,
            "vendor_library_same_arithmetic_ms": lib_ms, "vendor_library_tflops": (fl1 + fl2) / (lib_ms * 1e-3) / 1e12,
            "absorbed_query_gemm_us": ta * 1e3, "absorbed_output_gemm_us": tp * 1e3,
            "absorbed_query_gbs_l2_resident": ba / (ta * 1e-3) / 1e9, "absorbed_output_gbs_l2_resident": bp / (tp * 1e-3) / 1e9,
            "absorbed_workload": f"n={n} tokens, H={Hh}: [n,128]x[128,512] and [n,512]x[512,128] per head, CUDA-graph replay, "
                                 f"operands resident in L2 (42 MB)"}


def bench_moe_plumbing(dev, hbm_peak, iters=5):
    """The MoE kernels around the expert GEMMs at T=4096 tokens, E=256 experts, top-8, d=7168 bf16 (the shape of a
    DeepSeek-V3 MoE layer; capacity factor 1.25): gate, packing, row gather, weighted combine.  Algorithmic bytes:
    gate T E 4; gather (T + rows) x d x 2 (every token row once from HBM - its other reads hit L2 - and the packed
    rows out); combine (rows + 2 T) x d x 2 (packed rows and the shared output in, the result out)."""
    from flashdmla import moe
    T, E, k, d = 4096, 256, 8, 7168
    g = torch.Generator(device=dev).manual_seed(123)
    logits = torch.randn(T, E, generator=g, device=dev)
    x = (torch.randn(T, d, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    cap = int(1.25 * T * k / E)
    idx, w = moe.route_topk(logits, k)
    pos, perm, offs = moe.pack(idx, E, cap)
    rows = int(offs[-1])
    xp = moe.gather(x, perm, offs)
    sh = torch.zeros_like(x)

    def t_of(fn):
        ts = []
        for _ in range(iters + 2):
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b2.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b2))
        ts = sorted(ts[2:])
        return ts[len(ts) // 2]
    gate_ms = t_of(lambda: moe.route_topk(logits, k))
    pack_ms = t_of(lambda: moe.pack(idx, E, cap))
    gather_ms = t_of(lambda: moe.gather(x, perm, offs))
    scatter_ms = t_of(lambda: moe.scatter(x, pos, perm.shape[0]))
    comb_ms = t_of(lambda: moe.combine(xp, pos, w, sh))
    gb = lambda nbytes, ms: nbytes / (ms * 1e-3) / 1e9
    # a whole layer (padded packing, expert MLPs on the library's batched tensor-core GEMM, shared expert), smaller model
    layer = moe.MoEFFN(d_model=4096, d_ff=1024, n_experts=64, top_k=8, capacity_factor=1.25, device=dev, seed=1)
    xl = (torch.randn(T, 4096, generator=g, device=dev) * 0.1).to(torch.bfloat16)
    layer_ms = t_of(lambda: layer.forward_batched(xl))
    layer_grouped_ms = t_of(lambda: layer.forward(xl))
    del layer
    return {"layer_batched_ms": layer_ms, "layer_grouped_ms": layer_grouped_ms,
            "layer_grouped_how": "MoEFFN.forward: ragged packing, the expert MLPs as two launches of the grouped GEMM that reads "
                                 "the experts' row ranges on the device (no padding rows, no host read-back)",
            "layer_workload": "MoEFFN.forward_batched T=4096 d=4096 d_ff=1024 E=64 top-8 + shared expert, bf16",
            "workload": f"MoE plumbing T={T} E={E} top-{k} d={d} bf16, capacity {cap} ({rows} packed rows)",
            "gate_ms": gate_ms, "pack_ms": pack_ms, "gather_ms": gather_ms, "scatter_ms": scatter_ms, "combine_ms": comb_ms,
            "scatter_gbs": gb((T + rows) * d * 2.0, scatter_ms), "scatter_frac_of_hbm": gb((T + rows) * d * 2.0, scatter_ms) / hbm_peak,
            "gather_gbs": gb((T + rows) * d * 2.0, gather_ms), "combine_gbs": gb((rows + 2.0 * T) * d * 2, comb_ms),
            "gather_frac_of_hbm": gb((T + rows) * d * 2.0, gather_ms) / hbm_peak,
            "combine_frac_of_hbm": gb((rows + 2.0 * T) * d * 2, comb_ms) / hbm_peak}


if __name__ == "__main__":
    main()
