#!/usr/bin/env python3
"""Benchmark of the SSD chunked scan, forward + backward, in tokens/s.

    python bench.py --gpus N --steps K --warmup W [--config I] [--impl ours|reference]

One step = one forward + backward pass of the Mamba-2 style scan operator over one batch of
seeded synthetic input.  The default workload is the 1.3B-layer shape (batch 16 per GPU, weak
scaling: every rank runs its own batch, no data-path collective).  For N > 1 the script is
launched by torchrun, one rank per GPU.

``value``   : tokens/s with inputs resident in HBM (CUDA events, barrier + sync both sides, max over ranks)
``e2e``     : same metric through the public operator with HOST buffers; every step copies the inputs
              host->device from pinned memory and all results device->host, inside the timed region
``roofline``: the dominant kernel's algorithmic bytes / its CUDA-event duration vs the measured HBM peak
``cpu_baseline`` / ``--impl reference``: the CPU oracle (the reference's eager PyTorch SSD path restated)
              timed on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 0.0))), "measured"
    return FALLBACK_HBM_GBS, 1400.0, "fallback"


def dram_bytes_per_token(cfg_tag: str) -> dict[str, float]:
    """profiles/dram_traffic_per_token.txt: lines `<cfg tag> <kernel slot> <dram bytes per token>` taken from the
    ncu captures summarised beside it."""
    p = ROOT / "profiles" / "dram_traffic_per_token.txt"
    out = {}
    if p.exists():
        for line in p.read_text().splitlines():
            f = line.split()
            if len(f) >= 3 and not line.startswith("#") and f[0] == cfg_tag:
                out[f[1]] = float(f[2])
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower() == "active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_oracle_tokens_per_s(cfg, pkg, repeats: int = 3, target_s: float = 20.0):
    """Time the CPU oracle (forward + backward) on a bounded sample of the workload."""
    from oracle import ssd_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    batch, seqlen = 1, min(cfg.seqlen, 1024)
    small = pkg.shrink(cfg, batch, seqlen)
    inp = pkg.make_inputs(small)
    O.mamba2_fwd_bwd(inp, small.chunk)  # warm-up
    times = []
    t_begin = time.perf_counter()
    while len(times) < repeats or (time.perf_counter() - t_begin < target_s / 2 and len(times) < 20):
        t0 = time.perf_counter()
        O.mamba2_fwd_bwd(inp, small.chunk)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return small.tokens / med, threads, f"batch {batch} x seqlen {seqlen} of {cfg.name}, fp32 on bf16-rounded inputs, median of {len(times)}"


def run_reference(args, cfg, pkg, rank):
    """The reference arm: the reference's own eager CPU path (restated as the oracle), host cores only."""
    if rank != 0:
        return
    vals = []
    sample = ""
    threads = 1
    for i in range(args.warmup + args.steps):
        v, threads, sample = cpu_oracle_tokens_per_s(cfg, pkg, repeats=1, target_s=0.0)
        if i >= args.warmup:
            vals.append(v)
    value = statistics.median(vals)
    small_tokens = min(cfg.seqlen, 1024)
    line = {
        "impl": "reference", "metric": "ssd_scan_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * small_tokens / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "note": "CPU arm: the reference has no packaging to install; its eager PyTorch SSD "
                   "path (restated in oracle/ssd_oracle.py, pinned bit-exact against the imported reference) runs on the host cores"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_elementwise(args, cfg, pkg):
    """Rotation (fused_rope), trapezoidal coefficients (fused_trapezoidal) and the gated norm after the scan
    (fused_gate_norm), forward + backward, at the shapes of the block around the scan for this config: achieved HBM
    GB/s on the bytes each call must move."""
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    hbm_peak, _, peak_kind = measured_peaks()
    b, T, h, n = cfg.batch, cfg.seqlen, cfg.nheads, cfg.d_state
    dt = torch.bfloat16 if cfg.dtype == "bf16" else torch.float32
    es = 2 if cfg.dtype == "bf16" else 4
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(b, T, h, n, generator=g, device=dev).to(dt).requires_grad_(True)
    ang = torch.randn(b, T, h, n // 2, generator=g, device=dev).requires_grad_(True)
    gy = torch.randn(b, T, h, n, generator=g, device=dev).to(dt)
    dt_raw = torch.randn(b, T, h, generator=g, device=dev).to(dt).requires_grad_(True)
    lam_raw = torch.randn(b, T, h, generator=g, device=dev).to(dt).requires_grad_(True)
    bias = torch.zeros(h, device=dev, requires_grad=True)
    alog = torch.zeros(h, device=dev, requires_grad=True)
    g4 = [torch.randn(b, T, h, generator=g, device=dev).to(dt) for _ in range(4)]

    def rope_step():
        y = pkg.fused_rope(x, ang)
        torch.autograd.grad([y], [x, ang], [gy])

    def trap_step():
        outs = pkg.fused_trapezoidal(dt_raw, lam_raw, bias, alog)
        torch.autograd.grad(list(outs), [dt_raw, lam_raw, bias, alog], g4)

    yg = torch.randn(b * T, h * cfg.headdim, generator=g, device=dev).to(dt).requires_grad_(True)
    zg = torch.randn(b * T, h * cfg.headdim, generator=g, device=dev).to(dt).requires_grad_(True)
    wg = torch.ones(h * cfg.headdim, device=dev, requires_grad=True)
    gg_ = torch.randn(b * T, h * cfg.headdim, generator=g, device=dev).to(dt)

    def gate_step():
        o = pkg.fused_gate_norm(yg, zg, wg, 1e-6)
        torch.autograd.grad([o], [yg, zg, wg], [gg_])

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / args.steps

    nx, na, nt_ = b * T * h * n, b * T * h * (n // 2), b * T * h
    # rope: fwd reads x, angles, writes y; bwd reads x, angles, dy, writes dx, dangles (fp32 angles)
    rope_bytes = (2 * nx * es + na * 4) + (3 * nx * es + 2 * na * 4)
    # trapezoid: fwd reads 2, writes 4; bwd reads 2 + 4, writes 2
    trap_bytes = 14 * nt_ * es
    # gate norm: fwd reads y, z, writes out; bwd reads y, z, dout, writes dy, dz (the dw pass re-reads three of them)
    gate_bytes = 8 * b * T * h * cfg.headdim * es
    ms_r, ms_t, ms_g = timed(rope_step), timed(trap_step), timed(gate_step)
    # forward of the gated norm alone, with its own row statistic (two reads of y) and with the partial sums the scan's
    # forward leaves behind (one read of y), through the C ABI
    import ctypes as C
    cabi = importlib.import_module("dhammic-ai_b200._cabi")
    lib = cabi.load()
    rows, Dn = b * T, h * cfg.headdim
    ysq = torch.rand(rows // 128 * h * 2 * 128, device=dev)
    out_n = torch.empty_like(yg)
    rstd = torch.empty(rows, device=dev)
    code = cabi.BF16 if cfg.dtype == "bf16" else cabi.F32
    ptr = lambda t: C.c_void_p(t.data_ptr())
    stream = lambda: C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    wf = wg.detach().float().contiguous()

    def norm_fwd_own():
        cabi.check(lib.ssd_b200_rmsnorm_fwd(code, rows, Dn, 1e-6, ptr(yg), ptr(wf), ptr(zg), ptr(out_n), ptr(rstd), stream()))

    def norm_fwd_presummed():
        cabi.check(lib.ssd_b200_rmsnorm_fwd_presummed(code, rows, Dn, 1e-6, ptr(yg), ptr(wf), ptr(zg), ptr(ysq), h, ptr(out_n),
                                                      ptr(rstd), stream()))

    ms_n1, ms_n2 = timed(norm_fwd_own), timed(norm_fwd_presummed)
    fwd_bytes = 3 * rows * Dn * es
    line = {"metric": "elementwise_fwd_bwd_GBps", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "dtype": "bf16" if cfg.dtype == "bf16" else "f32", "data": "synthetic", "higher_is_better": True,
            "config": {"workload": cfg.name, "rope": [b, T, h, n], "trapezoid": [b, T, h],
                       "l2": "tensors larger than L2 (x %.0f MB)" % (nx * es / 1e6)},
            "rope": {"ms": ms_r, "GBps": rope_bytes / ms_r / 1e6, "frac_of_hbm": rope_bytes / ms_r / 1e6 / hbm_peak},
            "trapezoid": {"ms": ms_t, "GBps": trap_bytes / ms_t / 1e6, "frac_of_hbm": trap_bytes / ms_t / 1e6 / hbm_peak},
            "gate_norm": {"ms": ms_g, "GBps": gate_bytes / ms_g / 1e6, "frac_of_hbm": gate_bytes / ms_g / 1e6 / hbm_peak,
                          "shape": [b * T, h * cfg.headdim]},
            "gate_norm_forward": {"own_statistic_ms": ms_n1, "presummed_ms": ms_n2, "algorithmic_GB": fwd_bytes / 1e9,
                                  "own_statistic_frac_of_hbm": fwd_bytes / ms_n1 / 1e6 / hbm_peak,
                                  "presummed_frac_of_hbm": fwd_bytes / ms_n2 / 1e6 / hbm_peak},
            "peak": hbm_peak, "peak_kind": peak_kind}
    line["value"] = line["rope"]["GBps"]
    print(json.dumps(line))


def seq_parallel_record(pkg, dmod, cabi, args, dev, rank, world, barrier):
    """Config 4 (one sequence of 131,072 positions split contiguously over the ranks; per-rank state summaries cross
    NVLink through NCCL): tokens/s over all ranks, the same sequence on ONE GPU (rank 0, cut into segments that run
    as batch entries) for comparison, and where a step's time goes (library kernels by CUDA events on the launching
    stream, collectives by events on their side stream)."""
    import torch.distributed as dist
    full = pkg.CONFIGS[4]
    cfg = pkg.shrink(full, full.batch, full.seqlen // world)
    names = ("x", "dt", "A_head", "B", "C", "D", "dy")

    def make_step(c, seed_rank, comm):
        host = pkg.make_inputs(c, rank=seed_rank)
        d = {k: host[k].to(dev) for k in names}
        lv = {k: d[k].detach().requires_grad_(True) for k in names if k != "dy"}

        def step():
            y, _ = dmod.ssd_mamba2_sequence_parallel(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], c.chunk,
                                                     comm=comm, segments=0)
            return torch.autograd.grad([y], list(lv.values()), [d["dy"]])
        return step

    def timed(step, sync, steps, collective):
        for _ in range(max(3, args.warmup)):
            step()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if collective:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    steps = max(3, min(args.steps, 10))
    comm, comm_kind = dmod.make_comm(prefer_peer_stores=not args.nccl_exchange)
    step = make_step(cfg, rank, comm)
    ms = timed(step, barrier, steps, True)
    # phases of one step: kernels per slot, collectives from the communicator's own events
    cabi.profile_enable(True)
    comm.timings = []
    for _ in range(steps):
        step()
    torch.cuda.synchronize(dev)
    prof = cabi.profile_read()
    cabi.profile_enable(False)
    coll = comm.read_timings()
    comm.timings = None
    phases = {k: v[0] / steps for k, v in prof.items()}
    phases.update({f"comm_{k}": v / steps for k, v in coll.items()})
    del step
    torch.cuda.empty_cache()
    barrier()
    one_gpu = None
    if rank == 0:  # the whole sequence on one GPU, segments as batch entries, no communicator
        step1 = make_step(full, 0, dmod.LoopbackComm())
        ms1 = timed(step1, lambda: torch.cuda.synchronize(dev), steps, False)
        one_gpu = {"ms_per_step": ms1, "tokens_per_s": full.tokens / (ms1 * 1e-3)}
        del step1
        torch.cuda.empty_cache()
    barrier()
    return {"workload": full.name, "scaling": "strong", "n_gpus": world, "tokens_per_step": full.tokens,
            "ms_per_step": ms, "value": full.tokens / (ms * 1e-3), "unit": "tokens/s", "steps": steps,
            "one_gpu_segmented": one_gpu,
            "segments_per_rank": dmod.pick_segments(cfg.batch, cfg.nheads, cfg.seqlen),
            "exchange": "1 gather of one state per rank (forward) + 1 gather + 1 small all_reduce (backward) per step; gathers by "
                        + comm_kind,
            "exchange_status": comm.status() if hasattr(comm, "status") else 0,
            "phase_ms_per_step": phases}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=5, help="timed loops of --steps steps each; the median loop is reported")
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (debug)")
    ap.add_argument("--seqlen", type=int, default=0, help="override the sequence length (debug)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--micro-batches", type=int, default=8, help="e2e: micro-batches of the host pipeline")
    ap.add_argument("--no-seq-parallel", action="store_true", help="N > 1: skip the sequence-split sub-record")
    ap.add_argument("--nccl-exchange", action="store_true", help="sequence split: gather the summaries with NCCL instead of peer stores")
    ap.add_argument("--op", default="scan", choices=["scan", "elementwise"],
                    help="elementwise: time the rotation and trapezoidal-coefficient operators instead of the scan")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    pkg = importlib.import_module("dhammic-ai_b200")
    cfg = pkg.CONFIGS[args.config]
    if args.batch or args.seqlen:
        cfg = pkg.shrink(cfg, args.batch or None, args.seqlen or None)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, cfg, pkg, rank)
        return
    if args.op == "elementwise":
        run_elementwise(args, cfg, pkg)
        return

    import torch.distributed as dist
    cabi = importlib.import_module("dhammic-ai_b200._cabi")
    cabi.load()  # fails loudly if the CUDA library is missing
    pkg.set_kernel_path(args.path)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    seq_par = cfg.seq_parallel and world > 1
    if cfg.seq_parallel:
        if cfg.seqlen % (world * 128) != 0:
            raise SystemExit("sequence length must split into multiples of 128 per rank")
        cfg = pkg.shrink(cfg, cfg.batch, cfg.seqlen // world)  # this rank's contiguous slice
    dmod = importlib.import_module("dhammic-ai_b200.distributed")
    host = pkg.make_inputs(cfg, rank=rank)
    names = ("x", "dt", "A_head", "B", "C", "D", "dy") + (("raw_angles", "lam") if cfg.mamba3 else ())
    pinned = {k: host[k].pin_memory() for k in names}
    devin = {k: pinned[k].to(dev, non_blocking=True) for k in names}
    leaves = {k: devin[k].detach().requires_grad_(True) for k in names if k != "dy"}

    def scan(lv):
        if cfg.mamba3:  # rotary state angles + trapezoidal two-term form: two scans behind an element-wise prologue
            return pkg.ssd_mamba3(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], lv["raw_angles"], lv["lam"],
                                  cfg.chunk), None
        if seq_par:  # contiguous sequence split: per-rank states cross NVLink through NCCL
            return dmod.ssd_mamba2_sequence_parallel(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk,
                                                     segments=0)
        if cfg.seq_parallel:  # one GPU: the same schedule with the segments as extra batch entries
            return dmod.ssd_mamba2_segmented(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk)
        return pkg.ssd_mamba2(lv["x"], lv["dt"], lv["A_head"], lv["B"], lv["C"], lv["D"], cfg.chunk)

    def step_device():
        y, _ = scan(leaves)
        return y, torch.autograd.grad([y], list(leaves.values()), [devin["dy"]])

    # the sampler starts before the warm-up (the timed region is tens of milliseconds; nvidia-smi needs a moment to
    # come up) and keeps the samples taken from then to the end of the timed region, all of them under load
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step_device()
    barrier()
    launches0 = cabi.launch_count()
    # EXACTLY args.steps steps per timed loop, barrier + synchronise on both sides, CUDA events on the launching
    # stream, max over ranks; the loop is repeated and the median loop is reported (the spread goes into the line)
    loops = []
    for _ in range(max(1, args.repeats)):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step_device()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        loops.append(float(t.item()))
    launches = (cabi.launch_count() - launches0) // len(loops)
    clocks = sampler.stop() if rank == 0 else None
    ms_max = statistics.median(loops)
    tokens_all = cfg.tokens * world
    value = tokens_all * args.steps / (ms_max * 1e-3)

    # per-kernel durations (CUDA events inside the library, on the launching stream), same steps again
    cabi.profile_enable(True)
    for _ in range(args.steps):
        step_device()
    torch.cuda.synchronize(dev)
    prof = cabi.profile_read()
    cabi.profile_enable(False)
    hbm_peak, tc_peak, peak_kind = measured_peaks()
    total_kernel_ms = sum(v[0] for v in prof.values()) or 1.0
    kernels = {k: {"ms_per_launch": v[0] / v[1], "launches_per_step": v[1] / args.steps,
                   "share": v[0] / total_kernel_ms} for k, v in prof.items()}
    top = max(prof.items(), key=lambda kv: kv[1][0])[0]
    alg = pkg.kernel_algorithmic_bytes(cfg)
    top_bytes = alg.get(top, 0)
    top_ms = kernels[top]["ms_per_launch"]
    achieved = top_bytes / (top_ms * 1e-3) / 1e9 if top_bytes else 0.0
    step_bytes = cfg.bytes_per_token() * cfg.tokens
    step_flops = cfg.flops_per_token() * cfg.tokens
    ms_step = ms_max / args.steps
    # dram read + write of one launch, from the tracked ncu summary (bytes per token of this per-token shape,
    # captured at a smaller batch and scaled by tokens: traffic grows in proportion); None without a capture
    per_token = dram_bytes_per_token(cfg.name.split("_")[0])
    traffic = per_token[top] * cfg.tokens if top in per_token else None
    roofline = {
        "bound": "hbm", "kernel": top, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
        "frac": achieved / hbm_peak, "traffic": traffic, "peak_kind": peak_kind,
        "whole_step": {"algorithmic_GB": step_bytes / 1e9, "algorithmic_TFLOP": step_flops / 1e12,
                       "hbm_frac": step_bytes / (ms_step * 1e-3) / 1e9 / hbm_peak,
                       "tensor_frac": step_flops / (ms_step * 1e-3) / 1e12 / tc_peak if tc_peak else None},
        "kernels": kernels,
    }

    # end to end: host buffers in, host buffers out, through the public operator
    e2e = None
    if not args.no_e2e:
        h2d = sum(pinned[k].numel() * pinned[k].element_size() for k in names)
        e2e_steps = max(2, min(args.steps, 5))
        streamed = cfg.seq_parallel and world == 1 and cfg.seqlen % 16384 == 0
        plain = (cfg.mamba3 or cfg.seq_parallel) and not streamed
        if streamed:
            # one long sequence on one GPU: sequence slices streamed from host memory with the state carried across
            runner = pkg.SequenceStreamer(dev, slice_len=16384)
            out_host = pkg.HostPipeline.alloc_outputs(pinned)
            h2d = 2 * h2d - pinned["dy"].numel() * pinned["dy"].element_size()  # inputs cross twice (forward, backward)

            def step_e2e():
                runner.run(pinned, out_host, cfg.chunk)
        elif not plain:
            # the package's host-buffer entry: micro-batches, copies overlapped with the kernels on three streams
            pipe = pkg.HostPipeline(dev, micro_batches=args.micro_batches)
            out_host = pkg.HostPipeline.alloc_outputs(pinned)

            def step_e2e():
                pipe.run(pinned, out_host, cfg.chunk)
        else:
            out_host = None

            def step_e2e():
                nonlocal out_host
                d = {k: pinned[k].to(dev, non_blocking=True) for k in names}
                lv = {k: d[k].requires_grad_(True) for k in names if k != "dy"}
                y, _ = scan(lv)
                grads = torch.autograd.grad([y], list(lv.values()), [d["dy"]])
                outs = [y.detach(), *grads]
                if out_host is None:
                    out_host = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True) for o in outs]
                for o, hbuf in zip(outs, out_host):
                    hbuf.copy_(o, non_blocking=True)

        step_e2e()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            step_e2e()
        e1.record()
        barrier()
        t2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        outs_iter = out_host.values() if isinstance(out_host, dict) else out_host
        d2h = sum(o.numel() * o.element_size() for o in outs_iter)
        e2e = {"value": tokens_all * e2e_steps / (float(t2.item()) * 1e-3), "unit": "tokens/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "api": ("SequenceStreamer.run (16384-position slices, state carried across)" if streamed else
                       f"HostPipeline.run ({args.micro_batches} micro-batches, 3 streams)" if not plain else "operator call on pinned buffers")}

    # N > 1: the long-context configuration, whose sequence is split over the ranks (the only one with a collective
    # on the data path), rides along as a sub-record; `value` stays the batch-sharded configuration
    seq_record = None
    if world > 1 and not cfg.seq_parallel and not cfg.mamba3 and not args.no_seq_parallel:
        seq_record = seq_parallel_record(pkg, dmod, cabi, args, dev, rank, world, barrier)

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, threads, sample = cpu_oracle_tokens_per_s(cfg, pkg)
        cpu_base = {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": "ssd_scan_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if cfg.seq_parallel else "weak", "vs_baseline": None,
            "dtype": "bf16" if cfg.dtype == "bf16" else "f32",
            "data": "synthetic",
            "config": {"workload": cfg.name, "batch_per_gpu": cfg.batch, "seqlen": cfg.seqlen, "nheads": cfg.nheads,
                       "headdim": cfg.headdim, "d_state": cfg.d_state, "ngroups": cfg.ngroups, "chunk": cfg.chunk,
                       "parallelism": (f"sequence split x{world}, all_gather of per-rank states (NCCL)" if cfg.seq_parallel
                                       else f"batch-sharded x{world}, no data-path collective"),
                       "kernel_path": pkg.resolved_path_name(cfg), "accumulate": "fp32",
                       "l2": "inputs larger than L2 (x alone %.0f MB per GPU)" % (cfg.tokens * cfg.nheads * cfg.headdim * 2 / 1e6)},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_base,
            "timed_loops": {"count": len(loops), "ms_per_step_median": ms_step, "ms_per_step_min": min(loops) / args.steps,
                            "ms_per_step_max": max(loops) / args.steps},
        }
        if seq_record is not None:
            line["seq_parallel"] = seq_record
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
