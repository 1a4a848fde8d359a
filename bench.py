#!/usr/bin/env python
"""Headline benchmark: sampled rows/s at B=256, V=151936 (f32 logits, temperature 0.7, top-k 50,
top-p 0.9, frequency/presence penalties over 512-id histories -- the per-row recipe of the
batched stochastic configuration, at the batch size the metric is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the logits -> token chain over one batch.  With N > 1 (one process per
GPU under torchrun) every rank samples its own 256-row batch -- rows are independent, so there
is no data-path collective -- and the value is all ranks' rows over the slowest rank's time.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, VOCAB = 256, 151936
METRIC = "sampled rows/s at B=256,V=151936"
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (earlier measurement on this pool)"


def ncu_traffic_per_row():
    """DRAM bytes per row of the dominant kernel from the committed ncu summary, if there is one."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return float(json.load(f)["dram_bytes_per_row"])
    except Exception:
        return None


class ClockSampler:
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.path = f"/tmp/pgs_clocks_{os.getpid()}.csv"
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t0: float = 0.0, t1: float = 1e18) -> dict:
        """Summary over the samples taken inside [t0, t1] (all samples if none fall inside)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        import datetime
        sm, mx, reasons, sm_all, mx_all = [], [], set(), [], []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(p[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    a, b = float(p[1]), float(p[2])
                except ValueError:
                    continue
                sm_all.append(a); mx_all.append(b)
                if not (t0 - 0.05 <= ts <= t1 + 0.05):
                    continue
                sm.append(a); mx.append(b)
                for name, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        out["in_timed_region"] = bool(sm)
        if not sm:
            sm, mx = sm_all, mx_all
        if sm:
            out["sm_mhz"] = float(np.median(sm)); out["sm_max_mhz"] = float(max(mx))
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def cpu_port_rows_per_s(w, sample_rows: int, threads: int):
    """The CPU restatement of the reference chain on `sample_rows` rows of the workload."""
    from oracle import oracle
    sub = w.head(sample_rows)
    warm = w.head(min(threads, sample_rows))
    oracle.sample_batch(warm.logits_f32(), n_threads=threads, **warm.oracle_kwargs())  # page in
    t0 = time.perf_counter()
    oracle.sample_batch(sub.logits_f32(), n_threads=threads, **sub.oracle_kwargs())
    dt = time.perf_counter() - t0
    return sample_rows / dt, dt


def run_reference(args, rank, world):
    """--impl reference: the reference chain's CPU restatement on all host cores (the reference is
    Rust and no Rust toolchain exists here, so its own build cannot run)."""
    if rank != 0:
        return
    from pagoda_b200 import synth
    threads = os.cpu_count() or 1
    sample_rows = 64
    w = synth.headline(rows=sample_rows)
    for _ in range(max(args.warmup, 1)):
        cpu_port_rows_per_s(w, min(threads, sample_rows), threads)
    t_total, rows_total = 0.0, 0
    for _ in range(args.steps):
        rps, dt = cpu_port_rows_per_s(w, sample_rows, threads)
        t_total += dt; rows_total += sample_rows
    value = rows_total / t_total
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "headline: B=256 V=151936 f32, T=0.7 top-k 50 top-p 0.9 freq 0.2 pres 0.1, "
                                   "512-id histories", "sample": f"{sample_rows} rows per step"},
            "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                             "sample": f"{sample_rows} rows of the headline workload per step, rows spread over "
                                       f"{threads} host threads"},
            "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--phases", action="store_true",
                    help="print the fused kernel's in-kernel phase timers (cycles per row) for a few steps and exit")
    args = ap.parse_args()
    if args.phases:
        os.environ["PGS_PROFILE"] = "1"   # read when the sampler is created

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import pagoda_b200
    from pagoda_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sampler library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = synth.headline(seed=7 + rank, rows=ROWS, vocab=VOCAB)
    sampler = pagoda_b200.Sampler(device=local_rank, max_rows=ROWS, max_vocab=VOCAB, max_history=1024)

    def dev_t(a, dt=None):
        t = torch.from_numpy(np.ascontiguousarray(a))
        if dt is not None:
            t = t.view(dt)
        return t.to(dev)

    # input pools larger than L2 (3 x 155.6 MB): pool p is pool 0 rolled along the vocabulary axis
    n_pools = 3
    base = dev_t(w.logits)
    pools = [base] + [torch.roll(base, shifts=1009 * p, dims=1).contiguous() for p in range(1, n_pools)]
    common = dict(temperature=dev_t(w.temperature), top_k=dev_t(w.top_k.view(np.int32)), top_p=dev_t(w.top_p),
                  frequency_penalty=dev_t(w.frequency_penalty), presence_penalty=dev_t(w.presence_penalty),
                  repetition_penalty=dev_t(w.repetition_penalty), hist_offsets=dev_t(w.hist_offsets.view(np.int32)),
                  hist_ids=dev_t(w.hist_ids.view(np.int32)), uniform=dev_t(w.uniform))
    token = torch.zeros(ROWS, dtype=torch.int32, device=dev)
    status = torch.full((ROWS,), -1, dtype=torch.int32, device=dev)
    descs = [sampler.make_device_desc(p, token, status, **common) for p in pools]
    # time on the stream the kernels are launched on: the handle's own stream
    ext = torch.cuda.ExternalStream(sampler.stream_ptr, device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(ext)

    def step(i):
        sampler.launch_device(descs[i % n_pools], None)

    clocks = ClockSampler(local_rank) if rank == 0 else None
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    # parity of the benchmarked path on a few rows of pool 0, before timing
    step(0)
    torch.cuda.synchronize()
    assert (status.cpu().numpy() == 0).all(), "rows failed"
    if args.phases:
        sampler.read_phase_timers()       # clear what the warm-up left
        n = 6
        for i in range(n):
            step(i)
        t = sampler.read_phase_timers()
        act = t[t.sum(1) > 0]
        names = {12: "row barrier", 11: "parameters, copy issue, history table", 0: "slice check", 14: "  of which waiting for the copy",
                 1: "penalties", 2: "argmax", 3: "exchange 1", 13: "exchange 1 read", 15: "warp maxima ranked", 4: "bound -> cut",
                 5: "candidates + exponent pass", 6: "scan", 7: "exchange 2", 8: "fold", 9: "exchange 3 + refinement"}
        per_step = act.mean(0) / n
        print(f"{len(act)} CTAs active, {ROWS} rows per step; cycles per step and CTA (thread 0), mean over CTAs:", file=sys.stderr)
        for slot, name in names.items():
            print(f"  {name:42s} {per_step[slot]:9.0f}", file=sys.stderr)
        return
    if rank == 0:
        from oracle import oracle
        chk = 4
        sub = w.head(chk)
        want = oracle.sample_batch(sub.logits_f32(), n_threads=chk, **sub.oracle_kwargs())
        assert (token[:chk].cpu().numpy().view(np.uint32) == want["token"]).all(), "parity check failed"

    launches0 = sampler.counters()["kernel_launches"]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record(ext)
    for i in range(args.steps):
        step(i)
    e1.record(ext)
    torch.cuda.synchronize()
    t_wall1 = time.time()
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clock_info = clocks.stop(t_wall0, t_wall1) if clocks else None
    launches = sampler.counters()["kernel_launches"] - launches0

    # end to end through the host-memory side of the C ABI: pinned host logits in, tokens out
    pinned = torch.from_numpy(w.logits).pin_memory()
    host_logits = pinned.numpy()
    kw = w.sampler_kwargs()
    for _ in range(2):
        sampler.sample_batch(host_logits, **kw)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        res = sampler.sample_batch(host_logits, **kw)
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    assert (res.status == 0).all()
    h2d = int(w.logits.nbytes + ROWS * 4 * 8 + w.hist_offsets.nbytes + w.hist_ids.nbytes)
    d2h = int(ROWS * (4 + 4 + 1))

    if rank != 0:
        sampler.close()
        if world > 1:
            dist.destroy_process_group()
        return

    value = args.steps * ROWS * world / (ms * 1e-3)
    peak, peak_src = measured_peak()
    alg_bytes = w.algorithmic_bytes()
    # the step is four launches (fused row kernel ~94 % of the time, small-row finish kernel, and beside
    # it the large-row finish kernel and the work-list pass); dividing by the whole step keeps the
    # figure conservative for the dominant kernel
    per_launch_s = ms * 1e-3 / args.steps
    achieved = alg_bytes / per_launch_s / 1e9
    tpr = ncu_traffic_per_row()
    line = {
        "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "headline: B=256 V=151936 f32 per GPU, T=0.7 top-k 50 top-p 0.9 freq 0.2 pres 0.1, "
                               "512-id histories, one uniform per row",
                   "l2": f"{n_pools} input pools of {base.numel() * 4 / 1e6:.0f} MB rotated (larger than L2)",
                   "rows_per_gpu": ROWS, "vocab": VOCAB},
        "clocks": clock_info, "gpu_launches": int(launches),
        "e2e": {"value": args.e2e_steps * ROWS * world / e2e_s, "unit": "rows/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": args.e2e_steps},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if tpr is None else tpr * ROWS, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg_bytes,
                     "kernel": "fused_row_kernel (time of the whole step: + finish kernels + work-list pass)",
                     "launch_us": per_launch_s * 1e6},
    }
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        sample_rows = ROWS
        rps, dt = cpu_port_rows_per_s(w, sample_rows, threads)
        rps1, dt1 = cpu_port_rows_per_s(w, 4, 1)
        line["cpu_baseline"] = {"value": rps, "unit": "rows/s", "cores": threads, "kind": "port",
                                "sample": f"first {sample_rows} rows of the same workload over {threads} threads "
                                          f"({dt:.2f} s); single thread, as the reference runs it: {rps1:.1f} rows/s"}
    print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
