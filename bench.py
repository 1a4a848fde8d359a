#!/usr/bin/env python
"""Headline benchmark: sampled rows/s at B=256, V=151936 (f32 logits, temperature 0.7, top-k 50,
top-p 0.9, frequency/presence penalties over 512-id histories -- the per-row recipe of the
batched stochastic configuration, at the batch size the metric is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the logits -> token chain over one batch.  With N > 1 (one process per
GPU under torchrun) every rank samples its own 256-row batch -- rows are independent, so there
is no data-path collective -- and the value is all ranks' rows over the slowest rank's time.
Prints ONE JSON line on rank 0.  Beside the headline keys the line carries
  "configs"  (N = 1) the four single-GPU benchmark configurations at full size: time per step,
             algorithmic bytes, fraction of the HBM peak, and a parity bit against the CPU oracle;
  "strong"   one fixed B=256 batch split by rows over the N ranks (headline recipe and the
             heterogeneous bf16 configuration), with the efficiency against this run's 1-GPU time;
  "tp"       the vocabulary-sharded configuration at its 1024 rows over the N ranks: records
             exchanged by an NCCL all-gather and by peer stores, time per step, parity on rank 0.
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


HEADLINE_DESC = ("headline: B=256 V=151936 f32 per GPU, T=0.7 top-k 50 top-p 0.9 freq 0.2 pres 0.1, "
                 "512-id histories, one uniform per row")
TOL = 1e-5


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
    Rust and no Rust toolchain exists here, so its own build cannot run).  One step = the whole
    256-row batch of the headline workload."""
    if rank != 0:
        return
    from pagoda_b200 import synth
    threads = os.cpu_count() or 1
    w = synth.headline(rows=ROWS)
    for _ in range(max(min(args.warmup, 2), 1)):
        cpu_port_rows_per_s(w, ROWS, threads)
    t_total, rows_total = 0.0, 0
    for _ in range(args.steps):
        rps, dt = cpu_port_rows_per_s(w, ROWS, threads)
        t_total += dt; rows_total += ROWS
    value = rows_total / t_total
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": HEADLINE_DESC, "rows_per_gpu": ROWS, "vocab": VOCAB,
                       "sample": f"the whole {ROWS}-row batch per step"},
            "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                             "sample": f"all {ROWS} rows of the headline workload per step, rows spread over "
                                       f"{threads} host threads"},
            "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# device-resident workloads

class DeviceWorkload:
    """A workload with every array on the device, as rotating input pools larger than L2 (pool p is
    pool 0 rolled along the vocabulary axis), ready to be launched step after step."""

    def __init__(self, torch, sampler, w, dev, rows=None, min_pool_bytes=400e6, diagnostics=False):
        lo, hi = rows if rows is not None else (0, w.rows)
        self.w, self.lo, self.hi, self.sampler = w, lo, hi, sampler
        n = hi - lo

        def dev_t(a, dt=None):
            t = torch.from_numpy(np.ascontiguousarray(a))
            if dt is not None:
                t = t.view(dt)
            return t.to(dev)

        if w.is_bf16:
            base = dev_t(w.logits[lo:hi].view(np.int16)).view(torch.bfloat16)
        else:
            base = dev_t(w.logits[lo:hi])
        row_bytes = max(1, base.numel() * base.element_size())
        self.n_pools = int(min(512, max(2, -(-int(min_pool_bytes) // row_bytes))))
        self.pools = [base] + [torch.roll(base, shifts=1009 * p, dims=1).contiguous() for p in range(1, self.n_pools)]
        self.pool_bytes = row_bytes
        self.table_id = None
        common = dict(temperature=dev_t(w.temperature[lo:hi]), top_k=dev_t(w.top_k[lo:hi].view(np.int32)),
                      top_p=dev_t(w.top_p[lo:hi]), frequency_penalty=dev_t(w.frequency_penalty[lo:hi]),
                      presence_penalty=dev_t(w.presence_penalty[lo:hi]),
                      repetition_penalty=dev_t(w.repetition_penalty[lo:hi]), uniform=dev_t(w.uniform[lo:hi]),
                      eos_token_id=w.eos_token_id)
        if w.hist_offsets is not None:
            # offsets stay absolute: the slice of the offsets array points into the whole id array
            common.update(hist_offsets=dev_t(w.hist_offsets[lo:hi + 1].view(np.int32)), hist_ids=dev_t(w.hist_ids.view(np.int32)))
        if w.mask_state is not None:
            self.table_id = sampler.upload_mask_table(w.mask_words, w.state_flags)
            ms = w.mask_state[lo:hi]
            common.update(mask_table=dev_t(np.where(ms >= 0, self.table_id, -1).astype(np.int32)),
                          mask_state=dev_t(ms.astype(np.int32)))
        self.token = torch.zeros(n, dtype=torch.int32, device=dev)
        self.status = torch.full((n,), -1, dtype=torch.int32, device=dev)
        self.descs = [sampler.make_device_desc(p, self.token, self.status, **common) for p in self.pools]

    def step(self, i):
        self.sampler.launch_device(self.descs[i % self.n_pools], None)

    def close(self):
        if self.table_id is not None:
            self.sampler.free_mask_table(self.table_id)
            self.table_id = None


def timed_steps(torch, dist, world, ext, dev, step, steps, warmup):
    """ms for `steps` calls of step(i): CUDA events on the launching stream, barrier on both sides, max over ranks."""
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(ext)
    for i in range(steps):
        step(i)
    e1.record(ext)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def parity_bit(w, token, status, rows, threads):
    """Tokens of the first `rows` rows of pool 0 against the CPU oracle.  Greedy tokens, statuses and every
    stochastic row whose top-p / CDF decision is further than TOL from its boundary must agree."""
    from oracle import oracle
    sub = w.head(rows)
    want = oracle.sample_batch(sub.logits_f32(), n_threads=threads, **sub.oracle_kwargs())
    clear = (want["margin_p"] > TOL) & (want["margin_cdf"] > TOL)
    ok = bool((status[:rows] == want["status"]).all() and (token[:rows].view(np.uint32)[clear] == want["token"][clear]).all())
    return ok, int(rows), int((~clear).sum())


def bench_configs(torch, dist, sampler_of, ext_of, dev, peak, threads):
    """The four single-GPU configurations at their full sizes (N = 1 only)."""
    from pagoda_b200 import synth
    out = {}
    for key, make, check_rows, steps in (("1", synth.config1, 1, 400), ("2", synth.config2, 64, 200),
                                         ("3", synth.config3, 64, 200), ("4", synth.config4, 32, 100)):
        w = make()
        sampler = sampler_of(w)
        dw = DeviceWorkload(torch, sampler, w, dev)
        ext = ext_of(sampler)
        try:
            dw.step(0)
            torch.cuda.synchronize()
            ok, checked, skipped = parity_bit(w, dw.token.cpu().numpy(), dw.status.cpu().numpy(), check_rows, threads)
            ms = timed_steps(torch, dist, 1, ext, dev, dw.step, steps, 10) / steps
            alg = w.algorithmic_bytes()
            out[key] = {"workload": w.name, "rows": w.rows, "vocab": w.vocab, "dtype": "bf16" if w.is_bf16 else "f32",
                        "ms_per_step": ms, "rows_per_s": w.rows / (ms * 1e-3), "algorithmic_bytes": alg,
                        "achieved_gbs": alg / (ms * 1e-3) / 1e9, "frac": alg / (ms * 1e-3) / 1e9 / peak,
                        "parity": ok, "parity_rows": checked, "parity_rows_on_a_boundary": skipped,
                        "pools": dw.n_pools, "steps": steps}
        finally:
            dw.close()
    return out


def bench_strong(torch, dist, world, rank, sampler_of, ext_of, dev, weak_ms_per_step, threads):
    """One fixed 256-row batch split by rows over the ranks (no data-path collective): the headline recipe and the
    heterogeneous bf16 configuration.  Efficiency = (1-GPU time of the same batch) / (N x this time); the 1-GPU
    time of the headline batch is this run's own weak-scaling step (every rank ran all 256 rows)."""
    from pagoda_b200 import synth
    from pagoda_b200.parallel import row_shard
    out = {}
    for key, w, steps in (("headline", synth.headline(seed=7), 200), ("config4", synth.config4(), 100)):
        sampler = sampler_of(w)
        ext = ext_of(sampler)
        lo, hi = row_shard(w.rows, world, rank)
        dw = DeviceWorkload(torch, sampler, w, dev, rows=(lo, hi))
        one = None
        try:
            ms = timed_steps(torch, dist, world, ext, dev, dw.step, steps, 10) / steps
            if key == "headline":
                one = weak_ms_per_step
            elif world > 1 and rank == 0:   # the whole batch on this rank alone, for the efficiency
                full = DeviceWorkload(torch, sampler, w, dev)
                one = timed_steps(torch, dist, 1, ext, dev, full.step, steps, 10) / steps
                full.close()
            elif world == 1:
                one = ms
            if world > 1:   # timed_steps' collectives: keep the ranks together while rank 0 measures alone
                dist.barrier()
            rec = {"rows_total": w.rows, "rows_per_rank": hi - lo, "ms_per_step": ms, "rows_per_s": w.rows / (ms * 1e-3),
                   "steps": steps}
            if one is not None:
                rec["one_gpu_ms_per_step"] = one
                rec["efficiency"] = one / (world * ms)
            out[key] = rec
        finally:
            dw.close()
    return out


def bench_tp(torch, dist, world, rank, dev, threads, steps=50):
    """Vocabulary-sharded configuration at its full 1024 rows.  N >= 2: every rank holds V / N columns, emits its
    records, and the records travel (a) by an NCCL all-gather between the two kernels, (b) by stores into the peers'
    gather buffers and a flag wait in the merge kernel.  N = 1: the eight shards of an 8-way split are emitted one
    after the other on this GPU (no exchange), which gives the per-shard emit time and the merge time."""
    import pagoda_b200
    from pagoda_b200 import synth
    from pagoda_b200.parallel import PeerExchange, all_gather_records, column_shard
    w = synth.config5()
    rows, vocab, cand = w.rows, w.vocab, 64
    n_shards = world if world > 1 else 8
    sampler = pagoda_b200.Sampler(device=dev.index, max_rows=rows, max_vocab=vocab // n_shards, max_history=16)
    ext = torch.cuda.ExternalStream(sampler.stream_ptr, device=dev)
    torch.cuda.set_stream(ext)
    st = sampler.stream_ptr
    t = torch.from_numpy(w.temperature).to(dev)
    tp_, tu = torch.from_numpy(w.top_p).to(dev), torch.from_numpy(w.uniform).to(dev)
    draft = torch.from_numpy(w.extra["draft"].astype(np.int32)).to(dev)
    seqs, pos = draft.shape
    rec = {"rows": rows, "vocab": vocab, "n_shards": n_shards, "cand": cand, "steps": steps,
           "record_bytes": sampler.tp_record_bytes(cand)}

    outs = sampler.tp_outputs(rows, dev)   # reused by every step: no allocation inside the timed loops

    acc_out = (torch.zeros(seqs, dtype=torch.int32, device=dev), torch.zeros(seqs, dtype=torch.int32, device=dev))

    def finish(out):
        return sampler.draft_accept(out["argmax"].view(seqs, pos), draft, stream_ptr=st, out=acc_out)

    if world > 1:
        lo, hi = column_shard(vocab, world, rank)
        shard0 = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi])).to(dev)
        shards = [shard0, torch.roll(shard0, shifts=1009, dims=1).contiguous()] if shard0.numel() * 4 < 200e6 else [shard0]
        px = PeerExchange(sampler, rows, sampler.tp_record_bytes(cand), dev)
        state = {}

        def step_nccl(i):
            r = sampler.tp_partial(shards[i % len(shards)], vocab, world, rank, cand, temperature=t, stream_ptr=st)
            state["out"] = sampler.tp_merge(all_gather_records(r), vocab, world, rank, cand, temperature=t, top_p=tp_,
                                            uniform=tu, stream_ptr=st, out=outs)
            state["acc"] = finish(state["out"])

        def step_peer(i):
            epoch, par, rec_ptrs, flag_ptrs = px.next_step()
            sampler.tp_partial_push(shards[i % len(shards)], vocab, world, rank, cand, rec_ptrs, flag_ptrs, epoch,
                                    temperature=t, stream_ptr=st)
            state["out"] = sampler.tp_merge_wait(px.buf[par], px.flags[par], epoch, vocab, world, rank, cand, temperature=t,
                                                 top_p=tp_, uniform=tu, stream_ptr=st, out=outs)
            state["acc"] = finish(state["out"])

        step_nccl(0); torch.cuda.synchronize()
        out_nccl = {k: v.cpu().numpy() for k, v in state["out"].items()}
        step_peer(0); torch.cuda.synchronize()
        out_peer = {k: v.cpu().numpy() for k, v in state["out"].items()}
        acc, nxt = (x.cpu().numpy() for x in state["acc"])
        sampler.tp_exchange_status()
        rec["nccl_allgather_us_per_step"] = 1e3 * timed_steps(torch, dist, world, ext, dev, step_nccl, steps, 5) / steps
        rec["peer_store_us_per_step"] = 1e3 * timed_steps(torch, dist, world, ext, dev, step_peer, steps, 5) / steps
        sampler.tp_exchange_status()
        rec["paths_agree"] = bool((out_nccl["token"] == out_peer["token"]).all() and (out_nccl["status"] == out_peer["status"]).all())
        rec["roofline_us_per_gpu"] = rows * (vocab // world) * 4 / 6553e3
        px.close()
        tok, am, status = out_peer["token"], out_peer["argmax"], out_peer["status"]
    else:
        per = vocab // n_shards
        x = torch.from_numpy(w.logits).to(dev)
        views = [x[:, r * per:(r + 1) * per] for r in range(n_shards)]
        recs = torch.empty((n_shards, rows, sampler.tp_record_bytes(cand)), dtype=torch.uint8, device=dev)
        state = {}

        def emit(i):
            sampler.tp_partial(views[i % n_shards], vocab, n_shards, i % n_shards, cand, temperature=t, records=recs[i % n_shards],
                               stream_ptr=st)

        def merge(i):
            state["out"] = sampler.tp_merge(recs, vocab, n_shards, 0, cand, temperature=t, top_p=tp_, uniform=tu, stream_ptr=st,
                                            out=outs)
            state["acc"] = finish(state["out"])

        for r in range(n_shards):
            emit(r)
        merge(0)
        torch.cuda.synchronize()
        rec["emit_us_per_shard"] = 1e3 * timed_steps(torch, dist, 1, ext, dev, emit, 8 * 10, 8) / (8 * 10)
        rec["merge_us"] = 1e3 * timed_steps(torch, dist, 1, ext, dev, merge, steps, 5) / steps
        rec["exchange"] = "none: one GPU emits the 8 shards of an 8-way split in turn"
        rec["roofline_us_per_shard"] = rows * per * 4 / 6553e3
        tok, am, status = (state["out"][k].cpu().numpy() for k in ("token", "argmax", "status"))
        acc, nxt = (v.cpu().numpy() for v in state["acc"])
    if rank == 0:
        from oracle import oracle
        check = 48
        ok, skipped = True, 0
        for r in range(check):
            want = oracle.tp_sample_row(w.logits[r], n_shards, cand, float(w.temperature[r]), float(w.top_p[r]), float(w.uniform[r]))
            ok &= bool(status[r] == want.status and am[r] == want.argmax)
            if want.margin > TOL:
                ok &= bool(tok[r] == want.token)
            else:
                skipped += 1
        for s in range(check // pos):
            na, nx = oracle.draft_accept(am[pos * s:pos * s + pos].astype(np.uint32), w.extra["draft"][s])
            ok &= bool(acc[s] == na and nxt[s] == nx)
        rec.update(parity=bool(ok), parity_rows=check, parity_rows_on_a_boundary=skipped)
    torch.cuda.synchronize()
    sampler.close()
    return rec


def run_sweep(args):
    """Diagnostics, not the benchmark contract: plain text lines.  `--sweep variants`: the 256-row headline batch as
    greedy rows without penalties (the first pass alone), as stochastic rows without penalties, and as it is.
    `--sweep rows`: the headline recipe at other batch sizes.  With --sweep-steps 1 every case launches exactly once
    (no warm-up), which is the form to put under ncu for instruction counts."""
    import copy
    import torch
    import pagoda_b200
    from pagoda_b200 import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    n = args.sweep_steps
    cases = []
    if args.sweep == "variants":
        w = synth.headline(seed=7, rows=ROWS, vocab=VOCAB)
        g = copy.copy(w)
        g.temperature = np.zeros_like(w.temperature)
        g.hist_offsets = g.hist_ids = None
        st = copy.copy(w)
        st.hist_offsets = st.hist_ids = None
        cases = [("greedy rows, no penalties", g), ("stochastic rows, no penalties", st), ("headline rows", w)]
    else:
        for rows in (1, 8, 32, 64, 128, 148, 256, 296, 592, 1024, 2048):
            cases.append((f"{rows} rows", synth.headline(seed=7, rows=rows, vocab=VOCAB)))
    for name, w in cases:
        sampler = pagoda_b200.Sampler(device=0, max_rows=w.rows, max_vocab=VOCAB, max_history=1024)
        ext = torch.cuda.ExternalStream(sampler.stream_ptr, device=dev)
        dw = DeviceWorkload(torch, sampler, w, dev, min_pool_bytes=400e6 if w.rows <= 512 else 1)
        ms = timed_steps(torch, None, 1, ext, dev, dw.step, n, 0 if n == 1 else 20) / n
        print(f"{name:32s} {ms * 1e3:9.1f} us/step {ms * 1e6 / w.rows:9.1f} ns/row "
              f"{w.algorithmic_bytes() / (ms * 1e-3) / 1e9:8.0f} GB/s algorithmic", flush=True)
        dw.close(); sampler.close()
        del dw, sampler
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true", help="skip the configs / strong / tp records")
    ap.add_argument("--sweep", choices=["variants", "rows"], help="diagnostic tables (plain text), see run_sweep")
    ap.add_argument("--sweep-steps", type=int, default=100)
    ap.add_argument("--phases", action="store_true",
                    help="print the row kernel's in-kernel phase timers (cycles per step and CTA) and exit")
    args = ap.parse_args()
    if args.phases:
        os.environ["PGS_PROFILE"] = "1"   # read when the sampler is created

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.sweep:
        run_sweep(args)
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
    threads = os.cpu_count() or 1

    w = synth.headline(seed=7 + rank, rows=ROWS, vocab=VOCAB)
    sampler = pagoda_b200.Sampler(device=local_rank, max_rows=ROWS, max_vocab=VOCAB, max_history=1024)
    # time on the stream the kernels are launched on: the handle's own stream
    ext = torch.cuda.ExternalStream(sampler.stream_ptr, device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(ext)
    dw = DeviceWorkload(torch, sampler, w, dev)
    step = dw.step

    clocks = ClockSampler(local_rank) if rank == 0 else None
    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
    torch.cuda.synchronize()
    # parity of the benchmarked path, all rows of pool 0, before timing
    step(0)
    torch.cuda.synchronize()
    status_np, token_np = dw.status.cpu().numpy(), dw.token.cpu().numpy()
    assert (status_np == 0).all(), "rows failed"
    if args.phases:
        sampler.read_phase_timers()       # clear what the warm-up left
        n = 6
        for i in range(n):
            step(i)
        t = sampler.read_phase_timers()
        act = t[t.sum(1) > 0]
        names = {0: "gate + row barrier", 1: "history indexed", 2: "pass 1 (HBM)", 6: "reductions + argmax", 7: "top-k bound",
                 3: "fold table", 4: "pass 2 (L2)", 5: "finish"}
        per_step = act.mean(0) / n
        print(f"{len(act)} CTAs active, {ROWS} rows per step; cycles per step and CTA (thread 0), mean over CTAs:", file=sys.stderr)
        for slot, name in names.items():
            print(f"  {name:42s} {per_step[slot]:9.0f}", file=sys.stderr)
        return
    parity = None
    if rank == 0:
        ok, checked, skipped = parity_bit(w, token_np, status_np, ROWS, threads)
        assert ok, "parity check against the CPU oracle failed"
        parity = {"rows": checked, "rows_on_a_boundary": skipped, "ok": ok}

    # untimed steps until the GPU has been busy long enough to have left its idle clocks (a 20-step timed region is
    # under 2 ms, and the oracle check above left the GPU idle for a while), directly in front of the timed region
    if world > 1:
        dist.barrier()   # (rank 0 comes out of its oracle check: everybody ramps up together)
    ramp, t_ramp = 0, time.perf_counter()
    while time.perf_counter() - t_ramp < 0.25:
        for i in range(50):
            step(ramp + i)
        torch.cuda.synchronize()
        ramp += 50
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
    del pinned, host_logits

    peak, peak_src = measured_peak()
    extra = {}
    if not args.headline_only:
        big = {}

        def sampler_of(wl):   # the headline handle serves what fits it; the bf16 configuration gets its own
            if wl.vocab <= VOCAB and (wl.hist_offsets is None or int(np.diff(wl.hist_offsets).max()) <= 1024):
                return sampler
            if "s" not in big:
                big["s"] = pagoda_b200.Sampler(device=local_rank, max_rows=ROWS, max_vocab=256000, max_history=2048)
            return big["s"]

        def ext_of(s):
            return torch.cuda.ExternalStream(s.stream_ptr, device=dev)

        dw.close()
        del dw
        torch.cuda.empty_cache()
        if world == 1:
            extra["configs"] = bench_configs(torch, dist, sampler_of, ext_of, dev, peak, threads)
        extra["strong"] = bench_strong(torch, dist, world, rank, sampler_of, ext_of, dev, ms / args.steps, threads)
        if "s" in big:
            big["s"].close()
        torch.cuda.empty_cache()
        extra["tp"] = bench_tp(torch, dist, world, rank, dev, threads)

    if rank != 0:
        sampler.close()
        if world > 1:
            dist.destroy_process_group()
        return

    value = args.steps * ROWS * world / (ms * 1e-3)
    alg_bytes = w.algorithmic_bytes()
    # The step is three launches: the streaming row kernel (all of the time but a few microseconds) and the two
    # list passes behind it, which find their lists empty on this workload.  Dividing by the whole step keeps the
    # figure conservative for the row kernel.
    per_launch_s = ms * 1e-3 / args.steps
    achieved = alg_bytes / per_launch_s / 1e9
    tpr = ncu_traffic_per_row()
    line = {
        "metric": METRIC, "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": HEADLINE_DESC,
                   "l2": f"{dw_pools(ROWS, VOCAB)} input pools of {ROWS * VOCAB * 4 / 1e6:.0f} MB rotated (larger than L2)",
                   "rows_per_gpu": ROWS, "vocab": VOCAB,
                   "warmup_steps_run": warm + ramp + 1,
                   "parity_before_timing": parity},
        "clocks": clock_info, "gpu_launches": int(launches),
        "e2e": {"value": args.e2e_steps * ROWS * world / e2e_s, "unit": "rows/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": args.e2e_steps},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None if tpr is None else tpr * ROWS, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": alg_bytes,
                     "kernel": "stream_row_kernel (time of the whole step: + the finish and work-list passes)",
                     "launch_us": per_launch_s * 1e6},
    }
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        rps, dt = cpu_port_rows_per_s(w, ROWS, threads)
        rps1, dt1 = cpu_port_rows_per_s(w, 4, 1)
        line["cpu_baseline"] = {"value": rps, "unit": "rows/s", "cores": threads, "kind": "port",
                                "sample": f"all {ROWS} rows of the same workload over {threads} threads "
                                          f"({dt:.2f} s); single thread, as the reference runs it: {rps1:.1f} rows/s"}
    print(json.dumps(line), flush=True)
    sampler.close()
    if world > 1:
        dist.destroy_process_group()


def dw_pools(rows, vocab):
    return max(2, -(-int(400e6) // (rows * vocab * 4)))


if __name__ == "__main__":
    main()
