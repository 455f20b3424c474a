#!/usr/bin/env python
"""Throughput of the logits -> token hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the sampling path over one batch of B = 256 logits
rows (V = 128256, fp32) that already sit in HBM: the stream kernel and the two
finishing kernels behind it. The workload is the sampler configuration of the
single-row reference case at the metric's batch shape: rows ~ N(0, 2.5^2) with
8 ids per row boosted by +12, temperature 0.8, top_k 40, top_p 0.95 (top_k
takes precedence, as in the reference dispatch), repetition penalty 1.1 over a
64-token history, one xorshift64* draw per row. Inputs rotate over 8 distinct
logits sets (1.05 GB, far beyond the 126 MB L2). Both arms draw their rows from
the same numpy generator, so the reference arm samples the very bytes of the
first rows of input set 0.

Prints ONE JSON line. `value` is device-resident rows/s over all ranks (max
time over ranks); `e2e` is the same work through the session batcher with HOST
logits (pinned), host->device copies and the token read-back inside the timed
region, next to the host link's own copy rate; `roofline` compares algorithmic
bytes / measured step time with the measured HBM copy peak; `cpu_baseline`
times the reference's own CPU sampler (oracle/_ref, release flags) on a bounded
sample of the same rows; `configs` carries the other configurations of the
reference's table (device-resident time, HBM fraction, token parity with the
CPU checker on a row sample); with --gpus N > 1 `vocab_shards` is the
vocabulary-sharded variant of the 4096-row configuration (per-shard top-k ->
NCCL all-gather -> merge + draw, token ids compared with the unsharded launch
on every rank) and `row_shards_strong` the same 4096 rows split N ways.
With --impl reference the CPU sampler alone is timed (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

B, V, H = 256, 128256, 64
T, TOP_K, TOP_P, REP = 0.8, 40, 0.95, 1.1
N_SETS = 8
SEED = 1234
# algorithmic bytes per row: logits once + history ids + generator state in/out + token out
BYTES_PER_ROW = 4 * V + 4 * H + 16 + 4
# sample_stream_kernel alone: every session of the workload samples top-k 40, which the caller (here as in the
# session batcher) tells the launch with finish_hint = GREEDY_TOPK; the 256 rows are dealt out as whole rows, so the
# stream kernel's thread blocks finish them from their own candidate lists and no finishing kernel is launched.
# Without the hint the general finishing kernel runs behind it -- the "..., no hint" entries of `modes`
KERNELS_PER_STEP = 1
WORKLOAD = ("B=256 rows x V=128256 fp32 logits ~ N(0,2.5^2) with 8 ids/row +12; temperature 0.8, top_k 40, "
            "top_p 0.95 (top_k precedence), repetition penalty 1.1 over 64-token history, 1 draw/row, seed 1234")


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def ncu_traffic():
    """DRAM bytes of one step of this workload from the committed ncu summary (a bench run cannot measure them), and
    whether the kernel sources are still the ones the capture was taken with."""
    import hashlib
    p = ROOT / "profiles" / "traffic.json"
    try:
        d = json.loads(p.read_text())
        h = hashlib.sha256()
        for f in d["kernel_sources"]:
            h.update((ROOT / f).read_bytes())
        same = h.hexdigest() == d["kernel_sources_sha256"]
        return float(d["dram_bytes_per_step"]), d.get("source", p.name) + ("" if same else " [kernel sources changed since that capture]")
    except Exception:
        return None, "no ncu capture committed for this build"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons every 100 ms while the GPU works."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, windows):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        inside = [r for (t, r) in self.rows if any(a <= t <= b for a, b in windows)] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def gen_set(i: int, rank: int = 0, rows: int = B):
    """Logits set i of a rank: the same bytes in either arm."""
    import numpy as np
    rng = np.random.default_rng(SEED + 1000 * rank + i)
    x = rng.standard_normal((rows, V), dtype=np.float32) * np.float32(2.5)
    idx = rng.integers(0, V, (rows, 8))
    np.add.at(x, (np.arange(rows)[:, None], idx), np.float32(12.0))
    return x


def gen_hist(rank: int = 0, rows: int = B):
    import numpy as np
    return np.random.default_rng(SEED + 1000 * rank + 500).integers(0, V, (rows, H), dtype=np.int32)


def cpu_reference_rows(x_pen, states, threads):
    """The reference's CPU sampler on rows that already carry the penalties (the reference has none: they are
    applied by the checker before the clock starts), all host threads, one row per task."""
    import oracle
    ref = oracle.ref_release or oracle.ref
    if ref is not None:
        return ref.sample(x_pen, T, TOP_K, TOP_P, states, nthreads=threads), "reference"
    return oracle.port.sample_batch(x_pen, T, TOP_K, TOP_P, states, nthreads=threads), "port"


def penalised(x, hist):
    import numpy as np
    import oracle
    return np.stack([oracle.port.apply_penalties(x[r], hist[r], REP) for r in range(x.shape[0])])


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the path, timed alone."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from helpers import independent_states

    threads = os.cpu_count() or 1
    rows_per_step = min(B, max(64, 4 * threads))
    x = gen_set(0)[:rows_per_step]
    hist = gen_hist()[:rows_per_step]
    st = independent_states(oracle.port, SEED, rows_per_step)
    x_pen = penalised(x, hist)  # outside the timed region
    for _ in range(args.warmup):
        cpu_reference_rows(x_pen, st, threads)
    t0 = time.perf_counter()
    kind = "port"
    for _ in range(args.steps):
        _, kind = cpu_reference_rows(x_pen, st, threads)
    dt = time.perf_counter() - t0
    value = rows_per_step * args.steps / dt
    sample = (f"the first {rows_per_step} rows of input set 0 (the bytes the GPU arm samples) per step, {threads} host threads, "
              "one row per task; penalties applied before the clock starts")
    print(json.dumps({
        "impl": "reference", "metric": "sampled rows/s at B=256,V=128256 fp32", "value": value, "unit": "rows/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": rows_per_step, "penalties_in_timed_region": False},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-modes", action="store_true", help="skip the informational per-mode timings")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-logits leg (for profiler captures; the line then has no e2e value)")
    ap.add_argument("--no-configs", action="store_true", help="skip the other configurations and the multi-GPU legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    import oracle
    from geistlib_b200 import LIB_PATH, api
    from helpers import gumbel_logits, histories, independent_states, normal_logits, per_seq, seq_states, to_dev, u64_from_dev, u64_to_dev

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local) if rank == 0 else None
    port = oracle.port
    peak, peak_kind = measured_peak()

    ctx = api.Context(local)
    # everything timed runs on one explicit stream; events are recorded on the same stream
    work_stream = torch.cuda.Stream(dev)
    torch.cuda.set_stream(work_stream)
    sets_np0 = gen_set(0, rank)
    sets = [torch.from_numpy(sets_np0).to(dev)] + [torch.from_numpy(gen_set(i, rank)).to(dev) for i in range(1, N_SETS)]
    hist_np = gen_hist(rank)
    hist = torch.from_numpy(hist_np).to(dev)
    n_seq = B
    dT = torch.full((n_seq,), T, device=dev)
    dK = torch.full((n_seq,), TOP_K, device=dev, dtype=torch.int32)
    dP = torch.full((n_seq,), TOP_P, device=dev)
    dRep = torch.full((n_seq,), REP, device=dev)
    dHl = torch.full((n_seq,), H, device=dev, dtype=torch.int32)
    states = independent_states(port, SEED + 1000 * rank, n_seq)
    rng_a = u64_to_dev(states)
    stream = torch.cuda.current_stream(dev).cuda_stream

    # one prepared descriptor per input set; generator state ping-pongs a -> b -> a
    descs = []
    rng_b = None
    for i, x in enumerate(sets):
        src = rng_a if i % 2 == 0 else rng_b
        o = ctx.sample_batch(x, dT, dK, dP, src, rep=dRep, history=hist, history_len=dHl, launch=False, finish_hint=api.FINISH_GREEDY_TOPK)
        if i % 2 == 0:
            rng_b = o["rng_state"]
        else:
            o["_desc"].rng_out = rng_a.data_ptr()
        descs.append(o)

    def all_barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def timed_loop(launch, steps, warmup, collective=True):
        barrier = all_barrier if collective else (lambda: torch.cuda.synchronize(dev))
        for i in range(warmup):
            launch(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0 = time.time()
        e0.record()
        for i in range(steps):
            launch(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1 and collective:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, (w0, time.time())

    windows = []
    ms, w = timed_loop(lambda i: ctx.relaunch(descs[i % N_SETS], stream), args.steps, args.warmup)
    windows.append(w)
    bad = int((descs[0]["status"] & (api.ROW_INVALID | api.ROW_RETRY)).ne(0).sum().item())
    slow = int((descs[0]["status"] & api.ROW_SLOW_PATH).ne(0).sum().item())
    rows_per_s = world * B * args.steps / (ms * 1e-3)
    per_launch_s = ms * 1e-3 / args.steps
    achieved = B * BYTES_PER_ROW / per_launch_s / 1e9

    # ---- end to end: host logits -> session batcher -> host tokens
    e2e = None
    if not args.no_e2e:
        bt = api.Batcher(ctx, V, B, max_history=H + 8)
        sessions = [bt.open(temperature=T, top_p=TOP_P, top_k=TOP_K, seed=SEED + s, rep=REP) for s in range(B)]
        for s in sessions:
            bt.push_history(s, hist_np[s])
        host_sets = [torch.empty(B, V, dtype=torch.float32, pin_memory=True).copy_(sets[i]) for i in range(2)]
        e2e_steps = max(3, min(args.steps, 40))
        e2e_tok = []

        def e2e_launch(i):
            e2e_tok.append(bt.step(sessions, host_sets[i % 2], append_history=False))

        ms_e2e, w = timed_loop(e2e_launch, e2e_steps, 3)
        windows.append(w)
        e2e_rows_per_s = world * B * e2e_steps / (ms_e2e * 1e-3)
        # what the host link alone gives for the same bytes, all ranks at once: plain pinned -> device copies
        dst = torch.empty(B, V, dtype=torch.float32, device=dev)

        def link_launch(i):
            h = host_sets[i % 2]
            for c in range(0, B, 32):  # the batcher's chunking
                dst[c:c + 32].copy_(h[c:c + 32], non_blocking=True)

        ms_link, w = timed_loop(link_launch, e2e_steps, 3)
        host_link_gbs = B * V * 4 * e2e_steps / (ms_link * 1e-3) / 1e9  # per rank, while all ranks copy
        e2e_gbs = B * V * 4 * e2e_steps / (ms_e2e * 1e-3) / 1e9
        e2e = {"value": e2e_rows_per_s, "unit": "rows/s", "h2d_bytes_per_step": B * V * 4 + B * 4,
               "d2h_bytes_per_step": 2 * B * 4, "steps": e2e_steps, "ms_per_step": ms_e2e / e2e_steps,
               "host_link_gbs": host_link_gbs, "e2e_gbs": e2e_gbs, "e2e_frac_of_link": e2e_gbs / host_link_gbs,
               "link_note": "plain pinned->device copies of the same bytes in the same 32-row chunks, all ranks at once, per rank"}

    def time_desc_list(ds, steps, collective=True):
        m, ww = timed_loop(lambda i: ctx.relaunch(ds[i % len(ds)], stream), steps, 8, collective)
        windows.append(ww)
        return m * 1e-3 / steps

    # ---- informational: other modes on the same shape (device-resident)
    modes = {}
    keep = []
    if not args.no_modes:
        def mode(name, t, k, p, pen, hint=0):
            kw = dict(rep=dRep, history=hist, history_len=dHl) if pen else {}
            kw["finish_hint"] = hint
            mt = torch.full((n_seq,), t, device=dev)
            mk = torch.full((n_seq,), k, device=dev, dtype=torch.int32)
            mp = torch.full((n_seq,), p, device=dev)
            keep.extend([mt, mk, mp])
            ds = [ctx.sample_batch(x, mt, mk, mp, rng_a, launch=False, **kw) for x in sets]
            sec = time_desc_list(ds, max(8, min(args.steps, 400)))
            st = ds[0]["status"]
            modes[name] = {"rows_per_s": world * B / sec, "us_per_launch": sec * 1e6,
                           "hbm_frac": B * (4 * V + 20 + (4 * H if pen else 0)) / sec / 1e9 / peak,
                           "rows_on_slow_path": int((st & api.ROW_SLOW_PATH).ne(0).sum().item())}
        # every mode as the session batcher launches it (the batcher derives the finishing hint from its sessions'
        # sampler settings), and the same launch without a hint (what a bare sample_batch call without one gets)
        HINTS = {api.FINISH_AUTO: "AUTO", api.FINISH_GREEDY: "GREEDY", api.FINISH_GREEDY_TOPK: "GREEDY_TOPK", api.FINISH_GENERAL: "GENERAL"}
        for name, (t, k, p, pen, hint) in {
                "greedy": (0.0, 0, 1.0, False, api.FINISH_GREEDY),
                "greedy+penalties": (0.0, 0, 1.0, True, api.FINISH_GREEDY),
                "top_k40": (T, TOP_K, 1.0, False, api.FINISH_GREEDY_TOPK),
                "top_k40+penalties (the headline)": (T, TOP_K, TOP_P, True, api.FINISH_GREEDY_TOPK),
                "temperature": (T, 0, 1.0, False, api.FINISH_GENERAL),
                "top_p0.95_gaussian(wide nucleus)": (T, 0, TOP_P, False, api.FINISH_GENERAL)}.items():
            mode(name, t, k, p, pen, hint)
            modes[name]["finish_hint"] = HINTS[hint]
            mode(name + ", no hint", t, k, p, pen, api.FINISH_AUTO)
            modes[name + ", no hint"]["finish_hint"] = "AUTO"

    # ---- the other configurations of the reference's table (rank 0's GPU; device-resident)
    configs = {}
    if not args.no_configs and rank == 0:
        def run_cfg(name, xs_np, Tn, Kn, Pn, st_np, rows_per_seq=1, sample=None, hbytes=0, hint=0, **pen):
            rows, Vn = xs_np[0].shape
            nseq = rows // rows_per_seq
            cT, cK, cP = per_seq(nseq, Tn, Kn, Pn)
            kw, okw = {"finish_hint": hint}, {}  # the hint a caller that knows the sessions' settings gives (the batcher does)
            if "hist" in pen:
                kw["history"] = to_dev(pen["hist"])
                kw["history_len"] = to_dev(np.full(nseq, pen["hist"].shape[1], np.int32))
                okw["hist"] = pen["hist"]
            for k in ("rep", "freq", "pres"):
                if k in pen:
                    kw[k] = to_dev(np.full(nseq, pen[k], np.float32))
                    okw[k] = pen[k]
            dst_ = u64_to_dev(st_np)
            xs = [to_dev(x) for x in xs_np]
            ds = [ctx.sample_batch(x, cT, cK, cP, dst_, rows_per_seq=rows_per_seq, launch=False, **kw) for x in xs]
            sec = time_desc_list(ds, 100 if rows <= 1024 else 20, collective=False)
            out = ctx.sample_batch(xs[0], cT, cK, cP, dst_, rows_per_seq=rows_per_seq, **kw)
            tok = out["tokens"].cpu().numpy()
            sel = np.arange(rows) if sample is None else sample
            if rows_per_seq == 1:
                sub = {k: (v[sel] if k == "hist" else v) for k, v in okw.items()}
                o = port.sample_batch(xs_np[0][sel], np.broadcast_to(np.asarray(Tn, np.float32), (rows,))[sel], np.broadcast_to(np.asarray(Kn, np.int32), (rows,))[sel],
                                      np.broadcast_to(np.asarray(Pn, np.float32), (rows,))[sel], st_np[sel], **sub)
                match = bool(np.array_equal(tok[sel], o["tokens"]))
                checked = int(len(sel))
            else:
                o = port.sample_batch(xs_np[0], Tn, Kn, Pn, st_np, rows_per_seq=rows_per_seq, **okw)
                match = bool(np.array_equal(tok, o["tokens"]))
                checked = rows
            nbytes = rows * (4 * Vn + 4) + nseq * 16 + hbytes
            configs[name] = {"us_per_launch": sec * 1e6, "rows_per_s": rows / sec, "hbm_frac": nbytes / sec / 1e9 / peak,
                             "finish_hint": ["AUTO", "GREEDY_TOPK", "GENERAL", "GREEDY"][hint], "rows_checked_against_cpu": checked, "tokens_match_cpu": match,
                             "rows_invalid": int((out["status"] & api.ROW_INVALID).ne(0).sum().item()),
                             "rows_on_slow_path": int((out["status"] & api.ROW_SLOW_PATH).ne(0).sum().item())}
            del xs, ds, out
            torch.cuda.empty_cache()

        # config 2: batched greedy + frequency / presence penalties over 256-id histories, 64 x 151936
        run_cfg("c2_greedy_penalties_64x151936", [normal_logits(64, 151936, 3.0, 7 + i) for i in range(4)], 0.0, 0, 1.0,
                independent_states(port, 7, 64), hist=histories(64, 256, 151936, 7), freq=0.2, pres=0.3, hbytes=64 * 256 * 4, hint=api.FINISH_GREEDY)
        # config 3: nucleus sampling over heavy-tailed rows, 256 x 262144
        r3 = np.random.default_rng(99)
        run_cfg("c3_top_p_gumbel_256x262144", [gumbel_logits(256, 262144, 4.0, 99 + i) for i in range(2)],
                r3.uniform(0.5, 1.2, 256).astype(np.float32), 0, r3.uniform(0.8, 0.98, 256).astype(np.float32), seq_states(port, 99, 256),
                sample=np.arange(0, 256, 8), hint=api.FINISH_GENERAL)
        # config 4: speculative verify rows, 32 sequences x 7 rows x 128256, temperature 1
        def c4(seed):
            d = normal_logits(32 * 6, 128256, 2.5, seed).reshape(32, 6, 128256)
            t = np.empty((32, 7, 128256), np.float32)
            t[:, :6] = d + normal_logits(32 * 6, 128256, 0.5, seed + 1).reshape(32, 6, 128256)
            t[:, 6] = normal_logits(32, 128256, 2.5, seed + 2)
            return t.reshape(32 * 7, 128256)
        run_cfg("c4_verify_rows_32x7x128256", [c4(2024), c4(3024)], 1.0, 0, 1.0, independent_states(port, 2024, 32), rows_per_seq=7, hint=api.FINISH_GENERAL)
        # config 5: 4096 x 128256, top-k 50 + repetition penalty over 1024-id histories (every 128th row checked)
        run_cfg("c5_top_k50_penalties_4096x128256", [normal_logits(4096, 128256, 2.5, 31337)], 0.7, 50, 0.9, independent_states(port, 31337, 4096),
                hist=histories(4096, 1024, 128256, 31337), rep=1.15, sample=np.arange(0, 4096, 128), hbytes=4096 * 1024 * 4, hint=api.FINISH_GREEDY_TOPK)

    # ---- multi-GPU legs on configuration 5: vocabulary shards over NCCL, and its rows split N ways
    vocab_shards = None
    strong = None
    if world > 1 and not args.no_configs:
        rows5, V5, k5 = 4096, 128256, 50
        assert V5 % world == 0
        x5_np = normal_logits(rows5, V5, 2.5, 31337)  # the same matrix on every rank
        x5 = torch.from_numpy(x5_np).to(dev)
        h5_np = histories(rows5, 1024, V5, 31337)
        h5 = to_dev(h5_np)
        hl5 = to_dev(np.full(rows5, 1024, np.int32))
        rep5 = to_dev(np.full(rows5, 1.15, np.float32))
        st5_np = independent_states(port, 31337, rows5)
        st5 = u64_to_dev(st5_np)
        T5, K5, P5 = per_seq(rows5, 0.7, k5, 0.9)
        full = ctx.sample_batch(x5, T5, K5, P5, st5, rep=rep5, history=h5, history_len=hl5)
        Vs = V5 // world
        shard = x5[:, rank * Vs:(rank + 1) * Vs].contiguous()
        # the select's descriptor is filled once and launched again every iteration, like the headline's
        sel_out = ctx.sample_batch(shard, T5, K5, P5, st5, rep=rep5, history=h5, history_len=hl5, kept_cap=k5, vocab_offset=rank * Vs,
                                   select_only=True, launch=False)
        gv = torch.empty(world, rows5, k5, dtype=torch.float32, device=dev)
        gi = torch.empty(world, rows5, k5, dtype=torch.int32, device=dev)
        gn = torch.empty(world, rows5, dtype=torch.int32, device=dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        t_sel = t_gat = t_mrg = 0.0
        n_it = 12
        merged = None
        for it in range(n_it + 2):
            all_barrier()
            ev[0].record()
            ctx.relaunch(sel_out, stream)
            ev[1].record()
            dist.all_gather_into_tensor(gv, sel_out["kept_prob"])
            dist.all_gather_into_tensor(gi, sel_out["kept_idx"])
            dist.all_gather_into_tensor(gn, sel_out["kept_n"])
            ev[2].record()
            merged = ctx.shard_merge_sample(gv, gi, gn, T5, K5, st5, out=merged, sync=False)
            ev[3].record()
            torch.cuda.synchronize(dev)
            if it >= 2:
                t_sel += ev[0].elapsed_time(ev[1])
                t_gat += ev[1].elapsed_time(ev[2])
                t_mrg += ev[2].elapsed_time(ev[3])
        same = bool(torch.equal(merged["tokens"], full["tokens"]))
        flag = torch.tensor([1 if same else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        tt = torch.tensor([t_sel, t_gat, t_mrg], device=dev) / n_it
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        chk = np.arange(0, rows5, 256)
        o5 = port.sample_batch(x5_np[chk], 0.7, k5, 0.9, st5_np[chk], rep=1.15, hist=h5_np[chk]) if rank == 0 else None
        total_ms = float(tt.sum().item())
        vocab_shards = {"config": f"4096 x 128256 as {world} shards of {Vs} columns, 1024-id histories, rep 1.15, T 0.7, top-k 50",
                        "tokens_match_unsharded": bool(flag.item() == 1),
                        "tokens_match_cpu_sample": bool(np.array_equal(merged["tokens"].cpu().numpy()[chk], o5["tokens"])) if rank == 0 else None,
                        "ms_select": float(tt[0].item()), "ms_all_gather": float(tt[1].item()), "ms_merge_draw": float(tt[2].item()),
                        "rows_per_s": rows5 / (total_ms * 1e-3), "gathered_bytes_per_rank": int(world * rows5 * (k5 * 8 + 4))}
        # the same rows split over the ranks (strong scaling of configuration 5)
        a, b = rank * rows5 // world, (rank + 1) * rows5 // world
        part = ctx.sample_batch(x5[a:b], T5[a:b], K5[a:b], P5[a:b], st5[a:b], rep=rep5[a:b], history=h5[a:b], history_len=hl5[a:b], launch=False, finish_hint=api.FINISH_GREEDY_TOPK)
        sec = time_desc_list([part], 20)
        part_same = torch.tensor([1 if torch.equal(part["tokens"], full["tokens"][a:b]) else 0], device=dev)
        dist.all_reduce(part_same, op=dist.ReduceOp.MIN)
        strong = {"rows": rows5, "rows_per_rank": b - a, "us_per_launch": sec * 1e6, "rows_per_s": rows5 / sec,
                  "tokens_match_unsharded": bool(part_same.item() == 1)}

    clocks = sampler.stop(windows) if sampler else None

    # ---- CPU baseline on rank 0, bounded sample of the same rows, all host threads
    cpu = None
    parity = None
    if rank == 0:
        threads = os.cpu_count() or 1
        n_cpu = min(B, max(64, 8 * threads))
        x_pen = penalised(sets_np0[:n_cpu], hist_np[:n_cpu])  # the reference has no penalties: applied before the clock starts
        cpu_out, kind = cpu_reference_rows(x_pen, states[:n_cpu], threads)  # warm-up pass; its tokens feed the parity check
        if world == 1:  # the timed baseline belongs to the single-GPU line only
            t0 = time.perf_counter()
            passes = 2
            for _ in range(passes):
                cpu_reference_rows(x_pen, states[:n_cpu], threads)
            v = n_cpu * passes / (time.perf_counter() - t0)
            cpu = {"value": v, "unit": "rows/s", "cores": threads, "kind": kind,
                   "sample": f"first {n_cpu} rows of input set 0, {passes} passes after one warm-up pass, {threads} host threads, penalties applied outside the clock"}
        # the bench's own inputs double as a parity spot check (set 0 is sampled from the initial states)
        chk = ctx.sample_batch(sets[0], dT, dK, dP, u64_to_dev(states), rep=dRep, history=hist, history_len=dHl)
        parity = bool(np.array_equal(chk["tokens"][:n_cpu].cpu().numpy(), cpu_out["tokens"]))

    if rank == 0:
        traffic, traffic_src = ncu_traffic()
        line = {
            "metric": "sampled rows/s at B=256,V=128256 fp32", "value": rows_per_s, "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": B, "l2": f"inputs rotate over {N_SETS} sets of 131 MB (> 126 MB L2)",
                       "launch": {**api.plan(V, H), **api.grid(V, B, H)}, "finish_hint": "GREEDY_TOPK", "rows_invalid": bad, "rows_on_slow_path": slow,
                       "library": str(LIB_PATH)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_src, "peak_kind": peak_kind, "bytes_per_launch": B * BYTES_PER_ROW,
                         "us_per_launch": per_launch_s * 1e6,
                         "note": "one launch = one step: the stream kernel (every logit crosses HBM once), which also finishes the rows"},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": args.steps * KERNELS_PER_STEP,
            "clocks": clocks,
            "modes": modes,
            "configs": configs,
            "tokens_match_cpu_reference": parity,
        }
        if vocab_shards is not None:
            line["vocab_shards"] = vocab_shards
            line["row_shards_strong"] = strong
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
