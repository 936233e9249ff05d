#!/usr/bin/env python3
"""Benchmark of the sparse-ternary hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the GEMV shape sweep, batch 1, cold L2): the headline figure is the 6912x2560
sparse-ternary GEMV.  One step is one pass over `copies` distinct copies of that matrix
(together several times the L2), each copy one GEMV launch through the C-ABI, so every
launch streams its weights from HBM.  `value` is algorithmic bytes (the reference's own
count: both weight streams + x + y) over the device time of the timed steps, aggregated
over all ranks.  With N > 1 every rank runs the same per-GPU workload on its own GPU with no
data-path collective (weak scaling of independent replicas); time is the max over ranks.

Prints ONE JSON line.  `--impl reference` times the reference's own CPU implementation of
the same GEMV on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "sparse_ternary_gemv_hbm_gbs_6912x2560"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes one 6912x2560 GEMV launch moved under ncu (read 3.337 MB, write 0: y stays in L2)
NCU_DRAM_BYTES_PER_LAUNCH = 3.337e6


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.proc:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        rows = [l.strip().split(", ") for l in Path(self.file.name).read_text().splitlines() if l.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ---------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation on the host cores
# ---------------------------------------------------------------------------------------

def cpu_gemv_baseline(rows, cols, threads, budget_s, use_ref=True):
    """Times the reference's CPU GEMV (unpack_to_int8 + int32 dot, as its tests run it) on the
    metric shape.  Returns (GB/s, kind, reps, seconds)."""
    import oracle
    from spbitnet_b200 import synth
    rng = np.random.default_rng(0)
    w, mask = synth.ternary_weights_and_mask(rows, cols, rng)
    x = rng.integers(-127, 128, cols, dtype=np.int8)
    nbytes = synth.gemv_algorithmic_bytes(rows, cols)
    if use_ref and oracle.ref() is not None:
        kind = "reference"
        run = lambda reps: oracle.ref_cpu_sparse_gemv(w, mask, x, threads=threads, repeats=reps)
    else:
        kind = "port"
        meta, values = synth.pack_numpy(w, mask)
        def run(reps):
            for _ in range(reps):
                oracle.sparse_gemv(meta, values, x, rows, cols, threads=threads)
    t0 = time.perf_counter()
    run(1)
    one = time.perf_counter() - t0
    reps = max(1, int(budget_s / max(one, 1e-4)))
    t0 = time.perf_counter()
    run(reps)
    dt = time.perf_counter() - t0
    return nbytes * reps / dt / 1e9, kind, reps, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from spbitnet_b200 import synth
    rows, cols = synth.METRIC_SHAPE
    threads = os.cpu_count() or 1
    # each step: `reps` GEMVs of the metric shape on all host threads
    gbs1, kind, reps, _ = cpu_gemv_baseline(rows, cols, threads, 0.5)
    for _ in range(max(args.warmup - 1, 0)):
        cpu_gemv_baseline(rows, cols, threads, 0.2)
    vals, t_total = [], 0.0
    for _ in range(args.steps):
        g, kind, r, dt = cpu_gemv_baseline(rows, cols, threads, 1.0)
        vals.append((g, r, dt))
        t_total += dt
    total_bytes = sum(synth.gemv_algorithmic_bytes(rows, cols) * r for _, r, _ in vals)
    value = total_bytes / t_total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "gemv 6912x2560 batch 1, reference CPU path (unpack_to_int8 + int32 dot)",
                   "shape": [rows, cols]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{sum(r for _, r, _ in vals)} GEMVs of 6912x2560 in {t_total:.2f} s, row loop "
                                   f"split over {threads} threads"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from spbitnet_b200 import kernels as K, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    K.set_gemv_variant(args.variant)
    if args.no_pdl:
        K.set_pdl(False)
    if args.only_gemm:
        if rank == 0:
            l2 = torch.cuda.get_device_properties(local).L2_cache_size
            print(json.dumps({"metric": "sparse_ternary_gemm", "gemm": bench_gemm(args, l2), "n_gpus": world}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only_prefill:
        if rank == 0:
            print(json.dumps({"metric": "prefill_tok_s_2b4t_shape", "prefill": bench_prefill(args), "n_gpus": world}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only_decode:
        if rank == 0:
            print(json.dumps({"metric": "decode_tok_s_2b4t_shape", "decode": bench_decode(args), "n_gpus": world}))
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    l2_bytes = torch.cuda.get_device_properties(local).L2_cache_size
    rows, cols = synth.METRIC_SHAPE

    def dev_u32(a):
        return torch.from_numpy(np.ascontiguousarray(a).view(np.int32)).cuda()

    def make_set(r, c, min_bytes, seed=0):
        """`copies` distinct device copies of an r x c matrix totalling >= min_bytes."""
        case = synth.gemv_case(r, c, seed=seed)
        per = synth.gemv_algorithmic_bytes(r, c)
        copies = max(8, int(np.ceil(min_bytes / per)))
        meta = dev_u32(case["meta"])
        values = dev_u32(case["values"])
        # distinct storage per copy; contents are permuted rows so the copies are not identical
        metas = torch.stack([meta.roll(i, 0) for i in range(copies)]).contiguous()
        vals = torch.stack([values.roll(i, 0) for i in range(copies)]).contiguous()
        return case, copies, metas, vals, per

    stream = torch.cuda.current_stream()

    def launch_pass(metas, vals, xs, ys, r, c, ms, vs, copies):
        for i in range(copies):
            K.sparse_ternary_gemv_gpu(metas[i], vals[i], xs[i % xs.shape[0]], ys[i], r, c, ms, vs)

    def time_device(fn, steps, warmup):
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
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms

    # ---- headline: 6912 x 2560 over a rotating working set of 4x the L2 ------------------
    case, copies, metas, vals, per = make_set(rows, cols, max(4 * l2_bytes, 512 << 20))
    ms_, vs_ = case["meta_stride"], case["values_stride"]
    rng = np.random.default_rng(1)
    x_host = torch.from_numpy(rng.integers(-127, 128, (copies, cols), dtype=np.int8)).pin_memory()
    xs = x_host.cuda()
    ys = torch.zeros((copies, rows), dtype=torch.int32, device="cuda")
    y_host = torch.empty((copies, rows), dtype=torch.int32).pin_memory()

    # correctness spot check before timing (like benchmarks/bench_kernels.cu:221-232)
    launch_pass(metas, vals, xs, ys, rows, cols, ms_, vs_, copies)
    torch.cuda.synchronize()
    import oracle
    chk = oracle.sparse_gemv(case["meta"], case["values"], x_host[0].numpy(), rows, cols, threads=os.cpu_count() or 1)
    if not (ys[0].cpu().numpy() == chk).all():
        raise SystemExit("bench: GEMV result differs from the oracle; refusing to time it")

    branch_streams = [torch.cuda.Stream() for _ in range(max(args.chains, 1))]

    def capture(metas, vals, xs, ys, r, c, ms, vs, copies, chains):
        """One step as a CUDA graph: `copies` GEMV launches spread round-robin over `chains`
        parallel branches.  Launches of a branch are stream-ordered (PDL-chained); branches are
        independent, which the GEMVs of a step are (distinct weights and outputs)."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream()
            if chains <= 1:
                launch_pass(metas, vals, xs, ys, r, c, ms, vs, copies)
            else:
                for s in branch_streams[:chains]:
                    s.wait_stream(main)
                for i in range(copies):
                    with torch.cuda.stream(branch_streams[i % chains]):
                        K.sparse_ternary_gemv_gpu(metas[i], vals[i], xs[i % xs.shape[0]], ys[i], r, c, ms, vs)
                for s in branch_streams[:chains]:
                    main.wait_stream(s)
        return g

    graph = capture(metas, vals, xs, ys, rows, cols, ms_, vs_, copies, args.chains)
    graph_chain = capture(metas, vals, xs, ys, rows, cols, ms_, vs_, copies, 1) if args.chains > 1 else graph

    work = K.GemvWorkList([(metas[i], vals[i], xs[i], ys[i], rows, cols, ms_, vs_) for i in range(copies)])
    ys.zero_()
    K.sparse_ternary_gemv_batch_gpu(work)
    torch.cuda.synchronize()
    if not (ys[0].cpu().numpy() == chk).all() or not (ys[copies - 1].cpu().numpy() ==
            oracle.sparse_gemv(np.roll(case["meta"], copies - 1, 0), np.roll(case["values"], copies - 1, 0),
                               x_host[copies - 1].numpy(), rows, cols, threads=os.cpu_count() or 1)).all():
        raise SystemExit("bench: work-list GEMV result differs from the oracle; refusing to time it")
    ms_batch = time_device(lambda: K.sparse_ternary_gemv_batch_gpu(work), args.steps, args.warmup)
    batch_us = ms_batch * 1e3 / (args.steps * copies)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_graph = time_device(graph.replay, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else {}
    ms_stream = time_device(lambda: launch_pass(metas, vals, xs, ys, rows, cols, ms_, vs_, copies),
                            max(1, args.steps // 2), 1)
    ms_chain = time_device(graph_chain.replay, args.steps, args.warmup)
    chain_us = ms_chain * 1e3 / (args.steps * copies)
    step_bytes = per * copies
    value = world * step_bytes * args.steps / (ms_graph * 1e-3) / 1e9
    per_launch_us = ms_graph * 1e3 / (args.steps * copies)
    achieved = per / (per_launch_us * 1e-6) / 1e9
    stream_gbs = step_bytes * max(1, args.steps // 2) / (ms_stream * 1e-3) / 1e9

    # ---- e2e: host x batch in, host y batch out, every step --------------------------------
    # Steps are independent batches, so they are pipelined over two buffer sets: while the result of step k goes
    # back to the host on a copy stream, the inputs of step k + 1 come in and its GEMVs run.  Every step still
    # does its own H2D and D2H inside the timed region.
    xs_b, ys_b = torch.empty_like(xs), torch.zeros_like(ys)
    y_host_b = torch.empty_like(y_host).pin_memory()
    graph_b = capture(metas, vals, xs_b, ys_b, rows, cols, ms_, vs_, copies, args.chains)
    sets = [(xs, ys, y_host, graph), (xs_b, ys_b, y_host_b, graph_b)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(steps):
        main = torch.cuda.current_stream()
        for ev in ev_done + ev_out:
            ev.record(main)
        for k in range(steps):
            p = k & 1
            x_d, y_d, y_h, g = sets[p]
            s_in.wait_event(ev_done[p])      # the GEMVs that read this input buffer two steps ago are done
            with torch.cuda.stream(s_in):
                x_d.copy_(x_host, non_blocking=True)
                ev_in[p].record(s_in)
            main.wait_event(ev_in[p])
            main.wait_event(ev_out[p])       # the previous result in this output buffer has left
            g.replay()
            ev_done[p].record(main)
            s_out.wait_event(ev_done[p])
            with torch.cuda.stream(s_out):
                y_h.copy_(y_d, non_blocking=True)
                ev_out[p].record(s_out)
        main.wait_event(ev_out[0])
        main.wait_event(ev_out[1])

    def time_e2e(steps, warmup):
        e2e_run(warmup)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(steps)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms

    ms_e2e = time_e2e(args.steps, args.warmup)
    e2e_value = world * step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    if not (y_host[0].numpy() == chk).all() or not (y_host_b[0].numpy() == chk).all():
        raise SystemExit("bench: end-to-end result differs from the oracle")

    def e2e_step():  # the same step without overlap, for comparison
        xs.copy_(x_host, non_blocking=True)
        graph.replay()
        y_host.copy_(ys, non_blocking=True)
    ms_e2e_serial = time_device(e2e_step, args.steps, args.warmup)

    # ---- the other shapes of the sweep (rank 0 only, short) --------------------------------
    sweep = {}
    if rank == 0 and not args.no_sweep:
        for (r, c) in synth.GEMV_SHAPES:
            cs, cp, mt, vl, pb = make_set(r, c, max(2 * l2_bytes, 256 << 20), seed=0)
            xx = torch.from_numpy(rng.integers(-127, 128, (8, c), dtype=np.int8)).cuda()
            yy = torch.zeros((cp, r), dtype=torch.int32, device="cuda")
            launch_pass(mt, vl, xx, yy, r, c, cs["meta_stride"], cs["values_stride"], cp)
            torch.cuda.synchronize()
            g2 = capture(mt, vl, xx, yy, r, c, cs["meta_stride"], cs["values_stride"], cp, args.chains)
            for _ in range(3):
                g2.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                g2.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (5 * cp)
            gbs = pb / (us * 1e-6) / 1e9
            sweep[f"{r}x{c}"] = {"us_per_gemv": round(us, 3), "gbs": round(gbs, 1),
                                 "frac_measured": round(gbs / peak, 4), "frac_8tbs": round(gbs / NOMINAL_HBM_GBS, 4)}
            del mt, vl, yy, g2

    # ---- reference CUDA kernel on the same GPU (when the checker library is present) --------
    ref_cuda = None
    if rank == 0:
        try:
            import ctypes as C
            rc = oracle.refcuda()
            if rc is not None:
                sp = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                def ref_pass():
                    for i in range(copies):
                        rc.refcuda_gemv(C.c_void_p(metas[i].data_ptr()), C.c_void_p(vals[i].data_ptr()),
                                        C.c_void_p(xs[i].data_ptr()), C.c_void_p(ys[i].data_ptr()), rows, cols,
                                        ms_, vs_, sp)
                ms_ref = time_device(ref_pass, 2, 1) if world == 1 else None
                if ms_ref:
                    ref_cuda = {"us_per_gemv": ms_ref * 1e3 / (2 * copies),
                                "gbs": step_bytes * 2 / (ms_ref * 1e-3) / 1e9,
                                "what": "reference sparse_ternary_gemv_kernel recompiled for sm_100a, same buffers"}
        except Exception as exc:  # the checker is optional
            ref_cuda = {"error": str(exc)}

    # ---- CPU baseline (rank 0, N == 1) -------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        g1, kind, reps1, dt1 = cpu_gemv_baseline(rows, cols, 1, 4.0)
        gN, kind, repsN, dtN = cpu_gemv_baseline(rows, cols, threads, 4.0)
        cpu = {"value": gN, "unit": UNIT, "cores": threads, "kind": kind,
               "sample": f"{repsN} GEMVs of 6912x2560 in {dtN:.2f} s on {threads} threads "
                         f"(1 thread: {g1:.3f} GB/s over {reps1} GEMVs)"}

    gemm = None
    if rank == 0 and not args.no_gemm:
        try:
            gemm = bench_gemm(args, l2_bytes)
        except Exception as exc:
            gemm = {"error": repr(exc)}

    # ---- decode throughput on the 2B-4T-shape model (secondary figure) ----------------------
    decode = None
    if rank == 0 and not args.no_decode:
        try:
            decode = bench_decode(args)
        except Exception as exc:
            decode = {"error": repr(exc)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_graph / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "gemv shape sweep, batch 1; headline 6912x2560", "shape": [rows, cols],
                       "copies_per_step": copies, "working_set_mb": round(step_bytes / 2**20, 1),
                       "l2_mb": round(l2_bytes / 2**20, 1),
                       "cold_l2": "inputs larger than L2: every launch reads a different weight copy",
                       "launch": f"one CUDA graph replay per step: {copies} GEMV launches in {args.chains} independent "
                                 "branches (stream-ordered, PDL-chained inside a branch)",
                       "chains": args.chains, "gemv_variant": args.variant,
                       "seed": 0},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                           "kernel at 6912x2560 (profiles/gemv_mmasp_6912x2560_ncu_full.md)",
                         "algorithmic_bytes_per_launch": per, "us_per_launch": per_launch_us,
                         "frac_of_8tbs": achieved / NOMINAL_HBM_GBS},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel()),
                    "d2h_bytes_per_step": int(y_host.numel() * 4), "ms_per_step": ms_e2e / args.steps,
                    "pipeline": "two buffer sets: the D2H of step k overlaps the H2D and GEMVs of step k + 1",
                    "serial_value": world * step_bytes * args.steps / (ms_e2e_serial * 1e-3) / 1e9},
            "stream_launch_gbs": stream_gbs,
            "work_list": {"us_per_gemv": batch_us, "gbs": per / (batch_us * 1e-6) / 1e9,
                          "frac_measured": per / (batch_us * 1e-6) / 1e9 / peak,
                          "what": f"the same {copies} GEMVs as ONE persistent launch (spb_sparse_ternary_gemv_batch)"},
            "dependent_chain": {"us_per_gemv": chain_us, "gbs": per / (chain_us * 1e-6) / 1e9,
                                "what": "the same launches as ONE stream-ordered chain (each GEMV waits for the "
                                        "previous one before it reads x): the latency a decode step sees"},
            "gpu_launches": args.steps * copies,
            "clocks": clocks,
            "cpu_baseline": cpu,
            "ref_cuda_same_gpu": ref_cuda,
            "sweep": sweep,
            "gemm": gemm,
            "decode": decode,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def oracle_unpack(case, r, c):
    import oracle
    return oracle.unpack_to_int8(case["meta"], case["values"], r, c)


def library_gemm(Wd, X, r, c, n):
    """Library kernels on a dense int8 copy of the same weights (comparison only; weights stay resident in L2):
    cuBLASLt int8 (torch._int_mm) and cuSPARSELt 2:4 (torch._cslt_sparse_mm), which is the reference's batched path."""
    import torch
    res = {}

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 20
        return {"us": round(us, 2), "dense_equiv_tops": round(2.0 * r * c * n / us / 1e6, 2)}
    try:
        Wt = Wd.t()
        res["lib_cublaslt_dense"] = timed(lambda: torch._int_mm(X, Wt))
    except Exception as exc:
        res["lib_cublaslt_dense"] = {"error": str(exc)[:120]}
    try:
        comp = torch._cslt_compress(Wd)
        Xt = X.t()
        res["lib_cusparselt"] = timed(lambda: torch._cslt_sparse_mm(comp, Xt, out_dtype=torch.int32))
    except Exception as exc:
        res["lib_cusparselt"] = {"error": str(exc)[:120]}
    return res


def bench_gemm(args, l2_bytes):
    """Batched product (prefill) at the two FFN shapes, N in {1,4,16,64,256,1024}: us per call over a
    rotating set of weight copies larger than L2, weight-stream GB/s and dense-equivalent int8 TOP/s."""
    import torch
    from spbitnet_b200 import kernels as K, synth
    out = {}
    for (r, c) in synth.GEMM_SHAPES:
        case = synth.gemv_case(r, c, seed=0)
        per = r * 4 * (case["meta_stride"] + case["values_stride"])
        copies = max(4, int(np.ceil(1.5 * l2_bytes / per)))
        meta = torch.from_numpy(case["meta"].view(np.int32)).cuda()
        values = torch.from_numpy(case["values"].view(np.int32)).cuda()
        metas = torch.stack([meta.roll(i, 0) for i in range(copies)]).contiguous()
        vals = torch.stack([values.roll(i, 0) for i in range(copies)]).contiguous()
        Wd = torch.from_numpy(oracle_unpack(case, r, c)).cuda()  # dense int8 copy, what the reference hands to cuSPARSELt
        for n in synth.GEMM_BATCHES:
            X = torch.randint(-127, 128, (n, c), dtype=torch.int8, device="cuda")
            Y = torch.empty((n, r), dtype=torch.int32, device="cuda")
            row = {}
            for name, variant in (("auto", 0), ("simt", 1), ("tc_dense", 2), ("tc_sparse", 3), ("mma_sp", 4)):
                if (variant == 1 and n > 64) or (variant in (2, 3) and n < 16) or (variant == 4 and n > 256):
                    continue
                K.set_gemm_variant(variant)
                def run():
                    for i in range(copies):
                        K.sparse_ternary_gemm_gpu(metas[i], vals[i], X, Y, r, c, n, case["meta_stride"], case["values_stride"])
                run()
                torch.cuda.synchronize()
                # one CUDA graph of the `copies` calls (stream-ordered), so that the host's launch cost is not timed
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    run()
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 3
                e0.record()
                for _ in range(reps):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
                row[name] = {"us": round(us, 2), "weight_gbs": round(per / us / 1e3, 1),
                             "dense_equiv_tops": round(2.0 * r * c * n / us / 1e6, 2)}
            K.set_gemm_variant(0)
            if n >= 64:
                row.update(library_gemm(Wd, X, r, c, n))
            out[f"{r}x{c}_n{n}"] = row
        del metas, vals
    out["tc_timeouts"] = K.gemm_tc_timeouts()
    out["what"] = ("spb_sparse_ternary_gemm, us per call as a graph of stream-ordered calls over cold weights; auto = "
                   "warp-level sparse MMA (mma.sp) up to n = 32, tcgen05.mma.sp above; tc_dense = tcgen05 kind::i8 on "
                   "expanded int8 tiles; lib_* = library kernels on a dense int8 copy of the weights that stays in L2 "
                   "(comparison only); dense_equiv_tops counts 2*M*K*N")
    return out


def bench_decode(args):
    """Greedy decode of a random-init BitNet-2B-4T-shape model: 128-token prompt, 256 generated."""
    import torch
    from spbitnet_b200 import synth
    from spbitnet_b200.engine import DeviceModel, InferenceEngine
    cfg = dict(synth.BITNET_2B)
    if args.decode_layers > 0:
        cfg["num_hidden_layers"] = args.decode_layers
    model = synth.random_model(cfg, seed=0, shared_layer=True)
    dm = DeviceModel(model)
    eng = InferenceEngine(dm)
    prompt = np.random.default_rng(0).integers(0, cfg["vocab_size"], 128).astype(np.int32)
    n_gen = args.decode_tokens
    eng.generate(prompt, 8)  # warm-up: graph capture, page-in
    eng.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    toks = eng.generate(prompt, n_gen)
    dt = time.perf_counter() - t0
    steps = len(prompt) - 1 + n_gen
    weight_bytes = dm.sparse_bytes() + model["embed"].nbytes
    # the same job with the prompt fed as one batch (BitLinear layers as the batched product)
    eng.reset()
    eng.set_prefill_chunk(256)
    eng.generate(prompt, 2)
    eng.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    toks_b = eng.generate(prompt, n_gen)
    dt_b = time.perf_counter() - t0
    eng.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.prefill(prompt)
    dt_p = time.perf_counter() - t0
    eng.set_prefill_chunk(0)
    batched = {"tok_s": steps / dt_b, "ms_total": 1e3 * dt_b, "prefill_ms": 1e3 * dt_p,
               "prefill_tok_s": len(prompt) / dt_p, "same_tokens_as_serial": bool((toks_b == toks).all()),
               "decode_only_tok_s": (n_gen - 1) / max(dt_b - dt_p, 1e-9)}
    return {"tok_s": steps / dt, "batched_prompt": batched, "ms_per_token": 1e3 * dt / steps, "generated": int(len(toks)),
            "prompt": int(len(prompt)), "weight_mb_per_token": round(weight_bytes / 1e6, 1),
            "hbm_gbs": weight_bytes * steps / dt / 1e9,
            "what": "prefill (token-serial, as the reference) + decode, wall clock around generate() incl. prompt "
                    "H2D and token D2H; random-init 2B-4T shape, layer weights generated once and uploaded per layer"}


def bench_prefill(args):
    """The prompt as one batch through a random-init 2B-4T-shape model (engine.prefill), wall clock per call."""
    import torch
    from spbitnet_b200 import synth
    from spbitnet_b200.engine import DeviceModel, InferenceEngine
    cfg = dict(synth.BITNET_2B)
    if args.decode_layers > 0:
        cfg["num_hidden_layers"] = args.decode_layers
    model = synth.random_model(cfg, seed=0, shared_layer=True)
    eng = InferenceEngine(DeviceModel(model))
    n = args.prefill_tokens
    prompt = np.random.default_rng(0).integers(0, cfg["vocab_size"], n).astype(np.int32)
    for _ in range(3):  # direct launches, graph capture, first replay
        eng.reset()
        eng.prefill(prompt)
    times = []
    for _ in range(5):
        eng.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        eng.prefill(prompt)
        times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    return {"tokens": n, "layers": cfg["num_hidden_layers"], "ms": 1e3 * dt, "tok_s": n / dt,
            "what": "engine.prefill(prompt): token ids H2D, all layers over the batch, logits of the last token; "
                    "median of 5 calls after 3 warm-up calls"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--chains", type=int, default=8, help="independent branches per step graph")
    ap.add_argument("--variant", type=int, default=0,
                    help="GEMV kernel: 0 auto (warp-level sparse MMA), 1 SIMT pair, 2 SIMT group table, 3 tcgen05, 4 mma.sp")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-gemm", action="store_true")
    ap.add_argument("--only-gemm", action="store_true", help="only the batched-product section (profiling aid)")
    ap.add_argument("--only-decode", action="store_true", help="skip the GEMV sections (profiling aid)")
    ap.add_argument("--only-prefill", action="store_true", help="only the batched-prefill timing (profiling aid)")
    ap.add_argument("--prefill-tokens", type=int, default=128)
    ap.add_argument("--decode-layers", type=int, default=0, help="override the layer count of the decode model")
    ap.add_argument("--decode-tokens", type=int, default=256)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
