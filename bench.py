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
the same GEMV on the host cores instead (and imports nothing of the product).

Beside the headline the line carries: `sweep` (all nine shapes, each with the reference's own CUDA kernel
recompiled for sm_100a in the same graph), `cpu_baseline`, `gemm` (the batched product against cuBLASLt and
cuSPARSELt, every result checked against the CPU oracle before it is timed), `decode` (2B-4T-shape greedy decode,
one replica per rank) and `sharded` (the Llama-70B-shaped model row-sharded over the ranks of the run; with more
than one rank nothing is timed unless the sharded logits equal one rank's bit for bit).
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
NOMINAL_SPARSE_INT8_TOPS = 9000.0  # dense-equivalent; 4.5 POP/s dense int8 x 2
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
# reference arm: the reference's CPU implementation on the host cores.  Imports nothing of the product:
# the seeded inputs are drawn here with numpy (the rules of spbitnet_b200.synth, restated).
# ---------------------------------------------------------------------------------------

METRIC_ROWS, METRIC_COLS = 6912, 2560


def gemv_bytes(rows, cols):
    """The reference's byte count of one GEMV (benchmarks/bench_kernels.cu:248): both weight streams + x + y."""
    return rows * 4 * ((cols // 4 + 7) // 8 + (cols // 4 + 15) // 16) + cols + 4 * rows


def ternary_case_numpy(rows, cols, seed=0):
    """(weights int8 {-1,0,1}, keep-mask with two per group, x int8): P(0)=0.42, P(+1)=P(-1)=0.29; per group of
    four keep at most two non-zeros chosen uniformly, then zeros by ascending index until two are marked."""
    rng = np.random.default_rng(seed)
    u = rng.random((rows, cols))
    w = np.where(u < 0.42, 0, np.where(u < 0.71, 1, -1)).astype(np.int8)
    keys = rng.random((rows, cols))
    g = cols // 4
    nz = w.reshape(rows, g, 4) != 0
    order_key = np.where(nz, keys.reshape(rows, g, 4), 2.0 + np.arange(4)[None, None, :])
    order = np.argsort(order_key, axis=-1, kind="stable")
    keep = np.zeros((rows, g, 4), bool)
    np.put_along_axis(keep, order[:, :, :2], True, axis=-1)
    x = rng.integers(-127, 128, cols, dtype=np.int8)
    return w, keep.reshape(rows, cols), x


class CpuGemv:
    """The CPU GEMV of the reference (unpack_to_int8 + int32 dot, tests/test_sparse_ternary.cu:17-33) on the
    metric shape: through oracle/_ref (the reference's own header) when built, else the C port."""

    def __init__(self, rows, cols, threads):
        import oracle
        self.rows, self.cols, self.threads = rows, cols, threads
        w, mask, self.x = ternary_case_numpy(rows, cols, 0)
        self.bytes = gemv_bytes(rows, cols)
        if oracle.ref() is not None:
            self.kind = "reference"
            self.ctx = oracle.RefCpuGemv(w, mask, threads)
            self.run = lambda reps, dot_only=False: self.ctx.run(self.x, reps, dot_only)
        else:
            self.kind = "port"
            meta, values = oracle.pack_from_dense(w, mask)
            def run(reps, dot_only=False):
                for _ in range(reps):
                    oracle.sparse_gemv(meta, values, self.x, rows, cols, threads=threads)
            self.run = run

    def timed(self, budget_s, dot_only=False):
        """(GB/s, repeats, seconds) of about budget_s seconds of back-to-back GEMVs."""
        t0 = time.perf_counter()
        self.run(1, dot_only)
        one = time.perf_counter() - t0
        reps = max(1, int(budget_s / max(one, 1e-4)))
        t0 = time.perf_counter()
        self.run(reps, dot_only)
        dt = time.perf_counter() - t0
        return self.bytes * reps / dt / 1e9, reps, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows, cols = METRIC_ROWS, METRIC_COLS
    threads = os.cpu_count() or 1
    cpu = CpuGemv(rows, cols, threads)
    for _ in range(max(args.warmup, 0)):
        cpu.timed(0.2)
    vals, t_total = [], 0.0
    for _ in range(args.steps):  # each step: about a second of GEMVs of the metric shape on all host threads
        g, r, dt = cpu.timed(1.0)
        vals.append((g, r, dt))
        t_total += dt
    n_gemv = sum(r for _, r, _ in vals)
    value = cpu.bytes * n_gemv / t_total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "gemv shape sweep, batch 1; headline 6912x2560", "shape": [rows, cols],
                   "path": "reference CPU path: unpack_to_int8 + int32 dot, rows split over the host threads"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": cpu.kind,
                         "sample": f"{n_gemv} GEMVs of 6912x2560 in {t_total:.2f} s; every thread unpacks and "
                                   f"multiplies its own slice of the rows ({threads} threads)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def cpu_baselines(budget_s=4.0):
    """The CPU baselines of the metric shape, timed on this host: the reference's scalar GEMV as written (one
    thread), its dot product alone on pre-unpacked weights (one thread / all threads), and the same GEMV with the
    row loop split over all threads.  A baseline, not a target."""
    threads = os.cpu_count() or 1
    one, many = CpuGemv(METRIC_ROWS, METRIC_COLS, 1), CpuGemv(METRIC_ROWS, METRIC_COLS, threads)
    c1, r1, d1 = one.timed(budget_s)
    c2a, _, _ = one.timed(budget_s / 2, dot_only=True) if one.kind == "reference" else (None, 0, 0)
    c2b, _, _ = many.timed(budget_s / 2, dot_only=True) if many.kind == "reference" else (None, 0, 0)
    c3, r3, d3 = many.timed(budget_s)
    return {"value": c3, "unit": UNIT, "cores": threads, "kind": many.kind,
            "sample": f"{r3} GEMVs of 6912x2560 in {d3:.2f} s, unpack + dot with the rows split over {threads} threads",
            "one_thread_unpack_and_dot": c1, "one_thread_sample": f"{r1} GEMVs in {d1:.2f} s",
            "dot_only_one_thread": c2a, "dot_only_all_threads": c2b}


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
    if args.only_sharded:
        res = bench_sharded(args, rank, world, dist if world > 1 else None)
        if rank == 0:
            print(json.dumps({"metric": "sharded_decode_tok_s_70b_shape", "sharded": res, "n_gpus": world}))
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
            print(json.dumps({"metric": "decode_tok_s_2b4t_shape", "decode": bench_decode(args, with_cpu=not args.no_cpu), "n_gpus": world}))
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

    # ---- the shapes of the sweep (rank 0 only, short): ours, and the reference's own kernel recompiled for
    #      sm_100a, each as the same graph of launches (same branches, same weight copies, same x and y) -------
    import ctypes as C
    refcuda = oracle.refcuda() if rank == 0 else None

    def capture_ref(metas, vals, xs, ys, r, c, ms, vs, copies, chains):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            main = torch.cuda.current_stream()
            for st in branch_streams[:chains]:
                st.wait_stream(main)
            for i in range(copies):
                st = branch_streams[i % chains]
                refcuda.refcuda_gemv(C.c_void_p(metas[i].data_ptr()), C.c_void_p(vals[i].data_ptr()),
                                     C.c_void_p(xs[i % xs.shape[0]].data_ptr()), C.c_void_p(ys[i].data_ptr()), r, c,
                                     ms, vs, C.c_void_p(st.cuda_stream))
            for st in branch_streams[:chains]:
                main.wait_stream(st)
        return g

    def time_graph(g, reps, launches):
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * launches)

    sweep = {}
    if rank == 0 and not args.no_sweep:
        for (r, c) in synth.GEMV_SHAPES:
            cs, cp, mt, vl, pb = make_set(r, c, max(2 * l2_bytes, 256 << 20), seed=0)
            xh = rng.integers(-127, 128, (8, c), dtype=np.int8)
            xx = torch.from_numpy(xh).cuda()
            yy = torch.zeros((cp, r), dtype=torch.int32, device="cuda")
            launch_pass(mt, vl, xx, yy, r, c, cs["meta_stride"], cs["values_stride"], cp)
            torch.cuda.synchronize()
            want0 = oracle.sparse_gemv(cs["meta"], cs["values"], xh[0], r, c, threads=os.cpu_count() or 1)
            if not (yy[0].cpu().numpy() == want0).all():
                raise SystemExit(f"bench: {r}x{c} GEMV differs from the oracle; refusing to time it")
            g2 = capture(mt, vl, xx, yy, r, c, cs["meta_stride"], cs["values_stride"], cp, args.chains)
            us = time_graph(g2, 5, cp)
            gbs = pb / (us * 1e-6) / 1e9
            row = {"us_per_gemv": round(us, 3), "gbs": round(gbs, 1),
                   "frac_measured": round(gbs / peak, 4), "frac_8tbs": round(gbs / NOMINAL_HBM_GBS, 4)}
            if refcuda is not None:
                yy.zero_()
                g3 = capture_ref(mt, vl, xx, yy, r, c, cs["meta_stride"], cs["values_stride"], cp, args.chains)
                us_ref = time_graph(g3, 3, cp)
                ok = bool((yy[0].cpu().numpy() == want0).all())
                row["reference_kernel"] = {"us_per_gemv": round(us_ref, 3), "gbs": round(pb / (us_ref * 1e-6) / 1e9, 1),
                                           "frac_measured": round(pb / (us_ref * 1e-6) / 1e9 / peak, 4),
                                           "matches_oracle": ok, "speedup": round(us_ref / us, 2)}
                del g3
            sweep[f"{r}x{c}"] = row
            del mt, vl, yy, g2

    # ---- the GEMV on prepared weights (the packed format re-laid once, what an engine that owns its weights can
    #      use) beside the GEMV on the packed format, same graph of launches, on the shapes of the two models ----
    prepared = None
    if rank == 0 and not args.no_sweep:
        prepared = {"what": "us per GEMV / GB/s of algorithmic bytes, graph of launches in %d branches over weight copies "
                            "larger than L2; 'packed' is spb_sparse_ternary_gemv on the reference format, 'prepared' "
                            "spb_prepared_gemv on spb_prepare_weights' output (same bytes per weight)" % args.chains}
        for (r, c) in [(6912, 2560), (8192, 8192), (28672, 8192), (8192, 28672)]:
            try:
                meta, values = synth.device_sparse_matrix(r, c, seed=7)
                pb = synth.gemv_algorithmic_bytes(r, c)
                cp = min(64, max(8, int(np.ceil(max(2 * l2_bytes, 256 << 20) / pb))))
                mt = [meta.roll(i, 0) for i in range(cp)]
                vl = [values.roll(i, 0) for i in range(cp)]
                pr = [K.prepare_weights(mt[i], vl[i], r, c, c // 32, c // 64) for i in range(cp)]
                xx = torch.from_numpy(rng.integers(-127, 128, (8, c), dtype=np.int8)).cuda()
                ya = torch.zeros((cp, r), dtype=torch.int32, device="cuda")
                yb = torch.zeros((cp, r), dtype=torch.int32, device="cuda")
                row = {}
                for name in ("packed", "prepared"):
                    def one(i, name=name):
                        if name == "packed":
                            K.sparse_ternary_gemv_gpu(mt[i], vl[i], xx[i % 8], ya[i], r, c, c // 32, c // 64)
                        else:
                            K.prepared_gemv_gpu(pr[i], xx[i % 8], yb[i], r, c)
                    for i in range(cp):
                        one(i)
                    torch.cuda.synchronize()
                    g4 = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g4):
                        main = torch.cuda.current_stream()
                        for st in branch_streams[:args.chains]:
                            st.wait_stream(main)
                        for i in range(cp):
                            with torch.cuda.stream(branch_streams[i % max(args.chains, 1)]):
                                one(i)
                        for st in branch_streams[:args.chains]:
                            main.wait_stream(st)
                    us = time_graph(g4, 5, cp)
                    row[name] = {"us_per_gemv": round(us, 3), "gbs": round(pb / (us * 1e-6) / 1e9, 1),
                                 "frac_measured": round(pb / (us * 1e-6) / 1e9 / peak, 4)}
                    del g4
                row["same_result"] = bool((ya == yb).all().item())
                prepared[f"{r}x{c}"] = row
                del mt, vl, pr, ya, yb, meta, values
            except Exception as exc:
                prepared[f"{r}x{c}"] = {"error": repr(exc)[:160]}

    ref_cuda = None
    if refcuda is not None and "6912x2560" in sweep:
        ref_cuda = dict(sweep["6912x2560"].get("reference_kernel", {}),
                        what="reference sparse_ternary_gemv_kernel (src/kernels/sparse_ternary.cu:116-168) recompiled "
                             "for sm_100a, the same graph of launches over the same buffers as ours")

    # ---- CPU baselines (rank 0, N == 1) ------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baselines()

    gemm = None
    if rank == 0 and not args.no_gemm:
        try:
            gemm = bench_gemm(args, l2_bytes)
        except Exception as exc:
            gemm = {"error": repr(exc)}

    # ---- decode throughput on the 2B-4T-shape model: every rank runs its own replica -----------------
    decode = None
    if not args.no_decode:
        try:
            decode = bench_decode(args, with_reference=(rank == 0), with_cpu=(rank == 0 and world == 1 and not args.no_cpu))
        except Exception as exc:
            decode = {"error": repr(exc)}
        if world > 1:
            mine = torch.tensor([decode.get("tok_s", 0.0)], device="cuda", dtype=torch.float64)
            allv = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allv, mine)
            per_rank = [float(v.item()) for v in allv]
            decode["replicas"] = {"n": world, "tok_s_total": sum(per_rank), "tok_s_per_rank": per_rank,
                                  "what": "independent greedy-decode replicas, one per GPU, no communication"}

    # ---- the row-sharded 70B-shape decode on all ranks of this run ---------------------------------------
    sharded = None
    if not args.no_sharded:
        try:
            sharded = bench_sharded(args, rank, world, dist)
        except Exception as exc:
            sharded = {"error": repr(exc)[:300]}

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
            "sweep": sweep, "prepared_weights": prepared,
            "gemm": gemm,
            "decode": decode,
            "sharded": sharded,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def oracle_unpack(case, r, c):
    import oracle
    return oracle.unpack_to_int8(case["meta"], case["values"], r, c)


def _time_us(fn, reps=20, warm=3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def library_gemm(Wd, X, r, c, n, want):
    """Library kernels on a dense int8 copy of the same weights (comparison only; that copy stays resident in L2):
    cuBLASLt dense int8 (torch._int_mm) and cuSPARSELt 2:4 through oracle/cslt_shim.cpp, which follows the
    reference's CuSparseLtGemm: plan and compress once, then one cusparseLtMatmul per call, timed alone as a CUDA
    graph of 20 calls, result checked against the oracle."""
    import torch
    import oracle
    res = {}
    try:
        Wt = Wd.t()
        us = _time_us(lambda: torch._int_mm(X, Wt))
        res["lib_cublaslt_dense"] = {"us": round(us, 2), "dense_equiv_tops": round(2.0 * r * c * n / us / 1e6, 2)}
    except Exception as exc:
        res["lib_cublaslt_dense"] = {"error": str(exc)[:120]}
    try:
        if oracle.cslt() is None:
            raise RuntimeError("oracle/libspb_cslt.so not built or cuSPARSELt missing")
        gemm = oracle.CusparseLtGemm(r, c, n)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            gemm.prepare(Wd.data_ptr(), side.cuda_stream)
            D = torch.zeros((n, r), dtype=torch.int32, device="cuda")
            gemm.execute(X.data_ptr(), D.data_ptr(), side.cuda_stream)
            side.synchronize()
            ok = bool((D[:want.shape[0]].cpu().numpy() == want).all())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(20):
                    gemm.execute(X.data_ptr(), D.data_ptr(), side.cuda_stream)
            us = _time_us(g.replay, reps=5, warm=2) / 20
        torch.cuda.synchronize()
        res["lib_cusparselt"] = {"us": round(us, 2), "dense_equiv_tops": round(2.0 * r * c * n / us / 1e6, 2),
                                 "matches_oracle": ok}
        gemm.close()
    except Exception as exc:
        res["lib_cusparselt"] = {"error": str(exc)[:160]}
    return res


def sparse_int8_peak():
    """Empirical sparse-int8 tensor peak of this GPU: the library's own 2:4 kernel (cuSPARSELt through the shim) on
    a problem large enough to be compute-bound, in dense-equivalent TOP/s (2*M*K*N per call).  None when the
    library is missing."""
    import torch
    import oracle
    try:
        if oracle.cslt() is None:
            return None
        m = k = 8192
        n = 8192
        W = torch.zeros((m, k), dtype=torch.int8, device="cuda")
        W.view(m, k // 4, 4)[:, :, :2] = 1  # a valid 2:4 pattern
        X = torch.randint(-127, 128, (n, k), dtype=torch.int8, device="cuda")
        D = torch.empty((n, m), dtype=torch.int32, device="cuda")
        gemm = oracle.CusparseLtGemm(m, k, n)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            gemm.prepare(W.data_ptr(), side.cuda_stream)
            us = _time_us(lambda: gemm.execute(X.data_ptr(), D.data_ptr(), side.cuda_stream), reps=10, warm=3)
        torch.cuda.synchronize()
        gemm.close()
        return {"dense_equiv_tops": round(2.0 * m * k * n / us / 1e6, 1), "us": round(us, 1),
                "what": "cuSPARSELt int8 2:4, 8192 x 8192 x 8192, CUDA events over 10 calls"}
    except Exception as exc:
        return {"error": str(exc)[:160]}


def bench_gemm(args, l2_bytes):
    """Batched product (prefill) at the two FFN shapes, N in {1,4,16,64,256,1024}: us per call over a rotating set
    of weight copies larger than L2, weight-stream GB/s and dense-equivalent int8 TOP/s.  Every form's result is
    compared with the CPU oracle on a few activation rows before it is timed."""
    import torch
    import oracle
    from spbitnet_b200 import kernels as K, synth
    out = {}
    peak_hbm, _ = measured_peaks()
    sp_peak = None if args.gemm_shape else sparse_int8_peak()
    out["sparse_int8_peak"] = sp_peak
    peak_tops = (sp_peak or {}).get("dense_equiv_tops") or NOMINAL_SPARSE_INT8_TOPS
    threads = os.cpu_count() or 1
    shapes = synth.GEMM_SHAPES
    batches = synth.GEMM_BATCHES
    if args.gemm_shape:  # one shape, one batch size, no library arms: a small case for a profiler capture
        r_, c_ = (int(v) for v in args.gemm_shape.lower().split("x"))
        shapes, batches = [(r_, c_)], [args.gemm_n]
    for (r, c) in shapes:
        case = synth.gemv_case(r, c, seed=0)
        per = r * 4 * (case["meta_stride"] + case["values_stride"])
        copies = max(4, int(np.ceil(1.5 * l2_bytes / per)))
        meta = torch.from_numpy(case["meta"].view(np.int32)).cuda()
        values = torch.from_numpy(case["values"].view(np.int32)).cuda()
        metas = torch.stack([meta.roll(i, 0) for i in range(copies)]).contiguous()
        vals = torch.stack([values.roll(i, 0) for i in range(copies)]).contiguous()
        last_meta, last_values = np.roll(case["meta"], copies - 1, 0), np.roll(case["values"], copies - 1, 0)
        Wd = torch.from_numpy(oracle_unpack(case, r, c)).cuda()  # dense int8 copy, what the reference hands to cuSPARSELt
        for n in batches:
            X = torch.randint(-127, 128, (n, c), dtype=torch.int8, device="cuda")
            Y = torch.empty((n, r), dtype=torch.int32, device="cuda")
            Xh = X.cpu().numpy()
            probe = sorted({0, n // 2, n - 1})
            want = {j: oracle.sparse_gemv(last_meta, last_values, Xh[j], r, c, threads=threads) for j in probe}
            row = {}
            for name, variant in (("auto", 0), ("simt", 1), ("tc_sparse", 3), ("mma_sp", 4)):
                if args.gemm_shape and variant != 0:
                    continue
                if (variant == 1 and n > 64) or (variant == 3 and n < 16) or (variant == 4 and n > 256):
                    continue
                K.set_gemm_variant(variant)
                def run():
                    for i in range(copies):
                        K.sparse_ternary_gemm_gpu(metas[i], vals[i], X, Y, r, c, n, case["meta_stride"], case["values_stride"])
                Y.zero_()
                run()
                torch.cuda.synchronize()
                Yh = Y.cpu().numpy()  # the product with the last weight copy
                if any(not (Yh[j] == want[j]).all() for j in probe):
                    raise SystemExit(f"bench: batched product {r}x{c} n={n} ({name}) differs from the oracle; refusing to time it")
                # one CUDA graph of the `copies` calls (stream-ordered), so that the host's launch cost is not timed
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    run()
                us = _time_us(g.replay, reps=3, warm=1) / copies
                tops = 2.0 * r * c * n / us / 1e6
                gbs = (per + n * c + 4.0 * n * r) / us / 1e3
                row[name] = {"us": round(us, 2), "weight_gbs": round(per / us / 1e3, 1),
                             "dense_equiv_tops": round(tops, 2)}
                if name == "auto":
                    # the binding roof of this n: weights + X + Y over HBM, or 2*M*K*N over the sparse-int8 peak
                    t_hbm, t_tc = (per + n * c + 4.0 * n * r) / (peak_hbm * 1e3), 2.0 * r * c * n / (peak_tops * 1e6)
                    bound = "hbm" if t_hbm >= t_tc else "tensor"
                    row["roofline"] = {"bound": bound, "achieved": round(gbs if bound == "hbm" else tops, 1),
                                       "peak": peak_hbm if bound == "hbm" else peak_tops,
                                       "unit": "GB/s" if bound == "hbm" else "TOP/s (dense-equivalent)",
                                       "frac": round((t_hbm if bound == "hbm" else t_tc) / us, 4)}
            K.set_gemm_variant(0)
            if n >= 16 and not args.gemm_shape:
                # the libraries run on copy 0 of the weights
                w0 = oracle.sparse_gemv(case["meta"], case["values"], Xh[0], r, c, threads=threads)
                row.update(library_gemm(Wd, X, r, c, n, w0[None, :]))
            out[f"{r}x{c}_n{n}"] = row
        del metas, vals
    out["tc_timeouts"] = K.gemm_tc_timeouts()
    out["what"] = ("spb_sparse_ternary_gemm, us per call as a graph of stream-ordered calls over cold weights, each form "
                   "checked against the CPU oracle first; auto = warp-level sparse MMA (mma.sp) up to n = 32, tcgen05.mma.sp "
                   "above; lib_* = library kernels on a dense int8 copy of the weights that stays in L2 (comparison only: "
                   "cuBLASLt dense int8, and cuSPARSELt 2:4 planned and compressed once as the reference does); "
                   "dense_equiv_tops counts 2*M*K*N; roofline.peak for the tensor bound is sparse_int8_peak (measured "
                   "with the library) or the nominal 9000")
    return out


def bench_decode(args, with_reference=True, with_cpu=False):
    """Greedy decode of a random-init BitNet-2B-4T-shape model (every matrix of every layer with its own seed,
    generated on the GPU): 128-token prompt, 256 generated."""
    import torch
    from spbitnet_b200 import synth
    from spbitnet_b200.engine import InferenceEngine
    cfg = dict(synth.BITNET_2B)
    if args.decode_layers > 0:
        cfg["num_hidden_layers"] = args.decode_layers
    dm = synth.DeviceRandomModel(cfg, seed=0)
    eng = InferenceEngine(dm)
    prompt = np.random.default_rng(0).integers(0, cfg["vocab_size"], 128).astype(np.int32)
    n_gen = args.decode_tokens
    eng.generate(prompt, 8)  # warm-up: graph capture, page-in
    eng.reset()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    t0 = time.perf_counter()
    toks = eng.generate(prompt, n_gen)
    dt = time.perf_counter() - t0
    decode_clocks = sampler.stop()
    steps = len(prompt) - 1 + n_gen
    weight_bytes = dm.sparse_bytes() + dm.embed.numel() * 2
    # the same job with the layers of a token as one persistent kernel (opt-in mode of the engine)
    persistent = None
    try:
        eng.reset()
        eng.set_decode_mode(InferenceEngine.DECODE_PERSISTENT)
        eng.generate(prompt, 8)
        eng.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks_p = eng.generate(prompt, n_gen)
        dt_p2 = time.perf_counter() - t0
        persistent = {"tok_s": steps / dt_p2, "ms_per_token": 1e3 * dt_p2 / steps, "same_tokens": bool((toks_p == toks).all())}
    except Exception as exc:
        persistent = {"error": repr(exc)[:160]}
    # the default chain on the packed format (no prepared copies of the matrices)
    packed_chain = None
    try:
        eng.reset()
        eng.set_decode_mode(InferenceEngine.DECODE_AUTO)
        eng.set_prepared_weights(False)
        eng.generate(prompt, 8)
        eng.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks_p = eng.generate(prompt, n_gen)
        dt_p4 = time.perf_counter() - t0
        packed_chain = {"tok_s": steps / dt_p4, "ms_per_token": 1e3 * dt_p4 / steps, "same_tokens": bool((toks_p == toks).all())}
    except Exception as exc:
        packed_chain = {"error": repr(exc)[:160]}
    eng.set_prepared_weights(True)
    # ... and without grid barriers (stage outputs as tagged words)
    tagged = None
    try:
        eng.reset()
        eng.set_decode_mode(InferenceEngine.DECODE_PERSISTENT_TAGGED)
        eng.generate(prompt, 8)
        eng.reset()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks_p = eng.generate(prompt, n_gen)
        dt_p3 = time.perf_counter() - t0
        tagged = {"tok_s": steps / dt_p3, "ms_per_token": 1e3 * dt_p3 / steps, "same_tokens": bool((toks_p == toks).all())}
    except Exception as exc:
        tagged = {"error": repr(exc)[:160]}
    eng.reset()
    eng.set_decode_mode(InferenceEngine.DECODE_AUTO)
    # the same job with the prompt fed as one batch (BitLinear layers as the batched product)
    eng.reset()
    eng.set_prefill_chunk(256)
    for _ in range(2):  # the engine captures a prefill chunk's graph the second time it sees the same chunk: warm up past that
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
    peak, _ = measured_peaks()
    out = {"tok_s": steps / dt, "batched_prompt": batched, "ms_per_token": 1e3 * dt / steps, "generated": int(len(toks)),
           "prompt": int(len(prompt)), "weight_mb_per_token": round(weight_bytes / 1e6, 1),
           "step": "chain of five PDL-linked kernels per layer on prepared copies of the matrices", "chain_on_packed_weights": packed_chain, "persistent_kernel": persistent, "persistent_kernel_tagged_words": tagged, "clocks": decode_clocks,
           "hbm_gbs": weight_bytes * steps / dt / 1e9, "hbm_frac_measured": weight_bytes * steps / dt / 1e9 / peak,
           "what": "prefill (token-serial, as the reference) + decode, wall clock around generate() incl. prompt "
                   "H2D and token D2H; random-init 2B-4T shape, every matrix of every layer drawn with its own seed"}
    if with_reference:
        try:
            out["reference_engine_same_gpu"] = bench_reference_engine(dm, prompt)
        except Exception as exc:
            out["reference_engine_same_gpu"] = {"error": repr(exc)[:160]}
    if with_cpu:
        try:
            out["cpu_forward"] = bench_cpu_forward(dm)
        except Exception as exc:
            out["cpu_forward"] = {"error": repr(exc)[:160]}
    return out


def bench_reference_engine(dm, prompt, n_tokens=48):
    """The reference's forward pass op by op (src/inference.cu:123-283: ~28 launches + 2 copies per layer on the
    null stream, host arg-max as src/main.cpp:280-287) with the reference's own CUDA kernels recompiled for sm_100a,
    on the same device weights: tok/s over n_tokens greedy tokens after a 16-token prompt."""
    import torch
    import oracle
    if oracle.refcuda() is None:
        return None
    from oracle import ref_cuda_engine
    ref = ref_cuda_engine.RefCudaEngine(dm)
    for t in prompt[:16]:
        ref.forward(int(t))
    tok = int(prompt[16])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        tok = int(torch.argmax(ref.forward(tok)).item())
    dt = time.perf_counter() - t0
    return {"tok_s": n_tokens / dt, "ms_per_token": 1e3 * dt / n_tokens, "tokens": n_tokens,
            "what": "reference kernels (src/kernels/*.cu for sm_100a) in the reference's op order, launched from "
                    "Python through ctypes on the null stream, arg-max on the device; positions 16.."}


def bench_cpu_forward(dm):
    """The reference's forward pass on the host cores (the C port of src/inference.cu:123-283 in oracle/, one
    thread; python/baseline_pytorch.py InferenceEngine.forward is its Python twin): seconds per token at the
    model's full shape, one warm-up token and one timed token."""
    import oracle
    cpu = oracle.Engine(dm.to_host())
    cpu.forward(11)
    t0 = time.perf_counter()
    cpu.forward(12)
    dt = time.perf_counter() - t0
    return {"tok_s": 1.0 / dt, "s_per_token": dt, "cores": 1, "kind": "port",
            "sample": "one decode token at position 1 after one warm-up token, full model"}


def bench_sharded(args, rank, world, dist):
    """The Llama-70B-shaped ternary model (hidden 8192, 80 layers, 64 / 8 heads, FFN 28672, vocab 128256) row-sharded
    over the `world` GPUs of this run through spb_shard_engine (slices exchanged by peer stores + flags inside the
    captured step, no library collective on the data path): decode tok/s at batch 1 and batch 64 after a 512-token
    random-id prompt, and the fraction of the measured HBM bandwidth every GPU reaches on its own bytes.  With more
    than one rank a small model is first decoded sharded and on one rank: the logits must be bit-identical and the
    tokens the CPU oracle's, else nothing is timed."""
    import torch
    from spbitnet_b200 import synth
    from spbitnet_b200.shard_engine import ShardEngine
    peak, _ = measured_peaks()
    out = {"world": world}
    # The ranks' control plane here (barriers, the IPC handles, max over ranks) runs over a gloo group with a short
    # timeout: should a rank fail, the others get a Python exception within two minutes instead of sitting in a
    # device-side collective, and the run still prints its line.
    ctl = None
    if world > 1:
        import datetime
        torch.cuda.synchronize()
        dist.barrier()  # the ranks arrive here at different times (rank 0 ran the sweep and the batched product)
        ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=120))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=ctl)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ctl)
        return float(t.item())

    # ---- parity gate -------------------------------------------------------------------------------------
    if world > 1:
        small = dict(hidden_size=1024, num_hidden_layers=2, num_attention_heads=16, num_key_value_heads=8, head_dim=64,
                     intermediate_size=2048, vocab_size=4001, max_position_embeddings=64, rms_norm_eps=1e-5,
                     rope_theta=500000.0)
        dm = synth.DeviceRandomModel(small, seed=9)
        verdicts = []
        for batch in (1, 5):
            sharded, one = ShardEngine(dm, rank=rank, world=world, batch=batch, group=ctl), ShardEngine(dm, batch=batch)
            prompts = np.random.default_rng(7).integers(0, small["vocab_size"], (4, batch)).astype(np.int32)
            same = True
            for step in range(4):
                sharded.step(prompts[step])
                one.step(prompts[step])
                a, b = sharded.logits(), one.logits()
                same = same and bool((a.view(np.uint32) == b.view(np.uint32)).all())
            sharded.reset()
            one.reset()
            got = sharded.generate(prompts, 8)
            same = same and bool((got == one.generate(prompts, 8)).all())
            if rank == 0 and batch == 1:
                import oracle
                want, _ = oracle.Engine(dm.to_host()).generate(prompts[:, 0], 8)
                same = same and bool((got[:, 0] == want).all())
            verdicts.append(same)
            barrier()
            sharded.close()
            one.close()
        flag = torch.tensor([1.0 if all(verdicts) else 0.0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ctl)
        out["parity"] = "bit-identical" if flag.item() == 1.0 else "MISMATCH"
        out["parity_what"] = ("2-layer model (hidden 1024, 8 KV heads, vocab 4001), batch 1 and 5: logits of 4 steps equal "
                              "bit for bit to the same engine with one rank, 8 greedy tokens equal, batch-1 tokens equal to "
                              "the CPU oracle's")
        del dm
        if out["parity"] != "bit-identical":
            return out
    else:
        out["parity"] = "one rank (nothing to compare)"

    # ---- the 70B-shaped model: layer 0 drawn on the GPU, every further layer a separate copy of its slices -----
    cfg = dict(synth.LLAMA_70B_SHAPE, max_position_embeddings=args.shard_prompt + args.shard_tokens + 16)
    if args.shard_layers > 0:
        cfg["num_hidden_layers"] = args.shard_layers
    L = cfg["num_hidden_layers"]
    full = synth.DeviceRandomModel(dict(cfg, num_hidden_layers=1), seed=5)
    full.config = cfg
    full.layers = [full.layers[0]] * L  # ShardEngine clones the rank's slices layer by layer
    results = {}
    runs = [(1, 2), (64, 2)] + ([(1, 0)] if world > 1 else [])
    for batch, fold in runs:
        eng = ShardEngine(full, rank=rank, world=world, batch=batch, group=ctl)
        if fold != 2:  # the exchanges as launches of their own instead of in the producers' epilogues
            eng.set_exchange_fold(fold)
        rng = np.random.default_rng(11)
        prompts = rng.integers(0, cfg["vocab_size"], (args.shard_prompt, batch)).astype(np.int32)
        warm = eng.generate(prompts[:4], 2)  # graph capture, page-in
        eng.reset()
        barrier()
        t0 = time.perf_counter()
        first = eng.generate(prompts, 1)  # the prompt, step by step as the reference feeds it; one generated token
        t_prompt = max_over_ranks(time.perf_counter() - t0)
        barrier()
        t0 = time.perf_counter()
        toks = eng.generate(first[-1:], args.shard_tokens)
        dt = max_over_ranks(time.perf_counter() - t0)
        step_s = dt / args.shard_tokens
        kv_bytes = 2 * L * batch * (cfg["num_key_value_heads"] // world if world <= cfg["num_key_value_heads"] else 1) * \
            (args.shard_prompt + args.shard_tokens // 2) * cfg["head_dim"] * 2
        my_bytes = eng.weight_bytes() + kv_bytes
        results[f"batch{batch}" if fold == 2 else f"batch{batch}_exchange_as_launch"] = {
            "tok_s": batch * args.shard_tokens / dt, "ms_per_step": 1e3 * step_s,
            "prompt_s": t_prompt, "prompt_tok_s": batch * (args.shard_prompt - 1) / t_prompt,
            "per_gpu_bytes_per_step": int(my_bytes), "per_gpu_hbm_gbs": my_bytes / step_s / 1e9,
            "per_gpu_hbm_frac_measured": my_bytes / step_s / 1e9 / peak,
            "exchanges_per_step": 4 * L + 1, "tokens_checksum": int(np.asarray(toks, np.int64).sum() % 1000003)}
        eng.close()
        del eng
        torch.cuda.empty_cache()
    out.update(results)
    out["model"] = {"shape": "Llama-70B-shaped ternary 2:4", "layers": L, "hidden": cfg["hidden_size"],
                    "ffn": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "prompt": args.shard_prompt,
                    "generated": args.shard_tokens,
                    "weights": "one layer drawn at random, uploaded as a separate copy per layer (the HBM traffic is that "
                               "of distinct layers)"}
    out["what"] = ("row-sharded decode: every ternary matrix and the LM head split by output rows over the ranks, slices "
                   "exchanged inside the captured step over NVLink: the single-sequence step stores a slice from the epilogue "
                   "of the kernel that computes it, as tagged words, into every rank's staging area, where the consuming "
                   "kernel polls it (bounded); the batched step by a kernel that stores the slices into every peer's buffer "
                   "and waits (bounded) for the peers' flags; wall clock around generate(), max over ranks")
    return out


def bench_prefill(args):
    """The prompt as one batch through a random-init 2B-4T-shape model (engine.prefill), wall clock per call."""
    import torch
    from spbitnet_b200 import synth
    from spbitnet_b200.engine import InferenceEngine
    cfg = dict(synth.BITNET_2B)
    if args.decode_layers > 0:
        cfg["num_hidden_layers"] = args.decode_layers
    eng = InferenceEngine(synth.DeviceRandomModel(cfg, seed=0))
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
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--only-sharded", action="store_true", help="only the row-sharded 70B-shape decode")
    ap.add_argument("--shard-layers", type=int, default=0, help="override the layer count of the sharded model")
    ap.add_argument("--shard-prompt", type=int, default=512)
    ap.add_argument("--shard-tokens", type=int, default=48)
    ap.add_argument("--gemm-shape", default="", help="with --only-gemm: one ROWSxCOLS shape only, automatic form only")
    ap.add_argument("--gemm-n", type=int, default=1024, help="batch rows for --gemm-shape")
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
