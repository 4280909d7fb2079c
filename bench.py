"""Benchmark of the SVC -> vector-sparse SpMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the multi-GPU metric is quoted on): the conv-as-GEMM
set -- 8 pruned conv layers x sparsity {0.8, 0.9} x V {8, 16} = 32 products
C = A_vs * B with B = K x 25088 fp16 N(0,1), B and C sharded along N over the
ranks (strong scaling, no collective on the data path).  One step = all 32
products once.  The weights are compressed by the GPU SVC before timing.

One JSON line on stdout (rank 0).  `value` = useful TFLOP/s = 2*nnz*N_total summed
over the 32 products / device time of a step, operands resident in HBM; `e2e` =
the same with B coming from pinned host memory and C going back every step.
`--impl reference` times the reference's CPU path (restated in oracle/) on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import contextlib
import faulthandler
import io
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from sspmm_b200 import synthetic  # noqa: E402

METRIC = "useful_tflops_2nnzN"
UNIT = "TFLOP/s"
WORKLOAD = ("conv-as-GEMM pruned weights: 8 layers (Cout,K) in %s x sparsity {0.8,0.9} x V {8,16}, "
            "B = K x 25088 fp16 N(0,1), sharded along N" % (synthetic.CONV_LAYERS,))


def conv_problems():
    """(layer_id, sparsity_id, V) for the 32 products, ordered so that products
    sharing a layer are far apart within a step."""
    return [(l, s, V) for s in range(len(synthetic.CONV_SPARSITIES)) for V in (8, 16)
            for l in range(len(synthetic.CONV_LAYERS))]


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tensor_tflops": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "tensor_tflops_burst": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tensor_tflops": 1400.0, "tensor_tflops_burst": 1590.0, "source": "fallback"}


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in open(self.path):
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- #
# reference arm / CPU baseline (the only users of oracle/ in this file)
# --------------------------------------------------------------------------- #

def cpu_sample(n_cols: int = synthetic.CONV_N, target_rows: int = 32):
    """A bounded sample of the workload for the CPU: layer (512, 4608) at
    sparsity 0.9, V=16: the SVC of the whole layer, and the host SpMM on
    `target_rows` vector rows and `n_cols` columns of B."""
    from oracle import spmm_oracle, svc_oracle
    a = synthetic.conv_weight(3, 1)
    V = 16
    rows = a.row_lists()
    t0 = time.perf_counter()
    r = svc_oracle.cvse(a.M, a.K, a.nnz, rows, V)
    t_svc = time.perf_counter() - t0
    vals = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
    rng = np.random.default_rng(0)
    rhs = rng.normal(0, 1, (a.K, n_cols)).astype(np.float16)
    cores = os.cpu_count() or 1
    nrows = min(target_rows, r.num_vec_row)
    spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs, rows=(0, 1), threads=cores)  # warm
    t0 = time.perf_counter()
    spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs, rows=(0, nrows), threads=cores)
    t_spmm = time.perf_counter() - t0
    nnz_sample = int(a.row_ptr[nrows * V] - a.row_ptr[0])
    useful = 2.0 * nnz_sample * n_cols
    return {"svc_s": t_svc, "spmm_s": t_spmm, "useful_flops": useful, "cores": cores,
            "sample": f"layer (512,4608) s=0.9 V=16: SVC of the whole layer (1 core, CPython) + host fp32 SpMM on "
                      f"{nrows} of {r.num_vec_row} vector rows x {n_cols} of 25088 columns ({cores} OpenMP threads)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_sample(n_cols=128, target_rows=2)
    t_all, flops_all, last = 0.0, 0.0, None
    for _ in range(args.steps):
        last = cpu_sample()
        t_all += last["spmm_s"]
        flops_all += last["useful_flops"]
    val = flops_all / t_all / 1e12
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": last["sample"]},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": last["cores"], "kind": "port",
                             "sample": last["sample"], "svc_seconds_per_matrix": last["svc_s"]},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #

def run_ours(args):
    import torch
    import torch.distributed as dist

    from sspmm_b200 import build, capi, ops, parallel
    build.build()
    capi.lib()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    N_total = synthetic.CONV_N
    n0, n1 = parallel.shard_bounds(N_total, world)[rank]
    n_loc = n1 - n0
    peaks = load_peaks()

    # ---- operands: weights compressed on the GPU, one B and C per product
    probs = []
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    cache = {}
    todo = conv_problems()
    if args.only:
        todo = [tuple(int(x) for x in args.only.split(","))]
    for (l, s, V) in todo:
        if (l, s) not in cache:
            cache[(l, s)] = synthetic.conv_weight(l, s)
        a = cache[(l, s)]
        d_ptr = torch.from_numpy(a.row_ptr).to(dev)
        d_col = torch.from_numpy(a.col_idx).to(dev)
        d_val = torch.from_numpy(a.values).to(dev)
        vp, vc, vv, _ = ops.svc(d_ptr, d_col, d_val, a.M, a.K, V)
        m_vec = vp.numel() - 1
        nvec = vc.numel()
        B = torch.randn((a.K, n_loc), generator=g, device=dev, dtype=torch.float16)
        C = torch.empty((m_vec * V, n_loc), device=dev, dtype=torch.float16)
        k_used = int(torch.unique(vc).numel())
        probs.append(dict(l=l, s=s, V=V, M=a.M, K=a.K, nnz=a.nnz, m_vec=m_vec, nvec=nvec, k_used=k_used,
                          vp=vp, vc=vc, vv=vv, B=B, C=C))
    useful_flops_total = sum(2.0 * p["nnz"] * N_total for p in probs)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def launch(p):
        ops.sspmm(p["vp"], p["vc"], p["vv"], p["B"], p["V"], out=p["C"])

    # The products of a step are independent of one another, so they are issued round-robin on a few
    # streams (forked from and joined into the current stream): the tail of one product overlaps the head
    # of the next, and products with fewer tiles than SMs share the GPU.  With per-launch events
    # (evs != None) everything stays on the current stream so that each event pair brackets one product.
    side = [torch.cuda.Stream(device=dev) for _ in range(max(args.streams - 1, 0))]
    issue_order = list(range(len(probs)))

    def step(evs=None):
        if evs is not None or not side:
            for i, p in enumerate(probs):
                if evs is not None:
                    evs[i][0].record()
                launch(p)
                if evs is not None:
                    evs[i][1].record()
            return
        cur = torch.cuda.current_stream()
        lanes = [cur] + side
        for st in side:
            st.wait_stream(cur)
        for i, j in enumerate(issue_order):
            with torch.cuda.stream(lanes[i % len(lanes)]):
                launch(probs[j])
        for st in side:
            cur.wait_stream(st)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert ops.device_status() == 0

    # The 32 launches of a step are replayed from one CUDA graph (what a deployment
    # of a fixed layer stack does); falls back to eager launches if capture fails.
    run_step, graphed = step, False
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            torch.cuda.synchronize()
            run_step, graphed = graph.replay, True
        except Exception as exc:  # pragma: no cover - depends on driver support
            sys.stderr.write(f"CUDA graph capture failed, timing eager launches: {exc}\n")
            torch.cuda.synchronize()

    # ---- timed region: K steps, per-step and per-launch CUDA events on the launching stream
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    step_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    wall0 = time.perf_counter()
    for k in range(args.steps):
        flush.zero_()                       # evicts L2 between steps (outside the step's events)
        step_evs[k][0].record()
        run_step()
        step_evs[k][1].record()
    barrier()
    wall = time.perf_counter() - wall0
    # second, eager pass with an event pair around every launch: per-kernel durations for the roofline
    prof_steps = min(args.steps, 5)
    launch_evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in probs]
                  for _ in range(prof_steps)]
    step()                                  # one untimed eager step after the graph replays
    barrier()
    for k in range(prof_steps):
        flush.zero_()
        step(launch_evs[k])
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    step_ms = [a.elapsed_time(b) for a, b in step_evs]
    total_ms = float(sum(step_ms))
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = useful_flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel, from the per-launch events of this rank
    launch_ms = np.array([[a.elapsed_time(b) for a, b in row] for row in launch_evs])     # [steps, 32]
    per_prob_ms = launch_ms.mean(axis=0)
    f_alg = np.array([2.0 * p["nvec"] * p["V"] * n_loc for p in probs])
    b_alg = np.array([2.0 * p["V"] * p["nvec"] + 4.0 * p["nvec"] + 4.0 * (p["m_vec"] + 1) + 2.0 * p["k_used"] * n_loc
                      + 2.0 * p["m_vec"] * p["V"] * n_loc for p in probs])
    t_tensor = f_alg / (peaks["tensor_tflops"] * 1e12)
    t_hbm = b_alg / (peaks["hbm_gbs"] * 1e9)
    t_bound = np.maximum(t_tensor, t_hbm)
    # Duration of the step's kernels: the graph-replayed step (kernels back to back on the device).  The eager
    # per-launch events (per_prob_ms) also contain host launch gaps and are kept as the per-product breakdown.
    kernel_s = (float(sum(step_ms)) / args.steps if graphed else per_prob_ms.sum()) * 1e-3
    tensor_bound = bool(t_tensor.sum() >= t_hbm.sum())
    if tensor_bound:
        achieved = f_alg.sum() / kernel_s / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor_tflops"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tensor_tflops"]}
    else:
        achieved = b_alg.sum() / kernel_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"]}
    roof.update({"traffic": None, "peak_source": peaks["source"] + (" sustained bf16" if tensor_bound else " copy"),
                 "kernel": "sspmm_block_kernel (+ expand_transposed_kernel)", "t_bound_over_t": float(t_bound.sum() / kernel_s),
                 "algorithmic_flops_per_step": float(f_alg.sum()), "algorithmic_bytes_per_step": float(b_alg.sum()),
                 "kernel_ms_per_step": kernel_s * 1e3, "eager_per_launch_ms_per_step": float(per_prob_ms.sum()),
                 "launches_per_step": len(probs) * kernels_per_product()})
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        try:
            roof["traffic"] = json.load(open(traffic_file)).get("conv_step_dram_bytes")
        except Exception:
            pass

    # ---- end to end: B from pinned host memory, C back to the host, every step
    e2e = None
    e2e_steps = min(args.steps, 2)
    hostB = {}
    for p in probs:
        if p["K"] not in hostB:
            hostB[p["K"]] = torch.randn((p["K"], n_loc), dtype=torch.float16).pin_memory()
    hostC = {}
    for p in probs:
        key = p["m_vec"] * p["V"]
        if key not in hostC:
            hostC[key] = torch.empty((key, n_loc), dtype=torch.float16).pin_memory()
    h2d = sum(p["K"] * n_loc * 2 for p in probs)
    d2h = sum(p["m_vec"] * p["V"] * n_loc * 2 for p in probs)

    # Three streams: host->device copies, kernels, device->host copies; product p+1's B is on the wire while
    # product p computes and product p-1's C goes back (every product has its own device buffers).
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()

    def e2e_step():
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for p in probs:
            with torch.cuda.stream(s_in):
                p["B"].copy_(hostB[p["K"]], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            main.wait_event(ev_in)
            launch(p)
            ev_done = torch.cuda.Event()
            ev_done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done)
                hostC[p["m_vec"] * p["V"]].copy_(p["C"], non_blocking=True)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": useful_flops_total / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps}
    del hostB, hostC

    extras = {}
    if rank == 0:
        # ---- same-shape dense fp16 GEMM from the vendor library, for comparison only
        dense_ms = {}
        for p in probs:
            key = (p["m_vec"] * p["V"], p["K"])
            if key in dense_ms:
                continue
            A = torch.randn(key, device=dev, dtype=torch.float16)
            for _ in range(2):
                torch.matmul(A, p["B"])
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(5):
                torch.matmul(A, p["B"])
            a1.record()
            torch.cuda.synchronize()
            dense_ms[key] = a0.elapsed_time(a1) / 5
        dense_total = sum(dense_ms[(p["m_vec"] * p["V"], p["K"])] for p in probs)
        # the same 32 dense GEMMs issued like our step: round-robin on the same streams, replayed from a CUDA graph
        dense_A = {}
        for p in probs:
            key = (p["m_vec"] * p["V"], p["K"])
            if key not in dense_A:
                dense_A[key] = torch.randn(key, device=dev, dtype=torch.float16)

        def dense_step():
            cur = torch.cuda.current_stream()
            lanes = [cur] + side
            for st in side:
                st.wait_stream(cur)
            for i, p in enumerate(probs):
                with torch.cuda.stream(lanes[i % len(lanes)]):
                    torch.matmul(dense_A[(p["m_vec"] * p["V"], p["K"])], p["B"], out=p["C"])
            for st in side:
                cur.wait_stream(st)
        dense_streams_ms = None
        try:
            dense_step()
            torch.cuda.synchronize()
            dg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(dg):
                dense_step()
            dg.replay()
            torch.cuda.synchronize()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            tot = 0.0
            for _ in range(5):
                flush.zero_()
                a0.record()
                dg.replay()
                a1.record()
                torch.cuda.synchronize()
                tot += a0.elapsed_time(a1)
            dense_streams_ms = tot / 5
        except Exception as exc:  # pragma: no cover
            sys.stderr.write(f"dense comparator graph failed: {exc}\n")
            torch.cuda.synchronize()
        extras["comparators"] = {"cublas_dense_fp16": {
            "ms_per_step": dense_total, "ms_per_step_same_streams_graph": dense_streams_ms, "useful_tflops": 2.0 * sum(p["nnz"] for p in probs) * n_loc / dense_total / 1e9,
            "dense_tflops": sum(2.0 * p["m_vec"] * p["V"] * p["K"] * n_loc for p in probs) / dense_total / 1e9,
            "note": "torch.matmul (cuBLAS) on a dense M'xK matrix of the same shape, this rank's columns"}}
        extras["per_product"] = [
            {"layer": list(synthetic.CONV_LAYERS[p["l"]]), "sparsity": synthetic.CONV_SPARSITIES[p["s"]], "V": p["V"],
             "nvec": p["nvec"], "padding": p["nvec"] * p["V"] / p["nnz"], "us": float(per_prob_ms[i] * 1e3),
             "useful_tflops": 2.0 * p["nnz"] * n_loc / per_prob_ms[i] / 1e9,
             "vector_dense_tflops": float(f_alg[i] / per_prob_ms[i] / 1e9),
             "dense_equiv_tflops": 2.0 * p["M"] * p["K"] * n_loc / per_prob_ms[i] / 1e9,
             "gbs": float(b_alg[i] / per_prob_ms[i] / 1e6), "roofline_frac": float(t_bound[i] / (per_prob_ms[i] * 1e-3))}
            for i, p in enumerate(probs)]
        if not args.no_extras:
            extras["svc"] = bench_svc(torch, ops, dev)
            extras["ffn"] = bench_ffn(torch, ops, dev, peaks)
            extras["encoder_layer"] = bench_encoder(torch, dev)

    if not args.no_extras and not args.only:
        sweep = bench_sweep(torch, ops, dev, dist, rank, world)
        if rank == 0:
            extras["sweep"] = sweep

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        s = cpu_sample()
        cpu = {"value": s["useful_flops"] / s["spmm_s"] / 1e12, "unit": UNIT, "cores": s["cores"], "kind": "port",
               "sample": s["sample"], "svc_seconds_per_matrix": s["svc_s"]}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD if not args.only else "single product " + args.only, "N_total": N_total, "N_per_gpu": n_loc, "products_per_step": len(probs), "cuda_graph": graphed, "streams": args.streams,
                           "l2": "operands of a step exceed L2 and a 256 MiB buffer is written between steps",
                           "parallelism": f"B and C column-sharded over {world} GPU(s), A_vs replicated, no collective"},
                "roofline": roof, "cpu_baseline": cpu, "e2e": e2e,
                "gpu_launches": len(probs) * args.steps * kernels_per_product(), "clocks": clocks,
                "wall_s_timed_region": wall}
        line.update(extras)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def kernels_per_product() -> int:
    # block path: expansion kernel + GEMM kernel (the zero fill before them is a driver memset)
    return 2


def _cpu_svc_child(matrix_id, conn):
    """Child of cpu_svc_all_cores: builds its matrix, waits for the start signal, compresses, reports seconds."""
    from oracle import svc_oracle
    a = synthetic.sweep_matrix(matrix_id)
    rows = a.row_lists()
    conn.send("ready")
    conn.recv()
    t0 = time.perf_counter()
    svc_oracle.cvse(a.M, a.K, a.nnz, rows, 8)
    conn.send(time.perf_counter() - t0)
    conn.close()


def cpu_svc_all_cores(ids):
    """The CPython restatement on independent matrices, one process per matrix (the reference is single-threaded;
    a sweep can still be split over cores): matrices per second from the common start to the last finish."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")                      # the parent holds a CUDA context: no fork
    procs = []
    for i in ids:
        parent, child = ctx.Pipe()
        pr = ctx.Process(target=_cpu_svc_child, args=(i, child), daemon=True)
        pr.start()
        procs.append((pr, parent))
    for _, c in procs:
        if not c.poll(300):
            raise RuntimeError("CPU SVC worker did not start")
        c.recv()
    t0 = time.perf_counter()
    for _, c in procs:
        c.send("go")
    for _, c in procs:
        c.recv()
    wall = time.perf_counter() - t0
    for pr, _ in procs:
        pr.join(30)
    return len(ids) / wall


def bench_svc(torch, ops, dev, ids=(0, 1, 2, 3, 4, 5, 6, 7)):
    """SVC throughput on a sample of the power-law sweep (V=8): device-resident,
    through the host-buffer entry point, and the CPU oracle on one core."""
    from oracle import svc_oracle
    from sspmm_b200 import sparse_matrix_format as smf
    mats = [synthetic.sweep_matrix(i) for i in ids]
    dmats = [(torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev), torch.from_numpy(a.values).to(dev), a)
             for a in mats]
    for p, c, v, a in dmats:
        ops.svc(p, c, v, a.M, a.K, 8)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nbytes = 0
    for p, c, v, a in dmats:
        vp, vc, vv, _ = ops.svc(p, c, v, a.M, a.K, 8)
        nbytes += 4 * (a.M + 1) + 6 * a.nnz + 4 * vp.numel() + 4 * vc.numel() + 2 * vv.numel()
    torch.cuda.synchronize()
    t_dev = time.perf_counter() - t0
    # throughput mode: all matrices of the sample stacked into one pass
    batch_in = [(p, c, v, a.M, a.K) for p, c, v, a in dmats]
    ops.svc_batch(batch_in, 8)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        ops.svc_batch(batch_in, 8)
    torch.cuda.synchronize()
    t_batch = (time.perf_counter() - t0) / 3
    # larger stack: 32 matrices in one pass (the long vector rows of different matrices replay side by side)
    more = [synthetic.sweep_matrix(i) for i in range(len(ids), 32)]
    batch32 = batch_in + [(torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev),
                           torch.from_numpy(a.values).to(dev), a.M, a.K) for a in more]
    ops.svc_batch(batch32, 8)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(3):
        ops.svc_batch(batch32, 8)
    torch.cuda.synchronize()
    t_batch32 = (time.perf_counter() - t0) / 3
    del batch32, more
    # the SpMM of the same sweep matrices (B = n x 128)
    spmm = []
    for p, c, v, a in dmats:
        vp, vc, vv, _ = ops.svc(p, c, v, a.M, a.K, 8)
        B = torch.randn((a.K, 128), device=dev, dtype=torch.float16)
        C = torch.empty(((vp.numel() - 1) * 8, 128), device=dev, dtype=torch.float16)
        for _ in range(3):
            ops.sspmm(vp, vc, vv, B, 8, out=C)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.sspmm(vp, vc, vv, B, 8, out=C)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        b_alg = 2 * 8 * vc.numel() + 4 * vc.numel() + 4 * vp.numel() + 2 * a.K * 128 + 2 * C.numel()
        spmm.append({"n": a.M, "us": ms * 1e3, "useful_tflops": 2.0 * a.nnz * 128 / ms / 1e9,
                     "algorithmic_gbs": b_alg / ms / 1e6, "gather_gbs": 2.0 * vc.numel() * 128 / ms / 1e6})
    row_lists = [a.row_lists() for a in mats]          # the caller's data structure (lists of lists), built outside the clock
    t0 = time.perf_counter()
    for a, rows in zip(mats, row_lists):
        smf.CVSE(a.M, a.K, a.nnz, rows, 8)
    t_host_api = time.perf_counter() - t0
    t0 = time.perf_counter()
    for a, rows in zip(mats, row_lists):
        svc_oracle.cvse(a.M, a.K, a.nnz, rows, 8)
    t_cpu = time.perf_counter() - t0
    try:
        cpu_all = cpu_svc_all_cores(list(ids))
    except Exception as exc:  # pragma: no cover - depends on the host
        sys.stderr.write(f"all-core CPU SVC measurement skipped: {exc}\n")
        cpu_all = None
    return {"sample": f"sweep matrices {list(ids)} (n = {[a.M for a in mats]}), V=8",
            "device_matrices_per_s": len(mats) / t_dev, "device_gbs": nbytes / t_dev / 1e9,
            "device_batched_matrices_per_s": len(mats) / t_batch, "speedup_batched_vs_cpu": t_cpu / t_batch,
            "device_batched32_matrices_per_s": 32 / t_batch32,
            "python_entry_point_matrices_per_s": len(mats) / t_host_api,
            "cpu_oracle_matrices_per_s_1core": len(mats) / t_cpu, "speedup_device_vs_cpu": t_cpu / t_dev,
            "cpu_oracle_matrices_per_s_one_process_per_matrix": cpu_all, "cpu_cores": os.cpu_count(),
            "spmm_n128": spmm}


def bench_sweep(torch, ops, dev, dist, rank, world, per_rank=8):
    """The power-law sweep distributed over ranks (matrix_id mod world): every rank compresses its
    matrices (V=8) and multiplies each by B = n x 128; wall time of the slowest rank, device-resident
    inputs, no collective on the data path."""
    ids = [rank + world * k for k in range(per_rank)]
    mats = [synthetic.sweep_matrix(i) for i in ids]
    dmats = [(torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev), torch.from_numpy(a.values).to(dev),
              a, torch.randn((a.K, 128), device=dev, dtype=torch.float16)) for a in mats]

    def one_pass():
        # the rank's matrices are compressed in one stacked pass, then multiplied one by one
        parts, _ = ops.svc_batch([(p, c, v, a.M, a.K) for p, c, v, a, B in dmats], 8)
        for (vp, vc, vv), (p, c, v, a, B) in zip(parts, dmats):
            ops.sspmm(vp, vc, vv, B, 8)

    one_pass()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    one_pass()
    torch.cuda.synchronize()
    t = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
    nnz = torch.tensor([float(sum(a.nnz for a in mats))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nnz, op=dist.ReduceOp.SUM)
    sec = float(t.item())
    return {"matrices": per_rank * world, "matrices_per_rank": per_rank, "seconds_slowest_rank": sec,
            "svc_plus_spmm_matrices_per_s": per_rank * world / sec,
            "useful_tflops_n128": 2.0 * float(nnz.item()) * 128 / sec / 1e12,
            "note": "matrix_id mod world -> rank; SVC (V=8) of the rank's matrices in one stacked pass, then SpMM with B = n x 128 per matrix; weak scaling"}


def bench_encoder(torch, dev):
    """Sparse transformer encoder layer: hidden 768, FFN 3072, 12 heads, seq 512, batch 32, all six weight
    matrices pruned to 90 % and compressed at V=16; attention and LayerNorm dense."""
    from sspmm_b200.encoder import SparseEncoderLayer
    layer = SparseEncoderLayer(hidden=768, ffn=3072, heads=12, sparsity=0.9, vec_length=16, device=dev)
    batch, seq = 32, 512
    x = torch.randn(768, batch * seq, device=dev, dtype=torch.float16)

    def t(dense, it=10):
        for _ in range(3):
            layer.forward(x, batch, seq, dense=dense)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(it):
            layer.forward(x, batch, seq, dense=dense)
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / it
    ms_sparse, ms_dense = t(False), t(True)
    nnz = sum(l.nnz for l in layer.linears)
    return {"config": "hidden 768, ffn 3072, 12 heads, seq 512, batch 32, weights 90 % sparse, V=16",
            "ms_sparse_weights": ms_sparse, "ms_dense_weights_cublas": ms_dense,
            "linear_useful_tflops": 2.0 * nnz * batch * seq / ms_sparse / 1e9,
            "note": "whole layer incl. dense attention and LayerNorm; the useful-flop figure counts the six linears only"}


def bench_ffn(torch, ops, dev, peaks):
    """FFN configuration (V=16, N=256): single-call latency per matrix."""
    out = []
    for shape_id in range(2):
        for sid in range(len(synthetic.FFN_SPARSITIES)):
            a, rhs = synthetic.ffn(shape_id, sid)
            vp, vc, vv, _ = ops.svc(torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev),
                                    torch.from_numpy(a.values).to(dev), a.M, a.K, 16)
            B = torch.from_numpy(rhs).to(dev)
            C = torch.empty((vp.numel() - 1) * 16, 256, device=dev, dtype=torch.float16)
            A = torch.randn((a.M, a.K), device=dev, dtype=torch.float16)

            def t(fn, it=20):
                for _ in range(3):
                    fn()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(it):
                    fn()
                a1.record()
                torch.cuda.synchronize()
                return a0.elapsed_time(a1) / it

            def t_graph(fn, it=20):
                """Same call captured `it` times into one CUDA graph: device time per call without host launch cost."""
                try:
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        for _ in range(it):
                            fn()
                    g.replay()
                    torch.cuda.synchronize()
                    return t(g.replay, it=5) / it
                except Exception:
                    torch.cuda.synchronize()
                    return None
            Cd = torch.empty((a.M, 256), device=dev, dtype=torch.float16)
            ms = t(lambda: ops.sspmm(vp, vc, vv, B, 16, out=C))
            ms_d = t(lambda: torch.matmul(A, B, out=Cd))
            ms_g = t_graph(lambda: ops.sspmm(vp, vc, vv, B, 16, out=C))
            ms_dg = t_graph(lambda: torch.matmul(A, B, out=Cd))
            out.append({"shape": list(synthetic.FFN_SHAPES[shape_id]), "sparsity": synthetic.FFN_SPARSITIES[sid],
                        "us": ms * 1e3, "useful_tflops": 2.0 * a.nnz * 256 / ms / 1e9, "cublas_dense_us": ms_d * 1e3,
                        "cublas_useful_tflops": 2.0 * a.nnz * 256 / ms_d / 1e9, "padding": vc.numel() * 16 / a.nnz,
                        "us_in_graph": None if ms_g is None else ms_g * 1e3,
                        "cublas_dense_us_in_graph": None if ms_dg is None else ms_dg * 1e3})
    return {"note": "back-to-back launches, operands L2-resident (problem is ~1-4 MB): latency, not bandwidth",
            "cases": out}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--streams", type=int, default=8, help="streams the independent products of a step are issued on")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA graph of the step")
    ap.add_argument("--no-extras", action="store_true", help="skip the SVC and FFN side measurements")
    ap.add_argument("--only", default="", help="layer_id,sparsity_id,V: run a single product (profiling captures)")
    args = ap.parse_args()
    # a run that stalls ends with a traceback on stderr instead of holding the GPU until it is killed
    faulthandler.dump_traceback_later(1500, exit=True)
    # stdout carries exactly one JSON line: anything libraries print (NCCL banner, ...) goes to stderr
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        if args.impl == "reference":
            run_reference(args)
        else:
            run_ours(args)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    lines = [ln for ln in out.getvalue().splitlines() if ln.startswith("{")]
    if lines:
        print(lines[-1], flush=True)


if __name__ == "__main__":
    main()
