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

CPU_SAMPLE_COLS = 6272          # of 25088


def cpu_products():
    """The 32 products of the workload, compressed by the CPU oracle (CPython SVC, one core); returns the list
    and the seconds the 32 compressions took."""
    from oracle import svc_oracle
    out, t_svc, cache = [], 0.0, {}
    for (l, s, V) in conv_problems():
        if (l, s) not in cache:
            cache[(l, s)] = synthetic.conv_weight(l, s)
        a = cache[(l, s)]
        rows = a.row_lists()
        t0 = time.perf_counter()
        r = svc_oracle.cvse(a.M, a.K, a.nnz, rows, V)
        t_svc += time.perf_counter() - t0
        vals = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
        out.append(dict(l=l, s=s, V=V, a=a, ptr=np.asarray(r.vec_row_ptr, dtype=np.int32),
                        col=np.asarray(r.vec_colInd_list, dtype=np.int32), vals=vals))
    return out, t_svc


def cpu_step(prods, rhs_by_k, cores, n_cols=CPU_SAMPLE_COLS, keep=None):
    """One bounded pass of the reference's host SpMM over the SAME 32 products: for every product the first
    min(m_vec, cores) vector rows (one per OpenMP thread) times the first n_cols columns of B.  Returns
    (seconds, useful flops of the sample).  keep: dict that receives the computed rows (for validation)."""
    from oracle import spmm_oracle
    t_all, flops = 0.0, 0.0
    for i, p in enumerate(prods):
        a, V = p["a"], p["V"]
        m_vec = p["ptr"].size - 1
        nrows = min(m_vec, cores)
        rhs = rhs_by_k[a.K][:, :n_cols]
        t0 = time.perf_counter()
        ref = spmm_oracle.sspmm_host(V, p["ptr"], p["col"], p["vals"], rhs, rows=(0, nrows), threads=cores)
        t_all += time.perf_counter() - t0
        nnz_sample = int(a.row_ptr[min(nrows * V, a.M)] - a.row_ptr[0])
        flops += 2.0 * nnz_sample * n_cols
        if keep is not None:
            keep[i] = ref
    return t_all, flops


def cpu_sample_text(cores):
    return (f"all 32 products of the workload, each on its first min(m_vec, {cores}) vector rows x the first {CPU_SAMPLE_COLS} of "
            f"25088 columns of B (host fp32 SpMM, {cores} OpenMP threads); SVC of the 32 operands by the CPython restatement on 1 core")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    prods, t_svc = cpu_products()
    rng = np.random.default_rng(0)
    rhs_by_k = {}
    for p in prods:
        K = p["a"].K
        if K not in rhs_by_k:
            rhs_by_k[K] = rng.normal(0, 1, (K, CPU_SAMPLE_COLS)).astype(np.float16)
    for _ in range(args.warmup):
        cpu_step(prods, rhs_by_k, cores, n_cols=64)
    t_all, flops_all = 0.0, 0.0
    for _ in range(args.steps):
        t, f = cpu_step(prods, rhs_by_k, cores)
        t_all += t
        flops_all += f
    val = flops_all / t_all / 1e12
    sample = cpu_sample_text(cores)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * t_all / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": sample},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                             "svc_seconds_32_operands_1core": t_svc},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #

def numa_bind(local_rank: int):
    """Runs this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers
    allocated afterwards are local to the GPU's PCIe root.  Returns a short description (or why not)."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = getattr(torch.cuda.get_device_properties(local_rank), "pci_domain_id", 0)
        dev = getattr(torch.cuda.get_device_properties(local_rank), "pci_device_id", 0)
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return "GPU reports no NUMA node"
        cpus = open(f"/sys/devices/system/node/node{node}/cpulist").read().strip()
        ids = set()
        for part in cpus.split(","):
            lo, _, hi = part.partition("-")
            ids.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0) & ids
        if not allowed:
            return f"node {node}: none of its CPUs is available to this process"
        os.sched_setaffinity(0, allowed)
        return f"node {node} ({len(allowed)} CPUs)"
    except Exception as exc:  # pragma: no cover - depends on the host
        return f"not bound: {exc}"


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
    numa = numa_bind(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    N_total = synthetic.CONV_N
    n0, n1 = parallel.shard_bounds(N_total, world)[rank]
    n_loc = n1 - n0
    peaks = load_peaks()

    # ---- operands: weights compressed on the GPU; all B (and all C) of the rank in one buffer each, so that the
    # end-to-end path can move them with a few large copies
    todo = conv_problems()
    if args.only:
        todo = [tuple(int(x) for x in args.only.split(","))]
    cache, meta = {}, []
    for (l, s, V) in todo:
        if (l, s) not in cache:
            cache[(l, s)] = synthetic.conv_weight(l, s)
        a = cache[(l, s)]
        meta.append((l, s, V, a, (a.M + V - 1) // V))
    b_elems = [a.K * n_loc for (_, _, _, a, _) in meta]
    c_elems = [mv * V * n_loc for (_, _, V, _, mv) in meta]
    allB = torch.empty(sum(b_elems), device=dev, dtype=torch.float16)
    allC = torch.empty(sum(c_elems), device=dev, dtype=torch.float16)
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    allB.normal_(0, 1, generator=g)
    probs, bo, co = [], 0, 0
    for i, (l, s, V, a, m_vec) in enumerate(meta):
        d_ptr = torch.from_numpy(a.row_ptr).to(dev)
        d_col = torch.from_numpy(a.col_idx).to(dev)
        d_val = torch.from_numpy(a.values).to(dev)
        vp, vc, vv, _ = ops.svc(d_ptr, d_col, d_val, a.M, a.K, V)
        B = allB[bo: bo + b_elems[i]].view(a.K, n_loc)
        C = allC[co: co + c_elems[i]].view(m_vec * V, n_loc)
        plan = ops.Plan(vp, vc, V, a.K)
        probs.append(dict(l=l, s=s, V=V, M=a.M, K=a.K, nnz=a.nnz, m_vec=m_vec, nvec=vc.numel(),
                          k_used=int(torch.unique(vc).numel()), vp=vp, vc=vc, vv=vv, B=B, C=C, plan=plan,
                          b_off=bo, c_off=co))
        bo += b_elems[i]
        co += c_elems[i]
    useful_flops_total = sum(2.0 * p["nnz"] * N_total for p in probs)
    flush = L2Flush(torch, dev)

    # ---- one step = every product once = ONE group run = one persistent tensor-core launch (see sspmm_group_create)
    if not all(p["plan"].one_launch for p in probs):
        raise RuntimeError("a conv operand did not qualify for the grouped kernel")
    group = ops.Group([(p["plan"], p["vv"], p["B"], p["C"]) for p in probs], mode=args.group_mode)
    step = group.run
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert ops.device_status() == 0

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
            sys.stderr.write(f"CUDA graph capture failed, timing plain launches: {exc}\n")
            torch.cuda.synchronize()

    # ---- timed region: K steps, L2 flushed before each, CUDA events on the launching stream
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    step_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    wall0 = time.perf_counter()
    for k in range(args.steps):
        flush()                             # evicts L2 between steps (outside the step's events)
        step_evs[k][0].record()
        run_step()
        step_evs[k][1].record()
    barrier()
    wall = time.perf_counter() - wall0
    step_ms = [a.elapsed_time(b) for a, b in step_evs]
    c0_timed = probs[0]["C"].clone()        # result of the timed step, compared with the end-to-end path below
    ms_per_step = max_over_ranks(float(sum(step_ms))) / args.steps
    value = useful_flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- the same step back to back for about a second (operands of a step exceed L2, so no flush is needed):
    # what the kernels sustain under the power limit, with the clocks seen meanwhile
    reps = max(20, int(1000.0 / max(ms_per_step, 1e-3)))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s0.record()
    for _ in range(reps):
        run_step()
    s1.record()
    barrier()
    sustained_ms = max_over_ranks(s0.elapsed_time(s1)) / reps
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the dominant kernel (the grouped tensor-core kernel), live from the timed region
    launches_per_step = group.launches
    f_alg = np.array([2.0 * p["nvec"] * p["V"] * n_loc for p in probs])
    b_alg = np.array([2.0 * p["V"] * p["nvec"] + 4.0 * p["nvec"] + 4.0 * (p["m_vec"] + 1) + 2.0 * p["k_used"] * n_loc
                      + 2.0 * p["m_vec"] * p["V"] * n_loc for p in probs])
    step_s = float(sum(step_ms)) / args.steps * 1e-3            # this rank's own steps
    t_tensor = f_alg.sum() / (peaks["tensor_tflops_burst"] * 1e12)
    t_hbm = b_alg.sum() / (peaks["hbm_gbs"] * 1e9)
    tensor_bound = bool(t_tensor >= t_hbm)
    if tensor_bound:
        achieved = f_alg.sum() / step_s / 1e12
        roof = {"bound": "tensor", "achieved": achieved, "peak": peaks["tensor_tflops_burst"], "unit": "TFLOP/s",
                "frac": achieved / peaks["tensor_tflops_burst"],
                "peak_source": peaks["source"] + " bf16 burst (a step is a millisecond-scale region)"}
    else:
        achieved = b_alg.sum() / step_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"] + " copy"}
    sus_tf = f_alg.sum() / (sustained_ms * 1e-3) / 1e12
    roof.update({"traffic": None, "kernel": "sspmm_fused_pair_kernel" if args.group_mode == 3 else "sspmm_fused_kernel",
                 "t_hbm_over_t": float(t_hbm / step_s), "t_tensor_over_t": float(t_tensor / step_s),
                 "algorithmic_flops_per_step": float(f_alg.sum()), "algorithmic_bytes_per_step": float(b_alg.sum()),
                 "hbm_gbs_algorithmic": float(b_alg.sum() / step_s / 1e9),
                 "kernel_ms_per_step": step_s * 1e3, "launches_per_step": launches_per_step,
                 "sustained": {"ms_per_step": sustained_ms, "steps": reps, "achieved": sus_tf,
                               "peak": peaks["tensor_tflops"], "frac": sus_tf / peaks["tensor_tflops"],
                               "note": "same step back to back for about a second, against the sustained bf16 peak"}})
    # the slower-of rule product by product: the layers differ in flops per byte by a factor of nine, so the sum of the
    # per-product bounds is a tighter floor than the bound of the sums
    t_each = np.maximum(f_alg / (peaks["tensor_tflops_burst"] * 1e12), b_alg / (peaks["hbm_gbs"] * 1e9))
    roof["per_product_bound"] = {"ms_per_step": float(t_each.sum() * 1e3), "frac": float(t_each.sum() / step_s),
                                 "note": "sum over the products of max(F_alg / burst bf16 peak, B_alg / copy bandwidth), over the step time"}
    traffic_file = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(traffic_file):
        try:
            roof["traffic"] = json.load(open(traffic_file)).get("conv_step_dram_bytes")
        except Exception:
            pass

    # ---- per product, through the reference-signature entry point (sspmm_f16_f16), one after another: breakdown only
    prof_steps = min(args.steps, 3)
    launch_evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in probs]
                  for _ in range(prof_steps)]
    for p in probs:
        ops.sspmm(p["vp"], p["vc"], p["vv"], p["B"], p["V"], out=p["C"])
    barrier()
    for k in range(prof_steps):
        flush()
        for i, p in enumerate(probs):
            launch_evs[k][i][0].record()
            ops.sspmm(p["vp"], p["vc"], p["vv"], p["B"], p["V"], out=p["C"])
            launch_evs[k][i][1].record()
    barrier()
    per_prob_ms = np.array([[a.elapsed_time(b) for a, b in row] for row in launch_evs]).mean(axis=0)

    # ---- end to end: every step B comes from pinned host memory and C goes back, through the same C-ABI group
    # calls.  The products are cut into chunks that are contiguous in the operand buffers: one copy in, one group
    # run, one copy out per chunk, on three streams, so that chunk c+1 is on the wire while chunk c computes.
    e2e_steps = max(args.steps, 10)
    n_chunks = min(4, len(probs))
    bounds = [round(i * len(probs) / n_chunks) for i in range(n_chunks + 1)]
    chunks = []
    for c in range(n_chunks):
        ps = probs[bounds[c]: bounds[c + 1]]
        b0, b1 = ps[0]["b_off"], ps[-1]["b_off"] + ps[-1]["K"] * n_loc
        c0, c1 = ps[0]["c_off"], ps[-1]["c_off"] + ps[-1]["m_vec"] * ps[-1]["V"] * n_loc
        chunks.append(dict(group=ops.Group([(p["plan"], p["vv"], p["B"], p["C"]) for p in ps], mode=args.group_mode),
                           b=(b0, b1), c=(c0, c1)))
    hostB = torch.empty(allB.numel(), dtype=torch.float16).pin_memory()
    hostC = torch.empty(allC.numel(), dtype=torch.float16).pin_memory()
    hostB.copy_(allB)                       # the same operands, so the result can be checked below
    h2d, d2h = allB.numel() * 2, allC.numel() * 2
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()

    def e2e_step():
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for ch in chunks:
            with torch.cuda.stream(s_in):
                allB[ch["b"][0]: ch["b"][1]].copy_(hostB[ch["b"][0]: ch["b"][1]], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            main.wait_event(ev_in)
            ch["group"].run()
            ev_done = torch.cuda.Event()
            ev_done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done)
                hostC[ch["c"][0]: ch["c"][1]].copy_(allC[ch["c"][0]: ch["c"][1]], non_blocking=True)
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
    e2e_own_ms = e0.elapsed_time(e1) / e2e_steps
    e2e_ms = max_over_ranks(e2e_own_ms)
    e2e = {"value": useful_flops_total / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
           "ms_per_step": e2e_ms, "copies_per_step": 2 * n_chunks,
           "rank0_h2d_gbs_if_copy_bound": h2d / (e2e_own_ms * 1e-3) / 1e9, "rank0_d2h_gbs_if_copy_bound": d2h / (e2e_own_ms * 1e-3) / 1e9,
           "numa": numa, "note": "bytes are this rank's; copies in and out run concurrently with each other and with the kernels"}
    e2e_same = bool(torch.equal(hostC[: c0_timed.numel()].view_as(c0_timed), c0_timed.cpu()))
    e2e["first_product_bit_equal_to_timed_step"] = e2e_same
    del hostB, hostC, chunks

    extras = {}
    if rank == 0:
        # ---- comparators on the same GPU, for comparison only (never on the product path)
        comp = {}
        dense_A = {}
        for p in probs:
            key = (p["m_vec"] * p["V"], p["K"])
            if key not in dense_A:
                dense_A[key] = torch.randn(key, device=dev, dtype=torch.float16)

        def event_ms(fn, it=5):
            tot = 0.0
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(it):
                flush()
                a0.record()
                fn()
                a1.record()
                torch.cuda.synchronize()
                tot += a0.elapsed_time(a1)
            return tot / it

        dense_C = torch.empty(max(p["m_vec"] * p["V"] for p in probs) * n_loc, device=dev, dtype=torch.float16)
        lane_C = [dense_C] + [torch.empty_like(dense_C) for _ in range(7)]      # one output buffer per stream

        def dense_seq():
            for p in probs:
                M_ = p["m_vec"] * p["V"]
                torch.matmul(dense_A[(M_, p["K"])], p["B"], out=dense_C[: M_ * n_loc].view(M_, n_loc))
        dense_seq()
        dense_total = event_ms(dense_seq)
        # the same 32 dense GEMMs on eight streams, replayed from a CUDA graph (the best way found to issue them)
        side = [torch.cuda.Stream(device=dev) for _ in range(7)]

        def dense_streams():
            cur = torch.cuda.current_stream()
            lanes = [cur] + side
            for st in side:
                st.wait_stream(cur)
            for i, p in enumerate(probs):
                with torch.cuda.stream(lanes[i % len(lanes)]):
                    M_ = p["m_vec"] * p["V"]
                    torch.matmul(dense_A[(M_, p["K"])], p["B"], out=lane_C[i % len(lanes)][: M_ * n_loc].view(M_, n_loc))
            for st in side:
                cur.wait_stream(st)
        dense_streams_ms = None
        try:
            dense_streams()
            torch.cuda.synchronize()
            dg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(dg):
                dense_streams()
            dg.replay()
            torch.cuda.synchronize()
            dense_streams_ms = event_ms(dg.replay)
        except Exception as exc:  # pragma: no cover
            sys.stderr.write(f"dense comparator graph failed: {exc}\n")
            torch.cuda.synchronize()
        comp["cublas_dense_fp16"] = {
            "ms_per_step": dense_total, "ms_per_step_8_streams_graph": dense_streams_ms,
            "useful_tflops": 2.0 * sum(p["nnz"] for p in probs) * n_loc / dense_total / 1e9,
            "dense_tflops": sum(2.0 * p["m_vec"] * p["V"] * p["K"] * n_loc for p in probs) / dense_total / 1e9,
            "note": "torch.matmul (cuBLAS) on a dense M'xK matrix of the same shape, this rank's columns"}
        del lane_C, dense_C
        comp["reference_gpu_kernel"] = reference_kernel_comparator(torch, ops, probs, n_loc, dev, flush)
        extras["comparators"] = comp
        extras["per_product"] = [
            {"layer": list(synthetic.CONV_LAYERS[p["l"]]), "sparsity": synthetic.CONV_SPARSITIES[p["s"]], "V": p["V"],
             "nvec": p["nvec"], "padding": p["nvec"] * p["V"] / p["nnz"], "us": float(per_prob_ms[i] * 1e3),
             "useful_tflops": 2.0 * p["nnz"] * n_loc / per_prob_ms[i] / 1e9,
             "vector_dense_tflops": float(f_alg[i] / per_prob_ms[i] / 1e9),
             "dense_equiv_tflops": 2.0 * p["M"] * p["K"] * n_loc / per_prob_ms[i] / 1e9,
             "gbs": float(b_alg[i] / per_prob_ms[i] / 1e6)}
            for i, p in enumerate(probs)]
        extras["per_product_note"] = ("each product alone through sspmm_f16_f16 (the reference-signature entry point: "
                                      "expansion + GEMM launches, scratch from the stream-ordered allocator), one after another")
        if not args.no_extras:
            extras["svc"] = bench_svc(torch, ops, dev)
            extras["ffn"] = bench_ffn(torch, ops, dev, peaks)
            extras["encoder_layer"] = bench_encoder(torch, dev)

    if not args.no_extras and not args.only:
        sweep = bench_sweep(torch, ops, dev, dist, rank, world, args.sweep_matrices)
        if rank == 0:
            extras["sweep"] = sweep

    # ---- CPU baseline (rank 0, one GPU): the reference's CPU path on a bounded sample of the same 32 products,
    # and with it the check that what was timed is right: the CPU rows against the GPU's C of the timed step
    cpu, validated = None, None
    if rank == 0 and world == 1 and not args.no_cpu and not args.only:
        cores = os.cpu_count() or 1
        cprods, t_svc = cpu_products()
        rhs_by_k = {}
        for p in probs:                                  # the GPU's own B, products sharing K share the first one's
            if p["K"] not in rhs_by_k:
                rhs_by_k[p["K"]] = p["B"][:, :CPU_SAMPLE_COLS].cpu().numpy()
        keep = {}
        t_cpu, f_cpu = cpu_step(cprods, rhs_by_k, cores, keep=keep)
        cpu = {"value": f_cpu / t_cpu / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "sample": cpu_sample_text(cores),
               "seconds": t_cpu, "svc_seconds_32_operands_1core": t_svc}
        # the products that used that B on the GPU: rerun the group on it and compare
        first_of_k = {}
        for i, p in enumerate(probs):
            first_of_k.setdefault(p["K"], i)
        for i, p in enumerate(probs):
            src = probs[first_of_k[p["K"]]]["B"]
            if src is not p["B"]:
                p["B"].copy_(src)
        run_step()
        torch.cuda.synchronize()
        worst, checked = 0.0, 0
        for i, p in enumerate(probs):
            assert np.array_equal(cprods[i]["ptr"], p["vp"].cpu().numpy()) and np.array_equal(cprods[i]["col"], p["vc"].cpu().numpy()), \
                f"GPU SVC of product {i} differs from the CPU restatement"
            ref = keep[i]
            got = p["C"][: ref.shape[0], :CPU_SAMPLE_COLS].float().cpu().numpy()
            floor = 1e-3 * np.abs(ref).max(axis=1, keepdims=True) + 1e-30
            err = float((np.abs(got - ref) / np.maximum(np.abs(ref), floor)).max())
            worst = max(worst, err)
            checked += ref.size
        assert worst <= 1e-2, f"timed step differs from the CPU oracle: max rel err {worst:.3e}"
        validated = {"products": len(probs), "elements": checked, "max_rel_err": worst, "criterion": 1e-2,
                     "svc_bit_exact": True}
        validated["note"] = "GPU C of the grouped step against the host fp32 SpMM on the sampled rows and columns of all 32 products"
    if rank == 0:
        status = ops.device_status()
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": WORKLOAD if not args.only else "single product " + args.only, "N_total": N_total,
                           "N_per_gpu": n_loc, "products_per_step": len(probs), "cuda_graph": graphed,
                           "group": {"mode": ("automatic", "compressed", "expanded", "expanded, CTA pairs")[args.group_mode], "launches_per_step": launches_per_step,
                                     "tile_columns": group.tile_columns, "work_items": group.work_items, "ctas": group.ctas,
                                     "scratch_bytes": group.scratch_bytes},
                           "l2": "operands of a step exceed L2; between steps a 256 MiB buffer is written and read back (evicts L2 and leaves no dirty lines of the buffer behind)",
                           "parallelism": f"B and C column-sharded over {world} GPU(s), A_vs replicated, no collective"},
                "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "validated": validated,
                "gpu_launches": args.steps * launches_per_step, "clocks": clocks, "device_status": status,
                "wall_s_timed_region": wall}
        line.update(extras)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


class L2Flush:
    """Evicts L2 between timed launches: writes a buffer twice the size of L2, then reads it back.  The read pass
    matters: after the write alone, L2 is left full of dirty lines of this buffer, and the kernel timed next would
    pay for writing them back (about 126 MB, 30 us at HBM speed) on top of its own traffic."""

    def __init__(self, torch, dev, nbytes=256 << 20):
        self.torch = torch
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        self.sink = None

    def __call__(self):
        self.buf.zero_()
        self.sink = self.torch.sum(self.buf, dtype=self.torch.int64)


def reference_kernel_comparator(torch, ops, probs, n_loc, dev, flush):
    """The reference's own kernel (SSpMM/src/sspmm.cu compiled unmodified for sm_100a into oracle/_ref/ by
    oracle/Makefile) on the same products and the same B: microseconds per product and per step.  Its V = 16
    loader reads past the end of the last vector row, so its inputs are padded by 64 vectors; it needs
    N % 64 == 0 and is never given a product with an empty vector row."""
    import ctypes as C
    so = os.path.join(ROOT, "oracle", "_ref", "libsspmm_ref.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libsspmm_ref.so not built (needs a reference checkout at build time)"}
    if n_loc % 64 != 0:
        return {"unavailable": f"the reference kernel needs N % 64 == 0 (N per GPU = {n_loc})"}
    lib = C.CDLL(so)
    fn = getattr(lib, "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PK6__halfS4_PS2_")
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 4 + [C.c_void_p] * 6
    pad = 64
    per, total_ms, skipped, useful = [], 0.0, 0, 0.0
    for p in probs:
        lens = (p["vp"][1:] - p["vp"][:-1])
        if int(lens.min().item()) == 0:
            skipped += 1
            per.append(None)
            continue
        V, m_vec = p["V"], p["m_vec"]
        col = torch.cat([p["vc"], torch.zeros(pad, dtype=torch.int32, device=dev)])
        val = torch.cat([p["vv"], torch.zeros(pad * V, dtype=torch.float16, device=dev)])
        idx = torch.arange(m_vec, dtype=torch.int32, device=dev)
        out = torch.empty((m_vec * V, n_loc), dtype=torch.float16, device=dev)
        args_ = (m_vec, V, n_loc, p["K"], idx.data_ptr(), p["vp"].data_ptr(), col.data_ptr(), val.data_ptr(),
                 p["B"].data_ptr(), out.data_ptr())
        torch.cuda.synchronize()
        ms = []
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for k in range(4):                               # legacy default stream, as the reference driver
            flush()
            torch.cuda.synchronize()
            a0.record(torch.cuda.default_stream(dev))
            rc = fn(*args_)
            a1.record(torch.cuda.default_stream(dev))
            torch.cuda.synchronize()
            if rc != 0:
                return {"unavailable": f"reference kernel returned {rc}"}
            if k > 0:
                ms.append(a0.elapsed_time(a1))
        t = sum(ms) / len(ms)
        total_ms += t
        useful += 2.0 * p["nnz"] * n_loc
        per.append({"us": t * 1e3, "useful_tflops": 2.0 * p["nnz"] * n_loc / t / 1e9})
        if p is probs[0]:
            got = ops.sspmm_planned(p["plan"], p["vv"], p["B"]).float()
            per[-1]["max_abs_diff_vs_ours"] = float((out.float() - got).abs().max().item())
        del out, col, val
    return {"ms_per_step": total_ms, "products_timed": len(probs) - skipped, "products_skipped_empty_vector_row": skipped,
            "useful_tflops": useful / total_ms / 1e9 if total_ms else None, "per_product": per,
            "note": "spmm::SSpMM of the reference (mma.sync, one warp per CTA), fp16 output, one launch per product on the legacy "
                    "default stream, CUDA events, L2 flushed before each launch"}


def _cpu_svc_child(path, conn):
    """Child of cpu_svc_all_cores: loads its matrix, waits for the start signal, compresses, reports seconds."""
    from oracle import svc_oracle
    d = np.load(path)
    ptr, col = d["ptr"].tolist(), d["col"].tolist()
    M = len(ptr) - 1
    rows = [col[ptr[i]:ptr[i + 1]] for i in range(M)]
    conn.send("ready")
    conn.recv()
    t0 = time.perf_counter()
    svc_oracle.cvse(M, M, len(col), rows, 8)
    conn.send(time.perf_counter() - t0)
    conn.close()


def cpu_svc_all_cores(host_mats):
    """The CPython restatement on independent matrices, one process per matrix (the reference is single-threaded;
    a sweep can still be split over cores): matrices per second from the common start to the last finish."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")                      # the parent holds a CUDA context: no fork
    procs, files = [], []
    tmp = tempfile.mkdtemp()
    for k, (ptr, col) in enumerate(host_mats):
        path = os.path.join(tmp, f"m{k}.npz")
        np.savez(path, ptr=ptr, col=col)
        files.append(path)
        parent, child = ctx.Pipe()
        pr = ctx.Process(target=_cpu_svc_child, args=(path, child), daemon=True)
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
    for f in files:
        os.unlink(f)
    os.rmdir(tmp)
    return len(host_mats) / wall


def bench_svc(torch, ops, dev, ids=(0, 1, 2, 3, 4, 5, 6, 7)):
    """SVC throughput on a sample of the power-law sweep (V=8): device-resident one by one and stacked,
    through the Python entry point, and the CPU oracle on one core and on all cores; then the SpMM of the
    same matrices at N = 128 with its bounds."""
    from oracle import svc_oracle
    from sspmm_b200 import sparse_matrix_format as smf
    peaks = load_peaks()
    dm = [synthetic.sweep_matrix_device(i, dev) for i in range(32)]          # (n, row_ptr, col, values)
    dmats = [dm[i] for i in ids]
    for n, p, c, v in dmats:
        ops.svc(p, c, v, n, n, 8)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nbytes = 0
    for n, p, c, v in dmats:
        vp, vc, vv, _ = ops.svc(p, c, v, n, n, 8)
        nbytes += 4 * (n + 1) + 6 * c.numel() + 4 * vp.numel() + 4 * vc.numel() + 2 * vv.numel()
    torch.cuda.synchronize()
    t_dev = time.perf_counter() - t0

    def stacked(mats, reps=3):
        batch = [(p, c, v, n, n) for n, p, c, v in mats]
        ops.svc_batch(batch, 8)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            ops.svc_batch(batch, 8)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps
    t_batch, t_batch32 = stacked(dmats), stacked(dm)
    # the SpMM of the same sweep matrices (B = n x 128), caller-owned scratch, nothing read back
    spmm = []
    for n, p, c, v in dmats:
        vp, vc, vv, _ = ops.svc(p, c, v, n, n, 8)
        nvec = vc.numel()
        B = torch.randn((n, 128), device=dev, dtype=torch.float16)
        C = torch.empty(((vp.numel() - 1) * 8, 128), device=dev, dtype=torch.float16)
        wsb = ops.workspace_bytes(vp.numel() - 1, 8, 128, n, nvec)
        ws = torch.empty(max(wsb, 256), dtype=torch.uint8, device=dev)
        for _ in range(3):
            ops.sspmm_ws(vp, vc, vv, B, 8, nvec, ws, out=C)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.sspmm_ws(vp, vc, vv, B, 8, nvec, ws, out=C)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        b_alg = 2 * 8 * nvec + 4 * nvec + 4 * vp.numel() + 2 * n * 128 + 2 * C.numel()
        gather = 2.0 * nvec * 128
        spmm.append({"n": n, "nvec": nvec, "us": ms * 1e3, "useful_tflops": 2.0 * c.numel() * 128 / ms / 1e9,
                     "algorithmic_gbs": b_alg / ms / 1e6, "frac_of_hbm_peak": b_alg / ms / 1e6 / peaks["hbm_gbs"],
                     "gather_gbs": gather / ms / 1e6})
    host = [(p.cpu().numpy(), c.cpu().numpy()) for n, p, c, v in dmats]
    row_lists = []
    for ptr, col in host:                                # the caller's data structure (lists of lists), built outside the clock
        pl, cl = ptr.tolist(), col.tolist()
        row_lists.append([cl[pl[i]:pl[i + 1]] for i in range(len(pl) - 1)])
    t0 = time.perf_counter()
    for (ptr, col), rows in zip(host, row_lists):
        smf.CVSE(len(rows), len(rows), int(col.size), rows, 8)
    t_host_api = time.perf_counter() - t0
    t0 = time.perf_counter()
    for (ptr, col), rows in zip(host, row_lists):
        svc_oracle.cvse(len(rows), len(rows), int(col.size), rows, 8)
    t_cpu = time.perf_counter() - t0
    try:
        cpu_all = cpu_svc_all_cores(host)
    except Exception as exc:  # pragma: no cover - depends on the host
        sys.stderr.write(f"all-core CPU SVC measurement skipped: {exc}\n")
        cpu_all = None
    return {"sample": f"sweep matrices {list(ids)} (n = {[m[0] for m in dmats]}), V=8; stacks through svc_batch_begin/finish",
            "device_matrices_per_s": len(dmats) / t_dev, "device_gbs": nbytes / t_dev / 1e9,
            "device_batched_matrices_per_s": len(dmats) / t_batch, "speedup_batched_vs_cpu": t_cpu / t_batch,
            "device_batched32_matrices_per_s": 32 / t_batch32,
            "speedup_batched32_vs_cpu_1core": (32 / t_batch32) / (len(dmats) / t_cpu),
            "python_entry_point_matrices_per_s": len(dmats) / t_host_api,
            "cpu_oracle_matrices_per_s_1core": len(dmats) / t_cpu, "speedup_device_vs_cpu": t_cpu / t_dev,
            "cpu_oracle_matrices_per_s_one_process_per_matrix": cpu_all, "cpu_cores": os.cpu_count(),
            "spmm_n128": spmm,
            "spmm_n128_note": "every vector is a gathered 256-byte row of B for 8 output rows, so the kernel moves 2*nvec*N bytes "
                              "through L2 (gather_gbs) whatever HBM does; algorithmic_gbs counts B, C and A_vs once"}


def bench_sweep(torch, ops, dev, dist, rank, world, total=2000, batch=125):
    """The power-law sweep (BASELINE config 5): `total` seeded matrices, matrix_id mod world -> rank; every rank
    compresses its matrices (V=8) in stacked batches and multiplies each by B = n x 128.  Device-resident
    inputs, no collective on the data path; seconds are the slowest rank's."""
    ids = [i for i in range(total) if i % world == rank]
    t0 = time.perf_counter()
    mats = [synthetic.sweep_matrix_device(i, dev) for i in ids]
    torch.cuda.synchronize()
    t_gen = time.perf_counter() - t0
    n_max = max(m[0] for m in mats)
    Bs = [torch.randn((m[0], 128), device=dev, dtype=torch.float16) for m in mats]
    C = torch.empty((((n_max + 7) // 8) * 8, 128), device=dev, dtype=torch.float16)
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    batches = [list(range(k, min(k + batch, len(mats)))) for k in range(0, len(mats), batch)]

    def one_pass(with_spmm):
        for idx in batches:
            parts, _ = ops.svc_batch([(mats[k][1], mats[k][2], mats[k][3], mats[k][0], mats[k][0]) for k in idx], 8)
            if with_spmm:
                for k, (vp, vc, vv) in zip(idx, parts):
                    ops.sspmm_ws(vp, vc, vv, Bs[k], 8, vc.numel(), ws, out=C[: (vp.numel() - 1) * 8])

    def timed(with_spmm):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        one_pass(with_spmm)
        torch.cuda.synchronize()
        t = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    one_pass(True)                                       # warm-up
    sec_svc = min(timed(False), timed(False))
    sec_all = min(timed(True), timed(True))
    nnz = torch.tensor([float(sum(m[2].numel() for m in mats))], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(nnz, op=dist.ReduceOp.SUM)
    return {"matrices": total, "matrices_this_rank": len(ids), "stack_size": batch,
            "svc_matrices_per_s": total / sec_svc, "svc_plus_spmm_matrices_per_s": total / sec_all,
            "seconds_svc_slowest_rank": sec_svc, "seconds_svc_plus_spmm_slowest_rank": sec_all,
            "useful_tflops_n128": 2.0 * float(nnz.item()) * 128 / sec_all / 1e12,
            "generation_seconds_this_rank": t_gen,
            "note": "matrix_id mod world -> rank; seeded matrices drawn on the GPU (Zipf(2) row lengths, mean 16, uniform columns, "
                    "n log-uniform in [4096, 65536]); wall clock incl. the host side of svc_batch and of the per-matrix SpMM calls; "
                    "weak scaling per rank is by construction, the whole-job figure is matrices / slowest rank's seconds"}


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
    for _ in range(3):
        layer.forward_grouped(x, batch, seq)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(10):
        layer.forward_grouped(x, batch, seq)
    a1.record()
    torch.cuda.synchronize()
    ms_grouped = a0.elapsed_time(a1) / 10
    nnz = sum(l.nnz for l in layer.linears)
    return {"config": "hidden 768, ffn 3072, 12 heads, seq 512, batch 32, weights 90 % sparse, V=16",
            "ms_sparse_weights": ms_sparse, "ms_sparse_weights_grouped": ms_grouped, "ms_dense_weights_cublas": ms_dense,
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
            plan = ops.Plan(vp, vc, 16, a.K)
            ms_pg = ms_gg = None
            if plan.one_launch:
                grp = ops.Group([(plan, vv, B, C)], mode=ops.Group.COMPRESSED)
                ms_pg = t_graph(lambda: ops.sspmm_planned(plan, vv, B, out=C))
                ms_gg = t_graph(grp.run)
            out.append({"shape": list(synthetic.FFN_SHAPES[shape_id]), "sparsity": synthetic.FFN_SPARSITIES[sid],
                        "us": ms * 1e3, "useful_tflops": 2.0 * a.nnz * 256 / ms / 1e9, "cublas_dense_us": ms_d * 1e3,
                        "cublas_useful_tflops": 2.0 * a.nnz * 256 / ms_d / 1e9, "padding": vc.numel() * 16 / a.nnz,
                        "us_in_graph": None if ms_g is None else ms_g * 1e3,
                        "planned_one_launch_us_in_graph": None if ms_pg is None else ms_pg * 1e3,
                        "group_of_one_us_in_graph": None if ms_gg is None else ms_gg * 1e3,
                        "cublas_dense_us_in_graph": None if ms_dg is None else ms_dg * 1e3})
    return {"note": "back-to-back launches, operands L2-resident (problem is ~1-4 MB): latency, not bandwidth; us = sspmm_f16_f16 "
                    "(reference-signature entry point), planned = sspmm_planned (one launch, no scratch), group = sspmm_group_run (K cut into parts)",
            "cases": out}


def run_case(name: str):
    """Small fixed workloads for profiler captures (one kernel family, a few launches, a few GB at most):
         group_conv_shard   the 32 conv products as one group at the 8-GPU shard width N = 3136, three runs
         group_conv_full    the same at N = 25088 (the benchmark step), three runs
         group_conv_layer   conv layer (512, 4608) s = 0.8 V = 16, N = 18944, as a group, expanded and compressed
         planned_conv_layer the same layer through sspmm_planned (one launch, A tiles built in the kernel), N = 9472
         sweep_stack        32 sweep matrices: stacked SVC (svc_batch), then the SpMM of each at N = 128
         svc_stack8         stacked SVC of sweep matrices 0..7, twice (small enough for a full counter capture)
         svc_stack125       stacked SVC of sweep matrices 0..124, twice (one stack of the 2000-matrix sweep)
         gather_sweep       row-gather SpMM of sweep matrix 7 (n = 51970) at N = 128, four times
         svc_powerlaw       SVC of one power-law matrix, n = 65536, V = 8, three times
         gather_powerlaw    row-gather SpMM of that matrix at N = 1024, four times"""
    import torch
    from sspmm_b200 import build, capi, ops
    build.build()
    capi.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(0)
    flush = L2Flush(torch, dev)
    up = lambda a: (torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev), torch.from_numpy(a.values).to(dev))

    def conv_product(l, s, V, N):
        a = synthetic.conv_weight(l, s)
        vp, vc, vv, _ = ops.svc(*up(a), a.M, a.K, V)
        B = torch.randn((a.K, N), device=dev, dtype=torch.float16)
        C = torch.empty(((vp.numel() - 1) * V, N), device=dev, dtype=torch.float16)
        return ops.Plan(vp, vc, V, a.K), vv, B, C
    if name in ("group_conv_shard", "group_conv_full"):
        g = ops.Group([conv_product(l, s, V, 3136 if name == "group_conv_shard" else synthetic.CONV_N) for (l, s, V) in conv_problems()])
        for _ in range(3):
            flush()
            g.run()
    elif name == "group_conv_layer":
        prod = conv_product(3, 0, 16, 18944)
        for mode in (ops.Group.EXPANDED, ops.Group.COMPRESSED):
            g = ops.Group([prod], mode=mode)
            for _ in range(2):
                flush()
                g.run()
    elif name == "planned_conv_layer":
        plan, vv, B, C = conv_product(3, 0, 16, 9472)
        for _ in range(3):
            flush()
            ops.sspmm_planned(plan, vv, B, out=C)
    elif name == "sweep_stack":
        mats = [synthetic.sweep_matrix_device(i, dev) for i in range(32)]
        ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
        for _ in range(2):
            parts, _ = ops.svc_batch([(p, c, v, n, n) for n, p, c, v in mats], 8)
            for (n, p, c, v), (vp, vc, vv) in zip(mats, parts):
                B = torch.randn((n, 128), device=dev, dtype=torch.float16)
                ops.sspmm_ws(vp, vc, vv, B, 8, vc.numel(), ws)
    elif name in ("svc_stack8", "svc_stack125"):
        mats = [synthetic.sweep_matrix_device(i, dev) for i in range(8 if name == "svc_stack8" else 125)]
        for _ in range(2):
            ops.svc_batch([(p, c, v, n, n) for n, p, c, v in mats], 8)
    elif name == "gather_sweep":
        n, p, c, v = synthetic.sweep_matrix_device(7, dev)
        vp, vc, vv, _ = ops.svc(p, c, v, n, n, 8)
        B = torch.randn((n, 128), device=dev, dtype=torch.float16)
        ws = torch.empty(max(ops.workspace_bytes(vp.numel() - 1, 8, 128, n, vc.numel()), 256), dtype=torch.uint8, device=dev)
        for _ in range(4):
            ops.sspmm_ws(vp, vc, vv, B, 8, vc.numel(), ws)
    elif name in ("svc_powerlaw", "gather_powerlaw"):
        p, c, v = synthetic.power_law_device(65536, 65536, dev)
        for _ in range(3):
            vp, vc, vv, _ = ops.svc(p, c, v, 65536, 65536, 8)
        if name == "gather_powerlaw":
            B = torch.randn((65536, 1024), device=dev, dtype=torch.float16)
            C = torch.empty((65536, 1024), device=dev, dtype=torch.float16)
            ws = torch.empty(max(ops.workspace_bytes(8192, 8, 1024, 65536, vc.numel()), 256), dtype=torch.uint8, device=dev)
            for _ in range(4):
                ops.sspmm_ws(vp, vc, vv, B, 8, vc.numel(), ws, out=C)
    else:
        raise SystemExit(run_case.__doc__)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    print(json.dumps({"case": name, "status": "done"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--group-mode", type=int, default=0, choices=[0, 1, 2, 3],
                    help="0 automatic, 1 A tiles built in the kernel from the compressed operand, 2 dense copies of A written by "
                         "the kernel's loader warps every step, 3 as 2 with 256 x 256 tiles on CTA pairs")
    ap.add_argument("--sweep-matrices", type=int, default=2000, help="matrices of the power-law sweep (whole job)")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA graph of the step")
    ap.add_argument("--no-extras", action="store_true", help="skip the SVC and FFN side measurements")
    ap.add_argument("--case", default="", help="run one small fixed workload for a profiler capture and exit (see run_case)")
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
        if args.case:
            run_case(args.case)
        elif args.impl == "reference":
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
