#!/usr/bin/env python
"""Benchmark of the SpMM hot path: effective GFLOP/s (2*nnz*N) on seeded synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--scale-down k] [--no-workloads]

One "step" is one SpMM of the whole matrix.  With N > 1 (launched by torch.distributed.run, one
rank per GPU) the matrix is cut into N time-balanced row-window ranges, B is replicated and every
rank multiplies its own range; there is no data-path collective, total work is fixed (strong
scaling).  Rank 0 prints ONE JSON line.

  value       whole-job GFLOP/s with operands resident in HBM, CUDA-event timed, max over ranks
  e2e         the same through the host-buffer call: B copied from pinned host memory and C
              copied back inside the timed region (the converted matrix stays resident, like
              weights)
  roofline    algorithmic bytes of one launch / its duration against the measured HBM peak
  cpu_baseline  the CPU oracle's CSR SpMM on a bounded row sample, all host cores
  parity      the timed result itself against the CPU oracle (a row sample holding the heaviest
              rows, the first and the last window; every rank checks its own rows)
  workloads   (1 GPU) the four other benchmark configurations at full size, each with its time
              (L2 flushed between timed launches), roofline fraction, CPU baseline and parity record

--impl reference times that CPU path alone (the reference project has no CSR-level SpMM and
its GPU kernel is sm_90a-only and unfinished, so its own verifier arithmetic, restated in
oracle/, is what can run on the host cores).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))  # parity.py: the tolerance rules of the parity tests

DEFAULT_WORKLOAD = "rmat24_sharded_fp16"
OTHER_WORKLOADS = ("uniform_4096_fp16", "blocks_16384_tf32", "rmat20_gnn_fp16", "pruned_llm_fp16")
L2_FLUSH_BYTES = 512 << 20  # written between timed launches of the smaller workloads (L2 is 126 MB)


def log(*a):
    print("[bench]", *a, file=sys.stderr, flush=True)


def host_cores() -> int:
    """Cores this process may run on.  Taken from the machine, not from OMP_NUM_THREADS, which
    torch.distributed.run sets to 1 for every rank."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def measured_peaks():
    """(HBM GB/s, fp16/bf16 dense TFLOP/s, where they come from)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(nnz, rows, cols, n, a_size, b_size, c_size):
    """CSR-equivalent A once, B once, C written once."""
    return nnz * (a_size + 4) + 4 * (rows + 1) + cols * n * b_size + rows * n * c_size


def cpu_sample_rows(row_ptr_host: np.ndarray, target_nnz: int):
    """A contiguous block of rows from the middle of the matrix holding about target_nnz entries."""
    rows = len(row_ptr_host) - 1
    nnz = int(row_ptr_host[-1])
    if target_nnz >= nnz:
        return 0, rows
    mid = int(np.searchsorted(row_ptr_host, nnz // 2))
    lo = int(np.searchsorted(row_ptr_host, max(0, int(row_ptr_host[mid]) - target_nnz // 2)))
    hi = int(np.searchsorted(row_ptr_host, min(nnz, int(row_ptr_host[lo]) + target_nnz)))
    return lo, max(hi, lo + 1)


def time_cpu_oracle(rp, ci, v, B_host, steps, warmup, budget_s=12.0, threads=0):
    """GFLOP/s of the oracle's CSR SpMM on `threads` host threads (0: every core of the machine) on a
    row sample sized to the budget."""
    import oracle
    rows = len(rp) - 1
    n = B_host.shape[1]
    threads = threads or host_cores()
    lo, hi = cpu_sample_rows(rp, 1 << 20)  # probe
    t0 = time.perf_counter()
    oracle.spmm_csr(hi - lo, *slice_rows(rp, ci, v, lo, hi), B_host, n_threads=threads)
    probe = max(time.perf_counter() - t0, 1e-4)
    probe_nnz = int(rp[hi]) - int(rp[lo])
    per_step = budget_s / max(1, steps + warmup)
    target = int(min(int(rp[-1]), max(1 << 20, probe_nnz * per_step / probe)))
    lo, hi = cpu_sample_rows(rp, target)
    srp, sci, sv = slice_rows(rp, ci, v, lo, hi)
    nnz_s = int(srp[-1])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.spmm_csr(hi - lo, srp, sci, sv, B_host, n_threads=threads)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = float(np.mean(times))
    return {"value": 2.0 * nnz_s * n / t / 1e9, "unit": "GFLOP/s", "cores": threads, "kind": "port",
            "sample": f"rows [{lo}, {hi}) of {rows}: {nnz_s} of {int(rp[-1])} nnz, {len(times)} passes, "
                      f"{t * 1e3:.1f} ms each"}, t


def slice_rows(rp, ci, v, lo, hi):
    a, b = int(rp[lo]), int(rp[hi])
    return (np.asarray(rp[lo:hi + 1], dtype=np.int64) - a).astype(np.uint32), ci[a:b], v[a:b]


def parity_ranges(rows: int, rp, want_rows: int = 1 << 15):
    """Row ranges of the parity sample: the first rows (window 0; on the R-MAT matrices also the
    heaviest rows, which the generator puts at the low indices), the rows around the heaviest row if
    it lies elsewhere, a block from the middle and the last rows (the last, possibly ragged, window)."""
    if rows <= 4 * want_rows:
        return [(0, rows)]
    w = want_rows
    ranges = [(0, w), (rows // 2 // 16 * 16, rows // 2 // 16 * 16 + w), (rows - w, rows)]
    deg = np.diff(np.asarray(rp).astype(np.int64))
    hub = int(np.argmax(deg))
    if not any(a <= hub < b for a, b in ranges):
        a = max(0, min(rows - 64, hub // 16 * 16))
        ranges.append((a, a + 64))
    return sorted(ranges)


def parity_record(get_rows, rows, rp, ci, v, B_host):
    """Parity of a result against the CPU oracle on the sample rows; get_rows(a, b) returns C[a:b] as numpy."""
    import parity
    ranges = parity_ranges(rows, rp)
    got = np.concatenate([np.asarray(get_rows(a, b), dtype=np.float32) for a, b in ranges])
    try:
        st = parity.check_rows(got, rp, ci, v, B_host, ranges, threads=host_cores())
        st["ok"] = True
    except AssertionError as e:  # reported in the line; the bench exits non-zero at the end
        st = {"ok": False, "error": str(e), "checked_rows": int(got.shape[0])}
    st["rows_sampled"] = [[int(a), int(b)] for a, b in ranges]
    return st


def tf32_peak_tflops(dev):
    """Dense tf32 matmul throughput of this GPU (cuBLAS through torch, 8192^3, best of 5): the tensor
    peak of the tf32 workload, measured in the same run as the kernel it bounds."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        m = 8192
        a = torch.randn((m, m), device=dev)
        b = torch.randn((m, m), device=dev)
        for _ in range(2):
            torch.matmul(a, b)
        best = float("inf")
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2.0 * m ** 3 / (best * 1e-3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def roofline_record(nnz, rows, cols, n, esz, kernel_ms, hbm_gbs, tensor_tflops, peak_kind, tensor_note):
    """Fraction of the slower of the two rooflines: t_roof = max(bytes / HBM, flops / tensor peak)."""
    alg = algorithmic_bytes(nnz, rows, cols, n, esz, esz, 4)
    flops = 2.0 * nnz * n
    t_hbm = alg / (hbm_gbs * 1e9)
    t_tensor = flops / (tensor_tflops * 1e12)
    bound = "hbm" if t_hbm >= t_tensor else "tensor"
    t = kernel_ms * 1e-3
    if bound == "hbm":
        achieved, peak, unit = alg / t / 1e9, hbm_gbs, "GB/s"
    else:
        achieved, peak, unit = flops / t / 1e12, tensor_tflops, "TFLOP/s"
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
            "peak_source": f"of {peak_kind}" + (f"; tensor: {tensor_note}" if tensor_note else ""),
            "kernel_ms": kernel_ms, "algorithmic_bytes": alg, "t_hbm_us": t_hbm * 1e6, "t_tensor_us": t_tensor * 1e6}


def dram_traffic(workload, tiles, n_slabs):
    tpath = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(tpath):
        per_tile = json.load(open(tpath)).get(workload, {}).get("dram_bytes_per_tile")
        if per_tile:
            return float(per_tile) * tiles * n_slabs
    return None


def graph_replay_ms(plan, B, C_dev, steps):
    """The same launches replayed from a CUDA graph: what a launch-latency-bound product costs without
    the per-launch host work."""
    import torch
    try:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            plan.spmm(B, C_dev, sync=False)
            with torch.cuda.graph(g, stream=side):
                for _ in range(steps):
                    plan.spmm(B, C_dev, sync=False)
        torch.cuda.current_stream().wait_stream(side)
        g.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        g.replay()
        g1.record()
        torch.cuda.synchronize()
        ms = g0.elapsed_time(g1) / steps
        del g
        return ms
    except RuntimeError as e:  # reported, not fatal: the figure is an extra
        log(f"CUDA-graph replay not measured: {e}")
        return None


def capi_mod():
    from hopper_spmm_b200 import _capi
    return _capi


def run_other_workload(name, dev, steps, warmup, hbm_gbs, f16_tflops, tf32_tflops, peak_kind, flush_buf):
    """One of the smaller configurations at full size on one GPU: time (L2 flushed between the timed
    launches), roofline, CPU baseline, and the timed result checked whole against the CPU oracle."""
    import torch
    import hopper_spmm_b200 as hs
    from hopper_spmm_b200 import synth
    import parity
    dtype_name, n_feat, desc = synth.CONFIGS[name]
    csr, B = synth.make_config(name, 0, dev, 0)
    btcf = hs.DeviceBtcf(csr.rows, csr.cols, csr.row_ptr.to(torch.int32), csr.col_idx, csr.values, device=dev.index)
    plan = hs.SpmmPlan(btcf, device=dev.index)
    C_dev = torch.full((csr.rows, n_feat), float("nan"), dtype=torch.float32, device=dev)
    for _ in range(warmup):
        plan.spmm(B, C_dev, sync=False)
    plan.sync()
    cold = []
    for _ in range(steps):
        flush_buf.zero_()  # evicts operands and result from L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        plan.spmm(B, C_dev, sync=False)
        e1.record()
        plan.sync()
        cold.append(e0.elapsed_time(e1))
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0.record()
    for _ in range(steps):
        plan.spmm(B, C_dev, sync=False)
    h1.record()
    plan.sync()
    ms = float(np.mean(cold))
    ms_hot = h0.elapsed_time(h1) / steps
    # the reference's own protocol (src/common.h:48-49, src/fp16.cu:255-268): 3 warm-up launches, then 5
    # back to back between two events, issued by the library's C loop (no Python between the launches)
    proto = plan.bench(B, C_dev, hs.WARMUP_RUNS, hs.RUNS)
    info = plan.launch_info()
    esz = 2 if dtype_name == "f16" else 4
    tensor = f16_tflops if dtype_name == "f16" else tf32_tflops
    note = "" if dtype_name == "f16" else "tf32 matmul measured in this run"
    roof = roofline_record(csr.nnz, csr.rows, csr.cols, n_feat, esz, ms, hbm_gbs, tensor, peak_kind, note)
    flops = 2.0 * csr.nnz * n_feat
    rec = {"workload": name, "description": desc, "rows": csr.rows, "cols": csr.cols, "nnz": csr.nnz, "features": n_feat,
           "dtype": "f16" if dtype_name == "f16" else "tf32", "tiles": int(btcf.total_tiles),
           "fill": csr.nnz / max(1, btcf.total_tiles * 16 * btcf.col_window),
           "ms": ms, "ms_l2_warm": ms_hot, "ms_reference_protocol_3_5": proto.time / proto.runs,
           "l2": f"flushed between timed launches ({L2_FLUSH_BYTES >> 20} MB written)",
           "value": flops / (ms * 1e-3) / 1e9, "unit": "GFLOP/s", "roofline": roof,
           "kernel": {"n_ctas": info.n_ctas, "feature_slab": info.feature_slab, "n_slabs": info.n_slabs,
                      "stages": info.stages, "launches_per_step": int(info.kernel_launches),
                      "row_window": int(getattr(info, "row_window", 16) or 16)},
           "graph_replay_ms": graph_replay_ms(plan, B, C_dev, steps) if ms_hot < 0.2 else None}
    # executed MMA work: every tile of the kernel that ran is a dense (window rows x CW) block times all features
    win = rec["kernel"]["row_window"]
    if win == 16:
        ex_tiles = int(btcf.total_tiles)
    else:
        lib = capi_mod().lib()
        tinfo = capi_mod().BtcfInfo()
        getattr(lib, "b200spmm_plan_tall_info" if win == 128 else "b200spmm_plan_pair_info")(plan._p, ctypes.byref(tinfo))
        ex_tiles = int(tinfo.total_tiles)
    slab = int(info.feature_slab)
    rec["executed_mma_gflop"] = 2.0 * ex_tiles * win * btcf.col_window * (int(info.n_slabs) * slab) / 1e9
    rec["executed_mma_tflops"] = rec["executed_mma_gflop"] / ms
    rp, ci, v = csr.numpy()
    B_host = B.cpu().numpy()
    got = C_dev.cpu().numpy()
    try:
        st = parity.check(got, csr.rows, rp, ci, v, B_host, threads=host_cores())
        st.update(ok=True, checked_rows=csr.rows)
    except AssertionError as e:
        st = {"ok": False, "error": str(e), "checked_rows": csr.rows}
    rec["parity"] = st
    cpu, _ = time_cpu_oracle(rp, ci, v, B_host, 2, 1, budget_s=4.0)
    rec["cpu_baseline"] = cpu
    rec["vs_cpu"] = rec["value"] / cpu["value"]
    plan.close()
    btcf.close()
    del C_dev, B, csr
    torch.cuda.empty_cache()
    return rec


from hopper_spmm_b200.sharded import ROW_CHARGE as sharded_charge


def static_config(args, world, dtype_name, n_feat, desc, rows, cols, nnz):
    """What names the workload; the same keys and values in both arms."""
    return {"workload": args.workload, "description": desc, "scale_down": args.scale_down, "features": n_feat,
            "row_window": 16, "c_dtype": "f32", "rows": int(rows), "cols": int(cols), "nnz": int(nnz),
            "parallelism": f"row-window shards x{world} (balanced on nnz + {sharded_charge} per row), B replicated",
            "l2": "operands larger than L2 (no flush needed)" if args.scale_down == 0 and args.workload == DEFAULT_WORKLOAD
                  else "see workloads[].l2 / operands may fit L2 at this scale"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--scale-down", type=int, default=0)
    ap.add_argument("--no-allgather", action="store_true", help="skip the timing of the all-gather of the row-sharded C (N > 1)")
    ap.add_argument("--e2e-row-charge", type=int, default=-1,
                    help="entries a row is charged when the end-to-end step gets row ranges of its own (N > 1); "
                         "-1 = the ranges of the device-resident measurement")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the four other configurations (1 GPU, default workload only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    import torch
    from hopper_spmm_b200 import synth
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dtype_name, n_feat, desc = synth.CONFIGS[args.workload]

    if args.impl == "reference":
        if rank != 0:
            return
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        csr, B = synth.make_config(args.workload, 0, dev, args.scale_down)
        rp, ci, v = csr.numpy()
        cores = host_cores()
        base, t = time_cpu_oracle(rp, ci, v, B.cpu().numpy(), args.steps, args.warmup, budget_s=60.0, threads=cores)
        config = static_config(args, max(world, args.gpus), dtype_name, n_feat, desc, csr.rows, csr.cols, csr.nnz)
        line = {"impl": "reference", "metric": "SpMM effective GFLOP/s (2*nnz*N)", "value": base["value"],
                "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16" if dtype_name == "f16" else "tf32", "data": "synthetic", "config": config,
                "cpu_baseline": base, "gpu_launches": 0, "host_cores": cores,
                "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS"),
                "e2e": {"value": base["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    import torch.distributed as dist
    import hopper_spmm_b200 as hs
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- inputs: every rank generates the same matrix and keeps its own row range
    t0 = time.perf_counter()
    csr, B = synth.make_config(args.workload, 0, dev, args.scale_down)
    torch.cuda.synchronize()
    log(f"rank {rank}: generated {csr.rows}x{csr.cols}, nnz={csr.nnz} in {time.perf_counter() - t0:.1f}s")
    rp_full = csr.row_ptr.cpu().numpy().astype(np.uint32)
    from hopper_spmm_b200 import sharded
    cuts, r0, r1 = sharded.my_rows(csr.rows, rp_full, world, rank)
    part = csr.row_slice(r0, r1)
    total_nnz, total_rows = csr.nnz, csr.rows
    cols = B.shape[0]
    config = static_config(args, world, dtype_name, n_feat, desc, csr.rows, csr.cols, csr.nnz)
    # this rank's rows on the host: the parity sample and (1 GPU) the CPU baseline read them
    need_host = (not args.no_parity) or (rank == 0 and world == 1 and not args.no_cpu)
    host_csr = part.numpy() if need_host else None
    # Row ranges of the end-to-end step on several GPUs: the product's own, unless --e2e-row-charge
    # asks for others.  Charging the rows for their bytes of C over the rank's host link (201
    # entries per row at 128 fp16 features: 52 GB/s against 0.0253 ms per million entries) evens
    # out the row counts, but did not pay reliably: ms per step with the product's ranges / with
    # 201 per row, same box each pair: 109.5 / 97.7 on two GPUs (on other boxes 110 / 112-114 and
    # 112 / 90), 105.1 / 103.6 on four, 67.6 / 78.4 on eight, where the host's memory system, not
    # a rank's own link, limits the copies.
    e2e_charge = args.e2e_row_charge
    part_e2e, q0, q1 = None, r0, r1
    if world > 1 and not args.no_e2e and e2e_charge >= 0:
        _, q0, q1 = sharded.my_rows(csr.rows, rp_full, world, rank, row_charge=e2e_charge)
        part_e2e = csr.row_slice(q0, q1)
    del csr
    torch.cuda.empty_cache()
    # conversion on the device: CSR tensors -> condensed tiles, all in HBM
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    btcf = hs.DeviceBtcf(r1 - r0, cols, part.row_ptr.to(torch.int32), part.col_idx, part.values, device=local_rank)
    torch.cuda.synchronize()
    t_conv = time.perf_counter() - t0
    nnz_local = part.nnz
    del part
    torch.cuda.empty_cache()
    plan = hs.SpmmPlan(btcf, device=local_rank)
    log(f"rank {rank}: rows [{r0},{r1}) nnz={nnz_local} tiles={btcf.total_tiles} device convert {t_conv:.2f}s")
    tiles_local, rows_local = btcf.total_tiles, r1 - r0
    fill = nnz_local / max(1, tiles_local * 16 * btcf.col_window)
    C_dev = torch.full((rows_local, n_feat), float("nan"), dtype=torch.float32, device=dev)  # every row must be written

    # ---- device-resident timing (clocks are sampled from the warm-up to the end of the run)
    clocks = ClockSampler(local_rank)
    clocks.__enter__()
    for _ in range(args.warmup):
        plan.spmm(B, C_dev, sync=False)
    plan.sync()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for i in range(args.steps):
        plan.spmm(B, C_dev, sync=False)
        ev[i + 1].record()
    plan.sync()
    barrier()
    step_ms = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[-1])
    info = plan.launch_info()
    t_all = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    ms_per_step = float(t_all.item()) / args.steps
    rank_ms = [total_ms / args.steps]  # every rank's own time: shows how well the row cuts balance the GPUs
    if world > 1:
        gathered = [torch.zeros(1, dtype=torch.float64, device=dev) for _ in range(world)]
        dist.all_gather(gathered, torch.tensor([total_ms / args.steps], dtype=torch.float64, device=dev))
        rank_ms = [float(g.item()) for g in gathered]
    flops = 2.0 * total_nnz * n_feat
    value = flops / (ms_per_step * 1e-3) / 1e9

    # ---- parity of the timed result: this rank's rows against the CPU oracle (sample rows)
    B_host = B.cpu().numpy() if need_host else None
    parity_dev = None
    if not args.no_parity:
        parity_dev = parity_record(lambda a, b: C_dev[a:b].cpu().numpy(), rows_local, *host_csr, B_host)
        log(f"rank {rank}: parity of the device-resident result: {parity_dev}")

    graph_ms = graph_replay_ms(plan, B, C_dev, args.steps) if ms_per_step < 0.2 else None

    # ---- the collective: all-gather of the row-sharded C, timed on its own
    allgather_ms, allgather_bytes = None, None
    if world > 1 and not args.no_allgather:
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        full = sharded.allgather_rows(C_dev, cuts)  # untimed: the first exchange sets up the peer connections
        del full
        barrier()
        a0.record()
        full = sharded.allgather_rows(C_dev, cuts)
        a1.record()
        barrier()
        t_a = torch.tensor([a0.elapsed_time(a1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t_a, op=dist.ReduceOp.MAX)
        allgather_ms = float(t_a.item())
        allgather_bytes = int(full.numel() * full.element_size())
        # the gathered result holds this rank's rows where they belong
        assert torch.equal(full[r0:r1], C_dev), "all-gather misplaced this rank's rows"
        del full
        torch.cuda.empty_cache()

    # ---- end to end: B from pinned host memory in, C out to pinned host memory, every step
    e2e, parity_e2e = None, None
    if not args.no_e2e:
        hB = torch.empty(B.shape, dtype=B.dtype, pin_memory=True)
        hB.copy_(B)
        # the reference's operator keeps C in the matrix's element type (DENSE_MTX.values is MAT_VAL_TYPE,
        # src/utils/class.h:44-48: fp16 in the fp16 build): the host-buffer call is made the same way
        c_half = dtype_name == "f16"
        c_rows = C_dev.shape[0] if world == 1 else q1 - q0
        hC = torch.empty((c_rows, n_feat), dtype=torch.float16 if c_half else torch.float32, pin_memory=True)
        torch.cuda.synchronize()
        hBn, hCn = hB.numpy(), hC.numpy()
        if world == 1:
            step = lambda: plan.spmm_host(hBn, hCn, c_half=c_half)
            h2d_bytes = int(hB.numel() * hB.element_size())
        else:
            # N ranks behind one host: every rank uploads 1/N of the replicated B and the parts are
            # exchanged GPU to GPU (sharded.upload_replicated); then the rank's product, then its rows
            # of C back to the host.  Bytes are whole-job sums.
            plan_e = plan
            if part_e2e is not None:
                btcf_e = hs.DeviceBtcf(q1 - q0, cols, part_e2e.row_ptr.to(torch.int32), part_e2e.col_idx, part_e2e.values,
                                       device=local_rank)
                del part_e2e
                plan_e = hs.SpmmPlan(btcf_e, device=local_rank)
                log(f"rank {rank}: end-to-end rows [{q0},{q1}) (row charge {e2e_charge}) tiles={btcf_e.total_tiles}")
            dB = torch.empty_like(B)
            dC = torch.empty((q1 - q0, n_feat), dtype=hC.dtype, device=dev)

            def step():
                sharded.upload_replicated(hB, dB)
                plan_e.spmm(dB, dC, c_half=c_half, sync=False)
                hC.copy_(dC, non_blocking=True)
                plan_e.sync()
            h2d_bytes = int(hB.numel() * hB.element_size())
        step()  # warm-up: allocates the plan's device buffers
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        t_e = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        d2h = torch.tensor([float(hC.numel() * hC.element_size())], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
            dist.all_reduce(d2h, op=dist.ReduceOp.SUM)
        e_ms = float(t_e.item()) / args.steps
        e2e = {"value": flops / (e_ms * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(d2h.item()),
               "c_dtype": "f16" if c_half else "f32",
               "call": ("b200spmm_spmm_host (fp16_spmm / tf32_spmm with host B and C)" if world == 1 else
                        "per rank: 1/N of host B in + GPU-to-GPU exchange, b200spmm_spmm, its rows of C out to the host")}
        if world > 1:
            e2e["row_charge"] = e2e_charge if e2e_charge >= 0 else sharded.ROW_CHARGE
        if not args.no_parity and (q0, q1) == (r0, r1):  # the host-buffer result, same rows as above
            parity_e2e = parity_record(lambda a, b: hCn[a:b], rows_local, *host_csr, B_host)
            log(f"rank {rank}: parity of the end-to-end result: {parity_e2e}")
        else:
            assert bool(torch.isfinite(hC[:: max(1, hC.shape[0] // 4096)]).all())

    # ---- roofline of the SpMM kernel on this rank's launch
    hbm_gbs, f16_tflops, peak_kind = measured_peaks()
    esz = 2 if dtype_name == "f16" else 4
    tf32_tflops = None
    if dtype_name != "f16" or (world == 1 and not args.no_workloads and args.workload == DEFAULT_WORKLOAD):
        tf32_tflops = tf32_peak_tflops(dev)
    kernel_ms = float(np.mean(step_ms))
    roofline = roofline_record(nnz_local, rows_local, cols, n_feat, esz, kernel_ms, hbm_gbs,
                               f16_tflops if dtype_name == "f16" else tf32_tflops, peak_kind,
                               "" if dtype_name == "f16" else "tf32 matmul measured in this run")
    roofline["kernel"] = "spmm_sm100_kernel"
    roofline["traffic"] = dram_traffic(args.workload, tiles_local, info.n_slabs)
    # whole job: every rank's A and C bytes once, B once (it is replicated, not re-read by the algorithm),
    # against N GPUs' bandwidth
    alg_job = algorithmic_bytes(total_nnz, total_rows, cols, n_feat, esz, esz, 4)
    roofline["whole_job"] = {"algorithmic_bytes": alg_job, "achieved": alg_job / (ms_per_step * 1e-3) / 1e9,
                             "peak": hbm_gbs * world, "frac": alg_job / (ms_per_step * 1e-3) / 1e9 / (hbm_gbs * world)}
    if world > 1:
        roofline["note"] = "achieved/frac: rank 0's launch with the replicated B counted in full; whole_job counts B once"

    clocks.__exit__(None, None, None)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu, _ = time_cpu_oracle(*host_csr, B_host, 2, 1, budget_s=15.0)
        one, _ = time_cpu_oracle(*host_csr, B_host, 1, 1, budget_s=6.0, threads=1)  # the reference is single-threaded
        cpu["one_core"] = {"value": one["value"], "unit": one["unit"], "sample": one["sample"]}

    # ---- every rank's parity record goes to rank 0, which reports the worst
    def worst(rec):
        if rec is None:
            return None
        mine = [float(rec.get("ok", False)), float(rec.get("scaled_err", float("inf"))), float(rec.get("rule_failures", -1)),
                float(rec.get("checked_rows", 0))]
        if world == 1:
            return dict(rec, ranks=1)
        t = torch.tensor(mine, dtype=torch.float64, device=dev)
        allr = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        rows_ = [[float(x) for x in a.tolist()] for a in allr]
        return {"ok": all(r_[0] == 1.0 for r_ in rows_), "scaled_err": max(r_[1] for r_ in rows_),
                "rule_failures": int(max(r_[2] for r_ in rows_)), "checked_rows": int(sum(r_[3] for r_ in rows_)),
                "ranks": world, "rank0": rec}
    parity_dev, parity_e2e = worst(parity_dev), worst(parity_e2e)

    # ---- the other four configurations, full size, one GPU
    plan.close()
    btcf.close()
    del C_dev
    workloads = None
    if world == 1 and not args.no_workloads and args.workload == DEFAULT_WORKLOAD and args.scale_down == 0:
        del B
        torch.cuda.empty_cache()
        flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        workloads = []
        for name in OTHER_WORKLOADS:
            t0 = time.perf_counter()
            rec = run_other_workload(name, dev, args.steps, args.warmup, hbm_gbs, f16_tflops, tf32_tflops, peak_kind, flush_buf)
            log(f"{name}: {rec['ms'] * 1e3:.1f} us ({rec['ms_l2_warm'] * 1e3:.1f} us L2-warm), {rec['value']:.0f} GFLOP/s, "
                f"frac {rec['roofline']['frac']:.3f} ({rec['roofline']['bound']}), x{rec['vs_cpu']:.0f} CPU, "
                f"parity {rec['parity']}, {time.perf_counter() - t0:.1f}s")
            workloads.append(rec)

    failed = False
    if rank == 0:
        details = dict(tiles_rank0=int(tiles_local), fill_rank0=fill, n_ctas=info.n_ctas, feature_slab=info.feature_slab,
                       stages=info.stages, convert_s_rank0=t_conv, rank_ms=[round(x, 4) for x in rank_ms],
                       # what the tensor cores execute: every tile is a dense 16 x CW x n product
                       executed_mma_gflop_rank0=2.0 * tiles_local * 16 * btcf.col_window * n_feat / 1e9,
                       graph_replay_ms_per_step=graph_ms, allgather_c_ms=allgather_ms, allgather_c_bytes=allgather_bytes,
                       tf32_tflops_measured=tf32_tflops, host_cores=host_cores())
        line = {"metric": "SpMM effective GFLOP/s (2*nnz*N)", "value": value, "unit": "GFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16" if dtype_name == "f16" else "tf32",
                "data": "synthetic", "config": config, "details": details, "roofline": roofline, "cpu_baseline": cpu,
                "e2e": e2e, "parity": {"device_resident": parity_dev, "e2e": parity_e2e},
                "allgather_c_ms": allgather_ms, "workloads": workloads,
                "gpu_launches": int(args.steps * info.kernel_launches), "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
        recs = [parity_dev, parity_e2e] + [w["parity"] for w in (workloads or [])]
        failed = any(r is not None and not r.get("ok", False) for r in recs)
    if world > 1:
        dist.destroy_process_group()
    if failed:
        log("PARITY FAILED - see the parity records in the line above")
        sys.exit(1)


if __name__ == "__main__":
    main()
