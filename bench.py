"""Benchmark of the Newton constraint solve: world-steps/s on N B200s.

A "step" is one ``solve_with_scratch`` over one batch of worlds (the reference's
humanoid benchmark configuration: nv 34, njmax 64, 8192 worlds per GPU).  Inputs are
seeded synthetic solver states with that model's shapes; several distinct batches
are rotated so that consecutive steps never find their inputs in L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line is printed by rank 0.  ``--impl reference`` times the CPU
restatement of the reference's solver (the oracle) on all host cores.
"""

from __future__ import annotations

import argparse
import copy
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "newton_solver_world_steps_per_s"
UNIT = "world-steps/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one newton_kernel launch, from the ncu
# capture summarised in profiles/newton_kernel_humanoid.md: 138.8 MB for 16384 humanoid
# worlds (8.47 KB per world); traffic grows in proportion to the worlds of a launch.
NCU_TRAFFIC_BYTES_PER_WORLD = 140.06e6 / 16384


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--workload", default="humanoid", choices=["humanoid", "snu", "g1"])
    p.add_argument("--nworld", type=int, default=8192, help="worlds per GPU")
    p.add_argument("--batches", type=int, default=4, help="distinct input batches rotated per GPU")
    p.add_argument("--iterations", type=int, default=50)
    p.add_argument("--ls-iterations", type=int, default=50)
    p.add_argument("--tolerance", type=float, default=1e-8)
    p.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline sample length")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--sparse-hessian", default="on", choices=["on", "off"],
                   help="install the static-pattern sparse Hessian plan (single-body contact groups)")
    return p.parse_args()


def workload_config(args, m, d):
    return {
        "workload": f"{args.workload}: nv {m.nv}, nv_pad {m.nv_pad}, njmax {d.njmax}, "
        f"{args.nworld} worlds per GPU, one Newton solve per step "
        f"(iterations<={args.iterations}, ls_iterations<={args.ls_iterations}, tol {args.tolerance:g})",
        "worlds_per_gpu": args.nworld,
        "nv": m.nv,
        "njmax": d.njmax,
        "batches_rotated": args.batches,
        "l2": f"inputs of {args.batches} distinct batches rotate (> 126 MB L2 in total)",
        "sharding": "by world, no collective on the data path",
        "hessian_factor": "sparse-pattern L'DL" if args.sparse_hessian == "on" else "dense blocked Cholesky",
    }


def algorithmic_bytes(m, d) -> int:
    """Compulsory HBM bytes of one solve of batch ``d``: inputs read once, results
    written once, independent of the iteration count."""
    nefc = np.minimum(d.nefc, d.njmax).astype(np.int64)
    nv, nM = m.nv, m.nM
    read = nefc * nv + 3 * nefc + nM + 3 * nv + 3  # J; D, aref, frictionloss; M; 3 dof vectors; nefc/ne/nf
    write = 3 * nv + 2 * nefc + 2  # qacc, Ma, qfrc_constraint; force, state; niter, overflow
    return int(4 * (read + write).sum())


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def wait_started(self, timeout: float = 3.0) -> None:
        """nvidia-smi takes a few hundred ms to deliver its first row; a timed region of
        0.1-0.2 s would otherwise pass without a sample."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.rows and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self, t_begin: float, t_end: float):
        """Median SM clock and throttle reasons of the rows received in [t_begin, t_end]
        (host clock); when the window is too short to hold one, of all rows since the
        sampler started (warm-up and timed steps of the same workload), and says so."""
        inside = [r for t, r in self.rows if t_begin <= t <= t_end]
        window = "timed region"
        if not inside:
            inside = [r for _, r in self.rows]
            window = "warm-up and timed steps (no sample fell inside the timed region)"
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": window}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "window": window}


def make_batches(args, rank):
    from instantmimic_b200 import synthetic

    out = []
    for b in range(args.batches):
        m, d, _ = synthetic.make_workload(
            args.workload, args.nworld, seed=1000 * rank + b, iterations=args.iterations,
            ls_iterations=args.ls_iterations, tolerance=args.tolerance)
        out.append((m, d))
    return out


def run_reference(args):
    """The reference's CPU path for this solve, restated (oracle), on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    oracle.build()
    cores = os.cpu_count() or 1
    batches = make_batches(args, 0)
    m = batches[0][0]
    work = [copy.deepcopy(d) for _, d in batches]
    for k in range(min(args.warmup, 2)):
        oracle.solve(m, work[k % len(work)], threads=cores)
    steps = args.steps
    # bounded: stop once a few minutes are used; the steps actually timed are reported
    elapsed, done = 0.0, 0
    for k in range(steps):
        dd = copy.deepcopy(batches[k % len(batches)][1])
        t1 = time.perf_counter()
        oracle.solve(m, dd, threads=cores)
        elapsed += time.perf_counter() - t1
        done += 1
        if elapsed > 150.0:
            break
    value = args.nworld * done / elapsed
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": done,
        "warmup": min(args.warmup, 2),
        "ms_per_step": 1e3 * elapsed / done,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args, m, batches[0][1]),
        "cpu_baseline": {
            "value": value,
            "unit": UNIT,
            "cores": cores,
            "kind": "port",
            "sample": f"{done} steps of {args.nworld} worlds, OpenMP over worlds",
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference solver (MuJoCo / mujoco-warp are not installed)",
    }
    print(json.dumps(line))


def cpu_baseline(args, batches):
    from oracle import oracle

    oracle.build()
    cores = os.cpu_count() or 1
    m = batches[0][0]
    elapsed, solved, k = 0.0, 0, 0
    while elapsed < args.cpu_seconds:
        dd = copy.deepcopy(batches[k % len(batches)][1])
        t = time.perf_counter()
        oracle.solve(m, dd, threads=cores)
        elapsed += time.perf_counter() - t
        solved += args.nworld
        k += 1
    return {
        "value": solved / elapsed,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"{k} solves of {args.nworld} worlds ({elapsed:.1f} s), OpenMP over worlds, {cores} threads",
    }


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from instantmimic_b200 import _lib, mjw_model
    from instantmimic_b200 import mjw_step_optimized as runtime

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _lib.lib()

    host = make_batches(args, rank)
    m_host = host[0][0]
    md = mjw_model.to_device(m_host, device)
    dev = [mjw_model.to_device(d, device) for _, d in host]
    scratch = [runtime.make_optimized_fwd_position_scratch(md, dd, device) for dd in dev]
    if args.sparse_hessian == "on":
        groups = [[b] for b in range(1, len(m_host.body_dofadr))]
        for dd, sc in zip(dev, scratch):
            reason = runtime.refresh_sparse_hessian(md, dd, sc, groups, device)
            if reason != "enabled":
                # the model does not qualify (density, nv): the dense factor stays, as in the reference
                args.sparse_hessian = "off"
                break
    nb = len(dev)

    def step(k):
        runtime.solve_with_scratch(md, dev[k % nb], scratch[k % nb], use_optimized_kernel=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        clocks.wait_started()
        for k in range(args.warmup):
            step(k)
        barrier()
        t_begin = time.perf_counter()
        e0.record()
        for k in range(args.steps):
            step(k)
        e1.record()
        barrier()
        t_end = time.perf_counter()
    ms = max_over_ranks(e0.elapsed_time(e1))
    value = world * args.nworld * args.steps / (ms * 1e-3)
    niter = np.concatenate([dd.solver_niter.cpu().numpy() for dd in dev])

    # ---- end to end: host buffers in, host results out, every step -----------
    e2e = None
    if not args.no_e2e:
        in_names = ["nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M"]
        efc_in = ["J", "D", "aref", "frictionloss"]
        out_names = ["qacc", "qfrc_constraint", "solver_niter"]
        efc_out = ["force", "state", "Ma"]
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()  # noqa: E731
        hin = [
            ({n: pin(getattr(d, n)) for n in in_names}, {n: pin(getattr(d.efc, n)) for n in efc_in})
            for _, d in host
        ]
        # two slots (device buffers, stream, pinned result buffers): while slot A solves,
        # slot B's inputs are already crossing PCIe; the host consumes the results of
        # step k-1 while step k is in flight.  Every step's H2D and D2H is inside the
        # timed region.
        nslot = 2 if nb >= 2 else 1
        slots = []
        for i in range(nslot):
            slots.append({
                "dd": dev[i], "sc": scratch[i], "stream": torch.cuda.Stream(device=device),
                "done": torch.cuda.Event(),
                "out": ({n: pin(getattr(host[0][1], n)) for n in out_names},
                        {n: pin(getattr(host[0][1].efc, n)) for n in efc_out}),
            })
        h2d = sum(t.numel() * t.element_size() for part in hin[0] for t in part.values())
        d2h = sum(t.numel() * t.element_size() for part in slots[0]["out"] for t in part.values())
        checksum = 0.0

        def e2e_issue(k):
            sl = slots[k % nslot]
            a, b = hin[k % nb]
            with torch.cuda.stream(sl["stream"]):
                for n, t in a.items():
                    getattr(sl["dd"], n).copy_(t, non_blocking=True)
                for n, t in b.items():
                    getattr(sl["dd"].efc, n).copy_(t, non_blocking=True)
                runtime.solve_with_scratch(md, sl["dd"], sl["sc"], use_optimized_kernel=True, stream=sl["stream"])
                for n, t in sl["out"][0].items():
                    t.copy_(getattr(sl["dd"], n), non_blocking=True)
                for n, t in sl["out"][1].items():
                    t.copy_(getattr(sl["dd"].efc, n), non_blocking=True)
                sl["done"].record(sl["stream"])

        def e2e_consume(k):
            sl = slots[k % nslot]
            sl["done"].synchronize()  # the caller reads this step's results on the host
            return float(sl["out"][0]["solver_niter"][0])

        def e2e_run(n):
            total = 0.0
            for k in range(n):
                if k >= nslot:
                    total += e2e_consume(k - nslot)  # frees the slot step k is about to reuse
                e2e_issue(k)
            for k in range(max(n - nslot, 0), n):
                total += e2e_consume(k)
            return total

        torch.cuda.synchronize()
        e2e_steps = min(args.steps, 50)
        e2e_run(4)
        barrier()
        t0 = time.perf_counter()
        checksum = e2e_run(e2e_steps)
        barrier()
        dt = max_over_ranks(time.perf_counter() - t0)
        e2e = {
            "value": world * args.nworld * e2e_steps / dt,
            "unit": UNIT,
            "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h),
            "steps": e2e_steps,
            "ms_per_step": 1e3 * dt / e2e_steps,
            "pipeline": f"{nslot} slots (copy of step k+1 overlaps the solve of step k)",
            "h2d_gbs_per_gpu": float(h2d) * e2e_steps / dt / 1e9,  # the copy is the limit of this path
            "checksum": checksum,
        }

    # ---- the M-side kernels of the same path, timed alone on the same batches --------
    aux = None
    if world == 1:
        from instantmimic_b200.mjw_kernels import indexed_factor

        def timed(fn, reps=20):
            """Seconds per call on the device: the calls are recorded into a CUDA graph
            (they allocate nothing) and the replay is timed, so that host time per call
            (struct building, ctypes) does not hide the kernel's."""
            for k in range(3):
                fn(k)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for k in range(reps):
                    fn(k)
            graph.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) * 1e-3 / reps

        W, nv, nM = args.nworld, m_host.nv, m_host.nM
        aux = {}
        sc0 = scratch[0]
        if sc0.tree_factor_solve is not None:
            t = timed(lambda k: runtime._factor_solve_i_dense(
                md, dev[k % nb], dev[k % nb].M, dev[k % nb].qacc_smooth, dev[k % nb].qfrc_smooth, None,
                tree_factor_solve=sc0.tree_factor_solve))
            alg = 4.0 * W * (nM + 2 * nv)
            generated = sc0.tree_factor_solve.kernel is not None
            aux["tree_ldl_generated" if generated else "tree_ldl_kernel"] = {
                "ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg,
                "groups": sc0.tree_factor_solve.groups}
            if generated:
                # the same plan through the instruction-list interpreter (what runs without NVRTC)
                import dataclasses

                interp = dataclasses.replace(sc0.tree_factor_solve, kernel=None)
                t = timed(lambda k: runtime._factor_solve_i_dense(
                    md, dev[k % nb], dev[k % nb].M, dev[k % nb].qacc_smooth, dev[k % nb].qfrc_smooth, None,
                    tree_factor_solve=interp))
                aux["tree_ldl_kernel(interpreted)"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9,
                                                       "algorithmic_bytes": alg}
        if sc0.dense_factor_solve is not None:
            bs = sc0.dense_factor_solve
            t = timed(lambda k: indexed_factor.blocked_dense_factor_solve(
                dev[k % nb], dev[k % nb].M, dev[k % nb].qacc_smooth, dev[k % nb].qfrc_smooth, bs))
            alg = 4.0 * W * (nM + 2 * nv + bs.pad * bs.pad)
            aux["blocked_dense_kernel"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg}
        t = timed(lambda k: runtime._rowless_handoff(md, dev[k % nb]))
        alg = 4.0 * W * (nM + 4 * nv + 1)
        aux["mul_m_kernel(rowless hand-off)"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9,
                                                 "algorithmic_bytes": alg}

    if rank == 0:
        from instantmimic_b200.mjw_kernels import newton_fusion

        info = newton_fusion.solve_call(md, dev[0], scratch[0].solver_context, scratch[0].solver_nsolving,
                                        cache_on=scratch[0]).launch_info()
        alg = float(np.mean([algorithmic_bytes(m_host, d) for _, d in host]))
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured"
        else:
            peak, peak_src = 6650.0, "fallback"
        launch_s = (ms * 1e-3) / args.steps
        achieved = alg / launch_s / 1e9
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": workload_config(args, m_host, host[0][1]),
            "clocks": clocks.summary(t_begin, t_end),
            "e2e": e2e,
            "gpu_launches": 2 * args.steps,
            "roofline": {
                "kernel": "newton_kernel_resident" if info.j_resident else "newton_kernel_streamed",
                "bound": "hbm",
                "achieved": achieved,
                "peak": peak,
                "peak_source": peak_src,
                "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES_PER_WORLD * args.nworld if args.workload == "humanoid" else None,
                "algorithmic_bytes_per_launch": alg,
                "launch_ms": launch_s * 1e3,
            },
            "solver": {
                "niter_mean": float(niter.mean()),
                "niter_max": int(niter.max()),
                "smem_bytes_per_world": int(info.smem_bytes),
            },
        }
        if aux is not None:
            for v in aux.values():
                v["frac_of_hbm_peak"] = v["achieved_gbs"] / peak
            line["aux_kernels"] = aux
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args, host)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
