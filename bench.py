"""Benchmark of the Newton constraint solve: world-steps/s on N B200s.

A "step" is one ``solve_with_scratch`` over one batch of worlds (the reference's
humanoid benchmark configuration: nv 34, njmax 64, 8192 worlds per GPU).  Inputs are
seeded synthetic solver states with that model's shapes; several distinct batches
are rotated so that consecutive steps never find their inputs in L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload humanoid|snu|g1|sweep]

One JSON line is printed by rank 0.  The timed unit is a round of exactly K steps
between two CUDA events; rounds are repeated (at least nine, and until about a second
of device time has passed, so that the clock sampler sees the region) and
``ms_per_step`` is the median round, with p10 / p90 beside it.  ``--impl reference``
times the reference's CPU path: MuJoCo C ``mj_step`` when the ``mujoco`` package is
installed, else the CPU restatement of the solver (the oracle), on all host cores.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the humanoid solve kernel
# in an ncu capture of a 16384-world batch: 140.3 MB (128.33 read + 12.01 written), 8.56 KB
# per world.  DRAM traffic of
# this kernel grows in proportion to the worlds of a launch (every world's inputs are
# read once), so the figure is scaled by the worlds of the bench's launch.
NCU_TRAFFIC_BYTES_PER_WORLD_HUMANOID = 140.3e6 / 16384
STRONG_TOTAL_WORLDS = 8192


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--workload", default="humanoid", choices=["humanoid", "snu", "g1", "sweep"])
    p.add_argument("--nworld", type=int, default=8192, help="worlds per GPU")
    p.add_argument("--batches", type=int, default=4, help="distinct input batches rotated per GPU")
    p.add_argument("--iterations", type=int, default=50)
    p.add_argument("--ls-iterations", type=int, default=50)
    p.add_argument("--tolerance", type=float, default=1e-8)
    p.add_argument("--rounds", type=int, default=0, help="timed rounds of --steps steps (0: at least 9, ~1 s)")
    p.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU baseline sample length")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-aux", action="store_true")
    p.add_argument("--no-strong", action="store_true")
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--aux-nworld", type=int, default=65536, help="worlds of the M-side kernel timings")
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


def algorithmic_flops(m, d_host, niter, stats, state, plan) -> float:
    """Floating-point operations one solve of the batch needs, from the per-world work
    counters the kernel records (line-search passes, flipped rows, factorisations,
    gradient evaluations), the iteration counts and the final row states.  Per world:
    J qacc, M qacc, the initial Hessian over its QUADRATIC rows, per iteration M v, J v
    and ~20 operations per row and line-search step size, per gradient J^T f, per
    flipped row a rank-one update over the dofs the row touches, per factorisation the
    factor's multiply-adds (the plan's term count for the sparse factor, nv^3 / 3
    dense) and per gradient one forward + backward substitution."""
    nv, nM = m.nv, m.nM
    nefc = np.minimum(d_host.nefc, d_host.njmax).astype(np.float64)
    nM2 = 2 * nM - nv
    live = np.arange(d_host.njmax)[None, :] < nefc[:, None]
    J = d_host.efc.J[..., :nv]
    support = ((J != 0).sum(axis=2) * live).sum() / max(live.sum(), 1)  # dofs a row touches, mean
    nquad = ((state == 1) & live).sum(axis=1).astype(np.float64)
    if plan is not None:
        terms = float((plan.tables["run_kl"].astype(np.int64) >> 16).sum())
        f_factor = 3.0 * terms + 2.0 * plan.nfac
        f_solve = 4.0 * plan.nfac
    else:
        f_factor = nv**3 / 3.0
        f_solve = 2.0 * nv * nv
    passes, flips, nfactor, ngrad = (stats[:, k].astype(np.float64) for k in range(4))
    it = niter.astype(np.float64)
    # step sizes evaluated: one per pass for the first two passes of a search, three afterwards
    evals = np.maximum(passes, 0) + 2.0 * np.maximum(passes - 2.0 * it, 0)
    f = (2 * nefc * nv + 2 * nM2 + nquad * support * (support + 1)
         + it * (2 * nM2 + 2 * nefc * nv + 4 * nv)
         + 20.0 * nefc * evals
         + ngrad * (2 * nefc * nv + 3 * nv)
         + flips * support * (support + 1)
         + nfactor * f_factor + ngrad * f_solve)
    return float(f.sum())


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
        """nvidia-smi takes a few hundred ms to deliver its first row."""
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
        (host clock); when the window holds none, of all rows, and says so."""
        inside = [r for t, r in self.rows if t_begin <= t <= t_end]
        window = "timed region"
        if not inside:
            inside = [r for _, r in self.rows]
            window = "warm-up and timed steps (no sample fell inside the timed region)"
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                power.append(float(r[2]))
            except ValueError:
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "window": window}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm), "window": window, "power_w_median": float(np.median(power))}


def make_batches(args, rank, nworld=None, count=None):
    from instantmimic_b200 import synthetic

    out = []
    for b in range(count or args.batches):
        m, d, _ = synthetic.make_workload(
            args.workload, nworld or args.nworld, seed=1000 * rank + b, iterations=args.iterations,
            ls_iterations=args.ls_iterations, tolerance=args.tolerance)
        out.append((m, d))
    return out


# ------------------------------------------------------------------ reference arm


def mujoco_reference(args):
    """The reference's own CPU path: MuJoCo C ``mj_step`` (Newton, pyramidal, dense,
    same iteration limits and tolerance) over a thread pool, one MjData per thread.
    Returns None when the ``mujoco`` package is not installed."""
    try:
        import mujoco  # noqa: F401
    except Exception as e:  # not installed on this pool's boxes
        return None, f"{type(e).__name__}: {e}"
    # A humanoid with the workload's joint tree is generated as MJCF text: the model files
    # of the reference are not shipped with this repository.
    from concurrent.futures import ThreadPoolExecutor

    from instantmimic_b200 import synthetic

    xml = synthetic.humanoid_mjcf(iterations=args.iterations, ls_iterations=args.ls_iterations,
                                  tolerance=args.tolerance)
    model = mujoco.MjModel.from_xml_string(xml)
    cores = os.cpu_count() or 1
    datas = [mujoco.MjData(model) for _ in range(cores)]
    rng = np.random.default_rng(0)

    def work(i):
        d = datas[i]
        per = args.nworld // cores + (1 if i < args.nworld % cores else 0)
        for _ in range(per):
            mujoco.mj_resetData(model, d)
            d.qpos[2] = 0.9 + 0.1 * rng.random()
            d.qvel[:] = 0.5 * rng.standard_normal(model.nv)
            mujoco.mj_step(model, d)
        return per

    with ThreadPoolExecutor(cores) as pool:
        for _ in range(args.warmup):
            list(pool.map(work, range(cores)))
        t0 = time.perf_counter()
        done = 0
        for _ in range(args.steps):
            done += sum(pool.map(work, range(cores)))
            if time.perf_counter() - t0 > 150.0:
                break
        dt = time.perf_counter() - t0
    return {"value": done / dt, "cores": cores, "kind": "reference",
            "sample": f"{done} mj_step calls (generated humanoid MJCF), thread pool of {cores}", "dt": dt,
            "steps": done // max(args.nworld, 1)}, None


def run_reference(args):
    """The reference's CPU path for this solve on all host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    batches = make_batches(args, 0)
    m = batches[0][0]
    result, why_not = None, "workload has no generated MJCF"
    if args.workload == "humanoid":
        try:
            result, why_not = mujoco_reference(args)
        except Exception as e:  # a MuJoCo that rejects the generated model: keep the restated solver
            result, why_not = None, f"mj_step arm failed: {type(e).__name__}: {e}"
    if result is None:
        from oracle import oracle

        oracle.build()
        work = [copy.deepcopy(d) for _, d in batches]
        for k in range(args.warmup):
            oracle.solve(m, work[k % len(work)], threads=cores)
        elapsed, done = 0.0, 0
        for k in range(args.steps):
            dd = copy.deepcopy(batches[k % len(batches)][1])
            t1 = time.perf_counter()
            oracle.solve(m, dd, threads=cores)
            elapsed += time.perf_counter() - t1
            done += 1
            if elapsed > 150.0:  # bounded: the steps actually timed are reported
                break
        result = {"value": args.nworld * done / elapsed, "cores": cores, "kind": "port", "dt": elapsed,
                  "steps": done,
                  "sample": f"{done} steps of {args.nworld} worlds, OpenMP over worlds, {cores} threads"}
    value = result["value"]
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": result["steps"],
        "warmup": args.warmup,
        "ms_per_step": 1e3 * result["dt"] / max(result["steps"], 1),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32" if result["kind"] == "port" else "f64",
        "data": "synthetic",
        "config": workload_config(args, m, batches[0][1]),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": result["cores"], "kind": result["kind"],
                         "sample": result["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": ("MuJoCo C mj_step" if result["kind"] == "reference" else
                 f"CPU restatement of the reference solver; MuJoCo C unavailable ({why_not}); "
                 "reference Warp solver: unavailable on this box (not installed)"),
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
        solved += dd.nworld
        k += 1
    return {
        "value": solved / elapsed,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"{k} solves of {batches[0][1].nworld} worlds ({elapsed:.1f} s), OpenMP over worlds, {cores} threads",
    }


# ------------------------------------------------------------------ timing helpers


def percentiles(xs):
    xs = np.asarray(xs, dtype=np.float64)
    return float(np.median(xs)), float(np.percentile(xs, 10)), float(np.percentile(xs, 90))


class Timer:
    """Rounds of K calls between CUDA events on torch's current stream, bracketed by a
    device synchronisation and (multi-GPU) a barrier; per round the max over ranks."""

    def __init__(self, torch, dist, world, device):
        self.torch, self.dist, self.world, self.device = torch, dist, world, device

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, xs):
        if self.world == 1:
            return list(xs)
        t = self.torch.tensor(list(xs), dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def rounds(self, step, steps, rounds, min_seconds=0.0, max_rounds=400):
        """ms of each round of `steps` calls.  With rounds == 0: at least nine, then until
        `min_seconds` of device time (decided on rank 0's first round, same count on all)."""
        ev = self.torch.cuda.Event
        out = []
        k0 = 0

        def one():
            nonlocal k0
            e0, e1 = ev(enable_timing=True), ev(enable_timing=True)
            self.barrier()
            e0.record()
            for k in range(steps):
                step(k0 + k)
            e1.record()
            self.barrier()
            k0 += steps
            return e0.elapsed_time(e1)

        first = one()
        out.append(first)
        if rounds <= 0:
            first_max = self.max_over_ranks([first])[0]
            rounds = int(min(max_rounds, max(9, np.ceil(min_seconds * 1e3 / max(first_max, 1e-3)))))
        for _ in range(rounds - 1):
            out.append(one())
        return self.max_over_ranks(out)


def graph_of(torch, fn, reps):
    """`reps` calls recorded into one CUDA graph (they allocate nothing)."""
    for k in range(3):
        fn(k)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for k in range(reps):
            fn(k)
    graph.replay()
    torch.cuda.synchronize()
    return graph


def time_graph(torch, graph, reps, replays=5):
    """Median ms per call over `replays` replays of a graph of `reps` calls."""
    ms = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b) / reps)
    return float(np.median(ms))


# ------------------------------------------------------------------ sweep workload


SWEEP_NV = (27, 35, 64)
SWEEP_NEFC = (32, 128, 512)
SWEEP_WORLDS = (4096, 16384, 65536)


def stage_kernels(args, torch, md, m_host, device, timed):
    """The stages either side of the solve at the batch of the M-side timings: the
    implicit-fast tail (A = M - h qDeriv, advance) and the body-tree stages (com_vel,
    crb, rne).  Random device-resident state of the workload's shapes; one position
    servo per actuated dof."""
    from dataclasses import replace
    from types import SimpleNamespace

    import numpy as np

    from instantmimic_b200 import mjw_step_optimized as runtime
    from instantmimic_b200.mjw_kernels import tree_fusion, velocity_fusion

    W, nv, nM, nq = args.aux_nworld, m_host.nv, m_host.nM, m_host.nq
    nbody = int(np.asarray(m_host.body_parentid).size)
    nu = max(nv - 6, 1)
    gen = torch.Generator(device=device).manual_seed(11)
    rnd = lambda *s: torch.randn(*s, device=device, generator=gen)  # noqa: E731
    dofs = torch.arange(nv - nu, nv, device=device, dtype=torch.int32)

    def batch():
        qpos = rnd(W, nq)
        d = SimpleNamespace(
            nworld=W, M=rnd(W, nM), qvel=rnd(W, nv), qpos=qpos, time=torch.zeros(W, device=device),
            moment_rownnz=torch.ones(W, nu, dtype=torch.int32, device=device),
            moment_rowadr=torch.arange(nu, dtype=torch.int32, device=device).repeat(W, 1),
            moment_colind=dofs.repeat(W, 1).contiguous(), actuator_moment=torch.ones(W, nu, device=device),
            cinert=rnd(W, nbody, 10), crb=torch.empty(W, nbody, 10, device=device), cdof=rnd(W, nv, 6),
            cdof_dot=rnd(W, nv, 6), cvel=rnd(W, nbody, 6), cacc=torch.empty(W, nbody, 6, device=device),
            cfrc_int=torch.empty(W, nbody, 6, device=device), qfrc_bias=torch.empty(W, nv, device=device))
        return d

    big = [batch(), batch()]
    qacc = 1e-3 * rnd(W, nv)
    out = torch.empty(W, nM, device=device)
    mm = replace(md)
    mm.nu = nu
    mm.dof_damping = torch.rand(nv, device=device)
    sc = SimpleNamespace(implicit_actuator_vel=-10.0 * torch.rand(W, nu, device=device), advance_call=None,
                         pre_advance_modifier=None)
    tree = tree_fusion.create_tree_reduction_scratch(mm, deterministic=True)
    res = {}

    def put(name, t, floats_per_world):
        alg = 4.0 * W * floats_per_world
        res[name] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg}

    t = timed(lambda k: runtime.deriv_smooth_vel_dense_actuator_centric(mm, big[k % 2], out, sc))
    put("implicit_matrix_kernel", t, 2 * nM + 5 * nu)
    t = timed(lambda k: runtime._advance_with_scratch(mm, big[k % 2], qacc, sc))
    put("advance_kernel", t, 3 * nv + 2 * nq + 2)
    t = timed(lambda k: velocity_fusion.com_vel(mm, big[k % 2], tree))
    put("com_vel_kernel", t, nv + 12 * nv + 6 * nbody)
    t = timed(lambda k: tree_fusion.crb(mm, big[k % 2], tree))
    put("crb_kernel", t, 20 * nbody + 6 * nv + nM)
    t = timed(lambda k: tree_fusion.rne(mm, big[k % 2], tree))
    put("rne_kernel", t, 10 * nbody + 6 * nbody + 13 * nv + 12 * nbody + nv)
    return res


def run_sweep(args, torch, timer, world, rank, device, peak):
    """The isolated sweep: nv x nefc x batch, generic rows on tree-ancestor patterns,
    dense factor; worlds sharded over the ranks.  Inputs of 2048 generated worlds are
    repeated to the batch size on the device (generation on the host is what costs
    time; every world is still solved)."""
    from instantmimic_b200 import mjw_model, synthetic
    from instantmimic_b200 import mjw_step_optimized as runtime

    points = []
    base_worlds = 2048
    for nv in SWEEP_NV:
        for nefc in SWEEP_NEFC:
            m, d, _ = synthetic.make_sweep_point(nv, nefc, base_worlds, seed=rank, iterations=args.iterations,
                                                 ls_iterations=args.ls_iterations, tolerance=args.tolerance)
            md = mjw_model.to_device(m, device)
            bytes_per_world = algorithmic_bytes(m, d) / base_worlds
            for total in SWEEP_WORLDS:
                W = total // world
                reps = max(1, W // base_worlds)

                dev_arrays = mjw_model.to_device(d, device)  # one base copy on the device
                dd = copy.copy(dev_arrays)
                dd.nworld = W
                rep = lambda t: t.repeat((reps,) + (1,) * (t.dim() - 1))[:W].contiguous()  # noqa: E731
                for name in ("nefc", "ne", "nf", "qacc_smooth", "qacc_warmstart", "qfrc_smooth", "M", "qacc",
                             "qfrc_constraint", "solver_niter", "overflow"):
                    setattr(dd, name, rep(getattr(dev_arrays, name)))
                dd.efc = copy.copy(dev_arrays.efc)
                for name in ("J", "D", "aref", "frictionloss", "force", "state", "Ma"):
                    setattr(dd.efc, name, rep(getattr(dev_arrays.efc, name)))
                scratch = runtime.make_optimized_fwd_position_scratch(md, dd, device,
                                                                      include_optimized_kernel_scratch=False)
                step = lambda k: runtime.solve_with_scratch(md, dd, scratch, use_optimized_kernel=True)  # noqa: E731
                for _ in range(3):
                    step(0)
                ms = timer.rounds(step, 1, 5)
                med, p10, p90 = percentiles(ms)
                niter = float(dd.solver_niter.float().mean().item())
                points.append({
                    "nv": nv, "nefc": nefc, "worlds_total": total, "worlds_per_gpu": W, "ms": med, "ms_p10": p10,
                    "ms_p90": p90, "value": total / (med * 1e-3), "niter_mean": niter,
                    "achieved_gbs_per_gpu": bytes_per_world * W / (med * 1e-3) / 1e9,
                    "frac_of_hbm_peak": bytes_per_world * W / (med * 1e-3) / 1e9 / peak,
                })
                del dd, scratch, dev_arrays
                torch.cuda.empty_cache()
    return points


# ------------------------------------------------------------------ main


def main():
    args = parse_args()
    if args.impl == "reference":
        if args.workload == "sweep":
            args.workload = "humanoid"
        run_reference(args)
        return

    import torch
    import torch.distributed as dist

    from instantmimic_b200 import _lib, host_batch, mjw_model
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
    timer = Timer(torch, dist, world, device)
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    props = torch.cuda.get_device_properties(device)

    sweep_mode = args.workload == "sweep"
    if sweep_mode:
        args.workload = "humanoid"  # the headline line still carries the humanoid step

    host = make_batches(args, rank)
    m_host = host[0][0]
    md = mjw_model.to_device(m_host, device)
    dev = [mjw_model.to_device(d, device) for _, d in host]
    scratch = [runtime.make_optimized_fwd_position_scratch(md, dd, device) for dd in dev]
    groups = None
    if args.sparse_hessian == "on":
        groups = [[b] for b in range(1, len(m_host.body_dofadr))]
        for dd, sc in zip(dev, scratch):
            reason = runtime.refresh_sparse_hessian(md, dd, sc, groups, device)
            if reason != "enabled":
                # the model does not qualify (density, nv): the dense factor stays, as in the reference
                args.sparse_hessian, groups = "off", None
                break
    nb = len(dev)

    def step(k):
        runtime.solve_with_scratch(md, dev[k % nb], scratch[k % nb], use_optimized_kernel=True)

    with ClockSampler(local) as clocks:
        clocks.wait_started()
        for k in range(args.warmup):
            step(k)
        timer.barrier()
        t_begin = time.perf_counter()
        round_ms = timer.rounds(step, args.steps, args.rounds, min_seconds=1.2)
        t_end = time.perf_counter()
    ms, ms_p10, ms_p90 = percentiles(round_ms)
    value = world * args.nworld * args.steps / (ms * 1e-3)
    niter = np.concatenate([dd.solver_niter.cpu().numpy() for dd in dev])

    # the same steps as one CUDA-graph replay (the reference's step runs inside a graph)
    graph_ms = None
    if not args.no_graph:
        graph_steps = min(args.steps, 4 * nb)
        graph = graph_of(torch, step, graph_steps)
        graph_ms = timer.max_over_ranks([time_graph(torch, graph, graph_steps)])[0]

    # ---- strong scaling: a fixed total of worlds divided over the GPUs --------------
    strong = None
    if not args.no_strong and args.nworld >= STRONG_TOTAL_WORLDS // world and STRONG_TOTAL_WORLDS % world == 0:
        Ws = STRONG_TOTAL_WORLDS // world
        sdev = [mjw_model.slice_worlds(dd, 0, Ws) for dd in dev]
        ssc = [runtime.make_optimized_fwd_position_scratch(md, dd, device) for dd in sdev]
        if groups is not None:
            for dd, sc in zip(sdev, ssc):
                runtime.refresh_sparse_hessian(md, dd, sc, groups, device)
        sstep = lambda k: runtime.solve_with_scratch(md, sdev[k % nb], ssc[k % nb], use_optimized_kernel=True)  # noqa: E731
        for k in range(args.warmup):
            sstep(k)
        sms, sp10, sp90 = percentiles(timer.rounds(sstep, args.steps, 9))
        strong = {
            "total_worlds": STRONG_TOTAL_WORLDS, "worlds_per_gpu": Ws, "ms_per_step": sms / args.steps,
            "ms_per_step_p10": sp10 / args.steps, "ms_per_step_p90": sp90 / args.steps,
            "value": STRONG_TOTAL_WORLDS * args.steps / (sms * 1e-3),
            # one GPU solving all of them = this run's own step when it holds that many worlds per GPU
            "speedup_vs_one_gpu": (ms / sms) if args.nworld == STRONG_TOTAL_WORLDS else None,
            "note": "eager launches; a world is solved by one warp, so with few worlds per GPU the step "
                    "lasts as long as its slowest world's solve",
        }
        del sdev, ssc

    # ---- end to end: pinned host batches in, host results out, every step -----------
    e2e = None
    if not args.no_e2e:
        grouped = [host_batch.group_by_row_count(d)[0] for _, d in host]
        # pinned staging memory on the NUMA node of this rank's GPU (with one process per GPU
        # the ranks' copies otherwise all read one socket's memory)
        near = host_batch.host_near_device(local)
        near.__enter__()
        pinned = [host_batch.pin_batch(d, chunk=128) for d in grouped]
        ldj = int(dev[0].efc.J.stride(1))
        njmax = int(host[0][1].njmax)
        e2e_steps = min(args.steps, 50)

        def e2e_measure(mode):
            pipe = host_batch.HostBatchPipeline(md, grouped[0], device, slots=min(3, nb),
                                                sparse_groups=groups, mode=mode)
            nslot = len(pipe.slots)

            def run(n):
                total = 0.0
                for k in range(n):
                    if k >= nslot:
                        total += float(pipe.result(k - nslot)["solver_niter"][0])  # frees the slot step k reuses
                    pipe.submit(k, pinned[k % nb])
                for k in range(max(n - nslot, 0), n):
                    total += float(pipe.result(k)["solver_niter"][0])
                return total

            torch.cuda.synchronize()
            run(4)
            dts = []
            for _ in range(5):
                timer.barrier()
                t0 = time.perf_counter()
                checksum = run(e2e_steps)
                torch.cuda.synchronize()
                dts.append(time.perf_counter() - t0)
                timer.barrier()
            dt, dt10, dt90 = percentiles(timer.max_over_ranks(dts))
            h2d = float(np.mean([b.h2d_bytes(m_host.nv, ldj, m_host.nM, njmax, mode) for b in pinned]))
            del pipe
            return {
                "value": world * args.nworld * e2e_steps / dt,
                "unit": UNIT,
                "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(pinned[0].d2h_bytes(m_host.nv, njmax, mode)),
                "steps": e2e_steps,
                "ms_per_step": 1e3 * dt / e2e_steps,
                "ms_per_step_p10": 1e3 * dt10 / e2e_steps,
                "ms_per_step_p90": 1e3 * dt90 / e2e_steps,
                "h2d_gbs_per_gpu": h2d * e2e_steps / dt / 1e9,  # the copy is the limit of this path
                "copies": {"compact": "efc.J as the nefc rows of each world back to back on the host (the layout of "
                                      "MuJoCo C's mjData.efc_J), one contiguous copy, per-world offsets to the kernel",
                           "rows": "padded efc.J, rows [0, largest nefc of each chunk of 128 worlds) by strided "
                                   "copies, worlds grouped by descending row count on the host",
                           "whole": "whole padded arrays",
                           "sparse": "efc.J as values + column indices + row starts of the live rows on the host (MuJoCo "
                                     "C's sparse efc_J / efc_J_colind / efc_J_rowadr), expanded to dense rows on the "
                                     "device: only the nonzeros cross PCIe; all inputs in one pinned buffer (one copy each way)",
                           "sparse8": "efc.J as values + 8-bit column indices + row starts of the live rows on the host "
                                      "(nv <= 79 on the fused path), expanded to dense rows on the device: 5 bytes per "
                                      "nonzero cross PCIe; all inputs in one pinned buffer (one copy each way)"}[mode],
                "nslot": nslot,
                "checksum": checksum,
            }

        modes = {mode: e2e_measure(mode) for mode in ("sparse8", "sparse", "compact", "rows", "whole")}
        best = max(modes, key=lambda k: modes[k]["value"])
        e2e = dict(modes[best])
        near.__exit__(None, None, None)
        e2e["api"] = "instantmimic_b200.host_batch.HostBatchPipeline.submit / result"
        e2e["host_numa_node"] = near.node  # None: the platform does not say
        e2e["pipeline"] = f"{e2e.pop('nslot')} slots (copies of step k+1 overlap the solve of step k)"
        e2e["other_copy_modes"] = [
            {k: modes[mode][k] for k in ("copies", "value", "ms_per_step", "h2d_bytes_per_step", "h2d_gbs_per_gpu")}
            for mode in modes if mode != best]
        del pinned

    # ---- work counters -> flop count of one batch -------------------------------------
    counting = runtime.make_optimized_fwd_position_scratch(md, dev[0], device, with_stats=True)
    if groups is not None:
        runtime.refresh_sparse_hessian(md, dev[0], counting, groups, device)
    runtime.solve_with_scratch(md, dev[0], counting, use_optimized_kernel=True)
    torch.cuda.synchronize()
    stats = counting.solver_context.stats.cpu().numpy()
    state0 = dev[0].efc.state.cpu().numpy()
    plan0 = getattr(scratch[0].solver_context, "sparse_hessian_plan", None)
    flops = algorithmic_flops(m_host, host[0][1], dev[0].solver_niter.cpu().numpy(), stats, state0, plan0)

    # ---- the M-side kernels of the same path at a batch that exceeds L2 --------------
    aux = None
    if world == 1 and not args.no_aux:
        from instantmimic_b200.mjw_kernels import indexed_factor

        W, nv, nM = args.aux_nworld, m_host.nv, m_host.nM
        reps = max(1, W // args.nworld)
        rep = lambda t: t.repeat((reps,) + (1,) * (t.dim() - 1))[:W].contiguous()  # noqa: E731
        from types import SimpleNamespace

        big = [SimpleNamespace(nworld=W, M=rep(dev[i].M), y=rep(dev[i].qfrc_smooth), x=rep(dev[i].qacc_smooth))
               for i in range(2)]
        sc0 = scratch[0]
        aux = {"worlds": W, "batches_rotated": 2,
               "note": "timed as CUDA-graph replays of 8 calls over two rotating batches (M alone is "
                       f"{4 * W * nM / 1e6:.0f} MB per batch, so every call reads DRAM)"}

        def timed(fn):
            g = graph_of(torch, fn, 8)
            return time_graph(torch, g, 8) * 1e-3

        if sc0.tree_factor_solve is not None:
            t = timed(lambda k: runtime._factor_solve_i_dense(
                md, big[k % 2], big[k % 2].M, big[k % 2].x, big[k % 2].y, None,
                tree_factor_solve=sc0.tree_factor_solve))
            alg = 4.0 * W * (nM + 2 * nv)
            generated = sc0.tree_factor_solve.kernel is not None
            aux["tree_ldl_generated" if generated else "tree_ldl_kernel"] = {
                "ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg,
                "groups": sc0.tree_factor_solve.groups}
        if sc0.dense_factor_solve is not None:
            bs = indexed_factor.create_blocked_dense_factor_solve_scratch(md, big[0], device)
            t = timed(lambda k: indexed_factor.blocked_dense_factor_solve(
                big[k % 2], big[k % 2].M, big[k % 2].x, big[k % 2].y, bs))
            alg = 4.0 * W * (nM + 2 * nv + bs.pad * bs.pad)
            aux["blocked_dense_kernel"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg}
            del bs
        outv = torch.empty_like(big[0].x)
        t = timed(lambda k: runtime.mul_m(md, big[k % 2], outv, big[k % 2].y))
        alg = 4.0 * W * (nM + 2 * nv)
        aux["mul_m_kernel"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg}
        gen = runtime.generated_mul_m_kernel(md, big[0])
        if gen is not None:
            t = timed(lambda k: runtime.mul_m(md, big[k % 2], outv, big[k % 2].y, kernel=gen))
            aux["mul_m_generated"] = {"ms": t * 1e3, "achieved_gbs": alg / t / 1e9, "algorithmic_bytes": alg}
        del big, outv
        torch.cuda.empty_cache()
        aux.update(stage_kernels(args, torch, md, m_host, device, timed))
        torch.cuda.empty_cache()

    sweep = run_sweep(args, torch, timer, world, rank, device, peak) if sweep_mode else None

    if rank == 0:
        from instantmimic_b200.mjw_kernels import newton_fusion

        info = newton_fusion.solve_call(md, dev[0], scratch[0].solver_context, scratch[0].solver_nsolving,
                                        cache_on=scratch[0]).launch_info()
        alg = float(np.mean([algorithmic_bytes(m_host, d) for _, d in host]))
        launch_s = (ms * 1e-3) / args.steps
        achieved = alg / launch_s / 1e9
        fp32_peak = 2.0 * 128 * props.multi_processor_count * 1.965e9 / 1e12  # TFLOP/s at the max SM clock
        line = {
            "metric": METRIC,
            "value": value,
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms / args.steps,
            "ms_per_step_p10": ms_p10 / args.steps,
            "ms_per_step_p90": ms_p90 / args.steps,
            "rounds": len(round_ms),
            "timing": "median over rounds of exactly --steps eager steps between two CUDA events "
                      "(device synchronised and ranks joined on both sides; per round the max over ranks)",
            "graph_replay_ms_per_step": graph_ms,
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
                "traffic": NCU_TRAFFIC_BYTES_PER_WORLD_HUMANOID * args.nworld if args.workload == "humanoid" else None,
                "traffic_source": ("ncu capture of a 16384-world launch of the same kernel and workload, scaled by worlds"
                                   if args.workload == "humanoid" else None),
                "algorithmic_bytes_per_launch": alg,
                "launch_ms": launch_s * 1e3,
                "fp32": {
                    "algorithmic_flops_per_launch": flops,
                    "achieved_tflops": flops / launch_s / 1e12,
                    "peak_tflops": fp32_peak,
                    "peak_source": f"2 x 128 lanes x {props.multi_processor_count} SMs x 1.965 GHz",
                    "frac": flops / launch_s / 1e12 / fp32_peak,
                },
                "binding": "neither: the solve is a chain of dependent small-matrix steps per world, bound by "
                           "instruction issue and latency",
            },
            "solver": {
                "niter_mean": float(niter.mean()),
                "niter_max": int(niter.max()),
                "smem_bytes_per_world": int(info.smem_bytes),
                "line_search_passes_mean": float(stats[:, 0].mean()),
                "factorisations_mean": float(stats[:, 2].mean()),
            },
        }
        if strong is not None:
            line["strong"] = strong
        if aux is not None:
            for v in aux.values():
                if isinstance(v, dict):
                    v["frac_of_hbm_peak"] = v["achieved_gbs"] / peak
            line["aux_kernels"] = aux
        if sweep is not None:
            line["sweep"] = sweep
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args, host)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
