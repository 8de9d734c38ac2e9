"""Throughput of the eSCN-MD (UMA-s) energy+force path in atom-steps/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

A step is one energy+forces evaluation of the whole system: radius graph (rebuilt every step),
edge geometry, edge-degree embedding, 4 message-passing layers, energy head and the backward
pass that yields the forces, followed by a velocity-Verlet update of the positions (own
integrator).  The default workload is the 100,000-atom periodic water box; weights are seeded
random-init in the UMA-s shape, float32 (no dataset or checkpoint is read).

One JSON line is printed by rank 0 (see the keys below).  ``value`` is measured with the
positions resident on the device; ``e2e`` runs the same steps through the module interface with
host buffers: positions come from pinned host memory each step and energy+forces go back to the
host each step.  ``--impl reference`` times the CPU oracle (the reference's algorithm restated
for the host, checked against the reference's own outputs) on a bounded sample of the workload.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from fairchem_b200 import synthetic, weights  # noqa: E402

ACC = 9.648533e-3  # (eV/A)/amu -> A/fs^2
MASS = {1: 1.008, 6: 12.011, 7: 14.007, 8: 15.999, 24: 51.996, 25: 54.938, 26: 55.845, 27: 58.933, 28: 58.693, 29: 63.546}
CPU_SAMPLE_ATOMS = 1500
# DRAM bytes (read + write) per edge of one launch of so2_conv_fused_kernel, mean over its four convolution plans, from the
# ncu capture of 62 118-edge launches summarised in profiles/so2_conv_fused_kernel_bcc_alloy_2000.md:
# (1520 + 597) + (348 + 244) + (875 + 317) + (460 + 526) MB over 4 launches; traffic grows in proportion to the edges
FUSED_TRAFFIC_PER_EDGE_LAUNCH = (2117e6 + 592e6 + 1192e6 + 986e6) / 4 / 62118


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.rows, self.proc = [], None
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.cmd = ["nvidia-smi", f"--id={uuid}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"]
        except Exception:
            self.cmd = None

    def start(self):
        if self.cmd is None:
            return
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def masses_for(z: torch.Tensor) -> torch.Tensor:
    table = torch.full((120,), 12.0)
    for k, v in MASS.items():
        table[k] = v
    return table[z.cpu()].to(z.device)


class MDState:
    """Velocity-Verlet state (positions, velocities, accelerations) on one device."""

    def __init__(self, data, dt_fs: float = 0.5):
        self.data = data
        self.dt = dt_fs
        self.vel = torch.zeros_like(data["pos"])
        self.inv_m = (ACC / masses_for(data["atomic_numbers"])).view(-1, 1).to(data["pos"].dtype)
        self.box = torch.diagonal(data["cell"][0]).clone()
        self.periodic = bool(data["pbc"].all())

    @torch.no_grad()
    def advance(self, forces: torch.Tensor):
        """One force evaluation per step: v += dt*a, x += dt*v (leapfrog form of velocity Verlet)."""
        self.vel += self.dt * forces * self.inv_m
        pos = self.data["pos"].detach() + self.dt * self.vel
        if self.periodic:
            pos = pos - torch.floor(pos / self.box) * self.box
            pos = torch.where(pos >= self.box, torch.zeros_like(pos), pos)
        self.data["pos"] = pos.contiguous()


def run_b200(args):
    from fairchem_b200 import backbone as B
    from fairchem_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl b200 needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        # the per-layer exchanges are small all-to-alls and the reductions move 1.2 MB: nothing here gains from
        # in-switch reduction, and without it a rank that fails cannot fault its peers through a multicast binding
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    B.set_gemm_precision(args.precision)
    if args.conv_variant is not None:
        ops.CONV_VARIANT = args.conv_variant
    if args.edge_source_sums:
        from fairchem_b200 import backbone as _bb

        _bb._GemmState.node_sums = False
    if args.generic_kernels:
        from fairchem_b200 import ops as _ops

        _ops.set_generic_kernels(True)
    cfg, model_name = MODELS[args.model]
    sd = weights.random_init_state_dict(cfg, args.seed)
    bb, head = B.build_model(cfg, sd, device=dev, edge_chunk_size=args.chunk)
    host = synthetic.WORKLOADS[args.workload](args.seed)
    n_atoms = int(host["pos"].shape[0])
    if world > 1:
        from fairchem_b200 import parallel

        stepper = parallel.PartitionedStepper(bb, head, host, dev, rank, world)
    else:
        stepper = None
    data = host.to(dev)
    md = MDState(data)

    def one_step():
        if stepper is not None:
            energy, forces = stepper.step(data)
        else:
            out = head(data, bb(data))
            energy, forces = out["energy"], out["forces"]
        md.advance(forces)
        return energy, forces

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_step()
    barrier()
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        energy, _ = one_step()
    t1.record()
    barrier()
    ms = t0.elapsed_time(t1)
    clocks = sampler.stop() if rank == 0 else None
    # second pass, not part of `value`: the same steps with two CUDA events around every launch of this library's
    # kernels, for the per-kernel table and the roofline of the dominant kernel
    prof_steps = max(1, min(args.steps, 3))
    prof = ops.LaunchProfiler(timed=True)
    ops.set_profiler(prof)
    barrier()
    for _ in range(prof_steps):
        one_step()
    barrier()
    summary = prof.summary()
    ops.set_profiler(None)
    launches = prof.launches // prof_steps * args.steps  # launches inside the timed region (same steps, counted here)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    edges = int(bb.last_graph["edge_index"].shape[1]) if bb.last_graph else 0
    if world > 1:  # every rank holds the edges of its own targets only
        t = torch.tensor([edges], device=dev, dtype=torch.int64)
        torch.distributed.all_reduce(t)
        edges = int(t.item())

    # end to end through the public interface with host buffers
    from fairchem_b200.predict import B200PredictUnit

    unit = B200PredictUnit(bb, head, device=dev)
    pin_pos = data["pos"].detach().cpu().pin_memory()
    pin_f = torch.empty_like(pin_pos).pin_memory()
    pin_e = torch.empty(1, dtype=torch.float64).pin_memory()
    h2d = pin_pos.numel() * 4
    d2h = pin_f.numel() * 4 + 8
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        data["pos"] = pin_pos.to(dev, non_blocking=True)
        if stepper is not None:
            energy, forces = stepper.step(data)
        else:  # the call a calculator makes: predict-unit surface over the backbone (graph rebuilt every step, skin 0)
            out = unit.predict(data)
            energy, forces = out["energy"], out["forces"]
        pin_f.copy_(forces, non_blocking=True)
        pin_e.copy_(energy[:1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        # the host owns the integrator in this mode
        md.data["pos"] = data["pos"]
        md.advance(forces)
        pin_pos.copy_(md.data["pos"])
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        e2e_ms = float(t.item())

    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    peaks = load_peaks()
    # the fused convolution kernel is one kernel launched with four tile plans: one roofline entry for it
    by_kernel = {}
    for k, v in summary.items():
        # (the radial MLP's output layer runs on the same kernel but is bound by storing its wide output: own entry)
        key = "so2_conv_fused" if k.startswith("so2_conv_fused_conv") else k
        d = by_kernel.setdefault(key, {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
        for f in d:
            d[f] += v[f]
    top = max(by_kernel.items(), key=lambda kv: kv[1]["ms"]) if by_kernel else ("none", {"ms": 0.0, "bytes": 0, "flops": 0, "launches": 0})
    name, rec = top
    if name in ("gemm_f16x2", "gemm_f16x2_presplit", "so2_conv_fused", "so2_conv_fused_radial_out"):
        peak = peaks["bf16_tflops"]
        ach = rec["flops"] / (rec["ms"] * 1e-3) / 1e12 if rec["ms"] else 0.0
        traffic = None
        if name == "gemm_f16x2_presplit" and rec["launches"]:
            # ncu on a 62 119-edge chunk: 203.6 MB of DRAM traffic per launch, equal to the algorithmic bytes
            # (A_hi + A_lo + C once); per-launch traffic grows with the edges per launch
            n_chunks = max(1, -(-edges // args.chunk)) if world == 1 else None
            if n_chunks:
                traffic = 203.6e6 * (edges / n_chunks) / 62119.0
        if name == "so2_conv_fused" and rec["launches"] and FUSED_TRAFFIC_PER_EDGE_LAUNCH:
            per_rank = edges / world  # every rank launches over its own targets' edges
            traffic = FUSED_TRAFFIC_PER_EDGE_LAUNCH * per_rank / max(1, -(-int(per_rank) // args.chunk))
        roof = {"kernel": name + "_kernel", "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "traffic": traffic, "launches": rec["launches"], "issued": ach * 3, "frac_issued": ach * 3 / peak,
                "peak_source": f"{peaks['source']} bf16 sustained (kind::f16 issues at the bf16 rate)",
                "note": "achieved counts algorithmic float32 FLOPs; float32-accurate mode issues 3 half-precision MMAs per "
                        "product, so `issued` = 3 x achieved is what the tensor pipe executes; traffic is scaled from an ncu "
                        "capture of a 62 119-edge launch by the edges per launch"}
    elif name == "gemm_tf32":
        peak = peaks["bf16_tflops"] / 2.0
        ach = rec["flops"] / (rec["ms"] * 1e-3) / 1e12 if rec["ms"] else 0.0
        passes = 3 if args.precision == 3 else 1
        roof = {"kernel": "gemm_tf32_kernel", "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "traffic": None, "launches": rec["launches"],
                "issued": ach * passes, "frac_issued": ach * passes / peak,
                "peak_source": f"{peaks['source']} bf16 sustained / 2 (TF32 issues at half the bf16 rate; cuBLAS TF32 "
                               "measured 590-720 TFLOP/s on these shapes on this pool)",
                "note": "achieved counts algorithmic float32 FLOPs; float32-accurate mode issues 3 TF32 MMAs per product, "
                        "so `issued` = 3 x achieved is what the tensor pipe executes"}
    else:
        peak = peaks["hbm_gbs"]
        ach = rec["bytes"] / (rec["ms"] * 1e-3) / 1e9 if rec["ms"] else 0.0
        roof = {"kernel": name, "bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "traffic": None, "launches": rec["launches"], "peak_source": peaks["source"]}
    total_kernel_ms = sum(v["ms"] for v in summary.values())
    shares = {k: round(v["ms"] / total_kernel_ms, 4) for k, v in sorted(summary.items(), key=lambda kv: -kv[1]["ms"])} if total_kernel_ms else {}
    per_kernel = {}
    for k, v in summary.items():
        if not v["ms"]:
            continue
        per_kernel[k] = {"ms_per_step": round(v["ms"] / prof_steps, 3), "launches_per_step": v["launches"] // prof_steps,
                         "GBps": round(v["bytes"] / (v["ms"] * 1e-3) / 1e9, 1)}
        if v["flops"]:
            per_kernel[k]["TFLOPps"] = round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 2)
    cpu = cpu_baseline(args, reps=3, warmup=1) if world == 1 and not args.skip_cpu else None
    line = {
        "metric": "atom_steps_per_s", "value": n_atoms * args.steps / (ms * 1e-3), "unit": "atom-steps/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "atoms": n_atoms, "edges": edges, "model": model_name,
                   "cutoff": 6.0, "max_neighbors": 30, "gemm_precision": {3: "tf32x3", 2: "f16x3", 1: "tf32", 0: "cublas_fp32"}[args.precision],
                   "edge_chunk": args.chunk, "l2": "inputs larger than L2 (node and edge arrays of 0.4-2 GB per pass)",
                   "parallelism": f"gp{world}", "energy": float(energy[0]),
                   "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
                   "arithmetic": "float32 results; contractions as 3 half-precision tensor-core products per float32 "
                                 "product (22-bit operands, float32 accumulation), not IEEE float32"
                                 if args.precision == 2 else "float32"},
        "clocks": clocks,
        "e2e": {"value": n_atoms * args.steps / (e2e_ms * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": roof,
        "cpu_baseline": cpu,
        "kernel_time_share": shares,
        "per_kernel": per_kernel,
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 1e9, 2),
        "energy": float(energy[0]),
    }
    if args.profile_run:
        line["profile_run"] = True
    _emit(line)


MODELS = {
    "uma_s": (weights.UMA_S, "UMA-s shape (4 layers, C=128, lmax=mmax=2)"),
    "escn_md_l4": (weights.ESCN_MD_L4, "eSCN-MD shape (10 layers, C=128, lmax=4, mmax=2)"),
}


def _cpu_sample(args):
    """A bounded sample of the workload for the host: the same material at the same density with fewer atoms."""
    if args.workload.startswith("water"):
        return (synthetic.water_box(CPU_SAMPLE_ATOMS, seed=args.seed),
                f"{CPU_SAMPLE_ATOMS}-atom water box of the same density (graph + energy + forces)")
    if args.workload == "fcc_cu_20000":
        cells = (6, 6, 6) if args.model == "escn_md_l4" else (7, 7, 7)
        d = synthetic.fcc_cu(cells, seed=args.seed)
        return d, f"{int(d['pos'].shape[0])}-atom FCC Cu supercell of the same lattice (graph + energy + forces)"
    return synthetic.WORKLOADS[args.workload](args.seed), f"full {args.workload}"


def _reference_modules(cfg, sd):
    """The reference's own backbone + head on the CPU when a checkout is present (its location comes from the
    environment, see oracle/ref_shim.py); None otherwise."""
    try:
        from oracle import ref_shim
        if not ref_shim.available():
            return None
        overrides = {k: cfg[k] for k in cfg if k in ("lmax", "mmax", "num_layers", "sphere_channels", "hidden_channels")}
        bb, head = ref_shim.build_reference_model(0, **overrides)
        bsd, hsd = weights.split_head(sd)
        bb.load_state_dict(bsd, strict=False)
        head.energy_block.load_state_dict(hsd)
        return lambda sample: ref_shim.run_reference(bb, head, sample)
    except Exception:
        return None


def cpu_baseline(args, reps: int = 3, warmup: int = 1):
    """The reference's CPU path on a bounded sample of the workload (a box of the same density with fewer atoms):
    the reference's own modules when a checkout is importable (kind "reference"), else the CPU oracle, its pinned
    restatement (kind "port").  ``warmup`` untimed passes, then exactly ``reps`` timed ones."""
    from oracle import escn_md_oracle as oracle_model
    from oracle import radius_graph_oracle as oracle_graph

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample, what = _cpu_sample(args)
    cfg = MODELS[args.model][0]
    sd = weights.random_init_state_dict(cfg, args.seed)
    ref_step = _reference_modules(cfg, sd)

    def port_step(sample):
        ei, co, _, _ = oracle_graph.radius_graph(sample.pos.numpy(), sample.cell.numpy(), sample.pbc.numpy(),
                                                 sample.natoms.numpy(), 6.0, 30)
        oracle_model.energy_and_forces(sd, cfg, sample, torch.from_numpy(ei), torch.from_numpy(co))

    step = ref_step or port_step
    times = []
    for i in range(warmup + reps):
        t = time.perf_counter()
        step(sample)
        if i >= warmup:  # the first passes warm the allocator and thread pool
            times.append(time.perf_counter() - t)
    n = int(sample["pos"].shape[0])
    total = sum(times)
    return {"value": n * len(times) / total, "unit": "atom-steps/s", "cores": threads,
            "kind": "reference" if ref_step else "port", "sample": what, "s_per_step": total / len(times),
            "s_per_step_min": min(times), "s_per_step_median": statistics.median(times), "timed_steps": len(times),
            "warmup_steps": warmup}


def run_reference(args):
    """Reference arm: exactly ``--steps`` timed CPU steps after ``--warmup`` untimed ones; ``value`` is the mean rate over
    the timed steps (steps x atoms / total time), min and median are reported beside it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = cpu_baseline(args, reps=max(1, args.steps), warmup=max(0, args.warmup))
    n = int(_cpu_sample(args)[0]["pos"].shape[0])
    line = {
        "impl": "reference", "metric": "atom_steps_per_s", "value": cpu["value"], "unit": "atom-steps/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": cpu["timed_steps"], "warmup": cpu["warmup_steps"],
        "ms_per_step": cpu["s_per_step"] * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample_atoms": n, "model": MODELS[args.model][1]},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "atom-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit(line)


_JSON_FD = None


def _claim_stdout():
    """Keep the process's stdout for the one JSON line: libraries that print banners on fd 1 (NCCL's
    version line) are pointed at stderr instead."""
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)


def _emit(line: dict):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="water_100k", choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--model", default="uma_s", choices=sorted(MODELS),
                    help="uma_s: the configuration the metric is quoted on; escn_md_l4: the 10-layer lmax=4/mmax=2 shape")
    ap.add_argument("--precision", type=int, default=2, choices=[0, 1, 2, 3])
    ap.add_argument("--chunk", type=int, default=131072)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--edge-source-sums", action="store_true",
                    help="gather backward with the source half per edge plus a segmented sum instead of per-node sums (A/B measurement)")
    ap.add_argument("--generic-kernels", action="store_true",
                    help="route the lmax=2 model through the any-lmax edge-block kernels (A/B measurement)")
    ap.add_argument("--conv-variant", type=int, default=None, choices=[-1, 0, 1, 2],
                    help="launch form of the fused convolution kernel: 0 one CTA per 128-edge tile (32-deep stages), 1 CTA pairs, "
                         "2 64-deep stages, -1 the default choice per launch (A/B measurement)")
    ap.add_argument("--profile-run", action="store_true",
                    help="for runs under a profiler: allows fewer than 3 warm-up steps; the printed number is not a bench value")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "b200" and not args.profile_run:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
