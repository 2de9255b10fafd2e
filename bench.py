"""Benchmark of the sparse-convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = the whole hot path on one batch of synthetic rooms: coordinate hash
insert (SparseTensor construction) -> 3^3 kernel map (neighbour table + pair
lists) -> 64 -> 64 bf16 forward convolution, on a fresh coordinate manager every
step. The metric is forward throughput in Mvoxels/s (input voxels of all ranks
divided by the slowest rank's time). Under torchrun every rank runs its own batch
of rooms (weak scaling by sample; the forward pass needs no collective).

``--impl reference`` times the reference's own CPU implementation of the same
path (the unmodified reference sources behind ``oracle/_ref/ref_driver``; the
oracle's C restatement if that binary is absent) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sparse_conv_fwd_mvoxels_per_s"
UNIT = "Mvoxels/s"
N_SCENES, N_VOXELS = 8, 150_000
C_IN, C_OUT, KSIZE = 64, 64, 3
K_VOL = KSIZE ** 3
CPU_SAMPLE_SCENES = N_SCENES  # the reference arm runs the whole batch of one rank


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "indoor-room batch: 8 scenes x 150K voxels on a 200x200x60 grid per GPU, "
                    "3^3 stride-1 conv 64->64, hash insert + kernel map + forward",
        "scenes_per_gpu": N_SCENES, "voxels_per_scene": N_VOXELS, "kernel": "3x3x3", "stride": 1,
        "c_in": C_IN, "c_out": C_OUT, "sharding": f"by sample, {n_gpus} rank(s), no forward collective",
        "l2_policy": "inputs and tables (>200 MB per step) exceed the 126 MB L2; no explicit flush",
    }


def captured_traffic(*names: str):
    """DRAM bytes per launch (read + write) of the named kernels from the committed ncu capture of
    this exact workload (profiles/dram_traffic_indoor8x150k.json); None if the file is missing."""
    path = os.path.join(ROOT, "profiles", "dram_traffic_indoor8x150k.json")
    try:
        with open(path) as f:
            t = json.load(f)
        return int(sum(t[n]["dram_read_bytes"] + t[n]["dram_write_bytes"] for n in names))
    except (OSError, KeyError, ValueError):
        return None


class stdout_to_stderr:
    """Point file descriptor 1 at stderr for the duration of the block (native libraries write
    banners to stdout behind Python's back)."""

    def __enter__(self):
        sys.stdout.flush()
        self._saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self._saved, 1)
        os.close(self._saved)
        return False


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons while the timed region runs: an NVML
    polling thread (read-only queries, every 2 ms), or nvidia-smi if NVML cannot be loaded."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        import threading
        self.proc = None
        self.thread = None
        self.samples = []          # (sm_mhz, reasons bitmask)
        self.max_mhz = None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            # LOCAL_RANK indexes CUDA_VISIBLE_DEVICES; map it to the NVML index
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            nvml_index = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            handle = pynvml.nvmlDeviceGetHandleByIndex(nvml_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml

            def poll():
                while not self._stop.is_set():
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                        why = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.samples.append((float(mhz), int(why)))
                    except Exception:
                        break
                    time.sleep(0.002)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
            try:
                self.proc = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                     "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except OSError:
                self.proc = None

    def stop(self) -> dict:
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            n = self._nvml
            flags = {"hw_slowdown": n.nvmlClocksEventReasonHwSlowdown,
                     "hw_thermal_slowdown": n.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": n.nvmlClocksEventReasonSwThermalSlowdown,
                     "sw_power_cap": n.nvmlClocksEventReasonSwPowerCap}
            sm = [s[0] for s in self.samples]
            reasons = sorted(name for name, bit in flags.items() if any(s[1] & bit for s in self.samples))
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz,
                    "samples": len(sm), "reasons": reasons, "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


def bind_to_gpu_numa_node(local_rank: int) -> dict:
    """Pin this process to the CPUs of the NUMA node its GPU hangs off (read from sysfs; read-only queries),
    BEFORE any page-locked buffer is allocated, so that first touch places the staging buffers of the
    end-to-end path on the GPU's own node. Returns what was found for the bench line."""
    info = {"numa_node": None, "cpus_bound": None}
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = int(visible.split(",")[local_rank]) if visible and visible.split(",")[local_rank].isdigit() else local_rank
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(idx)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:      # NVML prints an 8-digit domain, sysfs a 4-digit one
            bus = bus[4:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info["numa_node"] = node
        if node >= 0:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["cpus_bound"] = len(allowed)
    except Exception as exc:  # no NVML / sysfs entry: run unbound
        info["error"] = str(exc)[:80]
    return info


def make_batch(rank: int):
    from riemannengine_b200 import synthetic
    coords = synthetic.indoor_batch(N_SCENES, N_VOXELS, seed=2000 + 100 * rank)
    feats = synthetic.features(2500 + rank, len(coords), C_IN)
    weights = synthetic.conv_weights(2600, K_VOL, C_IN, C_OUT)
    return coords, feats, weights


# ------------------------------------------------------------------------------------------
# reference arm: the reference's CPU implementation on the host cores
# ------------------------------------------------------------------------------------------
def cpu_reference_time(coords, feats, weights, steps: int, warmup: int):
    """Returns (seconds for `steps` steps, voxels per step, info dict)."""
    from oracle import refrun
    cores = os.cpu_count() or 1
    if refrun.available():
        out = refrun.run(coords, feats, weights, KSIZE, 1, 1, threads=0, reps=steps, warmup=warmup,
                         timing_only=True)
        per_step = out["times_all"][:, 0] + out["times_all"][:, 1]  # SparseTensor ctor + first forward
        return float(per_step.sum()) / 1e3, len(coords), {
            "kind": "reference", "cores": int(out["info"][1]), "hardware_concurrency": int(out["info"][0]),
            "phases_ms": {"sparse_tensor_ctor": float(out["times_ms"][0]), "first_forward": float(out["times_ms"][1]),
                          "cached_forward": float(out["times_ms"][2]), "forward_backward": float(out["times_ms"][3])}}
    from oracle import oracle as O
    total = 0.0
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        mapping, _ = O.insert_and_map(coords)
        uc = coords[mapping]
        ptr, a, q = O.conv_kernel_map(uc, uc, O.region_offsets(O.HYPER_CUBE, [KSIZE] * 3, [1] * 3, [1] * 3))
        O.conv_forward(feats[mapping], weights, ptr, a, q, len(uc))
        if it >= warmup:
            total += time.perf_counter() - t0
    return total, len(coords), {"kind": "port", "cores": 1, "hardware_concurrency": cores}


def cpu_sample():
    from riemannengine_b200 import synthetic
    coords = synthetic.indoor_batch(CPU_SAMPLE_SCENES, N_VOXELS, seed=2000)
    feats = synthetic.features(2500, len(coords), C_IN)
    weights = synthetic.conv_weights(2600, K_VOL, C_IN, C_OUT)
    return coords, feats, weights


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    coords, feats, weights = cpu_sample()
    seconds, voxels, info = cpu_reference_time(coords, feats, weights, args.steps, args.warmup)
    value = voxels * args.steps / seconds / 1e6
    sample = (f"all {CPU_SAMPLE_SCENES} scenes of one rank's batch ({voxels} voxels), fp32 features, "
              "SparseTensor construction + first forward (kernel map + convolution) per step")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": info["kind"],
                         "sample": sample, **{k: v for k, v in info.items() if k not in ("cores", "kind")}},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# training step of the headline workload and the other configurations (extra keys of the line)
# ------------------------------------------------------------------------------------------
def run_extras(args, C, dev, rank, world, coords, feats, weights_np, res, xf, conv) -> dict:
    """``train``: forward + backward (dX, dW) + weight-gradient all-reduce of the headline layer through the
    C++ host layer; ``configs``: the other benchmark configurations (riemannengine_b200/workloads.py). Times
    are the slowest rank's, voxels the sum over the ranks."""
    import torch
    import torch.distributed as dist

    from riemannengine_b200 import ops, workloads as W

    steps = max(3, min(args.steps, 10))
    warmup = 2

    def over_ranks(ms: float, voxels: float):
        t = torch.tensor([ms, voxels], dtype=torch.float64, device=dev)
        if world > 1:
            mx, sm = t.clone(), t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            return float(mx[0]), float(sm[1])
        return ms, voxels

    if world > 1:  # the layers reduce their weight gradients over this communicator in their backward pass
        box = [C.gradient_allreduce_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        with stdout_to_stderr():
            C.init_gradient_allreduce(box[0], rank, world, True)

    out = {}
    # ---- train: the headline layer, forward + backward + all-reduce ----------------------------------
    tconv = C.RiemannConvolution(C_IN, C_OUT, kernel_size=KSIZE, dimension=3)
    tconv.to(f"cuda:{dev.index}")
    tconv.to(torch.bfloat16)
    with torch.no_grad():
        tconv.kernel.copy_(torch.from_numpy(weights_np).to(dev))
    tfeats = feats.detach().clone().requires_grad_(True)
    grad_out = torch.randn(int(coords.size(0)), C_OUT, device=dev).bfloat16()  # stands in for the rest of a network

    def train_step():
        tconv.zero_grad()
        tfeats.grad = None
        y = tconv(C.SparseTensor(tfeats, coords))
        y.F.backward(grad_out)

    ms = W.time_steps(train_step, steps, warmup)
    ms_all, vox_all = over_ranks(ms, float(coords.size(0)))
    # the phases alone, on the cached map (device events, no host synchronisation in between)
    gy = grad_out
    wk = conv.kernel.detach()
    plan = ops.conv_plan_build(res.nbr, ops.region_offsets(0, [KSIZE] * 3, [1] * 3, [1] * 3))
    dw = ops.conv_backward_weight(xf, gy, res.nbr)
    fns = [lambda: ops.conv_forward(xf, wk, res.nbr, plan=plan),
           lambda: ops.conv_backward_input(gy, wk.flip(0), res.nbr, plan=plan),
           lambda: ops.conv_backward_weight(xf, gy, res.nbr),
           lambda: C.allreduce_gradients([dw])]
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(fns) + 1)] for _ in range(8)]
    for rep in marks:
        rep[0].record()
        for i, fn in enumerate(fns):
            fn()
            rep[i + 1].record()
    torch.cuda.synchronize()
    med = [statistics.median(rep[i].elapsed_time(rep[i + 1]) for rep in marks[2:]) for i in range(len(fns))]
    out["train"] = {
        "workload": "headline batch, 3^3 64->64 bf16: hash insert + kernel map + forward + backward (dX, dW) + "
                    "weight-gradient all-reduce, fresh manager every step, C++ host layer",
        "ms_per_step": ms_all, "mvoxels_per_s": vox_all / (ms_all / 1e3) / 1e6, "steps": steps,
        "phases_ms": {"forward_planned": med[0], "input_gradient_planned": med[1], "weight_gradient": med[2],
                      "allreduce_alone": med[3] if world > 1 else 0.0},
        "phases_note": "each phase timed alone on a cached map with a convolution plan; the step builds a fresh map, "
                       "for which the plan policy (two passes of one 64->64 layer) builds no plan",
        "allreduce_bytes": int(dw.numel() * 4) if world > 1 else 0,
        "allreduce": ("one ncclAllReduce per layer on a second stream behind the weight-gradient kernel, "
                      "overlapping the input-gradient kernel") if world > 1 else "single rank: none",
    }
    del tfeats, grad_out, dw, plan

    # ---- the other configurations ---------------------------------------------------------------------
    configs = {}
    runs = [("config1_sphere_shell_fp32", lambda: W.run_sphere_shell(C, dev, steps, warmup), "weak"),
            ("config3_lidar_chain_train", lambda: W.run_lidar_chain(C, dev, rank, steps, warmup), "weak"),
            ("config4_spatiotemporal_81_offsets", lambda: W.run_spatiotemporal(C, dev, rank, steps, warmup), "weak"),
            ("config5_unet_train", lambda: W.run_unet(C, dev, rank, world, max(3, steps // 2), 1), "strong")]
    for name, fn, scaling in runs:
        r = fn()
        torch.cuda.empty_cache()
        r["ms_per_step"], vox = over_ranks(r["ms_per_step"], float(r["voxels_per_step"]))
        r["voxels_per_step"] = vox
        r["mvoxels_per_s"] = vox / (r["ms_per_step"] / 1e3) / 1e6
        if "algorithmic_flops_per_step" in r:   # all ranks' flops over the slowest rank's time
            _, flops = over_ranks(0.0, float(r["algorithmic_flops_per_step"]))
            r["algorithmic_flops_per_step"] = flops
            r["algorithmic_tflops"] = flops / (r["ms_per_step"] / 1e3) / 1e12
            if r.get("dtype") == "bf16":          # the whole step (maps, norms, host gaps included) against the GEMM peak
                peak = load_peaks()
                r["frac_of_tensor_peak"] = r["algorithmic_tflops"] / (peak["bf16_tflops"] * world)
                r["peak_source"] = peak["source"]
        r["scaling"] = scaling
        r["n_gpus"] = world
        configs[name] = r
    if rank == 0 and world == 1:
        for name, base in cpu_baselines_of_configs().items():
            configs[name]["cpu_baseline"] = base
    out["configs"] = configs
    if world > 1:
        C.shutdown_gradient_allreduce()
    return out


def cpu_baselines_of_configs() -> dict:
    """The reference's CPU path (oracle/_ref/ref_driver) on a bounded sample of each of the other
    configurations, on the host cores of this box (rank 0, one GPU only): a reported baseline."""
    from oracle import refrun
    from riemannengine_b200 import synthetic, workloads as W
    if not refrun.available():
        return {}
    out = {}

    def entry(r, voxels, sample, fwd_bwd):
        ms = float(r["times_ms"][3]) + float(r["times_ms"][0]) if fwd_bwd else float(r["times_ms"][0] + r["times_ms"][1])
        return {"value": voxels / (ms / 1e3) / 1e6, "unit": UNIT, "cores": int(r["info"][1]), "kind": "reference",
                "ms": ms, "sample": sample}

    c, f, w = W.sphere_shell_inputs()
    r = refrun.run(c, f, w, 3, 1, 1, reps=3, warmup=1, timing_only=True)
    out["config1_sphere_shell_fp32"] = entry(r, len(c), "the whole configuration (101 930 voxels): SparseTensor "
                                             "construction + first forward, median of 3", False)
    c = W.lidar_batch(1, 3000)
    r = refrun.run(c, synthetic.features(1, len(c), 4), synthetic.conv_weights(2, 27, 4, 32), 3, 1, 1, reps=1,
                   timing_only=True)
    out["config3_lidar_chain_train"] = entry(r, len(c), "one sweep, first layer only (3^3 4->32, fp32): SparseTensor "
                                             "construction + forward + backward, one run", True)
    c = W.spatiotemporal_batch(1, 2, 4000)
    r = refrun.run(c, synthetic.features(3, len(c), 32), synthetic.conv_weights(4, 81, 32, 32), 3, 1, 1, reps=1,
                   timing_only=True)
    out["config4_spatiotemporal_81_offsets"] = entry(r, len(c), "one clip, two frames (300 K voxels), 3^4 32->32 fp32: "
                                                     "SparseTensor construction + first forward, one run", False)
    pts = synthetic.indoor_scene(5000, 150_000)
    c = np.concatenate([np.zeros((len(pts), 1), np.int32), pts], 1)
    r = refrun.run(c, synthetic.features(5, len(c), 32), synthetic.conv_weights(6, 27, 32, 32), 3, 1, 1, reps=1,
                   timing_only=True)
    out["config5_unet_train"] = entry(r, len(c), "one room, ONE 3^3 32->32 layer of the network (fp32): SparseTensor "
                                      "construction + forward + backward, one run (the network has 26 such passes at "
                                      "stride 1 alone)", True)
    return out


# ------------------------------------------------------------------------------------------
# product arm
# ------------------------------------------------------------------------------------------
def run_product(args) -> None:
    import torch
    import torch.distributed as dist

    from riemannengine_b200 import capi, engine as E, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    numa = bind_to_gpu_numa_node(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        with stdout_to_stderr():  # NCCL's version banner goes to stdout; stdout carries the JSON line only
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
    lib = capi.lib()

    coords_np, feats_np, weights_np = make_batch(rank)
    n_vox = len(coords_np)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(feats_np).to(dev).bfloat16()
    conv = E.RiemannConvolution(C_IN, C_OUT, kernel_size=KSIZE, dimension=3).to(dev).bfloat16()
    with torch.no_grad():
        conv.kernel.copy_(torch.from_numpy(weights_np).to(dev))
    offsets = ops.region_offsets(capi.HYPER_CUBE, [KSIZE] * 3, [1] * 3, [1] * 3)

    # The step runs through the C++ host layer (riemann_cpp) when it is built, else through the
    # Python mirror; both call the same C ABI.
    cpp_host = None
    if args.host != "py":
        try:
            from riemannengine_b200 import cpp as cpp_loader
            cpp_host = cpp_loader.load()
        except Exception as exc:  # pragma: no cover
            if args.host == "cpp":
                raise
            sys.stderr.write(f"C++ host layer unavailable ({exc}); using the Python host layer\n")
    if cpp_host is not None:
        cconv = cpp_host.RiemannConvolution(C_IN, C_OUT, kernel_size=KSIZE, dimension=3)
        cconv.to(f"cuda:{local_rank}")
        cconv.to(torch.bfloat16)
        with torch.no_grad():
            cconv.kernel.copy_(torch.from_numpy(weights_np).to(dev))

    def step(feats=feats, coords=coords):
        """Hot path on device-resident inputs: fresh manager, hash insert, kernel map, pair lists, forward."""
        if cpp_host is not None:
            x = cpp_host.SparseTensor(feats, coords)
            y = cconv(x)
            x.coordinate_manager.kernel_map_pairs(x.coordinate_map_key, y.coordinate_map_key, [KSIZE] * 3, [1] * 3,
                                                  [1] * 3)
            return x, y, None
        x = E.SparseTensor(feats, coords)
        y = conv(x)
        kmap = x.coordinate_manager.kernel_map(x.coordinate_map_key, y.coordinate_map_key, [KSIZE] * 3, [1] * 3,
                                               [1] * 3)
        kmap.pairs()
        return x, y, kmap

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            x, y, kmap = step()
        n_unique = len(x)
        table0 = ops.table_build(coords)
        total_pairs = int(ops.kmap_build(table0, table0.coords, offsets).pairs()[0][-1])
        del table0

        # ---- headline: K steps, device-resident inputs, CUDA events on the launching stream ----
        barrier()
        sampler = ClockSampler(local_rank) if rank == 0 else None
        launches0 = lib.rmn_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        launches = lib.rmn_launch_count() - launches0
        elapsed_ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if sampler else None

        # ---- per-phase timings ------------------------------------------------------------------
        # The phases of one step run back to back on the stream, as in the step itself, with an
        # event between them and no host synchronisation (every buffer is allocated beforehand);
        # the median over the repetitions is reported. The general kernel-map builder, which the
        # step does not use (its stride-1 layer takes the self-map builder), is timed at the end
        # of each repetition.
        table = ops.table_build(coords)
        res = ops.kmap_build(table, table.coords, offsets)
        res_self = ops.kmap_build(table, table.coords, offsets, self_map=True)
        assert torch.equal(res.nbr, res_self.nbr) and torch.equal(res.offset_ptr, res_self.offset_ptr)
        n_rows = int(coords.size(0))
        tbytes, wbytes = lib.rmn_table_bytes(n_rows), lib.rmn_table_build_workspace_bytes(n_rows)
        t_buf = torch.empty(tbytes, dtype=torch.uint8, device=dev)
        t_map = torch.empty(n_rows, dtype=torch.int64, device=dev)
        t_uniq = torch.empty((n_rows, 4), dtype=torch.int32, device=dev)
        t_ws = torch.empty(wbytes, dtype=torch.uint8, device=dev)
        cap = (torch.empty(total_pairs, dtype=torch.int32, device=dev),
               torch.empty(total_pairs, dtype=torch.int32, device=dev))
        xf = x.F
        P = ops._ptr

        def ph_hash():
            capi.check(lib.rmn_table_build(P(coords), n_rows, 4, P(t_buf), tbytes, P(t_map), None, P(t_uniq),
                                           P(t_ws), wbytes, ops._stream()), "rmn_table_build")

        def ph_pairs():
            capi.check(lib.rmn_kmap_pairs(P(res.nbr), res.n_query, res.K, P(res.offset_ptr), P(res.workspace),
                                          P(cap[0]), P(cap[1]), total_pairs, ops._stream()), "rmn_kmap_pairs")

        phase_fns = [ph_hash,
                     lambda: ops.kmap_build(table, table.coords, offsets, self_map=True),
                     ph_pairs,
                     lambda: ops.conv_forward(xf, conv.kernel, res.nbr),
                     lambda: ops.kmap_build(table, table.coords, offsets)]
        reps = max(5, min(args.steps, 20))
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(phase_fns) + 1)] for _ in range(reps + 2)]
        for rep in marks:
            rep[0].record()
            for i, fn in enumerate(phase_fns):
                fn()
                rep[i + 1].record()
        torch.cuda.synchronize()
        med = [statistics.median(rep[i].elapsed_time(rep[i + 1]) for rep in marks[2:]) for i in range(len(phase_fns))]
        t_hash, t_kmap, t_pairs, t_fwd, t_kmap_general = med

        # ---- side measurement: the workload's second layer, 2^3 stride-2 64 -> 128 -----------------
        # hash insert + strided coordinate map + kernel map (general builder, K = 8) + forward on a fresh manager
        down = E.RiemannConvolution(C_IN, 128, kernel_size=2, stride=2, dimension=3).to(dev).bfloat16()
        cdown = None
        if cpp_host is not None:
            cdown = cpp_host.RiemannConvolution(C_IN, 128, kernel_size=2, stride=2, dimension=3)
            cdown.to(f"cuda:{local_rank}")
            cdown.to(torch.bfloat16)

        def down_step():
            if cdown is not None:
                return cdown(cpp_host.SparseTensor(feats, coords))
            return down(E.SparseTensor(feats, coords))

        for _ in range(3):
            yd = down_step()
        n_down = len(yd)
        torch.cuda.synchronize()
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(args.steps):
            down_step()
        d1.record()
        torch.cuda.synchronize()
        down_ms = d0.elapsed_time(d1) / args.steps

        # ---- end to end through the public API with HOST buffers ----------------------------------
        h_coords = torch.from_numpy(coords_np).pin_memory()
        h_feats = torch.from_numpy(feats_np).bfloat16().pin_memory()
        h_out = torch.empty((n_unique, C_OUT), dtype=torch.bfloat16).pin_memory()

        def e2e_step():
            dc = h_coords.to(dev, non_blocking=True)
            df = h_feats.to(dev, non_blocking=True)
            yy = step(df, dc)[1]            # the same step as the headline's, pair lists included
            h_out.copy_(yy.F, non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.steps):
            e2e_step()
        f1.record()
        barrier()
        e2e_serial_ms = f0.elapsed_time(f1)

        # The same per-step work as an input pipeline: the host-to-device copy of step i+1 and the
        # device-to-host copy of step i-1 run on their own streams while step i computes (PCIe is
        # full duplex). Every step still copies its own inputs in and its own result out.
        s_main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        d_coords = [torch.empty_like(coords) for _ in range(2)]
        d_feats = [torch.empty_like(feats) for _ in range(2)]
        h_outs = [torch.empty((n_unique, C_OUT), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_used = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_used[b])          # the compute that last read this buffer pair
                d_coords[b].copy_(h_coords, non_blocking=True)
                d_feats[b].copy_(h_feats, non_blocking=True)
                ev_in[b].record(s_in)

        def run_pipelined(n_steps):
            prefetch(0)
            for i in range(n_steps):
                b = i % 2
                if i + 1 < n_steps:
                    prefetch(i + 1)
                s_main.wait_event(ev_in[b])
                yy = step(d_feats[b], d_coords[b])[1]
                ev_used[b].record(s_main)
                out_f = yy.F
                out_f.record_stream(s_out)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_used[b])
                    s_out.wait_event(ev_out[b])      # previous read-back into this host buffer
                    h_outs[b].copy_(out_f, non_blocking=True)
                    ev_out[b].record(s_out)
            s_main.wait_stream(s_out)
            s_main.wait_stream(s_in)

        # raw copy rates of this rank's page-locked buffers, all ranks copying at the same time
        barrier()
        c0, c1, c2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        c0.record()
        for _ in range(3):
            d_feats[0].copy_(h_feats, non_blocking=True)
        c1.record()
        for _ in range(3):
            h_outs[0].copy_(d_feats[0][:n_unique], non_blocking=True)
        c2.record()
        barrier()
        h2d_gbs = 3 * h_feats.numel() * 2 / (c0.elapsed_time(c1) / 1e3) / 1e9
        d2h_gbs = 3 * h_outs[0].numel() * 2 / (c1.elapsed_time(c2) / 1e3) / 1e9

        run_pipelined(3)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        run_pipelined(args.steps)
        g1.record()
        barrier()
        e2e_ms = g0.elapsed_time(g1)

        # ---- convolution plan: build time and the planned (cached-map) forward ---------------------
        plan_marks = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(reps + 2)]
        plan = ops.conv_plan_build(res.nbr, offsets)
        for rep in plan_marks:
            rep[0].record()
            ops.conv_plan_build(res.nbr, offsets)
            rep[1].record()
            ops.conv_forward(xf, conv.kernel, res.nbr, plan=plan)
            rep[2].record()
        torch.cuda.synchronize()
        t_plan = statistics.median(rep[0].elapsed_time(rep[1]) for rep in plan_marks[2:])
        t_fwd_planned = statistics.median(rep[1].elapsed_time(rep[2]) for rep in plan_marks[2:])
        assert torch.equal(ops.conv_forward(xf, conv.kernel, res.nbr, plan=plan), ops.conv_forward(xf, conv.kernel, res.nbr))
        # fraction of (512-row super-tile, offset) stages the planned kernel skips
        n_pos = (n_unique + 511) // 512 * 512
        tile_masks = plan[256 + ((n_pos * 4 + 255) & ~255):][:n_pos // 128 * 4].view(torch.int32).view(-1, 4)
        st_mask = tile_masks[:, 0] | tile_masks[:, 1] | tile_masks[:, 2] | tile_masks[:, 3]
        stages_run = int(sum(int(((st_mask >> k) & 1).sum()) for k in range(K_VOL)))
        stage_fraction = stages_run / float(st_mask.numel() * K_VOL)

    extras = run_extras(args, cpp_host, dev, rank, world, coords, feats, weights_np, res, xf, conv) \
        if cpp_host is not None and not args.no_extras else {}

    # ---- per-rank host-link figures (gathered to rank 0) ------------------------------------------
    link = torch.tensor([h2d_gbs, d2h_gbs, float(numa["numa_node"] if numa["numa_node"] is not None else -2)],
                        dtype=torch.float64, device=dev)
    links = [torch.zeros_like(link) for _ in range(world)] if world > 1 else [link]
    if world > 1:
        dist.all_gather(links, link)
    per_rank_link = [{"rank": r, "h2d_gbs": round(float(t[0]), 1), "d2h_gbs": round(float(t[1]), 1),
                      "gpu_numa_node": int(t[2])} for r, t in enumerate(links)]

    # ---- max over ranks ------------------------------------------------------------------------
    stats = torch.tensor([elapsed_ms, e2e_ms, float(n_vox), e2e_serial_ms], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        elapsed_ms, e2e_ms, total_vox, e2e_serial_ms = float(mx[0]), float(mx[1]), float(sm[2]), float(mx[3])
    else:
        total_vox = float(n_vox)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    value = total_vox * args.steps / (elapsed_ms / 1e3) / 1e6
    e2e_value = total_vox * args.steps / (e2e_ms / 1e3) / 1e6
    W = 4
    flops = 2.0 * total_pairs * C_IN * C_OUT
    bytes_hash = n_vox * (4 * W + 32)
    bytes_kmap = n_unique * 4 * W + n_unique * K_VOL * 32 + 8 * total_pairs
    phases = {"hash_insert_ms": t_hash, "kmap_probe_ms": t_kmap, "kmap_probe_general_ms": t_kmap_general,
              "kmap_pairs_ms": t_pairs, "conv_fwd_ms": t_fwd, "conv_plan_build_ms": t_plan,
              "conv_fwd_planned_ms": t_fwd_planned}
    planned_tflops = flops / (t_fwd_planned / 1e3) / 1e12
    fwd_tflops = flops / (t_fwd / 1e3) / 1e12
    kmap_gbs = bytes_kmap / ((t_kmap + t_pairs) / 1e3) / 1e9
    hash_gbs = bytes_hash / (t_hash / 1e3) / 1e9
    if t_fwd >= t_kmap + t_pairs:
        roofline = {"kernel": "conv_forward", "bound": "tensor", "achieved": fwd_tflops,
                    "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": fwd_tflops / peaks["bf16_tflops"],
                    "traffic": captured_traffic("conv_forward"), "peak_source": peaks["source"],
                    "algorithmic": f"2*P*Cin*Cout = {flops:.3e} flop per launch"}
    else:
        roofline = {"kernel": "kmap_probe+pairs", "bound": "hbm", "achieved": kmap_gbs, "peak": peaks["hbm_gbs"],
                    "unit": "GB/s", "frac": kmap_gbs / peaks["hbm_gbs"],
                    "traffic": captured_traffic("kmap_probe_self", "kmap_pairs"),
                    "peak_source": peaks["source"],
                    "algorithmic": f"N*4W + N*K*32 + 8P = {bytes_kmap:.3e} B per launch"}

    coords_s, feats_s, weights_s = cpu_sample()
    cpu_s, cpu_vox, info = cpu_reference_time(coords_s, feats_s, weights_s, steps=3, warmup=1)
    cpu_value = cpu_vox * 3 / cpu_s / 1e6

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "host_layer": "riemann_cpp (C++/LibTorch)" if cpp_host is not None else "python",
        "voxels_per_step": total_vox, "pairs_per_gpu": total_pairs,
        "phases_ms": phases,
        "kernel_map_build_ms": t_kmap + t_pairs,
        "fwd_cached_mvoxels_per_s": n_vox / (t_fwd / 1e3) / 1e6,
        "roofline": roofline,
        "roofline_all": {
            "hash_insert": {"bound": "hbm", "achieved": hash_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": hash_gbs / peaks["hbm_gbs"],
                            "traffic": captured_traffic("table_fill_range", "table_insert", "table_finalize")},
            "kernel_map": {"bound": "hbm", "achieved": kmap_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                           "frac": kmap_gbs / peaks["hbm_gbs"], "builder": "self-map (half the probes)",
                           # the same time against the bytes of the probes this builder actually issues
                           # (K/2 probes per row, the mirror entries come from 4-byte stores): the
                           # algorithmic figure above charges all K probes of 32 bytes each
                           "achieved_on_probes_issued": (n_unique * 4 * W + n_unique * (K_VOL // 2) * 32 + 8 * total_pairs)
                           / ((t_kmap + t_pairs) / 1e3) / 1e9,
                           "frac_on_probes_issued": (n_unique * 4 * W + n_unique * (K_VOL // 2) * 32 + 8 * total_pairs)
                           / ((t_kmap + t_pairs) / 1e3) / 1e9 / peaks["hbm_gbs"],
                           # compulsory bytes only (query rows in, pairs out): probes served by L2 do not count
                           "achieved_compulsory": (n_unique * 4 * W + 8 * total_pairs) / ((t_kmap + t_pairs) / 1e3) / 1e9,
                           "traffic": captured_traffic("kmap_probe_self", "kmap_pairs")},
            "kernel_map_general": {"bound": "hbm", "achieved": bytes_kmap / ((t_kmap_general + t_pairs) / 1e3) / 1e9,
                                   "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                   "frac": bytes_kmap / ((t_kmap_general + t_pairs) / 1e3) / 1e9 / peaks["hbm_gbs"]},
            "hash_and_kernel_map": {"bound": "hbm", "unit": "GB/s", "peak": peaks["hbm_gbs"],
                                    "achieved": (bytes_hash + bytes_kmap) / ((t_hash + t_kmap + t_pairs) / 1e3) / 1e9,
                                    "frac": (bytes_hash + bytes_kmap) / ((t_hash + t_kmap + t_pairs) / 1e3) / 1e9
                                    / peaks["hbm_gbs"]},
            "conv_forward": {"bound": "tensor", "achieved": fwd_tflops, "peak": peaks["bf16_tflops"],
                             "unit": "TFLOP/s", "frac": fwd_tflops / peaks["bf16_tflops"],
                             "note": "first use of a kernel map (what the timed step runs): no plan"},
            # the same layer on a map that has a convolution plan (second and later layers on a map, the
            # input-gradient pass): offsets at which no row of a 512-row super-tile has a neighbour are skipped
            "conv_forward_planned": {"bound": "tensor", "achieved": planned_tflops, "peak": peaks["bf16_tflops"],
                                     "unit": "TFLOP/s", "frac": planned_tflops / peaks["bf16_tflops"],
                                     "traffic": captured_traffic("conv_forward_planned"),
                                     "stages_run_fraction": stage_fraction,
                                     # MMAs issued (zero rows included) against the measured peak
                                     "executed_frac": (2.0 * stages_run * 512 * C_IN * C_OUT)
                                     / (t_fwd_planned / 1e3) / 1e12 / peaks["bf16_tflops"],
                                     "plan_build_ms": t_plan},
        },
        "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": info["cores"], "kind": info["kind"],
                         "sample": f"all {CPU_SAMPLE_SCENES} scenes of one rank's batch ({cpu_vox} voxels), fp32, "
                                   "SparseTensor construction + first forward, 3 steps after 1 warm-up",
                         **{k: v for k, v in info.items() if k not in ("cores", "kind")}},
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps,
                "pipelined": "H2D of step i+1 and D2H of step i-1 overlap the compute of step i (3 streams)",
                "serial_value": total_vox * args.steps / (e2e_serial_ms / 1e3) / 1e6,
                "serial_ms_per_step": e2e_serial_ms / args.steps,
                "h2d_bytes_per_step": int(h_coords.numel() * 4 + h_feats.numel() * 2),
                "d2h_bytes_per_step": int(h_out.numel() * 2),
                # each rank is pinned to the CPUs of its GPU's NUMA node before it allocates its page-locked
                # buffers; raw copy rates with all ranks copying at once
                "host_link_per_rank": per_rank_link, "numa_binding": numa},
        "gpu_launches": int(launches),
        "clocks": clocks,
        **extras,
        "strided_layer": {"layer": "2x2x2 stride-2 conv 64->128 on the same batch (hash insert + strided map + "
                                   "kernel map + forward, fresh manager)", "ms_per_step": down_ms,
                          "mvoxels_per_s": n_vox / (down_ms / 1e3) / 1e6, "output_voxels_per_gpu": int(n_down),
                          "note": "this rank only; not part of `value`"},
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# training step (side measurement, not the headline): hash + kernel map + forward + backward
# (input and weight gradients) + all-reduce of the weight gradients over the ranks
# ------------------------------------------------------------------------------------------
def run_train(args) -> None:
    import torch
    import torch.distributed as dist

    from riemannengine_b200 import capi, distributed as D, engine as E

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        with stdout_to_stderr():  # NCCL's version banner goes to stdout; stdout carries the JSON line only
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
    lib = capi.lib()
    coords_np, feats_np, weights_np = make_batch(rank)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(feats_np).to(dev).bfloat16().requires_grad_(True)
    conv = E.RiemannConvolution(C_IN, C_OUT, kernel_size=KSIZE, dimension=3).to(dev).bfloat16()
    with torch.no_grad():
        conv.kernel.copy_(torch.from_numpy(weights_np).to(dev))

    # a fixed upstream gradient stands in for the rest of the network (no loss kernels in the step)
    grad_out = torch.randn(len(coords_np), C_OUT, device=dev).bfloat16()

    def step():
        conv.zero_grad(set_to_none=True)
        feats.grad = None
        y = conv(E.SparseTensor(feats, coords))
        y.F.backward(grad_out)
        D.allreduce_gradients(conv.parameters(), average=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    l0 = lib.rmn_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    stats = torch.tensor([e0.elapsed_time(e1), float(len(coords_np))], dtype=torch.float64, device=dev)
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, vox = float(mx[0]), float(sm[1])
    else:
        ms, vox = float(stats[0]), float(stats[1])
    if rank == 0:
        print(json.dumps({
            "metric": "sparse_conv_fwd_bwd_mvoxels_per_s", "value": vox * args.steps / (ms / 1e3) / 1e6, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(world), workload="indoor-room batch, 3^3 64->64: hash insert + kernel map + "
                           "forward + backward (dX, dW) + weight-gradient all-reduce"),
            "gpu_launches": int(lib.rmn_launch_count() - l0)}))
    if world > 1:
        dist.destroy_process_group()


def run_kernels(args) -> None:
    """One pass over the kernels of the headline workload (for profilers: `ncu -k regex:<kernel> ...
    python bench.py --mode kernels`): table build, both kernel-map builders, pair lists, plan build, forward
    (plain and planned), input gradient, weight gradient - `--steps` times each after one warm-up, no timing."""
    import torch

    from riemannengine_b200 import capi, ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    coords_np, feats_np, weights_np = make_batch(0)
    coords = torch.from_numpy(coords_np).to(dev)
    feats = torch.from_numpy(feats_np).to(dev).bfloat16()
    w = torch.from_numpy(weights_np).to(dev).bfloat16()
    offsets = ops.region_offsets(capi.HYPER_CUBE, [KSIZE] * 3, [1] * 3, [1] * 3)
    gy = torch.randn(len(coords_np), C_OUT, device=dev).bfloat16()
    for _ in range(1 + max(args.steps, 1)):
        table = ops.table_build(coords)
        res = ops.kmap_build(table, table.coords, offsets, self_map=True)
        ops.kmap_build(table, table.coords, offsets)
        res.pairs()
        plan = ops.conv_plan_build(res.nbr, offsets)
        ops.conv_forward(feats, w, res.nbr)
        ops.conv_forward(feats, w, res.nbr, plan=plan)
        ops.conv_backward_input(gy, w.flip(0), res.nbr, plan=plan)
        ops.conv_backward_weight(feats, gy, res.nbr)
    torch.cuda.synchronize()
    print(json.dumps({"mode": "kernels", "voxels": len(coords_np), "passes": 1 + max(args.steps, 1)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="fwd", choices=["fwd", "train", "kernels"],
                    help="fwd: the headline forward metric; train: forward + backward + gradient all-reduce "
                         "(Python host layer); kernels: one untimed pass over every kernel, for profilers")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the training step and the other configurations (headline line only)")
    ap.add_argument("--host", default="auto", choices=["auto", "cpp", "py"],
                    help="host layer driving the step: the C++/LibTorch riemann_cpp module or the Python mirror")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.mode == "train":
        run_train(args)
    elif args.mode == "kernels":
        run_kernels(args)
    else:
        run_product(args)


if __name__ == "__main__":
    main()
