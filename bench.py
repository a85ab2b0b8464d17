"""Benchmark of the image-transform-and-batch path.

    python bench.py --gpus N --steps K --warmup W [--workload c5] [--impl reference]

One step = one batch of the named workload per GPU through the fused kernel
(resize / crop / flip / rotate -> batch + pad -> float32 cast).  The default arm
times this package: `value` with sources and batches resident in HBM, `e2e`
through the same public pipeline API with host samples in page-locked memory
and host batches out.  `--impl reference` times the reference's own CPU
pipeline (the build under oracle/_ref) on the host cores.  Rank 0 prints one
JSON line.
"""
import argparse
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one fused_fast_kernel launch per
# image of the workload, from an ncu capture of a 128-image launch (845.0 MB);
# the traffic of this kernel grows in proportion to the image count.
NCU_DRAM_BYTES_PER_IMAGE = {"c5": 845.0e6 / 128}


def load_package():
    if "mlx_data_b200" in sys.modules:
        return sys.modules["mlx_data_b200"]
    pkg_dir = os.path.join(ROOT, "mlx-data_b200")
    spec = importlib.util.spec_from_file_location(
        "mlx_data_b200", os.path.join(pkg_dir, "__init__.py"), submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["mlx_data_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def load_workloads():
    pkg_dir = os.path.join(ROOT, "mlx-data_b200")
    spec = importlib.util.spec_from_file_location("mlxd_workloads", os.path.join(pkg_dir, "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
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
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cast_kwargs(cast):
    if len(cast) == 0:
        return {}
    return {"mean": list(cast[0]), "std": list(cast[1])}


def build_pipeline(dx, samples, ops, batch, cast, native=True, prefetch=None):
    """The fluent chain as a user writes it.  `native` uses this package's fused
    cast (key_cast); otherwise the cast is the reference's numpy lambda."""
    ds = dx.buffer_from_vector(samples)
    for name, kw in ops:
        kw = dict(kw)
        if "angle_key" in kw:
            kw.setdefault("angle", 0.0)
        ds = getattr(ds, name)(**kw)
    ds = ds.batch(batch)
    if native:
        ds = ds.key_cast("image", **cast_kwargs(cast))
    else:
        if len(cast) == 0:
            ds = ds.key_transform("image", lambda x: x.astype("float32") / 255)
        else:
            mean = np.array(cast[0], dtype=np.float32)
            std = np.array(cast[1], dtype=np.float32)
            ds = ds.key_transform("image", lambda x: (x.astype("float32") / 255 - mean) / std)
    if prefetch:
        ds = ds.ordered_prefetch(*prefetch)
    return ds


def pool_shapes(wl, name, count):
    _, hs, ws = wl.image_sizes(name, "full", n=count)
    return [(int(h), int(w)) for h, w in zip(hs, ws)]


def sample_list(pool, extra, first_batch, n_batches, batch, world, rank):
    """Samples of the batches this rank owns: batch j of the global sequence
    belongs to rank j % world (sharding by sample index in whole batches)."""
    out = []
    for s in range(n_batches):
        j = (first_batch + s) * world + rank
        for i in range(batch):
            g = j * batch + i
            d = {"image": pool[g % len(pool)]}
            if extra is not None:
                d["angle"] = extra[g % len(extra)]
            out.append(d)
    return out


def reference_module():
    ref = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref, "mlx", "data")):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import mlx.data as dx
        return dx
    except Exception:
        return None


def cpu_pipeline_rate(wl, name, n_images, threads, repeats=1):
    """images/s of the reference CPU pipeline (oracle/_ref; the C restatement
    when that build is absent) on a bounded sample of the workload."""
    cfg = wl.CONFIGS[name]
    # the reference parallelises across batches (one prefetch worker builds a
    # whole batch), so the bounded sample uses batches small enough to keep
    # every worker busy
    batch = min(cfg["full"]["batch"], max(1, n_images // (2 * threads)))
    pool_n = min(n_images, 64)
    shapes = pool_shapes(wl, name, pool_n)
    rng = np.random.default_rng(7)
    pool = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for h, w in shapes]
    ops = wl.config_ops(name, "full")
    per_sample_angle = any("angle_key" in kw for _, kw in ops)
    dx = reference_module()
    if dx is not None:
        angles = np.random.default_rng(8).uniform(-30, 30, 16)
        samples = [{"image": pool[i % pool_n]} for i in range(n_images)]
        if per_sample_angle:
            # the reference op takes one angle per op instance: use a fixed one for timing
            ops = [(n, ({k: v for k, v in kw.items() if k != "angle_key"} | {"angle": float(angles[0])})
                    if "angle_key" in kw else kw) for n, kw in ops]
        best = 0.0
        for _ in range(repeats):
            dx.core.set_state(0)
            ds = build_pipeline(dx, samples, ops, batch, cfg["cast"], native=False)
            stream = ds.ordered_prefetch(threads, threads)
            t0 = time.perf_counter()
            n = 0
            for b in stream:
                n += b["image"].shape[0]
            dt = time.perf_counter() - t0
            best = max(best, n / dt)
        return best, "reference", threads, "%d images, batch %d, prefetch(%d,%d), numpy cast" % (
            n_images, batch, threads, threads)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    samples = [{"image": pool[i % pool_n], "angle": np.float64(3.0)} for i in range(n_images)]
    O.set_state(0)
    cast = {"image": None if len(cfg["cast"]) == 0 else (np.array(cfg["cast"][0], np.float32),
                                                         np.array(cfg["cast"][1], np.float32))}
    t0 = time.perf_counter()
    O.run_chain(samples, ops, batch, {"image": 0.0}, cast)
    dt = time.perf_counter() - t0
    return n_images / dt, "port", 1, "%d images, batch %d, single thread" % (n_images, batch)


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    cfg = wl.CONFIGS[name]
    threads = os.cpu_count() or 1
    per_step = args.cpu_images
    rates = []
    kind = cores = sample = None
    for s in range(args.warmup + args.steps):
        r, kind, cores, sample = cpu_pipeline_rate(wl, name, per_step, threads)
        if s >= args.warmup:
            rates.append(r)
    value = float(np.mean(rates))
    line = {
        "impl": "reference", "metric": "images_per_sec", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * per_step / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "images_per_step": per_step, "batch": cfg["full"]["batch"],
                   "note": "reference CPU pipeline on host cores; resize is the CPU restatement of the un-vendored stb routine"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--pool", type=int, default=0, help="distinct source images per GPU (0: workload default)")
    ap.add_argument("--batch", type=int, default=0,
                    help="images per step per GPU (0: the workload's batch size; smaller values are for profiling)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end leg (0: min(steps, 6))")
    ap.add_argument("--cpu-images", type=int, default=0, help="images per CPU-baseline run (0: workload default)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg")
    args = ap.parse_args()
    wl = load_workloads()
    name = args.workload
    cfg = wl.CONFIGS[name]
    if args.cpu_images == 0:
        args.cpu_images = {"c1": 2048, "c2": 1024, "c3": 128, "c4": 1024, "c5": 384}[name]
    if args.impl == "reference":
        return run_reference_arm(args, wl)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dx = load_package()
    dx.core.set_device(local)

    batch = args.batch or cfg["full"]["batch"]
    K, W = args.steps, max(args.warmup, 3)
    pool_n = args.pool or {"c1": 2048, "c2": 4096, "c3": 2048, "c4": 4096, "c5": 512}[name]
    shapes = pool_shapes(wl, name, pool_n)
    ops = wl.config_ops(name, "full")
    extra = None
    if name == "c4":
        extra = [np.float64(a) for a in np.random.default_rng(1000).uniform(-30.0, 30.0, 4096)]

    # ---------------- leg 1: sources and batches resident in HBM ----------------
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)
    pool = [torch.randint(0, 256, (h, w, 3), dtype=torch.uint8, device="cuda", generator=gen) for h, w in shapes]
    pool_bytes = sum(h * w * 3 for h, w in shapes)
    dx.core.set_state(rank)
    dx.core.set_device_output(True)
    dx.core.set_stream(torch.cuda.current_stream().cuda_stream, True)
    dx.core.set_timing(True)
    samples = sample_list(pool, extra, 0, W + K, batch, world, rank)
    pipe = build_pipeline(dx, samples, ops, batch, cfg["cast"], native=True)
    out = None
    for s in range(W):
        out = pipe[s]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    st0 = dx.core.stats()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0 = torch.cuda.Event(enable_timing=True)
    ev1 = torch.cuda.Event(enable_timing=True)
    ev0.record()
    for s in range(K):
        out = pipe[W + s]
    ev1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    st1 = dx.core.stats()
    out_shape = tuple(out["image"].shape)
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = world * K * batch / (ms_max / 1000.0)

    launches = st1["kernel_launches"] - st0["kernel_launches"]
    timed = max(1, st1["timed_launches"] - st0["timed_launches"])
    kernel_ms = (st1["kernel_ns"] - st0["kernel_ns"]) / 1e6 / timed
    algo_per_launch = ((st1["algo_src_bytes"] - st0["algo_src_bytes"]) +
                       (st1["algo_dst_bytes"] - st0["algo_dst_bytes"])) / max(1, launches)
    peak, peak_kind = measured_peak_gbs()
    achieved = algo_per_launch / (kernel_ms / 1000.0) / 1e9 if kernel_ms > 0 else 0.0

    # release the device leg before the host-fed one
    del pipe, samples, out
    dx.core.set_stream(0, False)
    dx.core.set_device_output(False)
    dx.core.set_timing(False)

    # ---------------- leg 2: end to end, host samples in, host batches out ----------------
    e2e = None
    if not args.no_e2e:
        Ke = args.e2e_steps or max(8, min(2 * K, 24))
        We = 1
        host_n = min(pool_n, {"c1": 2048, "c2": 1024, "c3": 512, "c4": 1024, "c5": 256}[name])
        rng = np.random.default_rng(99 + rank)
        host_pool = []
        for h, w in shapes[:host_n]:
            a = dx.core.pinned_empty([h, w, 3], "uint8")
            a[...] = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
            host_pool.append(a)
        lanes = int(os.environ.get("MLXD_BENCH_LANES", "4"))
        # Warm-up on a pipeline of its own, fully consumed.  Page-locked batch
        # buffers are expensive to allocate (about half a second per GB) and are
        # recycled afterwards; 2 * lanes + 2 batches bring the pool to the number
        # of buffers the steady state keeps alive (look-ahead ring + consumer).
        hw = build_pipeline(dx, sample_list(host_pool, extra, 0, 2 * lanes + 2, batch, world, rank), ops, batch,
                            cfg["cast"], native=True, prefetch=(lanes, lanes))
        held = None
        for b in hw:
            held = b
        del hw, held, b
        hs = sample_list(host_pool, extra, We, Ke, batch, world, rank)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s0 = dx.core.stats()
        # The timed region starts before the pipeline exists, so every copy and
        # launch of the Ke batches it delivers lies inside it (no look-ahead
        # work from before the clock started).
        t0 = time.perf_counter()
        hp = build_pipeline(dx, hs, ops, batch, cfg["cast"], native=True, prefetch=(lanes, lanes))
        n_img = 0
        checksum = 0.0
        for b in hp:
            n_img += b["image"].shape[0]
            checksum += float(b["image"][0, 0, 0, 0])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        s1 = dx.core.stats()
        t = torch.tensor([dt], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_max = float(t.item())
        # look-ahead batches count towards the copies but not the images: report bytes per delivered step
        steps_copied = max(1, s1["batches"] - s0["batches"])
        e2e = {"value": world * n_img / dt_max, "unit": "images/s",
               "h2d_bytes_per_step": int((s1["h2d_bytes"] - s0["h2d_bytes"]) / steps_copied),
               "d2h_bytes_per_step": int((s1["d2h_bytes"] - s0["d2h_bytes"]) / steps_copied),
               "steps": Ke, "host_threads": lanes, "host_memory": "page-locked"}
        del hp, hs, host_pool

    # ---------------- leg 3: the reference CPU pipeline on this host ----------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        r, kind, cores, sample = cpu_pipeline_rate(wl, name, args.cpu_images, threads)
        cpu = {"value": r, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample}

    if rank == 0:
        line = {
            "metric": "images_per_sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "ops": [n for n, _ in ops], "batch_per_gpu": batch,
                       "global_batch": batch * world, "output": list(out_shape),
                       "source_pool_images_per_gpu": pool_n, "source_pool_bytes_per_gpu": pool_bytes,
                       "l2": "inputs larger than L2: each step reads %d distinct sources and writes a fresh batch" % batch,
                       "sharding": "whole batches by index, batch j on rank j % n_gpus, no collective"},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS,
                         "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": algo_per_launch,
                         "traffic": (NCU_DRAM_BYTES_PER_IMAGE[name] * batch if name in NCU_DRAM_BYTES_PER_IMAGE else None),
                         "traffic_kind": "ncu dram bytes of a 128-image launch scaled by the image count"},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
