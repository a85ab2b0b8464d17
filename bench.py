"""Benchmark of the image-transform-and-batch path.

    python bench.py --gpus N --steps K --warmup W [--workload c5] [--impl reference]

One step = one batch of the named workload per GPU through the fused kernel
(resize / crop / flip / rotate -> batch + pad -> float32 cast).  The default arm
times this package: `value` with sources and batches resident in HBM (the K
steps are repeated until the timed region is about a second long), `e2e`
through the same public pipeline API with host samples in page-locked memory
and host batches out, with the same pipeline on ordinary numpy samples
(`e2e.pageable`) and with batches left in HBM (`e2e.device_output`) beside it.
Before the line is printed one full-size batch is compared with the CPU oracle
and the kernels' self-check word is read (`checked`).  `--impl reference`
times the reference's own CPU pipeline (the build under oracle/_ref) on the
host cores, at the workload's batch size.  Rank 0 prints one JSON line.
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
# image of the workload, from an ncu capture of a 128-image launch (852.6 MB);
# the traffic of this kernel grows in proportion to the image count.
NCU_DRAM_BYTES_PER_IMAGE = {"c5": 852.6e6 / 128}


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


def jpeg_fed_rate(dx, shapes, ops, batch, cast, lanes):
    """The chain fed from JPEG files held in memory: load_image (this package's
    decoder, one file per worker thread at a time) -> image ops -> batch -> cast,
    host float32 batches out.  Files: photographs are smooth, so the synthetic
    ones are coarse random colour fields with mild noise, 4:2:0, quality 90."""
    import io
    import torch
    from PIL import Image
    rng = np.random.default_rng(7)
    files = []
    for h, w in shapes[:16]:
        coarse = rng.integers(0, 256, (h // 16 + 2, w // 16 + 2, 3)).astype(np.float32)
        img = np.kron(coarse, np.ones((16, 16, 1), np.float32))[:h, :w] + rng.normal(0, 6, (h, w, 3))
        buf = io.BytesIO()
        Image.fromarray(np.clip(img, 0, 255).astype(np.uint8)).save(buf, format="JPEG", quality=90, subsampling=2)
        files.append(np.frombuffer(buf.getvalue(), dtype=np.uint8))
    threads = len(os.sched_getaffinity(0))
    n_batches = max(3, (1024 + batch - 1) // batch)
    samples = [{"image": files[i % len(files)]} for i in range(batch * n_batches)]

    def pipeline(some):
        ds = dx.buffer_from_vector(some).to_stream().load_image("image", from_memory=True).prefetch(threads, threads)
        for name, kw in ops:
            ds = getattr(ds, name)(**dict(kw))
        return ds.batch(batch).key_cast("image", **cast_kwargs(cast)).prefetch(lanes, lanes)

    for _ in pipeline(samples[:batch]):      # warm-up: staging pools, decoder code
        pass
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_img = 0
    for bb in pipeline(samples):
        n_img += bb["image"].shape[0]
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    return {"value": n_img / dt, "unit": "images/s", "decode_threads": threads, "images": n_img,
            "mean_file_bytes": int(np.mean([f.size for f in files])),
            "decoder": "this package's (pixel-equal to libjpeg-turbo's defaults)"}


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


def reference_full_batch_rate(wl, name, threads, n_batches):
    """images/s of the reference CPU pipeline at the workload's own batch size:
    n_batches batches from a shared pool of sources, prefetch(threads, threads)."""
    cfg = wl.CONFIGS[name]
    batch = cfg["full"]["batch"]
    dx = reference_module()
    if dx is None:
        return None
    pool_n = 64
    shapes = pool_shapes(wl, name, pool_n)
    rng = np.random.default_rng(7)
    pool = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for h, w in shapes]
    ops = wl.config_ops(name, "full")
    if any("angle_key" in kw for _, kw in ops):
        ops = [(n, ({k: v for k, v in kw.items() if k != "angle_key"} | {"angle": 17.0}) if "angle_key" in kw else kw)
               for n, kw in ops]
    samples = [{"image": pool[i % pool_n]} for i in range(batch * n_batches)]
    dx.core.set_state(0)
    ds = build_pipeline(dx, samples, ops, batch, cfg["cast"], native=False)
    stream = ds.ordered_prefetch(threads, threads)
    t0 = time.perf_counter()
    n = 0
    for b in stream:
        n += b["image"].shape[0]
    return n / (time.perf_counter() - t0)


def prefetch_threads_that_fit(wl, name, threads):
    """The reference keeps `threads` finished batches in flight; cap that by the host's free memory."""
    cfg = wl.CONFIGS[name]
    out_shape = {"c1": 224 * 224, "c2": 224 * 224, "c3": 2048 * 2048, "c4": 448 * 448, "c5": 512 * 512}[name]
    batch_bytes = cfg["full"]["batch"] * out_shape * 3 * 5          # uint8 batch + float32 batch
    try:
        import psutil
        free = psutil.virtual_memory().available
    except Exception:
        free = 64 << 30
    return max(1, min(threads, int(free * 0.5 / (3 * batch_bytes))))


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload
    cfg = wl.CONFIGS[name]
    cores = os.cpu_count() or 1
    # small-batch sample: every worker busy, bounded time
    small, kind, used, sample = cpu_pipeline_rate(wl, name, args.cpu_images, cores)
    # the stated configuration: the workload's own batch size, as many batches as workers (at least K)
    threads = prefetch_threads_that_fit(wl, name, cores)
    n_batches = max(threads, min(args.steps, 2 * threads))
    full = None
    if kind == "reference":
        for _ in range(max(0, min(args.warmup, 1))):
            reference_full_batch_rate(wl, name, threads, min(threads, 4))
        full = reference_full_batch_rate(wl, name, threads, n_batches)
    value = float(full if full is not None else small)
    batch = cfg["full"]["batch"]
    line = {
        "impl": "reference", "metric": "images_per_sec", "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * batch / value, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "batch": batch, "batches_timed": n_batches if full is not None else None,
                   "prefetch_threads": threads,
                   "note": "reference CPU pipeline on host cores at the workload's batch size; its resize is the CPU "
                           "restatement of the un-vendored stb routine (resize parity unpinned, stb absent)"},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": threads if full is not None else used,
                         "kind": kind,
                         "sample": ("%d batches of %d, prefetch(%d,%d), numpy cast" % (n_batches, batch, threads, threads))
                         if full is not None else sample,
                         "small_batch_sample": {"value": small, "sample": sample}},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def check_against_oracle(dx, wl, name, pipe_samples, ops, batch, cast, n_check):
    """One full-size batch through the same pipeline with a known seed; its first
    n_check slots against the CPU oracle (checker only: nothing here is timed)."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as O
    seed = 777
    dx.core.set_state(seed)
    pipe = build_pipeline(dx, pipe_samples[:batch], ops, batch, cast, native=True)
    out = pipe[0]["image"]
    torch.cuda.synchronize()
    got = torch.as_tensor(out, device="cuda")[:n_check].cpu().numpy()
    host = []
    for smp in pipe_samples[:n_check]:
        d = {"image": smp["image"].cpu().numpy()}
        if "angle" in smp:
            d["angle"] = smp["angle"]
        host.append(d)
    O.set_state(seed)
    c = {"image": None if len(cast) == 0 else (np.array(cast[0], np.float32), np.array(cast[1], np.float32))}
    # the oracle batches only the checked samples; the batch pads to the launch's slot size
    want = O.run_chain(host, ops, n_check, {"image": 0.0}, c)[0]["image"]
    h, w = want.shape[1], want.shape[2]
    has_resize = any(n.startswith("image_resize") for n, _ in ops)
    scale = 1.0 / 255 if len(cast) == 0 else 1.0 / 255 / min(cast[1])
    d = np.abs(got[:, :h, :w].astype(np.float64) - want.astype(np.float64))
    tol = scale * 1.0001 if has_resize else 0.0
    ok = bool(d.max() <= tol and (d > 0).mean() <= 1e-3)
    status = dx.core.stream_status(torch.cuda.current_stream().cuda_stream)
    return {"slots": n_check, "max_abs_diff": float(d.max()), "tolerance": tol,
            "differing_fraction": float((d > 0).mean()), "kernel_status": int(status),
            "ok": bool(ok and status == 0)}


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
    ap.add_argument("--quick-e2e", action="store_true", help="end-to-end leg without the device-output and pageable runs")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of one batch with the CPU oracle")
    ap.add_argument("--host-affinity", default="auto", choices=["auto", "on", "off"],
                    help="keep each rank's host threads on its GPU's NUMA node (auto: when more than one rank runs)")
    ap.add_argument("--from-jpeg", action="store_true",
                    help="add e2e.from_jpeg: the chain fed from JPEG files in memory through load_image (needs Pillow to write them)")
    ap.add_argument("--repeats", type=int, default=0, help="times the K steps are repeated inside the timed region (0: about one second)")
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
    numa = None
    if args.host_affinity == "on" or (args.host_affinity == "auto" and world > 1):
        # before any worker thread or page-locked block exists
        node, cpus = dx.core.bind_host_threads_to_device_node()
        numa = {"node": node, "cpus": cpus}

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
    wa = torch.cuda.Event(enable_timing=True)
    wb = torch.cuda.Event(enable_timing=True)
    for s in range(W):
        if s == W - 1:
            wa.record()
        out = pipe[s]
    wb.record()
    torch.cuda.synchronize()
    # The K steps are timed R times back to back inside one pair of events, so that
    # the timed region lasts about a second (clock samples, launch noise); the
    # ranks agree on R.
    est_ms = max(wa.elapsed_time(wb), 1e-3)
    r_t = torch.tensor([max(1.0, min(200.0, 1000.0 / (K * est_ms)))], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(r_t, op=dist.ReduceOp.MAX)
    R = int(args.repeats or round(float(r_t.item())))
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
    for _ in range(R):
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
    value = world * K * R * batch / (ms_max / 1000.0)

    launches = st1["kernel_launches"] - st0["kernel_launches"]
    timed = max(1, st1["timed_launches"] - st0["timed_launches"])
    kernel_ms = (st1["kernel_ns"] - st0["kernel_ns"]) / 1e6 / timed
    algo_per_launch = ((st1["algo_src_bytes"] - st0["algo_src_bytes"]) +
                       (st1["algo_dst_bytes"] - st0["algo_dst_bytes"])) / max(1, launches)
    peak, peak_kind = measured_peak_gbs()
    achieved = algo_per_launch / (kernel_ms / 1000.0) / 1e9 if kernel_ms > 0 else 0.0

    # one full-size batch against the CPU oracle, and the kernels' self-check word
    checked = None
    if rank == 0 and not args.no_check:
        n_check = {"c1": 8, "c2": 8, "c3": 2, "c4": 8, "c5": 4}[name]
        checked = check_against_oracle(dx, wl, name, samples, ops, batch, cfg["cast"], min(n_check, batch))

    # release the device leg before the host-fed one
    del pipe, samples, out
    dx.core.set_stream(0, False)
    dx.core.set_device_output(False)

    # ---------------- leg 2: end to end, host samples in, host batches out ----------------
    e2e = None
    if not args.no_e2e:
        Ke = args.e2e_steps or max(8, min(2 * K, 24))
        We = 1
        host_n = min(pool_n, {"c1": 2048, "c2": 1024, "c3": 512, "c4": 1024, "c5": 256}[name])
        rng = np.random.default_rng(99 + rank)
        host_pool, plain_pool = [], []
        for h, w in shapes[:host_n]:
            a = dx.core.pinned_empty([h, w, 3], "uint8")
            a[...] = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
            host_pool.append(a)
        lanes = int(os.environ.get("MLXD_BENCH_LANES", "4"))

        def run_host_leg(src_pool, n_steps, device_output):
            """Ke batches through the pipeline API from host samples; wall clock from
            before the pipeline exists until the last batch is delivered."""
            dx.core.set_device_output(device_output)
            # Warm-up on a pipeline of its own, fully consumed.  Page-locked batch
            # buffers are expensive to allocate (about half a second per GB) and are
            # recycled afterwards; 2 * lanes + 2 batches bring the pool to the number
            # of buffers the steady state keeps alive (look-ahead ring + consumer).
            hw = build_pipeline(dx, sample_list(src_pool, extra, 0, 2 * lanes + 2, batch, world, rank), ops, batch,
                                cfg["cast"], native=True, prefetch=(lanes, lanes))
            held = None
            for bb in hw:
                held = bb
            del hw, held
            hs = sample_list(src_pool, extra, We, n_steps, batch, world, rank)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            s0 = dx.core.stats()
            # The timed region starts before the pipeline exists, so every copy and
            # launch of the batches it delivers lies inside it (no look-ahead work
            # from before the clock started).
            t0 = time.perf_counter()
            hp = build_pipeline(dx, hs, ops, batch, cfg["cast"], native=True, prefetch=(lanes, lanes))
            n_img = 0
            checksum = 0.0
            for bb in hp:
                n_img += bb["image"].shape[0]
                if not device_output:
                    checksum += float(bb["image"][0, 0, 0, 0])   # the host reads the delivered batch
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            s1 = dx.core.stats()
            tt = torch.tensor([dt], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt_max = float(tt.item())
            # look-ahead batches count towards the copies but not the images: report bytes per delivered step
            nb = max(1, s1["batches"] - s0["batches"])
            tl = max(1, s1["timed_launches"] - s0["timed_launches"])
            h2d_b = (s1["h2d_bytes"] - s0["h2d_bytes"]) / nb
            d2h_b = (s1["d2h_bytes"] - s0["d2h_bytes"]) / nb
            h2d_ms = (s1["h2d_ns"] - s0["h2d_ns"]) / 1e6 / tl
            d2h_ms = (s1["d2h_ns"] - s0["d2h_ns"]) / 1e6 / tl
            k_ms = (s1["kernel_ns"] - s0["kernel_ns"]) / 1e6 / tl
            stage_ms = (s1["host_stage_ns"] - s0["host_stage_ns"]) / 1e6 / nb
            res = {"value": world * n_img / dt_max, "unit": "images/s",
                   "h2d_bytes_per_step": int(h2d_b), "d2h_bytes_per_step": int(d2h_b), "steps": n_steps,
                   "host_threads": lanes,
                   # per batch on this rank, device time from CUDA events on the lane's stream
                   "breakdown": {"h2d_ms": h2d_ms, "h2d_gbs": h2d_b / 1e6 / h2d_ms if h2d_ms > 0 else None,
                                 "kernel_ms": k_ms, "d2h_ms": d2h_ms,
                                 "d2h_gbs": d2h_b / 1e6 / d2h_ms if d2h_ms > 0 else None,
                                 "host_pack_ms": stage_ms, "wall_ms_per_batch": 1000.0 * dt / max(1, n_steps)}}
            del hp, hs
            return res

        e2e = run_host_leg(host_pool, Ke, False)
        e2e["host_memory"] = "page-locked (core.pinned_empty)"
        e2e["host_cpus"] = len(os.sched_getaffinity(0))
        e2e["numa"] = numa
        if world > 1:
            # every rank's breakdown, for the scaling picture
            gathered = [None] * world
            dist.all_gather_object(gathered, dict(e2e["breakdown"], numa=numa, host_cpus=e2e["host_cpus"]))
            e2e["breakdown_all_ranks"] = gathered
        if not args.quick_e2e:
            # batches left in HBM: what a trainer on the same GPU consumes
            e2e["device_output"] = run_host_leg(host_pool, Ke, True)
            # ordinary numpy samples, what an unmodified user script passes in
            for a in host_pool[:min(len(host_pool), 64)]:
                plain_pool.append(np.array(a, copy=True))
            e2e["pageable"] = run_host_leg(plain_pool, max(4, Ke // 2), False)
            e2e["pageable"]["host_memory"] = "ordinary numpy arrays, packed into page-locked blocks by the calling thread"
        dx.core.set_device_output(False)
        if args.from_jpeg and world == 1:
            e2e["from_jpeg"] = jpeg_fed_rate(dx, shapes, ops, batch, cfg["cast"], lanes)
        if world > 1:
            # What the host side can move at all: every rank copies page-locked
            # blocks to and from its GPU at the same time, nothing else running.
            blk = torch.empty(256 << 20, dtype=torch.uint8).pin_memory()
            dev_blk = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
            back = torch.empty(256 << 20, dtype=torch.uint8).pin_memory()
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            reps = 8
            for _ in range(reps):
                with torch.cuda.stream(s_in):
                    dev_blk.copy_(blk, non_blocking=True)
                with torch.cuda.stream(s_out):
                    back.copy_(dev_blk, non_blocking=True)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            tt = torch.tensor([dt], dtype=torch.float64, device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            per_dir = world * reps * (256 << 20) / float(tt.item()) / 1e9
            e2e["host_fabric"] = {"h2d_gbs_all_ranks": per_dir, "d2h_gbs_all_ranks": per_dir,
                                  "how": "all ranks copy 256 MiB page-locked blocks both ways at once, 8 times"}
        del host_pool, plain_pool
    dx.core.set_timing(False)

    # ---------------- leg 3: the reference CPU pipeline on this host ----------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        r, kind, cores, sample = cpu_pipeline_rate(wl, name, args.cpu_images, threads)
        cpu = {"value": r, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample}

    if rank == 0:
        line = {
            "metric": "images_per_sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_max / (K * R), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "ops": [n for n, _ in ops], "batch_per_gpu": batch,
                       "global_batch": batch * world, "output": list(out_shape),
                       "source_pool_images_per_gpu": pool_n, "source_pool_bytes_per_gpu": pool_bytes,
                       "timed_region": "%d x the %d steps inside one pair of CUDA events, %.0f ms" % (R, K, ms_max),
                       "l2": "inputs larger than L2: each step reads %d distinct sources and writes a fresh batch" % batch,
                       "sharding": "whole batches by index, batch j on rank j % n_gpus, no collective",
                       "resize": "parity unpinned: the reference's resize arithmetic (stb) is absent, the oracle "
                                 "restates its published behaviour"},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "checked": (checked["ok"] if checked is not None else None),
            "check": checked,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS,
                         "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": algo_per_launch,
                         "traffic": (NCU_DRAM_BYTES_PER_IMAGE[name] * batch if name in NCU_DRAM_BYTES_PER_IMAGE else None),
                         "traffic_kind": "ncu dram bytes of a 128-image launch scaled by the image count"},
            "cpu_baseline": cpu,
        }
        if checked is not None and not checked["ok"]:
            line["invalid"] = "the checked batch differs from the oracle or a kernel self-check failed"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
