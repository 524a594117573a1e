"""Benchmark of the KMeans hot path: Lloyd iterations/s on the n=10M, d=128, k=1024 fp32
configuration (synthetic blobs), on N GPUs of one box.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # CPU restatement of the reference, host cores

A step is one full Lloyd iteration over all samples: fused E-step + centroid accumulation,
merge of accumulator copies, all-reduce (N > 1), finalize, 32-byte status read.  Rows are
split into contiguous shards over the ranks (total work fixed: strong scaling).  Rank 0
prints one JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    # name: (n, d, k, dtype, cluster std, offset std, seed, description)
    "c3": dict(n=10_000_000, d=128, k=1024, dtype="f32", noise=1.0, spread=2.0, seed=2,
               desc="KMeans fp32 n=10M d=128 k=1024, x~N(0,1)+offset[cluster], offsets~N(0,4), "
                    "random-row init seed 2, tol=0"),
    "c2": dict(n=5_000_000, d=14, k=256, dtype="f32", noise=1.5, spread=None, seed=1,
               desc="KMeans fp32 n=5M d=14 k=256, blobs centres~U[-10,10] std 1.5, random-row "
                    "init seed 1, tol=0"),
    "c4": dict(n=2_000_000, d=32, k=64, dtype="f64", noise=None, spread=None, seed=3,
               desc="KMeans fp64 n=2M d=32 k=64, U[0,1] data, random-row init seed 3, tol=0"),
    "c1": dict(n=50_000, d=14, k=127, dtype="f32", noise=1.0, spread=None, seed=0,
               desc="KMeans fp32 n=50k d=14 k=127 blobs"),
    "c5": dict(n=20_000_000, d=64, k=4096, dtype="f32", noise=0.1, spread=None, seed=4,
               blobs=512, outliers=0.1, box=50.0,
               desc="KMeans fp32 n=20M d=64 k=4096: 90% from 512 tight blobs (std 0.1), 10% uniform "
                    "outliers in [-50,50]^64, k-means++ from seed 4"),
}
CHUNK = 1 << 20
# DRAM bytes (read + written) per sample row of one fused-step launch, from the ncu captures
# summarised under profiles/ (taken at a smaller n; the traffic grows in proportion to n).
DRAM_BYTES_PER_ROW = {
    ("tf32x3", 128): 540.4,     # lloyd_tc_kernel, n = 1 M, d = 128, k = 1024
    ("tf32x3", 14): 71.8,       # lloyd_tc_quads_kernel, n = 3 M, d = 14 padded to 16, k = 256
    ("cuda_core", 32): 266.5,   # lloyd_f64_kernel, n = 1 M, d = 32, k = 64, float64
}


def algorithmic_flops(n, d, k):
    return 2.0 * n * d * k


def algorithmic_bytes(n, d, k, s):
    # X once, labels read + written, centroids read + written, counts
    return n * d * s + 2 * 4 * n + 2 * k * d * s + k * s


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="MEASURED_PEAKS.json")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def measure_tf32_cublas(torch, device, size=8192, reps=10):
    """Dense TF32 GEMM rate of cuBLAS on this GPU (best of `reps`), for context next to the
    roofline denominator; MEASURED_PEAKS.json only holds the bf16 figure."""
    try:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn((size, size), device=device)
        b = torch.randn((size, size), device=device)
        best = None
        for _ in range(reps + 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None or ms < best else best
        torch.backends.cuda.matmul.allow_tf32 = prev
        return 2.0 * size ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def measure_fma_peak(torch, device, dtype_name):
    """FMA rate (TFLOP/s) of the CUDA cores in the compute dtype, measured now on this GPU."""
    import ctypes

    from sklearn_numba_dpex_b200._cabi import check, lib, ptr, stream_ptr

    out = ctypes.c_double(0.0)
    tdt = torch.float32 if dtype_name == "f32" else torch.float64
    scratch = torch.empty(8 * 256 * 256, dtype=tdt, device=device)
    try:
        check(lib.kmb_measure_fma_peak(0 if dtype_name == "f32" else 1, 10, ctypes.byref(out),
                                       ptr(scratch), stream_ptr(device)), "kmb_measure_fma_peak")
    except Exception:
        return None, None
    return out.value, None


# ----------------------------------------------------------------------------- data
def cluster_offsets(cfg, torch, device):
    g = torch.Generator(device="cpu").manual_seed(cfg["seed"] * 7919 + 1)
    d, k = cfg["d"], cfg.get("blobs", cfg["k"])
    if "box" in cfg:
        return ((torch.rand((k, d), generator=g) * 2.0 - 1.0) * cfg["box"]).to(device)
    if cfg["spread"] is not None:
        off = torch.randn((k, d), generator=g) * cfg["spread"]
    else:
        off = torch.rand((k, d), generator=g) * 20.0 - 10.0
    return off.to(device)


def generate_rows(cfg, start, stop, torch, device, dtype):
    """Rows [start, stop) of the synthetic data set; any rank can materialise any block
    because every CHUNK of rows has its own seed."""
    d, k = cfg["d"], cfg["k"]
    out = torch.empty((stop - start, d), dtype=dtype, device=device)
    offsets = cluster_offsets(cfg, torch, device).to(dtype)
    c0 = start // CHUNK
    pos = 0
    while start + pos < stop:
        chunk = (start + pos) // CHUNK
        lo, hi = chunk * CHUNK, min((chunk + 1) * CHUNK, cfg["n"])
        g = torch.Generator(device=device).manual_seed(cfg["seed"] * 1_000_003 + chunk)
        if cfg["noise"] is None:
            block = torch.rand((hi - lo, d), generator=g, device=device, dtype=dtype)
        else:
            ids = torch.randint(0, offsets.shape[0], (hi - lo,), generator=g, device=device)
            block = torch.randn((hi - lo, d), generator=g, device=device, dtype=dtype) * cfg["noise"]
            block += offsets[ids]
            if "outliers" in cfg:
                out_rows = torch.rand((hi - lo,), generator=g, device=device) < cfg["outliers"]
                uni = (torch.rand((hi - lo, d), generator=g, device=device, dtype=dtype) * 2 - 1) * cfg["box"]
                block = torch.where(out_rows[:, None], uni, block)
                del uni
        a, b = max(start, lo) - lo, min(stop, hi) - lo
        out[pos:pos + (b - a)] = block[a:b]
        pos += b - a
        del block
    return out


def initial_centres(cfg, X_shard, start, stop, torch, dist_mod):
    """Random distinct rows (numpy RandomState(seed).choice, the engine's "random" init);
    each rank contributes the rows it owns, one all-reduce assembles them."""
    idx = np.random.RandomState(cfg["seed"]).choice(cfg["n"], size=cfg["k"], replace=False)
    C = torch.zeros((cfg["k"], cfg["d"]), dtype=X_shard.dtype, device=X_shard.device)
    mine = np.nonzero((idx >= start) & (idx < stop))[0]
    if mine.size:
        C[torch.as_tensor(mine, device=C.device)] = X_shard[torch.as_tensor(idx[mine] - start,
                                                                           device=C.device)]
    dist_mod.all_reduce_sum_(C)
    return C


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fh = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = fh.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu_index)], stdout=fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        """Median SM clock and the throttle reasons seen between the two wall-clock times
        (all samples when none fall inside, e.g. a sub-second timed region)."""
        import datetime

        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(parts[1]), float(parts[2]), parts[5:9]))
                except ValueError:
                    continue
            os.unlink(self.path)
        except Exception:
            pass
        inside = [r for r in rows if t_begin is not None and t_begin - 0.05 <= r[0] <= t_end + 0.05]
        use = inside if inside else rows
        reasons = set()
        for _, _, _, flags in use:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), flags):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if use:
            out.update(sm_mhz=float(np.median([r[1] for r in use])),
                       sm_max_mhz=float(max(r[2] for r in use)), samples=len(use),
                       samples_in_timed_region=len(inside))
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------- CPU baseline
def host_threads():
    """Host threads this process may use.  Launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1; the CPU arms set their thread count from the affinity mask instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample(cfg, sample_rows):
    """`sample_rows` rows from the benchmark's own seeded generator (its CPU random stream; the
    GPU arm draws from the CUDA stream of the same generator) and initial centres drawn from
    them: what both CPU legs
    (the reference arm and the cpu_baseline of the GPU arm) and the provider-consistency check
    work on."""
    import torch

    key = (cfg["seed"], cfg["d"], cfg["k"], cfg["dtype"], int(sample_rows))
    if key not in _CPU_SAMPLES:
        dt = torch.float32 if cfg["dtype"] == "f32" else torch.float64
        sub = dict(cfg)
        sub["n"] = sample_rows
        X = generate_rows(sub, 0, sample_rows, torch, torch.device("cpu"), dt).numpy()
        idx = np.random.RandomState(cfg["seed"]).choice(sample_rows, size=cfg["k"], replace=False)
        _CPU_SAMPLES.clear()
        _CPU_SAMPLES[key] = (X, X[idx].copy())
    X, C = _CPU_SAMPLES[key]
    return X, C.copy()


_CPU_SAMPLES = {}


def cpu_reference_sample(cfg, sample_rows, iters, warmup=1):
    """Times the C restatement of the reference's Lloyd iteration on all host threads on a row
    sample of the workload and scales linearly in n to whole-job iterations/s."""
    from oracle import c_oracle

    threads = c_oracle.set_num_threads(host_threads())
    X, C = cpu_sample(cfg, sample_rows)
    first_labels = None
    for _ in range(max(warmup, 1)):
        first_labels, _, _, _ = c_oracle.lloyd_iteration(X, None, C)
    times = []
    for _ in range(iters):
        t0 = time.perf_counter()
        _, sums, counts, used = c_oracle.lloyd_iteration(X, None, C)
        times.append(time.perf_counter() - t0)
        nz = counts > 0
        C[nz] = sums[nz] / counts[nz, None]
    per_iter_full = float(np.mean(times)) * (cfg["n"] / sample_rows)
    base = dict(value=1.0 / per_iter_full, unit="iterations/s", cores=int(used), kind="port",
                extrapolated=bool(sample_rows < cfg["n"]),
                sample=f"{sample_rows} rows drawn by the benchmark's generator (same seed and "
                       f"distribution, CPU random stream), {iters} iterations of the C restatement "
                       f"on {used} threads, time scaled by n/{sample_rows}")
    sk = sklearn_lloyd_sample(X, cpu_sample(cfg, sample_rows)[1], min(iters, 5), int(used))
    if sk is not None:
        base["sklearn_lloyd"] = dict(value=1.0 / (sk * (cfg["n"] / sample_rows)), unit="iterations/s",
                                     threads=int(used),
                                     what="scikit-learn's own CPU Lloyd (_kmeans_single_lloyd, tol=0) on "
                                          "the same sample, for context")
    return base, times, first_labels


def sklearn_lloyd_sample(X, C, iters, threads):
    """Seconds per iteration of scikit-learn's CPU Lloyd loop on the sample, or None when this
    scikit-learn does not have the private entry point."""
    try:
        from sklearn.cluster._kmeans import _kmeans_single_lloyd
        from threadpoolctl import threadpool_limits
    except Exception:
        return None
    w = np.ones(X.shape[0], dtype=X.dtype)
    try:
        with threadpool_limits(limits=threads):
            _kmeans_single_lloyd(X, w, C.copy(), max_iter=1, tol=0.0, n_threads=threads)   # warm-up
            t0 = time.perf_counter()
            _, _, _, n_iter = _kmeans_single_lloyd(X, w, C.copy(), max_iter=iters, tol=0.0,
                                                   n_threads=threads)
        return (time.perf_counter() - t0) / max(int(n_iter), 1)
    except Exception:
        return None


def provider_consistency(cfg, sample_rows, cpu_labels, torch, device):
    """The check the reference's benchmark makes between providers (benchmark/kmeans.py:177-183
    there: every provider ran the same iterations and agrees): the first-iteration labels of the
    CUDA path on the CPU arm's sample, from the same centres, against the C restatement's.
    Labels may differ only where the two nearest centres tie within 1e-6 relative."""
    from oracle import reference_cpu as ref
    from sklearn_numba_dpex_b200.kmeans.drivers import get_labels_inertia

    X, C = cpu_sample(cfg, sample_rows)
    Xd, Cd = torch.as_tensor(X).to(device), torch.as_tensor(C).to(device)
    labels, _ = get_labels_inertia(Xd.T, Cd.T, None, False)
    ok, n_bad, n_unexplained = ref.labels_agree(labels.cpu().numpy(), cpu_labels, X, C)
    if not ok:
        raise AssertionError(f"providers disagree: {n_unexplained} of {n_bad} label mismatches on the "
                             f"{sample_rows}-row sample are not near-ties")
    return {"rows": int(sample_rows), "label_mismatches": int(n_bad), "unexplained": int(n_unexplained),
            "what": "first-iteration labels, CUDA path vs C restatement, same rows and centres"}


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_rows = max(cfg["k"] * 4, min(cfg["n"], args.cpu_sample_rows))
    base, times, _ = cpu_reference_sample(cfg, sample_rows, max(args.steps, 1), warmup=max(args.warmup, 1))
    ms = float(np.mean(times)) * (cfg["n"] / sample_rows) * 1e3
    line = {"impl": "reference", "metric": "Lloyd iterations/s", "value": base["value"],
            "unit": "iterations/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": cfg["desc"], "n": cfg["n"], "d": cfg["d"], "k": cfg["k"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "iterations/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, cfg):
    import torch
    import torch.distributed as tdist

    from sklearn_numba_dpex_b200 import dist as kdist
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState, lloyd

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        tdist.init_process_group("nccl", device_id=device)
        kdist.enable()
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float64
    esize = 4 if cfg["dtype"] == "f32" else 8
    n, d, k = cfg["n"], cfg["d"], cfg["k"]
    start, stop = kdist.shard_bounds(n, rank, world)
    X = generate_rows(cfg, start, stop, torch, device, dtype)
    C0 = initial_centres(cfg, X, start, stop, torch, kdist)
    state = LloydState(X, None, C0, args.algo)
    algo_name = {0: "auto", 1: "cuda_core", 2: "tf32x3"}[state.algo]

    def barrier():
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        state.step()
    barrier()
    launches0 = state.kernel_launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    # events around the fused kernel of every timed iteration (created ahead: the launch call
    # records them by handle)
    it0 = state.it
    for a, b in kev:
        a.record()
        b.record()
    state.step_events = {it0 + i: kev[i] for i in range(args.steps)}
    t_begin = time.time()
    ev0.record()
    out = state.run(args.steps, -1.0, pipelined=not args.no_pipeline, stop_on_strict=False)
    ev1.record()
    barrier()
    t_end = time.time()
    state.step_events = {}
    steps_run = out["n_iter"]
    assert steps_run == args.steps, (steps_run, args.steps)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    elapsed_ms = ev0.elapsed_time(ev1)
    kernel_ms = float(np.mean([a.elapsed_time(b) for a, b in kev]))
    launches = state.kernel_launches - launches0
    t = torch.tensor([elapsed_ms, kernel_ms], dtype=torch.float64, device=device)
    if world > 1:
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    elapsed_ms, kernel_ms = float(t[0]), float(t[1])
    ms_per_step = elapsed_ms / steps_run
    value = 1e3 / ms_per_step
    # the events bracket the fused kernel of every timed iteration: a kernel time that is not a
    # plausible share of the iteration means they were not recorded around it
    assert 0.2 * ms_per_step < kernel_ms <= 1.02 * ms_per_step, (kernel_ms, ms_per_step)

    # ---- end to end through the plugin: host buffers in, host results out
    e2e = None
    if not args.skip_e2e:
        n_local = stop - start
        Xh = torch.empty(X.shape, dtype=dtype).pin_memory()
        Xh.copy_(X)
        Ch = C0.cpu().pin_memory()
        # scaling cross-check, outside every timed region: the counts of the last step add up to
        # n and every rank holds the same total shift
        counts_total = float(state.packed_last[k * state.d: k * state.d + k].double().sum())
        shift_bits = torch.tensor([state.status_host.numpy().view(np.float64)[1]], dtype=torch.float64,
                                  device=device)
        if world > 1:
            lo, hi = shift_bits.clone(), shift_bits.clone()
            tdist.all_reduce(lo, op=tdist.ReduceOp.MIN)
            tdist.all_reduce(hi, op=tdist.ReduceOp.MAX)
            assert float(lo[0]) == float(hi[0]), "ranks disagree on the total shift"
        assert counts_total == float(n), (counts_total, n)
        del state
        del X
        torch.cuda.empty_cache()
        e2e_iters = args.steps
        X_np, C_np = Xh.numpy(), Ch.numpy()      # page-locked numpy views: what a user hands in

        phases = {}

        def engine_fit(copy_x, breakdown=False):
            from sklearn_numba_dpex_b200.kmeans import KMeans, KMeansEngine

            def mark(name, t_prev):
                # only in the (untimed) breakdown pass: wait for the device, note the phase
                if not breakdown:
                    return t_prev
                torch.cuda.synchronize()
                now = time.perf_counter()
                phases[name] = (now - t_prev) * 1e3
                return now

            KMeansEngine._CONFIG.update(device=local_rank, algo=args.algo)
            try:
                est = KMeans(n_clusters=k, init=C_np, n_init=1, max_iter=e2e_iters, tol=0.0,
                             copy_x=copy_x, algorithm="lloyd")
                barrier()
                t0 = time.perf_counter()
                engine = KMeansEngine(est)
                Xp, _, sw = engine.prepare_fit(X_np, sample_weight=None)
                tp = mark("validate_upload_centre_ms", t0)
                centers_init = engine.init_centroids(Xp, sw)
                labels, inertia, centers, n_iter = engine.kmeans_single(Xp, sw, centers_init)
                tp = mark("lloyd_loop_and_final_pass_ms", tp)
                engine.unshift_centers(Xp, centers)
                labels_h = labels.cpu()
                centres_h = centers.contiguous().cpu()
                torch.cuda.synchronize()
                dt_fit = time.perf_counter() - t0
                mark("unshift_and_read_back_ms", tp)
            finally:
                KMeansEngine._CONFIG.clear()
            # tol = 0 leaves strict convergence (labels unchanged) as the only early stop; well
            # separated data (the small configuration) reach it before max_iter
            t = torch.tensor([dt_fit], dtype=torch.float64, device=device)
            if world > 1:
                tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
            return float(t[0]), labels_h.numel(), centres_h.numel(), int(n_iter)

        def drivers_fit():
            wh = torch.ones(n_local, dtype=dtype).pin_memory()
            barrier()
            t0 = time.perf_counter()
            Xd = Xh.to(device, non_blocking=True)
            wd = wh.to(device, non_blocking=True)
            Cd = Ch.to(device, non_blocking=True)
            labels, inertia, C_t, n_iter = lloyd(Xd.T, wd, Cd.T, True, e2e_iters, False, 0.0,
                                                 algo=args.algo)
            labels.cpu()
            C_t.T.contiguous().cpu()
            torch.cuda.synchronize()
            dt_fit = time.perf_counter() - t0
            t = torch.tensor([dt_fit], dtype=torch.float64, device=device)
            if world > 1:
                tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
            return float(t[0]), int(n_iter)

        engine_fit(True)                          # untimed dry run (allocator, lazy initialisation)
        dt_copy, n_lab, n_cen, it_copy = engine_fit(True)
        dt_inplace, _, _, it_inplace = engine_fit(False)
        dt_drivers, it_drivers = drivers_fit()
        engine_fit(True, breakdown=True)          # untimed: the same call with a device wait per phase
        h2d = (Xh.numel() + Ch.numel()) * esize * world
        d2h = n_lab * 4 * world + n_cen * esize + esize
        e2e = {"value": it_copy / dt_copy, "unit": "iterations/s",
               "h2d_bytes_per_step": int(h2d // it_copy), "d2h_bytes_per_step": int(d2h // it_copy),
               "iterations_run": it_copy,
               "what": f"KMeansEngine.prepare_fit -> init_centroids (array) -> kmeans_single "
                       f"(max_iter={e2e_iters}, tol=0) -> unshift_centers on a page-locked numpy X "
                       "(validation, upload, centring, tolerance scaling, Lloyd loop, final assignment "
                       "and inertia), labels and centres copied back; copy_x=True",
               "breakdown_ms": {key: round(val, 3) for key, val in phases.items()},
               "copy_x_false": {"value": it_inplace / dt_inplace, "unit": "iterations/s"},
               "drivers_lloyd": {"value": it_drivers / dt_drivers, "unit": "iterations/s",
                                 "what": "one drivers.lloyd() call on tensors uploaded from pinned "
                                         "memory, no validation or centring"}}

    tf32_live = measure_tf32_cublas(torch, device) if (rank == 0 and algo_name == "tf32x3") else None
    if rank == 0:
        peaks = load_peaks()
        n_local = stop - start
        flops = algorithmic_flops(n_local, d, k)
        abytes = algorithmic_bytes(n_local, d, k, esize)
        tf_achieved = flops / (kernel_ms * 1e-3) / 1e12
        gb_achieved = abytes / (kernel_ms * 1e-3) / 1e9
        if algo_name == "tf32x3":
            # TF32 issues at half the bf16 rate and each product costs three MMAs (3xTF32).
            # The timed region is a fraction of a second, so the burst figure applies; the
            # fraction against the sustained (power-capped, ~1.34 GHz) figure is given too.
            peak = peaks["bf16_tflops"] / 6.0
            peak_sust = peaks["bf16_tflops_sustained"] / 6.0
            # DRAM bytes per sample row of the d=128 kernel from the ncu capture of n=1M
            # (summary kept with the other ncu summaries of this repository), growing in proportion to n
            traffic = DRAM_BYTES_PER_ROW.get(("tf32x3", d), 0) * n_local or None
            roofline = {"bound": "tensor", "achieved": tf_achieved, "peak": peak, "unit": "TFLOP/s",
                        "frac": tf_achieved / peak, "traffic": traffic,
                        "peak_source": f"{peaks['source']} bf16_tflops (burst) / 6: TF32 = half the "
                                       "bf16 rate, 3 MMAs per product (3xTF32)",
                        "frac_of_sustained_peak": tf_achieved / peak_sust,
                        "tf32_cublas_tflops_live": tf32_live,
                        "hbm_frac": gb_achieved / peaks["hbm_gbs"]}
        else:
            # CUDA-core step: the FMA pipe of the compute dtype binds long before HBM at this
            # arithmetic intensity; its ceiling is measured live by a register-resident kernel.
            fma_peak, fma_clock = measure_fma_peak(torch, device, cfg["dtype"])
            hbm_ms = abytes / peaks["hbm_gbs"] / 1e6
            fma_ms = flops / (fma_peak * 1e9) if fma_peak else None
            traffic = None
            if cfg["dtype"] == "f64":
                traffic = DRAM_BYTES_PER_ROW.get(("cuda_core", d), 0) * n_local or None
            if fma_peak and fma_ms >= hbm_ms:
                roofline = {"bound": "fma_pipe", "achieved": tf_achieved, "peak": fma_peak,
                            "unit": "TFLOP/s", "frac": tf_achieved / fma_peak, "traffic": traffic,
                            "peak_source": f"live {'FP32' if cfg['dtype'] == 'f32' else 'FP64'} FMA rate of "
                                           "a register-resident kernel (kmb_measure_fma_peak), best of 10",
                            "hbm_frac": gb_achieved / peaks["hbm_gbs"],
                            "ideal_ms": {"fma_pipe": fma_ms, "hbm": hbm_ms}}
            else:
                roofline = {"bound": "hbm", "achieved": gb_achieved, "peak": peaks["hbm_gbs"],
                            "unit": "GB/s", "frac": gb_achieved / peaks["hbm_gbs"], "traffic": traffic,
                            "peak_source": peaks["source"] + " hbm_gbs",
                            "fp_tflops_achieved": tf_achieved, "fma_peak_tflops": fma_peak}
        roofline["kernel_ms"] = kernel_ms
        line = {"metric": "Lloyd iterations/s", "value": value, "unit": "iterations/s",
                "n_gpus": world, "steps": steps_run, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
                "config": {"workload": cfg["desc"], "n": n, "d": d, "k": k, "algo": algo_name,
                           "rows_per_gpu": n_local,
                           "l2": "inputs larger than L2: every step streams this rank's X shard "
                                 f"({n_local * d * esize / 1e9:.2f} GB)"},
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline}
        if e2e is not None:
            line["e2e"] = e2e
        if world == 1 and not args.skip_cpu:
            rows = max(cfg["k"] * 4, min(n, args.cpu_sample_rows))
            line["cpu_baseline"], _, cpu_labels = cpu_reference_sample(cfg, rows, 3)
            line["provider_consistency"] = provider_consistency(cfg, rows, cpu_labels, torch, device)
        print(json.dumps(line), flush=True)
    if world > 1:
        tdist.barrier()
        tdist.destroy_process_group()


def run_fit_arm(args, cfg):
    """Whole-fit timing through the drivers: k-means++ seeding then `steps` Lloyd iterations
    (tol=0), rows sharded over the ranks.  Used for the seeding / relocation stress
    configuration; prints its own JSON line (not the headline metric)."""
    import torch
    import torch.distributed as tdist

    from sklearn_numba_dpex_b200 import dist as kdist
    from sklearn_numba_dpex_b200.kmeans.drivers import kmeans_plusplus, lloyd

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        tdist.init_process_group("nccl", device_id=device)
        kdist.enable()
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float64
    n, d, k = cfg["n"], cfg["d"], cfg["k"]
    start, stop = kdist.shard_bounds(n, rank, world)
    X = generate_rows(cfg, start, stop, torch, device, dtype)
    w = torch.ones(X.shape[0], dtype=dtype, device=device)

    def sync():
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    sync()
    t0 = time.perf_counter()
    centers_t, indices = kmeans_plusplus(X.T, w, k, np.random.RandomState(cfg["seed"]))
    sync()
    t1 = time.perf_counter()
    stats = {}
    labels, inertia, C_t, n_iter = lloyd(X.T, w, centers_t, True, args.steps, False, 0.0, algo=args.algo,
                                         stats=stats)
    sync()
    t2 = time.perf_counter()
    distinct = int(torch.unique(indices).numel())
    if rank == 0:
        print(json.dumps({
            "mode": "fit", "n_gpus": world, "config": {"workload": cfg["desc"], "n": n, "d": d, "k": k},
            "kmeanspp_seconds": t1 - t0, "kmeanspp_rounds_per_s": (k - 1) / (t1 - t0),
            "kmeanspp_distinct_centres": distinct,
            "lloyd_seconds_incl_final_pass": t2 - t1, "lloyd_iterations": int(n_iter),
            "lloyd_iterations_per_s": n_iter / (t2 - t1), "inertia": float(inertia),
            "n_relocation_events": stats.get("n_relocation_events"),
            "n_empty_max": stats.get("n_empty_max"),
            "data": "synthetic"}), flush=True)
    if world > 1:
        tdist.barrier()
        tdist.destroy_process_group()


def run_rowscan_arm(args, cfg):
    """Times the two row-scan kernels alone on one GPU, on rows of the configuration's shape:
    the k-means++ pass (`kmb_kpp_step`) for t = 1, 4, 8, 10 candidates and the inertia kernel.
    One JSON line; bytes are the algorithmic ones (X once, closest in, t outputs)."""
    import torch

    from sklearn_numba_dpex_b200._cabi import check, lib, ptr, stream_ptr, workspace_for

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    dtype = torch.float32 if cfg["dtype"] == "f32" else torch.float64
    code, esize = (0, 4) if dtype == torch.float32 else (1, 8)
    n, d, k = cfg["n"], cfg["d"], cfg["k"]
    X = generate_rows(cfg, 0, n, torch, device, dtype)
    w = torch.ones(n, dtype=dtype, device=device)
    nb = (n + lib.kmb_kpp_block_rows() - 1) // lib.kmb_kpp_block_rows()
    s = stream_ptr(device)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    out = {"mode": "rowscan", "config": {"workload": cfg["desc"], "n": n, "d": d, "k": k},
           "l2": "inputs larger than L2" if n * d * esize > 126e6 else "inputs fit L2", "kpp_step": {}}
    for t in (1, 4, 8, 10):
        M0 = torch.rand((t, n), dtype=dtype, device=device)
        M1 = torch.empty((t, n), dtype=dtype, device=device)
        bs = torch.empty((t, nb), dtype=torch.float64, device=device)
        best = torch.zeros(1, dtype=torch.int32, device=device)
        rows = X[:t].contiguous()
        ms = timed(lambda: check(lib.kmb_kpp_step(code, ptr(X), ptr(w), ptr(rows), ptr(M0), ptr(best),
                                                  ptr(M1), ptr(bs), n, d, t, s)))
        gb = (n * d * esize + 2 * n * esize + t * n * esize) / 1e9
        out["kpp_step"][f"t={t}"] = {"ms": ms, "GB/s": gb / ms * 1e3}
    C = X[:k].contiguous()
    labels = torch.randint(0, k, (n,), device=device, dtype=torch.int32)
    ws, wsb = workspace_for(device, n, d, k)
    tot = torch.empty(1, dtype=dtype, device=device)
    ms = timed(lambda: check(lib.kmb_inertia(code, ptr(X), ptr(w), ptr(C), ptr(labels), None, ptr(tot),
                                             n, d, k, ptr(ws), wsb, s)))
    out["inertia"] = {"ms": ms, "GB/s": (n * d * esize + 2 * n * esize) / 1e9 / ms * 1e3}
    peak = load_peaks()["hbm_gbs"]

    def line(ms_, nbytes):
        return {"ms": ms_, "GB/s": nbytes / 1e9 / ms_ * 1e3, "frac_of_hbm_peak": nbytes / 1e9 / ms_ * 1e3 / peak}

    # column sums (centring) and the in-place shift
    col = torch.empty(d, dtype=torch.float64, device=device)
    ms = timed(lambda: check(lib.kmb_col_sums(code, ptr(X), n, d, ptr(col), ptr(ws), wsb, s)))
    out["col_sums"] = line(ms, n * d * esize)
    vec = torch.zeros(d, dtype=dtype, device=device)
    ms = timed(lambda: check(lib.kmb_add_row_vector(code, ptr(X), n, d, ptr(vec), 1.0, s)))
    out["add_row_vector"] = line(ms, 2 * n * d * esize)
    # radix top-k over n values (the relocation's search), m = 1, 64, 4096
    vals = torch.rand(n, dtype=dtype, device=device)
    out["topk"] = {}
    for m in (1, 64, 4096):
        tws = torch.empty(lib.kmb_topk_workspace_bytes(1, n, m) + 256, dtype=torch.uint8, device=device)
        idx = torch.empty(m, dtype=torch.int64, device=device)
        ms = timed(lambda: check(lib.kmb_topk(code, ptr(vals), 1, n, m, None, ptr(idx), ptr(tws),
                                              tws.numel(), s)))
        out["topk"][f"m={m}"] = line(ms, n * esize)
    # euclidean distances (transform): n x k outputs, chunked so that the output stays modest
    kt = min(k, 256)
    rows = min(n, max(1, (1 << 30) // (kt * esize)))
    Y = X[:kt].contiguous()
    Dt = torch.empty((kt, rows), dtype=dtype, device=device)
    Xr = X[:rows]
    ms = timed(lambda: check(lib.kmb_euclidean_distances(code, ptr(Xr), ptr(Y), ptr(Dt), rows, d, kt, rows, s)))
    out["euclidean_distances"] = dict(line(ms, rows * d * esize + rows * kt * esize), rows=rows, k=kt,
                                      fma_tflops=3.0 * rows * d * kt / ms / 1e9,
                                      note="direct squared differences: 3 flops (subtract, multiply, add) "
                                           "per sample x centroid x feature on the FMA pipe")
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--n", "--rows", dest="n", type=int, default=None,
                    help="override the number of samples (use --rows under torchrun, whose own "
                         "parser claims the --n prefix)")
    ap.add_argument("--k", type=int, default=None, help="override the number of clusters")
    ap.add_argument("--algo", default="auto", choices=["auto", "cuda_core", "tf32x3"])
    ap.add_argument("--cpu-sample-rows", type=int, default=1_000_000)
    ap.add_argument("--mode", default="step", choices=["step", "fit", "rowscan"],
                    help="step: the headline per-iteration benchmark; fit: k-means++ + Lloyd; "
                         "rowscan: the k-means++ pass and the inertia kernel alone (1 GPU)")
    ap.add_argument("--no-pipeline", action="store_true",
                    help="read every iteration's status before enqueuing the next one")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config])
    if args.n:
        cfg["n"] = args.n
        cfg["desc"] += f" [n overridden to {args.n}]"
    if args.k:
        cfg["k"] = args.k
        cfg["desc"] += f" [k overridden to {args.k}]"
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    elif args.mode == "fit":
        run_fit_arm(args, cfg)
    elif args.mode == "rowscan":
        run_rowscan_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
