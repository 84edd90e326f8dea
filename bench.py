"""Headline benchmark: decode matmul effective HBM TB/s (weights + scales streamed per product / time).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path over one batch of synthetic input: for the default workload (the INT8 weight-only
product, K = 4096, N = 14336, M in {1, 8, 32}) one product per M against a weight copy that has not been touched for
at least 1 GiB of other weights, so every byte comes from HBM. With N > 1 GPUs (launched under torchrun) the weight
rows are split over the ranks and the output slices meet in an NCCL all-gather inside the timed region.

Prints ONE JSON line (rank 0). `value` is the whole-job figure with inputs resident in HBM; `e2e` is the same metric
through the host-buffer API (pinned host activations copied in, outputs copied out, every step); `roofline` is the
streaming kernel alone against the measured HBM copy bandwidth; `cpu_baseline` is the reference's own CPU backend on
the host cores of this machine. `--impl reference` times that CPU backend on the same steps instead.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from dromos_b200 import abi  # noqa: E402

WORKLOADS = {
    # name: (weight format, N, K, Ms, description)
    "c1_bf16": (abi.W_BF16, 4096, 4096, (1,), "BF16 GEMV M=1 K=4096 N=4096"),
    "c2_int8": (abi.W_INT8, 14336, 4096, (1, 8, 32), "INT8 weight-only gemm_w M in {1,8,32} K=4096 N=14336"),
    "c3_fp8": (abi.W_FP8, 28672, 8192, (1, 16, 64), "FP8 E4M3 (per-row scale) gemm_w M in {1,16,64} K=8192 N=28672"),
    "c3_nvfp4": (abi.W_NVFP4, 28672, 8192, (1, 16, 64), "NVFP4 gemm_w M in {1,16,64} K=8192 N=28672"),
    "c4_bf16x": (abi.W_BF16X, 14336, 4096, (1,), "BF16X lossless GEMV M=1 K=4096 N=14336"),
}
MOE_WORKLOADS = {
    # name: (weight format, E, top_k, L, I, T, description)
    "c5_moe_fp8": (abi.W_FP8, 64, 8, 4096, 1536, 32, "MoE routed experts E=64 top-8 L=4096 I=1536 FP8 (per-row scale), T=32"),
}
DTYPE = {abi.W_BF16: "bf16", abi.W_INT8: "int8xbf16->s32/f32", abi.W_FP8: "e4m3xbf16->f32", abi.W_NVFP4: "e2m1xbf16->f32",
         abi.W_BF16X: "bf16"}
ROTATE_BYTES = 1 << 30  # weights touched between two uses of the same copy (L2 is 126 MB)


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the workload's dominant kernel, from an ncu capture
# (profiles/tc_direct_kernel_c2_int8_m1.md); workloads without a capture report null.
NCU_TRAFFIC = {"c2_int8": 58.864e6 + 0.071e6}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def hold_load(fn, once_ms, seconds=0.6):
    """The K timed steps last a few milliseconds, less than one nvidia-smi sample: the same work is repeated (untimed)
    for a moment while the clock sampler still runs, so that the clocks it reports are clocks under this load. The
    number of repetitions comes from the measured time (the same on every rank, so collectives inside fn stay matched)."""
    import torch

    for _ in range(max(1, min(2000, int(seconds * 1e3 / max(once_ms, 1e-3))))):
        fn()
    torch.cuda.synchronize()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm),
                "window": "the timed steps and 0.6 s of the same steps repeated right after them"}


# ---------------------------------------------------------------------------------------------------------------------
# The reference's CPU backend (oracle/_ref) on host arrays: the cpu_baseline leg and the --impl reference arm.
# ---------------------------------------------------------------------------------------------------------------------


def cpu_library():
    path = os.path.join(ROOT, "oracle", "_ref", "libdromos_cpu.so")
    return abi.Library(path) if os.path.exists(path) else None


def cpu_inputs(wtype, N, K, Ms, copies):
    """Seeded host inputs in the stored format, quantized by the CPU library itself."""
    from oracle import dromos_oracle as O

    rng = np.random.default_rng(0)
    lib = cpu_library()
    weights = []
    for _ in range(copies):
        w = O.f32_to_bf16_bits((rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)))
        if wtype == abi.W_BF16:
            weights.append((abi.make_weight(wtype, w), w, None))
        elif wtype == abi.W_BF16X:
            n = lib.lx_bf16x_bytes(abi.ptr(w), N, K, None)
            buf = np.zeros(n, dtype=np.uint8)
            assert lib.lx_bf16x_encode(abi.ptr(w), N, K, abi.ptr(buf), n, None) == 0
            weights.append((abi.make_weight(wtype, buf), buf, None))
        else:
            data = np.zeros(N * (K // 2 if wtype == abi.W_NVFP4 else K), dtype=np.uint8)
            scale = np.zeros(N * K // 16, dtype=np.uint8) if wtype == abi.W_NVFP4 else np.zeros(N, dtype=np.float32)
            lw = abi.make_weight(wtype, data, scale)
            assert lib.lx_quantize_weight(abi.ptr(w), ctypes.byref(lw), N, K, None) == 0
            weights.append((lw, data, scale))
    xs = {M: O.f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32)) for M in Ms}
    ys = {M: np.zeros((M, N), dtype=np.float32) for M in Ms}
    return lib, weights, xs, ys


def cpu_step(lib, weights, xs, ys, N, K, Ms, i):
    for j, M in enumerate(Ms):
        lw = weights[(i * len(Ms) + j) % len(weights)][0]
        if M <= 8:
            st = lib.lx_gemv_w(abi.ptr(xs[M]), abi.BF16, K, ctypes.byref(lw), None, abi.BF16, abi.ptr(ys[M]), abi.F32, N, M, N, K,
                               1.0, 0.0, None)
        else:
            st = lib.lx_gemm_w(abi.ptr(xs[M]), abi.BF16, K, ctypes.byref(lw), abi.MATH_BF16, None, abi.BF16, abi.ptr(ys[M]), abi.F32,
                               N, M, N, K, 1.0, 0.0, None, None)
        assert st == 0, st


def weight_bytes(wtype, N, K, bf16x_bytes=None):
    from oracle import dromos_oracle as O

    return O.weight_bytes(wtype, N, K, bf16x_bytes)


def run_cpu(wtype, N, K, Ms, steps, warmup, bf16x_bytes=None):
    """Times `steps` steps of the reference CPU backend; returns (TB/s, ms per step, cores, sample text)."""
    one = weight_bytes(wtype, N, K, bf16x_bytes)
    copies = max(3, min(8, -(-(256 << 20) // one)))  # rotate at least 256 MiB so reads come from DRAM
    lib, weights, xs, ys = cpu_inputs(wtype, N, K, Ms, copies)
    for i in range(warmup):
        cpu_step(lib, weights, xs, ys, N, K, Ms, i)
    t0 = time.perf_counter()
    for i in range(steps):
        cpu_step(lib, weights, xs, ys, N, K, Ms, warmup + i)
    dt = time.perf_counter() - t0
    cores = os.cpu_count() or 1
    tbs = one * len(Ms) * steps / dt / 1e12
    return tbs, dt / steps * 1e3, cores, f"{steps} steps of the full workload ({len(Ms)} products each), {copies} weight copies rotated"


# ---------------------------------------------------------------------------------------------------------------------


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_int8", choices=sorted(WORKLOADS) + sorted(MOE_WORKLOADS))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.workload in MOE_WORKLOADS:
        return main_moe(args)
    wtype, N, K, Ms, desc = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = "decode matmul effective HBM TB/s"
    config = {"workload": desc, "rotation": "weight copies >= 1 GiB between reuses (inputs larger than L2)",
              "parallelism": "single GPU"}
    if world > 1:
        if os.environ.get("LX_BENCH_SCALING", "weak") == "strong":
            config["parallelism"] = f"the configuration's {N} rows of W split over {world} GPUs, all-gather of y"
        else:
            config["parallelism"] = f"{world} x {N} rows of W, {N} per GPU (the configuration's size on every GPU), all-gather of y"

    if args.impl == "reference":
        if rank != 0:
            return
        if cpu_library() is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libdromos_cpu.so is not built (make -C oracle ref)"}))
            return
        steps = max(1, min(args.steps, 20))
        tbs, ms, cores, sample = run_cpu(wtype, N, K, Ms, steps, min(args.warmup, 3))
        print(json.dumps({"impl": "reference", "metric": metric, "value": tbs, "unit": "TB/s", "n_gpus": args.gpus, "steps": steps,
                          "warmup": min(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": DTYPE[wtype], "data": "synthetic", "config": config,
                          "cpu_baseline": {"value": tbs, "unit": "TB/s", "cores": cores, "kind": "reference", "sample": sample},
                          "e2e": {"value": tbs, "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    import torch.distributed as dist

    from dromos_b200 import host

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = abi.Library()  # raises when the CUDA library is missing: there is no other path
    dev = torch.device("cuda", local)

    # ---- synthetic weights: each rank draws the rows it keeps ----
    # Weak scaling (default): the matrix grows with the job, world x N rows, so every GPU streams a shard of the
    # configuration's own size (a model world times wider on world GPUs); LX_BENCH_SCALING=strong splits the
    # configuration's N rows instead (29 MB per GPU at two GPUs: fixed costs, not bytes).
    strong = world > 1 and os.environ.get("LX_BENCH_SCALING", "weak") == "strong"
    N_job = N if strong or world == 1 else N * world
    n0, n1 = host.shard_rows(N_job, rank, world)
    gen = torch.Generator(device=dev).manual_seed(rank)
    w_shard = (torch.randn((n1 - n0, K), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    gen.manual_seed(0)  # the activations are the same on every rank
    first = host.store_weight(lib, w_shard, wtype)
    shard_bytes = first.nbytes()
    copies = max(3, -(-ROTATE_BYTES // (shard_bytes * len(Ms))) * len(Ms))
    stored = [first]
    for _ in range(copies - 1):
        stored.append(host.StoredWeight(wtype, first.data.clone(), None if first.scale is None else first.scale.clone(), first.glob,
                                        rows=first.rows, cols=first.cols))
    layers = [host.Linear(lib, s, n1 - n0, K) for s in stored]
    xs = {M: torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16) for M in Ms}
    ys = {M: torch.empty((M, n1 - n0), dtype=torch.float32, device=dev) for M in Ms}
    gathered = {M: torch.empty((world, M, n1 - n0), dtype=torch.float32, device=dev) for M in Ms} if world > 1 else None
    # whole-job bytes a step streams: every shard of every product (all ranks' shards are the same size up to rounding)
    total_step_bytes = torch.tensor([float(shard_bytes * len(Ms))], device=dev)
    if world > 1:
        dist.all_reduce(total_step_bytes)
    total_step_bytes = float(total_step_bytes.item())

    # More than one GPU: the products store their slices straight into every rank's y (the all-gather is the kernel's
    # epilogue, NVLink peer stores, no collective kernel). Where that is not available (format, symmetric memory) the
    # slices meet in an NCCL all-gather instead. Measured at 2 GPUs on this workload the NCCL exchange is the faster one
    # (93.6 us per step against 101.5 us), so it is the default; LX_BENCH_FUSED=1 takes the epilogue.
    fused = None
    if world > 1 and os.environ.get("LX_BENCH_FUSED", "0") == "1":
        try:
            fused = [host.FusedShardedLinear(lib, None, wtype, N_job, K, max(Ms), stored=sw) for sw in stored]
            for M in Ms:
                fused[0](xs[M])
            torch.cuda.synchronize()
        except Exception as e:
            print(f"[bench] all-gather epilogue unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
            fused = None
        ok = torch.tensor([1 if fused is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # every rank takes the same path
        if int(ok.item()) == 0:
            fused = None
    config["exchange"] = "all-gather epilogue (peer stores over NVLink)" if fused is not None else ("NCCL all-gather" if world > 1 else "none")
    if world > 1 and fused is None and os.environ.get("LX_BENCH_OVERLAP", "0") == "1":
        config["exchange"] += ", overlapped with the next (independent) product of the step"

    overlap = world > 1 and os.environ.get("LX_BENCH_OVERLAP", "0") == "1"
    pending = []

    def step(i):
        for j, M in enumerate(Ms):
            c = (i * len(Ms) + j) % copies
            if fused is not None:
                fused[c](xs[M])
                continue
            layers[c](xs[M], ys[M])
            if world > 1:
                # The three products of a step are independent, so a product's all-gather runs (on NCCL's own stream)
                # under the next product when LX_BENCH_OVERLAP=1 (measured at 2 GPUs: no gain, the products fill every SM).
                work = dist.all_gather_into_tensor(gathered[M].view(world * M, n1 - n0), ys[M], async_op=overlap)
                if overlap:
                    pending.append(work)
        while pending:
            pending.pop(0).wait()

    # The decode loop is launch-bound from Python (a product is ~15 us of GPU time), so, like the reference engine's
    # decode loop, the steps are captured once into CUDA graphs (one per rotation position, programmatic dependent
    # launch edges included) and replayed; LX_BENCH_GRAPHS=0 launches every kernel from Python instead.
    use_graphs = os.environ.get("LX_BENCH_GRAPHS", "1") != "0"

    all_graphs = []

    def capture(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        all_graphs.append(g)
        return g

    def replayer(fn, period):
        """fn(i) for i in range(period) captured as graphs; returns run(i) that replays graph i % period, and how many
        of this library's kernels one pass over the period launches."""
        for i in range(period):  # every allocation (workspaces, the status word) happens before capture
            fn(i)
        torch.cuda.synchronize()
        before = lib.lx_b200_kernel_launches()
        if not use_graphs:
            fn(0)
            return fn, (lib.lx_b200_kernel_launches() - before) * period
        try:
            graphs = [capture(lambda i=i: fn(i)) for i in range(period)]
        except Exception as e:  # e.g. a collective that cannot be captured: fall back to eager launches
            print(f"[bench] graph capture failed ({type(e).__name__}: {e}); launching eagerly", file=sys.stderr)
            torch.cuda.synchronize()
            return fn, 0
        return (lambda i: graphs[i % period].replay()), lib.lx_b200_kernel_launches() - before

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    period = copies // len(Ms)  # steps until the rotation comes back to the first weight copy
    run_step, launches_per_period = replayer(step, period)
    for i in range(args.warmup):
        run_step(i)
    # The K timed steps are ONE graph (the reference's method, bench/bench_gemv.py:74-119: every launch of the timed
    # region in one graph), so that no host round trip sits between two steps; eager when graphs are off or the capture
    # fails (then every step is a host launch).
    whole = None
    if use_graphs:
        try:
            whole = capture(lambda: [step(args.warmup + i) for i in range(args.steps)])
            whole.replay()  # once untimed: the graph's own first-launch cost
        except Exception as e:
            print(f"[bench] capture of the timed region failed ({type(e).__name__}: {e}); replaying per step", file=sys.stderr)
            torch.cuda.synchronize()
            whole = None
    with ClockSampler(local) as clocks:
        if whole is not None:
            ms = timed(lambda i: whole.replay(), 1)
        else:
            ms = timed(lambda i: run_step(args.warmup + i), args.steps)
        hold_load(whole.replay if whole is not None else (lambda: run_step(0)), ms if whole is not None else ms / args.steps)
    launches = launches_per_period * args.steps // period
    value = total_step_bytes * args.steps / (ms * 1e-3) / 1e12

    # ---- the product kernels alone, per M (events on the launching stream, no collective): one graph holds a pass
    # over every weight copy ----
    per_m, k_bytes, k_ms = {}, 0.0, 0.0
    reps = max(2, min(20, int(4e9 // (shard_bytes * copies))))
    for M in Ms:
        def sweep(_, M=M):
            for c in range(copies):
                layers[c](xs[M], ys[M])
        run_sweep, _ = replayer(sweep, 1)
        for i in range(2):
            run_sweep(i)
        t = timed(run_sweep, reps) / (reps * copies)
        per_m[str(M)] = {"us": t * 1e3, "GB/s": shard_bytes / (t * 1e-3) / 1e9}
        k_bytes += shard_bytes
        k_ms += t
    peak, peak_kind = measured_peak_gbs()
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    dominant = "tc_direct_kernel" if wtype in (abi.W_INT8, abi.W_FP8) else "stream_kernel"
    # DRAM bytes per launch of the dominant kernel from the ncu capture summarised under profiles/ (read + write)
    traffic = NCU_TRAFFIC.get(args.workload) if world == 1 else None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "peak_source": f"{peak_kind} copy bandwidth (burst)", "kernel": dominant, "per_m": per_m,
                "algorithmic_bytes_per_launch": shard_bytes}

    # ---- end to end through the host-buffer API: pinned activations in, outputs out, every step ----
    xh = {M: xs[M].cpu().pin_memory() for M in Ms}
    yh = {M: torch.empty((M, (n1 - n0) * (world if world > 1 else 1)), dtype=torch.float32).pin_memory() for M in Ms}
    xd = {M: torch.empty_like(xs[M]) for M in Ms}

    # The device-to-host copy of a product's outputs runs on a second stream under the next product of the step (largest
    # outputs first, so that the longest copy has the most to hide behind); the step ends when every copy has landed.
    copy_stream = torch.cuda.Stream() if world == 1 else None

    def e2e_work(i):
        main = torch.cuda.current_stream()
        for j, M in sorted(enumerate(Ms), key=lambda jm: -jm[1]):
            xd[M].copy_(xh[M], non_blocking=True)
            if fused is not None:
                src = fused[(i * len(Ms) + j) % copies](xd[M])
            else:
                layers[(i * len(Ms) + j) % copies](xd[M], ys[M])
                src = ys[M]
                if world > 1:
                    dist.all_gather_into_tensor(gathered[M].view(world * M, n1 - n0), ys[M])
                    src = gathered[M].permute(1, 0, 2).reshape(M, -1)
            if world > 1:  # with collectives in the step everything stays on one stream
                yh[M].copy_(src, non_blocking=True)
                continue
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                yh[M].copy_(src, non_blocking=True)
        if world == 1:
            main.wait_stream(copy_stream)

    run_e2e, _ = replayer(e2e_work, period)

    def e2e_step(i):
        run_e2e(i)
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step

    for i in range(3):
        e2e_step(i)
    e2e_ms = timed(e2e_step, args.steps)
    e2e = {"value": total_step_bytes * args.steps / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s",
           "h2d_bytes_per_step": sum(M * K * 2 for M in Ms), "d2h_bytes_per_step": sum(M * N * 4 for M in Ms)}

    status = lib.lx_b200_last_error()

    def leave():
        """Graphs that hold NCCL kernels must be gone before the communicator is: release them, meet, then leave the
        process without running NCCL's destructors (which can wait for ever on a communicator a graph once captured)."""
        torch.cuda.synchronize()
        for g in all_graphs:
            g.reset()
        all_graphs.clear()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        leave()
        return
    out = {"metric": metric, "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if strong else "weak",
           "vs_baseline": None, "dtype": DTYPE[wtype], "data": "synthetic", "config": config, "roofline": roofline, "e2e": e2e,
           "gpu_launches": int(launches), "launch": "CUDA graphs" if use_graphs else "eager", "clocks": clocks.summary(), "pct_of_8TBs": value / 8.0 / max(world, 1),
           "kernel_status": status}
    if world == 1:
        if cpu_library() is not None:
            bx = shard_bytes if wtype == abi.W_BF16X else None
            tbs, _, cores, sample = run_cpu(wtype, N, K, Ms, 8, 2, bx)
            out["cpu_baseline"] = {"value": tbs, "unit": "TB/s", "cores": cores, "kind": "reference", "sample": sample}
        else:
            out["cpu_baseline"] = {"value": None, "unit": "TB/s", "cores": os.cpu_count(), "kind": "reference",
                                   "sample": "oracle/_ref/libdromos_cpu.so not built"}
    print(json.dumps(out), flush=True)
    leave()


def main_moe(args):
    """The routed-experts workload (C5): a step is lx_moe_route + lx_moe_experts_grouped on T tokens with fresh logits
    and the next copy of the expert stacks (>= 1 GiB of other weights between two uses of a copy). Bytes of a step =
    the weights and scales of the experts the step's routing touches (the reference's accounting, model/traffic.cpp:23-58).
    With N > 1 ranks the experts are split over the ranks (expert parallel: two all-to-all exchanges per step)."""
    wtype, E, top_k, L, I, T, desc = MOE_WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    metric = "decode matmul effective HBM TB/s"
    config = {"workload": desc, "rotation": "expert stack copies >= 1 GiB between reuses (inputs larger than L2)",
              "parallelism": f"experts split over {world} GPU(s), all-to-all of routed rows" if world > 1 else "single GPU"}
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm of bench.py times the dense workloads only"}))
        return
    import torch
    import torch.distributed as dist

    from dromos_b200 import host

    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = abi.Library()
    dev = torch.device("cuda", local)
    e0, e1 = host.expert_range(E, rank, world)
    gen = torch.Generator(device=dev).manual_seed(0)
    per_expert = (2 * I * L + L * I) + 4 * (2 * I + L)  # bytes of one expert: both stacks and their row scales
    local_bytes = per_expert * (e1 - e0)
    copies = max(2, -(-ROTATE_BYTES // local_bytes) + 1)
    stacks = []
    for c in range(copies):
        if c == 0:
            gu = host.store_weight(lib, (torch.randn((e1 - e0, 2 * I, L), generator=gen, device=dev) * 0.02).to(torch.bfloat16), wtype)
            dn = host.store_weight(lib, (torch.randn((e1 - e0, L, I), generator=gen, device=dev) * 0.02).to(torch.bfloat16), wtype)
        else:
            gu = host.StoredWeight(wtype, stacks[0][0].data.clone(), stacks[0][0].scale.clone(), stacks[0][0].glob, rows=stacks[0][0].rows, cols=L)
            dn = host.StoredWeight(wtype, stacks[0][1].data.clone(), stacks[0][1].scale.clone(), stacks[0][1].glob, rows=stacks[0][1].rows, cols=I)
        stacks.append((gu, dn))
    t0, t1 = T * rank // world, T * (rank + 1) // world  # this rank's tokens
    periods = 8  # distinct routings
    logits = [torch.randn((T, E), generator=torch.Generator(device=dev).manual_seed(100 + i), device=dev)[t0:t1].contiguous()
              for i in range(periods)]
    latent = torch.randn((T, L), generator=gen, device=dev).to(torch.bfloat16)[t0:t1].contiguous()
    if world == 1:
        engines = [host.Experts(lib, gu, dn, E, L, I, top_k) for gu, dn in stacks]
    else:
        engines = [host.ExpertParallel(lib, gu, dn, E, L, I, top_k) for gu, dn in stacks]
    router = host.Experts(lib, stacks[0][0], stacks[0][1], E, L, I, top_k)
    out = torch.empty((t1 - t0, L), dtype=torch.float32, device=dev)
    touched = []
    for i in range(periods):  # the experts each routing touches, whole job (the same seeds on every rank give the same T x E logits)
        full = torch.randn((T, E), generator=torch.Generator(device=dev).manual_seed(100 + i), device=dev)
        touched.append(int(torch.unique(torch.topk(full, top_k, dim=1).indices).numel()))

    def step(i):
        ids, w = router.route(logits[i % periods])
        if world == 1:
            engines[i % copies](latent, ids, w, out)
        else:
            out.copy_(engines[i % copies](latent, ids, w))

    use_graphs = world == 1 and os.environ.get("LX_BENCH_GRAPHS", "1") != "0"
    period = periods * copies
    for i in range(min(period, 4)):
        step(i)
    torch.cuda.synchronize()
    before = lib.lx_b200_kernel_launches()
    step(0)
    launches_per_step = lib.lx_b200_kernel_launches() - before
    if use_graphs:
        graphs = []
        for i in range(period):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step(i)
            graphs.append(g)
        run = lambda i: graphs[i % period].replay()
    else:
        run = step

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(n):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for i in range(args.warmup):
        run(i)
    whole = None
    if use_graphs:  # the timed steps as one graph, no host round trip between steps
        whole = torch.cuda.CUDAGraph()
        with torch.cuda.graph(whole):
            for i in range(args.steps):
                step(args.warmup + i)
        whole.replay()
    with ClockSampler(local) as clocks:
        ms = timed((lambda i: whole.replay()), 1) if whole is not None else timed(lambda i: run(args.warmup + i), args.steps)
        hold_load(whole.replay if whole is not None else (lambda: run(0)), ms if whole is not None else ms / args.steps)
    step_bytes = [per_expert * touched[(args.warmup + i) % periods] for i in range(args.steps)]
    value = sum(step_bytes) / (ms * 1e-3) / 1e12
    peak, peak_kind = measured_peak_gbs()
    achieved = sum(step_bytes) / (ms * 1e-3) / 1e9 / world
    # end to end: logits and latent from pinned host memory in, the tokens' outputs out, every step
    lh = [x.cpu().pin_memory() for x in logits]
    xh = latent.cpu().pin_memory()
    oh = torch.empty(out.shape, dtype=torch.float32).pin_memory()
    ld, xd = torch.empty_like(logits[0]), torch.empty_like(latent)

    def e2e_step(i):
        ld.copy_(lh[i % periods], non_blocking=True)
        xd.copy_(xh, non_blocking=True)
        ids, w = router.route(ld)
        if world == 1:
            engines[i % copies](xd, ids, w, out)
        else:
            out.copy_(engines[i % copies](xd, ids, w))
        oh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    e2e_ms = timed(e2e_step, args.steps)
    status = lib.lx_b200_last_error()
    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": value, "unit": "TB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": DTYPE[wtype], "data": "synthetic", "config": config,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "peak_source": f"{peak_kind} copy bandwidth (burst)", "kernel": "tc_expert_kernel (whole step: route + 6 kernels)",
                         "algorithmic_bytes_per_launch": sum(step_bytes) / len(step_bytes)},
            "e2e": {"value": sum(step_bytes) / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s",
                    "h2d_bytes_per_step": T * E * 4 + T * L * 2, "d2h_bytes_per_step": T * L * 4},
            "gpu_launches": int(launches_per_step * args.steps), "launch": "CUDA graphs" if use_graphs else "eager",
            "clocks": clocks.summary(), "pct_of_8TBs": value / 8.0 / max(world, 1), "kernel_status": status,
            "cpu_baseline": {"value": None, "unit": "TB/s", "cores": os.cpu_count(), "kind": "reference",
                             "sample": "not timed for this workload (the dense workloads time the reference CPU backend)"}}))
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
