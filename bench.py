"""Headline benchmark: decode matmul effective HBM TB/s (weights + scales streamed per product / time).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--only NAME[,NAME..]]

One run times all six workloads of the decode path and prints ONE JSON line (rank 0):

  c1_bf16   BF16 GEMV, M = 1, K = 4096, N = 4096
  c2_int8   INT8 weight-only, M in {1, 8, 32}, K = 4096, N = 14336
  c3_fp8    FP8 E4M3 (per-row scale), M in {1, 16, 64}, K = 8192, N = 28672      <- the headline: value, roofline, e2e
  c3_nvfp4  NVFP4, same shape
  c4_bf16x  BF16X lossless GEMV, M = 1, K = 4096, N = 14336
  c5_moe_fp8  routed experts, E = 64, top-8, L = 4096, I = 1536, FP8, T = 32

A step is one pass of the hot path over one batch of synthetic input: one product per M of the workload (for c5: route
+ experts) against a weight copy that has not been touched for at least 1 GiB of other weights, so every byte comes
from HBM. The K timed steps of the headline are one replayed CUDA graph, timed with CUDA events on the launching stream.
`value` is the whole-job figure with inputs resident in HBM; `e2e` is the same metric through the host-buffer API
(pinned host activations copied in, outputs copied out, every step); `roofline` is the product kernels alone against
the measured HBM copy bandwidth and against the read-only ceiling measured in the same run (lx_bandwidth_probe);
`cpu_baseline` is the reference's own CPU backend on the host cores of this machine. `per_config` carries the same
figures for each workload. `--impl reference` times that CPU backend on the same workloads instead.

With N > 1 GPUs (torchrun) the headline is the STRONG split: the configuration's rows of W are split over the ranks,
the activations are replicated and the output slices meet in lx_b200_exchange_slices (one kernel of peer stores over
NVLink; LX_BENCH_EXCHANGE=nccl takes NCCL's all-gather instead); c3_nvfp4 likewise, c2_int8 also as the weak split
(every GPU streams a shard of the configuration's own size), c5 expert-parallel. Outside the timed region every rank
recomputes a peer's slice from the peer's seed with its own kernel and compares it bit for bit with what arrived
(`parity_check`); a mismatch ends the run with a non-zero exit code.
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

DENSE = {
    # name: (weight format, N, K, Ms, description)
    "c1_bf16": (abi.W_BF16, 4096, 4096, (1,), "BF16 GEMV M=1 K=4096 N=4096"),
    "c2_int8": (abi.W_INT8, 14336, 4096, (1, 8, 32), "INT8 weight-only gemm_w M in {1,8,32} K=4096 N=14336"),
    "c3_fp8": (abi.W_FP8, 28672, 8192, (1, 16, 64), "FP8 E4M3 (per-row scale) gemm_w M in {1,16,64} K=8192 N=28672"),
    "c3_nvfp4": (abi.W_NVFP4, 28672, 8192, (1, 16, 64), "NVFP4 gemm_w M in {1,16,64} K=8192 N=28672"),
    "c4_bf16x": (abi.W_BF16X, 14336, 4096, (1,), "BF16X lossless GEMV M=1 K=4096 N=14336"),
}
MOE = {
    # name: (weight format, E, top_k, L, I, T, description)
    "c5_moe_fp8": (abi.W_FP8, 64, 8, 4096, 1536, 32, "MoE routed experts E=64 top-8 L=4096 I=1536 FP8 (per-row scale), T=32"),
}
HEADLINE = "c3_fp8"
ORDER = ["c1_bf16", "c2_int8", "c3_fp8", "c3_nvfp4", "c4_bf16x", "c5_moe_fp8"]
DTYPE = {abi.W_BF16: "bf16", abi.W_INT8: "int8xbf16->f32", abi.W_FP8: "e4m3xbf16->f32", abi.W_NVFP4: "e2m1xbf16->f32", abi.W_BF16X: "bf16"}
KERNELS = {"c1_bf16": "gemv_kernel<bf16>", "c2_int8": "tc_direct_kernel<int8>", "c3_fp8": "tc_direct_kernel<fp8> (M=16,64), gemv_kernel<fp8> (M=1)",
           "c3_nvfp4": "tc_nvfp4_ss_kernel (M=16,64), gemv_ring8_kernel<nvfp4> (M=1)", "c4_bf16x": "gemv_x16_kernel",
           "c5_moe_fp8": "tc_expert_kernel (whole step: route, group, 2 x (prepare, experts), ordered sum)"}
ROTATE_BYTES = 1 << 30  # weights touched between two uses of the same copy (L2 is 126 MB)
METRIC = "decode matmul effective HBM TB/s"

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of a workload's dominant kernel, from ncu captures of this
# library on a B200 (the summaries under profiles/; bytes; mean of the captured launches). c3_fp8: tc_direct_kernel,
# the M = 16 and M = 64 launches; c3_nvfp4: tc_nvfp4_ss_kernel at M = 16; c5_moe_fp8: the gate/up plus the down launch of
# one step. The few MB written are mostly lines the setup left dirty in L2: the kernels write 0.1-7 MB of outputs.
NCU_TRAFFIC = {"c1_bf16": 33.59e6, "c2_int8": 58.854e6 + 0.105e6, "c3_fp8": (235.69e6 + 5.20e6 + 237.49e6 + 6.77e6) / 2, "c3_nvfp4": 132.46e6 + 3.55e6,
               "c4_bf16x": 88.87e6 + 3.47e6, "c5_moe_fp8": 400.74e6 + 7.10e6 + 840.85e6 + 4.11e6}


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def config_of(name, world, scaling, exchange):
    desc = (DENSE.get(name) or MOE.get(name))[-1]
    if world == 1:
        par = "single GPU"
    elif name in MOE:
        par = f"experts split over {world} GPUs, routing and tokens replicated, weighted rows exchanged"
    elif scaling == "strong":
        par = f"the configuration's rows of W split over {world} GPUs, activations replicated, y slices exchanged"
    else:
        par = f"{world} x the configuration's rows of W, one configuration-sized shard per GPU, y slices exchanged"
    return {"workload": desc, "rotation": "weight copies >= 1 GiB between reuses (inputs larger than L2)", "parallelism": par,
            "exchange": exchange}


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
# The reference's CPU backend (oracle/_ref) on host arrays: the cpu_baseline legs and the --impl reference arm.
# ---------------------------------------------------------------------------------------------------------------------


def reference_cuda_library():
    """The reference's own CUDA backend (oracle/_ref/libdromos_kernels_ref.so, `make -C oracle cuda_ref`), timed beside this
    library's kernels only when --reference-cuda asks for it: a reported baseline like the CPU one, never part of `value`."""
    path = os.path.join(ROOT, "oracle", "_ref", "libdromos_kernels_ref.so")
    return abi.Library(path) if os.path.exists(path) else None


def cpu_library():
    path = os.path.join(ROOT, "oracle", "_ref", "libdromos_cpu.so")
    return abi.Library(path) if os.path.exists(path) else None


def _bf16_normal_host(rng, shape, std):
    from oracle import dromos_oracle as O

    out = np.empty(shape, dtype=np.uint16)
    flat = out.reshape(-1)
    step = 1 << 24
    for i in range(0, flat.size, step):  # in pieces: a whole f32 copy of the larger matrices would be gigabytes
        n = min(step, flat.size - i)
        flat[i:i + n] = O.f32_to_bf16_bits(rng.standard_normal(n, dtype=np.float32) * np.float32(std))
    return out


def _cpu_store(lib, w_bits, wtype, rows, cols):
    """A bf16 [rows, cols] host matrix in a stored format, converted by the CPU library itself."""
    if wtype == abi.W_BF16:
        return abi.make_weight(wtype, w_bits), (w_bits, None)
    if wtype == abi.W_BF16X:
        n = lib.lx_bf16x_bytes(abi.ptr(w_bits), rows, cols, None)
        buf = np.zeros(n, dtype=np.uint8)
        assert lib.lx_bf16x_encode(abi.ptr(w_bits), rows, cols, abi.ptr(buf), n, None) == 0
        return abi.make_weight(wtype, buf), (buf, None)
    data = np.zeros(rows * (cols // 2 if wtype == abi.W_NVFP4 else cols), dtype=np.uint8)
    scale = np.zeros(rows * cols // 16, dtype=np.uint8) if wtype == abi.W_NVFP4 else np.zeros(rows, dtype=np.float32)
    lw = abi.make_weight(wtype, data, scale)
    assert lib.lx_quantize_weight(abi.ptr(w_bits), ctypes.byref(lw), rows, cols, None) == 0
    return lw, (data, scale)


def cpu_dense(name, steps, warmup):
    """`steps` steps of a dense workload on the reference CPU backend: (TB/s, ms per step, cores, sample text)."""
    from oracle import dromos_oracle as O

    wtype, N, K, Ms, _ = DENSE[name]
    lib = cpu_library()
    rng = np.random.default_rng(0)
    lw0, keep0 = _cpu_store(lib, _bf16_normal_host(rng, (N, K), 0.02), wtype, N, K)
    one = int(keep0[0].nbytes + (keep0[1].nbytes if keep0[1] is not None else 0) + (4 if wtype == abi.W_NVFP4 else 0))
    copies = max(1, min(8, -(-(256 << 20) // one)))  # rotate >= 256 MiB so reads come from DRAM (one copy when it is that large)
    weights, keep = [lw0], [keep0]
    for _ in range(copies - 1):
        d, s = keep0[0].copy(), None if keep0[1] is None else keep0[1].copy()
        keep.append((d, s))
        weights.append(abi.make_weight(wtype, d, s, lw0.glob))
    xs = {M: _bf16_normal_host(rng, (M, K), 1.0) for M in Ms}
    ys = {M: np.zeros((M, N), dtype=np.float32) for M in Ms}
    ws = np.zeros(max(1, max(lib.lx_gemm_workspace_bytes(M, K, abi.MATH_BF16) for M in Ms)), dtype=np.uint8)

    def step(i):
        for j, M in enumerate(Ms):
            lw = weights[(i * len(Ms) + j) % copies]
            if M <= 8:
                st = lib.lx_gemv_w(abi.ptr(xs[M]), abi.BF16, K, ctypes.byref(lw), None, abi.BF16, abi.ptr(ys[M]), abi.F32, N, M, N, K, 1.0, 0.0, None)
            else:
                st = lib.lx_gemm_w(abi.ptr(xs[M]), abi.BF16, K, ctypes.byref(lw), abi.MATH_BF16, None, abi.BF16, abi.ptr(ys[M]), abi.F32, N, M, N, K,
                                   1.0, 0.0, abi.ptr(ws), None)
            assert st == 0, st

    for i in range(warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(steps):
        step(warmup + i)
    dt = time.perf_counter() - t0
    del keep
    return one * len(Ms) * steps / dt / 1e12, dt / steps * 1e3, os.cpu_count() or 1, \
        f"{steps} steps of the full workload ({len(Ms)} products each) after {warmup} warm-up steps, {copies} weight cop{'y' if copies == 1 else 'ies'} rotated"


def cpu_moe(name, steps, warmup):
    """`steps` steps (lx_moe_route + lx_moe_experts_grouped) of the routed-experts workload on the reference CPU backend."""
    wtype, E, top_k, L, I, T, _ = MOE[name]
    lib = cpu_library()
    rng = np.random.default_rng(0)
    gu, keep_gu = _cpu_store(lib, _bf16_normal_host(rng, (E * 2 * I, L), 0.02), wtype, E * 2 * I, L)
    dn, keep_dn = _cpu_store(lib, _bf16_normal_host(rng, (E * L, I), 0.02), wtype, E * L, I)
    latent = _bf16_normal_host(rng, (T, L), 1.0)
    logits = [rng.standard_normal((T, E), dtype=np.float32) for _ in range(8)]
    ids, wts = np.zeros((T, top_k), dtype=np.int32), np.zeros((T, top_k), dtype=np.float32)
    ent, conf = np.zeros(T, dtype=np.float32), np.zeros(T, dtype=np.float32)
    out = np.zeros((T, L), dtype=np.float32)
    ws = np.zeros(max(256, lib.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, abi.MATH_BF16)), dtype=np.uint8)
    per_expert = (2 * I * L + L * I) + 4 * (2 * I + L)
    touched = []

    def step(i):
        lg = logits[i % len(logits)]
        assert lib.lx_moe_route(abi.ptr(lg), None, abi.ptr(ids), abi.ptr(wts), abi.ptr(ent), abi.ptr(conf), T, E, top_k, None) == 0
        assert lib.lx_moe_experts_grouped(abi.ptr(latent), abi.ptr(ids), abi.ptr(wts), ctypes.byref(gu), ctypes.byref(dn), abi.MATH_BF16,
                                          abi.ptr(out), abi.ptr(ws), T, L, I, E, top_k, None) == 0
        return len(np.unique(ids))

    for i in range(warmup):
        step(i)
    t0 = time.perf_counter()
    for i in range(steps):
        touched.append(step(warmup + i))
    dt = time.perf_counter() - t0
    del keep_gu, keep_dn
    return per_expert * sum(touched) / dt / 1e12, dt / steps * 1e3, os.cpu_count() or 1, \
        f"{steps} steps of the full workload (route + experts, {sum(touched) / len(touched):.1f} experts touched per step) after {warmup} warm-up steps"


def cpu_leg(name, steps, warmup):
    if cpu_library() is None:
        return {"value": None, "unit": "TB/s", "cores": os.cpu_count(), "kind": "reference", "sample": "oracle/_ref/libdromos_cpu.so not built"}, None
    try:
        tbs, ms, cores, sample = (cpu_moe if name in MOE else cpu_dense)(name, steps, warmup)
    except Exception as exc:  # a reported baseline: its failure is recorded beside the GPU numbers, which stay valid
        return {"value": None, "unit": "TB/s", "cores": os.cpu_count(), "kind": "reference", "sample": f"failed: {type(exc).__name__}: {exc}"[:200]}, None
    return {"value": tbs, "unit": "TB/s", "cores": cores, "kind": "reference", "sample": sample}, ms


# ---------------------------------------------------------------------------------------------------------------------
# GPU legs
# ---------------------------------------------------------------------------------------------------------------------


class Gpu:
    """Process-wide state of the GPU arm: library, device, process group, timing helpers."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.lib = abi.Library()  # raises when the CUDA library is missing: there is no other path
        self.graphs = []
        self.use_graphs = os.environ.get("LX_BENCH_GRAPHS", "1") != "0"

    def capture(self, fn):
        g = self.torch.cuda.CUDAGraph()
        with self.torch.cuda.graph(g):
            fn()
        self.graphs.append(g)
        return g

    def timed(self, fn, n):
        """n calls of fn between two events on the current stream, after a barrier; the slowest rank's milliseconds."""
        torch = self.torch
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def replayer(self, fn, period):
        """fn(i) for i in range(period), captured as graphs; run(i) replays graph i % period. Also how many kernels of
        this library one pass over the period launches."""
        for i in range(period):  # every allocation (workspaces, the status word) happens before capture
            fn(i)
        self.torch.cuda.synchronize()
        before = self.lib.lx_b200_kernel_launches()
        if not self.use_graphs:
            for i in range(period):
                fn(i)
            return fn, self.lib.lx_b200_kernel_launches() - before
        graphs = [self.capture(lambda i=i: fn(i)) for i in range(period)]
        return (lambda i: graphs[i % period].replay()), self.lib.lx_b200_kernel_launches() - before

    def timed_steps(self, step, steps, warmup, period):
        """`warmup` untimed steps, then exactly `steps` steps as ONE replayed graph between events (the reference's own
        method: every launch of the timed region in one graph, bench/bench_gemv.py:74-119). Returns (ms, launches, run)."""
        run, launches_per_period = self.replayer(step, period)
        for i in range(warmup):
            run(i)
        whole = self.capture(lambda: [step(warmup + i) for i in range(steps)]) if self.use_graphs else None
        if whole is not None:
            whole.replay()  # once untimed: the graph's own first-launch cost
            ms = self.timed(lambda i: whole.replay(), 1)
            again = whole.replay
        else:
            ms = self.timed(lambda i: run(warmup + i), steps)
            again = lambda: [run(i) for i in range(steps)]
        return ms, launches_per_period * steps // period, again

    def leave(self):
        """Graphs that hold NCCL kernels must be gone before the communicator is: release them, meet, then leave the
        process without running NCCL's destructors (which can wait for ever on a communicator a graph once captured)."""
        self.torch.cuda.synchronize()
        for g in self.graphs:
            g.reset()
        self.graphs.clear()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)


def hold_load(G, again, once_ms, seconds=0.6):
    """The timed steps last a few milliseconds, less than one nvidia-smi sample: the same work is repeated (untimed) for a
    moment while the clock sampler still runs, so that the clocks it reports are clocks under this load. The repetition
    count comes from the measured time (the same on every rank, so exchanges inside stay matched)."""
    for _ in range(max(1, min(2000, int(seconds * 1e3 / max(once_ms, 1e-3))))):
        again()
    G.torch.cuda.synchronize()


def dense_leg(G, name, steps, warmup, scaling, peaks, sampler=None, parity=False):
    """One dense workload on the GPU(s). scaling: 'single', 'strong' (the configuration's rows split over the ranks) or
    'weak' (a configuration-sized shard per rank). Returns the per-config record (rank 0's view, times max over ranks)."""
    from dromos_b200 import host

    torch, dist, lib, dev, world, rank = G.torch, G.dist, G.lib, G.dev, G.world, G.rank
    wtype, N, K, Ms, _ = DENSE[name]
    N_job = N * world if scaling == "weak" else N
    n0, n1 = host.shard_rows(N_job, rank, world) if world > 1 else (0, N)
    rows = n1 - n0

    def shard_of(r):
        a, b = host.shard_rows(N_job, r, world) if world > 1 else (0, N)
        gen = torch.Generator(device=dev).manual_seed(1000 + r)
        return (torch.randn((b - a, K), generator=gen, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    first = host.store_weight(lib, shard_of(rank), wtype)
    shard_bytes = first.nbytes()
    copies = max(3, -(-ROTATE_BYTES // (shard_bytes * len(Ms))) * len(Ms))
    stored = [first] + [host.StoredWeight(wtype, first.data.clone(), None if first.scale is None else first.scale.clone(), first.glob,
                                          rows=first.rows, cols=first.cols) for _ in range(copies - 1)]
    gen = torch.Generator(device=dev).manual_seed(7)  # the activations are the same on every rank
    xs = {M: torch.randn((M, K), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16) for M in Ms}
    total_step_bytes = torch.tensor([float(shard_bytes * len(Ms))], device=dev)
    if world > 1:
        dist.all_reduce(total_step_bytes)
    total_step_bytes = float(total_step_bytes.item())

    exchange, layers, gathered = "none", None, None
    local = [host.Linear(lib, s, rows, K) for s in stored]
    ys = {M: torch.empty((M, rows), dtype=torch.float32, device=dev) for M in Ms}
    if world > 1:
        if os.environ.get("LX_BENCH_EXCHANGE", "peer") == "peer":
            try:
                buffers = host.PeerBuffers(N_job, max(Ms), dev)
                layers = [host.PeerShardedLinear(lib, s, N_job, K, buffers) for s in stored]
                exchange = "one kernel over peer memory: lx_b200_exchange_packets (flag-in-data packets) for small slices, lx_b200_exchange_slices (stores + semaphore) for large"
            except Exception as e:
                print(f"[bench] peer exchange unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
                layers = None
            ok = torch.tensor([1 if layers is not None else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # every rank takes the same path
            if int(ok.item()) == 0:
                layers = None
        if layers is None:
            exchange = "NCCL all-gather"
            gathered = {M: torch.empty((world, M, rows), dtype=torch.float32, device=dev) for M in Ms}

    def product(c, M, x=None):
        """The workload's product on weight copy c: this rank's whole y [M, N_job] (valid on the stream)."""
        x = xs[M] if x is None else x
        if world == 1:
            return local[c](x, ys[M])
        if layers is not None:
            return layers[c](x)
        local[c](x, ys[M])
        dist.all_gather_into_tensor(gathered[M].view(world * M, rows), ys[M])
        return gathered[M].permute(1, 0, 2).reshape(M, -1)

    def step(i):
        for j, M in enumerate(Ms):
            product((i * len(Ms) + j) % copies, M)

    period = copies // len(Ms)
    if sampler is not None:
        with sampler:
            ms, launches, again = G.timed_steps(step, steps, warmup, period)
            hold_load(G, again, ms)
    else:
        ms, launches, again = G.timed_steps(step, steps, warmup, period)
    value = total_step_bytes * steps / (ms * 1e-3) / 1e12

    # ---- the product kernels alone, per M (no exchange): one graph holds a pass over every weight copy ----
    per_m, k_bytes, k_ms = {}, 0.0, 0.0
    reps = max(2, min(20, int(4e9 // (shard_bytes * copies))))
    peak, peak_kind, read_only = peaks
    for M in Ms:
        def sweep(_, M=M):
            for c in range(copies):
                local[c](xs[M], ys[M])
        run_sweep, _ = G.replayer(sweep, 1)
        for i in range(2):
            run_sweep(i)
        t = G.timed(run_sweep, reps) / (reps * copies)
        gbs = shard_bytes / (t * 1e-3) / 1e9
        per_m[str(M)] = {"us": t * 1e3, "GB/s": gbs, "frac": gbs / peak}
        k_bytes += shard_bytes
        k_ms += t
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    reference_cuda = None
    if getattr(G, "refcuda", None) is not None and world == 1:  # the same sweep on the reference's own CUDA kernels
        theirs = [host.Linear(G.refcuda, s_, rows, K) for s_ in stored]
        ref_m, ref_ms = {}, 0.0
        for M in Ms:
            def ref_sweep(_, M=M):
                for c in range(copies):
                    theirs[c](xs[M], ys[M])
            run_ref, _ = G.replayer(ref_sweep, 1)
            for i in range(2):
                run_ref(i)
            t = G.timed(run_ref, reps) / (reps * copies)
            ref_m[str(M)] = {"us": t * 1e3, "GB/s": shard_bytes / (t * 1e-3) / 1e9, "speedup_of_this_library": t * 1e3 / per_m[str(M)]["us"]}
            ref_ms += t
        reference_cuda = {"kind": "the reference's engine/cuda compiled unmodified for architecture 100 (its kernels of the 80 / 89 / 90 families)",
                          "per_m": ref_m, "GB/s": k_bytes / (ref_ms * 1e-3) / 1e9, "speedup_of_this_library": ref_ms / k_ms}
        del theirs
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC.get(name) if world == 1 else None, "peak_source": f"{peak_kind} copy bandwidth (burst)",
                "read_only_peak": read_only, "frac_of_read_only": achieved / read_only if read_only else None,
                "kernel": KERNELS[name], "per_m": per_m, "algorithmic_bytes_per_launch": shard_bytes,
                "achieved_is": "weight + scale bytes of one launch / mean launch time of the product kernels over the workload's M, CUDA events"}

    # ---- end to end through the host-buffer API: pinned activations in, outputs out, every step ----
    xh = {M: xs[M].cpu().pin_memory() for M in Ms}
    yh = {M: torch.empty((M, rows if world > 1 else N), dtype=torch.float32).pin_memory() for M in Ms}
    xd = {M: torch.empty_like(xs[M]) for M in Ms}
    copy_stream = torch.cuda.Stream()

    def e2e_work(i):
        # The device-to-host copy of a product's outputs runs on a second stream under the next product of the step
        # (largest outputs first); with several ranks each rank brings home its own columns of the whole y.
        main = torch.cuda.current_stream()
        for j, M in sorted(enumerate(Ms), key=lambda jm: -jm[1]):
            xd[M].copy_(xh[M], non_blocking=True)
            y = product((i * len(Ms) + j) % copies, M, xd[M])
            src = y[:, n0:n1] if world > 1 else y
            copy_stream.wait_stream(main)
            with torch.cuda.stream(copy_stream):
                yh[M].copy_(src, non_blocking=True)
        main.wait_stream(copy_stream)

    run_e2e, _ = G.replayer(e2e_work, period)

    def e2e_step(i):
        run_e2e(i)
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step

    for i in range(3):
        e2e_step(i)
    e2e_steps = min(steps, 20)
    e2e_ms = G.timed(e2e_step, e2e_steps)
    e2e = {"value": total_step_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s",
           "h2d_bytes_per_step": sum(M * K * 2 for M in Ms), "d2h_bytes_per_step": sum(M * rows * 4 for M in Ms)}

    out = {"workload": DENSE[name][-1], "scaling": scaling, "value": value, "unit": "TB/s", "ms_per_step": ms / steps, "steps": steps,
           "pct_of_8TBs": value / 8.0 / max(world, 1) * 100.0, "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches),
           "exchange": exchange, "dtype": DTYPE[wtype]}
    if reference_cuda is not None:
        out["reference_cuda"] = reference_cuda

    # ---- correctness of what the exchange delivered: a peer's slice, recomputed here from the peer's seed ----
    if parity and world > 1:
        peer = (rank + 1) % world
        p0, p1 = host.shard_rows(N_job, peer, world)
        pl = host.Linear(lib, host.store_weight(lib, shard_of(peer), wtype), p1 - p0, K)
        bad, cols = 0, 0
        for M in Ms:
            whole = product(0, M).clone()  # copy 0 holds what every rank drew from its seed
            mine = torch.empty((M, p1 - p0), dtype=torch.float32, device=dev)
            pl(xs[M], mine)
            torch.cuda.synchronize()
            bad += int((whole[:, p0:p1].view(torch.int32) != mine.view(torch.int32)).sum().item())
            cols += (p1 - p0) * M
        verdict = torch.tensor([bad, cols], device=dev, dtype=torch.int64)
        dist.all_reduce(verdict)
        out["parity_check"] = {"ok": int(verdict[0].item()) == 0, "columns": int(verdict[1].item()), "mismatches": int(verdict[0].item()),
                               "how": "every rank recomputes its neighbour's rows (weights redrawn from the neighbour's seed) with its own kernel and compares the outputs bit for bit with what arrived"}
    del stored, local, layers
    torch.cuda.empty_cache()
    return out


def moe_leg(G, name, steps, warmup, peaks):
    """The routed-experts workload: a step is lx_moe_route + lx_moe_experts_grouped on T tokens with fresh logits and the
    next copy of the expert stacks. Bytes of a step = weights and scales of the experts the step's routing touches (the
    reference's accounting, model/traffic.cpp:23-58). With several ranks the experts are split over the ranks."""
    from dromos_b200 import host

    torch, dist, lib, dev, world, rank = G.torch, G.dist, G.lib, G.dev, G.world, G.rank
    wtype, E, top_k, L, I, T, desc = MOE[name]
    e0, e1 = host.expert_range(E, rank, world)
    gen = torch.Generator(device=dev).manual_seed(0)  # the same stacks, tokens and logits on every rank
    per_expert = (2 * I * L + L * I) + 4 * (2 * I + L)  # bytes of one expert: both stacks and their row scales
    local_bytes = per_expert * (e1 - e0)
    copies = max(2, -(-ROTATE_BYTES // local_bytes) + 1)
    whole_gu = host.store_weight(lib, (torch.randn((E, 2 * I, L), generator=gen, device=dev) * 0.02).to(torch.bfloat16), wtype)
    whole_dn = host.store_weight(lib, (torch.randn((E, L, I), generator=gen, device=dev) * 0.02).to(torch.bfloat16), wtype)

    def own_slice(s, rows_per, cols):  # this rank's experts of a stored stack (row-wise formats: the rows and their scales)
        data = s.data.view(E, -1)[e0:e1].contiguous().view(-1)
        scale = None if s.scale is None else s.scale.view(E, -1)[e0:e1].contiguous().view(-1)
        return host.StoredWeight(wtype, data, scale, s.glob, rows=(e1 - e0) * rows_per, cols=cols)

    stacks = [(own_slice(whole_gu, 2 * I, L), own_slice(whole_dn, L, I)) if world > 1 else (whole_gu, whole_dn)]
    for c in range(1, copies):
        g0, d0 = stacks[0]
        stacks.append((host.StoredWeight(wtype, g0.data.clone(), None if g0.scale is None else g0.scale.clone(), g0.glob, rows=g0.rows, cols=L),
                       host.StoredWeight(wtype, d0.data.clone(), None if d0.scale is None else d0.scale.clone(), d0.glob, rows=d0.rows, cols=I)))
    t0, t1 = T * rank // world, T * (rank + 1) // world  # the tokens whose outputs this rank hands back end to end
    periods = 8  # distinct routings
    logits = [torch.randn((T, E), generator=torch.Generator(device=dev).manual_seed(100 + i), device=dev) for i in range(periods)]
    latent = torch.randn((T, L), generator=gen, device=dev).to(torch.bfloat16)
    if world == 1:
        engines = [host.Experts(lib, gu, dn, E, L, I, top_k) for gu, dn in stacks]
    else:  # routing and tokens replicated, each rank its own experts, the weighted rows exchanged as packets over peer memory
        engines = [host.ReplicatedExpertParallel(lib, gu, dn, E, L, I, top_k, T, dev) for gu, dn in stacks]
    router = host.Experts(lib, whole_gu, whole_dn, E, L, I, top_k)
    out = torch.empty((T, L), dtype=torch.float32, device=dev)
    touched = [int(torch.unique(torch.topk(lg, top_k, dim=1).indices).numel()) for lg in logits]  # experts each routing touches, whole job

    def step(i):
        ids, w = router.route(logits[i % periods])
        engines[i % copies](latent, ids, w, out)

    parity = None
    if world > 1:  # every rank holds the whole stacks once: the split result must be one GPU's, bit for bit
        ids, w = router.route(logits[0])
        want = router(latent, ids, w)
        got = engines[0](latent, ids, w, out)
        torch.cuda.synchronize()
        bad = int((got.view(torch.int32) != want.view(torch.int32)).sum().item())
        flag = torch.tensor([bad], device=dev)
        dist.all_reduce(flag)
        parity = {"ok": int(flag.item()) == 0, "columns": T * L, "mismatches": int(flag.item()),
                  "how": "every rank also runs lx_moe_experts_grouped on the whole stacks and compares its split result bit for bit"}
    if world == 1:
        del whole_gu, whole_dn
    ms, launches, _ = G.timed_steps(step, steps, warmup, periods * copies)
    step_bytes = [per_expert * touched[(warmup + i) % periods] for i in range(steps)]
    value = sum(step_bytes) / (ms * 1e-3) / 1e12
    peak, peak_kind, read_only = peaks
    achieved = sum(step_bytes) / (ms * 1e-3) / 1e9 / world
    # end to end: logits and latent from pinned host memory in, the tokens' outputs out, every step
    lh = [x.cpu().pin_memory() for x in logits]
    xh = latent.cpu().pin_memory()
    oh = torch.empty((t1 - t0, L), dtype=torch.float32).pin_memory()
    ld, xd = torch.empty_like(logits[0]), torch.empty_like(latent)

    def e2e_step(i):
        ld.copy_(lh[i % periods], non_blocking=True)
        xd.copy_(xh, non_blocking=True)
        ids, w = router.route(ld)
        engines[i % copies](xd, ids, w, out)
        oh.copy_(out[t0:t1], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    e2e_steps = min(steps, 20)
    e2e_ms = G.timed(e2e_step, e2e_steps)
    e2e_bytes = sum(per_expert * touched[i % periods] for i in range(e2e_steps))
    rec = {"workload": desc, "scaling": "single" if world == 1 else "strong", "value": value, "unit": "TB/s", "ms_per_step": ms / steps, "steps": steps,
           "pct_of_8TBs": value / 8.0 / max(world, 1) * 100.0,
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(name),
                        "peak_source": f"{peak_kind} copy bandwidth (burst)", "read_only_peak": read_only,
                        "frac_of_read_only": achieved / read_only if read_only else None, "kernel": KERNELS[name],
                        "algorithmic_bytes_per_launch": sum(step_bytes) / len(step_bytes),
                        "achieved_is": "bytes of the experts a step's routing touches / step time (all kernels of the step), CUDA events"},
           "e2e": {"value": e2e_bytes / (e2e_ms * 1e-3) / 1e12, "unit": "TB/s", "h2d_bytes_per_step": T * (E * 4 + L * 2),
                   "d2h_bytes_per_step": (t1 - t0) * L * 4},
           "gpu_launches": int(launches),
           "exchange": "none" if world == 1 else "lx_b200_moe_exchange_rows (routing and tokens replicated; weighted rows as flag-in-data packets over peer memory)",
           "dtype": DTYPE[wtype]}
    if parity is not None:
        rec["parity_check"] = parity
    if getattr(G, "refcuda", None) is not None and world == 1:
        theirs = [host.Experts(G.refcuda, gu, dn, E, L, I, top_k) for gu, dn in stacks]
        their_router = host.Experts(G.refcuda, stacks[0][0], stacks[0][1], E, L, I, top_k)

        def ref_step(i):
            ids, w = their_router.route(logits[i % periods])
            theirs[i % copies](latent, ids, w, out)

        ref_ms, _, _ = G.timed_steps(ref_step, steps, warmup, periods * copies)
        rec["reference_cuda"] = {"kind": "the reference's engine/cuda compiled unmodified for architecture 100", "ms_per_step": ref_ms / steps,
                                 "value": sum(step_bytes) / (ref_ms * 1e-3) / 1e12, "speedup_of_this_library": ref_ms / ms}
        del theirs, their_router
    del stacks, engines
    torch.cuda.empty_cache()
    return rec


def read_only_ceiling(G):
    """The read-only DRAM bandwidth of this GPU, measured now (lx_bandwidth_probe: 16-byte loads over a 4 GiB buffer)."""
    read, spec = ctypes.c_double(0.0), ctypes.c_double(0.0)
    st = G.lib.lx_bandwidth_probe(4 << 30, 5, ctypes.byref(read), ctypes.byref(spec), ctypes.c_void_p(G.torch.cuda.current_stream().cuda_stream))
    G.torch.cuda.synchronize()
    return float(read.value) if st == 0 and read.value > 0 else None


# ---------------------------------------------------------------------------------------------------------------------


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="", help="comma-separated workloads to time besides the headline (default: all six)")
    ap.add_argument("--reference-cuda", action="store_true", help="also time the reference's own CUDA kernels (oracle/_ref/libdromos_kernels_ref.so) on every workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    names = [n for n in ORDER if not args.only or n in args.only.split(",") or n == HEADLINE]
    side_steps = max(3, min(args.steps, 20))
    exchange_name = "none" if world == 1 else None

    if args.impl == "reference":
        # The reference's own CPU backend on the host cores, rank 0 only: the same workloads, the same steps and warm-up.
        if rank != 0:
            return
        if cpu_library() is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libdromos_cpu.so is not built (make -C oracle ref)"}))
            return
        per_config = {}
        for n in names:
            st = args.steps if n == HEADLINE else max(2, min(side_steps, 5))
            leg, ms = cpu_leg(n, st, args.warmup if n == HEADLINE else 2)
            per_config[n] = {"workload": (DENSE.get(n) or MOE.get(n))[-1], "value": leg["value"], "unit": "TB/s", "ms_per_step": ms, "cpu_baseline": leg}
        head = per_config[HEADLINE]
        exch = "none" if world == 1 else os.environ.get("LX_BENCH_EXCHANGE_NAME", "one kernel over peer memory: lx_b200_exchange_packets (flag-in-data packets) for small slices, lx_b200_exchange_slices (stores + semaphore) for large")
        print(json.dumps({"impl": "reference", "metric": METRIC, "value": head["value"], "unit": "TB/s", "n_gpus": args.gpus, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": DTYPE[DENSE[HEADLINE][0]], "data": "synthetic",
                          "config": config_of(HEADLINE, world, "strong", exch), "cpu_baseline": head["cpu_baseline"],
                          "e2e": {"value": head["value"], "unit": "TB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                          "per_config": per_config}))
        return

    G = Gpu()
    G.refcuda = reference_cuda_library() if args.reference_cuda else None
    peak, peak_kind = measured_peak_gbs()
    read_only = read_only_ceiling(G)
    peaks = (peak, peak_kind, read_only)
    per_config = {}
    sampler = ClockSampler(G.local)
    scaling = "single" if world == 1 else "strong"
    head = dense_leg(G, HEADLINE, args.steps, args.warmup, scaling, peaks, sampler=sampler, parity=True)
    for n in names:
        if n == HEADLINE:
            per_config[n] = head
        elif n in MOE:
            per_config[n] = moe_leg(G, n, side_steps, 3, peaks)
        elif world == 1:
            per_config[n] = dense_leg(G, n, side_steps, 3, "single", peaks)
        elif n == "c3_nvfp4":
            per_config[n] = dense_leg(G, n, side_steps, 3, "strong", peaks, parity=True)
        elif n == "c2_int8":
            per_config[n + "_weak"] = dense_leg(G, n, side_steps, 3, "weak", peaks, parity=True)
        # (the two single-row GEMV workloads are single-GPU configurations: they are timed at N = 1 only)
    status = G.lib.lx_b200_last_error()
    parity_ok = all(v.get("parity_check", {}).get("ok", True) for v in per_config.values())
    if rank != 0:
        G.leave()
        if not parity_ok:
            sys.exit(3)
        return
    if world == 1:  # the reference's CPU backend beside every workload (bounded samples: the whole run stays within minutes)
        for n in names:
            per_config[n]["cpu_baseline"], _ = cpu_leg(n, 5 if n != HEADLINE else 8, 2)
    line = {"metric": METRIC, "value": head["value"], "unit": "TB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": head["dtype"], "data": "synthetic", "config": config_of(HEADLINE, world, "strong", head["exchange"]), "roofline": head["roofline"],
            "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "launch": "CUDA graphs" if G.use_graphs else "eager", "clocks": sampler.summary(),
            "pct_of_8TBs": head["pct_of_8TBs"], "kernel_status": status, "per_config": per_config}
    if world == 1:
        line["cpu_baseline"] = head["cpu_baseline"]
    else:
        line["parity_check"] = {"ok": parity_ok, "columns": sum(v.get("parity_check", {}).get("columns", 0) for v in per_config.values())}
    print(json.dumps(line), flush=True)
    G.leave()
    if not parity_ok:
        sys.exit(3)


if __name__ == "__main__":
    main()
