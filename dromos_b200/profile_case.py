"""One product shape, launched a few times on rotating weight copies: the small, fixed case to put under a profiler or to
time quickly.

    python -m dromos_b200.profile_case FORMAT N K M [launches] [copies]     a dense product (lx_gemv_w for M <= 8, else lx_gemm_w)
    python -m dromos_b200.profile_case moe FORMAT E TOP_K L I T [launches]  route + routed experts (lx_moe_experts_grouped)

FORMAT is bf16, int8, fp8, nvfp4 or bf16x. The launches run one by one on the current stream first (what a profiler
captures: name the kernel with its own filter, e.g. ncu -k regex:gemv_kernel -c 2), then once more as a replayed graph
between CUDA events, and the time per launch of that replay is printed. `copies` weight copies are used in turn so that a
launch reads its weights from DRAM when copies x weight bytes exceeds the L2 (126 MB).
"""

import sys

import torch

from dromos_b200 import abi, host

FORMATS = {"bf16": abi.W_BF16, "int8": abi.W_INT8, "fp8": abi.W_FP8, "nvfp4": abi.W_NVFP4, "bf16x": abi.W_BF16X}


def timed_graph(run, launches):
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            run(i)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / launches


def copies_of(s, n, cols):
    return [s] + [host.StoredWeight(s.wtype, s.data.clone(), None if s.scale is None else s.scale.clone(), s.glob, rows=s.rows, cols=cols)
                  for _ in range(n - 1)]


def dense(lib, argv):
    fmt, N, K, M = FORMATS[argv[0]], int(argv[1]), int(argv[2]), int(argv[3])
    launches = int(argv[4]) if len(argv) > 4 else 6
    copies = int(argv[5]) if len(argv) > 5 else 3
    g = torch.Generator(device="cuda").manual_seed(0)
    w = (torch.randn((N, K), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    layers = [host.Linear(lib, s, N, K) for s in copies_of(host.store_weight(lib, w, fmt), copies, K)]
    del w
    x = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    run = lambda i: layers[i % copies](x, y)
    for i in range(launches):
        run(i)
    us = timed_graph(run, launches)
    print(f"{argv[0]} N={N} K={K} M={M}: {us:.2f} us per product in a replayed graph, kernel status {lib.lx_b200_last_error()}")


def moe(lib, argv):
    fmt, E, top_k, L, I, T = FORMATS[argv[0]], *(int(a) for a in argv[1:6])
    launches = int(argv[6]) if len(argv) > 6 else 4
    g = torch.Generator(device="cuda").manual_seed(0)
    gu = host.store_weight(lib, (torch.randn((E, 2 * I, L), generator=g, device="cuda") * 0.02).to(torch.bfloat16), fmt)
    dn = host.store_weight(lib, (torch.randn((E, L, I), generator=g, device="cuda") * 0.02).to(torch.bfloat16), fmt)
    engines = [host.Experts(lib, a, b, E, L, I, top_k) for a, b in zip(copies_of(gu, 2, L), copies_of(dn, 2, I))]
    latent = torch.randn((T, L), generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), generator=g, device="cuda")
    out = torch.empty((T, L), dtype=torch.float32, device="cuda")

    def run(i):
        ids, w = engines[0].route(logits)
        engines[i % 2](latent, ids, w, out)

    for i in range(launches):
        run(i)
    us = timed_graph(run, launches)
    print(f"moe {argv[0]} E={E} top_k={top_k} L={L} I={I} T={T}: {us:.2f} us per step in a replayed graph, kernel status {lib.lx_b200_last_error()}")


def main(argv):
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    lib = abi.Library()
    if argv[0] == "moe":
        moe(lib, argv[1:])
    else:
        dense(lib, argv)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
