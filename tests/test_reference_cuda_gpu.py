"""The library against the reference project's OWN CUDA backend on the same inputs, on the GPU: the parity statement of the
path in its strongest form. oracle/_ref/libdromos_kernels_ref.so is the reference's engine/cuda compiled unmodified
(`make -C oracle cuda_ref`); where it is absent these tests skip (the CPU-backend and float64 checks still run).

Bit-exact: quantized weights and their scales (INT8, FP8, NVFP4), dequantized bf16 values, BF16X encodings and their
decoding, quantized activations, routing picks. Within the acceptance bound (rel-L2 <= 1e-3, max-abs <= 2e-2 of outputs of
order one; in practice both libraries agree to a few 1e-6): every product entry point on every format.
"""

import ctypes
import os

import numpy as np
import pytest
import torch

from dromos_b200 import abi, host
from tests import util

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_PATH = os.path.join(ROOT, "oracle", "_ref", "libdromos_kernels_ref.so")
FORMATS = {"bf16": abi.W_BF16, "int8": abi.W_INT8, "fp8": abi.W_FP8, "nvfp4": abi.W_NVFP4, "bf16x": abi.W_BF16X}


@pytest.fixture(scope="module")
def refcuda():
    if not os.path.exists(REF_PATH):
        pytest.skip("oracle/_ref/libdromos_kernels_ref.so not built (make -C oracle cuda_ref needs the reference checkout)")
    return abi.Library(REF_PATH)


def bf16(shape, std, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * std).to(torch.bfloat16)


def close(got, want, what):
    got, want = got.double(), want.double()
    rel = float((got - want).norm() / want.norm().clamp_min(1e-30))
    worst = float((got - want).abs().max())
    assert torch.isfinite(got).all() and rel <= 1e-3 and worst <= 2e-2 * max(1.0, float(want.abs().max())), f"{what}: rel-L2 {rel:.3e}, max-abs {worst:.3e}"


@pytest.mark.parametrize("name", ["int8", "fp8", "nvfp4", "bf16x"])
def test_stored_weights_are_the_same_bytes(lx, refcuda, name):
    rows, K = 300, 2048
    w = bf16((rows, K), 0.02, 3)
    w[7] = 0
    w[9, 5] = 1e-30  # a patch for BF16X, a tiny value for the quantizers
    a, b = host.store_weight(lx, w, FORMATS[name]), host.store_weight(refcuda, w, FORMATS[name])
    assert torch.equal(a.data, b.data), "stored bytes differ"
    if a.scale is not None:
        assert torch.equal(a.scale.view(torch.uint8), b.scale.view(torch.uint8)), "scales differ"
        assert np.float32(a.glob).tobytes() == np.float32(b.glob).tobytes(), "global scale differs"
    # and both libraries give back the same bf16 values from them
    outs = []
    for lib in (lx, refcuda):
        out = torch.zeros((rows, K), dtype=torch.bfloat16, device="cuda")
        if name == "bf16x":
            assert lib.lx_bf16x_decode(abi.ptr(a.data), rows, K, abi.ptr(out), util.stream_ptr()) == 0
        else:
            assert lib.lx_dequantize_weight(a.ref(), abi.ptr(out), rows, K, util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append(out)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    if name == "bf16x":
        assert torch.equal(outs[0].view(torch.int16), w.view(torch.int16)), "the lossless format lost bits"


@pytest.mark.parametrize("math", [abi.MATH_INT8, abi.MATH_FP8, abi.MATH_FP4], ids=["int8", "fp8", "fp4"])
def test_quantized_activations_are_the_same_bytes(lx, refcuda, math):
    M, K = 7, 1536
    x = bf16((M, K), 1.0, 5)
    x[3] = 0
    outs = []
    for lib in (lx, refcuda):
        q = torch.zeros((M, K), dtype=torch.uint8, device="cuda")
        s = torch.zeros(M, dtype=torch.float32, device="cuda")
        bs = torch.zeros((M, K // 16), dtype=torch.uint8, device="cuda")
        ld_q = K // 2 if math == abi.MATH_FP4 else K
        assert lib.lx_quantize_act(abi.ptr(x), abi.BF16, K, math, abi.ptr(q), ld_q, abi.ptr(s), abi.ptr(bs), K // 16, M, K, util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append((q, s, bs))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_routing_picks_are_the_same(lx, refcuda):
    T, E, top_k = 40, 64, 8
    logits = torch.randn((T, E), generator=torch.Generator(device="cuda").manual_seed(6), device="cuda")
    bias = torch.randn(E, generator=torch.Generator(device="cuda").manual_seed(7), device="cuda") * 0.1
    outs = []
    for lib in (lx, refcuda):
        ids = torch.zeros((T, top_k), dtype=torch.int32, device="cuda")
        w, ent, conf = torch.zeros((T, top_k), device="cuda"), torch.zeros(T, device="cuda"), torch.zeros(T, device="cuda")
        assert lib.lx_moe_route(abi.ptr(logits), abi.ptr(bias), abi.ptr(ids), abi.ptr(w), abi.ptr(ent), abi.ptr(conf), T, E, top_k, util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append((ids, w, ent, conf))
    assert torch.equal(outs[0][0], outs[1][0]), "picks differ"
    for a, b in zip(outs[0][1:], outs[1][1:]):
        assert float((a - b).abs().max()) <= 1e-5


@pytest.mark.parametrize("name", list(FORMATS))
@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(1000, 2048), (520, 4096)])
def test_decode_gemv_agrees(lx, refcuda, name, M, N, K):
    stored = host.store_weight(lx, bf16((N, K), 0.02, N + K), FORMATS[name])
    x = bf16((M, K), 1.0, M)
    bias = bf16((N,), 0.5, 9)
    outs = []
    for lib in (lx, refcuda):
        y = torch.full((M, N), 0.25, device="cuda")
        assert lib.lx_gemv_w(abi.ptr(x), abi.BF16, K, stored.ref(), abi.ptr(bias), abi.BF16, abi.ptr(y), abi.F32, N, M, N, K, 0.5, 2.0, util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append(y)
    close(outs[0], outs[1], f"lx_gemv_w {name} M={M}")
    util.check_status(lx)


@pytest.mark.parametrize("name,math", [("bf16", abi.MATH_BF16), ("int8", abi.MATH_BF16), ("fp8", abi.MATH_BF16), ("nvfp4", abi.MATH_BF16),
                                       ("int8", abi.MATH_INT8), ("fp8", abi.MATH_FP8)], ids=["bf16", "w8a16_int8", "w8a16_fp8", "w4a16", "int8", "fp8"])
@pytest.mark.parametrize("M", [16, 70])
def test_gemm_w_agrees(lx, refcuda, name, math, M):
    N, K = 776, 2048
    stored = host.store_weight(lx, bf16((N, K), 0.02, 11), FORMATS[name])
    x = bf16((M, K), 1.0, 12)
    bias = torch.randn(N, generator=torch.Generator(device="cuda").manual_seed(13), device="cuda")
    outs = []
    for lib in (lx, refcuda):
        y = torch.full((M, N), float("nan"), device="cuda")
        ws = torch.zeros(max(256, lib.lx_gemm_workspace_bytes(M, K, math)), dtype=torch.uint8, device="cuda")
        assert lib.lx_gemm_w(abi.ptr(x), abi.BF16, K, stored.ref(), math, abi.ptr(bias), abi.F32, abi.ptr(y), abi.F32, N, M, N, K, 1.0, 0.0, abi.ptr(ws),
                             util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append(y)
    close(outs[0], outs[1], f"lx_gemm_w {name} math {math} M={M}")
    util.check_status(lx)


@pytest.mark.parametrize("name,math", [("bf16", abi.MATH_BF16), ("fp8", abi.MATH_BF16), ("int8", abi.MATH_BF16), ("fp8", abi.MATH_FP8), ("int8", abi.MATH_INT8)],
                         ids=["bf16", "w8a16_fp8", "w8a16_int8", "fp8", "int8"])
def test_grouped_experts_agree(lx, refcuda, name, math):
    T, L, I, E, top_k = 24, 512, 384, 16, 4
    gu = host.store_weight(lx, bf16((E, 2 * I, L), 1.0 / L**0.5, 21), FORMATS[name])
    dn = host.store_weight(lx, bf16((E, L, I), 1.0 / I**0.5, 22), FORMATS[name])
    latent = bf16((T, L), 1.0, 23)
    ids, weights = host.Experts(lx, gu, dn, E, L, I, top_k).route(torch.randn((T, E), generator=torch.Generator(device="cuda").manual_seed(24), device="cuda"))
    outs = []
    for lib in (lx, refcuda):
        out = torch.full((T, L), float("nan"), device="cuda")
        ws = torch.zeros(max(256, lib.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, math)), dtype=torch.uint8, device="cuda")
        assert lib.lx_moe_experts_grouped(abi.ptr(latent), abi.ptr(ids), abi.ptr(weights), gu.ref(), dn.ref(), math, abi.ptr(out), abi.ptr(ws), T, L, I, E, top_k,
                                          util.stream_ptr()) == 0
        torch.cuda.synchronize()
        outs.append(out)
    # experts: 2e-3 of the largest output (8e-3 under FP8 math, where a tipped e4m3 rounding of an intermediate moves a row): the reference suite's own bound
    tol = (8e-3 if math == abi.MATH_FP8 else 2e-3) * float(outs[1].abs().max())
    assert torch.isfinite(outs[0]).all() and float((outs[0] - outs[1]).abs().max()) <= tol
    util.check_status(lx)


def test_bf16x_gemv_equals_bf16_gemv_in_both_libraries(lx, refcuda):
    """The lossless format's product is the bf16 product bit for bit, in the reference and here (each library against itself:
    the two libraries add in different orders)."""
    N, K, M = 640, 4096, 4
    w = bf16((N, K), 0.02, 31)
    x = bf16((M, K), 1.0, 32)
    for lib in (lx, refcuda):
        plain, packed = host.store_weight(lib, w, abi.W_BF16), host.store_weight(lib, w, abi.W_BF16X)
        ys = []
        for s in (plain, packed):
            y = torch.full((M, N), float("nan"), device="cuda")
            assert lib.lx_gemv_w(abi.ptr(x), abi.BF16, K, s.ref(), None, abi.BF16, abi.ptr(y), abi.F32, N, M, N, K, 1.0, 0.0, util.stream_ptr()) == 0
            torch.cuda.synchronize()
            ys.append(y)
        assert torch.equal(ys[0].view(torch.int32), ys[1].view(torch.int32))
