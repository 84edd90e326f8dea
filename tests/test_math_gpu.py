"""The low-precision maths of lx_gemm_w and lx_moe_experts_grouped: INT8 weights x per-token int8 activations
(LX_MATH_INT8) and FP8 weights x per-token e4m3 activations (LX_MATH_FP8), and which (math, format, architecture)
combinations answer "not supported".

Mirrors the reference's tests/kernels/test_gemm_w.py (PAIRS, arch override, 2e-4 of the largest output) and
test_moe_grouped.py (2e-3 under INT8 math, 8e-3 under FP8 math, where one tipped e4m3 rounding of an intermediate moves
its token's row).
"""

import ctypes

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu
NOT_SUPPORTED, INVALID = 801, 1
QUANT = [(O.W_INT8, abi.MATH_INT8, "int8"), (O.W_FP8, abi.MATH_FP8, "fp8")]


def gemm_w(lx, x, x_dtype, wt, math, M, N, K, bias=None, alpha=1.0, beta=0.0, y0=None, workspace=True):
    dw = util.DeviceWeight(wt)
    x_dev = util.dev(x)
    y = torch.full((M, N), float("nan"), device="cuda") if y0 is None else util.dev(y0)
    ws = torch.full((max(1, lx.lx_gemm_workspace_bytes(M, K, math)),), 0xFF, dtype=torch.uint8, device="cuda") if workspace else None
    bias_dev = None if bias is None else util.dev(bias)
    st = lx.lx_gemm_w(abi.ptr(x_dev), x_dtype, K, dw.ref(), math, abi.ptr(bias_dev), abi.F32, abi.ptr(y), abi.F32, N, M, N, K, alpha, beta,
                      abi.ptr(ws), util.stream_ptr())
    torch.cuda.synchronize()
    return st, util.host(y)


@pytest.mark.parametrize("wtype,math,name", QUANT, ids=[q[2] for q in QUANT])
@pytest.mark.parametrize("shape", [(1, 264, 1024), (8, 1000, 2304), (33, 520, 4096), (64, 9605, 1040), (100, 300, 528)],
                         ids=lambda s: f"M{s[0]}N{s[1]}K{s[2]}")
@pytest.mark.parametrize("x_f32", [False, True], ids=["xbf16", "xf32"])
def test_gemm_w_quantized_math(lx, wtype, math, name, shape, x_f32):
    """Against float64 on the operands the math sees (the per-token quantization of the oracle, which the activation
    quantizer's own test pins bit for bit): what is left is the f32 epilogue, so 2e-4 of the largest output."""
    M, N, K = shape
    wt = util.make_weight(util.bf16_normal((N, K), 0.02, 5 + M), wtype)
    x = util.f32_normal((M, K), 1.0, 6 + M) if x_f32 else util.bf16_normal((M, K), 1.0, 6 + M)
    xf = x if x_f32 else O.bf16_bits_to_f32(x)
    bias = util.f32_normal((N,), 0.5, 7)
    y0 = util.f32_normal((M, N), 1.0, 8)
    st, got = gemm_w(lx, x, abi.F32 if x_f32 else abi.BF16, wt, math, M, N, K, bias=bias, alpha=0.5, beta=0.25, y0=y0)
    assert st == 0, st
    util.check_status(lx)
    want = 0.5 * (O.product_f64(O.act_operand(xf, math), wt) + bias.astype(np.float64)[None, :]) + 0.25 * y0.astype(np.float64)
    tol = 2e-4 * np.abs(want).max()
    assert np.all(np.isfinite(got)) and np.abs(got - want).max() <= tol, f"{name} {shape}: {np.abs(got - want).max():.3e} > {tol:.3e}"


@pytest.mark.parametrize("wtype,math,name", QUANT, ids=[q[2] for q in QUANT])
def test_quantized_rows_do_not_depend_on_batch_and_zero_rows(lx, wtype, math, name):
    """A row's bits are the same alone and in a batch of 70 (two passes); an all-zero row gives exactly the bias."""
    N, K = 520, 2048
    wt = util.make_weight(util.bf16_normal((N, K), 0.02, 41), wtype)
    x = util.bf16_normal((70, K), 1.0, 42)
    x[3] = 0
    bias = util.f32_normal((N,), 0.5, 43)
    st, big = gemm_w(lx, x, abi.BF16, wt, math, 70, N, K, bias=bias)
    assert st == 0
    assert np.array_equal(big[3], bias)
    for m in (0, 3, 64, 69):
        st, one = gemm_w(lx, x[m : m + 1], abi.BF16, wt, math, 1, N, K, bias=bias)
        assert st == 0 and np.array_equal(one[0].view(np.uint32), big[m].view(np.uint32)), f"{name}: row {m}"
    util.check_status(lx)


def test_pairs_and_architectures(lx):
    """The reference's table (engine/cuda/gemm_w.cuh:274-289) on a part of the 10x family: INT8 math needs INT8 weights,
    FP8 math FP8 weights and architecture 89; FP4 math and FP8 math on NVFP4 weights belong to the 12x family; below 80
    nothing runs. A quantized math without a workspace is an invalid call."""
    M, N, K = 16, 256, 512
    w_bits = util.bf16_normal((N, K), 0.02, 1)
    x = util.bf16_normal((M, K), 1.0, 2)
    weights = {t: util.make_weight(w_bits, t) for t in (O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4)}
    ok = {(abi.MATH_BF16, O.W_BF16), (abi.MATH_BF16, O.W_INT8), (abi.MATH_BF16, O.W_FP8), (abi.MATH_BF16, O.W_NVFP4),
          (abi.MATH_INT8, O.W_INT8), (abi.MATH_FP8, O.W_FP8)}
    for math in (abi.MATH_BF16, abi.MATH_INT8, abi.MATH_FP8, abi.MATH_FP4):
        for t, wt in weights.items():
            st, _ = gemm_w(lx, x, abi.BF16, wt, math, M, N, K)
            assert st == (0 if (math, t) in ok else NOT_SUPPORTED), (math, t, st)
    st, _ = gemm_w(lx, x, abi.BF16, weights[O.W_INT8], abi.MATH_INT8, M, N, K, workspace=False)
    assert st == INVALID
    real = lx.lx_arch()
    try:
        assert lx.lx_set_arch_override(80) == 80
        assert gemm_w(lx, x, abi.BF16, weights[O.W_INT8], abi.MATH_INT8, M, N, K)[0] == 0
        assert gemm_w(lx, x, abi.BF16, weights[O.W_FP8], abi.MATH_FP8, M, N, K)[0] == NOT_SUPPORTED
        assert gemm_w(lx, x, abi.BF16, weights[O.W_FP8], abi.MATH_BF16, M, N, K)[0] == 0
        assert lx.lx_set_arch_override(89) == 89
        assert gemm_w(lx, x, abi.BF16, weights[O.W_FP8], abi.MATH_FP8, M, N, K)[0] == 0
        assert lx.lx_set_arch_override(75) == 75
        for t, wt in weights.items():
            assert gemm_w(lx, x, abi.BF16, wt, abi.MATH_BF16, M, N, K)[0] == NOT_SUPPORTED
    finally:
        assert lx.lx_set_arch_override(0) == real
    util.check_status(lx)


def grouped(lx, wtype, math, T, L, I, E, top_k, seed):
    gu = O.quantize_weight(util.bf16_normal((E, 2 * I, L), 1.0 / L**0.5, seed), wtype)
    dn = O.quantize_weight(util.bf16_normal((E, L, I), 1.0 / I**0.5, seed + 1), wtype)
    latent = util.bf16_normal((T, L), 1.0, seed + 2)
    ids, weights, _, _ = O.moe_route(util.f32_normal((T, E), 1.0, seed + 3), None, top_k)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    out = torch.full((T, L), float("nan"), device="cuda")
    ws = torch.full((lx.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, math),), 0xFF, dtype=torch.uint8, device="cuda")
    latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)
    st = lx.lx_moe_experts_grouped(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(), math, abi.ptr(out), abi.ptr(ws),
                                   T, L, I, E, top_k, util.stream_ptr())
    torch.cuda.synchronize()
    return st, util.host(out), (latent, ids, weights, gu, dn)


@pytest.mark.parametrize("wtype,math,name", QUANT, ids=[q[2] for q in QUANT])
@pytest.mark.parametrize("shape", [(1, 256, 128, 8, 2), (9, 512, 384, 16, 4), (40, 384, 272, 8, 8)], ids=lambda s: f"T{s[0]}L{s[1]}I{s[2]}E{s[3]}k{s[4]}")
def test_grouped_experts_quantized_math(lx, wtype, math, name, shape):
    T, L, I, E, top_k = shape
    st, got, (latent, ids, weights, gu, dn) = grouped(lx, wtype, math, T, L, I, E, top_k, seed=T)
    assert st == 0, st
    util.check_status(lx)
    want = O.moe_experts_reference(latent, ids, weights, gu, dn, I, math=math)
    tol = (2e-3 if math == abi.MATH_INT8 else 8e-3) * np.abs(want).max()
    assert np.all(np.isfinite(got)) and np.abs(got - want).max() <= tol, f"{name} {shape}: {np.abs(got - want).max():.3e} > {tol:.3e}"


def test_grouped_experts_pairs(lx):
    """One math for both stacks; a stack in another format, FP4 math, BF16X stacks and architectures below the pair's
    first are all "not supported" (BF16X even when its scale pointer is null)."""
    T, L, I, E, top_k = 4, 256, 128, 8, 2
    assert grouped(lx, O.W_INT8, abi.MATH_FP8, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
    assert grouped(lx, O.W_FP8, abi.MATH_INT8, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
    assert grouped(lx, O.W_BF16, abi.MATH_INT8, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
    assert grouped(lx, O.W_NVFP4, abi.MATH_FP4, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
    assert grouped(lx, O.W_NVFP4, abi.MATH_FP8, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
    real = lx.lx_arch()
    try:
        lx.lx_set_arch_override(80)
        assert grouped(lx, O.W_FP8, abi.MATH_FP8, T, L, I, E, top_k, 1)[0] == NOT_SUPPORTED
        assert grouped(lx, O.W_INT8, abi.MATH_INT8, T, L, I, E, top_k, 1)[0] == 0
    finally:
        assert lx.lx_set_arch_override(0) == real
    # a BF16X stack: the type is refused before anything else about the weight is looked at
    some = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    gu = abi.make_weight(O.W_BF16X, some, None, 1.0)
    out = torch.zeros((T, L), device="cuda")
    ids = torch.zeros((T, top_k), dtype=torch.int32, device="cuda")
    wts = torch.zeros((T, top_k), device="cuda")
    st = lx.lx_moe_experts_grouped(abi.ptr(some), abi.ptr(ids), abi.ptr(wts), ctypes.byref(gu), ctypes.byref(gu), abi.MATH_BF16,
                                   abi.ptr(out), abi.ptr(some), T, L, I, E, top_k, util.stream_ptr())
    assert st == NOT_SUPPORTED
