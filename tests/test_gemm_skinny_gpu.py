"""lx_gemm_skinny (bf16 weights, bf16 activations, any M): parity, the f32 epilogue, and the contract that a row's bits
depend on nothing but that row, the weight and the epilogue (kernels.h:457-475). Mirrors the reference's
tests/kernels/test_gemm_skinny.py:72-107 on smaller shapes (the CPU oracle multiplies in float64)."""

import ctypes

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def skinny(lx, x_dev, dw, y_dev, y_dt, M, N, K, bias=None, bias_dt=abi.F32, alpha=1.0, beta=0.0, x_dt=abi.BF16):
    return lx.lx_gemm_skinny(abi.ptr(x_dev), x_dt, K, dw.ref(), abi.ptr(bias), bias_dt, abi.ptr(y_dev), y_dt, N, M, N, K, alpha, beta,
                             util.stream_ptr())


@pytest.mark.parametrize("N,K", [(1024, 1024), (2560, 2560), (256, 6400), (10304, 2048)])
@pytest.mark.parametrize("M", [1, 2, 8, 16, 32, 64, 100])
def test_bf16_matches_reference(lx, N, K, M):
    w_bits = util.bf16_normal((N, K), 0.02, N + K)
    dw = util.DeviceWeight(O.Weight(O.W_BF16, w_bits))
    x = util.bf16_normal((M, K), 1.0, M)
    y = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    assert skinny(lx, util.dev(x), dw, y, abi.BF16, M, N, K) == 0
    util.check_status(lx)
    got = O.bf16_bits_to_f32(util.host(y, np.uint16))
    want = O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), O.Weight(O.W_BF16, w_bits))
    tol = 2.0**-8 * float(np.abs(want).max())  # half a bf16 ulp of the largest output, the reference suite's bound
    assert float(np.abs(got - want).max()) <= tol


@pytest.mark.parametrize("N,K", [(2560, 2560), (10304, 2048)])
def test_bias_alpha_beta_f32_output(lx, N, K):
    M = 16
    w_bits = util.bf16_normal((N, K), 0.02, 3)
    dw = util.DeviceWeight(O.Weight(O.W_BF16, w_bits))
    x = util.bf16_normal((M, K), 1.0, 4)
    bias = util.bf16_normal((N,), 1.0, 5)
    y0 = util.f32_normal((M, N), 1.0, 6)
    y = util.dev(y0.copy())
    assert skinny(lx, util.dev(x), dw, y, abi.F32, M, N, K, bias=util.dev(bias), bias_dt=abi.BF16, alpha=0.5, beta=2.0) == 0
    util.check_status(lx)
    want = O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), O.Weight(O.W_BF16, w_bits), O.bf16_bits_to_f32(bias).astype(np.float64),
                            y0, 0.5, 2.0)
    assert float(np.abs(util.host(y) - want).max()) <= 2e-4 * float(np.abs(want).max())


@pytest.mark.parametrize("N,K", [(2560, 2560), (10304, 2048), (256, 6400)])
def test_rows_are_batch_invariant(lx, N, K):
    """A row's bits do not depend on M, on its position in the launch, or on the other rows: at M = 1, 2, 8, 16, 32, 64
    against the M = 100 launch (which crosses a chunk of 64), and rows alone."""
    w_bits = util.bf16_normal((N, K), 0.02, 7)
    dw = util.DeviceWeight(O.Weight(O.W_BF16, w_bits))
    x = util.bf16_normal((100, K), 1.0, 8)
    x_dev = util.dev(x)
    full = torch.zeros((100, N), dtype=torch.int16, device="cuda")
    assert skinny(lx, x_dev, dw, full, abi.BF16, 100, N, K) == 0
    full_h = util.host(full, np.uint16)
    for M in (1, 2, 8, 16, 32, 64):
        y = torch.zeros((M, N), dtype=torch.int16, device="cuda")
        assert skinny(lx, x_dev, dw, y, abi.BF16, M, N, K) == 0
        assert np.array_equal(util.host(y, np.uint16), full_h[:M]), f"M={M}: rows differ from the M=100 launch"
    for r in (0, 1, 37, 63, 64, 99):
        alone = torch.zeros((1, N), dtype=torch.int16, device="cuda")
        assert skinny(lx, util.dev(x[r:r + 1]), dw, alone, abi.BF16, 1, N, K) == 0
        assert np.array_equal(util.host(alone, np.uint16), full_h[r:r + 1]), f"row {r} alone differs from its row in the M=100 launch"
    # and the same bits as the decode GEMV entry point gives the row
    gv = torch.zeros((8, N), dtype=torch.int16, device="cuda")
    assert util.gemv(lx, x_dev, abi.BF16, K, dw, gv, abi.BF16, N, 8, N, K) == 0
    assert np.array_equal(util.host(gv, np.uint16), full_h[:8])
    util.check_status(lx)


def test_unsupported_shapes_are_refused(lx):
    """N not a multiple of 16, K not a multiple of 64, f32 activations and other formats are outside the contract: the
    call says so (801), it does not guess."""
    w_bits = util.bf16_normal((64, 2048), 0.02, 1)
    dw = util.DeviceWeight(O.Weight(O.W_BF16, w_bits))
    x = util.dev(util.bf16_normal((4, 2048), 1.0, 2))
    y = torch.zeros((4, 64), dtype=torch.int16, device="cuda")
    assert skinny(lx, x, dw, y, abi.BF16, 4, 8, 2048) == abi.ERR_NOT_SUPPORTED      # N = 8
    assert skinny(lx, x, dw, y, abi.BF16, 4, 64, 2016) == abi.ERR_NOT_SUPPORTED     # K % 64 != 0
    xf = util.dev(util.f32_normal((4, 2048), 1.0, 3))
    assert skinny(lx, xf, dw, y, abi.BF16, 4, 64, 2048, x_dt=abi.F32) == abi.ERR_NOT_SUPPORTED
    d8 = util.DeviceWeight(util.make_weight(w_bits, O.W_INT8))
    assert skinny(lx, x, d8, y, abi.BF16, 4, 64, 2048) == abi.ERR_NOT_SUPPORTED
    assert skinny(lx, x, dw, y, abi.BF16, 0, 64, 2048) == 0                          # nothing to do
    assert lx.lx_gemm_skinny(abi.ptr(x), abi.BF16, 2047, dw.ref(), None, abi.F32, abi.ptr(y), abi.BF16, 64, 4, 64, 2048, 1.0, 0.0,
                             util.stream_ptr()) == abi.ERR_INVALID               # ld_x < K
