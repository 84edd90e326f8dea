"""Every registered variant of the five decode GEMV kernels, forced through the variant table (lx_tune_force), against the
float64 oracle, bitwise across M = 1..8, and bitwise against the other variants of its order class; and the admission
rule of lx_tune_set on a GPU. Mirrors the reference's tests/kernels/test_gemv_w.py:200-318 (every variant, rows do not
depend on the batch, the order class is the same for every batch size)."""

import re

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu

KERNELS = {O.W_BF16: b"gemv_w_bf16", O.W_INT8: b"gemv_w_int8", O.W_FP8: b"gemv_w_fp8", O.W_NVFP4: b"gemv_w_nvfp4", O.W_BF16X: b"gemv_bf16x"}
NAMES = {O.W_BF16: "bf16", O.W_INT8: "int8", O.W_FP8: "fp8", O.W_NVFP4: "nvfp4", O.W_BF16X: "bf16x"}


def variants(lx, kernel):
    return [lx.lx_tune_variant_name(kernel, i) for i in range(lx.lx_tune_variants(kernel))]


@pytest.fixture(autouse=True)
def _clean_table(lx):
    lx.lx_tune_clear()
    yield
    lx.lx_tune_clear()


@pytest.mark.parametrize("fmt", list(KERNELS), ids=lambda f: NAMES[f])
@pytest.mark.parametrize("shape", [(320, 2048), (9605, 1152)], ids=["N320", "N9605"])
@pytest.mark.parametrize("x_f32", [False, True], ids=["xbf16", "xf32"])
def test_every_variant(lx, fmt, shape, x_f32):
    N, K = shape
    kernel = KERNELS[fmt]
    w_bits = util.bf16_normal((N, K), 0.02, 50 + fmt)
    if fmt == O.W_BF16X:  # a few patches and one row with more patches than its header holds
        w_bits[3, 100] = O.f32_to_bf16_bits(np.float32([2.0**-60]))[0]
        w_bits[17, ::9] = O.f32_to_bf16_bits(np.float32([2.0**-90]))[0]
    wt = util.make_weight(w_bits, fmt)
    dw = util.DeviceWeight(wt)
    if x_f32:
        xh = util.f32_normal((8, K), 1.0, 60)
        xv = xh.astype(np.float64)
    else:
        xh = util.bf16_normal((8, K), 1.0, 60)
        xv = O.bf16_bits_to_f32(xh).astype(np.float64)
    x_dev = util.dev(xh)
    x_dt = abi.F32 if x_f32 else abi.BF16
    want = O.gemv_reference(xv, util.reference_weight(w_bits, wt))
    names = variants(lx, kernel)
    by_class = {}
    for v, name in enumerate(names):
        for M in (1, 2, 4, 8):  # one entry per M bucket
            assert lx.lx_tune_force(kernel, M, N, K, v) == 0
        outs = {}
        for M in range(1, 9):
            assert lx.lx_tune_get(kernel, M, N, K) == v
            y = torch.full((M, N), float("nan"), device="cuda")
            assert util.gemv(lx, x_dev, x_dt, K, dw, y, abi.F32, N, M, N, K) == 0, f"{name} M={M}"
            outs[M] = util.host(y)
        util.check_status(lx)
        util.assert_close(outs[8], want, what=f"{NAMES[fmt]} variant {name.decode()}")
        for M in range(1, 8):
            assert np.array_equal(outs[M].view(np.uint32), outs[8][:M].view(np.uint32)), f"variant {name.decode()}: rows at M={M} differ from M=8"
        cls = 0 if re.match(rb"(s16)?d\d+c\d+", name) else name
        by_class.setdefault(cls, []).append(outs[8].view(np.uint32).copy())
        lx.lx_tune_clear()
    same = by_class[0]
    assert len(same) >= 2
    for other in same[1:]:
        assert np.array_equal(same[0], other), "two variants of one order class give different bits"


def test_bf16x_variants_keep_bf16_bits(lx):
    """Whatever variant of one class is named for either kernel, lx_gemv_bf16x equals lx_gemv on the same matrix bit for bit."""
    N, K = 2500, 2048
    w_bits = util.bf16_normal((N, K), 0.02, 70)
    w_bits[5, 77] = O.f32_to_bf16_bits(np.float32([2.0**-70]))[0]
    d16 = util.DeviceWeight(util.make_weight(w_bits, O.W_BF16))
    dx = util.DeviceWeight(util.make_weight(w_bits, O.W_BF16X))
    x_dev = util.dev(util.bf16_normal((8, K), 1.0, 71))
    n16, nx = variants(lx, b"gemv_w_bf16"), variants(lx, b"gemv_bf16x")
    same16 = [i for i, n in enumerate(n16) if re.match(rb"(s16)?d\d+c\d+", n)]
    samex = [i for i, n in enumerate(nx) if re.match(rb"(s16)?d\d+c\d+", n)]
    for a in same16:
        for b in samex:
            lx.lx_tune_clear()
            assert lx.lx_tune_set(b"gemv_w_bf16", 8, N, K, a) == 0 and lx.lx_tune_set(b"gemv_bf16x", 8, N, K, b) == 0
            ya = torch.full((8, N), float("nan"), device="cuda")
            yb = torch.full((8, N), float("nan"), device="cuda")
            assert util.gemv(lx, x_dev, abi.BF16, K, d16, ya, abi.F32, N, 8, N, K) == 0
            assert util.gemv(lx, x_dev, abi.BF16, K, dx, yb, abi.F32, N, 8, N, K) == 0
            assert np.array_equal(util.host(ya).view(np.uint32), util.host(yb).view(np.uint32)), (n16[a], nx[b])
    util.check_status(lx)


def test_order_class_admission_on_the_device(lx):
    """lx_tune_set admits exactly the variants whose bits equal the default's for the shape (engine/cuda/tunable.cu:104-118):
    the decode GEMV's own variants where it is the default, the tcgen05 product for INT8 weights wide enough for it."""
    K = 4096
    for kernel in KERNELS.values():
        names = variants(lx, kernel)
        gemv = [i for i, n in enumerate(names) if re.match(rb"(s16)?d\d+c\d+", n)]
        # a narrow weight: the GEMV is the default for every format
        for v in gemv:
            assert lx.lx_tune_set(kernel, 1, 1024, K, v) == 0
        if kernel == b"gemv_bf16x":  # only its own order-keeping forms are listed: every one is admitted at every key
            assert len(gemv) == len(names)
            for v in gemv:
                assert lx.lx_tune_set(kernel, 4, 14336, K, v) == 0 and lx.lx_tune_set(kernel, 2, 300, 1040, v) == 0
            assert lx.lx_tune_set(kernel, 1, 14336, K, len(names)) == abi.ERR_TUNE_VARIANT
            continue
        tc, ring = names.index(b"s1tc"), names.index(b"s8ring")
        assert lx.lx_tune_set(kernel, 1, 1024, K, tc) == abi.ERR_TUNE_REJECTED
        assert lx.lx_tune_set(kernel, 1, 1024, K, ring) == abi.ERR_TUNE_REJECTED
        # a wide weight: INT8 runs on the tcgen05 product by default, so there only "tc" keeps the bits
        splits = {int(re.match(rb"s(\d+)", names[v]).group(1)) for v in gemv}
        assert len(splits) == 1, "variants admitted together carry one split in their names"
        wide_default_tc = kernel == b"gemv_w_int8"
        assert lx.lx_tune_set(kernel, 8, 14336, K, tc) == (0 if wide_default_tc else abi.ERR_TUNE_REJECTED)
        for v in gemv:
            assert lx.lx_tune_set(kernel, 4, 14336, K, v) == (abi.ERR_TUNE_REJECTED if wide_default_tc else 0)
        assert lx.lx_tune_set(kernel, 1, 14336, K, len(names)) == abi.ERR_TUNE_VARIANT
