"""Parity of the decode products (lx_gemv_w, lx_gemv_bf16x, lx_gemm_w) against the float64 oracle, through the C ABI.

Mirrors the reference's tests/kernels/test_gemv_w.py and test_gemm_w.py: dtype matrix, every M, strided rows with a
"wrote past N" check, epilogue constants, determinism and batch invariance, plus the configurations the headline
metric is quoted on, checked on sampled rows at full size.
"""

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu

FORMATS = [O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4, O.W_BF16X]
NAMES = {O.W_BF16: "bf16", O.W_INT8: "int8", O.W_FP8: "fp8", O.W_NVFP4: "nvfp4", O.W_BF16X: "bf16x"}


def run(lx, fmt, M, N, K, x_f32=False, y_f32=True, bias_dtype=None, alpha=1.0, beta=0.0, seed=0, fn="lx_gemv_w",
        ld_pad=0, w_bits=None):
    w_bits = util.bf16_normal((N, K), 0.02, seed) if w_bits is None else w_bits
    wt = util.make_weight(w_bits, fmt)
    dw = util.DeviceWeight(wt)
    ld_x, ld_y = K + ld_pad, N + ld_pad
    if x_f32:
        xh = np.zeros((M, ld_x), dtype=np.float32)
        xh[:, :K] = util.f32_normal((M, K), 1.0, seed + 1)
        x_vals = xh[:, :K].astype(np.float64)
        if fn == "lx_gemm_w":  # BF16 math rounds f32 activations to bf16 first (engine/cuda/gemm_w.cu:213-252); the GEMV does not
            x_vals = O.bf16_bits_to_f32(O.f32_to_bf16_bits(xh[:, :K])).astype(np.float64)
    else:
        xh = np.zeros((M, ld_x), dtype=np.uint16)
        xh[:, :K] = util.bf16_normal((M, K), 1.0, seed + 1)
        x_vals = O.bf16_bits_to_f32(xh[:, :K]).astype(np.float64)
    bias_h = bias_v = None
    if bias_dtype is not None:
        if bias_dtype == abi.F32:
            bias_h = util.f32_normal((N,), 0.5, seed + 2)
            bias_v = bias_h.astype(np.float64)
        else:
            bias_h = util.bf16_normal((N,), 0.5, seed + 2)
            bias_v = O.bf16_bits_to_f32(bias_h).astype(np.float64)
    y_old = util.f32_normal((M, ld_y), 1.0, seed + 3)
    if not y_f32:
        y_old_bits = O.f32_to_bf16_bits(y_old)
        y_old = O.bf16_bits_to_f32(y_old_bits)
    # y pre-filled with NaN when beta == 0: it must not be read
    y_init = y_old.copy() if beta != 0.0 else np.full((M, ld_y), np.nan, dtype=np.float32)
    y_dev = util.dev(y_init if y_f32 else O.f32_to_bf16_bits(y_init))
    x_dev = util.dev(xh)
    bias_dev = None if bias_h is None else util.dev(bias_h)
    ws = torch.empty(max(1, lx.lx_gemm_workspace_bytes(M, K, 0)), dtype=torch.uint8, device="cuda")
    st = util.gemv(lx, x_dev, abi.F32 if x_f32 else abi.BF16, ld_x, dw, y_dev, abi.F32 if y_f32 else abi.BF16, ld_y, M, N, K,
                   bias=bias_dev, bias_dtype=bias_dtype if bias_dtype is not None else abi.BF16, alpha=alpha, beta=beta,
                   fn=fn, workspace=ws)
    assert st == 0, f"status {st}"
    util.check_status(lx)
    got_full = util.host(y_dev) if y_f32 else O.bf16_bits_to_f32(util.host(y_dev, np.uint16))
    want = O.gemv_reference(x_vals, util.reference_weight(w_bits, wt), bias_v, y_old[:, :N], alpha, beta)
    return got_full, want, y_init


def check(got_full, want, y_init, N, y_f32, what):
    got = got_full[:, :N]
    scale = max(1e-30, float(np.abs(want).max()))
    # the reference suite's own bound (2^-8 of max|y| for bf16 outputs, 2e-4 for f32) and the acceptance bound
    tol = (2.0**-8 if not y_f32 else 2e-4) * scale
    assert np.all(np.isfinite(got)), f"{what}: non-finite"
    err = float(np.abs(got - want).max())
    assert err <= tol, f"{what}: max abs err {err:.3e} > {tol:.3e}"
    if y_f32:
        util.assert_close(got, want, what=what)
    # columns past N keep what they held (compare bit patterns: NaN != NaN)
    if got_full.shape[1] > N:
        a = np.ascontiguousarray(got_full[:, N:]).view(np.uint32)
        b = np.ascontiguousarray(y_init[:, N:]).view(np.uint32)
        assert np.array_equal(a, b) or not y_f32, f"{what}: wrote past N"


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8])
def test_gemv_every_m(lx, fmt, M):
    N, K = 320, 2048
    got, want, y0 = run(lx, fmt, M, N, K, seed=M)
    check(got, want, y0, N, True, f"{NAMES[fmt]} M={M}")


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("x_f32", [False, True])
@pytest.mark.parametrize("y_f32", [False, True])
@pytest.mark.parametrize("bias_dtype", [None, abi.F32, abi.BF16])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (0.5, 0.75)])
def test_gemv_dtype_matrix(lx, fmt, x_f32, y_f32, bias_dtype, alpha, beta):
    M, N, K = 3, 136, 1024
    got, want, y0 = run(lx, fmt, M, N, K, x_f32, y_f32, bias_dtype, alpha, beta, seed=7)
    check(got, want, y0, N, y_f32, NAMES[fmt])


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("K", [32, 48, 256, 528, 768, 4096 + 256])
def test_gemv_k_boundaries(lx, fmt, K):
    if fmt == O.W_NVFP4 and K % 16:
        pytest.skip("NVFP4 needs K % 16 == 0")
    M, N = 2, 77
    got, want, y0 = run(lx, fmt, M, N, K, seed=K)
    check(got, want, y0, N, True, f"{NAMES[fmt]} K={K}")


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
def test_gemv_strided_rows_and_tail(lx, fmt):
    M, N, K = 4, 100, 512
    got, want, y0 = run(lx, fmt, M, N, K, ld_pad=24, seed=3)
    check(got, want, y0, N, True, NAMES[fmt])


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("M", [9, 16, 17, 32, 33, 64, 70])
def test_gemm_w_small_m(lx, fmt, M):
    if fmt == O.W_BF16X:
        pytest.skip("lx_gemm_w takes BF16X through lx_bf16x_decode in the engine")
    N, K = 264, 1024
    got, want, y0 = run(lx, fmt, M, N, K, seed=M, fn="lx_gemm_w")
    check(got, want, y0, N, True, f"{NAMES[fmt]} M={M}")


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("case", [(16, 264, 4096, False), (24, 1000, 2304, False), (20, 1000, 2304, True), (64, 520, 8192, False)],
                         ids=lambda c: f"M{c[0]}N{c[1]}K{c[2]}{'f32' if c[3] else ''}")
def test_gemm_w_odd_tiles_and_long_k(lx, fmt, case):
    """Shapes with few, ragged tiles (N not a multiple of the tile rows, fewer tiles than SMs), K ending inside a stage,
    f32 activations and 64 rows, with bias, alpha and beta, twice in a row on the same workspace: the two results are
    bitwise equal."""
    if fmt == O.W_BF16X:
        pytest.skip("lx_gemm_w takes BF16X through lx_bf16x_decode in the engine")
    M, N, K, x_f32 = case
    outs = []
    for _ in range(2):
        got, want, y0 = run(lx, fmt, M, N, K, seed=7, fn="lx_gemm_w", x_f32=x_f32, bias_dtype=abi.F32, alpha=0.5, beta=0.25)
        check(got, want, y0, N, True, f"{NAMES[fmt]} {case}")
        outs.append(got.view(np.uint32).copy())
    assert np.array_equal(outs[0], outs[1]), "two runs differ"


WIDE = [O.W_INT8, O.W_FP8]  # formats that also have a tcgen05 product for up to 8 rows when N gives every SM >= 40 rows


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("x_f32", [False, True], ids=["xbf16", "xf32"])
def test_gemv_wide_weight(lx, fmt, M, x_f32):
    """N large enough that every CTA has several 16-row units with a ragged last one, K ending inside a warp's slice,
    with bias, alpha and beta."""
    N, K = 9605, 1152
    got, want, y0 = run(lx, fmt, M, N, K, seed=20 + M, x_f32=x_f32, bias_dtype=abi.BF16, alpha=1.5, beta=-0.5)
    check(got, want, y0, N, True, f"{NAMES[fmt]} M={M}")


@pytest.mark.parametrize("fmt", WIDE, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("x_f32", [False, True], ids=["xbf16", "xf32"])
def test_gemv_wide_weight_tensor_core_variant(lx, fmt, M, x_f32):
    """The tcgen05 product for up to 8 rows (tiles of 65 rows, a ragged last tile, K ending inside a stage), reached
    through the variant table."""
    N, K = 9605, 1040
    kernel = b"gemv_w_int8" if fmt == O.W_INT8 else b"gemv_w_fp8"
    names = [lx.lx_tune_variant_name(kernel, i) for i in range(lx.lx_tune_variants(kernel))]
    assert lx.lx_tune_force(kernel, M, N, K, names.index(b"s1tc")) == 0
    try:
        got, want, y0 = run(lx, fmt, M, N, K, seed=20 + M, x_f32=x_f32, bias_dtype=abi.BF16, alpha=1.5, beta=-0.5)
    finally:
        lx.lx_tune_clear()
    check(got, want, y0, N, True, f"{NAMES[fmt]} M={M}")


@pytest.mark.parametrize("fmt", [O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4], ids=lambda f: NAMES[f])
def test_gemm_w_rows_do_not_depend_on_batch(lx, fmt):
    """Within lx_gemm_w (a workspace given) a row's bits are the same in a call of 1, 5, 8, 9 or 16 rows: every row count
    runs on the tcgen05 product (the reference promises this under LX_BATCH_INVARIANT=1, engine/cuda/gemm_w.cu:160-168)."""
    N, K = 9605, 1024
    w_bits = util.bf16_normal((N, K), 0.02, 31)
    dw = util.DeviceWeight(util.make_weight(w_bits, fmt))
    x = util.bf16_normal((16, K), 1.0, 32)
    x_dev = util.dev(x)
    big = torch.full((16, N), float("nan"), device="cuda")
    ws = torch.empty(lx.lx_gemm_workspace_bytes(16, K, 0), dtype=torch.uint8, device="cuda")
    assert util.gemv(lx, x_dev, abi.BF16, K, dw, big, abi.F32, N, 16, N, K, fn="lx_gemm_w", workspace=ws) == 0
    want = util.host(big).view(np.uint32)
    for M in (1, 5, 8, 9):
        y = torch.full((M, N), float("nan"), device="cuda")
        assert util.gemv(lx, x_dev, abi.BF16, K, dw, y, abi.F32, N, M, N, K, fn="lx_gemm_w", workspace=ws) == 0
        assert np.array_equal(util.host(y).view(np.uint32), want[:M]), f"rows at M={M} differ from the same rows at M=16"
    util.check_status(lx)


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
@pytest.mark.parametrize("K", [2048, 4096], ids=["K2048", "K4096"])
@pytest.mark.parametrize("x_f32", [False, True], ids=["xbf16", "xf32"])
@pytest.mark.parametrize("N", [256, 2500])
def test_rows_do_not_depend_on_batch_and_runs_repeat(lx, fmt, K, x_f32, N):
    """A row's bits are the same at every M = 1..8, for bf16 and for f32 activations, whether the weight is a few rows
    (one short unit per CTA) or thousands, and a second run repeats the first bit for bit."""
    w_bits = util.bf16_normal((N, K), 0.02, 11)
    wt = util.make_weight(w_bits, fmt)
    dw = util.DeviceWeight(wt)
    x_dev = util.dev(util.f32_normal((8, K), 1.0, 12)) if x_f32 else util.dev(util.bf16_normal((8, K), 1.0, 12))
    x_dt = abi.F32 if x_f32 else abi.BF16
    outs = {}
    for M in range(1, 9):
        y = torch.full((M, N), float("nan"), device="cuda")
        assert util.gemv(lx, x_dev, x_dt, K, dw, y, abi.F32, N, M, N, K) == 0
        outs[M] = util.host(y).view(np.uint32).copy()
    y2 = torch.full((8, N), float("nan"), device="cuda")
    assert util.gemv(lx, x_dev, x_dt, K, dw, y2, abi.F32, N, 8, N, K) == 0
    util.check_status(lx)
    assert np.array_equal(outs[8], util.host(y2).view(np.uint32)), "two runs differ"
    for M in range(1, 8):
        assert np.array_equal(outs[M], outs[8][:M]), f"rows at M={M} differ from the same rows at M=8"


@pytest.mark.parametrize("N,K", [(512, 4096), (520, 1536), (264, 8192), (77, 1536), (40, 14336), (2400, 512)],
                         ids=["aligned", "short_last_unit", "records_8_aligned", "odd_rows", "long_rows", "many_units"])
def test_bf16x_product_equals_bf16_product_bitwise(lx, N, K):
    """Records that start on 16-byte boundaries (header a multiple of 16 bytes: K = 4096, 512) and records that do not
    (K = 1536, 8192, 14336: every other record starts 8 bytes off), a last unit of fewer than 16 rows, an odd number of
    8-aligned records (the copy of the last one would end past the matrix: the in-register kernel takes those)."""
    w_bits = util.bf16_normal((N, K), 0.02, 5)
    # patches: a few values far below their block's largest, one row with more patches than its slots
    w_bits[3, 100] = O.f32_to_bf16_bits(np.float32([2.0**-60]))[0]
    w_bits[3, 1000 % K] = O.f32_to_bf16_bits(np.float32([-(2.0**-70)]))[0]
    w_bits[17, ::9] = O.f32_to_bf16_bits(np.float32([2.0**-90]))[0]
    w_bits[N - 1, K - 1] = O.f32_to_bf16_bits(np.float32([2.0**-80]))[0]
    w_bits[N - 2, 0] = O.f32_to_bf16_bits(np.float32([-(2.0**-80)]))[0]
    dw16 = util.DeviceWeight(util.make_weight(w_bits, O.W_BF16))
    dwx = util.DeviceWeight(util.make_weight(w_bits, O.W_BF16X))
    for x_dt, x_dev in ((abi.BF16, util.dev(util.bf16_normal((8, K), 1.0, 6))), (abi.F32, util.dev(util.f32_normal((8, K), 1.0, 6)))):
        for M in (1, 5, 8):
            ya = torch.full((M, N), float("nan"), device="cuda")
            yb = torch.full((M, N), float("nan"), device="cuda")
            assert util.gemv(lx, x_dev, x_dt, K, dw16, ya, abi.F32, N, M, N, K) == 0
            assert util.gemv(lx, x_dev, x_dt, K, dwx, yb, abi.F32, N, M, N, K) == 0
            util.check_status(lx)
            assert np.array_equal(util.host(ya).view(np.uint32), util.host(yb).view(np.uint32))


@pytest.mark.parametrize("fmt", FORMATS, ids=lambda f: NAMES[f])
def test_scalar_path_agrees(lx, fmt, monkeypatch):
    """The scalar kernel (unaligned / odd shapes) and the streaming kernel are two implementations of one contract."""
    M, N, K = 3, 96, 1024
    got_a, want, y0 = run(lx, fmt, M, N, K, seed=21)
    monkeypatch.setenv("LX_B200_FORCE_SCALAR", "1")
    got_b, _, _ = run(lx, fmt, M, N, K, seed=21)
    check(got_b, want, y0, N, True, f"{NAMES[fmt]} scalar")
    scale = float(np.abs(want).max())
    assert float(np.abs(got_a[:, :N] - got_b[:, :N]).max()) <= 1e-4 * scale


def test_argument_errors(lx):
    N, K = 64, 256
    dw = util.DeviceWeight(util.make_weight(util.bf16_normal((N, K), 0.02, 1), O.W_INT8))
    x = util.dev(util.bf16_normal((8, K), 1.0, 2))
    y = torch.zeros((8, N), device="cuda")
    assert util.gemv(lx, x, abi.BF16, K, dw, y, abi.F32, N, 0, N, K) == 0           # nothing to do
    assert util.gemv(lx, x, abi.BF16, K, dw, y, abi.F32, N, 9, N, K) == abi.ERR_INVALID   # GEMV is M <= 8
    assert util.gemv(lx, x, abi.BF16, K - 1, dw, y, abi.F32, N, 1, N, K) == abi.ERR_INVALID  # ld_x < K
    assert util.gemv(lx, x, abi.BF16, K, dw, y, abi.F32, N - 1, 1, N, K) == abi.ERR_INVALID  # ld_y < N
    no_scale = abi.make_weight(O.W_INT8, dw.data, None)
    import ctypes
    assert lx.lx_gemv_w(abi.ptr(x), abi.BF16, K, ctypes.byref(no_scale), None, abi.BF16, abi.ptr(y), abi.F32, N, 1, N, K,
                        1.0, 0.0, util.stream_ptr()) == abi.ERR_INVALID
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    assert util.gemv(lx, x, abi.BF16, K, dw, y, abi.F32, N, 8, N, K, fn="lx_gemm_w", math=abi.MATH_FP4,
                     workspace=ws) == abi.ERR_NOT_SUPPORTED


@pytest.mark.parametrize("fmt", [O.W_BF16, O.W_INT8, O.W_FP8], ids=lambda f: NAMES[f])
@pytest.mark.parametrize("M", [3, 20])
def test_allgather_epilogue_on_one_gpu(lx, fmt, M):
    """lx_b200_linear_allgather with the two "ranks" played one after the other on one GPU: each stores its row shard's
    outputs into its columns of the one whole y and counts itself; lx_b200_wait_arrivals takes both rounds' arrivals.
    The slices equal the same products through lx_gemm_w bit for bit (the same kernels, another epilogue)."""
    import ctypes

    N, K = 19210, 1024  # two shards of 9605 rows: wide enough for up to 8 rows to take the tensor-core GEMV
    half = N // 2
    w_bits = util.bf16_normal((N, K), 0.02, 41)
    x = util.bf16_normal((M, K), 1.0, 42)
    x_dev = util.dev(x)
    y = torch.full((M, N), float("nan"), device="cuda")
    counter = torch.zeros(4, dtype=torch.int32, device="cuda")
    ws = torch.empty(lx.lx_gemm_workspace_bytes(M, K, 0), dtype=torch.uint8, device="cuda")
    y_all = (ctypes.c_void_p * 1)(y.data_ptr())
    c_all = (ctypes.c_void_p * 1)(counter.data_ptr())
    total, shards = 0, []
    for r in range(2):
        dw = util.DeviceWeight(util.make_weight(w_bits[r * half:(r + 1) * half], fmt))
        shards.append(dw)
        added = ctypes.c_int(0)
        st = lx.lx_b200_linear_allgather(abi.ptr(x_dev), abi.BF16, K, dw.ref(), None, abi.BF16, y_all, c_all, 1, 0, r * half, abi.F32, N, M,
                                         half, K, 1.0, abi.ptr(ws), ctypes.byref(added), util.stream_ptr())
        assert st == 0 and added.value > 0
        total += added.value
    assert lx.lx_b200_wait_arrivals(counter.data_ptr(), total, util.stream_ptr()) == 0
    util.check_status(lx)
    assert int(counter[0].item()) == 0 and int(counter[1].item()) == 0  # the wait took what the products added; the warp count is back to zero
    got = util.host(y)
    for r in range(2):
        ref = torch.full((M, half), float("nan"), device="cuda")
        assert util.gemv(lx, x_dev, abi.BF16, K, shards[r], ref, abi.F32, half, M, half, K, fn="lx_gemm_w", workspace=ws) == 0
        assert np.array_equal(got[:, r * half:(r + 1) * half].view(np.uint32), util.host(ref).view(np.uint32)), f"shard {r}"
    want = O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), util.reference_weight(w_bits, util.make_weight(w_bits, fmt)))
    util.assert_close(got, want, what=NAMES[fmt])
