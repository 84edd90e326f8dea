"""Bit-exact checks of the load-time conversions through the C ABI: lx_quantize_weight / lx_dequantize_weight /
lx_quantize_w8 / lx_quantize_act against the oracle's bytes, and the BF16X encoder / decoder (byte-exact encoding,
exact round trip on trained-like, wide-range and special values, overflow records, stacked experts).

Mirrors the reference's tests/kernels/test_quant.py, test_quant_act.py and test_bf16x.py, which have no tolerances.
"""

import ctypes

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def quantize_on_gpu(lx, w_bits, wtype):
    rows, K = w_bits.reshape(-1, w_bits.shape[-1]).shape
    w_dev = util.dev(w_bits)
    data = torch.zeros(rows * (K // 2 if wtype == O.W_NVFP4 else K), dtype=torch.uint8, device="cuda")
    if wtype == O.W_NVFP4:
        scale = torch.zeros(rows * K // 16, dtype=torch.uint8, device="cuda")
    else:
        scale = torch.zeros(rows, dtype=torch.float32, device="cuda")
    lw = abi.make_weight(wtype, data, scale)
    assert lx.lx_quantize_weight(abi.ptr(w_dev), ctypes.byref(lw), rows, K, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    return data, scale, lw


@pytest.mark.parametrize("wtype", [O.W_INT8, O.W_FP8, O.W_NVFP4])
@pytest.mark.parametrize("rows,K", [(1, 16), (33, 48), (96, 512), (64, 4096)])
def test_quantize_weight_bytes_and_dequantized_values(lx, wtype, rows, K):
    w = util.bf16_normal((rows, K), 0.02, rows + K)
    if rows > 4:
        w[3] = 0            # an all-zero row keeps scale 1
        w[4, : K // 2] = 0  # zero blocks
        w[2, 5] = 0x8000    # -0.0
    want = O.quantize_weight(w, wtype)
    data, scale, lw = quantize_on_gpu(lx, w, wtype)
    assert np.array_equal(util.host(data), want.data.view(np.uint8).reshape(-1)), "quantized bytes differ"
    assert np.array_equal(util.host(scale).view(np.uint8), want.scale.view(np.uint8).reshape(-1)), "scales differ"
    if wtype == O.W_NVFP4:
        assert np.float32(lw.glob).tobytes() == np.float32(want.glob).tobytes(), "global differs"
    out = torch.zeros((rows, K), dtype=torch.int16, device="cuda")
    assert lx.lx_dequantize_weight(ctypes.byref(lw), abi.ptr(out), rows, K, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(util.host(out, np.uint16), O.dequantize_weight(want)), "dequantized bf16 values differ"


def test_nvfp4_tie_cases(lx):
    """The reference's own known answer (tests/kernels/test_quant.py:107-126): a block with amax 2688 sets the global to 1;
    a block with amax 12 gets the e4m3 scale 2 (byte 0x40) and its values / 2 sit on midpoints of the e2m1 grid: ties go
    to the even code, and -0.25 rounds to a zero stored without a sign. Asserted as literal bytes on the GPU quantizer
    and on the oracle."""
    K = 16
    vals = np.zeros((2, K), dtype=np.float32)
    vals[0, 0] = 2688.0
    vals[1, 0] = 12.0
    vals[1, 1:8] = [0.5, 1.5, 2.5, 3.5, 5.0, 7.0, 10.0]
    vals[1, 8:15] = [-0.5, -1.5, -2.5, -3.5, -5.0, -7.0, -10.0]
    w = O.f32_to_bf16_bits(vals)
    want = O.quantize_weight(w, O.W_NVFP4)
    data, scale, lw = quantize_on_gpu(lx, w, O.W_NVFP4)
    for name, d, sc, g in (("oracle", want.data.reshape(2, K // 2), want.scale.reshape(2, 1), float(want.glob)),
                           ("gpu", util.host(data).reshape(2, K // 2), util.host(scale).reshape(2, 1), float(lw.glob))):
        assert g == 1.0, f"{name}: global {g}"
        codes = np.stack([d & 15, d >> 4], axis=-1).reshape(2, K)
        assert codes[1, 0] == 7, f"{name}: 12 / 2 is 6, the largest code"
        assert codes[1, 1:8].tolist() == [0, 2, 2, 4, 4, 6, 6], f"{name}: positive ties {codes[1, 1:8].tolist()}"
        assert codes[1, 8:15].tolist() == [0, 8 + 2, 8 + 2, 8 + 4, 8 + 4, 8 + 6, 8 + 6], f"{name}: negative ties {codes[1, 8:15].tolist()}"
        assert int(sc[1, 0]) == 0x40, f"{name}: block scale byte {int(sc[1, 0]):#x}"
    assert np.array_equal(util.host(data), want.data.reshape(-1))
    assert np.array_equal(util.host(scale), want.scale.reshape(-1))


def test_quantize_w8_matches(lx):
    rows, K = 40, 200
    w = util.bf16_normal((rows, K), 0.02, 9)
    want = O.quantize_weight(w, O.W_INT8)
    q = torch.zeros((rows, K), dtype=torch.int8, device="cuda")
    s = torch.zeros(rows, dtype=torch.float32, device="cuda")
    w_dev = util.dev(w)
    assert lx.lx_quantize_w8(abi.ptr(w_dev), abi.ptr(q), abi.ptr(s), rows, K, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert np.array_equal(util.host(q), want.data) and np.array_equal(util.host(s), want.scale)


@pytest.mark.parametrize("math", [O.MATH_INT8, O.MATH_FP8, O.MATH_FP4])
@pytest.mark.parametrize("x_f32", [False, True])
def test_quantize_act_bytes(lx, math, x_f32):
    M, K = 5, 512
    if x_f32:
        x = util.f32_normal((M, K), 1.0, 4)
        x[2] = 0
        xv = x
    else:
        xb = util.bf16_normal((M, K), 1.0, 4)
        xb[2] = 0
        x, xv = xb, O.bf16_bits_to_f32(xb)
    q_want, s_want, bs_want = O.quantize_act(xv, math)
    ld_q = K // 2 if math == O.MATH_FP4 else K
    q = torch.zeros((M, ld_q), dtype=torch.uint8, device="cuda")
    s = torch.zeros(M, dtype=torch.float32, device="cuda")
    bs = torch.zeros((M, K // 16), dtype=torch.uint8, device="cuda")
    x_dev = util.dev(x)
    st = lx.lx_quantize_act(abi.ptr(x_dev), abi.F32 if x_f32 else abi.BF16, K, math, abi.ptr(q), ld_q, abi.ptr(s),
                            abi.ptr(bs), K // 16, M, K, util.stream_ptr())
    assert st == 0
    torch.cuda.synchronize()
    assert np.array_equal(util.host(q), q_want)
    assert np.array_equal(util.host(s).view(np.uint32), s_want.view(np.uint32))
    if bs_want is not None:
        assert np.array_equal(util.host(bs), bs_want)


# ---- BF16X -----------------------------------------------------------------------------------------------------


def trained_like(rows, K, seed):
    return util.bf16_normal((rows, K), 0.02, seed)


def wide_range(rows, K, seed):
    g = torch.Generator().manual_seed(seed)
    mant = torch.randn((rows, K), generator=g)
    expo = torch.randint(-60, 20, (rows, K), generator=g).float()
    return O.f32_to_bf16_bits((mant * torch.exp2(expo)).numpy().astype(np.float32))


def specials(rows, K, seed):
    w = trained_like(rows, K, seed)
    pool = np.array([0x0000, 0x8000, 0x0001, 0x8001, 0x007F, 0x7F80, 0xFF80, 0x7FC0, 0xFFC1, 0x7F7F, 0x0080], dtype=np.uint16)
    rng = np.random.default_rng(seed)
    mask = rng.random((rows, K)) < 0.05
    w[mask] = pool[rng.integers(0, len(pool), mask.sum())]
    return w


def encode(lx, w):
    rows, K = w.shape
    w_dev = util.dev(w)
    n = lx.lx_bf16x_bytes(abi.ptr(w_dev), rows, K, util.stream_ptr())
    assert n > 0, f"lx_bf16x_bytes returned {n}"
    buf = torch.full((n + 16,), 0xAB, dtype=torch.uint8, device="cuda")
    assert lx.lx_bf16x_encode(abi.ptr(w_dev), rows, K, abi.ptr(buf), n, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert bool((buf[n:] == 0xAB).all()), "encoder wrote past the size it reported"
    return buf[:n]


def decode(lx, data, rows, K):
    out = torch.zeros((rows, K), dtype=torch.int16, device="cuda")
    assert lx.lx_bf16x_decode(abi.ptr(data), rows, K, abi.ptr(out), util.stream_ptr()) == 0
    torch.cuda.synchronize()
    return util.host(out, np.uint16)


@pytest.mark.parametrize("make", [trained_like, wide_range, specials], ids=["trained", "wide", "specials"])
@pytest.mark.parametrize("rows,K", [(1, 1), (7, 13), (100, 256), (37, 1000), (512, 2048), (64, 4096), (16, 6400), (3, 20000)])
def test_bf16x_encoding_is_byte_exact_and_round_trips(lx, make, rows, K):
    w = make(rows, K, rows * 3 + K)
    data = encode(lx, w)
    want = O.bf16x_encode(w)
    got = util.host(data)
    assert got.size == want.size, f"size {got.size} != {want.size}"
    assert np.array_equal(got, want), f"{int((got != want).sum())} bytes differ"
    assert np.array_equal(decode(lx, data, rows, K), w), "round trip changed bits"
    assert lx.lx_bf16x_row_bytes(K) == O.bf16x_row_bytes(K)


def test_bf16x_overflow_rows(lx):
    rows, K = 4, 2048
    w = trained_like(rows, K, 1)
    w[1, ::7] = O.f32_to_bf16_bits(np.float32([2.0**-100]))[0]
    w[1, 0::128] = O.f32_to_bf16_bits(np.float32([1.0]))[0]
    w[3, 5] = O.f32_to_bf16_bits(np.float32([-(2.0**-120)]))[0]
    data = encode(lx, w)
    assert data.numel() > rows * O.bf16x_row_bytes(K), "expected an overflow record"
    assert np.array_equal(util.host(data), O.bf16x_encode(w))
    assert np.array_equal(decode(lx, data, rows, K), w)


def test_bf16x_stack_is_rows_and_size_query_limits(lx):
    w = trained_like(6 * 64, 512, 2)
    data = encode(lx, w)
    assert np.array_equal(decode(lx, data, 6 * 64, 512), w)
    assert lx.lx_bf16x_row_bytes(0) == -1 and lx.lx_bf16x_row_bytes(1 << 23) == -1
    assert lx.lx_bf16x_row_bytes(4096) == 6192 and lx.lx_bf16x_row_bytes(8192) == 12376 and lx.lx_bf16x_row_bytes(1536) == 2328


def test_bf16x_bits_per_value_on_trained_like_weights(lx):
    w = trained_like(256, 4096, 0)
    data = encode(lx, w)
    bits = data.numel() * 8 / w.size
    assert 12.0 <= bits <= 12.2, bits
