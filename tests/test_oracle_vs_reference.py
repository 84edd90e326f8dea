"""Pins the oracle: the numpy restatement against the reference project's own CPU backend, compiled unmodified from the
reference checkout by oracle/Makefile (skipped where that library has not been built). Bit-exact for every byte and
index the path defines; 1e-5 for the routing weights; float round-off for the products."""

import ctypes

import numpy as np
import pytest

from dromos_b200 import abi
from oracle import dromos_oracle as O


def bf16_normal(rng, shape, std):
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32))


@pytest.mark.parametrize("wt", [O.W_INT8, O.W_FP8, O.W_NVFP4])
@pytest.mark.parametrize("N,K", [(1, 16), (33, 48), (96, 512), (16, 4096)])
def test_quantize_dequantize(ref, wt, N, K):
    rng = np.random.default_rng(N * 7 + K)
    w = bf16_normal(rng, (N, K), 0.02)
    if N > 4:
        w[3] = 0
        w[4, : K // 2] = 0
    o = O.quantize_weight(w, wt)
    data, scale = np.zeros_like(o.data), np.zeros_like(o.scale)
    lw = abi.make_weight(wt, data, scale)
    assert ref.lx_quantize_weight(abi.ptr(w), ctypes.byref(lw), N, K, None) == 0
    assert np.array_equal(data.view(np.uint8), o.data.view(np.uint8))
    assert np.array_equal(scale.view(np.uint8), o.scale.view(np.uint8))
    assert np.float32(lw.glob).tobytes() == np.float32(o.glob).tobytes()
    out = np.zeros((N, K), dtype=np.uint16)
    assert ref.lx_dequantize_weight(ctypes.byref(lw), abi.ptr(out), N, K, None) == 0
    assert np.array_equal(out, O.dequantize_weight(o))


@pytest.mark.parametrize("rows,K", [(1, 1), (7, 13), (100, 256), (37, 1000), (64, 4096), (3, 20000)])
def test_bf16x(ref, rows, K):
    rng = np.random.default_rng(rows + K)
    w = bf16_normal(rng, (rows, K), 0.02)
    w[0, ::3] = O.f32_to_bf16_bits(np.float32([2.0**-100]))[0]
    if K > 5:
        w[rows - 1, 5] = O.f32_to_bf16_bits(np.float32([-(2.0**-120)]))[0]
    n = ref.lx_bf16x_bytes(abi.ptr(w), rows, K, None)
    buf = np.zeros(n, dtype=np.uint8)
    assert ref.lx_bf16x_encode(abi.ptr(w), rows, K, abi.ptr(buf), n, None) == 0
    assert np.array_equal(O.bf16x_encode(w), buf)
    assert np.array_equal(O.bf16x_decode(buf, rows, K), w)
    assert O.bf16x_row_bytes(K) == ref.lx_bf16x_row_bytes(K)


@pytest.mark.parametrize("math", [1, 2, 3])
def test_quantize_act(ref, math):
    rng = np.random.default_rng(math)
    x = rng.standard_normal((5, 256)).astype(np.float32)
    x[2] = 0
    q, s, bs = O.quantize_act(x, math)
    q2, s2, bs2 = np.zeros_like(q), np.zeros_like(s), np.zeros((5, 16), dtype=np.uint8)
    assert ref.lx_quantize_act(abi.ptr(x), 0, 256, math, abi.ptr(q2), q2.shape[1], abi.ptr(s2), abi.ptr(bs2), 16, 5, 256, None) == 0
    assert np.array_equal(q, q2) and np.array_equal(s, s2) and (bs is None or np.array_equal(bs, bs2))


@pytest.mark.parametrize("with_bias", [False, True])
def test_route(ref, with_bias):
    rng = np.random.default_rng(5)
    T, E, k = 33, 64, 8
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0] = 0.5
    bias = (rng.standard_normal(E) * 0.1).astype(np.float32) if with_bias else None
    ids, w, ent, conf = O.moe_route(logits, bias, k)
    ids2, w2 = np.zeros((T, k), dtype=np.int32), np.zeros((T, k), dtype=np.float32)
    e2, c2 = np.zeros(T, dtype=np.float32), np.zeros(T, dtype=np.float32)
    assert ref.lx_moe_route(abi.ptr(logits), abi.ptr(bias), abi.ptr(ids2), abi.ptr(w2), abi.ptr(e2), abi.ptr(c2), T, E, k, None) == 0
    assert np.array_equal(ids, ids2)
    assert np.abs(w - w2).max() <= 1e-5 and np.abs(ent - e2).max() <= 1e-5 and np.abs(conf - c2).max() <= 1e-5


@pytest.mark.parametrize("wt", [O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4])
def test_gemv_product(ref, wt):
    rng = np.random.default_rng(9)
    M, N, K = 3, 40, 512
    w = bf16_normal(rng, (N, K), 0.02)
    o = O.quantize_weight(w, wt)
    lw = abi.make_weight(wt, o.data, o.scale, o.glob)
    x = bf16_normal(rng, (M, K), 1.0)
    y = np.zeros((M, N), dtype=np.float32)
    assert ref.lx_gemv_w(abi.ptr(x), abi.BF16, K, ctypes.byref(lw), None, abi.BF16, abi.ptr(y), abi.F32, N, M, N, K, 1.0, 0.0, None) == 0
    want = O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), o)
    assert O.rel_l2(y, want) <= 1e-5


@pytest.mark.parametrize("wt", [O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4])
def test_routed_experts(ref, wt):
    """The oracle's routed experts against the reference's few-token and grouped entry points on its CPU backend."""
    rng = np.random.default_rng(13)
    T, E, L, I, k = 5, 6, 128, 64, 3
    gu = O.quantize_weight(bf16_normal(rng, (E, 2 * I, L), 0.02), wt)
    dn = O.quantize_weight(bf16_normal(rng, (E, L, I), 0.02), wt)
    latent = bf16_normal(rng, (T, L), 1.0)
    ids, weights, _, _ = O.moe_route(rng.standard_normal((T, E)).astype(np.float32), None, k)
    want = O.moe_experts_reference(latent, ids, weights, gu, dn, I)
    lgu, ldn = abi.make_weight(wt, gu.data, gu.scale, gu.glob), abi.make_weight(wt, dn.data, dn.scale, dn.glob)
    out = np.zeros((T, L), dtype=np.float32)
    ws = np.zeros(max(int(ref.lx_moe_decode_workspace_bytes(T, I, k)), 16), dtype=np.uint8)
    assert ref.lx_moe_experts_decode(abi.ptr(latent), abi.ptr(ids), abi.ptr(weights), ctypes.byref(lgu), ctypes.byref(ldn),
                                     abi.ptr(out), abi.ptr(ws), T, L, I, k, None) == 0
    assert O.rel_l2(out, want) <= 1e-5
    out2 = np.zeros((T, L), dtype=np.float32)
    ws2 = np.zeros(max(int(ref.lx_moe_grouped_workspace_bytes(T, L, I, E, k, abi.MATH_BF16)), 16), dtype=np.uint8)
    assert ref.lx_moe_experts_grouped(abi.ptr(latent), abi.ptr(ids), abi.ptr(weights), ctypes.byref(lgu), ctypes.byref(ldn),
                                      abi.MATH_BF16, abi.ptr(out2), abi.ptr(ws2), T, L, I, E, k, None) == 0
    assert O.rel_l2(out2, want) <= 1e-5
