"""CPU restatement of the Dromos decode weight-streaming path. TEST INFRASTRUCTURE ONLY.

This module is the checker the parity tests, the smoke test and the CPU-baseline leg of the bench compare
the CUDA library against. The product never imports it. Everything here is numpy on the host; integer and
byte arithmetic is bit-exact by construction, floating point is float32 with IEEE division where the
reference divides, and float64 for the dot products (the "exact values the stored bytes stand for").

Parity pin: every function below is checked bit for bit (bytes, ids) or to float32 round-off (weights)
against the reference project's own CPU backend, compiled unmodified by oracle/Makefile into
oracle/_ref/libdromos_cpu.so, by tests/test_oracle_vs_reference.py, and against the committed fixtures under
tests/golden/ that were produced by calling that library (tests/golden/make_golden.py).

Reference citations are paths inside lernex/dromos.
"""

from __future__ import annotations

import numpy as np

W_BF16, W_INT8, W_FP8, W_NVFP4, W_BF16X = 0, 1, 2, 3, 4
MATH_BF16, MATH_INT8, MATH_FP8, MATH_FP4 = 0, 1, 2, 3

E2M1_GRID = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
E2M1_MIDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)

# ---------------------------------------------------------------------------------------------------
# bf16 <-> f32 (a bf16 is the top half of an f32; engine/cpu/cpu.h bf16_to_f32 / f32_to_bf16)
# ---------------------------------------------------------------------------------------------------


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 values."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (NaN stays NaN)."""
    u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16
    nan = (u & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
    return np.where(nan, (u >> 16) | np.uint32(0x40), rounded).astype(np.uint16)


# ---------------------------------------------------------------------------------------------------
# e4m3 ("fn": no inf, max 448) and e2m1 (engine/cpu/quant.cpp:11-54)
# ---------------------------------------------------------------------------------------------------


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """engine/cpu/quant.cpp:11-16, engine/cuda/wformat.cuh:26-29."""
    b = b.astype(np.uint32)
    mag = b & 0x7F
    normal = ((mag << 20) + np.uint32(120 << 23)).view(np.float32)
    sub = mag.astype(np.float32) * np.float32(2.0**-9)
    v = np.where(mag >= 8, normal, sub).astype(np.float32)
    return np.where((b & 0x80) != 0, -v, v).astype(np.float32)


def f32_to_e4m3(f: np.ndarray) -> np.ndarray:
    """Round to nearest even, saturating at 448; engine/cpu/quant.cpp:18-37."""
    f = np.ascontiguousarray(f, dtype=np.float32)
    u = f.view(np.uint32).copy()
    sign = ((u >> 24) & 0x80).astype(np.uint8)
    u &= np.uint32(0x7FFFFFFF)
    a = u.view(np.float32)
    out = np.zeros(f.shape, dtype=np.uint8)
    nan = u > np.uint32(0x7F800000)
    sat = (~nan) & (a >= np.float32(448.0))
    sub = (~nan) & (a < np.float32(2.0**-6))
    nor = ~(nan | sat | sub)
    out[nan] = 0x7F
    out[sat] = 0x7E
    out[sub] = np.rint(a[sub] * np.float32(512.0)).astype(np.uint8)
    un = u[nor]
    un = un + np.uint32(0x7FFFF) + ((un >> 20) & np.uint32(1))
    un &= np.uint32(0xFFF00000)
    e = (un >> 23).astype(np.int32) - 127 + 7
    m = ((un >> 20) & 7).astype(np.int32)
    code = ((e << 3) | m).astype(np.uint8)
    code[(e > 15) | ((e == 15) & (m == 7))] = 0x7E
    out[nor] = code
    return out | sign


def e2m1_to_f32(code: np.ndarray) -> np.ndarray:
    """engine/cpu/quant.cpp:39-43."""
    code = code.astype(np.uint8)
    v = E2M1_GRID[code & 7]
    return np.where((code & 8) != 0, -v, v).astype(np.float32)


def f32_to_e2m1(x: np.ndarray) -> np.ndarray:
    """Nearest e2m1, midpoints to the even code, saturating at 6, no sign on a zero result;
    engine/cpu/quant.cpp:45-54, engine/cuda/quant.cu:28-43."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    mag = np.minimum(np.abs(x), np.float32(6.0))
    idx = np.zeros(x.shape, dtype=np.int32)
    for mid in E2M1_MIDS:
        idx += mag > mid
    at_mid = np.zeros(x.shape, dtype=bool)
    for i, mid in enumerate(E2M1_MIDS):
        at_mid |= (idx == i) & (mag == mid) & bool(i & 1)
    idx = idx + at_mid
    sign = np.where((x < 0) & (idx > 0), 8, 0)
    return (idx | sign).astype(np.uint8)


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    """[..., K] 4-bit codes -> [..., K/2] bytes, the even k in the low nibble (kernels.h "Weight formats")."""
    c = codes.astype(np.uint8)
    return np.ascontiguousarray(c[..., 0::2] | (c[..., 1::2] << 4))


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    lo = packed & 0x0F
    hi = packed >> 4
    return np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], -1)


# ---------------------------------------------------------------------------------------------------
# Weight quantizers (engine/cpu/quant.cpp:66-140, engine/cuda/quant.cu:45-189, gemv.cu:700-720)
# ---------------------------------------------------------------------------------------------------


class Weight:
    """One weight (or stack) in a stored format: the fields of lx_weight (engine/cuda/kernels.h:411-417)."""

    def __init__(self, wtype, data, scale=None, glob=1.0, expert_global=None):
        self.wtype = wtype
        self.data = np.ascontiguousarray(data)
        self.scale = None if scale is None else np.ascontiguousarray(scale)
        self.glob = np.float32(glob)
        self.expert_global = expert_global


def quantize_weight(w_bits: np.ndarray, wtype: int) -> Weight:
    """w_bits: uint16 bf16 bits [..., N, K]. Returns the stored bytes the reference's lx_quantize_weight writes."""
    w = bf16_bits_to_f32(w_bits)
    if wtype == W_BF16:
        return Weight(W_BF16, w_bits)
    if wtype in (W_INT8, W_FP8):
        qmax = np.float32(127.0 if wtype == W_INT8 else 448.0)
        amax = np.abs(w).max(axis=-1).astype(np.float32)
        scale = np.where(amax > 0, amax / qmax, np.float32(1.0)).astype(np.float32)
        v = (w / scale[..., None]).astype(np.float32)
        if wtype == W_INT8:
            q = np.clip(np.rint(v), -127, 127).astype(np.int8)
        else:
            q = f32_to_e4m3(np.clip(v, np.float32(-448.0), np.float32(448.0)))
        return Weight(wtype, q, scale)
    if wtype == W_NVFP4:
        K = w.shape[-1]
        assert K % 16 == 0
        glob = np.float32(np.abs(w).max()) / np.float32(2688.0)
        blocks = w.reshape(*w.shape[:-1], K // 16, 16)
        bmax = np.abs(blocks).max(axis=-1).astype(np.float32)
        with np.errstate(divide="ignore", invalid="ignore"):
            s8 = f32_to_e4m3((bmax / (np.float32(6.0) * glob)).astype(np.float32))
            eff = (e4m3_to_f32(s8) * glob).astype(np.float32)
            codes = f32_to_e2m1((blocks / eff[..., None]).astype(np.float32))
        codes = np.where(eff[..., None] > 0, codes, 0).astype(np.uint8)
        return Weight(W_NVFP4, pack_nibbles(codes.reshape(w.shape)), s8, glob)
    raise ValueError(wtype)


def weight_values(wt: Weight) -> tuple[np.ndarray, np.ndarray]:
    """(v, row_factor): v float32 [..., N, K] are the exact per-element values WITHOUT the per-row factor
    (engine/cuda/wformat.cuh:4-8), row_factor float32 broadcastable to [..., N, 1]."""
    if wt.wtype == W_BF16:
        return bf16_bits_to_f32(wt.data), np.float32(1.0)
    if wt.wtype == W_INT8:
        return wt.data.astype(np.float32), wt.scale[..., None]
    if wt.wtype == W_FP8:
        return e4m3_to_f32(wt.data), wt.scale[..., None]
    if wt.wtype == W_NVFP4:
        vals = e2m1_to_f32(unpack_nibbles(wt.data))
        Kk = vals.shape[-1]
        s = e4m3_to_f32(wt.scale)
        v = (vals.reshape(*vals.shape[:-1], Kk // 16, 16) * s[..., None]).reshape(vals.shape).astype(np.float32)
        if wt.expert_global is not None:
            g = np.asarray(wt.expert_global, dtype=np.float32).reshape(-1, 1, 1)
        else:
            g = wt.glob
        return v, g
    raise ValueError(f"no direct values for weight type {wt.wtype} (decode BF16X with bf16x_decode first)")


def dequantize_weight(wt: Weight) -> np.ndarray:
    """bf16 bits of element * row factor, the f32 product rounded once (engine/cpu/quant.cpp:247-269)."""
    v, rf = weight_values(wt)
    if wt.wtype == W_BF16:
        return wt.data.copy()
    return f32_to_bf16_bits((v * np.float32(rf)).astype(np.float32))


def weight_f64(wt: Weight) -> np.ndarray:
    """The weight's exact values as float64 [..., N, K]."""
    v, rf = weight_values(wt)
    return v.astype(np.float64) * np.asarray(rf, dtype=np.float64)


# ---------------------------------------------------------------------------------------------------
# Activation quantizer (engine/cpu/quant.cpp:159-203, engine/cuda/kernels.h:479-493)
# ---------------------------------------------------------------------------------------------------


def quantize_act(x: np.ndarray, math: int):
    """x float32 [M, K] (bf16 inputs widened first) -> (q uint8, scale f32 [M], block_scale uint8 or None)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    a = np.abs(x).max(axis=-1).astype(np.float32)
    if math in (MATH_INT8, MATH_FP8):
        qmax = np.float32(127.0 if math == MATH_INT8 else 448.0)
        with np.errstate(divide="ignore"):
            inv = np.where(a > 0, qmax / a, np.float32(0.0)).astype(np.float32)
        v = (x * inv[:, None]).astype(np.float32)
        if math == MATH_INT8:
            q = np.clip(np.rint(v), -127, 127).astype(np.int8).view(np.uint8)
        else:
            q = f32_to_e4m3(v)
        scale = np.where(a > 0, a / qmax, np.float32(1.0)).astype(np.float32)
        return q, scale, None
    M, K = x.shape
    assert K % 16 == 0
    g = np.where(a > 0, a / np.float32(2688.0), np.float32(1.0)).astype(np.float32)
    blocks = x.reshape(M, K // 16, 16)
    bmax = np.abs(blocks).max(axis=-1).astype(np.float32)
    s8 = f32_to_e4m3((bmax / (np.float32(6.0) * g[:, None])).astype(np.float32))
    d = (e4m3_to_f32(s8) * g[:, None]).astype(np.float32)
    with np.errstate(divide="ignore"):
        r = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    codes = f32_to_e2m1((blocks * r[..., None]).astype(np.float32))
    codes = np.where(d[..., None] > 0, codes, 0).astype(np.uint8)
    return pack_nibbles(codes.reshape(M, K)), g, s8


def act_operand(x: np.ndarray, math: int) -> np.ndarray:
    """The activations as a product's math sees them, float64: x itself under BF16 math, else the per-row quantization
    of quantize_act times its scale (the reference's tests/kernels/wformats.py:174-180; INT8 and FP8 maths)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if math == MATH_BF16:
        return x.astype(np.float64)
    assert math in (MATH_INT8, MATH_FP8), "FP4 math is a product of other parts only"
    q, scale, _ = quantize_act(x, math)
    vals = q.view(np.int8).astype(np.float64) if math == MATH_INT8 else e4m3_to_f32(q).astype(np.float64)
    return vals * scale.astype(np.float64)[:, None]


# ---------------------------------------------------------------------------------------------------
# BF16X, the lossless encoding (engine/cuda/bf16x.cuh:13-49, engine/cpu/bf16x.cpp:60-199)
# ---------------------------------------------------------------------------------------------------

BF16X_BLOCK, BF16X_BLOCK_BYTES, BF16X_NO_PATCH, BF16X_MAX_K = 128, 192, 0xFFFFFFFF, 1 << 23


def bf16x_layout(K: int):
    """(B blocks, P patch slots, base offset, H header bytes, row bytes); engine/cuda/bf16x.cuh:42-49."""
    B = (K + 127) // 128
    H = (4 * (2 + K // 2048) + B + 7) // 8 * 8
    P = (H - B) // 4
    return B, P, 4 * P, H, H + 192 * B


def bf16x_row_bytes(K: int) -> int:
    return bf16x_layout(K)[4] if 0 < K < BF16X_MAX_K else -1


def _record_bytes(patches: int) -> int:
    return (4 * (patches + 2) + 7) // 8 * 8


def bf16x_encode(w_bits: np.ndarray) -> np.ndarray:
    """uint16 [rows, K] -> the encoding's bytes (rows * row_bytes, then overflow records in row order)."""
    rows, K = w_bits.shape
    B, P, bo, H, rb = bf16x_layout(K)
    Kp = 128 * B
    up = np.zeros((rows, Kp), dtype=np.uint32)
    up[:, :K] = w_bits
    valid = np.zeros((rows, Kp), dtype=bool)
    valid[:, :K] = True
    e = (up >> 7) & 0xFF
    e0 = np.where(valid, e, 0).reshape(rows, B, 128).max(axis=-1)
    e0k = np.repeat(e0, 128, axis=1)
    diff = e0k.astype(np.int64) - e.astype(np.int64)
    patched = valid & (diff > 15)
    code = np.where(valid & ~patched, diff, 0).astype(np.uint8)
    sm = np.where(valid, ((up >> 8) & 0x80) | (up & 0x7F), 0).astype(np.uint8)

    out = np.zeros((rows, rb), dtype=np.uint8)
    out[:, bo : bo + B] = e0.astype(np.uint8)
    blocks = np.zeros((rows, B, 192), dtype=np.uint8)
    blocks[:, :, :128] = sm.reshape(rows, B, 128)
    c = code.reshape(rows, B, 16, 8)
    blocks[:, :, 128:] = (c[..., :4] | (c[..., 4:] << 4)).reshape(rows, B, 64)
    out[:, H:] = blocks.reshape(rows, B * 192)

    slots = np.full((rows, P), BF16X_NO_PATCH, dtype=np.uint32)
    overflow = []
    region, offset = rows * rb, 0
    for r in np.nonzero(patched.any(axis=1))[0].tolist():
        ks = np.nonzero(patched[r])[0]
        entries = ((ks.astype(np.uint32) << 8) | e[r, ks]).astype(np.uint32)
        if len(entries) <= P:
            slots[r, : len(entries)] = entries
        else:
            size = _record_bytes(len(entries))
            rec = np.zeros(size // 4, dtype=np.uint32)
            rec[0] = len(entries)
            rec[1 : 1 + len(entries)] = entries
            rec[1 + len(entries)] = BF16X_NO_PATCH
            slots[r, 0] = 0x80000000 | ((region + offset - r * rb) // 8)
            overflow.append(rec)
            offset += size
    out[:, :bo] = slots.astype("<u4").view(np.uint8).reshape(rows, bo)
    flat = out.reshape(-1)
    if overflow:
        flat = np.concatenate([flat, np.concatenate(overflow).astype("<u4").view(np.uint8)])
    return flat


def bf16x_decode(data: np.ndarray, rows: int, K: int) -> np.ndarray:
    """The encoding's bytes -> uint16 [rows, K], every bit of the original (engine/cpu/bf16x.cpp:153-199)."""
    B, P, bo, H, rb = bf16x_layout(K)
    data = np.ascontiguousarray(data, dtype=np.uint8)
    recs = data[: rows * rb].reshape(rows, rb)
    bases = recs[:, bo : bo + B].astype(np.int32)
    blocks = recs[:, H:].reshape(rows, B, 192)
    sm = blocks[:, :, :128].astype(np.uint32)
    cw = blocks[:, :, 128:].reshape(rows, B, 16, 4)
    codes = np.concatenate([cw & 0x0F, cw >> 4], axis=-1).reshape(rows, B, 128).astype(np.int32)
    e = ((bases[:, :, None] - codes) & 0xFF).astype(np.uint32)
    vals = (((sm & 0x80) << 8) | (e << 7) | (sm & 0x7F)).astype(np.uint16).reshape(rows, B * 128)[:, :K].copy()
    slots = recs[:, :bo].copy().view("<u4").reshape(rows, P)
    for r in np.nonzero(slots[:, 0] != BF16X_NO_PATCH)[0].tolist():
        s0 = int(slots[r, 0])
        if s0 & 0x80000000:
            at = r * rb + (s0 & 0x7FFFFFFF) * 8
            n = int(data[at : at + 4].view("<u4")[0])
            lst = data[at + 4 : at + 4 + 4 * n].view("<u4")
        else:
            lst = slots[r]
        for p in lst.tolist():
            if p == BF16X_NO_PATCH:
                break
            k = p >> 8
            if k < K:
                vals[r, k] = (int(vals[r, k]) & 0x807F) | ((p & 0xFF) << 7)
    return vals


# ---------------------------------------------------------------------------------------------------
# Products (engine/cpu/gemm.cpp:21-34 epilogue; engine/cuda/gemv.cu:71-80, 511-513)
# ---------------------------------------------------------------------------------------------------


def product_f64(x: np.ndarray, wt: Weight) -> np.ndarray:
    """x float64 [M, K] times the weight's exact values: float64 [M, N], the row factor applied."""
    v, rf = weight_values(wt)
    N = v.shape[0]
    out = np.empty((x.shape[0], N), dtype=np.float64)
    step = max(1, (1 << 24) // max(1, v.shape[1]))
    for n0 in range(0, N, step):
        out[:, n0 : n0 + step] = x @ v[n0 : n0 + step].astype(np.float64).T
    return out * np.asarray(rf, dtype=np.float64).reshape(1, -1)


def gemv_reference(x, wt: Weight, bias=None, y_old=None, alpha=1.0, beta=0.0) -> np.ndarray:
    """y = alpha * (x @ W^T + bias) + beta * y_old in float64 (kernels.h lx_gemv_w / lx_gemm_w contract)."""
    t = product_f64(np.asarray(x, dtype=np.float64), wt)
    if bias is not None:
        t = t + np.asarray(bias, dtype=np.float64)[None, :]
    v = alpha * t
    if beta != 0.0:
        v = v + beta * np.asarray(y_old, dtype=np.float64)
    return v


# ---------------------------------------------------------------------------------------------------
# MoE: routing, grouping, experts (engine/cuda/route.cuh:18-81, moe_grouped.cu:1-17, 208-281; kernels.h:203-225)
# ---------------------------------------------------------------------------------------------------


def moe_route(logits: np.ndarray, bias, top_k: int):
    """ids int32 [T, top_k] (exact rule: descending logits + bias in f32, ties to the lower index), weights f32
    (softmax over the picks of the unbiased logits), entropy, confidence."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    T, E = logits.shape
    m = logits.max(axis=1, keepdims=True)
    ex = np.exp((logits - m).astype(np.float32)).astype(np.float32)
    z = ex.sum(axis=1, dtype=np.float32, keepdims=True)
    p = (ex / z).astype(np.float32)
    entropy = -(p * np.log(np.maximum(p, np.float32(1e-9)))).sum(axis=1, dtype=np.float32)
    confidence = (np.float32(1.0) / z[:, 0]).astype(np.float32)
    score = logits if bias is None else (logits + np.asarray(bias, dtype=np.float32)[None, :]).astype(np.float32)
    # stable argsort of -score: equal scores keep ascending index order
    order = np.argsort(-score.astype(np.float64), axis=1, kind="stable")
    ids = order[:, :top_k].astype(np.int32)
    picked = np.take_along_axis(logits, ids.astype(np.int64), axis=1)
    pe = np.exp((picked - picked.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float32)
    weights = (pe / pe.sum(axis=1, dtype=np.float32, keepdims=True)).astype(np.float32)
    return ids, weights, entropy.astype(np.float32), confidence


def moe_group(ids: np.ndarray, E: int):
    """The grouping the grouped expert GEMM sorts by: pairs p = t * top_k + k stably sorted by expert.
    Returns (counts [E], offsets [E + 1], pairs [P]); engine/cuda/moe_grouped.cu:1-6, 110-254."""
    flat = ids.reshape(-1).astype(np.int64)
    counts = np.bincount(flat, minlength=E).astype(np.int32)
    offsets = np.zeros(E + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    pairs = np.argsort(flat, kind="stable").astype(np.int32)
    return counts, offsets, pairs


def silu(v):
    return v / (1.0 + np.exp(-v))


def moe_experts_reference(latent_bits, ids, weights, gate_up: Weight, down: Weight, I: int, math: int = MATH_BF16) -> np.ndarray:
    """out[t] = sum_k w[t, k] * down[e] @ bf16(silu(gate . x) * (up . x)), float64 except the one bf16 rounding of
    the intermediate (kernels.h:217-225, 495-511). gate_up [E, 2I, L], down [E, L, I]. Under the INT8 / FP8 maths the
    latent (per token) and the rounded intermediate (per pair row) are what act_operand makes of them
    (engine/cuda/moe_grouped.cu:434-490; tests/kernels/test_moe_grouped.py:99-118)."""
    x = act_operand(bf16_bits_to_f32(latent_bits), math)
    T, L = x.shape
    gu = weight_f64(gate_up)
    dn = weight_f64(down)
    out = np.zeros((T, L), dtype=np.float64)
    for t in range(T):
        for k in range(ids.shape[1]):
            e = int(ids[t, k])
            h = gu[e] @ x[t]
            mid = (silu(h[:I]) * h[I:]).astype(np.float32)
            mid = act_operand(bf16_bits_to_f32(f32_to_bf16_bits(mid))[None, :], math)[0]
            out[t] += float(weights[t, k]) * (dn[e] @ mid)
    return out


# ---------------------------------------------------------------------------------------------------
# Algorithmic bytes (bench/bench_gemv.py:51-56, engine/model/traffic.cpp:23-52 of the reference)
# ---------------------------------------------------------------------------------------------------


def weight_bytes(wtype: int, N: int, K: int, bf16x_total: int | None = None) -> int:
    if wtype == W_BF16:
        return 2 * N * K
    if wtype in (W_INT8, W_FP8):
        return N * K + 4 * N
    if wtype == W_NVFP4:
        return N * K // 2 + N * K // 16 + 4
    if wtype == W_BF16X:
        return bf16x_total if bf16x_total is not None else N * bf16x_row_bytes(K)
    raise ValueError(wtype)


# ---------------------------------------------------------------------------------------------------
# Comparison helpers shared by the tests
# ---------------------------------------------------------------------------------------------------


def rel_l2(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    d = np.linalg.norm(want.ravel())
    return float(np.linalg.norm((got - want).ravel()) / (d if d > 0 else 1.0))


def max_abs(got, want) -> float:
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - np.asarray(want, dtype=np.float64)))) if np.size(got) else 0.0
