"""Generates the golden fixtures under tests/golden/ by calling the reference project's own CPU backend
(oracle/_ref/libdromos_cpu.so, built by `make -C oracle ref` from the reference checkout) on seeded inputs.

    python tests/golden/make_golden.py

Each .npz holds the inputs' seeds / bits and the reference's outputs: quantized bytes and scales, dequantized bf16,
BF16X encodings (with patches and overflow records), activation quantization, routing, and decode products. The
fixtures let the oracle (and through it the CUDA library) be checked on machines that have neither the reference
checkout nor its compiled backend.
"""

import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from dromos_b200 import abi  # noqa: E402
from oracle import dromos_oracle as O  # noqa: E402


def bf16_normal(rng, shape, std):
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32))


def main():
    ref = abi.Library(os.path.join(ROOT, "oracle", "_ref", "libdromos_cpu.so"))
    rng = np.random.default_rng(20240607)

    # ---- weight quantizers and dequantization ----
    N, K = 48, 256
    w = bf16_normal(rng, (N, K), 0.02)
    w[3] = 0
    w[5, 7] = 0x8000
    w[6, :64] = 0
    out = {"w": w}
    for name, wt in (("int8", O.W_INT8), ("fp8", O.W_FP8), ("nvfp4", O.W_NVFP4)):
        data = np.zeros(N * (K // 2 if wt == O.W_NVFP4 else K), dtype=np.uint8)
        scale = np.zeros(N * K // 16, dtype=np.uint8) if wt == O.W_NVFP4 else np.zeros(N, dtype=np.float32)
        lw = abi.make_weight(wt, data, scale)
        assert ref.lx_quantize_weight(abi.ptr(w), ctypes.byref(lw), N, K, None) == 0
        deq = np.zeros((N, K), dtype=np.uint16)
        assert ref.lx_dequantize_weight(ctypes.byref(lw), abi.ptr(deq), N, K, None) == 0
        out[f"{name}_data"], out[f"{name}_scale"], out[f"{name}_deq"] = data, scale, deq
        out[f"{name}_global"] = np.float32(lw.glob)
        # decode products of the reference on its own stored weights (f32 outputs), M = 3
        x = bf16_normal(rng, (3, K), 1.0)
        y = np.zeros((3, N), dtype=np.float32)
        assert ref.lx_gemv_w(abi.ptr(x), abi.BF16, K, ctypes.byref(lw), None, abi.BF16, abi.ptr(y), abi.F32, N, 3, N, K, 1.0, 0.0,
                             None) == 0
        out[f"{name}_x"], out[f"{name}_y"] = x, y
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **out)

    # ---- BF16X ----
    out = {}
    for i, (rows, Kx) in enumerate([(7, 13), (20, 256), (5, 1000), (4, 2048), (6, 4096)]):
        wx = bf16_normal(rng, (rows, Kx), 0.02)
        wx[0, ::5] = O.f32_to_bf16_bits(np.float32([2.0**-100]))[0]           # more patches than slots: overflow record
        if Kx > 5:
            wx[rows - 1, 5] = O.f32_to_bf16_bits(np.float32([-(2.0**-120)]))[0]  # one patch in the header slots
        wx[rows // 2, 0] = 0x7FC0                                              # NaN
        wx[rows // 2, 1 % Kx] = 0xFF80                                         # -inf
        n = ref.lx_bf16x_bytes(abi.ptr(wx), rows, Kx, None)
        buf = np.zeros(n, dtype=np.uint8)
        assert ref.lx_bf16x_encode(abi.ptr(wx), rows, Kx, abi.ptr(buf), n, None) == 0
        back = np.zeros((rows, Kx), dtype=np.uint16)
        assert ref.lx_bf16x_decode(abi.ptr(buf), rows, Kx, abi.ptr(back), None) == 0
        assert np.array_equal(back, wx)
        out[f"w{i}"], out[f"enc{i}"] = wx, buf
        out[f"row_bytes{i}"] = np.int64(ref.lx_bf16x_row_bytes(Kx))
    np.savez_compressed(os.path.join(HERE, "bf16x.npz"), **out)

    # ---- activation quantizer ----
    M, Ka = 5, 256
    x = rng.standard_normal((M, Ka)).astype(np.float32)
    x[2] = 0
    out = {"x": x}
    for math in (1, 2, 3):
        q = np.zeros((M, Ka // 2 if math == 3 else Ka), dtype=np.uint8)
        s = np.zeros(M, dtype=np.float32)
        bs = np.zeros((M, Ka // 16), dtype=np.uint8)
        assert ref.lx_quantize_act(abi.ptr(x), abi.F32, Ka, math, abi.ptr(q), q.shape[1], abi.ptr(s), abi.ptr(bs), Ka // 16, M, Ka,
                                   None) == 0
        out[f"q{math}"], out[f"s{math}"], out[f"bs{math}"] = q, s, bs
    np.savez_compressed(os.path.join(HERE, "quantize_act.npz"), **out)

    # ---- routing and routed experts ----
    T, E, k = 33, 64, 8
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[0, :] = 0.5
    logits[1, 3] = logits[1, 9]
    bias = (rng.standard_normal(E) * 0.1).astype(np.float32)
    out = {"logits": logits, "bias": bias}
    for tag, b in (("nobias", None), ("bias", bias)):
        ids = np.zeros((T, k), dtype=np.int32)
        wts = np.zeros((T, k), dtype=np.float32)
        ent = np.zeros(T, dtype=np.float32)
        conf = np.zeros(T, dtype=np.float32)
        assert ref.lx_moe_route(abi.ptr(logits), abi.ptr(b), abi.ptr(ids), abi.ptr(wts), abi.ptr(ent), abi.ptr(conf), T, E, k, None) == 0
        out[f"ids_{tag}"], out[f"weights_{tag}"], out[f"entropy_{tag}"], out[f"confidence_{tag}"] = ids, wts, ent, conf
    # experts: fp8 stacks, reference grouped kernel under BF16 math
    Te, L, I, Ee, ke = 6, 128, 64, 8, 2
    gu_bits = bf16_normal(rng, (Ee, 2 * I, L), 0.02)
    dn_bits = bf16_normal(rng, (Ee, L, I), 0.02)
    latent = bf16_normal(rng, (Te, L), 1.0)
    lg = rng.standard_normal((Te, Ee)).astype(np.float32)
    ids = np.zeros((Te, ke), dtype=np.int32)
    wts = np.zeros((Te, ke), dtype=np.float32)
    assert ref.lx_moe_route(abi.ptr(lg), None, abi.ptr(ids), abi.ptr(wts), abi.ptr(np.zeros(Te, np.float32)),
                            abi.ptr(np.zeros(Te, np.float32)), Te, Ee, ke, None) == 0
    stacks = []
    for bits, rows, cols in ((gu_bits, Ee * 2 * I, L), (dn_bits, Ee * L, I)):
        data = np.zeros(rows * cols, dtype=np.uint8)
        scale = np.zeros(rows, dtype=np.float32)
        lw = abi.make_weight(O.W_FP8, data, scale)
        assert ref.lx_quantize_weight(abi.ptr(bits), ctypes.byref(lw), rows, cols, None) == 0
        stacks.append((lw, data, scale))
    need = ref.lx_moe_grouped_workspace_bytes(Te, L, I, Ee, ke, 0)
    ws = np.zeros(max(need, 1 << 20), dtype=np.uint8)
    outp = np.zeros((Te, L), dtype=np.float32)
    assert ref.lx_moe_experts_grouped(abi.ptr(latent), abi.ptr(ids), abi.ptr(wts), ctypes.byref(stacks[0][0]), ctypes.byref(stacks[1][0]),
                                      0, abi.ptr(outp), abi.ptr(ws), Te, L, I, Ee, ke, None) == 0
    out.update({"e_gate_up": gu_bits, "e_down": dn_bits, "e_latent": latent, "e_ids": ids, "e_weights": wts, "e_out": outp})
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
