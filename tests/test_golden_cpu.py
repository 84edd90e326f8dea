"""The oracle against the committed golden fixtures (outputs of the reference's own CPU backend on seeded inputs,
made by tests/golden/make_golden.py). Runs without a GPU and without the reference checkout."""

import os

import numpy as np

from oracle import dromos_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLDEN, name))


def test_weight_quantizers_and_dequantized_values_bit_exact():
    g = load("quantizers.npz")
    w = g["w"]
    for name, wt in (("int8", O.W_INT8), ("fp8", O.W_FP8), ("nvfp4", O.W_NVFP4)):
        q = O.quantize_weight(w, wt)
        assert np.array_equal(q.data.view(np.uint8).reshape(-1), g[f"{name}_data"]), name
        assert np.array_equal(q.scale.view(np.uint8).reshape(-1), g[f"{name}_scale"].view(np.uint8).reshape(-1)), name
        assert np.float32(q.glob).tobytes() == np.float32(g[f"{name}_global"]).tobytes(), name
        assert np.array_equal(O.dequantize_weight(q), g[f"{name}_deq"]), name


def test_products_match_reference_outputs():
    g = load("quantizers.npz")
    w = g["w"]
    for name, wt in (("int8", O.W_INT8), ("fp8", O.W_FP8), ("nvfp4", O.W_NVFP4)):
        q = O.quantize_weight(w, wt)
        x = O.bf16_bits_to_f32(g[f"{name}_x"]).astype(np.float64)
        want = g[f"{name}_y"]
        got = O.gemv_reference(x, q)
        assert O.rel_l2(got, want) <= 1e-5 and O.max_abs(got, want) <= 1e-4 * np.abs(want).max(), name


def test_bf16x_encoding_byte_exact_and_lossless():
    g = load("bf16x.npz")
    i = 0
    while f"w{i}" in g:
        w, enc = g[f"w{i}"], g[f"enc{i}"]
        mine = O.bf16x_encode(w)
        assert mine.size == enc.size and np.array_equal(mine, enc), f"case {i}"
        assert np.array_equal(O.bf16x_decode(enc, *w.shape), w), f"case {i}"
        assert O.bf16x_row_bytes(w.shape[1]) == int(g[f"row_bytes{i}"])
        i += 1
    assert i == 5
    assert O.bf16x_row_bytes(4096) == 6192 and O.bf16x_row_bytes(8192) == 12376 and O.bf16x_row_bytes(1536) == 2328
    assert O.bf16x_row_bytes(0) == -1 and O.bf16x_row_bytes(1 << 23) == -1


def test_activation_quantizer_bit_exact():
    g = load("quantize_act.npz")
    for math in (1, 2, 3):
        q, s, bs = O.quantize_act(g["x"], math)
        assert np.array_equal(q, g[f"q{math}"]) and np.array_equal(s.view(np.uint32), g[f"s{math}"].view(np.uint32))
        if bs is not None:
            assert np.array_equal(bs, g[f"bs{math}"])


def test_routing_ids_exact_and_weights_close():
    g = load("moe.npz")
    for tag, b in (("nobias", None), ("bias", g["bias"])):
        ids, w, ent, conf = O.moe_route(g["logits"], b, 8)
        assert np.array_equal(ids, g[f"ids_{tag}"])
        assert np.abs(w - g[f"weights_{tag}"]).max() <= 1e-5
        assert np.abs(ent - g[f"entropy_{tag}"]).max() <= 1e-5 and np.abs(conf - g[f"confidence_{tag}"]).max() <= 1e-5


def test_routed_experts_match_reference_outputs():
    g = load("moe.npz")
    gu = O.quantize_weight(g["e_gate_up"], O.W_FP8)
    dn = O.quantize_weight(g["e_down"], O.W_FP8)
    got = O.moe_experts_reference(g["e_latent"], g["e_ids"], g["e_weights"], gu, dn, 64)
    want = g["e_out"]
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()


def test_grouping_is_a_stable_sort_by_expert():
    ids = np.array([[3, 1], [1, 3], [0, 3], [1, 1]], dtype=np.int32)
    counts, offsets, pairs = O.moe_group(ids, 4)
    assert counts.tolist() == [1, 4, 0, 3] and offsets.tolist() == [0, 1, 5, 5, 8]
    assert pairs.tolist() == [4, 1, 2, 6, 7, 0, 3, 5]


def test_number_formats_round_trip_every_code():
    codes = np.arange(256, dtype=np.uint8)
    finite = (codes & 0x7F) != 0x7F
    assert np.array_equal(O.f32_to_e4m3(O.e4m3_to_f32(codes[finite])), np.where(codes[finite] == 0x80, 0x80, codes[finite]))
    nib = np.arange(16, dtype=np.uint8)
    back = O.f32_to_e2m1(O.e2m1_to_f32(nib))
    assert np.array_equal(back, np.where(nib == 8, 0, nib))  # minus zero carries no sign
    # ties go to the even code
    assert O.f32_to_e2m1(np.float32([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25])).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 0]
