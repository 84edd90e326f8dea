"""Few-token routed experts through the C ABI: lx_moe_experts_decode on every stored format, lx_moe_experts_bf16x,
lx_moe_experts_decode_bf16 and lx_moe_experts, against the float64 oracle (intermediate rounded to bf16 as the contract
says) and against each other bit for bit where the contract promises it.

Mirrors the reference's tests/kernels/test_moe_decode.py (shapes, repeated experts, mixed formats per stack, per-expert
NVFP4 globals, batch invariance, the refused cases) and the expert part of tests/kernels/test_bf16x.py.
"""

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu
FORMATS = {"bf16": O.W_BF16, "int8": O.W_INT8, "fp8": O.W_FP8, "nvfp4": O.W_NVFP4}
METIS = (1024, 512, 4)  # L, I, top_k of the reference's small model


def stacks(gu_type, dn_type, E, L, I, seed):
    gu_bits = util.bf16_normal((E, 2 * I, L), 0.02, seed)
    dn_bits = util.bf16_normal((E, L, I), 0.02, seed + 1)
    return O.quantize_weight(gu_bits, gu_type), O.quantize_weight(dn_bits, dn_type)


def make_inputs(T, E, L, top_k, seed, pool=None):
    rng = np.random.default_rng(seed)
    latent = util.bf16_normal((T, L), 1.0, seed + 2)
    choose = np.arange(E) if pool is None else np.asarray(pool)
    ids = np.stack([rng.permutation(choose)[:top_k] for _ in range(T)]).astype(np.int32)
    w = rng.standard_normal((T, top_k)).astype(np.float32)
    w = np.exp(w - w.max(axis=1, keepdims=True))
    weights = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return latent, ids, weights


def run_decode(lx, latent, ids, weights, dgu, ddn, I, expect=0):
    """The kernel in a workspace of exactly the reported size, filled with 0xFF bytes first; out starts as NaN."""
    T, L = latent.shape
    top_k = ids.shape[1]
    nbytes = lx.lx_moe_decode_workspace_bytes(T, I, top_k)
    assert nbytes >= 2 * T * top_k * I
    ws = torch.full((max(nbytes, 16),), 0xFF, dtype=torch.uint8, device="cuda")
    out = torch.full((T, L), float("nan"), device="cuda")
    latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)
    st = lx.lx_moe_experts_decode(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(), abi.ptr(out),
                                  abi.ptr(ws), T, L, I, top_k, util.stream_ptr())
    assert st == expect, st
    util.check_status(lx)
    return util.host(out)


def check(lx, latent, ids, weights, gu, dn, I):
    got = run_decode(lx, latent, ids, weights, util.DeviceWeight(gu), util.DeviceWeight(dn), I)
    want = O.moe_experts_reference(latent, ids, weights, gu, dn, I)
    # the reference suite's bound: 1e-3 of max|out| absolute plus 1e-3 relative; and the acceptance bound
    assert np.all(np.abs(got - want) <= 1e-3 * np.abs(want).max() + 1e-3 * np.abs(want))
    util.assert_close(got, want, what="decode experts")
    return got


@pytest.mark.parametrize("fmt", list(FORMATS))
@pytest.mark.parametrize("T", [1, 2, 4, 8])
def test_model_shapes(lx, T, fmt):
    L, I, top_k = METIS
    E = 32
    gu, dn = stacks(FORMATS[fmt], FORMATS[fmt], E, L, I, seed=T + 1)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=T * 13)
    check(lx, latent, ids, weights, gu, dn, I)


@pytest.mark.parametrize("T,E,L,I,top_k", [(1, 1, 16, 16, 1), (3, 5, 48, 32, 2), (5, 9, 64, 48, 3), (8, 8, 32, 64, 8), (2, 6, 1024, 16, 4)])
@pytest.mark.parametrize("fmt", list(FORMATS))
def test_odd_shapes(lx, T, E, L, I, top_k, fmt):
    gu, dn = stacks(FORMATS[fmt], FORMATS[fmt], E, L, I, seed=E + 3)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=T + E)
    check(lx, latent, ids, weights, gu, dn, I)


@pytest.mark.parametrize("gu_fmt,dn_fmt", [("nvfp4", "fp8"), ("fp8", "nvfp4"), ("int8", "bf16"), ("bf16", "nvfp4")])
def test_mixed_formats_per_stack(lx, gu_fmt, dn_fmt):
    T, E = 4, 16
    L, I, top_k = METIS
    gu, dn = stacks(FORMATS[gu_fmt], FORMATS[dn_fmt], E, L, I, seed=21)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=23)
    check(lx, latent, ids, weights, gu, dn, I)


def test_repeated_experts(lx):
    """Tokens share a small pool of experts: most expert rows serve several pairs in one pass."""
    T, E = 8, 128
    L, I, top_k = METIS
    gu, dn = stacks(O.W_NVFP4, O.W_NVFP4, E, L, I, seed=31)
    pool = np.random.default_rng(33).permutation(E)[:6]
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=33, pool=pool)
    check(lx, latent, ids, weights, gu, dn, I)


def test_an_expert_named_twice_by_one_token(lx):
    """More member pairs of one expert than tokens: nine pairs name expert 2 (one token names it twice)."""
    T, E, L, I, top_k = 8, 6, 256, 64, 3
    gu, dn = stacks(O.W_FP8, O.W_INT8, E, L, I, seed=35)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=36)
    ids[:, 0] = 2
    ids[:, 1] = np.where(ids[:, 1] == 2, 3, ids[:, 1])
    ids[:, 2] = np.where(ids[:, 2] == 2, 4, ids[:, 2])
    ids[5, 2] = 2
    check(lx, latent, ids, weights, gu, dn, I)


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_deterministic_and_token_independent(lx, fmt):
    T, E = 8, 32
    L, I, top_k = METIS
    gu, dn = stacks(FORMATS[fmt], FORMATS[fmt], E, L, I, seed=41)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=43)
    first = run_decode(lx, latent, ids, weights, dgu, ddn, I)
    second = run_decode(lx, latent, ids, weights, dgu, ddn, I)
    assert np.array_equal(first.view(np.uint32), second.view(np.uint32))
    head = run_decode(lx, latent[:1], ids[:1], weights[:1], dgu, ddn, I)
    assert np.array_equal(head.view(np.uint32), first[:1].view(np.uint32))


@pytest.mark.parametrize("fmt", list(FORMATS))
def test_rows_do_not_depend_on_the_batch(lx, fmt):
    """Each token of a batch of T (1 to 8) equals that token run alone, with experts shared between tokens (E = 12)."""
    L, I, top_k = METIS
    E = 12
    gu, dn = stacks(FORMATS[fmt], FORMATS[fmt], E, L, I, seed=51)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    latent, ids, weights = make_inputs(8, E, L, top_k, seed=53)
    alone = np.concatenate([run_decode(lx, latent[t:t + 1], ids[t:t + 1], weights[t:t + 1], dgu, ddn, I) for t in range(8)])
    for T in range(1, 9):
        out = run_decode(lx, latent[:T], ids[:T], weights[:T], dgu, ddn, I)
        assert np.array_equal(out.view(np.uint32), alone[:T].view(np.uint32)), f"a token of a T={T} batch differs from the token alone"


def test_rejects_more_than_eight_tokens_and_nine_experts_per_token(lx):
    L, I, top_k = METIS
    gu, dn = stacks(O.W_BF16, O.W_BF16, 16, L, I, seed=51)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    latent, ids, weights = make_inputs(9, 16, L, top_k, seed=53)
    run_decode(lx, latent, ids, weights, dgu, ddn, I, expect=1)
    latent, ids, weights = make_inputs(2, 16, L, 9, seed=54)
    run_decode(lx, latent, ids, weights, dgu, ddn, I, expect=1)


def test_global_is_per_expert(lx):
    """The down stack's per-expert NVFP4 global enters linearly: doubling expert 1's doubles the output exactly; expert 3,
    which has weight 0, changes nothing."""
    T, E = 1, 4
    L, I, _ = METIS
    gu, dn = stacks(O.W_NVFP4, O.W_NVFP4, E, L, I, seed=61)
    dn.expert_global = np.full(E, dn.glob, dtype=np.float32)
    latent, _, _ = make_inputs(T, E, L, 2, seed=63)
    ids = np.array([[1, 3]], dtype=np.int32)
    weights = np.array([[1.0, 0.0]], dtype=np.float32)
    dgu = util.DeviceWeight(gu)
    base = run_decode(lx, latent, ids, weights, dgu, util.DeviceWeight(dn), I)
    dn.expert_global[3] *= 2.0
    assert np.array_equal(run_decode(lx, latent, ids, weights, dgu, util.DeviceWeight(dn), I), base)
    dn.expert_global[1] *= 2.0
    assert np.array_equal(run_decode(lx, latent, ids, weights, dgu, util.DeviceWeight(dn), I), base * 2.0)


def plain_call(lx, fn, latent, ids, weights, gu_d, dn_d, I, with_ws=True):
    T, L = latent.shape
    top_k = ids.shape[1]
    out = torch.full((T, L), float("nan"), device="cuda")
    latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)
    args = [abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), abi.ptr(gu_d), abi.ptr(dn_d), abi.ptr(out)]
    if with_ws:
        ws = torch.full((max(lx.lx_moe_bf16x_workspace_bytes(T, I, top_k), 16),), 0xFF, dtype=torch.uint8, device="cuda")
        args.append(abi.ptr(ws))
    st = getattr(lx, fn)(*args, T, L, I, top_k, util.stream_ptr())
    assert st == 0, st
    util.check_status(lx)
    return util.host(out)


def lossless_stacks(E, L, I, seed, wide=False):
    """bf16 stacks and their BF16X encodings (stacks are rows back to back: [E * 2I, L] and [E * L, I]). wide: a few
    values far below their block's largest exponent, in a few rows more of them than the header has slots for, so that
    rows with patches in the header and rows with an overflow record both occur."""
    gu_bits = util.bf16_normal((E, 2 * I, L), 0.02, seed)
    dn_bits = util.bf16_normal((E, L, I), 0.02, seed + 1)
    if wide:
        rng = np.random.default_rng(seed)
        tiny = O.f32_to_bf16_bits(np.array([1e-30, -3e-28, 2e-25], dtype=np.float32))
        for bits in (gu_bits, dn_bits):
            flat = bits.reshape(-1, bits.shape[-1])
            for r in rng.choice(flat.shape[0], size=12, replace=False):
                n = 2 if r % 3 else min(40, flat.shape[1] // 2)
                cols = rng.choice(flat.shape[1], size=n, replace=False)
                flat[r, cols] = tiny[rng.integers(0, 3, size=n)]
    gu_enc = O.bf16x_encode(gu_bits.reshape(-1, L))
    dn_enc = O.bf16x_encode(dn_bits.reshape(-1, I))
    return gu_bits, dn_bits, gu_enc, dn_enc


@pytest.mark.parametrize("T,E,L,I,top_k,wide", [(4, 8, 256, 128, 2, False), (3, 6, 384, 200, 3, True), (8, 16, 1024, 512, 4, True)])
def test_lossless_stacks_give_the_bits_of_the_bf16_stacks(lx, T, E, L, I, top_k, wide):
    gu_bits, dn_bits, gu_enc, dn_enc = lossless_stacks(E, L, I, seed=5 + T, wide=wide)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=21)
    gu_d, dn_d, gue_d, dne_d = util.dev(gu_bits), util.dev(dn_bits), util.dev(gu_enc), util.dev(dn_enc)
    plain = plain_call(lx, "lx_moe_experts", latent, ids, weights, gu_d, dn_d, I, with_ws=False)
    decode = plain_call(lx, "lx_moe_experts_decode_bf16", latent, ids, weights, gu_d, dn_d, I)
    lossless = plain_call(lx, "lx_moe_experts_bf16x", latent, ids, weights, gue_d, dne_d, I)
    assert np.array_equal(decode.view(np.uint32), plain.view(np.uint32))
    assert np.array_equal(lossless.view(np.uint32), plain.view(np.uint32))
    # and through lx_moe_experts_decode: BF16X descriptors run the lossless experts, bf16 descriptors the same sums
    gu_w, dn_w = O.Weight(O.W_BF16, gu_bits), O.Weight(O.W_BF16, dn_bits)
    via_bf16 = run_decode(lx, latent, ids, weights, util.DeviceWeight(gu_w), util.DeviceWeight(dn_w), I)
    via_x = run_decode(lx, latent, ids, weights, util.DeviceWeight(O.Weight(O.W_BF16X, gu_enc)),
                       util.DeviceWeight(O.Weight(O.W_BF16X, dn_enc)), I)
    assert np.array_equal(via_bf16.view(np.uint32), plain.view(np.uint32))
    assert np.array_equal(via_x.view(np.uint32), plain.view(np.uint32))
    want = O.moe_experts_reference(latent, ids, weights, gu_w, dn_w, I)
    util.assert_close(plain, want, what="bf16 experts")


def test_bf16_experts_of_any_length(lx):
    """lx_moe_experts takes any T (more pairs than the decode kernels scan for shared experts) and any top_k."""
    T, E, L, I, top_k = 37, 12, 256, 96, 9
    gu_bits, dn_bits, _, _ = lossless_stacks(E, L, I, seed=9)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=22)
    got = plain_call(lx, "lx_moe_experts", latent, ids, weights, util.dev(gu_bits), util.dev(dn_bits), I, with_ws=False)
    want = O.moe_experts_reference(latent, ids, weights, O.Weight(O.W_BF16, gu_bits), O.Weight(O.W_BF16, dn_bits), I)
    util.assert_close(got, want, what="lx_moe_experts")
    head = plain_call(lx, "lx_moe_experts", latent[:1], ids[:1], weights[:1], util.dev(gu_bits), util.dev(dn_bits), I, with_ws=False)
    assert np.array_equal(head.view(np.uint32), got[:1].view(np.uint32))


def test_mixed_lossless_pair_is_refused(lx):
    T, E, L, I, top_k = 2, 4, 128, 64, 2
    gu_bits, dn_bits, gu_enc, _ = lossless_stacks(E, L, I, seed=5)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=23)
    dgu = util.DeviceWeight(O.Weight(O.W_BF16X, gu_enc))
    ddn = util.DeviceWeight(O.Weight(O.W_BF16, dn_bits))
    run_decode(lx, latent, ids, weights, dgu, ddn, I, expect=801)


def test_short_rows_are_refused_as_the_reference_refuses_them(lx):
    """Rows that are not whole 8-byte words (bf16 K % 4, 8-bit K % 8): invalid value, nothing launched."""
    T, E, L, I, top_k = 1, 2, 20, 16, 1
    gu, dn = stacks(O.W_FP8, O.W_FP8, E, L, I, seed=3)
    latent, ids, weights = make_inputs(T, E, L, top_k, seed=4)
    run_decode(lx, latent, ids, weights, util.DeviceWeight(gu), util.DeviceWeight(dn), I, expect=1)
