"""Mixture-of-experts parity through the C ABI: lx_moe_route (ids exact, weights / entropy / confidence to 1e-5), the
grouping the expert GEMM sorts by (exact), and lx_moe_experts_grouped against the float64 oracle.

Mirrors the reference's tests/kernels/test_moe.py and test_moe_grouped.py.
"""

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu
NAMES = {O.W_BF16: "bf16", O.W_INT8: "int8", O.W_FP8: "fp8", O.W_NVFP4: "nvfp4"}


def route(lx, logits, bias, top_k):
    T, E = logits.shape
    ids = torch.full((T, top_k), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros((T, top_k), dtype=torch.float32, device="cuda")
    ent = torch.zeros(T, dtype=torch.float32, device="cuda")
    conf = torch.zeros(T, dtype=torch.float32, device="cuda")
    logits_d = util.dev(logits)
    bias_d = None if bias is None else util.dev(bias)
    st = lx.lx_moe_route(abi.ptr(logits_d), abi.ptr(bias_d), abi.ptr(ids), abi.ptr(w), abi.ptr(ent), abi.ptr(conf), T, E, top_k,
                         util.stream_ptr())
    assert st == 0
    torch.cuda.synchronize()
    return util.host(ids), util.host(w), util.host(ent), util.host(conf)


@pytest.mark.parametrize("T,E,top_k", [(1, 8, 2), (5, 64, 8), (32, 64, 8), (33, 128, 4), (7, 1000, 32)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_route_matches_oracle(lx, T, E, top_k, with_bias):
    logits = util.f32_normal((T, E), 1.0, T + E)
    bias = util.f32_normal((E,), 0.1, 3) if with_bias else None
    ids, w, ent, conf = route(lx, logits, bias, top_k)
    ids_o, w_o, ent_o, conf_o = O.moe_route(logits, bias, top_k)
    assert np.array_equal(ids, ids_o)
    assert np.abs(w - w_o).max() <= 1e-5 and np.abs(ent - ent_o).max() <= 1e-5 and np.abs(conf - conf_o).max() <= 1e-5


def test_route_ties_go_to_the_lower_index(lx):
    logits = np.zeros((2, 6), dtype=np.float32)
    logits[0] = [1.0, 3.0, 3.0, 0.0, 3.0, -1.0]
    logits[1] = 0.5
    ids, w, _, _ = route(lx, logits, None, 3)
    assert ids[0].tolist() == [1, 2, 4] and ids[1].tolist() == [0, 1, 2]
    assert np.allclose(w, 1.0 / 3.0, atol=1e-6)
    bias = np.array([0, 0, 0, 10.0, 0, 0], dtype=np.float32)  # the bias picks, the unbiased logits weigh
    ids, w, _, _ = route(lx, logits[:1], bias, 2)
    assert ids[0].tolist() == [3, 1]
    e = np.exp(np.array([0.0, 3.0]) - 3.0)
    assert np.allclose(w[0], e / e.sum(), atol=1e-6)


def experts_case(lx, wtype, T, L, I, E, top_k, seed=0, ids_override=None, per_expert_global=False):
    gu_bits = util.bf16_normal((E, 2 * I, L), 0.02, seed)
    dn_bits = util.bf16_normal((E, L, I), 0.02, seed + 1)
    gu, dn = O.quantize_weight(gu_bits, wtype), O.quantize_weight(dn_bits, wtype)
    if per_expert_global and wtype == O.W_NVFP4:
        gu.expert_global = (np.float32(gu.glob) * (1.0 + 0.25 * np.arange(E))).astype(np.float32)
    latent = util.bf16_normal((T, L), 1.0, seed + 2)
    logits = util.f32_normal((T, E), 1.0, seed + 3)
    ids, weights, _, _ = O.moe_route(logits, None, top_k)
    if ids_override is not None:
        ids = ids_override(ids)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    out = torch.full((T, L), float("nan"), device="cuda")
    nbytes = lx.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, abi.MATH_BF16)
    ws = torch.full((nbytes,), 0xFF, dtype=torch.uint8, device="cuda")  # garbage: nothing may be assumed zero
    latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)  # kept alive across the call
    st = lx.lx_moe_experts_grouped(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(), abi.MATH_BF16,
                                   abi.ptr(out), abi.ptr(ws), T, L, I, E, top_k, util.stream_ptr())
    assert st == 0, st
    util.check_status(lx)
    want = O.moe_experts_reference(latent, ids, weights, gu, dn, I)
    return util.host(out), want, (ws, ids, E)


@pytest.mark.parametrize("wtype", [O.W_BF16, O.W_INT8, O.W_FP8, O.W_NVFP4], ids=lambda w: NAMES[w])
@pytest.mark.parametrize("T,L,I,E,top_k", [(5, 256, 256, 8, 2), (1, 512, 128, 16, 4), (32, 512, 256, 64, 8), (40, 256, 96, 6, 3)])
def test_grouped_experts_match_oracle(lx, wtype, T, L, I, E, top_k):
    got, want, _ = experts_case(lx, wtype, T, L, I, E, top_k, seed=T + E)
    # the reference suite's bound is 2e-3 of max|out| under BF16 math; the acceptance bound is rel-L2 1e-3
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()
    util.assert_close(got, want, what=NAMES[wtype])


@pytest.mark.parametrize("wtype", [O.W_BF16, O.W_INT8, O.W_FP8], ids=lambda w: NAMES[w])
def test_grouped_experts_many_tiles_and_chunks(lx, wtype):
    """Shapes that give the tensor-core path several row tiles per expert with a ragged last one (I = 400, L = 1024:
    tiles of fewer than 128 rows), K ending inside a stage (400 = 256 + 144), and an expert with more than 16 rows
    (two chunks)."""
    def crowd(ids):
        ids = ids.copy()
        ids[:20, 0] = 2  # 20 rows for expert 2: two chunks
        return ids

    got, want, _ = experts_case(lx, wtype, 24, 1024, 400, 12, 3, seed=17, ids_override=crowd)
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()
    util.assert_close(got, want, what=NAMES[wtype])


def test_grouping_tables_are_exact(lx):
    T, L, I, E, top_k = 32, 256, 64, 64, 8
    _, _, (ws, ids, E) = experts_case(lx, O.W_FP8, T, L, I, E, top_k, seed=5)
    counts, offsets, pairs = O.moe_group(ids, E)
    raw = util.host(ws)
    got_offsets = raw[: 4 * (E + 1)].view(np.int32)
    at = (4 * (E + 1) + 255) // 256 * 256
    at = at + (4 * E + 255) // 256 * 256
    got_pairs = raw[at : at + 4 * T * top_k].view(np.int32)
    assert np.array_equal(got_offsets, offsets) and np.array_equal(got_pairs, pairs)


def test_skewed_routing_and_an_expert_chosen_twice(lx):
    def skew(ids):
        ids = ids.copy()
        ids[:, 0] = 1          # every token picks expert 1: more rows than one column tile
        ids[3, 1] = 1          # and one token picks it twice
        return ids

    got, want, _ = experts_case(lx, O.W_INT8, 24, 256, 128, 8, 2, seed=9, ids_override=skew)
    util.assert_close(got, want, what="skewed")


def test_per_expert_nvfp4_globals(lx):
    got, want, _ = experts_case(lx, O.W_NVFP4, 6, 256, 256, 4, 2, seed=2, per_expert_global=True)
    util.assert_close(got, want, what="expert_global")


def test_token_bits_do_not_depend_on_batch(lx):
    T, L, I, E, top_k = 8, 512, 256, 16, 4
    gu = O.quantize_weight(util.bf16_normal((E, 2 * I, L), 0.02, 1), O.W_FP8)
    dn = O.quantize_weight(util.bf16_normal((E, L, I), 0.02, 2), O.W_FP8)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    latent = util.bf16_normal((T, L), 1.0, 3)
    ids, weights, _, _ = O.moe_route(util.f32_normal((T, E), 1.0, 4), None, top_k)
    outs = {}
    for t in (1, 3, 8):
        out = torch.full((t, L), float("nan"), device="cuda")
        ws = torch.empty(lx.lx_moe_grouped_workspace_bytes(t, L, I, E, top_k, 0), dtype=torch.uint8, device="cuda")
        latent_d, ids_d, weights_d = util.dev(latent[:t]), util.dev(ids[:t]), util.dev(weights[:t])
        assert lx.lx_moe_experts_grouped(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(), 0,
                                         abi.ptr(out), abi.ptr(ws), t, L, I, E, top_k, util.stream_ptr()) == 0
        util.check_status(lx)
        outs[t] = util.host(out).view(np.uint32).copy()
    assert np.array_equal(outs[1], outs[8][:1]) and np.array_equal(outs[3], outs[8][:3])


def router_case(lx, M, E, K, top_k, with_bias, seed, tie=False):
    rng = np.random.default_rng(seed)
    ld_x = K + 3
    w = (rng.standard_normal((E, K)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(E).astype(np.float32) if with_bias else None
    sel = (rng.standard_normal(E) * 0.3).astype(np.float32) if with_bias else None
    if tie:  # experts 16.. repeat experts 0..15: equal logits and biases tie, the lower index wins; a NaN bias is never picked
        dup = np.arange(16, E) % 16
        w[16:], bias[16:], sel[16:] = w[dup], bias[dup], sel[dup]
        sel[5] = np.nan
    x = rng.standard_normal((M, ld_x)).astype(np.float32)
    x_d, w_d = util.dev(x), util.dev(w)
    bias_d = None if bias is None else util.dev(bias)
    sel_d = None if sel is None else util.dev(sel)
    logits = torch.full((M, E), float("nan"), device="cuda")
    ids = torch.full((M, top_k), -7, dtype=torch.int32, device="cuda")
    weights = torch.full((M, top_k), float("nan"), device="cuda")
    ent = torch.full((M,), float("nan"), device="cuda")
    conf = torch.full((M,), float("nan"), device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):  # twice on the same ticket: the call leaves it at zero
        st = lx.lx_router_route(abi.ptr(x_d), ld_x, abi.ptr(w_d), abi.ptr(bias_d), abi.ptr(logits), abi.ptr(sel_d), abi.ptr(ids),
                                abi.ptr(weights), abi.ptr(ent), abi.ptr(conf), abi.ptr(ticket), M, E, K, top_k, util.stream_ptr())
        assert st == 0, st
        torch.cuda.synchronize()
        assert int(ticket.item()) == 0
    want = x[:, :K].astype(np.float64) @ w.astype(np.float64).T + (0.0 if bias is None else bias.astype(np.float64))
    got = util.host(logits)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    # the logits are lx_spec_gemv_f32's, bit for bit (kernels.h:211-213)
    two = torch.full((M, E), float("nan"), device="cuda")
    assert lx.lx_spec_gemv_f32(abi.ptr(x_d), ld_x, abi.ptr(w_d), abi.ptr(bias_d), abi.ptr(two), E, M, E, K, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.equal(two.view(torch.int32), logits.view(torch.int32))
    # the routing is lx_moe_route on these logits, bit for bit
    ids2 = torch.full((M, top_k), -1, dtype=torch.int32, device="cuda")
    w2, e2, c2 = torch.zeros((M, top_k), device="cuda"), torch.zeros(M, device="cuda"), torch.zeros(M, device="cuda")
    assert lx.lx_moe_route(abi.ptr(logits), abi.ptr(sel_d), abi.ptr(ids2), abi.ptr(w2), abi.ptr(e2), abi.ptr(c2), M, E, top_k,
                           util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.equal(ids, ids2)
    for a, b in ((weights, w2), (ent, e2), (conf, c2)):
        assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    return util.host(ids), got, sel


@pytest.mark.parametrize("E,K,top_k", [(128, 1280, 4), (192, 1280, 4), (128, 1000, 4), (64, 300, 8), (1024, 2048, 32)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_router_in_one_launch(lx, E, K, top_k, with_bias):
    """lx_router_route for every row count of a decode-sized step (mirrors the reference's tests/kernels/test_moe.py:255-284)."""
    for M in range(1, 9):
        ids, logits, sel = router_case(lx, M, E, K, top_k, with_bias, seed=M + E)
        ids_o, _, _, _ = O.moe_route(logits, sel, top_k)
        assert np.array_equal(ids, ids_o)


def test_router_breaks_ties_like_the_route_call(lx):
    for M in (1, 5, 8):
        ids, _, _ = router_case(lx, M, 128, 1280, 4, True, seed=2 + M, tie=True)
        assert not np.any(ids == 5)


@pytest.mark.parametrize("N,K", [(300, 5000), (1000, 4096), (7, 33)])
def test_rows_gemv_f32_rows_do_not_depend_on_batch(lx, N, K):
    """lx_spec_gemv_f32 beyond the router's sizes: close to float64, and a row alone equals the row in a batch of 8."""
    rng = np.random.default_rng(N + K)
    x, w, bias = rng.standard_normal((8, K)).astype(np.float32), (rng.standard_normal((N, K)) * 0.05).astype(np.float32), rng.standard_normal(N).astype(np.float32)
    x_d, w_d, b_d = util.dev(x), util.dev(w), util.dev(bias)
    big = torch.full((8, N + 5), float("nan"), device="cuda")
    assert lx.lx_spec_gemv_f32(abi.ptr(x_d), K, abi.ptr(w_d), abi.ptr(b_d), abi.ptr(big), N + 5, 8, N, K, util.stream_ptr()) == 0
    got = util.host(big)
    want = x.astype(np.float64) @ w.astype(np.float64).T + bias
    assert np.abs(got[:, :N] - want).max() <= 1e-5 * max(1.0, np.abs(want).max()) and np.all(np.isnan(got[:, N:]))
    for m in (0, 3, 7):
        one = torch.full((1, N), float("nan"), device="cuda")
        assert lx.lx_spec_gemv_f32(abi.ptr(x_d[m : m + 1]), K, abi.ptr(w_d), abi.ptr(b_d), abi.ptr(one), N, 1, N, K, util.stream_ptr()) == 0
        assert np.array_equal(util.host(one)[0].view(np.uint32), got[m, :N].view(np.uint32))
    z = torch.zeros(16, device="cuda")
    assert lx.lx_spec_gemv_f32(abi.ptr(z), 4, abi.ptr(z), None, abi.ptr(z), 4, 9, 4, 4, None) == 1   # more than eight rows
    assert lx.lx_spec_gemv_f32(abi.ptr(z), 3, abi.ptr(z), None, abi.ptr(z), 4, 1, 4, 4, None) == 1   # a stride shorter than the row
    assert lx.lx_spec_gemv_f32(abi.ptr(z), 4, abi.ptr(z), None, abi.ptr(z), 4, 0, 4, 4, None) == 0


def test_router_refuses_what_the_reference_refuses(lx):
    z = torch.zeros(16, device="cuda")
    zi = torch.zeros(16, dtype=torch.int32, device="cuda")
    args = lambda M, E, K, k, ld: (abi.ptr(z), ld, abi.ptr(z), None, abi.ptr(z), None, abi.ptr(zi), abi.ptr(z), None, None, abi.ptr(zi), M, E, K, k, None)
    assert lx.lx_router_route(*args(9, 4, 4, 1, 4)) == 1       # more than eight rows
    assert lx.lx_router_route(*args(1, 2000, 4, 1, 4)) == 1    # more experts than the epilogue stages
    assert lx.lx_router_route(*args(1, 4, 4, 1, 3)) == 1       # a row stride shorter than the row
    assert lx.lx_router_route(*args(0, 4, 4, 1, 4)) == 0       # nothing to do
