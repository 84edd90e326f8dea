"""The routed-experts entry point for callers that must not allocate (lx_b200_moe_experts_grouped_static).

Such callers have given all free device memory to their own arena, or may not enter the driver's allocator from their
decode loop, so the library keeps this call's scratch in a fixed array of its own image. The test calls it through the
C ABI twice in a row (the array is shared and keeps the previous call's contents) and checks every bit of the output
against lx_moe_experts_grouped, which runs the same kernels on a caller workspace; it also checks that a problem too
large for the array is refused. This file sorts last so that a run that stops at the first failure has already run
every other test; it passes alone in a fresh process as well as after the others.
"""

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def case(T, L, I, E, top_k, wtype, seed):
    gu = O.quantize_weight(util.bf16_normal((E, 2 * I, L), 0.02, seed), wtype)
    dn = O.quantize_weight(util.bf16_normal((E, L, I), 0.02, seed + 1), wtype)
    latent = util.bf16_normal((T, L), 1.0, seed + 2)
    ids, weights, _, _ = O.moe_route(util.f32_normal((T, E), 1.0, seed + 3), None, top_k)
    return gu, dn, latent, ids, weights


@pytest.mark.parametrize("wtype", [O.W_FP8, O.W_BF16])
def test_static_scratch_matches_workspace_entry_point_twice(lx, wtype):
    T, L, I, E, top_k = 32, 512, 256, 16, 4
    results = []
    for call in range(2):  # two calls in a row: the second finds the first one's leftovers in the array
        gu, dn, latent, ids, weights = case(T, L, I, E, top_k, wtype, 10 * call)
        dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
        latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)
        want = torch.full((T, L), float("nan"), device="cuda")
        ws = torch.empty(lx.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, abi.MATH_BF16), dtype=torch.uint8, device="cuda")
        assert lx.lx_moe_experts_grouped(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(), abi.MATH_BF16,
                                         abi.ptr(want), abi.ptr(ws), T, L, I, E, top_k, util.stream_ptr()) == 0
        got = torch.full((T, L), float("nan"), device="cuda")
        assert lx.lx_b200_moe_experts_grouped_static(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(),
                                                     abi.MATH_BF16, abi.ptr(got), T, L, I, E, top_k, util.stream_ptr()) == 0
        util.check_status(lx)
        g, w = util.host(got), util.host(want)
        assert np.all(np.isfinite(g))
        assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), f"call {call}: outputs differ"
        util.assert_close(g, O.moe_experts_reference(latent, ids, weights, gu, dn, I), what=f"call {call}")
        results.append(g)
    assert not np.array_equal(results[0], results[1])  # the two calls really were different problems


def test_static_scratch_refuses_what_does_not_fit(lx):
    T, L, I, E, top_k = 512, 4096, 1536, 64, 8
    assert lx.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, abi.MATH_BF16) > lx.lx_b200_moe_static_scratch_bytes()
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    w = abi.make_weight(abi.W_BF16, dummy)
    import ctypes
    st = lx.lx_b200_moe_experts_grouped_static(abi.ptr(dummy), abi.ptr(dummy), abi.ptr(dummy), ctypes.byref(w), ctypes.byref(w),
                                               abi.MATH_BF16, abi.ptr(dummy), T, L, I, E, top_k, util.stream_ptr())
    assert st == abi.ERR_SCRATCH
