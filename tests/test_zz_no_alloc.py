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


@pytest.mark.parametrize("wtype", [O.W_FP8, O.W_BF16, O.W_NVFP4])
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


def test_static_scratch_call_allocates_nothing(lx):
    """What the entry point is for: after a first call (which looks the array up), further calls neither take nor give
    back device memory, and they can be captured in a graph (a capture refuses cudaMalloc)."""
    T, L, I, E, top_k = 16, 512, 256, 8, 2
    gu, dn, latent, ids, weights = case(T, L, I, E, top_k, O.W_FP8, 3)
    dgu, ddn = util.DeviceWeight(gu), util.DeviceWeight(dn)
    latent_d, ids_d, weights_d = util.dev(latent), util.dev(ids), util.dev(weights)
    out = torch.full((T, L), float("nan"), device="cuda")

    def call():
        assert lx.lx_b200_moe_experts_grouped_static(abi.ptr(latent_d), abi.ptr(ids_d), abi.ptr(weights_d), dgu.ref(), ddn.ref(),
                                                     abi.MATH_BF16, abi.ptr(out), T, L, I, E, top_k, util.stream_ptr()) == 0

    call()  # the first call on the device: address lookup, function attributes
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
    first = util.host(out).copy()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        out.fill_(float("nan"))
        with torch.cuda.graph(g, stream=side):
            call()
        g.replay()
    torch.cuda.synchronize()
    assert np.array_equal(util.host(out).view(np.uint32), first.view(np.uint32))
    util.check_status(lx)


def test_static_scratch_status_word_is_reported(lx):
    """A bounded wait that gives up inside this entry point leaves its code in the array's first word, not in the
    library's own status word: lx_b200_last_error() must report and clear both. The test plants a code there (nothing
    is made to time out) and reads it back through the public call."""
    import ctypes

    base = lx.lx_b200_moe_static_scratch_ptr()
    assert base, "the array's address could not be looked up"
    assert lx.lx_b200_last_error() == 0
    planted = torch.tensor([5], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    cudart = ctypes.CDLL("libcudart.so.12")  # the runtime the library itself is linked against (already loaded)
    cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    cudart.cudaMemcpy.restype = ctypes.c_int
    assert cudart.cudaMemcpy(base, planted.data_ptr(), 4, 3) == 0  # device to device: 4 bytes into word 0 of the array
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 5, "the static array's status word was not read"
    assert lx.lx_b200_last_error() == 0, "the status word was not cleared"


def test_static_scratch_refuses_what_does_not_fit(lx):
    T, L, I, E, top_k = 512, 4096, 1536, 64, 8
    assert lx.lx_moe_grouped_workspace_bytes(T, L, I, E, top_k, abi.MATH_BF16) > lx.lx_b200_moe_static_scratch_bytes()
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    w = abi.make_weight(abi.W_BF16, dummy)
    import ctypes
    st = lx.lx_b200_moe_experts_grouped_static(abi.ptr(dummy), abi.ptr(dummy), abi.ptr(dummy), ctypes.byref(w), ctypes.byref(w),
                                               abi.MATH_BF16, abi.ptr(dummy), T, L, I, E, top_k, util.stream_ptr())
    assert st == abi.ERR_SCRATCH
