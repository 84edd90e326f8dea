"""The exchange kernels of the multi-GPU paths, on ONE GPU: two "ranks" whose buffers all live on this GPU (a peer-mapped
pointer is just a pointer) call in turn. Kernels of one GPU must not wait for each other, so the rank that calls first
finds nobody there: its bounded wait gives up after a few milliseconds and says so (that is the first thing checked); the
rank that calls second finds the first one's data already delivered and completes (the second thing). Both directions are
played, which covers send, poll, unpack, the sequence numbers and the alternating halves of the receive buffers.
Nothing here faults or hangs the GPU."""

import ctypes

import numpy as np
import pytest
import torch

from dromos_b200 import abi, host
from tests import util

pytestmark = pytest.mark.gpu


def ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("dtype,M,N", [(torch.float32, 3, 520), (torch.bfloat16, 5, 1024), (torch.float32, 1, 64)], ids=["f32", "bf16", "tiny"])
def test_packet_exchange_between_two_ranks_in_turn(lx, monkeypatch, dtype, M, N):
    monkeypatch.setenv("LX_B200_WAIT_MS", "20")
    assert lx.lx_b200_last_error() == 0
    esz = 2 if dtype == torch.bfloat16 else 4
    y_dt = abi.BF16 if dtype == torch.bfloat16 else abi.F32
    bounds, region, ok = host.packet_plan(N, 2, esz, M, 1 << 20)
    assert ok
    b_arr = (ctypes.c_int64 * 3)(*bounds)
    whole = torch.randn((M, N), device="cuda").to(dtype)
    boxes = [torch.zeros((2, 2, region, 4), dtype=torch.int32, device="cuda") for _ in range(2)]
    words = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    y = [torch.zeros((M, N), dtype=dtype, device="cuda") for _ in range(2)]

    def call(rank):
        return lx.lx_b200_exchange_packets(abi.ptr(y[rank]), ptrs(boxes), region, abi.ptr(words[rank]), abi.ptr(words[rank][32:]), 2, rank, b_arr,
                                           y_dt, N, M, util.stream_ptr())

    for first in (1, 0, 1):  # three rounds: the halves of the receive buffers alternate with the sequence number
        second = 1 - first
        for r in range(2):  # every rank has its own columns of a fresh whole y, the rest zero
            y[r].zero_()
            y[r][:, bounds[r] : bounds[r + 1]] = whole[:, bounds[r] : bounds[r + 1]]
        assert call(first) == 0
        torch.cuda.synchronize()
        assert lx.lx_b200_last_error() == 7, "the rank that called first should have given up on its peer"
        assert call(second) == 0
        torch.cuda.synchronize()
        assert lx.lx_b200_last_error() == 0
        assert torch.equal(y[second].view(torch.uint8), whole.view(torch.uint8)), "the second caller's y is not whole"
        assert torch.equal(y[first][:, bounds[second] : bounds[second + 1]], torch.zeros_like(y[first][:, bounds[second] : bounds[second + 1]]))
        assert int(words[0][0].item()) == int(words[1][0].item()) and int(words[0][32].item()) == 0 and int(words[1][32].item()) == 0
        whole = torch.randn((M, N), device="cuda").to(dtype)
    assert int(words[0][0].item()) == 3


def test_packet_exchange_refuses_what_it_cannot_send(lx):
    z = torch.zeros(4096, dtype=torch.int32, device="cuda")
    boxes = ptrs([z, z])
    ok_bounds = (ctypes.c_int64 * 3)(0, 8, 16)
    odd_bounds = (ctypes.c_int64 * 3)(0, 7, 16)
    args = lambda bounds, region, ranks, rank: (abi.ptr(z), boxes, region, abi.ptr(z), abi.ptr(z[32:]), ranks, rank, bounds, abi.F32, 16, 2, None)
    assert lx.lx_b200_exchange_packets(*args(odd_bounds, 64, 2, 0)) == 801   # a slice that is not whole 8-byte pieces
    assert lx.lx_b200_exchange_packets(*args(ok_bounds, 4, 2, 0)) == 1       # regions too small for the slices
    assert lx.lx_b200_exchange_packets(*args(ok_bounds, 64, 2, 2)) == 1      # a rank outside the ranks
    assert lx.lx_b200_exchange_packets(*args(ok_bounds, 64, 9, 0)) == 1      # more ranks than the kernel addresses
    one = (ctypes.c_int64 * 2)(0, 16)
    assert lx.lx_b200_exchange_packets(abi.ptr(z), ptrs([z]), 64, abi.ptr(z), abi.ptr(z[32:]), 1, 0, one, abi.F32, 16, 2, None) == 0  # alone: nothing to exchange
    torch.cuda.synchronize()
    assert int(z[0].item()) == 1 and lx.lx_b200_last_error() == 0  # the sequence number still advances


def test_semaphore_exchange_between_two_ranks_in_turn(lx, monkeypatch):
    monkeypatch.setenv("LX_B200_WAIT_MS", "20")
    M, N = 4, 776
    bounds = [0, 388, 776]
    whole = torch.randn((M, N), device="cuda")
    y = [torch.zeros((M, N), device="cuda") for _ in range(2)]
    counters = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(2)]
    for r in range(2):
        y[r][:, bounds[r] : bounds[r + 1]] = whole[:, bounds[r] : bounds[r + 1]]

    def call(rank):
        return lx.lx_b200_exchange_slices(ptrs(y), ptrs(counters), 2, rank, bounds[rank], bounds[rank + 1] - bounds[rank], abi.F32, N, M, util.stream_ptr())

    assert call(1) == 0
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 6  # nobody else has arrived: rank 1 gives up and takes nothing
    assert [int(c[0].item()) for c in counters] == [1, 1]
    assert torch.equal(y[0], whole), "rank 1's stores did not make rank 0's y whole"
    assert call(0) == 0
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 0
    assert torch.equal(y[1], whole)
    assert [int(c[0].item()) for c in counters] == [0, 2]  # rank 0 took its two arrivals; rank 1's are what it left behind


def test_row_exchange_of_split_experts_in_turn(lx, monkeypatch):
    """Experts split over two "ranks" of one GPU: each computes its own experts' rows, the rank that exchanges second gets the
    first one's rows as packets and its ordered sum equals lx_moe_experts_grouped on all experts, bit for bit."""
    monkeypatch.setenv("LX_B200_WAIT_MS", "20")
    T, L, I, E, top_k = 11, 256, 128, 8, 3
    gu_bf = (torch.randn((E, 2 * I, L), device="cuda") * 0.03).to(torch.bfloat16)
    dn_bf = (torch.randn((E, L, I), device="cuda") * 0.03).to(torch.bfloat16)
    latent = torch.randn((T, L), device="cuda").to(torch.bfloat16)
    plain = host.Experts(lx, host.store_weight(lx, gu_bf, abi.W_FP8), host.store_weight(lx, dn_bf, abi.W_FP8), E, L, I, top_k)
    ids, weights = plain.route(torch.randn((T, E), device="cuda"))
    want = plain(latent, ids, weights)
    cut = 5
    eng = [host.ReplicatedExpertParallel(lx, host.store_weight(lx, gu_bf[a:b].contiguous(), abi.W_FP8), host.store_weight(lx, dn_bf[a:b].contiguous(), abi.W_FP8),
                                         E, L, I, top_k, T, latent.device) for a, b in ((0, cut), (cut, E))]
    half_packets = T * top_k * (L // 2)
    boxes = [torch.zeros((2, half_packets, 4), dtype=torch.int32, device="cuda") for _ in range(2)]
    bounds = (ctypes.c_int * 3)(0, cut, E)
    eng[0].owned(latent, ids, weights, 0, cut)
    eng[1].owned(latent, ids, weights, cut, E)

    def exchange(rank):
        e = eng[rank]
        return lx.lx_b200_moe_exchange_rows(abi.ptr(e.rows), abi.ptr(e.ws), ptrs(boxes), half_packets, abi.ptr(e.seq), abi.ptr(e.seq[32:]), 2, rank, bounds,
                                            T, L, I, E, top_k, util.stream_ptr())

    assert exchange(1) == 0
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 8  # rank 0 has not sent yet
    assert exchange(0) == 0
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 0
    got = eng[0].sum(T, torch.empty_like(want))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # bad arguments
    assert lx.lx_b200_moe_exchange_rows(abi.ptr(eng[0].rows), abi.ptr(eng[0].ws), ptrs(boxes), half_packets - 1, abi.ptr(eng[0].seq), abi.ptr(eng[0].seq[32:]),
                                        2, 0, bounds, T, L, I, E, top_k, None) == 1
    bad = (ctypes.c_int * 3)(0, cut, E - 1)
    assert lx.lx_b200_moe_exchange_rows(abi.ptr(eng[0].rows), abi.ptr(eng[0].ws), ptrs(boxes), half_packets, abi.ptr(eng[0].seq), abi.ptr(eng[0].seq[32:]),
                                        2, 0, bad, T, L, I, E, top_k, None) == 1
