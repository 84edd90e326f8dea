"""The host-side mirror on one GPU: Linear picks the entry point by row count, ShardedLinear and ExpertParallel with a
world of one reduce to the plain layers (their exchanges are covered by the two-rank gloo tests on CPU)."""

import numpy as np
import pytest
import torch

from dromos_b200 import abi, host
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("wtype", [abi.W_BF16, abi.W_INT8, abi.W_FP8, abi.W_NVFP4, abi.W_BF16X])
def test_linear_matches_oracle_at_every_row_count(lx, wtype):
    N, K = 320, 1024
    w_bits = util.bf16_normal((N, K), 0.02, 1)
    w = torch.from_numpy(w_bits.view(np.int16)).cuda().view(torch.bfloat16)
    layer = host.Linear(lx, host.store_weight(lx, w, wtype), N, K)
    wt = util.make_weight(w_bits, wtype)
    for M in (1, 8, 9, 40):
        x_bits = util.bf16_normal((M, K), 1.0, 2 + M)
        x = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
        y = layer(x)
        torch.cuda.synchronize()
        want = O.gemv_reference(O.bf16_bits_to_f32(x_bits).astype(np.float64), util.reference_weight(w_bits, wt))
        util.assert_close(y.cpu().numpy(), want, what=f"wtype {wtype} M={M}")
    util.check_status(lx)


def test_sharded_linear_with_one_rank_is_the_plain_layer(lx):
    N, K, M = 512, 512, 4
    w = (torch.randn((N, K), device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    plain = host.Linear(lx, host.store_weight(lx, w, abi.W_FP8), N, K)(x)
    sharded = host.ShardedLinear(lx, w, abi.W_FP8, N, K)(x)
    torch.cuda.synchronize()
    assert torch.equal(plain, sharded)


def test_expert_parallel_with_one_rank_matches_the_grouped_experts(lx):
    T, L, I, E, top_k = 16, 512, 256, 8, 2
    gu = host.store_weight(lx, (torch.randn((E, 2 * I, L), device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    dn = host.store_weight(lx, (torch.randn((E, L, I), device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    latent = torch.randn((T, L), device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), device="cuda")
    plain = host.Experts(lx, gu, dn, E, L, I, top_k)
    ids, weights = plain.route(logits)
    want = plain(latent, ids, weights)
    got = host.ExpertParallel(lx, gu, dn, E, L, I, top_k)(latent, ids, weights)
    torch.cuda.synchronize()
    # the owner runs one pair per row (top_k = 1) and the home rank adds the k rows: same products, same order of the sum
    assert torch.allclose(got, want, rtol=0, atol=2e-3 * float(want.abs().max()))
    util.check_status(lx)


@pytest.mark.parametrize("wtype", [abi.W_BF16, abi.W_INT8, abi.W_FP8], ids=["bf16", "int8", "fp8"])
@pytest.mark.parametrize("cuts", [(0, 8), (0, 3, 8), (0, 2, 2, 5, 8)], ids=["whole", "two", "four-one-empty"])
def test_owned_experts_of_every_split_add_up_to_the_grouped_experts(lx, wtype, cuts):
    """The expert-parallel path without its exchange, on one GPU: each "rank" computes the rows of its own experts from
    its own slice of the stacks into one shared rows buffer, then the ordered sum: bit for bit lx_moe_experts_grouped,
    however the experts are cut (an empty range and a range whose experts nobody chose included)."""
    T, L, I, E, top_k = 19, 512, 256, 8, 3
    gu_bf = (torch.randn((E, 2 * I, L), device="cuda") * 0.02).to(torch.bfloat16)
    dn_bf = (torch.randn((E, L, I), device="cuda") * 0.02).to(torch.bfloat16)
    latent = torch.randn((T, L), device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), device="cuda")
    logits[:, 6] = -50.0  # nobody chooses expert 6
    plain = host.Experts(lx, host.store_weight(lx, gu_bf, wtype), host.store_weight(lx, dn_bf, wtype), E, L, I, top_k)
    ids, weights = plain.route(logits)
    want = plain(latent, ids, weights)
    shared = None
    for e0, e1 in zip(cuts[:-1], cuts[1:]):
        if e1 == e0:
            continue
        eng = host.ReplicatedExpertParallel(lx, host.store_weight(lx, gu_bf[e0:e1].contiguous(), wtype), host.store_weight(lx, dn_bf[e0:e1].contiguous(), wtype),
                                            E, L, I, top_k, T, latent.device)
        if shared is None:
            shared = eng
            shared.rows.fill_(float("nan"))
        else:
            eng.rows = shared.rows
        eng.owned(latent, ids, weights, e0, e1)
    got = shared.sum(T, torch.empty_like(want))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    util.check_status(lx)


def test_a_rank_without_experts_still_writes_the_grouping_tables(lx):
    """More ranks than experts: the rank's owned range is empty and it holds no stacks; the call groups (the row exchange reads
    the tables on every rank) and multiplies nothing."""
    T, L, I, E, top_k = 6, 256, 128, 4, 2
    eng = host.ReplicatedExpertParallel(lx, None, None, E, L, I, top_k, T, torch.device("cuda"))
    eng.ws.fill_(0xFF)
    latent = torch.randn((T, L), device="cuda").to(torch.bfloat16)
    ids = torch.tensor([[0, 1], [2, 3], [1, 0], [3, 3], [2, 0], [1, 2]], dtype=torch.int32, device="cuda")
    w = torch.ones((T, top_k), device="cuda")
    eng.owned(latent, ids, w, 2, 2)
    torch.cuda.synchronize()
    offsets = eng.ws[: 4 * (E + 1)].view(torch.int32).tolist()
    assert offsets == [0, 3, 6, 9, 12]  # pairs per expert: 3, 3, 3, 3
    util.check_status(lx)


def test_owned_experts_refuse_what_they_cannot_take(lx):
    T, L, I, E, top_k = 4, 256, 128, 8, 2
    gu = host.store_weight(lx, (torch.randn((E, 2 * I, L), device="cuda") * 0.02).to(torch.bfloat16), abi.W_NVFP4)
    dn = host.store_weight(lx, (torch.randn((E, L, I), device="cuda") * 0.02).to(torch.bfloat16), abi.W_NVFP4)
    eng = host.ReplicatedExpertParallel(lx, gu, dn, E, L, I, top_k, T, torch.device("cuda"))
    latent = torch.randn((T, L), device="cuda").to(torch.bfloat16)
    ids = torch.zeros((T, top_k), dtype=torch.int32, device="cuda")
    w = torch.ones((T, top_k), device="cuda")
    args = lambda own0, own1: (abi.ptr(latent), abi.ptr(ids), abi.ptr(w), gu.ref(), dn.ref(), abi.MATH_BF16, abi.ptr(eng.rows), abi.ptr(eng.ws), T, L, I,
                               E, own0, own1, top_k, None)
    assert lx.lx_b200_moe_experts_owned(*args(0, 8)) == 801   # NVFP4 stacks: not a format the expert tensor-core kernels read as stored
    assert lx.lx_b200_moe_experts_owned(*args(5, 3)) == 1     # an empty-negative range
    assert lx.lx_b200_moe_experts_owned(*args(0, 9)) == 1     # beyond the experts
    assert lx.lx_b200_moe_sum_rows(abi.ptr(eng.rows), None, T, L, top_k, None) == 1
