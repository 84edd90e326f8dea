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
