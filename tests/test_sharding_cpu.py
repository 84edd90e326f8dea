"""The multi-GPU host logic on CPU: row sharding arithmetic, and the expert-parallel dispatch / combine exchanges run as
two `gloo` ranks whose "experts" are computed by the oracle instead of the CUDA library. Checks that the sharded results
equal the unsharded ones."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dromos_b200 import host
from oracle import dromos_oracle as O


def test_shard_rows_cover_everything_once():
    for N in (4096, 14336, 28672, 100, 7):
        for world in (1, 2, 4, 8):
            edges = [host.shard_rows(N, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == N
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
    assert host.shard_rows(28672, 3, 8) == (10752, 14336)
    assert [host.expert_range(64, r, 8) for r in (0, 7)] == [(0, 8), (56, 64)]


def test_remap_for_owner():
    ids = torch.tensor([[0, 5], [9, 6]], dtype=torch.int32)
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5]])
    lid, lw, mine = host.remap_for_owner(ids, w, 4, 8)
    assert lid.tolist() == [[0, 1], [0, 2]] and lw.tolist() == [[0.0, 0.75], [0.0, 0.5]] and mine.tolist() == [[False, True], [False, True]]


class OracleExperts:
    """Stands in for host.Experts on CPU: same call signature, computed by the oracle."""

    def __init__(self, gu, dn, I):
        self.gu, self.dn, self.I = gu, dn, I

    def __call__(self, latent, ids, weights, out):
        lat = latent.view(torch.int16).numpy().view(np.uint16)
        res = O.moe_experts_reference(lat, ids.numpy(), weights.numpy(), self.gu, self.dn, self.I)
        out.copy_(torch.from_numpy(res.astype(np.float32)))
        return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T, L, I, E, k = 8, 64, 32, 8, 2
        rng = np.random.default_rng(0)
        bits = lambda shape, std: O.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32))
        gu_bits, dn_bits = bits((E, 2 * I, L), 0.05), bits((E, L, I), 0.05)
        latent = bits((T, L), 1.0)
        ids, weights, _, _ = O.moe_route(rng.standard_normal((T, E)).astype(np.float32), None, k)
        want = O.moe_experts_reference(latent, ids, weights, O.Weight(O.W_BF16, gu_bits), O.Weight(O.W_BF16, dn_bits), I)
        # this rank's experts and tokens
        e0, e1 = host.expert_range(E, rank, world)
        t0, t1 = T * rank // world, T * (rank + 1) // world
        ep = host.ExpertParallel.__new__(host.ExpertParallel)
        ep.dist, ep.group, ep.world, ep.rank = dist, None, world, rank
        ep.E, ep.L, ep.I, ep.top_k, ep.e0, ep.e1 = E, L, I, k, e0, e1
        ep.local = OracleExperts(O.Weight(O.W_BF16, gu_bits[e0:e1]), O.Weight(O.W_BF16, dn_bits[e0:e1]), I)
        lat_t = torch.from_numpy(latent[t0:t1].view(np.int16)).view(torch.bfloat16)
        got = ep(lat_t, torch.from_numpy(ids[t0:t1]), torch.from_numpy(weights[t0:t1]))
        err = np.abs(got.numpy() - want[t0:t1]).max() / np.abs(want).max()
        # dense: row shards gathered equal the whole product
        N, K = 24, 64
        w = bits((N, K), 0.05)
        x = bits((3, K), 1.0)
        full = O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), O.Weight(O.W_BF16, w))
        n0, n1 = host.shard_rows(N, rank, world)
        mine = torch.from_numpy(O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), O.Weight(O.W_BF16, w[n0:n1])).astype(np.float32))
        gathered = torch.empty((world, 3, n1 - n0))
        dist.all_gather_into_tensor(gathered.view(world * 3, n1 - n0), mine.contiguous())
        dense_err = np.abs(gathered.permute(1, 0, 2).reshape(3, N).numpy() - full).max()
        ret[rank] = (float(err), float(dense_err))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_expert_parallel_and_row_sharding_two_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        err, dense_err = ret[r]
        assert err <= 1e-6, f"rank {r}: expert-parallel output differs from the unsharded one ({err})"
        assert dense_err <= 1e-5
