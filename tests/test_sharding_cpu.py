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


def test_packet_plan_geometry():
    """Which exchanges travel as packets: by what a rank sends, not by the slice alone; odd splits fall back."""
    # C3 on 2 GPUs, f32 y, up to 64 rows, 3 MB limit: M = 1 and 16 as packets, M = 64 (3.7 MB sent) not
    bounds, region, ok = host.packet_plan(28672, 2, 4, 64, 3 << 20)
    assert bounds == [0, 14336, 28672] and ok and region == (3 << 20) // (14336 * 4) * (14336 * 4 // 8)
    assert [host.travels_as_packets(M, bounds, region, ok, 4, 3 << 20) for M in (1, 16, 64)] == [True, True, False]
    # 8 GPUs: a rank sends its slice seven times
    bounds, region, ok = host.packet_plan(28672, 8, 4, 64, 3 << 20)
    assert bounds[1] == 3584 and [host.travels_as_packets(M, bounds, region, ok, 4, 3 << 20) for M in (1, 16, 64)] == [True, True, False]
    # slices that are not whole 8-byte pieces (bf16, a bound at an odd column) never travel as packets
    bounds, region, ok = host.packet_plan(30, 4, 2, 8, 3 << 20)
    assert not ok and not host.travels_as_packets(1, bounds, region, ok, 2, 3 << 20)
    # one rank: nothing to send, packets trivially fit
    bounds, region, ok = host.packet_plan(64, 1, 4, 8, 1 << 20)
    assert bounds == [0, 64] and ok


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
        # experts over ranks with routing and tokens replicated (what host.ReplicatedExpertParallel does on GPUs): every rank
        # computes the weighted rows of the pairs whose expert it owns, the rows meet (here: a sum of zero-filled buffers,
        # exact because the owners are disjoint), and every rank adds a token's rows in k order. Bit for bit the single-rank sum.
        def pair_rows(e_lo, e_hi):
            rows = np.zeros((T * k, L), dtype=np.float32)
            for p in range(T * k):
                e = int(ids.reshape(-1)[p])
                if e_lo <= e < e_hi:
                    one = O.moe_experts_reference(latent[p // k : p // k + 1], np.array([[e]], dtype=np.int32), weights.reshape(-1)[p : p + 1].reshape(1, 1),
                                                  O.Weight(O.W_BF16, gu_bits), O.Weight(O.W_BF16, dn_bits), I)
                    rows[p] = one[0].astype(np.float32)
            return rows

        def k_ordered_sum(rows):
            acc = np.zeros((T, L), dtype=np.float32)
            for j in range(k):
                acc = (acc + rows.reshape(T, k, L)[:, j]).astype(np.float32)
            return acc

        mine_rows = torch.from_numpy(pair_rows(e0, e1))
        dist.all_reduce(mine_rows)
        split = k_ordered_sum(mine_rows.numpy())
        whole = k_ordered_sum(pair_rows(0, E))
        rep_equal = bool(np.array_equal(split.view(np.uint32), whole.view(np.uint32)))
        rep_err = float(np.abs(split - want).max() / np.abs(want).max())
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
        ret[rank] = (float(err), float(dense_err), rep_equal, rep_err)
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
        err, dense_err, rep_equal, rep_err = ret[r]
        assert err <= 1e-6, f"rank {r}: expert-parallel output differs from the unsharded one ({err})"
        assert dense_err <= 1e-5
        assert rep_equal and rep_err <= 1e-6, f"rank {r}: replicated-routing expert split differs from one rank's sum ({rep_err})"
