"""Child of tests/test_multi_gpu.py: one process per GPU (launched by torch.distributed.run). Checks on real peers what
the single-GPU suite cannot: the one-kernel exchange of output slices against the unsharded product, bit for bit, and a
peer that never arrives (the wait gives up, reports, and the next round works). Nothing here faults or hangs a GPU: the
rank that "never arrives" simply skips one call and stays alive; NVLS / multicast are off."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

from dromos_b200 import abi, host  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    lib = abi.Library()
    failures = []
    N, K = 2 * 8192 + 72, 2048  # every shard wide enough that shard and whole weight pick the same kernel
    gen = torch.Generator(device=dev).manual_seed(5)  # the same on every rank
    w = (torch.randn((N, K), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    n0, n1 = host.shard_rows(N, rank, world)
    for wtype in (abi.W_BF16, abi.W_INT8, abi.W_FP8, abi.W_NVFP4, abi.W_BF16X):
        buffers = host.PeerBuffers(N, 64, dev)
        whole = host.Linear(lib, host.store_weight(lib, w, wtype), N, K)
        if wtype == abi.W_NVFP4:  # a shard of an NVFP4 checkpoint keeps the whole matrix's global scale: slice the stored rows
            s = whole.weight
            shard = host.StoredWeight(wtype, s.data.view(N, K // 2)[n0:n1].contiguous(), s.scale.view(N, K // 16)[n0:n1].contiguous(), s.glob,
                                      rows=n1 - n0, cols=K)
        else:
            shard = host.store_weight(lib, w[n0:n1].contiguous(), wtype)
        layer = host.PeerShardedLinear(lib, shard, N, K, buffers)
        for rnd, M in enumerate((1, 8, 3, 16, 64, 5, 2, 33)):
            x = torch.randn((M, K), generator=gen, device=dev).to(torch.bfloat16)
            layer.packets = [None, True, False][rnd % 3]  # the default choice, packets forced, the semaphore exchange forced
            if layer.packets and M * ((n1 - n0) * 4 // 8) > buffers.region:
                layer.packets = None
            got = layer(x).clone()
            want = whole(x)
            torch.cuda.synchronize()
            ok = torch.equal(got.view(torch.int32), want.view(torch.int32))
            if not ok:
                failures.append(f"rank {rank} wtype {wtype} round {rnd} M={M}: exchanged y differs from the unsharded product "
                                f"(max abs {float((got - want).abs().max()):.3e})")
        if lib.lx_b200_last_error() != 0:
            failures.append(f"rank {rank} wtype {wtype}: a bounded wait ran out")
        dist.barrier()

    # ---- a peer that never arrives ----
    os.environ["LX_B200_WAIT_MS"] = "50"
    buffers = host.PeerBuffers(N, 8, dev)
    layer = host.PeerShardedLinear(lib, host.store_weight(lib, w[n0:n1].contiguous(), abi.W_FP8), N, K, buffers)
    x = torch.randn((2, K), generator=gen, device=dev).to(torch.bfloat16)
    want = host.Linear(lib, host.store_weight(lib, w, abi.W_FP8), N, K)(x)
    for packets, code_wanted in ((False, 6), (True, 7)):
        layer.packets = packets
        layer(x)
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            layer(x)  # the others skip this round: rank 0 waits 50 ms, gives up and says so
            torch.cuda.synchronize()
            code = lib.lx_b200_last_error()
            if code != code_wanted:
                failures.append(f"rank 0: expected status {code_wanted} after a round nobody joined, got {code}")
        else:
            buffers.next_half()  # keep the buffer halves in step with rank 0
        dist.barrier()
        if packets:
            # the sequence numbers live on each rank: the ranks that skipped the call put theirs forward by hand, which a
            # caller that abandons a round has to do (here: both buffers' words from rank 0, whose count is right)
            seq = buffers.seq.clone()
            dist.broadcast(seq, src=0)
            buffers.seq[0:1].copy_(seq[0:1])
        else:
            # rank 0's lone arrival is still in everyone's semaphore: drain it, then a normal round works again
            buffers.counter.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        got = layer(x).clone()
        torch.cuda.synchronize()
        if not torch.equal(got.view(torch.int32), want.view(torch.int32)) or lib.lx_b200_last_error() != 0:
            failures.append(f"rank {rank}: the round after the abandoned one is wrong (packets={packets})")
    # ---- experts split over the ranks: replicated routing and tokens, rows exchanged as packets ----
    os.environ["LX_B200_WAIT_MS"] = "1000"
    E, top_k, L, I = 16, 4, 512, 384
    gu_bf = (torch.randn((E, 2 * I, L), generator=gen, device=dev) * 0.03).to(torch.bfloat16)
    dn_bf = (torch.randn((E, L, I), generator=gen, device=dev) * 0.03).to(torch.bfloat16)
    e0, e1 = host.expert_range(E, rank, world)
    for wtype in (abi.W_BF16, abi.W_FP8, abi.W_INT8):
        plain = host.Experts(lib, host.store_weight(lib, gu_bf, wtype), host.store_weight(lib, dn_bf, wtype), E, L, I, top_k)
        split = host.ReplicatedExpertParallel(lib, host.store_weight(lib, gu_bf[e0:e1].contiguous(), wtype), host.store_weight(lib, dn_bf[e0:e1].contiguous(), wtype),
                                              E, L, I, top_k, 40, dev)
        for T in (1, 32, 5, 40, 8, 8):
            latent = torch.randn((T, L), generator=gen, device=dev).to(torch.bfloat16)
            ids, weights = plain.route(torch.randn((T, E), generator=gen, device=dev))
            want = plain(latent, ids, weights)
            got = split(latent, ids, weights)
            torch.cuda.synchronize()
            if not torch.equal(got.view(torch.int32), want.view(torch.int32)):
                failures.append(f"rank {rank} experts wtype {wtype} T={T}: split experts differ from one GPU's (max abs {float((got - want).abs().max()):.3e})")
        if lib.lx_b200_last_error() != 0:
            failures.append(f"rank {rank} experts wtype {wtype}: a bounded wait ran out")
        dist.barrier()
    # a round only rank 0 joins: its polls give up (status 8); the others put their sequence word forward; the next round is right
    os.environ["LX_B200_WAIT_MS"] = "50"
    if rank == 0:
        split(latent, ids, weights)
        torch.cuda.synchronize()
        code = lib.lx_b200_last_error()
        if code != 8:
            failures.append(f"rank 0: expected status 8 after a row exchange nobody joined, got {code}")
    dist.barrier()
    seq = split.seq.clone()
    dist.broadcast(seq, src=0)
    split.seq[0:1].copy_(seq[0:1])
    torch.cuda.synchronize()
    dist.barrier()
    got = split(latent, ids, weights)
    torch.cuda.synchronize()
    if not torch.equal(got.view(torch.int32), want.view(torch.int32)) or lib.lx_b200_last_error() != 0:
        failures.append(f"rank {rank}: the row exchange after the abandoned one is wrong")
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    for f in failures:
        print("FAIL", f, flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("MGPU_OK" if int(flag.item()) == 0 else "MGPU_FAILED", flush=True)
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
