"""Host-side mirror of the reference's operator interface for the decode weight-streaming path.

The reference engine reaches the path through three calls of its backend ABI (lernex/dromos
engine/model/metis.cpp:1232-1310): `linear()` picks lx_gemv_w for M <= 8 rows (in chunks of 8) and lx_gemm_w above,
and `routed_experts()` picks lx_moe_experts_grouped for more than 8 tokens. The classes here make the same choices
on top of the C ABI of this package's library, own the device buffers a caller of the engine would own (weights,
workspaces), and add what the reference does not have: weights sharded by output rows over the ranks of a
torch.distributed group (each rank streams N / G rows, the slices meet in an all-gather) and experts sharded over
ranks (each rank runs the experts it owns on the tokens routed to them; per-pair rows return to every rank and are
summed in k order).

torch is used for device memory, streams and the process group only. Nothing here computes a product on the host.
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import abi

GEMV_MAX_ROWS = 8  # lx_gemv_w takes at most 8 activation rows (engine/cuda/gemv.cu:59)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class StoredWeight:
    """A weight in one stored format on the device: the buffers and the lx_weight that points at them."""

    def __init__(self, wtype: int, data: torch.Tensor, scale: torch.Tensor | None = None, glob: float = 1.0,
                 expert_global: torch.Tensor | None = None, rows: int = 0, cols: int = 0):
        self.wtype, self.data, self.scale, self.glob, self.expert_global = wtype, data, scale, float(glob), expert_global
        self.rows, self.cols = rows, cols
        self.struct = abi.make_weight(wtype, data, scale, glob, expert_global)

    def ref(self):
        return ctypes.byref(self.struct)

    def nbytes(self) -> int:
        """Bytes a product streams from this weight: values and their scales (the reference's accounting,
        bench/bench_gemv.py:51-56)."""
        n = self.data.numel() * self.data.element_size()
        if self.scale is not None:
            n += self.scale.numel() * self.scale.element_size()
        return n + (4 if self.wtype == abi.W_NVFP4 else 0)


def store_weight(lib: abi.Library, w_bf16: torch.Tensor, wtype: int) -> StoredWeight:
    """Converts a bf16 [rows, cols] (or stacked [E, rows, cols]) device tensor into a stored format with the library's
    own load-time entry points (lx_quantize_weight / lx_bf16x_encode)."""
    assert w_bf16.is_cuda and w_bf16.dtype == torch.bfloat16 and w_bf16.is_contiguous()
    cols = w_bf16.shape[-1]
    rows = w_bf16.numel() // cols
    if wtype == abi.W_BF16:
        return StoredWeight(wtype, w_bf16, rows=rows, cols=cols)
    if wtype == abi.W_BF16X:
        n = lib.lx_bf16x_bytes(abi.ptr(w_bf16), rows, cols, _stream())
        if n <= 0:
            raise RuntimeError(f"lx_bf16x_bytes failed: {n}")
        data = torch.empty(n, dtype=torch.uint8, device=w_bf16.device)
        st = lib.lx_bf16x_encode(abi.ptr(w_bf16), rows, cols, abi.ptr(data), n, _stream())
        if st:
            raise RuntimeError(f"lx_bf16x_encode failed: {st}")
        return StoredWeight(wtype, data, rows=rows, cols=cols)
    if wtype == abi.W_NVFP4:
        data = torch.empty(rows * cols // 2, dtype=torch.uint8, device=w_bf16.device)
        scale = torch.empty(rows * cols // 16, dtype=torch.uint8, device=w_bf16.device)
    else:
        data = torch.empty(rows * cols, dtype=torch.uint8, device=w_bf16.device)
        scale = torch.empty(rows, dtype=torch.float32, device=w_bf16.device)
    lw = abi.make_weight(wtype, data, scale)
    st = lib.lx_quantize_weight(abi.ptr(w_bf16), ctypes.byref(lw), rows, cols, _stream())
    if st:
        raise RuntimeError(f"lx_quantize_weight failed: {st}")
    return StoredWeight(wtype, data, scale, lw.glob, rows=rows, cols=cols)


class Linear:
    """y = x @ W^T for one stored weight [N, K], choosing the entry point as the engine's linear() does."""

    def __init__(self, lib: abi.Library, weight: StoredWeight, N: int, K: int):
        self.lib, self.weight, self.N, self.K = lib, weight, N, K
        self._ws = None

    def __call__(self, x: torch.Tensor, y: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 or f32 [M, K] on the device; y: f32 [M, N] (allocated when absent)."""
        M = x.shape[0]
        if y is None:
            y = torch.empty((M, self.N), dtype=torch.float32, device=x.device)
        x_dt = abi.BF16 if x.dtype == torch.bfloat16 else abi.F32
        y_dt = abi.BF16 if y.dtype == torch.bfloat16 else abi.F32
        ld_x, ld_y = x.stride(0), y.stride(0)
        if M <= GEMV_MAX_ROWS or self.weight.wtype == abi.W_BF16X:
            for m0 in range(0, M, GEMV_MAX_ROWS):  # chunks of 8 rows (metis.cpp:1234-1253)
                mc = min(GEMV_MAX_ROWS, M - m0)
                st = self.lib.lx_gemv_w(abi.ptr(x[m0:]), x_dt, ld_x, self.weight.ref(), None, abi.BF16, abi.ptr(y[m0:]), y_dt,
                                        ld_y, mc, self.N, self.K, 1.0, 0.0, _stream())
                if st:
                    raise RuntimeError(f"lx_gemv_w failed: {st}")
            return y
        need = self.lib.lx_gemm_workspace_bytes(M, self.K, abi.MATH_BF16)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
        st = self.lib.lx_gemm_w(abi.ptr(x), x_dt, ld_x, self.weight.ref(), abi.MATH_BF16, None, abi.BF16, abi.ptr(y), y_dt, ld_y,
                                M, self.N, self.K, 1.0, 0.0, abi.ptr(self._ws), _stream())
        if st:
            raise RuntimeError(f"lx_gemm_w failed: {st}")
        return y


def shard_rows(N: int, rank: int, world: int) -> tuple[int, int]:
    """The contiguous range of output rows rank `rank` of `world` owns: [n0, n1)."""
    return N * rank // world, N * (rank + 1) // world


class ShardedLinear:
    """A Linear whose rows are split over the ranks of a process group. Each rank holds rows [n0, n1) of the weight (with
    their scales; a BF16X shard is encoded on its own), multiplies the replicated activations by them and the slices
    meet in an all-gather: no collective touches the weight stream."""

    def __init__(self, lib, w_bf16_shard: torch.Tensor, wtype: int, N: int, K: int, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N, self.K = N, K
        self.n0, self.n1 = shard_rows(N, self.rank, self.world)
        assert w_bf16_shard.shape == (self.n1 - self.n0, K)
        self.local = Linear(lib, store_weight(lib, w_bf16_shard, wtype), self.n1 - self.n0, K)
        self.uniform = N % self.world == 0

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        M = x.shape[0]
        y_local = self.local(x)  # [M, N / G]
        if self.world == 1:
            return y_local
        if self.uniform:
            gathered = torch.empty((self.world, M, self.n1 - self.n0), dtype=y_local.dtype, device=y_local.device)
            self.dist.all_gather_into_tensor(gathered.view(self.world * M, self.n1 - self.n0), y_local, group=self.group)
            return gathered.permute(1, 0, 2).reshape(M, self.N)
        parts = [torch.empty((M, shard_rows(self.N, r, self.world)[1] - shard_rows(self.N, r, self.world)[0]),
                             dtype=y_local.dtype, device=y_local.device) for r in range(self.world)]
        self.dist.all_gather(parts, y_local, group=self.group)
        return torch.cat(parts, dim=1)


class Experts:
    """Routed experts on stored stacks gate_up [E, 2I, L] and down [E, L, I] (lx_moe_route + lx_moe_experts_grouped)."""

    def __init__(self, lib, gate_up: StoredWeight, down: StoredWeight, E: int, L: int, I: int, top_k: int):
        self.lib, self.gate_up, self.down, self.E, self.L, self.I, self.top_k = lib, gate_up, down, E, L, I, top_k
        self._ws = None

    def route(self, logits: torch.Tensor, bias: torch.Tensor | None = None):
        T = logits.shape[0]
        ids = torch.empty((T, self.top_k), dtype=torch.int32, device=logits.device)
        weights = torch.empty((T, self.top_k), dtype=torch.float32, device=logits.device)
        # entropy and confidence are required outputs of the reference's entry point (its kernel writes them without a null
        # check, engine/cuda/moe.cu:67), so they are always passed; the last call's values stay readable as self.stats
        self.stats = torch.empty((2, T), dtype=torch.float32, device=logits.device)
        st = self.lib.lx_moe_route(abi.ptr(logits), abi.ptr(bias), abi.ptr(ids), abi.ptr(weights), abi.ptr(self.stats[0]), abi.ptr(self.stats[1]), T,
                                   logits.shape[1], self.top_k, _stream())
        if st:
            raise RuntimeError(f"lx_moe_route failed: {st}")
        return ids, weights

    def __call__(self, latent: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, out: torch.Tensor | None = None):
        T = latent.shape[0]
        if out is None:
            out = torch.empty((T, self.L), dtype=torch.float32, device=latent.device)
        need = self.lib.lx_moe_grouped_workspace_bytes(T, self.L, self.I, self.E, self.top_k, abi.MATH_BF16)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=latent.device)
        st = self.lib.lx_moe_experts_grouped(abi.ptr(latent), abi.ptr(ids), abi.ptr(weights), self.gate_up.ref(), self.down.ref(),
                                             abi.MATH_BF16, abi.ptr(out), abi.ptr(self._ws), T, self.L, self.I, self.E,
                                             self.top_k, _stream())
        if st:
            raise RuntimeError(f"lx_moe_experts_grouped failed: {st}")
        return out


def expert_range(E: int, rank: int, world: int) -> tuple[int, int]:
    return E * rank // world, E * (rank + 1) // world


def remap_for_owner(ids: torch.Tensor, weights: torch.Tensor, e0: int, e1: int):
    """The routing as the owner of experts [e0, e1) sees it: pairs routed elsewhere keep a valid local expert id but
    weight zero, so they add nothing; owned pairs keep their weight. Pure index arithmetic (also used by the CPU tests)."""
    mine = (ids >= e0) & (ids < e1)
    local_ids = torch.where(mine, ids - e0, torch.zeros_like(ids))
    local_w = torch.where(mine, weights, torch.zeros_like(weights))
    return local_ids, local_w, mine


class ReplicatedExpertParallel:
    """Experts split over ranks with routing and tokens replicated: rank g holds the stacks of experts [g E / G, (g + 1) E / G)
    and every rank calls with the same latent, ids and weights of all T tokens. Three library calls, no host read-back
    (so the call can be captured in a graph): the weighted rows of this rank's experts, their exchange as flag-in-data
    packets over peer memory, the sum of each token's rows in k order: bit for bit what Experts gives on one GPU.

    The receive buffers (torch symmetric memory, plain peer mappings) are sized for max_tokens."""

    def __init__(self, lib, gate_up_local: StoredWeight, down_local: StoredWeight, E: int, L: int, I: int, top_k: int, max_tokens: int,
                 device, group=None, math: int = abi.MATH_BF16):
        import torch.distributed as dist

        self.lib, self.gate_up, self.down, self.E, self.L, self.I, self.top_k, self.math = lib, gate_up_local, down_local, E, L, I, top_k, math
        self.dist, self.group = dist, group
        multi = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        if self.world > 8:
            raise RuntimeError("the row exchange addresses at most 8 ranks")
        self.bounds = [expert_range(E, r, self.world)[0] for r in range(self.world)] + [E]
        self.bounds_array = (ctypes.c_int * (self.world + 1))(*self.bounds)
        self.max_tokens = max_tokens
        self.rows = torch.empty((max_tokens * top_k, L), dtype=torch.float32, device=device)
        self.ws = torch.empty(max(256, lib.lx_moe_grouped_workspace_bytes(max_tokens, L, I, E, top_k, math)), dtype=torch.uint8, device=device)
        self.seq = torch.zeros((64,), dtype=torch.int32, device=device)  # word 0: sequence, word 32: CTA counter
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            self.packets = max_tokens * top_k * (L // 2)
            self.boxes = symm.empty((2, self.packets, 4), dtype=torch.int32, device=device)
            self.boxes.zero_()
            hb = symm.rendezvous(self.boxes, group if group is not None else dist.group.WORLD)
            self.box_array = (ctypes.c_void_p * self.world)(*[int(p) for p in hb.buffer_ptrs])
            torch.cuda.synchronize()
            dist.barrier(group)

    def owned(self, latent, ids, weights, e0: int | None = None, e1: int | None = None):
        """The first call alone: this rank's (or the given range's) weighted rows into self.rows."""
        T = latent.shape[0]
        assert T <= self.max_tokens
        e0 = self.bounds[self.rank] if e0 is None else e0
        e1 = self.bounds[self.rank + 1] if e1 is None else e1
        gu = self.gate_up.ref() if self.gate_up is not None else None  # a rank that owns no expert holds no stacks
        dn = self.down.ref() if self.down is not None else None
        st = self.lib.lx_b200_moe_experts_owned(abi.ptr(latent), abi.ptr(ids), abi.ptr(weights), gu, dn, self.math,
                                                abi.ptr(self.rows), abi.ptr(self.ws), T, self.L, self.I, self.E, e0, e1, self.top_k, _stream())
        if st:
            raise RuntimeError(f"lx_b200_moe_experts_owned failed: {st}")

    def sum(self, T: int, out: torch.Tensor):
        st = self.lib.lx_b200_moe_sum_rows(abi.ptr(self.rows), abi.ptr(out), T, self.L, self.top_k, _stream())
        if st:
            raise RuntimeError(f"lx_b200_moe_sum_rows failed: {st}")
        return out

    def __call__(self, latent: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """latent bf16 [T, L], ids / weights [T, top_k] of ALL tokens (the same on every rank) -> f32 [T, L] on every rank."""
        T = latent.shape[0]
        if out is None:
            out = torch.empty((T, self.L), dtype=torch.float32, device=latent.device)
        self.owned(latent, ids, weights)
        if self.world > 1:
            st = self.lib.lx_b200_moe_exchange_rows(abi.ptr(self.rows), abi.ptr(self.ws), self.box_array, self.packets, abi.ptr(self.seq),
                                                    abi.ptr(self.seq[32:]), self.world, self.rank, self.bounds_array, T, self.L, self.I, self.E,
                                                    self.top_k, _stream())
            if st:
                raise RuntimeError(f"lx_b200_moe_exchange_rows failed: {st}")
        return self.sum(T, out)


class ExpertParallel:
    """Experts split over ranks: rank g holds experts [g E / G, (g + 1) E / G). Tokens are split over ranks too (rank g
    is home to tokens [g T / G, (g + 1) T / G)); the routed rows are exchanged with one all-to-all each way:

      dispatch  every rank sends each peer the latent rows of its own tokens that route to that peer's experts, with
                the pair's local expert id, weight and home position;
      compute   the owner runs its experts on the rows it received (one pair per row, top_k = 1);
      combine   the weighted rows go back to the token's home rank, which adds each token's top_k rows in k order.

    Routing itself is replicated: every rank computes lx_moe_route on its own tokens' logits."""

    def __init__(self, lib, gate_up_local: StoredWeight, down_local: StoredWeight, E: int, L: int, I: int, top_k: int, group=None):
        import torch.distributed as dist

        self.dist, self.group = dist, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.E, self.L, self.I, self.top_k = E, L, I, top_k
        self.e0, self.e1 = expert_range(E, self.rank, self.world)
        # the owner sees one (expert, weight) pair per received row
        self.local = Experts(lib, gate_up_local, down_local, self.e1 - self.e0, L, I, 1)

    def plan(self, ids: torch.Tensor):
        """Which of this rank's (token, k) pairs go to which rank, in destination order. Returns (order, counts): `order`
        lists pair indices sorted by destination rank (stable), counts[r] how many go to rank r."""
        flat = ids.reshape(-1).to(torch.int64)
        dest = torch.zeros_like(flat)
        for r in range(1, self.world):
            dest += (flat >= expert_range(self.E, r, self.world)[0]).to(torch.int64)
        order = torch.sort(dest, stable=True).indices
        counts = torch.bincount(dest, minlength=self.world)
        return order, counts

    def __call__(self, latent: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """latent bf16 [T_local, L], ids / weights [T_local, top_k] of this rank's tokens -> f32 [T_local, L]."""
        dist, W = self.dist, self.world
        T, k = ids.shape
        order, counts = self.plan(ids)
        send_counts = counts.tolist()
        recv_counts_t = torch.empty_like(counts)
        if W > 1:
            dist.all_to_all_single(recv_counts_t, counts, group=self.group)
        else:
            recv_counts_t = counts.clone()
        recv_counts = recv_counts_t.tolist()
        n_send, n_recv = sum(send_counts), sum(recv_counts)
        tok = torch.div(order, k, rounding_mode="floor")
        send_rows = latent[tok].contiguous()                                   # [n_send, L] bf16
        send_meta = torch.stack([ids.reshape(-1)[order].to(torch.float32), weights.reshape(-1)[order]], dim=1).contiguous()
        recv_rows = torch.empty((n_recv, self.L), dtype=latent.dtype, device=latent.device)
        recv_meta = torch.empty((n_recv, 2), dtype=torch.float32, device=latent.device)
        if W > 1:
            dist.all_to_all_single(recv_rows, send_rows, recv_counts, send_counts, group=self.group)
            dist.all_to_all_single(recv_meta, send_meta, recv_counts, send_counts, group=self.group)
        else:
            recv_rows, recv_meta = send_rows, send_meta
        out_rows = torch.zeros((n_recv, self.L), dtype=torch.float32, device=latent.device)
        if n_recv:
            local_ids = (recv_meta[:, 0].to(torch.int32) - self.e0).reshape(n_recv, 1).contiguous()
            local_w = recv_meta[:, 1].reshape(n_recv, 1).contiguous()
            self.local(recv_rows, local_ids, local_w, out_rows)
        back = torch.empty((n_send, self.L), dtype=torch.float32, device=latent.device)
        if W > 1:
            dist.all_to_all_single(back, out_rows, send_counts, recv_counts, group=self.group)
        else:
            back = out_rows
        # back[i] belongs to pair order[i]; add each token's rows in k order (fixed order: deterministic)
        per_pair = torch.empty((T * k, self.L), dtype=torch.float32, device=latent.device)
        per_pair[order] = back
        per_pair = per_pair.reshape(T, k, self.L)
        out = per_pair[:, 0].clone()
        for j in range(1, k):
            out += per_pair[:, j]
        return out


def packet_plan(N: int, world: int, elem_bytes: int, max_rows: int, packet_bytes: int):
    """The geometry of the packet exchange for an [max_rows, N] output split over `world` ranks: the column bounds of the
    ranks' slices, the packets a rank's region of a receive buffer holds (rows that may travel as packets x 8-byte pieces of
    the widest slice), and whether slices are whole 8-byte pieces at all. Pure arithmetic (tested on CPU)."""
    bounds = [shard_rows(N, r, world)[0] for r in range(world)] + [N]
    widest = max(bounds[r + 1] - bounds[r] for r in range(world))
    rows = min(max_rows, max(1, packet_bytes // max(1, widest * elem_bytes * max(1, world - 1))))
    region = rows * ((widest * elem_bytes + 7) // 8)
    ok = all((b * elem_bytes) % 8 == 0 for b in bounds) and (N * elem_bytes) % 8 == 0
    return bounds, region, ok


def travels_as_packets(M: int, bounds, region: int, ok: bool, elem_bytes: int, packet_bytes: int) -> bool:
    """The default choice between the two exchanges for M rows: packets when the slices fit the regions and what a rank sends
    (its slice to every peer) is at most packet_bytes."""
    world = len(bounds) - 1
    widest = max(bounds[r + 1] - bounds[r] for r in range(world))
    fits = ok and M * ((widest * elem_bytes + 7) // 8) <= region
    return fits and M * widest * elem_bytes * max(1, world - 1) <= packet_bytes


class PeerBuffers:
    """What the ranks of a row-sharded layer share: two whole-y buffers used in turn (so that a rank one call ahead never
    overwrites the y a slower rank still reads) and the arrival counters, all torch symmetric memory (plain peer mappings,
    multicast off), exchanged once at construction. One set serves any number of layers of the same output width.

    The y buffer of a call is picked here, on the host, by the count of calls: a captured graph that is replayed back to
    back must hold an even number of calls, or the last call of one replay and the first of the next share a buffer and
    a peer one call ahead stores into a y this rank may still read. (The packet exchange has no such rule: peers never
    write into y, and the half of the receive buffer is picked on the device from the sequence number.)"""

    def __init__(self, N: int, max_rows: int, device, dtype=torch.float32, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.dist, self.group = dist, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise RuntimeError("the exchange kernel addresses at most 8 ranks")
        self.N, self.max_rows, self.dtype = N, max_rows, dtype
        self.y = symm.empty((2, max_rows, N), dtype=dtype, device=device)
        self.counter = symm.empty((64,), dtype=torch.int32, device=device)
        self.counter.zero_()
        hy, hc = symm.rendezvous(self.y, self.group), symm.rendezvous(self.counter, self.group)
        self.y_ptrs, self.c_ptrs = [int(p) for p in hy.buffer_ptrs], [int(p) for p in hc.buffer_ptrs]
        self.c_array = (ctypes.c_void_p * self.world)(*self.c_ptrs)
        # the packet exchange of small slices: per y buffer a receive buffer of one region per rank, a sequence word and a
        # CTA counter (both this rank's own). Slices above packet_bytes go through the store-and-semaphore exchange.
        # Measured on two B200s (f32 y, N = 28672 split in two): 57 KB slices 4.9 us as packets against 14.4 us; 0.9 MB 7.3
        # against 16.6; 1.8 MB 10.3 against 17.8; 3.7 MB 18.7 against 19.8. Packets put twice the bytes on the wire, once
        # per peer, so the limit is on what a rank sends.
        self.packet_bytes = int(os.environ.get("LX_B200_PACKET_BYTES", str(3 << 20)))
        self.bounds, self.region, self.packets_ok = packet_plan(N, self.world, self.y.element_size(), max_rows, self.packet_bytes)
        self.boxes = symm.empty((2, self.world, self.region, 4), dtype=torch.int32, device=device)
        self.boxes.zero_()
        hb = symm.rendezvous(self.boxes, self.group)
        self.b_ptrs = [int(p) for p in hb.buffer_ptrs]
        self.seq = torch.zeros((64,), dtype=torch.int32, device=device)  # word 0: sequence, word 32: CTA counter (separate lines)
        self.box_array = (ctypes.c_void_p * self.world)(*self.b_ptrs)
        self.bounds_array = (ctypes.c_int64 * (self.world + 1))(*self.bounds)
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def next_half(self) -> int:
        half = self.calls & 1
        self.calls += 1
        return half

    def y_array(self, half: int):
        stride = self.max_rows * self.N * self.y.element_size()
        return (ctypes.c_void_p * self.world)(*[p + half * stride for p in self.y_ptrs])

    def exchange(self, lib, half: int, M: int, packets: bool | None = None):
        """Makes y[half, :M] whole on every rank (every rank has written its own columns). packets: force one of the two
        exchanges; by default slices of at most packet_bytes travel as packets."""
        y_dt = abi.BF16 if self.dtype == torch.bfloat16 else abi.F32
        n0, n1 = self.bounds[self.rank], self.bounds[self.rank + 1]
        esz = self.y.element_size()
        widest = max(self.bounds[r + 1] - self.bounds[r] for r in range(self.world))
        if packets is None:
            packets = travels_as_packets(M, self.bounds, self.region, self.packets_ok, esz, self.packet_bytes)
        if packets:
            if not (self.packets_ok and M * ((widest * esz + 7) // 8) <= self.region):
                raise RuntimeError("the slices do not fit the packet buffers")
            st = lib.lx_b200_exchange_packets(abi.ptr(self.y[half]), self.box_array, self.region, abi.ptr(self.seq), abi.ptr(self.seq[32:]),
                                              self.world, self.rank, self.bounds_array, y_dt, self.N, M, _stream())
        else:
            st = lib.lx_b200_exchange_slices(self.y_array(half), self.c_array, self.world, self.rank, n0, n1 - n0, y_dt, self.N, M, _stream())
        if st:
            raise RuntimeError(f"the exchange of output slices failed: {st}")


class PeerShardedLinear:
    """ShardedLinear without the collective library: the product writes this rank's columns straight into its own copy of
    the whole y, and lx_b200_exchange_slices (one kernel: peer stores over NVLink, one arrival per rank, a bounded wait)
    makes every rank's copy whole. Any weight format and row count: the product is the plain Linear."""

    def __init__(self, lib, stored: StoredWeight, N: int, K: int, buffers: PeerBuffers, packets: bool | None = None):
        self.lib, self.buf, self.N, self.K, self.packets = lib, buffers, N, K, packets
        self.n0, self.n1 = shard_rows(N, buffers.rank, buffers.world)
        self.local = Linear(lib, stored, self.n1 - self.n0, K)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """x: bf16 or f32 [M, K], the same on every rank. Returns this rank's whole y [M, N] (valid on the stream)."""
        M, b = x.shape[0], self.buf
        assert M <= b.max_rows
        half = b.next_half()
        self.local(x, b.y[half, :M, self.n0:self.n1])
        b.exchange(self.lib, half, M, self.packets)
        return b.y[half, :M]


class FusedShardedLinear:
    """ShardedLinear without the collective: every rank's product stores its slice of y straight into every rank's copy
    of the whole y (lx_b200_linear_allgather: NVLink stores from the kernel's epilogue through peer-mapped pointers) and
    counts itself on every rank's arrival counter; lx_b200_wait_arrivals then holds the stream until all slices are in.
    The buffers and counters are torch symmetric memory (one allocation per layer, exchanged once at construction).

    Each layer owns two whole-y buffers used in turn, so that a rank one call ahead never overwrites the y a slower rank
    is still reading. Raises if symmetric memory or the tensor-core product is not available for this weight; callers
    then use ShardedLinear (NCCL all-gather)."""

    def __init__(self, lib, w_bf16_shard: torch.Tensor | None, wtype: int, N: int, K: int, max_rows: int, group=None,
                 stored: StoredWeight | None = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only
        self.lib, self.dist, self.group = lib, dist, group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 8:
            raise RuntimeError("the all-gather epilogue addresses at most 8 ranks")
        self.N, self.K, self.max_rows = N, K, max_rows
        self.n0, self.n1 = shard_rows(N, self.rank, self.world)
        self.weight = stored if stored is not None else store_weight(lib, w_bf16_shard.contiguous(), wtype)
        dev = self.weight.data.device
        self.y = symm.empty((2, max_rows, N), dtype=torch.float32, device=dev)
        self.counter = symm.empty((64,), dtype=torch.int32, device=dev)
        self.counter.zero_()
        hy, hc = symm.rendezvous(self.y, self.group), symm.rendezvous(self.counter, self.group)
        self._y_ptrs, self._c_ptrs = [int(p) for p in hy.buffer_ptrs], [int(p) for p in hc.buffer_ptrs]
        self._c_array = (ctypes.c_void_p * self.world)(*self._c_ptrs)
        self._calls, self._total = 0, {}
        self._ws = None
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """x: bf16 or f32 [M, K], the same on every rank. Returns this rank's whole y, f32 [M, N] (valid on the stream)."""
        M = x.shape[0]
        assert M <= self.max_rows
        half = self._calls & 1
        self._calls += 1
        stride = self.max_rows * self.N * 4
        y_array = (ctypes.c_void_p * self.world)(*[p + half * stride for p in self._y_ptrs])
        need = self.lib.lx_gemm_workspace_bytes(M, self.K, abi.MATH_BF16)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
        added = ctypes.c_int(0)
        x_dt = abi.BF16 if x.dtype == torch.bfloat16 else abi.F32
        st = self.lib.lx_b200_linear_allgather(abi.ptr(x), x_dt, x.stride(0), self.weight.ref(), None, abi.BF16, y_array, self._c_array,
                                               self.world, self.rank, self.n0, abi.F32, self.N, M, self.n1 - self.n0, self.K, 1.0,
                                               abi.ptr(self._ws),
                                               ctypes.byref(added), _stream())
        if st:
            raise RuntimeError(f"lx_b200_linear_allgather failed: {st}")
        if M not in self._total:  # what one round adds to a counter: every rank's share, exchanged once per row count
            shares = [None] * self.world
            self.dist.all_gather_object(shares, int(added.value), group=self.group)
            self._total[M] = int(sum(shares))
        st = self.lib.lx_b200_wait_arrivals(self._c_ptrs[self.rank], self._total[M], _stream())
        if st:
            raise RuntimeError(f"lx_b200_wait_arrivals failed: {st}")
        return self.y[half, :M]
