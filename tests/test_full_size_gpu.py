"""The configurations the headline metric is quoted on, at full size (C1 - C4 of the baseline), through the C ABI.

The float64 oracle takes seconds per full matrix, so at these sizes parity is checked three ways that do not grow with
N: (1) a sample of output rows against the oracle, computed from the very bytes the device holds for those rows;
(2) homogeneity, y(2 x) = 2 y(x) bit for bit over the whole output (a power of two passes through every scaling,
digit and rounding step exactly); (3) batch invariance, row 0 of the largest batch equals the single-row call bit for
bit where the contract promises it (up to 8 rows through lx_gemv_w; every row count through lx_gemm_w).
"""

import numpy as np
import pytest
import torch

from dromos_b200 import abi, host
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu

CONFIGS = [
    ("c1_bf16", abi.W_BF16, 4096, 4096, (1,)),
    ("c2_int8", abi.W_INT8, 14336, 4096, (1, 8, 32)),
    ("c3_fp8", abi.W_FP8, 28672, 8192, (1, 16, 64)),
    ("c3_nvfp4", abi.W_NVFP4, 28672, 8192, (1, 16, 64)),
    ("c4_bf16x", abi.W_BF16X, 14336, 4096, (1,)),
]


def sampled_weight(sw, w_bf16, rows, K):
    """The oracle's view of the sampled rows, from the bytes on the device (BF16X: from the bf16 source, the format is
    lossless and its codec is tested byte for byte elsewhere)."""
    idx = torch.as_tensor(rows, device="cuda")
    if sw.wtype in (abi.W_BF16, abi.W_BF16X):
        return O.Weight(O.W_BF16, w_bf16[idx].view(torch.int16).cpu().numpy().view(np.uint16))
    if sw.wtype == abi.W_NVFP4:
        data = sw.data.view(-1, K // 2)[idx].cpu().numpy()
        scale = sw.scale.view(-1, K // 16)[idx].cpu().numpy()
        return O.Weight(O.W_NVFP4, data, scale, sw.glob)
    data = sw.data.view(-1, K)[idx].cpu().numpy()
    data = data.view(np.int8) if sw.wtype == abi.W_INT8 else data
    return O.Weight(sw.wtype, data, sw.scale[idx].cpu().numpy())


@pytest.mark.parametrize("name,wtype,N,K,Ms", CONFIGS, ids=[c[0] for c in CONFIGS])
def test_full_size_configuration(lx, name, wtype, N, K, Ms):
    gen = torch.Generator(device="cuda").manual_seed(7)
    w = (torch.randn((N, K), generator=gen, device="cuda") * 0.02).to(torch.bfloat16)
    sw = host.store_weight(lx, w, wtype)
    layer = host.Linear(lx, sw, N, K)
    rows = np.sort(np.random.default_rng(3).choice(N, size=48, replace=False))
    rows[0], rows[-1] = 0, N - 1
    wt = sampled_weight(sw, w, rows, K)
    m_max = max(Ms)
    x = torch.randn((m_max, K), generator=gen, device="cuda").to(torch.bfloat16)
    xv = O.bf16_bits_to_f32(x.view(torch.int16).cpu().numpy().view(np.uint16)).astype(np.float64)
    first = {}
    for M in Ms:
        y = layer(x[:M]).clone()
        y2 = layer((x[:M].float() * 2).to(torch.bfloat16)).clone()
        torch.cuda.synchronize()
        util.check_status(lx)
        got = y.cpu().numpy()
        assert np.all(np.isfinite(got)), f"{name} M={M}: non-finite"
        want = O.gemv_reference(xv[:M], wt)
        util.assert_close(got[:, rows], want, what=f"{name} M={M}, sampled rows")
        assert torch.equal(y2, y * 2), f"{name} M={M}: y(2x) != 2 y(x)"
        first[M] = got[0].view(np.uint32).copy()
    small = [M for M in Ms if M <= 8]
    for M in small[1:]:
        assert np.array_equal(first[M], first[small[0]]), f"{name}: row 0 at M={M} differs from M={small[0]}"
    large = [M for M in Ms if M > 8]
    for M in large[1:]:
        assert np.array_equal(first[M], first[large[0]]), f"{name}: row 0 at M={M} differs from M={large[0]}"


def test_full_size_routed_experts(lx):
    """C5: E = 64, top-8, L = 4096, I = 1536, FP8 stacks, T = 32. Two sampled tokens against the float64 oracle computed
    from the device's own bytes of the experts those tokens picked (SwiGLU is not homogeneous, so there is no doubling
    check here); and a token's bits do not depend on its batch: the same token routed alone gives the same row."""
    E, top_k, L, I, T = 64, 8, 4096, 1536, 32
    gen = torch.Generator(device="cuda").manual_seed(11)
    gu = host.store_weight(lx, (torch.randn((E, 2 * I, L), generator=gen, device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    dn = host.store_weight(lx, (torch.randn((E, L, I), generator=gen, device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    layer = host.Experts(lx, gu, dn, E, L, I, top_k)
    latent = torch.randn((T, L), generator=gen, device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), generator=gen, device="cuda")
    ids, weights = layer.route(logits)
    out = layer(latent, ids, weights).clone()
    torch.cuda.synchronize()
    util.check_status(lx)
    got = out.cpu().numpy()
    assert np.all(np.isfinite(got))
    ids_h, w_h = ids.cpu().numpy(), weights.cpu().numpy()
    lat_h = O.bf16_bits_to_f32(latent.view(torch.int16).cpu().numpy().view(np.uint16)).astype(np.float64)
    gu_data, gu_scale = gu.data.view(E, 2 * I, L), gu.scale.view(E, 2 * I)
    dn_data, dn_scale = dn.data.view(E, L, I), dn.scale.view(E, L)
    for t in (0, T - 1):
        want = np.zeros(L, dtype=np.float64)
        for k in range(top_k):
            e = int(ids_h[t, k])
            wg = O.weight_f64(O.Weight(O.W_FP8, gu_data[e].cpu().numpy(), gu_scale[e].cpu().numpy()))
            wd = O.weight_f64(O.Weight(O.W_FP8, dn_data[e].cpu().numpy(), dn_scale[e].cpu().numpy()))
            h = wg @ lat_h[t]
            g, u = h[:I], h[I:]
            mid = O.bf16_bits_to_f32(O.f32_to_bf16_bits((g / (1.0 + np.exp(-g)) * u).astype(np.float32))).astype(np.float64)
            want += float(w_h[t, k]) * (wd @ mid)
        util.assert_close(got[t], want, what=f"c5_moe_fp8 token {t}")
    # the last token alone: same bits
    alone = layer(latent[T - 1:].contiguous(), ids[T - 1:].contiguous(), weights[T - 1:].contiguous()).clone()
    torch.cuda.synchronize()
    assert torch.equal(alone[0], out[T - 1]), "a token's bits depend on its batch"


def test_full_size_few_token_experts(lx):
    """The C5 stacks (E = 64, top-8, L = 4096, I = 1536, FP8) through lx_moe_experts_decode at T = 1 and T = 8: sampled
    tokens against the float64 oracle on the device's own bytes of the experts they picked, and every token of the batch
    equal to that token alone, bit for bit."""
    E, top_k, L, I, T = 64, 8, 4096, 1536, 8
    gen = torch.Generator(device="cuda").manual_seed(12)
    gu = host.store_weight(lx, (torch.randn((E, 2 * I, L), generator=gen, device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    dn = host.store_weight(lx, (torch.randn((E, L, I), generator=gen, device="cuda") * 0.02).to(torch.bfloat16), abi.W_FP8)
    latent = torch.randn((T, L), generator=gen, device="cuda").to(torch.bfloat16)
    logits = torch.randn((T, E), generator=gen, device="cuda")
    ids, weights = host.Experts(lx, gu, dn, E, L, I, top_k).route(logits)
    ws = torch.full((lx.lx_moe_decode_workspace_bytes(T, I, top_k),), 0xFF, dtype=torch.uint8, device="cuda")

    def decode(t0, t1):
        out = torch.full((t1 - t0, L), float("nan"), device="cuda")
        st = lx.lx_moe_experts_decode(abi.ptr(latent[t0:t1]), abi.ptr(ids[t0:t1]), abi.ptr(weights[t0:t1]), gu.ref(), dn.ref(),
                                      abi.ptr(out), abi.ptr(ws), t1 - t0, L, I, top_k, util.stream_ptr())
        assert st == 0, st
        util.check_status(lx)
        return out

    batch = decode(0, T)
    for t in range(T):
        assert torch.equal(decode(t, t + 1)[0], batch[t]), f"token {t} of the batch differs from the token alone"
    got = batch.cpu().numpy()
    ids_h, w_h = ids.cpu().numpy(), weights.cpu().numpy()
    lat_h = O.bf16_bits_to_f32(latent.view(torch.int16).cpu().numpy().view(np.uint16)).astype(np.float64)
    gu_data, gu_scale = gu.data.view(E, 2 * I, L), gu.scale.view(E, 2 * I)
    dn_data, dn_scale = dn.data.view(E, L, I), dn.scale.view(E, L)
    for t in (0, T - 1):
        want = np.zeros(L, dtype=np.float64)
        for k in range(top_k):
            e = int(ids_h[t, k])
            wg = O.weight_f64(O.Weight(O.W_FP8, gu_data[e].cpu().numpy(), gu_scale[e].cpu().numpy()))
            wd = O.weight_f64(O.Weight(O.W_FP8, dn_data[e].cpu().numpy(), dn_scale[e].cpu().numpy()))
            h = wg @ lat_h[t]
            g, u = h[:I], h[I:]
            mid = O.bf16_bits_to_f32(O.f32_to_bf16_bits((g / (1.0 + np.exp(-g)) * u).astype(np.float32))).astype(np.float64)
            want += float(w_h[t, k]) * (wd @ mid)
        util.assert_close(got[t], want, what=f"few-token experts, token {t}")
