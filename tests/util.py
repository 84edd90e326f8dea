"""Shared helpers of the tests: seeded inputs generated on the host (so the oracle and the GPU see the same bits),
device buffers, and calls through the C ABI."""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O

TORCH_OF = {np.dtype(np.uint16): torch.int16, np.dtype(np.uint8): torch.uint8, np.dtype(np.int8): torch.int8,
            np.dtype(np.float32): torch.float32, np.dtype(np.int32): torch.int32}


def bf16_normal(shape, std, seed):
    """bf16 bit patterns (uint16) of N(0, std) drawn with a seeded CPU generator."""
    g = torch.Generator().manual_seed(seed)
    t = (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def f32_normal(shape, std, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).numpy().copy()


def dev(a: np.ndarray) -> torch.Tensor:
    """A device copy of a host array (uint16 travels as int16: same bits)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).cuda()
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).cuda()
    return torch.from_numpy(a).cuda()


def host(t: torch.Tensor, dtype=None) -> np.ndarray:
    a = t.detach().cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class DeviceWeight:
    """An oracle Weight copied to the device, with its lx_weight struct."""

    def __init__(self, w: O.Weight):
        self.host = w
        self.data = dev(w.data)
        self.scale = None if w.scale is None else dev(w.scale)
        self.expert_global = None if w.expert_global is None else dev(np.asarray(w.expert_global, dtype=np.float32))
        self.struct = abi.make_weight(w.wtype, self.data, self.scale, float(w.glob), self.expert_global)

    def ref(self):
        return ctypes.byref(self.struct)


def make_weight(w_bits: np.ndarray, wtype: int) -> O.Weight:
    """The stored form of a bf16 matrix in a format, by the oracle's quantizers / encoder."""
    if wtype == O.W_BF16X:
        rows, K = w_bits.reshape(-1, w_bits.shape[-1]).shape
        return O.Weight(O.W_BF16X, O.bf16x_encode(w_bits.reshape(rows, K)))
    return O.quantize_weight(w_bits, wtype)


def reference_weight(w_bits: np.ndarray, wt: O.Weight) -> O.Weight:
    """The weight whose exact values a product on `wt` must use (BF16X stands for the bf16 matrix itself)."""
    return O.Weight(O.W_BF16, w_bits) if wt.wtype == O.W_BF16X else wt


def gemv(lx, x_dev, x_dtype, ld_x, dw: DeviceWeight, y_dev, y_dtype, ld_y, M, N, K, bias=None, bias_dtype=abi.BF16,
         alpha=1.0, beta=0.0, fn="lx_gemv_w", math=None, workspace=None):
    if fn == "lx_gemm_w":
        return lx.lx_gemm_w(abi.ptr(x_dev), x_dtype, ld_x, dw.ref(), math or 0, abi.ptr(bias), bias_dtype, abi.ptr(y_dev),
                            y_dtype, ld_y, M, N, K, alpha, beta, abi.ptr(workspace), stream_ptr())
    return lx.lx_gemv_w(abi.ptr(x_dev), x_dtype, ld_x, dw.ref(), abi.ptr(bias), bias_dtype, abi.ptr(y_dev), y_dtype, ld_y,
                        M, N, K, alpha, beta, stream_ptr())


def check_status(lx):
    torch.cuda.synchronize()
    assert lx.lx_b200_last_error() == 0, "a bounded wait inside a kernel ran out"


def assert_close(got, want, rel_l2=1e-3, max_abs=2e-2, what=""):
    """The acceptance bound of the decode products: rel-L2 <= 1e-3 and max-abs <= 2e-2 against the float64 oracle."""
    r, a = O.rel_l2(got, want), O.max_abs(got, want)
    assert np.all(np.isfinite(np.asarray(got, dtype=np.float64))), f"{what}: non-finite output"
    assert r <= rel_l2 and a <= max_abs, f"{what}: rel-L2 {r:.3e} (<= {rel_l2}), max-abs {a:.3e} (<= {max_abs})"
