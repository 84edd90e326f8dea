"""ctypes bindings for the Dromos kernel C ABI (the hot-path subset declared in include/dromos_b200.h).

The same bindings load any library that exports the ABI of lernex/dromos engine/cuda/kernels.h: this
package's CUDA library (device pointers) or the reference's CPU backend (host pointers), which is how the
parity tests drive both sides with one harness, as the reference's own tests/kernels/conftest.py does.
Nothing here computes anything: a missing library or symbol raises.
"""

from __future__ import annotations

import ctypes
import os

W_BF16, W_INT8, W_FP8, W_NVFP4, W_BF16X = 0, 1, 2, 3, 4
MATH_BF16, MATH_INT8, MATH_FP8, MATH_FP4 = 0, 1, 2, 3
F32, BF16 = 0, 1
ERR_INVALID, ERR_NOT_SUPPORTED, ERR_TUNE_REJECTED, ERR_TUNE_VARIANT = 1, 801, 802, 803

c_int, c_i64, c_f32, c_ptr = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p


class LxWeight(ctypes.Structure):
    """lx_weight (engine/cuda/kernels.h:411-417): a host struct whose pointers are device pointers."""

    _fields_ = [("type", c_int), ("data", c_ptr), ("scale", c_ptr), ("glob", c_f32), ("expert_global", c_ptr)]


class LxTuneProblem(ctypes.Structure):
    """lx_tune_problem (engine/cuda/tunable.h:57-62)."""

    _fields_ = [("M", c_int), ("N", c_int), ("K", c_int), ("experts", c_int), ("weight", c_int), ("math", c_int)]


# name -> (restype, argtypes). The argument lists are those of kernels.h / tunable.h, in order.
_W = ctypes.POINTER(LxWeight)
SIGNATURES = {
    "lx_gemv_w": (c_int, [c_ptr, c_int, c_int, _W, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr]),
    "lx_gemv": (c_int, [c_ptr, c_int, c_int, c_ptr, c_int, c_ptr, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr]),
    "lx_gemv_bf16x": (c_int, [c_ptr, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr]),
    "lx_gemv_decode_bf16": (c_int, [c_ptr, c_int, c_int, c_ptr, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr]),
    "lx_gemm_w": (c_int, [c_ptr, c_int, c_int, _W, c_int, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr, c_ptr]),
    "lx_gemm_workspace_bytes": (c_i64, [c_int, c_int, c_int]),
    "lx_gemm_skinny": (c_int, [c_ptr, c_int, c_int, _W, c_ptr, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_f32, c_f32, c_ptr]),
    "lx_quantize_act": (c_int, [c_ptr, c_int, c_int, c_int, c_ptr, c_int, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr]),
    "lx_quantize_weight": (c_int, [c_ptr, _W, c_i64, c_int, c_ptr]),
    "lx_dequantize_weight": (c_int, [_W, c_ptr, c_i64, c_int, c_ptr]),
    "lx_quantize_w8": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_int, c_ptr]),
    "lx_bf16x_row_bytes": (c_i64, [c_int]),
    "lx_bf16x_bytes": (c_i64, [c_ptr, c_i64, c_int, c_ptr]),
    "lx_bf16x_encode": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_i64, c_ptr]),
    "lx_bf16x_decode": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_ptr]),
    "lx_spec_gemv_f32": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_route": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_ptr]),
    "lx_router_route": (c_int, [c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_experts_grouped": (c_int, [c_ptr, c_ptr, c_ptr, _W, _W, c_int, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_grouped_workspace_bytes": (c_i64, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "lx_moe_experts_decode": (c_int, [c_ptr, c_ptr, c_ptr, _W, _W, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_decode_workspace_bytes": (c_i64, [c_int, c_int, c_int]),
    "lx_moe_experts_bf16x": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_experts_decode_bf16": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_moe_bf16x_workspace_bytes": (c_i64, [c_int, c_int, c_int]),
    "lx_moe_experts": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_arch": (c_int, []),
    "lx_set_arch_override": (c_int, [c_int]),
    "lx_tune_get": (c_int, [ctypes.c_char_p, c_int, c_int, c_int]),
    "lx_tune_set": (c_int, [ctypes.c_char_p, c_int, c_int, c_int, c_int]),
    "lx_tune_force": (c_int, [ctypes.c_char_p, c_int, c_int, c_int, c_int]),
    "lx_tune_clear": (None, []),
    "lx_tune_kernels": (c_int, [ctypes.POINTER(ctypes.c_char_p), c_int]),
    "lx_tune_variants": (c_int, [ctypes.c_char_p]),
    "lx_tune_variant_name": (ctypes.c_char_p, [ctypes.c_char_p, c_int]),
    "lx_tune_run": (c_int, [ctypes.c_char_p, c_int, ctypes.POINTER(LxTuneProblem), c_ptr, c_ptr]),
    "lx_tune_runnable": (c_int, [ctypes.c_char_p]),
    "lx_tune_key": (c_int, [ctypes.c_char_p, ctypes.POINTER(LxTuneProblem), ctypes.c_char_p, c_int]),
    "lx_rt_backend": (c_int, []),
    "lx_rt_device_count": (c_int, []),
    "lx_bandwidth_probe": (c_int, [c_i64, c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double), c_ptr]),
}

# Entry points that exist only in this package's library (declared in include/dromos_b200.h, no reference counterpart).
EXTENSIONS = {
    "lx_b200_kernel_launches": (c_i64, []),
    "lx_b200_last_error": (c_int, []),
    "lx_b200_gemv_ring_plan": (c_int, [c_int, c_int, c_int, c_int, c_ptr]),
    "lx_b200_moe_experts_grouped_static": (c_int, [c_ptr, c_ptr, c_ptr, _W, _W, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_b200_moe_static_scratch_bytes": (c_i64, []),
    "lx_b200_moe_static_scratch_ptr": (c_ptr, []),
    # x, x_dtype, ld_x, w, bias, bias_dtype, y_all, arrivals, ranks, rank, col0, y_dtype, ld_y, M, N, K, alpha, workspace, arrivals_added, stream
    "lx_b200_linear_allgather": (c_int, [c_ptr, c_int, c_int, _W, c_ptr, c_int, c_ptr, c_ptr, c_int, c_int, c_i64, c_int, c_int, c_int, c_int,
                                         c_int, ctypes.c_float, c_ptr, c_ptr, c_ptr]),
    "lx_b200_wait_arrivals": (c_int, [c_ptr, c_int, c_ptr]),
    # y_all, arrivals, ranks, rank, col0, cols, y_dtype, ld_y, M, stream
    "lx_b200_exchange_slices": (c_int, [c_ptr, c_ptr, c_int, c_int, c_i64, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_b200_moe_experts_owned": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_b200_moe_exchange_rows": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_int, c_int, c_ptr, c_int, c_int, c_int, c_int, c_int, c_ptr]),
    "lx_b200_moe_sum_rows": (c_int, [c_ptr, c_ptr, c_int, c_int, c_int, c_ptr]),
    "lx_b200_exchange_packets": (c_int, [c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_int, c_int, c_ptr, c_int, c_int, c_int, c_ptr]),
}
ERR_SCRATCH = 804


def default_library_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "libdromos_b200.so")


def ptr(a):
    """A device/host address as c_void_p from a torch tensor, a numpy array, an int or None."""
    if a is None:
        return c_ptr(None)
    if isinstance(a, (int,)):
        return c_ptr(a)
    if hasattr(a, "data_ptr"):
        return c_ptr(a.data_ptr())
    if hasattr(a, "ctypes"):
        return c_ptr(a.ctypes.data)
    if isinstance(a, c_ptr):
        return a
    raise TypeError(type(a))


class Library:
    """A loaded backend library with typed entry points. `lib.lx_gemv_w(...)` calls the C function; buffers
    pass through ptr(). Raises if the file or a requested symbol is missing: there is no fallback."""

    def __init__(self, path: str | None = None, require=None):
        self.path = path or os.environ.get("LX_KERNELS") or default_library_path()
        if not os.path.exists(self.path):
            raise FileNotFoundError(f"kernel library not found: {self.path} (build it: python -m dromos_b200.build)")
        self.cdll = ctypes.CDLL(self.path)
        self._fns = {}
        for name in require or ():
            self.fn(name)

    def has(self, name: str) -> bool:
        return hasattr(self.cdll, name)

    def fn(self, name: str):
        f = self._fns.get(name)
        if f is None:
            sig = SIGNATURES.get(name) or EXTENSIONS.get(name)
            if sig is None:
                raise AttributeError(f"{name}: not part of the bound ABI")
            if not hasattr(self.cdll, name):
                raise AttributeError(f"{self.path} does not export {name}")
            f = getattr(self.cdll, name)
            f.restype, f.argtypes = sig
            self._fns[name] = f
        return f

    def __getattr__(self, name):
        if name.startswith("lx_"):
            return self.fn(name)
        raise AttributeError(name)


def make_weight(wtype: int, data, scale=None, glob: float = 1.0, expert_global=None) -> LxWeight:
    """An lx_weight over the given buffers (tensors or arrays; the caller keeps them alive)."""
    return LxWeight(wtype, ptr(data), ptr(scale), float(glob), ptr(expert_global))
