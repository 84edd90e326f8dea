"""The shared-memory plans of the decode GEMV kernels that bring their weights in with bulk copies (lx_b200_gemv_ring_plan:
the geometry functions the launches use, nothing launched), swept over K, M and activation dtype on the CPU: everything a
kernel would address lies inside the 226 KB its launch opts in to, on the alignments bulk copies and 16-byte reads need."""

import ctypes

import numpy as np

from dromos_b200 import abi

SMEM_MAX = 226 * 1024  # what the launches opt in to (an SM has 227 KB)


def plan(lib, wtype, K, M, x_bf16):
    out = (ctypes.c_int32 * 12)()
    assert lib.lx_b200_gemv_ring_plan(wtype, K, M, int(x_bf16), out) == 0
    return list(out)


def test_bad_arguments():
    lib = abi.Library(abi.default_library_path())
    out = (ctypes.c_int32 * 12)()
    assert lib.lx_b200_gemv_ring_plan(abi.W_FP8, 4096, 1, 1, None) == abi.ERR_INVALID
    assert lib.lx_b200_gemv_ring_plan(abi.W_FP8, 0, 1, 1, out) == abi.ERR_INVALID
    assert lib.lx_b200_gemv_ring_plan(abi.W_FP8, 4096, 9, 1, out) == abi.ERR_INVALID
    assert plan(lib, abi.W_BF16, 4096, 1, True)[0] == 0  # plain bf16 has no such kernel


def test_lossless_plans():
    lib = abi.Library(abi.default_library_path())
    seen_whole = seen_rows = 0
    for K in list(range(64, 4097, 64)) + [5120, 6144, 7168, 8192, 11008, 12288, 14336, 16384]:
        row = lib.lx_bf16x_row_bytes(K)
        nblk = (K + 127) // 128
        hb = row - 192 * nblk
        for M in range(1, 9):
            for x_bf16 in (True, False):
                S, whole, cb, spu, stride, slot, hstride, hslot, hdr_off, ring_off, bar_off, total = plan(lib, abi.W_BF16X, K, M, x_bf16)
                if S == 0:
                    continue
                assert S >= 2 and total <= SMEM_MAX and bar_off + 8 * (2 * S + 8) + 4 <= total
                assert ring_off % 128 == 0 and bar_off == ring_off + S * slot and bar_off % 8 == 0
                if whole:
                    seen_whole += 1
                    assert spu == 1 and cb == nblk and stride == row and slot >= 16 * row and slot % 128 == 0
                else:
                    seen_rows += 1
                    assert S >= 3 and 1 <= cb <= 32 and (spu - 1) * cb < nblk <= spu * cb
                    assert stride >= cb * 192 + 16 and stride % 128 == 64 and slot == 16 * stride  # 8 bytes before, 8 after; odd rows on the other banks
                    assert hstride >= hb + 8 and hstride % 16 == 0 and hslot == 16 * hstride
                    assert hdr_off % 128 == 0 and hdr_off + 2 * hslot <= ring_off
    assert seen_whole and seen_rows
    # the measured case: K = 4096, one bf16 activation row: two whole units of 16 records
    S, whole, *_ = plan(lib, abi.W_BF16X, 4096, 1, True)
    assert (S, whole) == (2, 1)


def test_plans_of_the_quantized_formats():
    lib = abi.Library(abi.default_library_path())
    fits = 0
    for wtype in (abi.W_INT8, abi.W_FP8, abi.W_NVFP4):
        for K in range(128, 16385, 128):
            row = K // 2 if wtype == abi.W_NVFP4 else K
            for M in range(1, 9):
                for x_bf16 in (True, False):
                    S, whole, cb, spu, stride, slot, scale_off, _, _, ring_off, bar_off, total = plan(lib, wtype, K, M, x_bf16)
                    if S == 0:
                        continue
                    fits += 1
                    assert 2 <= S <= 6 and whole == 1 and spu == 1 and stride == row and total <= SMEM_MAX
                    assert slot == 16 * row + (K if wtype == abi.W_NVFP4 else 0) and scale_off == 16 * row
                    assert ring_off % 128 == 0 and slot % 128 == 0 and scale_off % 16 == 0 and bar_off == ring_off + S * slot and bar_off % 8 == 0
                    assert bar_off + 8 * (2 * S + 4) + 4 <= total
                    if wtype == abi.W_NVFP4:
                        assert K % 256 == 0
    assert fits
    assert plan(lib, abi.W_FP8, 4096, 1, True)[0] == 3 and plan(lib, abi.W_FP8, 8192, 1, True)[0] == 0
    assert plan(lib, abi.W_NVFP4, 8192, 1, True)[0] == 2
