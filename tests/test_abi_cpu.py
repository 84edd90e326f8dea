"""The C-ABI library loads without a GPU and exports every symbol include/dromos_b200.h declares, with the bindings of
dromos_b200/abi.py covering each of them. No compute call is made here."""

import os
import re

from dromos_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dromos_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"LX_API[^;(]*?\b(lx_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = abi.Library(abi.default_library_path())
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert lib.has(name), f"{name} is declared in include/dromos_b200.h but not exported"
        lib.fn(name)  # and bound with a signature


def test_no_binding_without_a_declaration():
    names = set(declared_symbols())
    for name in list(abi.SIGNATURES) + list(abi.EXTENSIONS):
        assert name in names, f"{name} is bound in abi.py but not declared in the header"


def test_host_only_entry_points_answer_without_a_gpu():
    lib = abi.Library(abi.default_library_path())
    assert lib.lx_rt_backend() == 0
    assert lib.lx_bf16x_row_bytes(4096) == 6192 and lib.lx_bf16x_row_bytes(0) == -1
    assert lib.lx_gemm_workspace_bytes(0, 4096, 0) == 0 and lib.lx_gemm_workspace_bytes(32, 4096, 0) > 0
    assert lib.lx_moe_grouped_workspace_bytes(32, 4096, 1536, 64, 8, 0) > 0
    n = lib.lx_tune_kernels(None, 0)
    assert n == 11  # five decode GEMV kernels and the six lx_gemm_w families
    assert lib.lx_tune_variants(b"gemm_w.f8.sm100") == 1 and lib.lx_tune_set(b"gemm_w.f8.sm100", 200, 384, 1024, 0) == 0
    assert lib.lx_tune_variants(b"gemv_w_fp8") >= 1 and lib.lx_tune_variants(b"nope") == 0
    names = [lib.lx_tune_variant_name(b"gemv_w_fp8", i) for i in range(lib.lx_tune_variants(b"gemv_w_fp8"))]
    assert re.match(rb"s16d\d+c\d+", names[0]) and b"s8ring" in names and b"s1tc" in names and b"s16d1c1" in names
    lossless = [lib.lx_tune_variant_name(b"gemv_bf16x", i) for i in range(lib.lx_tune_variants(b"gemv_bf16x"))]
    assert lossless == [b"d4c2", b"d8c1", b"d1c1"]  # its own forms, no split in the name: every one keeps the bf16 kernel's order
    assert lib.lx_tune_variant_name(b"gemv_w_fp8", len(names)) is None
    assert lib.lx_tune_set(b"gemv_w_fp8", 1, 64, 64, 10**6) == abi.ERR_TUNE_VARIANT
    assert lib.lx_tune_set(b"gemv_w_fp8", 3, 64, 64, 1) == 0 and lib.lx_tune_get(b"gemv_w_fp8", 4, 64, 64) == 1  # M bucket 4
    lib.lx_tune_clear()
    assert lib.lx_tune_get(b"gemv_w_fp8", 4, 64, 64) == -1


def test_tune_set_refuses_another_summation_order():
    """The order-class rule (engine/cuda/tunable.cu:104-118, tests/kernels/test_gemv_w.py:293-318): lx_tune_set stores a
    variant only if it adds a row's products in the order of the shape's default; lx_tune_force stores anything."""
    lib = abi.Library(abi.default_library_path())
    lib.lx_tune_clear()
    for kernel in (b"gemv_w_bf16", b"gemv_w_int8", b"gemv_w_fp8", b"gemv_w_nvfp4", b"gemv_bf16x"):
        n = lib.lx_tune_variants(kernel)
        names = [lib.lx_tune_variant_name(kernel, i) for i in range(n)]
        same = [i for i, nm in enumerate(names) if re.match(rb"(s16)?d\d+c\d+", nm)]
        other = [i for i in range(n) if i not in same]
        assert same and (other or kernel == b"gemv_bf16x")  # the lossless kernel lists only its own order-keeping forms
        for v in same:  # K = 4096: every format's decode GEMV takes it
            assert lib.lx_tune_set(kernel, 1, 4096, 4096, v) == 0
            assert lib.lx_tune_get(kernel, 1, 4096, 4096) == v
        for v in other:
            assert lib.lx_tune_set(kernel, 1, 4096, 4096, v) == abi.ERR_TUNE_REJECTED
            assert lib.lx_tune_get(kernel, 1, 4096, 4096) == same[-1]  # the table is unchanged
            assert lib.lx_tune_force(kernel, 8, 4096, 4096, v) == 0 and lib.lx_tune_get(kernel, 8, 4096, 4096) == v
        # K = 40 is not whole 64-byte steps for any format: the default there is the other kernel family
        if other:
            assert lib.lx_tune_set(kernel, 1, 4096, 40, names.index(b"s8ring")) == 0
            assert lib.lx_tune_set(kernel, 1, 4096, 40, names.index(b"s1tc")) == abi.ERR_TUNE_REJECTED
        for v in same:  # naming a decode GEMV form for a shape it cannot take changes nothing: admitted
            assert lib.lx_tune_set(kernel, 1, 4096, 40, v) == 0
    lib.lx_tune_clear()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "dromos_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("# oracle", ""), f"{f} mentions the oracle"
