"""CPU-side checks of the drop-in boundary: the library builds, loads and exports what the header declares,
and the product refuses to compute without a GPU (no fallback).  No kernel runs here."""
import ctypes
import os
import re

import numpy as np
import pytest

import zeninfer_b200
from zeninfer_b200 import backend, blocks, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib_path():
    return build.build()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "zen_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zen_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_symbols() == sorted(backend.ABI_SYMBOLS)


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_header_compiles_as_plain_c(tmp_path):
    # the boundary must be bindable from C (cgo, JNI and ctypes all see it as C)
    src = tmp_path / "t.c"
    src.write_text('#include "zen_cuda.h"\nint main(void){zen_cuda_gemv_task t; (void)t; return ZEN_CUDA_MAX_BATCH == 8 ? 0 : 1;}\n')
    import subprocess
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_no_gpu_means_loud_failure(lib_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = backend.load_library(lib_path)
    assert lib.zen_cuda_init() == 0
    assert b"CUDA" in lib.zen_cuda_last_error()
    w = np.zeros(34, np.uint8)
    x = np.zeros(32, np.float32)
    y = np.full(1, 123456.0, np.float32)
    assert lib.zen_cuda_gemv_q8_0(w.ctypes.data, x.ctypes.data, y.ctypes.data, 1, 32) == 0
    assert y[0] == 123456.0  # nothing computed, nothing written
    with pytest.raises(zeninfer_b200.BackendError):
        zeninfer_b200.Backend(lib_path)


def test_missing_library_is_an_error(tmp_path):
    with pytest.raises(zeninfer_b200.BackendError):
        backend.load_library(str(tmp_path / "nope.so"))


def test_product_never_touches_the_oracle():
    # the package must not import, read or execute anything under oracle/
    pkg = os.path.join(ROOT, "zeninfer_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text and "libzenref" not in text, f


def test_block_sizes_match_reference_registry():
    # src/quant.cpp:253,257,259
    assert (blocks.BLOCK_ELEMENTS[blocks.Q4_0], blocks.BLOCK_BYTES[blocks.Q4_0]) == (32, 18)
    assert (blocks.BLOCK_ELEMENTS[blocks.Q8_0], blocks.BLOCK_BYTES[blocks.Q8_0]) == (32, 34)
    assert (blocks.BLOCK_ELEMENTS[blocks.Q6_K], blocks.BLOCK_BYTES[blocks.Q6_K]) == (256, 210)
    assert blocks.row_bytes(blocks.Q8_0, 4096) == 4352 and blocks.row_bytes(blocks.Q4_0, 4096) == 2304 and blocks.row_bytes(blocks.Q6_K, 4096) == 3360
    assert blocks.row_bytes(blocks.Q8_0, 48) == 0 and blocks.row_bytes(blocks.Q6_K, 4096 + 32) == 0


def test_workspace_sizes_are_plain_arithmetic(lib_path):
    # the size queries need no device: callers size their workspaces before anything is resident
    lib = backend.load_library(lib_path)
    ACT_INT8, ACT_FP32 = backend.ACT_INT8, backend.ACT_FP32
    for tokens, rows, cols in [(9, 128, 256), (40, 300, 4096), (512, 14336, 4096), (129, 4096, 14336), (16, 100, 544)]:
        g = lib.zen_cuda_gemm_workspace_bytes_act(tokens, cols, ACT_FP32)
        i8 = lib.zen_cuda_gemm_workspace_bytes_act(tokens, cols, ACT_INT8)
        assert lib.zen_cuda_gemm_workspace_bytes(tokens, cols) == i8
        assert g >= i8 >= tokens * cols                                   # at least one int8 plane of the activations
        if cols % 256 == 0:
            assert i8 >= 2 * tokens * cols                                # the group-scale kernel: two digit planes in either mode
        # the per-format products: never less than what the group-scale kernel needs, and room for the widened codes
        assert lib.zen_cuda_gemm_q4_0_workspace_bytes(tokens, rows, cols) >= rows * cols + 2 * tokens * cols
        assert lib.zen_cuda_gemm_kquant_workspace_bytes(tokens, rows, cols) >= rows * cols + 2 * rows * (cols // 32) * 4 + 2 * tokens * cols
        assert lib.zen_cuda_gemm_q6_k_workspace_bytes(tokens, cols) >= 4 * tokens * cols     # a token is two columns of two digits
        bigger = lib.zen_cuda_gemm_workspace_bytes_act(tokens + 1, cols, ACT_FP32)
        assert bigger >= g
