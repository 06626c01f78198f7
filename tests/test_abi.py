"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "schedforge_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sfb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(sfb):
    lib = sfb.load()
    declared = header_symbols()
    assert len(declared) >= 50
    missing = [name for name in declared if not hasattr(lib, name)]
    assert missing == []
    assert sorted(sfb.EXPORTS) == declared  # the Python binding lists exactly the header's functions


def test_version_and_error_channel(sfb):
    lib = sfb.load()
    assert b"sm_100a" in lib.sfb_version()
    status = lib.sfb_k_add(None, None, None, C.c_int64(0), 0, None)
    assert status == sfb.SFB_INVALID_ARGUMENT
    assert b"residual shape mismatch" in lib.sfb_last_error()


def test_no_cpu_fallback(sfb):
    """Without a CUDA device a compute entry point must fail loudly, never compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    x = np.ones(16, np.float32)
    status = sfb.load().sfb_k_add(x.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p),
                                  x.ctypes.data_as(C.c_void_p), C.c_int64(16), 0, None)
    assert status == sfb.SFB_CUDA_ERROR
    assert np.all(x == 1.0)


def test_struct_layouts_match_header(sfb):
    """ctypes mirrors: field counts and sizes follow the C structs (natural alignment)."""
    assert C.sizeof(sfb.DecoderConfig) == 14 * 4
    assert C.sizeof(sfb.DecoderData) == 16 * 8
    assert C.sizeof(sfb.CompileOptions) == 17 * 4
    assert C.sizeof(sfb.AttentionConfig) == 9 * 4
    assert C.sizeof(sfb.MoeConfig) == 5 * 4
    assert C.sizeof(sfb.GraphSummary) == 7 * 4
    assert C.sizeof(sfb.DecoderResult) == 9 * 8 + 8
    assert C.sizeof(sfb.GemmArgs) % 8 == 0 and sfb.GemmArgs.kv_num_blocks.offset == C.sizeof(sfb.GemmArgs) - 4


def test_weight_layout_and_scratch_size_helpers_need_no_device(sfb):
    """Element count of the 64x64-blocked weight copy and the byte count of the few-row GEMM scratch."""
    lib = sfb.load()
    assert lib.sfb_tiled_weight_elems(128, 64) == 2 * 4096
    assert lib.sfb_tiled_weight_elems(130, 65) == 3 * 2 * 4096     # ragged edges are padded to whole blocks
    assert lib.sfb_tiled_weight_elems(0, 64) == 0
    one_tile = 128 * 128 * 4
    assert lib.sfb_gemm_stream_workspace_bytes(128) == one_tile + 16
    assert lib.sfb_gemm_stream_workspace_bytes(4096) == 32 * one_tile + 128
    assert lib.sfb_gemm_stream_workspace_bytes(0) == 0
