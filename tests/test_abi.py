"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol the header
declares, and fails the way the header says without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    src = open(os.path.join(ROOT, "include", "wick_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(wick_cuda_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported(cuda_lib):
    names = _header_functions()
    assert len(names) >= 30
    for n in names:
        assert hasattr(cuda_lib, n), f"{n} declared in include/wick_cuda.h but not exported"


def test_binding_covers_header(cuda_lib):
    from wick_b200 import _lib
    assert set(_header_functions()) == set(_lib.ALL_SYMBOLS)


def test_no_cpu_fallback_in_package():
    """The product must not import or call the oracle."""
    pkg = os.path.join(ROOT, "wick_b200")
    for dp, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".h")):
                txt = open(os.path.join(dp, f), errors="replace").read()
                assert not re.search(r"(from|import)\s+oracle|libwick_oracle|oracle[/.]|orc_[a-z]", txt), f"{f} uses the oracle"


def test_bad_arguments_do_not_touch_cuda(cuda_lib):
    from wick_b200 import _lib
    h = C.c_void_p()
    assert cuda_lib.wick_cuda_model_create(None, 0, 16, 0, C.byref(h)) == _lib.ERR_BAD_ARG
    junk = (C.c_uint8 * 64)(*([1] * 64))
    assert cuda_lib.wick_cuda_model_create(C.addressof(junk), 64, 16, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
    assert b"GGUF" in cuda_lib.wick_cuda_last_error()
    tiny = (C.c_uint8 * 8)()
    assert cuda_lib.wick_cuda_model_create(C.addressof(tiny), 8, 16, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
    assert cuda_lib.wick_cuda_model_create_from_file(b"/nonexistent/model.gguf", 16, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
    assert cuda_lib.wick_cuda_forward(None, 0, 0, None) == _lib.ERR_BAD_ARG
    assert cuda_lib.wick_cuda_reset(None) == _lib.ERR_BAD_ARG
    cuda_lib.wick_cuda_model_destroy(None)  # NULL is allowed
    w = C.c_void_p()
    raw = np.zeros(18, np.uint8)
    assert cuda_lib.wick_cuda_weight_create(3, raw.ctypes.data, 1, 32, C.byref(w)) == _lib.ERR_UNSUPPORTED_DTYPE
    assert cuda_lib.wick_cuda_weight_create(2, raw.ctypes.data, 1, 33, C.byref(w)) == _lib.ERR_BAD_ARG


def test_gguf_version_and_truncation_are_rejected(cuda_lib, model_dir):
    from wick_b200 import _lib, gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir)
    data = bytearray(open(path, "rb").read())
    h = C.c_void_p()
    v2 = bytearray(data)
    v2[4] = 2
    buf = (C.c_uint8 * len(v2)).from_buffer(v2)
    assert cuda_lib.wick_cuda_model_create(C.addressof(buf), len(v2), 64, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
    assert b"version" in cuda_lib.wick_cuda_last_error()
    cut = bytearray(data[: len(data) // 2])
    buf = (C.c_uint8 * len(cut)).from_buffer(cut)
    assert cuda_lib.wick_cuda_model_create(C.addressof(buf), len(cut), 64, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
    assert b"beyond file" in cuda_lib.wick_cuda_last_error()


def test_model_load_without_gpu_fails_loudly(cuda_lib, model_dir):
    """On a machine without a CUDA device loading reports a CUDA error instead of falling back."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from wick_b200 import gguf_synth as gs
    from wick_b200.model import CudaLfm2Model, WickCudaError
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir)
    with pytest.raises(WickCudaError) as e:
        CudaLfm2Model(path, 64)
    assert e.value.code in (-2, -1)


def test_gguf_wrapping_tensor_shape_is_rejected(cuda_lib, model_dir):
    """A tensor whose dimensions multiply to more than 2^64 (the product wraps to a tiny element count) must not pass
    the 'fits in the file' check."""
    import struct
    from wick_b200 import _lib, gguf_synth as gs
    path = gs.cached_model("tiny", "q4_0", 0, cache_dir=model_dir)
    data = bytearray(open(path, "rb").read())
    name = b"token_embd.weight"
    at = data.find(struct.pack("<Q", len(name)) + name)
    assert at > 0
    dims_at = at + 8 + len(name)
    (n_dims,) = struct.unpack_from("<I", data, dims_at)
    assert n_dims == 2
    h = C.c_void_p()
    for d0, d1 in ((1 << 63, 2), (1 << 32, 1 << 32), (1 << 31, 64)):
        bad = bytearray(data)
        struct.pack_into("<QQ", bad, dims_at + 4, d0, d1)
        buf = (C.c_uint8 * len(bad)).from_buffer(bad)
        assert cuda_lib.wick_cuda_model_create(C.addressof(buf), len(bad), 64, 0, C.byref(h)) == _lib.ERR_BAD_GGUF
        assert b"implausible shape" in cuda_lib.wick_cuda_last_error()
