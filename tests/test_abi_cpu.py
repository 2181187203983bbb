"""CPU tests of the drop-in boundary: the shared library builds, loads and exports every entry point the header
declares (no compute call is made: there is no GPU here), the ctypes table matches the header, and the Python host
side rejects bad arguments with the reference's exception types and message substrings before touching the GPU
(reference: tests/test_decode.py:118-128, nvfp4_mla/__init__.py:78-79, 89-90)."""
import ctypes
import pathlib
import re

import pytest
import torch

import nvfp4_mla_b200 as mla
from nvfp4_mla_b200 import _lib, build

ROOT = pathlib.Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "nvfp4_mla_b200.h"


def header_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"NVFP4_MLA_API\s+[\w\s\*]+?\b(nvfp4_mla_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    build.build()  # no-op when the library is up to date; nvcc cross-compiles without a GPU
    return ctypes.CDLL(str(_lib.LIB_PATH))


def test_header_declares_the_expected_entry_points():
    names = header_symbols()
    for must in ("nvfp4_mla_decode", "nvfp4_mla_decode_workspace_bytes", "nvfp4_mla_dequantize", "nvfp4_mla_combine",
                 "nvfp4_mla_quantize_append", "nvfp4_mla_last_error", "nvfp4_mla_version", "nvfp4_mla_decode_static"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    missing = [n for n in header_symbols() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_ctypes_table_matches_header():
    assert set(_lib.SIGNATURES) <= set(header_symbols())


def test_version_and_error_string_need_no_gpu(lib):
    lib.nvfp4_mla_version.restype = ctypes.c_int
    assert lib.nvfp4_mla_version() == 100
    lib.nvfp4_mla_last_error.restype = ctypes.c_char_p
    assert isinstance(lib.nvfp4_mla_last_error(), bytes)


def cpu_args(heads=16, q_dtype=torch.bfloat16, table_dtype=torch.int32, cache_dtype=torch.float8_e4m3fn):
    B, P, ps = 2, 4, 16
    return (torch.zeros(B, heads, 512, dtype=q_dtype), torch.zeros(B, heads, 64, dtype=q_dtype),
            torch.zeros(P, ps, 256, dtype=torch.uint8), torch.zeros(P, ps, 32, dtype=torch.uint8).view(cache_dtype),
            torch.zeros(P, ps, 64, dtype=torch.uint8).view(torch.float8_e4m3fn), torch.zeros(B, 2, dtype=table_dtype),
            torch.ones(B, dtype=torch.int32), 0.1)


def test_python_host_rejects_bad_arguments_before_any_gpu_call():
    """What can be rejected without a GPU: the precision and dtype names (ValueError, as the reference raises them)
    and host-resident caches (RuntimeError). The dtype / shape messages are checked by the GPU tests."""
    with pytest.raises(ValueError, match="precision must be one of"):
        mla.decode(*cpu_args(), precision="fp4-qk")
    with pytest.raises(ValueError, match="precision must be one of"):
        mla.decode_partial(*cpu_args(), precision="int8")
    with pytest.raises(RuntimeError, match="CUDA"):
        mla.decode(*cpu_args(), max_kv_len=8)
    a = cpu_args()
    with pytest.raises(ValueError, match="dtype"):
        mla.dequantize(a[2], a[3], a[4], dtype=torch.float16)
    with pytest.raises(RuntimeError, match="float32"):
        mla.combine(torch.zeros(2, 4, 512, dtype=torch.float16), torch.zeros(2, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        mla.combine(torch.zeros(2, 4, 512), torch.zeros(2, 4))


def test_reference_style_imports_resolve():
    """The import forms the reference's own tests and benchmarks use (tests/test_decode.py:8-10, benchmarks/bench.py:31)."""
    import nvfp4_mla
    from nvfp4_mla.testing import SM_SCALE, RandomCache, rel_l2
    import nvfp4_mla_b200.testing as T
    assert nvfp4_mla.decode is mla.decode and nvfp4_mla.dequantize is mla.dequantize
    assert RandomCache is T.SyntheticCache and rel_l2 is T.rel_l2 and SM_SCALE == T.SM_SCALE
    c = RandomCache([5, 40], 16, 16, seed=1)
    assert c.ckv_cache.dtype == torch.uint8 and c.ckv_cache.shape[1:] == (16, 256)


def test_dequantize_rejects_a_misaligned_cache_before_any_launch(lib):
    """A ckv_cache pointer that is 2- but not 4-byte aligned must come back as an error code: the bf16 kernel loads
    4-byte words from it, and a misaligned device address would fault the GPU."""
    lib.nvfp4_mla_dequantize.restype = ctypes.c_int
    lib.nvfp4_mla_dequantize.argtypes = _lib.SIGNATURES["nvfp4_mla_dequantize"][1]
    lib.nvfp4_mla_last_error.restype = ctypes.c_char_p
    rc = lib.nvfp4_mla_dequantize(0x10002, 0x20000, 0x30000, 64, 1.0, 1.0, 1, 0x40000, 0x50000, None)
    assert rc != 0 and b"aligned" in lib.nvfp4_mla_last_error()
