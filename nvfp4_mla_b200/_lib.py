"""ctypes binding of libnvfp4_mla_b200.so (the C ABI declared in include/nvfp4_mla_b200.h).

There is no fallback: if the library is missing or an entry point fails, the caller gets an exception.
"""
import ctypes
import functools
import pathlib

LIB_PATH = pathlib.Path(__file__).resolve().parent / "libnvfp4_mla_b200.so"

_vp, _i32, _i64, _f32, _u32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_uint32

# name -> (restype, argtypes); mirrors include/nvfp4_mla_b200.h
SIGNATURES = {
    "nvfp4_mla_version": (_i32, []),
    "nvfp4_mla_last_error": (ctypes.c_char_p, []),
    "nvfp4_mla_decode_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "nvfp4_mla_decode_launches": (_i32, [_i32, _i32, _i32, _i32, _i32]),
    "nvfp4_mla_decode": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _i64, _vp, _i32, _i32, _f32, _f32, _f32,
                                _i32, _i32, _i32, _vp, _vp, _vp, _vp, _i64, _vp]),
    "nvfp4_mla_decode_static": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp, _i64, _vp, _i32, _i32, _f32, _f32, _f32,
                                       _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "nvfp4_mla_decode_static_capacity": (_i64, []),
    "nvfp4_mla_decode_static_status": (_i32, [_vp]),
    "nvfp4_mla_workspace_status": (_i32, [_vp, _vp]),
    "nvfp4_mla_profile_begin": (_i32, [_i32]),
    "nvfp4_mla_profile_end": (_i32, [_vp, _i32]),
    "nvfp4_mla_dequantize": (_i32, [_vp, _vp, _vp, _i64, _f32, _f32, _i32, _vp, _vp, _vp]),
    "nvfp4_mla_combine": (_i32, [_vp, _vp, _i32, _i64, _vp, _vp, _vp, _vp]),
    "nvfp4_mla_combine_strided": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "nvfp4_mla_combine_records": (_i32, [_vp, _i32, _i64, _vp, _vp, _vp, _vp]),
    "nvfp4_mla_combine_records_signalled": (_i32, [_vp, _vp, _i32, _u32, _i64, _i32, _i64, _vp, _vp, _vp, _vp, _vp]),
    "nvfp4_mla_quantize_append": (_i32, [_vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i32, _vp, _vp, _i32, _f32, _f32,
                                         _vp, _vp]),
}


@functools.lru_cache(maxsize=None)
def load():
    """Loads the shared library (built by ``python -m nvfp4_mla_b200.build``) and types its entry points."""
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m nvfp4_mla_b200.build` "
                           "(there is no fallback implementation)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def check(code):
    """Raises RuntimeError with the library's message if an entry point returned non-zero."""
    if code != 0:
        raise RuntimeError(load().nvfp4_mla_last_error().decode())
