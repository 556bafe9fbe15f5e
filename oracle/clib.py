"""ctypes access to the compiled CPU checkers.  TEST INFRASTRUCTURE ONLY.

``c_port()``  -> oracle/libkivi_oracle_c.so (plain-C restatement, kivi_ref.c)
``ref_tile()`` -> oracle/_ref/libkivi_ref_tile.so (the reference's own
quant_tile.hpp compiled against oracle/sycl_shim), or None when it was never
built.  Both are built by ``make -C oracle``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32 = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8 = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")


def reference_dir():
    """Where the reference project's tree is: $KIVI_REFERENCE_DIR, else a
    checkout named ``reference`` next to this repository; None when neither
    exists (the reference-derived checker is then not rebuilt)."""
    cand = os.environ.get("KIVI_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(cand) else None


def build(reference=None):
    reference = reference or reference_dir()
    cmd = ["make", "-s", "-C", _HERE]
    if reference:
        cmd.append(f"REFERENCE={reference}")
    subprocess.run(cmd, check=True)


def c_port():
    path = os.path.join(_HERE, "libkivi_oracle_c.so")
    if not os.path.exists(path):
        build()
    lib = ctypes.CDLL(path)
    lib.kivi_c_quantize_groups.argtypes = [_f32, _u8, _f32, _f32, ctypes.c_long, ctypes.c_int, ctypes.c_int]
    lib.kivi_c_dequantize_groups.argtypes = [_u8, _f32, _f32, _f32, ctypes.c_long, ctypes.c_int]
    lib.kivi_c_roundtrip_groups.argtypes = [_f32, _f32, ctypes.c_long, ctypes.c_int, ctypes.c_int]
    for f in (lib.kivi_c_quantize_groups, lib.kivi_c_dequantize_groups, lib.kivi_c_roundtrip_groups):
        f.restype = None
    return lib


def ref_tile():
    path = os.path.join(_HERE, "_ref", "libkivi_ref_tile.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    lib.ref_quantize_groups.argtypes = [_f32, _u8, _f32, _f32, ctypes.c_long, ctypes.c_int]
    lib.ref_roundtrip_groups.argtypes = [_f32, _f32, ctypes.c_long, ctypes.c_int]
    lib.ref_quantize_groups.restype = None
    lib.ref_roundtrip_groups.restype = None
    return lib


def c_quantize(x: np.ndarray, G: int, half_even: bool = False, lib=None):
    lib = lib or c_port()
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    n = x.size // G
    packed = np.empty(x.size // 4, np.uint8)
    scales = np.empty(n, np.float32)
    zeros = np.empty(n, np.float32)
    lib.kivi_c_quantize_groups(x, packed, scales, zeros, n, G, int(half_even))
    return packed, scales, zeros


def c_dequantize(packed, scales, zeros, G: int, lib=None):
    lib = lib or c_port()
    out = np.empty(scales.size * G, np.float32)
    lib.kivi_c_dequantize_groups(np.ascontiguousarray(packed).reshape(-1),
                                 np.ascontiguousarray(scales).reshape(-1),
                                 np.ascontiguousarray(zeros).reshape(-1), out, scales.size, G)
    return out


def c_roundtrip(x: np.ndarray, G: int, half_even: bool = False, lib=None):
    lib = lib or c_port()
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib.kivi_c_roundtrip_groups(x.reshape(-1), out.reshape(-1), x.size // G, G, int(half_even))
    return out


def ref_quantize(x: np.ndarray, G: int):
    lib = ref_tile()
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    n = x.size // G
    packed = np.empty(x.size // 4, np.uint8)
    scales = np.empty(n, np.float32)
    zeros = np.empty(n, np.float32)
    lib.ref_quantize_groups(x, packed, scales, zeros, n, G)
    return packed, scales, zeros


def ref_roundtrip(x: np.ndarray, G: int):
    lib = ref_tile()
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib.ref_roundtrip_groups(x.reshape(-1), out.reshape(-1), x.size // G, G)
    return out
