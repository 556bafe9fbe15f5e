"""Single import seam for the compiled extension (kivi_cuda._C).

Mirrors the reference's seam (src/kivi_sycl/extension/loader.py:8-19): every
module that needs the native operators imports ``kivi_native`` from here, so a
missing build is explained in exactly one place.  The extension is built
in-tree on first use when nvcc and g++ are available; there is no fallback
implementation.
"""
import importlib

try:
    kivi_native = importlib.import_module("intel_kivi_hybrid_b200._C")
except ImportError:
    try:
        from intel_kivi_hybrid_b200 import _build
        _build.build_all()
        kivi_native = importlib.import_module("intel_kivi_hybrid_b200._C")
    except Exception as exc:
        raise ImportError(
            "kivi_cuda._C (the compiled CUDA extension) was not found and could not be built.\n"
            "Build it in-place with:\n\n"
            "  python -m intel_kivi_hybrid_b200._build\n\n"
            "(needs nvcc with sm_100a support, g++ and the installed torch headers)."
        ) from exc

__all__ = ["kivi_native"]
