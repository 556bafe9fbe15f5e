"""B200-native KIVI 2-bit KV-cache engine: drop-in for the kivi_sycl API.

    from kivi_cuda import KiviCache, generate          # or: from kivi_sycl import ...
    from kivi_cuda import _C                           # the twelve native operators

Importing the package does not touch the GPU; the native library is loaded (and
built in-tree if missing) when ``KiviCache``, ``generate``, ``_C`` or ``cabi`` is
first used.  There is no CPU fallback.
"""
__version__ = "0.1.0"

__all__ = ["KiviCache", "generate", "__version__"]


def __getattr__(name):
    if name == "KiviCache":
        from .cache.manager import KiviCache
        return KiviCache
    if name == "generate":
        from .generation.generate import generate
        return generate
    if name == "_C":
        from .extension.loader import kivi_native
        return kivi_native
    raise AttributeError(name)
