"""Alias of intel_kivi_hybrid_b200 under the name callers of the reference use
(`from kivi_sycl import KiviCache, generate`, `from kivi_sycl import _C`)."""
import intel_kivi_hybrid_b200 as _impl
from intel_kivi_hybrid_b200 import __version__

__all__ = ["KiviCache", "generate", "__version__"]


def __getattr__(name):
    return getattr(_impl, name)
