"""B200-native KIVI 2-bit KV-cache engine (drop-in for the kivi_sycl API)."""
__version__ = "0.1.0"
