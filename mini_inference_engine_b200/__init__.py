"""B200-native (sm_100a) continuous-batching hot path for a Qwen3-4B-FP8 serving engine.

The kernels live in ``csrc/`` and are exported through the C-ABI declared in
``include/mie_b200.h``.  ``engine/`` mirrors the reference engine's Python
operator interface (same module names, function names, signatures and error
behaviour) on top of that library, and ``install`` rebinds those operators
inside an imported copy of the reference package.
"""

from ._lib import MieLibraryError, exported_symbols, library_path, load  # noqa: F401

__all__ = ["MieLibraryError", "exported_symbols", "library_path", "load"]
