"""nv_embedding_cache_b200 — B200-native embedding lookup hot path behind the NV Embedding Cache API.

The product is ``libnve_b200.so`` (C ABI declared in ``include/nve_c_api.h`` and
``include/nve_b200_ops.h``).  This package holds its sources (``csrc/``), the build recipe
(``build.py``), a ctypes binding of the C ABI (``capi``), the Python layer classes that mirror the
reference's pynve bindings (``pynve``) and seeded synthetic workload generators (``datagen``).
There is no CPU fallback: importing ``capi`` without the built library raises.
"""

__all__ = ["capi", "datagen", "build"]
__version__ = "26.9.0"
