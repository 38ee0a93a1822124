"""B200 (sm_100a) compressed-KV kernels behind the TurboCAG C API.

`TurboQuantWrapper` mirrors the reference's ctypes wrapper
(tq_backend/turboquant_wrapper.py) on top of this package's libturboquant.so;
`BlockTable` is the host page allocator / block table.  Build the library with
``python -m turborag_b200.build``.
"""
from .wrapper import (BlockTable, TQConfig, TQTurbomsePageLayout, TQTurboProdPageLayout,
                      TurboQuantWrapper, load_library, DEFAULT_LIB_PATH, PARTIAL_STRIDE)

__all__ = ["BlockTable", "TQConfig", "TQTurbomsePageLayout", "TQTurboProdPageLayout",
           "TurboQuantWrapper", "load_library", "DEFAULT_LIB_PATH", "PARTIAL_STRIDE"]
