"""hexagon_mlir_b200 — the hexagon-mlir operator hot path on B200 (sm_100a).

The product is ``libb200mlir.so`` (hand-written CUDA behind the C ABI declared
in ``include/b200mlir_capi.h``); this package is its Python binding and the
mirror of the reference's launch surface.  Importing it loads the shared
library and raises if it has not been built.
"""
from . import _capi
from ._capi import B200Error, LIB_PATH
from .launcher import *  # noqa: F401,F403

_capi.lib()  # fail loudly at import when the extension is missing
