"""ctypes binding of libflowwalker.so, the C ABI declared in include/flowwalker.h.

This is the harness side used by the tests and the bench; the product is the
shared library.  Nothing here computes a walk: every call goes to the CUDA
engine, and loading fails loudly when the library has not been built.
"""
from ._binding import (  # noqa: F401
    APP_DEEPWALK, APP_METAPATH, APP_NODE2VEC, APP_PPR, ENGINE_MANAGED, GROUP_EDGE, GROUP_STRIP,
    Engine, FlowWalkerError, Graph, WalkStats, lib, lib_path, lognormal_weights, make_params, rmat,
)
