"""B200 (sm_100a) implementation of MC-Sparse's token-sparse attention hot path.

The compute lives in hand-written CUDA kernels behind a C ABI
(``include/mcsparse_b200.h``, built into ``libmcsparse_b200.so``); this package
holds the build step, the ctypes binding and a host-side mirror of the
reference's ``mcsparse.kernels`` / ``mcsparse.h3`` entry points for the path.
Submodules are not imported at package load time, so that logic-only code works
without the shared library.
"""

__version__ = "0.1.0"

__all__: list[str] = []
